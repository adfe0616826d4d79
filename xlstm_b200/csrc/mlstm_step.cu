// mLSTM single-token decode step: one streaming pass over the C state per (stream, head).
//
//   m' = max(logsig(f) + m, i);  f' = exp(logsig(f) + m - m');  i' = exp(i - m')
//   C' = f' C + i' k v^T;  n' = f' n + i' k;  h = (q~^T C') / (max(|q~^T n'|, exp(-m')) + eps),  q~ = q / sqrt(DHQK)
//
// The kernel is HBM-bound: 8 bytes move per state element against 4 flops, so the layout is chosen for
// coalesced 128-bit accesses.  A CTA owns a 128-column slice of one C matrix; a warp reads one 512-byte
// row segment per instruction (lane -> float4), rows are strided over the 8 warps and unrolled so that
// several independent 16-byte loads per thread are in flight.  The row update, the rank-1 term and the
// q~-weighted column reduction are done in the same pass; the 8 partial column sums meet in shared memory.
#include "common.cuh"

namespace xl {

constexpr int STEP_THREADS = 256;
constexpr int STEP_WARPS = STEP_THREADS / 32;
constexpr int STEP_COLS = 128;   // columns of C per CTA (32 lanes x float4)
constexpr int STEP_UNROLL = 8;   // rows in flight per warp

template <typename T>
__global__ void __launch_bounds__(STEP_THREADS) mlstm_step_kernel(const xl_mlstm_step_params p) {
  extern __shared__ float smem[];
  float* s_q = smem;                 // DHQK   q~ (scaled)
  float* s_k = s_q + p.DHQK;         // DHQK   i' * k
  float* s_red = s_k + p.DHQK;       // STEP_WARPS * STEP_COLS partial column sums
  __shared__ float s_scalar[STEP_WARPS];

  const int b = blockIdx.z, head = blockIdx.y, col0 = blockIdx.x * STEP_COLS;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int DHQK = p.DHQK, DHV = p.DHV;
  const int64_t row = p.slot ? (int64_t)p.slot[b] : (int64_t)b;
  if (p.slot && (row < 0 || row >= p.n_slots)) {
    // a negative slot marks an inactive stream: nothing of the pool is touched, h is zero.  A slot beyond the pool is
    // an error of the caller: the row is skipped all the same and the status word says so.
    T* hz = reinterpret_cast<T*>(p.h) + b * p.h_sb + head * p.h_sh;
    if (tid < STEP_COLS && col0 + tid < p.DHV) hz[col0 + tid] = from_float<T>(0.f);
    if (row >= p.n_slots && tid == 0 && p.status) atomicExch(p.status, 2);
    return;
  }
  const int64_t sidx = row * p.NH + head;

  const T* q = reinterpret_cast<const T*>(p.q) + b * p.q_sb + head * p.q_sh;
  const T* k = reinterpret_cast<const T*>(p.k) + b * p.k_sb + head * p.k_sh;
  const T* v = reinterpret_cast<const T*>(p.v) + b * p.v_sb + head * p.v_sh;
  T* h = reinterpret_cast<T*>(p.h) + b * p.h_sb + head * p.h_sh;

  const float ig = p.igate[b * p.g_sb + head * p.g_sh];
  const float fg = p.fgate[b * p.g_sb + head * p.g_sh];
  const float m_old = p.m_in ? p.m_in[sidx] : 0.f;
  const float logf = log_sigmoid(fg);
  const float m_new = fmaxf(logf + m_old, ig);
  const float f_act = expf(logf + m_old - m_new);
  const float i_act = expf(ig - m_new);
  const float qscale = rsqrtf((float)DHQK);

  // stage q~ and i'k, update n, and accumulate q~ . n'
  const float* n_in = p.n_in ? p.n_in + sidx * DHQK : nullptr;
  float* n_out = p.n_out + sidx * DHQK;
  float qn = 0.f;
  for (int d = tid; d < DHQK; d += STEP_THREADS) {
    const float qd = to_float(q[d]) * qscale;
    const float kd = to_float(k[d]) * i_act;
    s_q[d] = qd;
    s_k[d] = kd;
    const float nn = f_act * (n_in ? n_in[d] : 0.f) + kd;
    if (blockIdx.x == 0) n_out[d] = nn;
    qn += qd * nn;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) qn += __shfl_xor_sync(0xffffffffu, qn, o);
  if (lane == 0) s_scalar[warp] = qn;
  __syncthreads();
  qn = 0.f;
#pragma unroll
  for (int w = 0; w < STEP_WARPS; ++w) qn += s_scalar[w];
  const float inv_den = 1.f / (fmaxf(fabsf(qn), expf(-m_new)) + p.eps);
  if (blockIdx.x == 0 && tid == 0) p.m_out[sidx] = m_new;

  // streaming pass over this CTA's column slice of C
  const int col = col0 + lane * 4;
  const bool col_ok = col < DHV;  // DHV % 4 == 0 is checked on the host
  float4 vv = make_float4(0.f, 0.f, 0.f, 0.f);
  if (col_ok) {
    if constexpr (sizeof(T) == 4) {
      vv = *reinterpret_cast<const float4*>(v + col);
    } else {
      const uint2 raw = *reinterpret_cast<const uint2*>(v + col);
      const float2 a = unpack_bf16x2(raw.x), c = unpack_bf16x2(raw.y);
      vv = make_float4(a.x, a.y, c.x, c.y);
    }
  }
  const float* c_in = p.c_in ? p.c_in + sidx * (int64_t)DHQK * DHV + col : nullptr;
  float* c_out = p.c_out + sidx * (int64_t)DHQK * DHV + col;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  if (col_ok) {
    for (int r0 = warp; r0 < DHQK; r0 += STEP_WARPS * STEP_UNROLL) {
      float4 c[STEP_UNROLL];
#pragma unroll
      for (int u = 0; u < STEP_UNROLL; ++u) {
        const int r = r0 + u * STEP_WARPS;
        c[u] = (c_in && r < DHQK) ? __ldcs(reinterpret_cast<const float4*>(c_in + (int64_t)r * DHV))
                                  : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < STEP_UNROLL; ++u) {
        const int r = r0 + u * STEP_WARPS;
        if (r < DHQK) {
          const float kr = s_k[r], qr = s_q[r];
          float4 o;
          o.x = fmaf(f_act, c[u].x, kr * vv.x);
          o.y = fmaf(f_act, c[u].y, kr * vv.y);
          o.z = fmaf(f_act, c[u].z, kr * vv.z);
          o.w = fmaf(f_act, c[u].w, kr * vv.w);
          __stcs(reinterpret_cast<float4*>(c_out + (int64_t)r * DHV), o);
          acc.x = fmaf(qr, o.x, acc.x);
          acc.y = fmaf(qr, o.y, acc.y);
          acc.z = fmaf(qr, o.z, acc.z);
          acc.w = fmaf(qr, o.w, acc.w);
        }
      }
    }
  }
  reinterpret_cast<float4*>(s_red)[warp * 32 + lane] = acc;
  __syncthreads();
  if (tid < STEP_COLS && col0 + tid < DHV) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < STEP_WARPS; ++w) s += s_red[w * STEP_COLS + tid];
    h[col0 + tid] = from_float<T>(s * inv_den);
  }
}

}  // namespace xl

extern "C" int xl_mlstm_step(const xl_mlstm_step_params* p, void* cuda_stream) {
  using namespace xl;
  if (!p || !p->q || !p->k || !p->v || !p->h || !p->igate || !p->fgate || !p->c_out || !p->n_out || !p->m_out)
    return XL_ERR_NULL_POINTER;
  const bool any_in = p->c_in || p->n_in || p->m_in, all_in = p->c_in && p->n_in && p->m_in;
  if (any_in && !all_in) return XL_ERR_NULL_POINTER;
  if (all_in && (p->n_in == p->n_out || p->m_in == p->m_out)) return XL_ERR_ALIASING;
  if (p->B <= 0 || p->NH <= 0 || p->DHQK <= 0 || p->DHV <= 0) return XL_ERR_BAD_SHAPE;
  if (p->slot && p->n_slots <= 0) return XL_ERR_BAD_SHAPE;
  if (p->DHV % 4 != 0 || p->DHQK > 4096 || p->NH > 65535 || p->B > 65535) return XL_ERR_BAD_SHAPE;
  if (p->dtype != XL_F32 && p->dtype != XL_BF16) return XL_ERR_BAD_DTYPE;
  const int esz = p->dtype == XL_F32 ? 4 : 2;
  // v is read with one 4-element vector load per thread; C with float4
  if (p->v_sb % 4 || p->v_sh % 4) return XL_ERR_BAD_STRIDE;
  if ((reinterpret_cast<uintptr_t>(p->v) % (4 * esz)) != 0) return XL_ERR_BAD_ALIGNMENT;
  if (!aligned16(p->c_out) || (p->c_in && !aligned16(p->c_in))) return XL_ERR_BAD_ALIGNMENT;

  dim3 grid((p->DHV + STEP_COLS - 1) / STEP_COLS, p->NH, p->B), block(STEP_THREADS);
  const size_t smem = (2 * (size_t)p->DHQK + STEP_WARPS * STEP_COLS) * sizeof(float);
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  if (p->dtype == XL_F32)
    mlstm_step_kernel<float><<<grid, block, smem, st>>>(*p);
  else
    mlstm_step_kernel<__nv_bfloat16><<<grid, block, smem, st>>>(*p);
  return check_launch("xl_mlstm_step");
}
