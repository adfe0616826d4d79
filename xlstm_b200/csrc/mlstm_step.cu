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

// What the fused decode cell does around the step (FUSED = true): the soft cap of the two gate pre-activations in front
// of it, and the per-head norm, its weight and the output gate behind it.  The thread blocks of a head (one per 128
// columns of DHV) then form a cluster and exchange their partial sums through distributed shared memory.
struct StepFused {
  const void* gates_raw; const void* gate_bias; const void* ogate; const void* norm_weight; void* hg;
  long long gr_sb, o_sb, hg_sb;
  float gate_cap, norm_eps;
};

__device__ __forceinline__ float step_block_sum(float v, float* s_scalar, int warp, int lane) {   // all STEP_THREADS threads call
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();   // (s_scalar may still be read from the previous use)
  if (lane == 0) s_scalar[warp] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int w = 0; w < STEP_WARPS; ++w) t += s_scalar[w];
  return t;
}

template <typename T, bool FUSED>
__global__ void __launch_bounds__(STEP_THREADS) mlstm_step_kernel(const xl_mlstm_step_params p, const StepFused fx) {
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
    // (all thread blocks of a head take this branch together: nobody is left waiting in the cluster barriers below)
    if (tid < STEP_COLS && col0 + tid < p.DHV) {
      if constexpr (FUSED) reinterpret_cast<T*>(fx.hg)[b * fx.hg_sb + (long long)head * p.DHV + col0 + tid] = from_float<T>(0.f);   // the norm of a zero row
      else (reinterpret_cast<T*>(p.h) + b * p.h_sb + head * p.h_sh)[col0 + tid] = from_float<T>(0.f);
    }
    if (row >= p.n_slots && tid == 0 && p.status) atomicExch(p.status, 2);
    return;
  }
  const int64_t sidx = row * p.NH + head;

  const T* q = reinterpret_cast<const T*>(p.q) + b * p.q_sb + head * p.q_sh;
  const T* k = reinterpret_cast<const T*>(p.k) + b * p.k_sb + head * p.k_sh;
  const T* v = reinterpret_cast<const T*>(p.v) + b * p.v_sb + head * p.v_sh;

  float ig, fg;
  if constexpr (FUSED) {
    // cap * tanh(x / cap) in fp32 on the projection's output (+ bias, rounded to T as the Linear rounds it)
    const T* gr = reinterpret_cast<const T*>(fx.gates_raw) + b * fx.gr_sb;
    const T* gbias = reinterpret_cast<const T*>(fx.gate_bias);
    float xi = to_float(gr[head]), xf = to_float(gr[p.NH + head]);
    if (gbias) {
      xi = to_float(from_float<T>(xi + to_float(gbias[head])));
      xf = to_float(from_float<T>(xf + to_float(gbias[p.NH + head])));
    }
    ig = fx.gate_cap * tanhf(xi / fx.gate_cap);
    fg = fx.gate_cap * tanhf(xf / fx.gate_cap);
  } else {
    ig = p.igate[b * p.g_sb + head * p.g_sh];
    fg = p.fgate[b * p.g_sb + head * p.g_sh];
  }
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
  const bool owner = tid < STEP_COLS && col0 + tid < DHV;
  float hv = 0.f;
  if (owner) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < STEP_WARPS; ++w) s += s_red[w * STEP_COLS + tid];
    hv = to_float(from_float<T>(s * inv_den));   // the cell's output in its own dtype
  }
  if constexpr (!FUSED) {
    if (owner) (reinterpret_cast<T*>(p.h) + b * p.h_sb + head * p.h_sh)[col0 + tid] = from_float<T>(hv);
  } else {
    // per-head norm over all DHV columns (MultiHeadLayerNorm of xlstm_large/components.py:188-242: mean, then the
    // centred second moment), its weight and the output gate (model.py:435-449), with the eager sequence's rounding.
    // Every block of the head sends its partial sum to every block (itself included) and all meet at a cluster barrier.
    __shared__ float s_stat[2][8];
    const uint32_t rank = cluster_ctarank(), nblk = gridDim.x;
    const float part = step_block_sum(hv, s_scalar, warp, lane);
    if (tid < (int)nblk) st_cluster_f32(mapa_u32(smem_u32(&s_stat[0][rank]), (uint32_t)tid), part);
    cluster_sync_all();
    float mean = 0.f;
    for (uint32_t r = 0; r < nblk; ++r) mean += s_stat[0][r];
    mean /= (float)DHV;
    const float d = owner ? hv - mean : 0.f;
    const float part2 = step_block_sum(d * d, s_scalar, warp, lane);
    if (tid < (int)nblk) st_cluster_f32(mapa_u32(smem_u32(&s_stat[1][rank]), (uint32_t)tid), part2);
    cluster_sync_all();
    float var = 0.f;
    for (uint32_t r = 0; r < nblk; ++r) var += s_stat[1][r];
    const float rstd = rsqrtf(var / (float)DHV + fx.norm_eps);
    if (owner) {
      const long long c = (long long)head * DHV + col0 + tid;
      const float w = to_float(reinterpret_cast<const T*>(fx.norm_weight)[c]);
      const float o = to_float(reinterpret_cast<const T*>(fx.ogate)[b * fx.o_sb + c]);
      const float nw = to_float(from_float<T>(to_float(from_float<T>((hv - mean) * rstd)) * w));
      const float g = to_float(from_float<T>(sigmoid_for<T>(o)));
      reinterpret_cast<T*>(fx.hg)[b * fx.hg_sb + c] = from_float<T>(g * nw);
    }
  }
}

static int validate_step(const xl_mlstm_step_params* p, bool fused) {
  if (!p || !p->q || !p->k || !p->v || !p->c_out || !p->n_out || !p->m_out) return XL_ERR_NULL_POINTER;
  if (!fused && (!p->h || !p->igate || !p->fgate)) return XL_ERR_NULL_POINTER;
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
  return XL_OK;
}

}  // namespace xl

extern "C" int xl_mlstm_step(const xl_mlstm_step_params* p, void* cuda_stream) {
  using namespace xl;
  const int rc = validate_step(p, false);
  if (rc != XL_OK) return rc;
  dim3 grid((p->DHV + STEP_COLS - 1) / STEP_COLS, p->NH, p->B), block(STEP_THREADS);
  const size_t smem = (2 * (size_t)p->DHQK + STEP_WARPS * STEP_COLS) * sizeof(float);
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  const StepFused none = {};
  if (p->dtype == XL_F32)
    mlstm_step_kernel<float, false><<<grid, block, smem, st>>>(*p, none);
  else
    mlstm_step_kernel<__nv_bfloat16, false><<<grid, block, smem, st>>>(*p, none);
  return check_launch("xl_mlstm_step");
}

extern "C" int xl_mlstm_decode_cell(const xl_mlstm_decode_cell_params* f, void* cuda_stream) {
  using namespace xl;
  if (!f) return XL_ERR_NULL_POINTER;
  const xl_mlstm_step_params* p = &f->step;
  const int rc = validate_step(p, true);
  if (rc != XL_OK) return rc;
  if (!f->gates_raw || !f->ogate || !f->norm_weight || !f->hg) return XL_ERR_NULL_POINTER;
  if (!(f->gate_cap > 0.f)) return XL_ERR_BAD_SHAPE;
  const unsigned nblk = (unsigned)((p->DHV + STEP_COLS - 1) / STEP_COLS);
  if (nblk > 8) return XL_ERR_UNSUPPORTED;   // the blocks of a head form one (portable) cluster: DHV <= 1024
  if (f->gr_sb < 2 * p->NH || f->o_sb < (int64_t)p->NH * p->DHV || f->hg_sb < (int64_t)p->NH * p->DHV) return XL_ERR_BAD_STRIDE;
  dim3 grid(nblk, p->NH, p->B), block(STEP_THREADS);
  const size_t smem = (2 * (size_t)p->DHQK + STEP_WARPS * STEP_COLS) * sizeof(float);
  StepFused fx;
  fx.gates_raw = f->gates_raw; fx.gate_bias = f->gate_bias; fx.ogate = f->ogate; fx.norm_weight = f->norm_weight; fx.hg = f->hg;
  fx.gr_sb = f->gr_sb; fx.o_sb = f->o_sb; fx.hg_sb = f->hg_sb;
  fx.gate_cap = f->gate_cap; fx.norm_eps = f->norm_eps;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = static_cast<cudaStream_t>(cuda_stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = nblk; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  if (p->dtype == XL_F32) (void)cudaLaunchKernelEx(&cfg, mlstm_step_kernel<float, true>, *p, fx);
  else (void)cudaLaunchKernelEx(&cfg, mlstm_step_kernel<__nv_bfloat16, true>, *p, fx);
  return check_launch("xl_mlstm_decode_cell");
}
