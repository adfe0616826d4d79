// mLSTM token-by-token recurrence over a sequence, fp32 arithmetic throughout.
//
// One CTA owns a REC_COLS-wide column slice of one document's C matrix and keeps it in shared memory for
// the whole document: per token it applies  C' = f'C + i' k v^T,  accumulates q~^T C' for its columns,
// updates n and writes h.  Only q,k,v,i,f are read from and h written to global memory per token; the
// state touches HBM once at the start (initial state) and once at the end (final state).
// It serves (a) fp32 models, where the tensor-core chunkwise kernel's bf16 operands would break the 1e-4
// tolerance, (b) head sizes the chunkwise kernel does not cover, and it is the on-device cross-check for
// the chunkwise kernel in the tests.
#include "common.cuh"

namespace xl {

constexpr int REC_THREADS = 256;
constexpr int REC_COLS = 64;                      // C columns per CTA
constexpr int REC_RG = REC_THREADS / REC_COLS;    // row groups (4)

template <typename T>
__global__ void __launch_bounds__(REC_THREADS) mlstm_recurrent_kernel(const xl_mlstm_seq_params p) {
  extern __shared__ __align__(16) float smem[];
  const int DHQK = p.DHQK, DHV = p.DHV;
  float* s_C = smem;                                 // DHQK x REC_COLS
  float* s_n = s_C + (size_t)DHQK * REC_COLS;        // DHQK
  float* s_q = s_n + DHQK;                           // 2 x DHQK (double buffered by token parity)
  float* s_k = s_q + 2 * DHQK;                       // 2 x DHQK
  float* s_part = s_k + 2 * DHQK;                    // REC_RG x REC_COLS
  __shared__ float s_red[REC_THREADS / 32];

  const int doc = blockIdx.z, head = blockIdx.y, col0 = blockIdx.x * REC_COLS;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int c = tid % REC_COLS, rg = tid / REC_COLS;
  const int col = col0 + c;
  const bool col_ok = col < DHV;

  // document -> (batch row, first token, length)
  int64_t tok0, len;
  int b;
  if (p.cu_seqlens) {
    const int64_t s = p.cu_seqlens[doc], e = p.cu_seqlens[doc + 1];
    b = (int)(s / p.S);
    tok0 = s - (int64_t)b * p.S;
    len = e - s;
  } else {
    b = doc; tok0 = 0; len = p.S;
  }
  const T* q = reinterpret_cast<const T*>(p.q) + b * p.q_sb + head * p.q_sh + tok0 * p.q_st;
  const T* k = reinterpret_cast<const T*>(p.k) + b * p.k_sb + head * p.k_sh + tok0 * p.k_st;
  const T* v = reinterpret_cast<const T*>(p.v) + b * p.v_sb + head * p.v_sh + tok0 * p.v_st;
  T* h = reinterpret_cast<T*>(p.h) + b * p.h_sb + head * p.h_sh + tok0 * p.h_st;
  const float* ig = p.igate + b * p.g_sb + head * p.g_sh + tok0 * p.g_st;
  const float* fg = p.fgate + b * p.g_sb + head * p.g_sh + tok0 * p.g_st;
  const int64_t sidx = (int64_t)doc * p.NH + head;

  // initial state
  for (int r = rg; r < DHQK; r += REC_RG)
    s_C[r * REC_COLS + c] = (p.c0 && col_ok) ? p.c0[(sidx * DHQK + r) * DHV + col] : 0.f;
  for (int d = tid; d < DHQK; d += REC_THREADS) s_n[d] = p.n0 ? p.n0[sidx * DHQK + d] : 0.f;
  float m = p.m0 ? p.m0[sidx] : 0.f;
  const float qscale = rsqrtf((float)DHQK);

  // prefetch token 0 into buffer 0
  if (len > 0)
    for (int d = tid; d < DHQK; d += REC_THREADS) {
      s_q[d] = to_float(q[d]) * qscale;
      s_k[d] = to_float(k[d]);
    }
  __syncthreads();

  for (int64_t t = 0; t < len; ++t) {
    const int cur = (int)(t & 1), nxt = cur ^ 1;
    const float* sq = s_q + cur * DHQK;
    const float* sk = s_k + cur * DHQK;
    // issue next token's loads early (registers), store them to the other buffer after the math
    float qn_[2], kn_[2];  // up to 2 elements per thread (DHQK <= 512)
    const bool more = t + 1 < len;
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int d = tid + u * REC_THREADS;
      if (more && d < DHQK) {
        qn_[u] = to_float(q[(t + 1) * p.q_st + d]) * qscale;
        kn_[u] = to_float(k[(t + 1) * p.k_st + d]);
      }
    }
    const float vv = col_ok ? to_float(v[t * p.v_st + col]) : 0.f;
    const float logf = log_sigmoid(fg[t * p.g_st]);
    const float iv = ig[t * p.g_st];
    const float m_new = fmaxf(logf + m, iv);
    const float f_act = expf(logf + m - m_new);
    const float i_act = expf(iv - m_new);

    // column slice update + partial q~^T C'
    float acc = 0.f;
    const float iv_v = i_act * vv;
#pragma unroll 8
    for (int r = rg; r < DHQK; r += REC_RG) {
      const float cn = fmaf(f_act, s_C[r * REC_COLS + c], sk[r] * iv_v);
      s_C[r * REC_COLS + c] = cn;
      acc = fmaf(sq[r], cn, acc);
    }
    s_part[rg * REC_COLS + c] = acc;
    // n update and q~ . n'
    float qn = 0.f;
    for (int d = tid; d < DHQK; d += REC_THREADS) {
      const float nn = fmaf(f_act, s_n[d], i_act * sk[d]);
      s_n[d] = nn;
      qn = fmaf(sq[d], nn, qn);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) qn += __shfl_xor_sync(0xffffffffu, qn, o);
    if (lane == 0) s_red[warp] = qn;
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int d = tid + u * REC_THREADS;
      if (more && d < DHQK) {
        s_q[nxt * DHQK + d] = qn_[u];
        s_k[nxt * DHQK + d] = kn_[u];
      }
    }
    __syncthreads();
    if (tid < REC_COLS && col0 + tid < DHV) {
      float tot = 0.f;
#pragma unroll
      for (int w = 0; w < REC_THREADS / 32; ++w) tot += s_red[w];
      float num = 0.f;
#pragma unroll
      for (int g = 0; g < REC_RG; ++g) num += s_part[g * REC_COLS + tid];
      const float den = fmaxf(fabsf(tot), expf(-m_new)) + p.eps;
      h[t * p.h_st + col0 + tid] = from_float<T>(num / den);
    }
    m = m_new;
    __syncthreads();
  }

  // final state
  for (int r = rg; r < DHQK; r += REC_RG)
    if (col_ok) p.c_out[(sidx * DHQK + r) * DHV + col] = s_C[r * REC_COLS + c];
  if (blockIdx.x == 0) {
    for (int d = tid; d < DHQK; d += REC_THREADS) p.n_out[sidx * DHQK + d] = s_n[d];
    if (tid == 0) p.m_out[sidx] = m;
  }
}

int validate_seq_common(const xl_mlstm_seq_params* p) {
  if (!p || !p->q || !p->k || !p->v || !p->h || !p->igate || !p->fgate || !p->c_out || !p->n_out || !p->m_out)
    return XL_ERR_NULL_POINTER;
  const bool any0 = p->c0 || p->n0 || p->m0, all0 = p->c0 && p->n0 && p->m0;
  if (any0 && !all0) return XL_ERR_NULL_POINTER;
  if (all0 && (p->n0 == p->n_out || p->m0 == p->m_out)) return XL_ERR_ALIASING;
  if (p->B <= 0 || p->NH <= 0 || p->S <= 0 || p->DHQK <= 0 || p->DHV <= 0) return XL_ERR_BAD_SHAPE;
  if (p->cu_seqlens && p->num_docs <= 0) return XL_ERR_BAD_SHAPE;
  if (p->NH > 65535) return XL_ERR_BAD_SHAPE;
  const int nd = p->cu_seqlens ? p->num_docs : p->B;
  if (nd > 65535) return XL_ERR_TOO_LARGE;
  if (p->dtype != XL_F32 && p->dtype != XL_BF16) return XL_ERR_BAD_DTYPE;
  return XL_OK;
}

}  // namespace xl

extern "C" int xl_mlstm_recurrent(const xl_mlstm_seq_params* p, void* cuda_stream) {
  using namespace xl;
  int rc = validate_seq_common(p);
  if (rc != XL_OK) return rc;
  if (p->DHQK > 2 * REC_THREADS) return XL_ERR_BAD_SHAPE;
  const int nd = p->cu_seqlens ? p->num_docs : p->B;
  const size_t smem = ((size_t)p->DHQK * REC_COLS + 5 * (size_t)p->DHQK + REC_RG * REC_COLS) * sizeof(float);
  if (smem > 200 * 1024) return XL_ERR_BAD_SHAPE;
  dim3 grid((p->DHV + REC_COLS - 1) / REC_COLS, p->NH, nd), block(REC_THREADS);
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  if (p->dtype == XL_F32) {
    XL_CUDA_TRY(cudaFuncSetAttribute(mlstm_recurrent_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    mlstm_recurrent_kernel<float><<<grid, block, smem, st>>>(*p);
  } else {
    XL_CUDA_TRY(cudaFuncSetAttribute(mlstm_recurrent_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    mlstm_recurrent_kernel<__nv_bfloat16><<<grid, block, smem, st>>>(*p);
  }
  return check_launch("xl_mlstm_recurrent");
}
