// y = x W^T for a handful of rows of x (one decode step of a few streams): a weight-streaming kernel.
//
// The linear layers of a decode step (xlstm/xlstm_large/model.py:268-277 feed-forward, 383-396 q/k/v/gate projections,
// 443-449 out_proj, 144-151 lm_head) multiply 8 activation rows by matrices of 30-180 MB: the time is the time to read
// the weights once.  Here a thread block owns 16 consecutive output features; its eight warps split the contraction,
// every thread reads 16-byte pieces of two weight rows straight from global memory into `mma.sync.m16n8k16` A fragments
// (the weight tile is the 16-row operand, the activations the 8-column one), partial sums meet in shared memory.  Loading
// 16 contiguous bytes per thread permutes the contraction index inside a 32-wide step; the activation fragment is loaded
// with the same permutation, so the dot products are unchanged.  (tcgen05 is not used on purpose: with M = 8..32 rows the
// tensor pipe is idle either way and a UMMA would want the weights staged in shared memory first.)
#include "common.cuh"

namespace xl {

constexpr int GV_THREADS = 256;   // 8 warps: K is split eight ways
constexpr int GV_ROWS = 16;       // output features per block (MMA M)

__device__ __forceinline__ uint4 ldg_stream16(const void* p) {   // weights: read once, do not keep in L1
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// NT: 8-row tiles of x (M <= 8 NT)
template <int NT>
__global__ void __launch_bounds__(GV_THREADS) decode_gemv_kernel(const xl_gemv_params p) {
  __shared__ float red[GV_THREADS / 32][NT][GV_ROWS][8 + 1];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, tig = lane & 3;
  const int n0 = blockIdx.x * GV_ROWS;
  const __nv_bfloat16* W = reinterpret_cast<const __nv_bfloat16*>(p.w);
  const __nv_bfloat16* X = reinterpret_cast<const __nv_bfloat16*>(p.x);
  const int K = p.K;
  // this thread's two weight rows (clamped: rows past N are computed from row N-1 and never written)
  const int r0 = min(n0 + g, p.N - 1), r1 = min(n0 + g + 8, p.N - 1);
  const __nv_bfloat16* w0 = W + (long long)r0 * p.w_rs + 8 * tig;
  const __nv_bfloat16* w1 = W + (long long)r1 * p.w_rs + 8 * tig;
  // activation rows of this thread's B fragments: row g of every tile (rows past M read row M-1, never written)
  const __nv_bfloat16* xr[NT];
#pragma unroll
  for (int t = 0; t < NT; ++t) xr[t] = X + (long long)min(8 * t + g, p.M - 1) * p.x_rs + 8 * tig;
  // the warp's share of the contraction, in 32-wide steps
  const int steps = (K + 31) / 32;
  const int s_begin = (int)((long long)warp * steps / 8), s_end = (int)((long long)(warp + 1) * steps / 8);
  float acc[NT][4];
#pragma unroll
  for (int t = 0; t < NT; ++t)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[t][i] = 0.f;

  constexpr int UNROLL = 8;
  for (int s0 = s_begin; s0 < s_end; s0 += UNROLL) {
    uint4 a[UNROLL], b[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {   // all weight loads of the batch first: 16 x 16 bytes in flight per thread
      const int k = (s0 + u) * 32;
      const bool in = (s0 + u < s_end) && (k + 8 * tig + 8 <= K);
      a[u] = in ? ldg_stream16(w0 + k) : make_uint4(0u, 0u, 0u, 0u);
      b[u] = in ? ldg_stream16(w1 + k) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int k = (s0 + u) * 32;
      const bool in = (s0 + u < s_end) && (k + 8 * tig + 8 <= K);
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        const uint4 xv = in ? __ldg(reinterpret_cast<const uint4*>(xr[t] + k)) : make_uint4(0u, 0u, 0u, 0u);
        mma_bf16_16816(acc[t], a[u].x, b[u].x, a[u].y, b[u].y, xv.x, xv.y);
        mma_bf16_16816(acc[t], a[u].z, b[u].z, a[u].w, b[u].w, xv.z, xv.w);
      }
    }
  }
  // partial sums of the eight warps meet in shared memory: fragment (row g / g+8, columns 2 tig, 2 tig + 1)
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    red[warp][t][g][2 * tig] = acc[t][0];
    red[warp][t][g][2 * tig + 1] = acc[t][1];
    red[warp][t][g + 8][2 * tig] = acc[t][2];
    red[warp][t][g + 8][2 * tig + 1] = acc[t][3];
  }
  __syncthreads();
  __nv_bfloat16* Y = reinterpret_cast<__nv_bfloat16*>(p.y);
  for (int e = tid; e < NT * 8 * GV_ROWS; e += GV_THREADS) {
    const int m = e / GV_ROWS, r = e % GV_ROWS;   // consecutive threads: consecutive features of one activation row
    if (m < p.M && n0 + r < p.N) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < GV_THREADS / 32; ++w) s += red[w][m >> 3][r][m & 7];
      Y[(long long)m * p.y_rs + n0 + r] = __float2bfloat16_rn(s);
    }
  }
}

}  // namespace xl

extern "C" int xl_decode_gemv(const xl_gemv_params* p, void* cuda_stream) {
  using namespace xl;
  if (!p || !p->x || !p->w || !p->y) return XL_ERR_NULL_POINTER;
  if (p->dtype != XL_BF16) return XL_ERR_BAD_DTYPE;
  if (p->M < 1 || p->N < 1 || p->K < 8) return XL_ERR_BAD_SHAPE;
  if (p->M > 32) return XL_ERR_TOO_LARGE;
  if (p->K % 8 != 0 || p->x_rs % 8 != 0 || p->w_rs % 8 != 0 || p->x_rs < p->K || p->w_rs < p->K || p->y_rs < p->N) return XL_ERR_BAD_STRIDE;
  if (!aligned16(p->x) || !aligned16(p->w)) return XL_ERR_BAD_ALIGNMENT;
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  const unsigned grid = (unsigned)((p->N + GV_ROWS - 1) / GV_ROWS);
  if (p->M <= 8) decode_gemv_kernel<1><<<grid, GV_THREADS, 0, st>>>(*p);
  else if (p->M <= 16) decode_gemv_kernel<2><<<grid, GV_THREADS, 0, st>>>(*p);
  else decode_gemv_kernel<4><<<grid, GV_THREADS, 0, st>>>(*p);
  return check_launch("xl_decode_gemv");
}
