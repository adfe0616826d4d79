// Shared by the sLSTM forward and backward kernels: the thread mapping constants, the layout of the training
// cache and the small device helpers both use.
#pragma once
#include "common.cuh"

namespace xl {

constexpr int SL_THREADS = 128;         // 4 warps; warp w owns units [8w, 8w+8) of the CTA's 32
constexpr int SL_UNITS = 32;            // hidden units per CTA
constexpr int SL_ROWS = 16;             // batch rows per cluster (mma M)
constexpr int SL_RING = 8;              // Wx prefetch depth in time steps
constexpr int SL_WX_ROW_BYTES = 4 * SL_UNITS * 2 + 16;  // 4 gates x 32 units bf16 + 16 B pad (bank spread)
constexpr int SL_WX_STEP_BYTES = SL_ROWS * SL_WX_ROW_BYTES;
// Training cache: one record per (step, thread): 4 x bf16x2 gates of batch row a (i', raw f, tanh z, sigmoid o), the same
// for row b, h' of rows a and b (bf16x2 each) + 8 B pad, then c'[4], n'[4], m'[4] in fp32 for the thread's four
// (row, unit) pairs.  Records of a CTA are contiguous: [cluster][CTA][step][thread].
constexpr int SL_REC_BYTES = 96;

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
// Bounded wait without back-off: this wait is the per-step latency chain, a sleep would land on it in full.
__device__ __forceinline__ bool sl_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t it = 0; it < (1u << 26); ++it)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
// 4-byte store into (another) CTA's shared memory that adds its 4 bytes to the transaction count of an mbarrier there
__device__ __forceinline__ void st_async_u32(uint32_t addr, uint32_t v, uint32_t remote_bar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];" ::"r"(addr), "r"(v), "r"(remote_bar)
               : "memory");
}
// 16-byte version of the same store
__device__ __forceinline__ void st_async_v4(uint32_t addr, const uint32_t (&v)[4], uint32_t remote_bar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];" ::"r"(addr), "r"(v[0]),
               "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(remote_bar)
               : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float fast_tanh(float x) {
  // 1 - 2/(1+e^{2x}); saturates cleanly for large |x|
  const float e = __expf(2.f * x);
  return 1.f - __fdividef(2.f, 1.f + e);
}
__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fast_logsigmoid(float x) { return fminf(x, 0.f) - __logf(1.f + __expf(-fabsf(x))); }


}  // namespace xl
