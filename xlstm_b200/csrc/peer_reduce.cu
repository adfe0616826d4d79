// Tensor-parallel decode: all-reduce of the row-parallel projection's partial sums, the residual add and the RMSNorm of
// the next sub-block in ONE kernel over peer memory (NVLink / NVSwitch), in place of an NCCL all-reduce launch followed by
// the add + norm launch.
//
// The partial sums of a decode step are tiny (a few rows of D values), so the all-reduce is pure latency.  One-shot, push
// based: the thread block of row i writes its rank's partial row i into the receive area of EVERY rank (plain peer stores),
// publishes a flag there, then waits until the flags of all ranks for row i have arrived in its OWN receive area, and sums
// the partial rows from local memory in rank order (the same order on every rank: all ranks get the same bits), adds the
// residual and normalises -- the arithmetic of xl_add_rmsnorm with y = the reduced sum (reference:
// xlstm/xlstm_large/model.py:499-510, components.py:70-97; the reference itself has no tensor parallelism).
//
// Ordering.  Every row keeps an epoch counter in this rank's memory; call number e of a row uses receive buffer e & 1 and
// the flag value e + 1 (never zero, so zero-initialised flags match nothing).  A rank can be at most one call ahead of a
// peer on a row (to finish call e + 1 it needs the peer's push of call e + 1, which the peer issues only after it has
// finished reading call e), so two buffers are enough and nothing is ever cleared.  Writes: data, then
// __threadfence_system, then a releasing store of the flag at system scope; the reader acquires the flag at system scope
// before it touches the data.  Every wait is bounded (about two seconds): on expiry the status word is set and the block
// carries on with whatever it has, so a missing peer becomes an error the host sees, never a hang.
#include "common.cuh"

namespace xl {

constexpr int PR_THREADS = 256, PR_MAXC = 4, PR_MAX_WORLD = 8;

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

template <typename T> struct PrVec;
template <> struct PrVec<float> { static constexpr int N = 4; };
template <> struct PrVec<__nv_bfloat16> { static constexpr int N = 8; };

template <typename T, int NC>
__global__ void __launch_bounds__(PR_THREADS) peer_reduce_add_rmsnorm_kernel(const xl_peer_reduce_params p) {
  constexpr int V = PrVec<T>::N;
  __shared__ float s_part[PR_THREADS / 32];
  __shared__ uint32_t s_epoch;
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) s_epoch = p.epoch[row];
  __syncthreads();
  const uint32_t e = s_epoch, want = e + 1u;
  const int par = (int)(e & 1u);
  // receive areas: [2 buffers][world source ranks][rows_max][D] elements; flags: [2][world][rows_max]
  const long long slot = ((long long)par * p.world + p.rank) * p.rows_max + row;   // where MY partial goes on every rank
  const T* mine = static_cast<const T*>(p.partial) + (long long)row * p.partial_sr;

  // ---- push this rank's partial row to every rank (itself included), then the flag
  uint4 pv[NC];
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    const int el = (c * PR_THREADS + tid) * V;
    if (el < p.D) pv[c] = *reinterpret_cast<const uint4*>(mine + el);
  }
  for (int r = 0; r < p.world; ++r) {
    T* dst = static_cast<T*>(p.peer_recv[r]) + slot * p.D;
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      const int el = (c * PR_THREADS + tid) * V;
      if (el < p.D) *reinterpret_cast<uint4*>(dst + el) = pv[c];
    }
  }
  __threadfence_system();
  __syncthreads();
  if (tid < p.world) st_release_sys(p.peer_flags[tid] + slot, want);

  // ---- meanwhile: the residual row and the weights
  const T* x = static_cast<const T*>(p.x) + (long long)row * p.x_sr;
  uint4 xv[NC], wv[NC];
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    const int el = (c * PR_THREADS + tid) * V;
    if (el < p.D) {
      xv[c] = *reinterpret_cast<const uint4*>(x + el);
      wv[c] = *reinterpret_cast<const uint4*>(static_cast<const T*>(p.weight) + el);
    }
  }

  // ---- wait for every rank's row (bounded), thread r polls the flag of source rank r
  bool ok = true;
  if (tid < p.world) {
    const uint32_t* f = p.flags_local + ((long long)par * p.world + tid) * p.rows_max + row;
    const long long t0 = clock64();
    while (ld_acquire_sys(f) != want) {
      if (clock64() - t0 > 4000000000LL) { ok = false; break; }
      __nanosleep(20);
    }
  }
  if (!__syncthreads_and(ok ? 1 : 0) && tid == 0 && p.status) atomicExch(p.status, 3);

  // ---- sum the partial rows in rank order (fp32), add the residual, RMSNorm
  T* xo = static_cast<T*>(p.x_out) + (long long)row * p.xo_sr;
  T* nd = static_cast<T*>(p.normed) + (long long)row * p.n_sr;
  float xs[NC][V];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    const int el = (c * PR_THREADS + tid) * V;
    if (el < p.D) {
      float acc[V];
#pragma unroll
      for (int i = 0; i < V; ++i) acc[i] = 0.f;
      for (int r = 0; r < p.world; ++r) {
        const T* src = static_cast<const T*>(p.recv_local) + (((long long)par * p.world + r) * p.rows_max + row) * p.D + el;
        T v[V];
        *reinterpret_cast<uint4*>(v) = __ldcg(reinterpret_cast<const uint4*>(src));   // L2 only: peers wrote it, L1 may be stale
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] += to_float(v[i]);
      }
      const T* xe = reinterpret_cast<const T*>(&xv[c]);
      T outv[V];
#pragma unroll
      for (int i = 0; i < V; ++i) {
        // the reduced sum is rounded to T (what an all-reduce hands back), then added to the residual and rounded again
        outv[i] = from_float<T>(to_float(xe[i]) + to_float(from_float<T>(acc[i])));
        xs[c][i] = to_float(outv[i]);
        ss = fmaf(xs[c][i], xs[c][i], ss);
      }
      *reinterpret_cast<uint4*>(xo + el) = *reinterpret_cast<const uint4*>(outv);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (lane == 0) s_part[warp] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < PR_THREADS / 32; ++i) tot += s_part[i];
  const float rinv = rsqrtf(tot / (float)p.D + p.eps);
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    const int el = (c * PR_THREADS + tid) * V;
    if (el < p.D) {
      const T* we = reinterpret_cast<const T*>(&wv[c]);
      T outv[V];
#pragma unroll
      for (int i = 0; i < V; ++i) outv[i] = from_float<T>(to_float(from_float<T>(xs[c][i] * rinv)) * to_float(we[i]));
      *reinterpret_cast<uint4*>(nd + el) = *reinterpret_cast<const uint4*>(outv);
    }
  }
  if (tid == 0) p.epoch[row] = want;
}

}  // namespace xl

extern "C" int xl_peer_reduce_add_rmsnorm(const xl_peer_reduce_params* p, void* cuda_stream) {
  using namespace xl;
  if (!p || !p->partial || !p->peer_recv || !p->recv_local || !p->peer_flags || !p->flags_local || !p->epoch || !p->x ||
      !p->weight || !p->x_out || !p->normed)
    return XL_ERR_NULL_POINTER;
  if (p->dtype != XL_F32 && p->dtype != XL_BF16) return XL_ERR_BAD_DTYPE;
  const int V = p->dtype == XL_F32 ? 4 : 8;
  if (p->world < 1 || p->rank < 0 || p->rank >= p->world || p->rows <= 0 || p->D <= 0 || p->D % V != 0) return XL_ERR_BAD_SHAPE;
  if (p->world > PR_MAX_WORLD || p->rows > p->rows_max || p->D > PR_THREADS * PR_MAXC * V) return XL_ERR_TOO_LARGE;
  if (p->partial_sr % V || p->x_sr % V || p->xo_sr % V || p->n_sr % V) return XL_ERR_BAD_STRIDE;
  if (!aligned16(p->partial) || !aligned16(p->recv_local) || !aligned16(p->x) || !aligned16(p->weight) || !aligned16(p->x_out) ||
      !aligned16(p->normed))
    return XL_ERR_BAD_ALIGNMENT;
  if (p->normed == p->x || p->normed == p->x_out) return XL_ERR_ALIASING;
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  const int nc = (p->D + PR_THREADS * V - 1) / (PR_THREADS * V);
#define XL_PR_LAUNCH(T)                                                                                   \
  do {                                                                                                    \
    if (nc <= 1) peer_reduce_add_rmsnorm_kernel<T, 1><<<p->rows, PR_THREADS, 0, st>>>(*p);                  \
    else if (nc <= 2) peer_reduce_add_rmsnorm_kernel<T, 2><<<p->rows, PR_THREADS, 0, st>>>(*p);             \
    else peer_reduce_add_rmsnorm_kernel<T, 4><<<p->rows, PR_THREADS, 0, st>>>(*p);                          \
  } while (0)
  if (p->dtype == XL_F32) XL_PR_LAUNCH(float);
  else XL_PR_LAUNCH(__nv_bfloat16);
#undef XL_PR_LAUNCH
  return check_launch("xl_peer_reduce_add_rmsnorm");
}
