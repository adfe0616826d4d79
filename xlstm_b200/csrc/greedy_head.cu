// Greedy sampling head: token[r] = argmax over the vocabulary of soft_cap(logits[r, :]).
//
// The reference caps the logits (xlstm/xlstm_large/model.py:149-151, components.py:5-22: cap * tanh(x / cap), quotient,
// tanh and product each rounded to the model dtype) and takes torch.argmax of the last position
// (xlstm/xlstm_large/generate.py:13-15).  Rounding makes ties, and argmax returns the FIRST maximal index, so the capped,
// rounded values are what is compared here, with the lower index winning a tie.
//
// A row of 50 304 logits is too little work for the whole GPU and too much for one thread block when only a handful of
// streams decode: every row is cut into `parts` slices, one thread block each.  A block leaves its (value, index)
// candidate in SCRATCH memory and takes a ticket from the row's counter there; the block that draws the last ticket
// reduces the row's candidates, writes the token and puts the counter back to zero for the next call.
#include "common.cuh"

namespace xl {

constexpr int GH_THREADS = 256, GH_MAX_PARTS = 32;

struct GhCand {
  float val;
  int idx;
};
// Scratch of one row.  Candidates and counter of a row sit together so that the counter of row r is at the same place
// whatever the number of rows of a call: a counter must never land where an earlier call left candidates.
struct GhRow {
  GhCand cand[GH_MAX_PARTS];
  unsigned int counter;
  unsigned int pad;
};

__device__ __forceinline__ bool gh_better(float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); }

template <typename T> __device__ __forceinline__ float gh_capped(T x, float cap) {
  const T q = from_float<T>(to_float(x) / cap);
  const T t = from_float<T>(tanhf(to_float(q)));
  return to_float(from_float<T>(cap * to_float(t)));
}

template <typename T>
__global__ void __launch_bounds__(GH_THREADS) greedy_head_kernel(const xl_greedy_params p, GhRow* __restrict__ scratch) {
  __shared__ GhCand s_c[GH_THREADS / 32];
  __shared__ int s_last;
  const int row = blockIdx.y, part = blockIdx.x, parts = gridDim.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const T* x = static_cast<const T*>(p.logits) + (long long)row * p.row_stride;
  GhRow* mine = scratch + row;
  // slice of this block, in whole 16-byte vectors where the row allows it
  constexpr int V16 = 16 / (int)sizeof(T);
  const bool vec = (p.V % V16 == 0) && (p.row_stride % V16 == 0) && ((reinterpret_cast<uintptr_t>(p.logits) & 15u) == 0);
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  if (vec) {
    const int nvec = p.V / V16, per = (nvec + parts - 1) / parts;
    const int v0 = part * per, v1 = min(nvec, v0 + per);
    for (int v = v0 + tid; v < v1; v += GH_THREADS) {
      T e[V16];
      *reinterpret_cast<uint4*>(e) = *reinterpret_cast<const uint4*>(x + (long long)v * V16);
#pragma unroll
      for (int i = 0; i < V16; ++i) {
        const float y = gh_capped<T>(e[i], p.cap);
        if (gh_better(y, v * V16 + i, bv, bi)) { bv = y; bi = v * V16 + i; }
      }
    }
  } else {
    const int per = (p.V + parts - 1) / parts;
    const int v0 = part * per, v1 = min(p.V, v0 + per);
    for (int v = v0 + tid; v < v1; v += GH_THREADS) {
      const float y = gh_capped<T>(x[v], p.cap);
      if (gh_better(y, v, bv, bi)) { bv = y; bi = v; }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (gh_better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
  }
  if (lane == 0) { s_c[warp].val = bv; s_c[warp].idx = bi; }
  __syncthreads();
  if (tid == 0) {
    for (int w = 1; w < GH_THREADS / 32; ++w)
      if (gh_better(s_c[w].val, s_c[w].idx, bv, bi)) { bv = s_c[w].val; bi = s_c[w].idx; }
    mine->cand[part].val = bv;
    mine->cand[part].idx = bi;
    __threadfence();                                    // the candidate is visible before the ticket is
    s_last = atomicAdd(&mine->counter, 1u) == (unsigned)(parts - 1);
  }
  __syncthreads();
  if (!s_last) return;
  // the last block of the row: reduce the candidates of all parts (parts <= 32: one warp)
  if (warp == 0) {
    __threadfence();
    float v = -INFINITY;
    int i = 0x7fffffff;
    if (lane < parts) {
      const volatile GhCand* c = mine->cand + lane;
      v = c->val; i = c->idx;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oi = __shfl_xor_sync(0xffffffffu, i, o);
      if (gh_better(ov, oi, v, i)) { v = ov; i = oi; }
    }
    if (lane == 0) {
      p.tokens[row] = (long long)(i == 0x7fffffff ? 0 : i);
      mine->counter = 0u;                               // ready for the next call
    }
  }
}

static int gh_parts(int rows) {
  int parts = (2 * 148 + rows - 1) / rows;   // about two blocks per SM in all
  return parts < 1 ? 1 : (parts > GH_MAX_PARTS ? GH_MAX_PARTS : parts);
}

static int gh_validate(const xl_greedy_params* p) {
  if (!p || !p->logits || !p->tokens) return XL_ERR_NULL_POINTER;
  if (p->dtype != XL_F32 && p->dtype != XL_BF16) return XL_ERR_BAD_DTYPE;
  if (p->rows <= 0 || p->V <= 0 || !(p->cap > 0.f) || p->row_stride < p->V) return XL_ERR_BAD_SHAPE;
  if (p->rows > 65535) return XL_ERR_TOO_LARGE;
  return XL_OK;
}

static int gh_launch(const xl_greedy_params* p, GhRow* scratch, cudaStream_t st) {
  const dim3 grid((unsigned)gh_parts(p->rows), (unsigned)p->rows);
  if (p->dtype == XL_F32) greedy_head_kernel<float><<<grid, GH_THREADS, 0, st>>>(*p, scratch);
  else greedy_head_kernel<__nv_bfloat16><<<grid, GH_THREADS, 0, st>>>(*p, scratch);
  return check_launch("xl_softcap_argmax");
}

}  // namespace xl

extern "C" int64_t xl_softcap_argmax_scratch_bytes(int32_t rows) {
  return rows <= 0 ? 0 : (int64_t)rows * (int64_t)sizeof(xl::GhRow);
}

extern "C" int xl_softcap_argmax(const xl_greedy_params* p, void* cuda_stream) {
  using namespace xl;
  int rc = gh_validate(p);
  if (rc != XL_OK) return rc;
  if (!p->scratch) return XL_ERR_NULL_POINTER;
  if (p->scratch_bytes < xl_softcap_argmax_scratch_bytes(p->rows)) return XL_ERR_TOO_LARGE;
  if (reinterpret_cast<uintptr_t>(p->scratch) & 7u) return XL_ERR_BAD_ALIGNMENT;
  return gh_launch(p, static_cast<GhRow*>(p->scratch), static_cast<cudaStream_t>(cuda_stream));
}

// ---------------------------------------------------------------------------------------------
// The same head for callers that cannot allocate device memory.
//
// Its scratch is a file-scope array in device memory, part of the library image: every GPU on which the library is
// loaded holds GH_STATIC_MAX_ROWS * sizeof(GhRow) = 270 336 bytes of it until the process exits.  In host code the name
// of the array is only a stand-in for the symbol, not a device address, so the address is asked for once per device
// (cudaGetSymbolAddress, with that device current) and handed to the kernel like any other scratch pointer.
// ---------------------------------------------------------------------------------------------
namespace xl {

constexpr int GH_STATIC_MAX_ROWS = 1024;
constexpr int GH_MAX_DEVICES = 64;
static __device__ __align__(256) GhRow g_gh_static_scratch[GH_STATIC_MAX_ROWS];
static GhRow* g_gh_static_ptr[GH_MAX_DEVICES];   // device address of the array, per device; filled on first use

}  // namespace xl

extern "C" int32_t xl_softcap_argmax_noalloc_max_rows(void) { return xl::GH_STATIC_MAX_ROWS; }

extern "C" int xl_softcap_argmax_noalloc(const xl_greedy_params* p, void* cuda_stream) {
  using namespace xl;
  int rc = gh_validate(p);
  if (rc != XL_OK) return rc;
  if (p->rows > GH_STATIC_MAX_ROWS) return XL_ERR_TOO_LARGE;   // the built-in scratch holds GH_STATIC_MAX_ROWS rows
  int dev = -1;
  XL_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= GH_MAX_DEVICES) return XL_ERR_TOO_LARGE;
  if (!g_gh_static_ptr[dev]) {   // set-up, once per device, with that device current (it is: cudaGetDevice said so)
    void* sym = nullptr;
    XL_CUDA_TRY(cudaGetSymbolAddress(&sym, g_gh_static_scratch));
    g_gh_static_ptr[dev] = static_cast<GhRow*>(sym);
  }
  GhRow* scratch = g_gh_static_ptr[dev];
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  // The array keeps what the last call left.  A call that ran to its end left the counters at zero, but nothing here
  // relies on that: the rows this call uses are cleared first, in stream order.
  XL_CUDA_TRY(cudaMemsetAsync(scratch, 0, (size_t)p->rows * sizeof(GhRow), st));
  return gh_launch(p, scratch, st);
}
