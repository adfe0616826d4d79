// Operators next to the mLSTM cell in the reference's layer, each fused into one pass over its data:
//   xl_add_rmsnorm    residual add + RMSNorm                      (xlstm/xlstm_large/model.py:499-510, components.py:70-97)
//   xl_soft_cap       cap * tanh(x / cap) of gate pre-activations and logits  (components.py:5-22)
//   xl_headnorm_gate  per-head LayerNorm of the cell output read through its (B,NH,S,DH) strides, weight, output gate
//                     (xlstm/xlstm_large/model.py:435-449, components.py:171-242)
//   xl_causal_conv1d  depthwise causal convolution over time + SiLU in front of the sLSTM cell, with document
//                     boundaries (xlstm/components/conv.py:110-129, xlstm/blocks/slstm/layer.py:133-142)
//   xl_swiglu         silu(gate) * up of the feed-forward block (xlstm/xlstm_large/model.py:268-277)
// Both are bound by HBM traffic: every element is read once with 16-byte loads, kept in registers across the
// reduction, and written once.  Rounding points are those of the reference's eager operator sequence (fp32
// reductions; the normalised value rounded to the model dtype, then the weight product rounded, then the gate).
#include "common.cuh"

namespace xl {

constexpr int ADJ_MAXC = 4;  // most 16-byte vectors per thread (kernels are instantiated for 1, 2 and 4)

template <typename T> struct Vec16;
template <> struct Vec16<float> {
  static constexpr int N = 4;
  float v[4];
};
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  __nv_bfloat16 v[8];
};

template <typename T>
__device__ __forceinline__ Vec16<T> load16(const T* p) {
  Vec16<T> r;
  *reinterpret_cast<uint4*>(r.v) = *reinterpret_cast<const uint4*>(p);
  return r;
}
template <typename T>
__device__ __forceinline__ void store16(T* p, const Vec16<T>& r) {
  *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(r.v);
}

// The gate is rounded to T right away: for bf16 the hardware exponential and reciprocal (a few fp32 ulp) are far
// inside the rounding step and keep the kernel on the memory roofline (with expf and an IEEE division the kernel
// was bound by instruction issue: 0.49 ms against 0.25 ms of traffic at the 7B shapes); fp32 keeps the exact forms.
// out = round(round(sigmoid(o)) * round(round((h - mean) * r) * w)), the eager reference's rounding sequence.
__device__ __forceinline__ Vec16<float> normalise_weight_gate(const Vec16<float>& h, const Vec16<float>& o,
                                                              const Vec16<float>& w, float mean, float r) {
  Vec16<float> y;
#pragma unroll
  for (int i = 0; i < 4; ++i) y.v[i] = sigmoid_for<float>(o.v[i]) * (((h.v[i] - mean) * r) * w.v[i]);
  return y;
}
// bf16: two elements per instruction where the hardware has it -- one packed conversion per rounding point and
// packed bf16 multiplies (the product of two bf16 values rounded once, which is what "multiply in fp32, round to
// bf16" gives).  Element by element, with a conversion per rounding, the kernel was bound by instruction issue.
__device__ __forceinline__ Vec16<__nv_bfloat16> normalise_weight_gate(const Vec16<__nv_bfloat16>& h, const Vec16<__nv_bfloat16>& o,
                                                                      const Vec16<__nv_bfloat16>& w, float mean, float r) {
  Vec16<__nv_bfloat16> y;
  const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(h.v);
  const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(o.v);
  const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(w.v);
  __nv_bfloat162* y2 = reinterpret_cast<__nv_bfloat162*>(y.v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 hf = __bfloat1622float2(h2[i]), of = __bfloat1622float2(o2[i]);
    const __nv_bfloat162 nw = __hmul2(__floats2bfloat162_rn((hf.x - mean) * r, (hf.y - mean) * r), w2[i]);
    const __nv_bfloat162 g = __floats2bfloat162_rn(sigmoid_for<__nv_bfloat16>(of.x), sigmoid_for<__nv_bfloat16>(of.y));
    y2[i] = __hmul2(g, nw);
  }
  return y;
}

// Without a gate (o == NULL): out = round((h - mean) * r * w), one rounding, as a group norm computes it
// (F.group_norm in MultiHeadLayerNorm.forward, xlstm/components/ln.py:52-68).
template <typename T>
__device__ __forceinline__ Vec16<T> normalise_weight(const Vec16<T>& h, const Vec16<T>& w, float mean, float r) {
  Vec16<T> y;
#pragma unroll
  for (int i = 0; i < Vec16<T>::N; ++i) y.v[i] = from_float<T>(((to_float(h.v[i]) - mean) * r) * to_float(w.v[i]));
  return y;
}

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

// ------------------------------------------------------------------------------------------------------------
// residual add + RMSNorm: one CTA of 256 threads per row
// ------------------------------------------------------------------------------------------------------------
constexpr int RMS_THREADS = 256;

template <typename T, int NC>
__global__ void __launch_bounds__(RMS_THREADS) add_rmsnorm_kernel(const xl_add_rmsnorm_params p) {
  constexpr int V = Vec16<T>::N;
  __shared__ float s_part[RMS_THREADS / 32];
  const long long row = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const T* x = static_cast<const T*>(p.x) + row * p.x_sr;
  const T* y = p.y ? static_cast<const T*>(p.y) + row * p.y_sr : nullptr;
  const T* w = static_cast<const T*>(p.weight);
  T* xo = p.x_out ? static_cast<T*>(p.x_out) + row * p.xo_sr : nullptr;
  T* nd = static_cast<T*>(p.normed) + row * p.n_sr;

  // every load of the row is issued before the first use (x, y and the weights: up to 12 vectors in flight per thread)
  Vec16<T> xv[NC], yv[NC], wv[NC];
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    const int e = (c * RMS_THREADS + tid) * V;
    if (e < p.D) {
      xv[c] = load16(x + e);
      if (y) yv[c] = load16(y + e);
    }
  }
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    const int e = (c * RMS_THREADS + tid) * V;
    if (e < p.D) wv[c] = load16(w + e);
  }
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    const int e = (c * RMS_THREADS + tid) * V;
    if (e < p.D) {
      if (y) {
#pragma unroll
        for (int i = 0; i < V; ++i) xv[c].v[i] = from_float<T>(to_float(xv[c].v[i]) + to_float(yv[c].v[i]));
        store16(xo + e, xv[c]);
      }
#pragma unroll
      for (int i = 0; i < V; ++i) {
        const float f = to_float(xv[c].v[i]);
        ss = fmaf(f, f, ss);
      }
    }
  }
  ss = warp_sum(ss);
  if (lane == 0) s_part[warp] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < RMS_THREADS / 32; ++i) tot += s_part[i];
  const float r = rsqrtf(tot / (float)p.D + p.eps);
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    const int e = (c * RMS_THREADS + tid) * V;
    if (e < p.D) {
      Vec16<T> o;
#pragma unroll
      for (int i = 0; i < V; ++i)
        o.v[i] = from_float<T>(to_float(from_float<T>(to_float(xv[c].v[i]) * r)) * to_float(wv[c].v[i]));
      store16(nd + e, o);
    }
  }
}

// ------------------------------------------------------------------------------------------------------------
// per-head LayerNorm + weight + output gate: one warp per (batch, token, head)
// ------------------------------------------------------------------------------------------------------------
constexpr int HNG_WARPS = 8;

template <typename T, int NC>
__global__ void __launch_bounds__(HNG_WARPS * 32) headnorm_gate_kernel(const xl_headnorm_gate_params p) {
  constexpr int V = Vec16<T>::N;
  const int lane = threadIdx.x & 31;
  // 32-bit index arithmetic on purpose (grid.y = batch row): with 64-bit divisions for (batch, token, head) the index
  // computation alone was more than half of the warp's instructions
  const unsigned unit = blockIdx.x * HNG_WARPS + (threadIdx.x >> 5);   // (token, head) within the batch row
  if (unit >= (unsigned)p.S * (unsigned)p.NH) return;
  const unsigned s = unit / (unsigned)p.NH, head = unit - s * (unsigned)p.NH;
  const long long b = blockIdx.y;
  const T* h = static_cast<const T*>(p.h) + b * p.h_sb + head * p.h_sh + s * p.h_st;
  const T* o = static_cast<const T*>(p.o) + b * p.o_sb + s * p.o_st + (long long)head * p.DH;
  const T* w = static_cast<const T*>(p.weight) + (long long)head * p.DH;
  T* out = static_cast<T*>(p.out) + ((b * p.S + s) * p.NH + head) * p.DH;

  // every load of the row is issued before the first use
  Vec16<T> hv[NC], ov[NC], wv[NC];
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    const int e = (c * 32 + lane) * V;
    if (e < p.DH) {
      hv[c] = load16(h + e);
      if (p.o) ov[c] = load16(o + e);
      wv[c] = load16(w + e);
    }
  }
  float sum = 0.f;
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    const int e = (c * 32 + lane) * V;
    if (e < p.DH) {
#pragma unroll
      for (int i = 0; i < V; ++i) sum += to_float(hv[c].v[i]);
    }
  }
  const float mean = warp_sum(sum) / (float)p.DH;
  float sq = 0.f;
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    const int e = (c * 32 + lane) * V;
    if (e < p.DH) {
#pragma unroll
      for (int i = 0; i < V; ++i) {
        const float d = to_float(hv[c].v[i]) - mean;
        sq = fmaf(d, d, sq);
      }
    }
  }
  const float r = rsqrtf(warp_sum(sq) / (float)p.DH + p.eps);
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    const int e = (c * 32 + lane) * V;
    if (e < p.DH) {
      store16(out + e, p.o ? normalise_weight_gate(hv[c], ov[c], wv[c], mean, r) : normalise_weight<T>(hv[c], wv[c], mean, r));
    }
  }
}

// ------------------------------------------------------------------------------------------------------------
// soft cap: cap * tanh(x / cap), each operator's result rounded to T
// ------------------------------------------------------------------------------------------------------------
template <typename T, typename O, bool ROUND_EACH>
__global__ void __launch_bounds__(256) soft_cap_kernel(const T* __restrict__ x, O* __restrict__ out, long long n, float cap,
                                                       long long cols, long long x_row_stride, const T* __restrict__ bias) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    // (rows of `cols` elements `x_row_stride` apart: a column slice of a wider projection output; a bias per column is
    // added first, rounded to T as the reference's Linear rounds its output)
    float v;
    if (cols > 0) {
      const long long r = i / cols, c = i - r * cols;
      v = to_float(x[r * x_row_stride + c]);
      if (bias) v = to_float(from_float<T>(v + to_float(bias[c])));
    } else {
      v = to_float(x[i]);
    }
    if (ROUND_EACH) {
      const T q = from_float<T>(v / cap);
      const T t = from_float<T>(tanhf(to_float(q)));
      out[i] = from_float<O>(to_float(from_float<T>(cap * to_float(t))));
    } else {
      out[i] = from_float<O>(cap * tanhf(v / cap));
    }
  }
}

// ---------------------------------------------------------------------------------------------
// SwiGLU: out[r, j] = round(round(silu(gz[r, j])) * gz[r, F + j]) -- the eager sequence of the reference's feed-forward
// (act_fn(proj_up_gate(x)) * proj_up(x), xlstm/xlstm_large/model.py:268-277) on the output of the fused up-projection.
// One pass: reads 2F, writes F per row.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) swiglu_kernel(const T* __restrict__ gz, T* __restrict__ out, long long rows, int F,
                                                     long long gz_row_stride) {
  constexpr int V = Vec16<T>::N;
  const long long nvec = rows * (long long)(F / V), stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    const long long r = i / (F / V);
    const int c = (int)(i - r * (F / V)) * V;
    const Vec16<T> g = load16(gz + r * gz_row_stride + c), z = load16(gz + r * gz_row_stride + F + c);
    Vec16<T> o;
#pragma unroll
    for (int k = 0; k < V; ++k) {
      const float gv = to_float(g.v[k]);
      const float sl = to_float(from_float<T>(gv * sigmoid_for<T>(gv)));
      o.v[k] = from_float<T>(sl * to_float(z.v[k]));
    }
    store16(out + r * (long long)F + c, o);
  }
}

// ---------------------------------------------------------------------------------------------
// Depthwise causal convolution over time, optional SiLU, document boundaries.
//   y[b,t,f] = bias[f] + sum_{lag=0}^{K-1} w[f][K-1-lag] x[b,t-lag,f]      (taps that reach in front of the first token of
//   the document -- or of the row -- read zero), out = silu(round(y)).
// A thread owns one 16-byte vector of features and walks CONV_TILE consecutive tokens with the last K-1 inputs in
// registers, so x is read once (plus a K-1 token halo per tile) and out written once: HBM-bound.
// ---------------------------------------------------------------------------------------------
constexpr int CONV_THREADS = 128, CONV_TILE = 64, CONV_MAXK = 8;

template <typename T>
__global__ void __launch_bounds__(CONV_THREADS) causal_conv1d_kernel(const xl_conv1d_params p) {
  constexpr int V = Vec16<T>::N;
  const int f0 = (blockIdx.x * CONV_THREADS + threadIdx.x) * V;
  if (f0 >= p.F) return;
  const int b = blockIdx.z, K = p.K;
  const int t0 = blockIdx.y * CONV_TILE, t1 = min(p.S, t0 + CONV_TILE);
  const T* x = static_cast<const T*>(p.x) + (long long)b * p.x_sb + f0;
  T* out = static_cast<T*>(p.out) + (long long)b * p.o_sb + f0;
  // weights by lag: wl[l] multiplies x[t-l] (tap K-1-l of the convolution's weight; zero beyond the kernel size, so that
  // every index below is a compile-time constant and the arrays stay in registers); win[l-1] = x[t-l]
  float wl[CONV_MAXK][V], bias[V], win[CONV_MAXK - 1][V];
#pragma unroll
  for (int i = 0; i < V; ++i) {
    bias[i] = p.bias ? to_float(static_cast<const T*>(p.bias)[f0 + i]) : 0.f;
#pragma unroll
    for (int l = 0; l < CONV_MAXK; ++l) wl[l][i] = l < K ? to_float(static_cast<const T*>(p.weight)[(long long)(f0 + i) * K + (K - 1 - l)]) : 0.f;
  }
  // tokens since the first token of the document that holds (b, t0); the next boundary on the flattened axis
  long long since = t0, next_b = 0x7fffffffffffffffLL;
  int idx = 0;
  const long long flat0 = (long long)b * p.S + t0;
  if (p.cu_seqlens) {
    int lo = 0, hi = p.num_docs;   // last offset <= flat0
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if ((long long)p.cu_seqlens[mid] <= flat0) lo = mid; else hi = mid - 1;
    }
    idx = lo;
    since = flat0 - (long long)p.cu_seqlens[idx];
    if (since > t0) since = t0;   // a row start is a start whatever the offsets say
    next_b = idx + 1 <= p.num_docs ? (long long)p.cu_seqlens[idx + 1] : next_b;
  }
#pragma unroll
  for (int l = 1; l < CONV_MAXK; ++l) {
    const int t = t0 - l;
    Vec16<T> v;
#pragma unroll
    for (int i = 0; i < V; ++i) v.v[i] = from_float<T>(0.f);
    if (l < K && t >= 0) v = load16(x + (long long)t * p.x_st);
#pragma unroll
    for (int i = 0; i < V; ++i) win[l - 1][i] = to_float(v.v[i]);
  }
  for (int t = t0; t < t1; ++t) {
    const long long flat = (long long)b * p.S + t;
    while (flat >= next_b) {   // a document starts here (empty documents are stepped over)
      since = flat - next_b;
      ++idx;
      next_b = idx + 1 <= p.num_docs ? (long long)p.cu_seqlens[idx + 1] : 0x7fffffffffffffffLL;
    }
    const Vec16<T> cur = load16(x + (long long)t * p.x_st);
    Vec16<T> o;
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const float c = to_float(cur.v[i]);
      float acc = bias[i];
      acc = fmaf(wl[0][i], c, acc);
#pragma unroll
      for (int l = 1; l < CONV_MAXK; ++l)
        if (l <= since) acc = fmaf(wl[l][i], win[l - 1][i], acc);
      float y = to_float(from_float<T>(acc));            // the convolution's output is rounded to T ...
      if (p.act) y = y * sigmoid_for<T>(y);               // ... before the activation
      o.v[i] = from_float<T>(y);
#pragma unroll
      for (int l = CONV_MAXK - 1; l >= 2; --l) win[l - 1][i] = win[l - 2][i];
      win[0][i] = c;
    }
    store16(out + (long long)t * p.o_st, o);
    ++since;
  }
}

}  // namespace xl

extern "C" int xl_add_rmsnorm(const xl_add_rmsnorm_params* p, void* cuda_stream) {
  using namespace xl;
  if (!p || !p->x || !p->weight || !p->normed) return XL_ERR_NULL_POINTER;
  if (p->y && !p->x_out) return XL_ERR_NULL_POINTER;
  if (p->dtype != XL_F32 && p->dtype != XL_BF16) return XL_ERR_BAD_DTYPE;
  const int V = p->dtype == XL_F32 ? 4 : 8;
  if (p->rows < 0 || p->D <= 0 || p->D % V != 0) return XL_ERR_BAD_SHAPE;
  if (p->D > RMS_THREADS * ADJ_MAXC * V) return XL_ERR_TOO_LARGE;
  if (p->rows > 0x7fffffffLL) return XL_ERR_TOO_LARGE;
  if (p->x_sr % V || p->n_sr % V || (p->y && (p->y_sr % V || p->xo_sr % V))) return XL_ERR_BAD_STRIDE;
  if (!aligned16(p->x) || !aligned16(p->weight) || !aligned16(p->normed) || (p->y && (!aligned16(p->y) || !aligned16(p->x_out))))
    return XL_ERR_BAD_ALIGNMENT;
  if (p->normed == p->x || (p->y && p->normed == p->x_out)) return XL_ERR_ALIASING;
  if (p->rows == 0) return XL_OK;
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  const int nc = (p->D + RMS_THREADS * V - 1) / (RMS_THREADS * V);
  const unsigned grid = (unsigned)p->rows;
#define XL_RMS_LAUNCH(T)                                                              \
  do {                                                                                \
    if (nc <= 1) add_rmsnorm_kernel<T, 1><<<grid, RMS_THREADS, 0, st>>>(*p);          \
    else if (nc <= 2) add_rmsnorm_kernel<T, 2><<<grid, RMS_THREADS, 0, st>>>(*p);     \
    else add_rmsnorm_kernel<T, 4><<<grid, RMS_THREADS, 0, st>>>(*p);                  \
  } while (0)
  if (p->dtype == XL_F32) XL_RMS_LAUNCH(float);
  else XL_RMS_LAUNCH(__nv_bfloat16);
#undef XL_RMS_LAUNCH
  return check_launch("xl_add_rmsnorm");
}

extern "C" int xl_headnorm_gate(const xl_headnorm_gate_params* p, void* cuda_stream) {
  using namespace xl;
  if (!p || !p->h || !p->weight || !p->out) return XL_ERR_NULL_POINTER;
  if (p->dtype != XL_F32 && p->dtype != XL_BF16) return XL_ERR_BAD_DTYPE;
  const int V = p->dtype == XL_F32 ? 4 : 8;
  if (p->B <= 0 || p->NH <= 0 || p->S <= 0 || p->DH <= 0 || p->DH % V != 0) return XL_ERR_BAD_SHAPE;
  if (p->DH > 32 * ADJ_MAXC * V) return XL_ERR_TOO_LARGE;
  if (p->h_sb % V || p->h_sh % V || p->h_st % V || (p->o && (p->o_sb % V || p->o_st % V))) return XL_ERR_BAD_STRIDE;
  if (!aligned16(p->h) || (p->o && !aligned16(p->o)) || !aligned16(p->weight) || !aligned16(p->out)) return XL_ERR_BAD_ALIGNMENT;
  if (p->out == p->h || p->out == p->o) return XL_ERR_ALIASING;
  const long long per_row = (long long)p->S * p->NH;
  if (per_row > 0x7fffffffLL || p->B > 65535) return XL_ERR_TOO_LARGE;
  const dim3 blocks((unsigned)((per_row + HNG_WARPS - 1) / HNG_WARPS), (unsigned)p->B);
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  const int nc = (p->DH + 32 * V - 1) / (32 * V);
#define XL_HNG_LAUNCH(T)                                                                              \
  do {                                                                                                \
    if (nc <= 1) headnorm_gate_kernel<T, 1><<<blocks, HNG_WARPS * 32, 0, st>>>(*p);         \
    else if (nc <= 2) headnorm_gate_kernel<T, 2><<<blocks, HNG_WARPS * 32, 0, st>>>(*p);    \
    else headnorm_gate_kernel<T, 4><<<blocks, HNG_WARPS * 32, 0, st>>>(*p);                 \
  } while (0)
  if (p->dtype == XL_F32) XL_HNG_LAUNCH(float);
  else XL_HNG_LAUNCH(__nv_bfloat16);
#undef XL_HNG_LAUNCH
  return check_launch("xl_headnorm_gate");
}

extern "C" int xl_soft_cap(const xl_soft_cap_params* p, void* cuda_stream) {
  using namespace xl;
  if (!p || !p->x || !p->out) return XL_ERR_NULL_POINTER;
  if (p->dtype != XL_F32 && p->dtype != XL_BF16) return XL_ERR_BAD_DTYPE;
  if (p->n < 0 || !(p->cap > 0.f) || p->out_f32 < 0 || p->out_f32 > 2) return XL_ERR_BAD_SHAPE;
  if (p->cols < 0 || (p->cols > 0 && (p->n % p->cols != 0 || p->x_row_stride < p->cols))) return XL_ERR_BAD_SHAPE;
  if (p->bias && p->cols <= 0) return XL_ERR_BAD_SHAPE;
  if (p->n == 0) return XL_OK;
  if (p->out == p->x && ((p->dtype == XL_BF16 && p->out_f32) || (p->cols > 0 && p->x_row_stride != p->cols))) return XL_ERR_ALIASING;
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  const long long want = (p->n + 255) / 256;
  const unsigned grid = (unsigned)(want < 148 * 16 ? want : 148 * 16);
  const long long cols = p->cols, rs = p->x_row_stride;
  if (p->dtype == XL_F32)
    soft_cap_kernel<float, float, false><<<grid, 256, 0, st>>>(static_cast<const float*>(p->x), static_cast<float*>(p->out), p->n, p->cap, cols, rs, static_cast<const float*>(p->bias));
  else if (p->out_f32 == 2)
    soft_cap_kernel<__nv_bfloat16, float, false><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(p->x), static_cast<float*>(p->out), p->n, p->cap, cols, rs, static_cast<const __nv_bfloat16*>(p->bias));
  else if (p->out_f32)
    soft_cap_kernel<__nv_bfloat16, float, true><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(p->x), static_cast<float*>(p->out), p->n, p->cap, cols, rs, static_cast<const __nv_bfloat16*>(p->bias));
  else
    soft_cap_kernel<__nv_bfloat16, __nv_bfloat16, true><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(p->x), static_cast<__nv_bfloat16*>(p->out), p->n, p->cap, cols, rs, static_cast<const __nv_bfloat16*>(p->bias));
  return check_launch("xl_soft_cap");
}

extern "C" int xl_swiglu(const xl_swiglu_params* p, void* cuda_stream) {
  using namespace xl;
  if (!p || !p->gz || !p->out) return XL_ERR_NULL_POINTER;
  if (p->dtype != XL_F32 && p->dtype != XL_BF16) return XL_ERR_BAD_DTYPE;
  const int V = p->dtype == XL_F32 ? 4 : 8;
  if (p->rows < 0 || p->F <= 0 || p->F % V != 0 || p->gz_row_stride < 2LL * p->F || p->gz_row_stride % V != 0) return XL_ERR_BAD_SHAPE;
  if (!aligned16(p->gz) || !aligned16(p->out)) return XL_ERR_BAD_ALIGNMENT;
  if (p->out == p->gz) return XL_ERR_ALIASING;
  if (p->rows == 0) return XL_OK;
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  const long long want = (p->rows * (long long)(p->F / V) + 255) / 256;
  const unsigned grid = (unsigned)(want < 148 * 16 ? want : 148 * 16);
  if (p->dtype == XL_F32) swiglu_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(p->gz), static_cast<float*>(p->out), p->rows, p->F, p->gz_row_stride);
  else swiglu_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(p->gz), static_cast<__nv_bfloat16*>(p->out), p->rows, p->F, p->gz_row_stride);
  return check_launch("xl_swiglu");
}

extern "C" int xl_causal_conv1d(const xl_conv1d_params* p, void* cuda_stream) {
  using namespace xl;
  if (!p || !p->x || !p->weight || !p->out) return XL_ERR_NULL_POINTER;
  if (p->dtype != XL_F32 && p->dtype != XL_BF16) return XL_ERR_BAD_DTYPE;
  const int V = p->dtype == XL_F32 ? 4 : 8;
  if (p->B <= 0 || p->S <= 0 || p->F <= 0 || p->F % V != 0 || p->K < 1) return XL_ERR_BAD_SHAPE;
  if (p->K > CONV_MAXK || p->B > 65535) return XL_ERR_TOO_LARGE;
  if (p->cu_seqlens && p->num_docs <= 0) return XL_ERR_BAD_SHAPE;
  if (p->x_sb % V || p->x_st % V || p->o_sb % V || p->o_st % V || p->x_st < p->F || p->o_st < p->F) return XL_ERR_BAD_STRIDE;
  if (!aligned16(p->x) || !aligned16(p->out)) return XL_ERR_BAD_ALIGNMENT;
  if (p->out == p->x) return XL_ERR_ALIASING;   // a tile's halo is read by the neighbouring thread block
  const dim3 grid((unsigned)((p->F / V + CONV_THREADS - 1) / CONV_THREADS), (unsigned)((p->S + CONV_TILE - 1) / CONV_TILE), (unsigned)p->B);
  if (grid.y > 65535) return XL_ERR_TOO_LARGE;
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  if (p->dtype == XL_F32) causal_conv1d_kernel<float><<<grid, CONV_THREADS, 0, st>>>(*p);
  else causal_conv1d_kernel<__nv_bfloat16><<<grid, CONV_THREADS, 0, st>>>(*p);
  return check_launch("xl_causal_conv1d");
}
