/*
 * xlstm_b200 -- C ABI of the sm_100a recurrent-cell kernels for xLSTM.
 *
 * Every entry point takes plain device pointers, sizes and element strides,
 * validates them on the host, enqueues its kernels on the given CUDA stream
 * and returns immediately: 0 on success, a negative xl_status otherwise
 * (nothing is launched when a negative code is returned).  No entry point
 * synchronises, allocates or frees device memory.
 *
 * Conventions shared by all mLSTM entry points
 *   - q,k are (B, NH, S, DHQK), v and h are (B, NH, S, DHV); the innermost
 *     dimension is contiguous, the other three are given as ELEMENT strides,
 *     so the transposed views the reference's layer produces
 *     (xlstm/xlstm_large/model.py:415-419) are consumed without a copy.
 *   - gate pre-activations are fp32 (B, NH, S) with element strides.
 *   - states are fp32 and contiguous: C (N, NH, DHQK, DHV), n (N, NH, DHQK),
 *     m (N, NH); an absent initial state means C = 0, n = 0, m = 0
 *     (xlstm/blocks/mlstm/backends.py:185-194).
 *   - the 1/sqrt(DHQK) factor is applied to q; C and n hold un-scaled keys
 *     (xlstm/blocks/mlstm/backends.py:168).  This is the convention of the third-party mlstm_kernels package
 *     the reference's xLSTM-Large model calls; the older step function recurrent_step_stabilized_simple
 *     (xlstm/blocks/mlstm/backends.py:134-137) scales k instead, so its C and n differ from these by sqrt(DHQK)
 *     and states are NOT interchangeable with xlstm.blocks.mlstm step states.
 *   - packed ragged batches: cu_seqlens (device, int32, num_docs + 1 entries)
 *     lists document boundaries on the flattened (B * S) token axis; a
 *     document must not straddle two rows.  Every document starts from the
 *     zero state (or its own row of the initial-state arrays) and leaves its
 *     own final state; states then have N = num_docs rows.  Without
 *     cu_seqlens every batch row is one document and N = B.
 */
#ifndef XLSTM_B200_H
#define XLSTM_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum xl_status {
  XL_OK = 0,
  XL_ERR_NULL_POINTER = -1,
  XL_ERR_BAD_SHAPE = -2,       /* a dimension is zero/negative or not supported by the kernel */
  XL_ERR_BAD_STRIDE = -3,      /* stride not compatible with 16-byte vector / TMA access */
  XL_ERR_BAD_ALIGNMENT = -4,   /* base pointer not 16-byte aligned */
  XL_ERR_BAD_DTYPE = -5,
  XL_ERR_UNSUPPORTED = -6,     /* valid request, but not by this entry point (use the one named in the docs) */
  XL_ERR_CUDA = -7,            /* a CUDA runtime/driver call failed; see xl_last_cuda_error() */
  XL_ERR_TOO_LARGE = -8,       /* exceeds a fixed capacity of the entry point */
  XL_ERR_ALIASING = -9         /* an output overlaps an input that other thread blocks still read */
} xl_status;

typedef enum xl_dtype { XL_F32 = 0, XL_BF16 = 1 } xl_dtype;

/* Human-readable text for a status code (never NULL). */
const char* xl_strerror(int status);
/* Text of the last CUDA error seen by this library on the calling thread ("" if none). */
const char* xl_last_cuda_error(void);
/* ABI version of this header; bumped on any incompatible change. */
int xl_abi_version(void);

/* ------------------------------------------------------------------------------------------------
 * mLSTM over a sequence (prefill).
 * Replaces the kernels the reference selects through mLSTMBackendConfig.chunkwise_kernel and
 * .sequence_kernel (xlstm/xlstm_large/model.py:56-64, call site model.py:425-434); arithmetic as in
 * xlstm/blocks/mlstm/backends.py:149-263.
 * ---------------------------------------------------------------------------------------------- */
typedef struct xl_mlstm_seq_params {
  const void* q; const void* k; const void* v;  /* dtype `dtype` */
  void* h;                                      /* out, dtype `dtype` */
  const float* igate; const float* fgate;       /* pre-activations */
  const float* c0; const float* n0; const float* m0;   /* all three NULL, or all three set */
  float* c_out; float* n_out; float* m_out;     /* final state per document; c_out may alias c0, but n_out and
                                                   m_out must not alias n0/m0 (several thread blocks read those) */
  const int32_t* cu_seqlens;                    /* device pointer or NULL */
  int32_t* status;                              /* device word, or NULL: set non-zero if a bounded wait expired */
  int32_t B, NH, S, DHQK, DHV;
  int32_t num_docs;                             /* used only with cu_seqlens */
  int64_t q_sb, q_sh, q_st;                     /* element strides: batch, head, token */
  int64_t k_sb, k_sh, k_st;
  int64_t v_sb, v_sh, v_st;
  int64_t h_sb, h_sh, h_st;
  int64_t g_sb, g_sh, g_st;                     /* shared by igate and fgate */
  float eps;                                    /* normaliser epsilon (reference default 1e-6) */
  int32_t dtype;                                /* xl_dtype of q,k,v,h */
} xl_mlstm_seq_params;

/* Chunkwise-parallel form on tcgen05 tensor cores (TMA-fed, C state resident in tensor memory).
 * Requires dtype = XL_BF16, DHQK in {64,128,256}, DHV a multiple of 128, strides that are multiples
 * of 8 elements and 16-byte aligned bases.  Any S >= 1 and any document lengths: a trailing partial
 * chunk is handled inside the kernel, so the same call also covers what the reference hands to its
 * sequence kernel.  Returns XL_ERR_UNSUPPORTED for other shapes (use xl_mlstm_recurrent). */
int xl_mlstm_chunkwise(const xl_mlstm_seq_params* p, void* cuda_stream);

/* Token-by-token recurrence with the C state held on chip (exact fp32 arithmetic; the reference's
 * `native_sequence__native` contract).  dtype XL_F32 or XL_BF16, any DHQK <= 512, any DHV. */
int xl_mlstm_recurrent(const xl_mlstm_seq_params* p, void* cuda_stream);

/* ------------------------------------------------------------------------------------------------
 * mLSTM single-token step (decode).  Replaces the kernel selected by mLSTMBackendConfig.step_kernel
 * (xlstm/xlstm_large/model.py:65-68); arithmetic as in xlstm/blocks/mlstm/backends.py:93-146 with the
 * scale moved to q.  One pass over C: read, update, reduce against q, write.
 * ---------------------------------------------------------------------------------------------- */
typedef struct xl_mlstm_step_params {
  const void* q; const void* k; const void* v;  /* (B, NH, DHQK|DHV), dtype `dtype` */
  void* h;                                      /* out (B, NH, DHV) */
  const float* igate; const float* fgate;       /* (B, NH) */
  const float* c_in; const float* n_in; const float* m_in;  /* state pool (NSLOT, NH, ...) */
  float* c_out; float* n_out; float* m_out;     /* c_out may alias c_in (in-place update of the large state);
                                                   n_out/m_out must not alias n_in/m_in */
  const int32_t* slot;                          /* device (B) row of the pool per stream, or NULL = identity.
                                                   slot[b] < 0: stream b is inactive (its pool rows are not touched, its
                                                   h is zero).  slot[b] >= n_slots: skipped likewise and *status = 2.
                                                   Two active streams must not name the same row (they would race). */
  int32_t* status;                              /* device word or NULL */
  int32_t B, NH, DHQK, DHV;
  int32_t n_slots;                              /* rows of the state pool; used only with `slot` */
  int64_t q_sb, q_sh, k_sb, k_sh, v_sb, v_sh, h_sb, h_sh, g_sb, g_sh;
  float eps;
  int32_t dtype;
} xl_mlstm_step_params;

int xl_mlstm_step(const xl_mlstm_step_params* p, void* cuda_stream);

/* One decode step of the mLSTM LAYER's cell part in one kernel: soft cap of the two gate pre-activations
 * (xlstm/xlstm_large/model.py:389-394; fp32 arithmetic on the projection's output + bias), the step above, and behind it
 * the per-head norm, its weight and the output gate (model.py:435-449, components.py:188-242), written as the
 * (B, NH*DHV) input of out_proj.  `step.igate`, `step.fgate` and `step.h` are not used.  The thread blocks of a head
 * exchange the norm's partial sums through distributed shared memory (one cluster per (stream, head)): DHV <= 1024. */
typedef struct xl_mlstm_decode_cell_params {
  xl_mlstm_step_params step;
  const void* gates_raw;    /* (B, 2*NH): input-gate pre-activations of all heads, then forget-gate; row stride gr_sb */
  const void* gate_bias;    /* (2*NH) or NULL */
  const void* ogate;        /* (B, NH*DHV) output-gate pre-activations; row stride o_sb */
  const void* norm_weight;  /* (NH*DHV) */
  void* hg;                 /* out (B, NH*DHV); row stride hg_sb */
  int64_t gr_sb, o_sb, hg_sb;
  float gate_cap, norm_eps;
} xl_mlstm_decode_cell_params;

int xl_mlstm_decode_cell(const xl_mlstm_decode_cell_params* p, void* cuda_stream);

/* ------------------------------------------------------------------------------------------------
 * sLSTM forward over a sequence, one persistent kernel: one thread-block cluster per (head, group of 16 batch
 * rows), each CTA's slice of the recurrent matrix resident in registers as tensor-core fragments, the new h
 * exchanged every time step through asynchronous distributed-shared-memory stores that complete on mbarriers.
 * Replaces sLSTMFunc.forward (xlstm/blocks/slstm/src/cuda/slstm.cc:53-135), i.e. the host loop
 * ForwardPass::Run (slstm_forward.cu:217-267) + SLSTMPointwiseForward (slstm_pointwise.cu:24-116).
 * ---------------------------------------------------------------------------------------------- */
typedef struct xl_slstm_params {
  const void* wx;        /* (B, S, 4, NH, DH) gate pre-activations, gates ordered i,f,z,o; dtype `dtype` */
  const void* R;         /* (NH, DH_in, 4, DH_out) recurrent matrix, dtype `dtype` */
  const float* bias;     /* (NH, 4, DH) */
  const float* state0;   /* (4, B, NH*DH) ordered h,c,n,m; or NULL = zeros */
  void* h_out;           /* (B, NH, S, DH), dtype `dtype` */
  float* state_out;      /* (4, B, NH*DH) final state */
  const int32_t* cu_seqlens;  /* device, or NULL; boundaries on the flattened (B*S) axis reset h,c,n,m */
  int32_t* status;
  int32_t B, S, NH, DH;
  int32_t num_docs;
  int32_t dtype;
  void* train_cache;     /* NULL for inference.  Training: xl_slstm_cache_bytes(B,S,NH,DH) bytes, 16-byte aligned, that the
                            forward fills with what xl_slstm_backward needs (activated gates and states of every step; the
                            reference's `states` and gate caches, slstm.cc:88-101).  Not with cu_seqlens. */
} xl_slstm_params;

/* Requires DH in {64,128,256}; any B (batch rows are tiled into groups of 16), dtype XL_BF16. */
int xl_slstm_forward(const xl_slstm_params* p, void* cuda_stream);

/* Size of the training cache of one forward call (0 for unsupported shapes).  Host only, no CUDA call. */
int64_t xl_slstm_cache_bytes(int32_t B, int32_t S, int32_t NH, int32_t DH);

/* sLSTM backward through time, one persistent kernel with the forward's mapping.  Replaces sLSTMFunc.backward
 * (xlstm/blocks/slstm/src/cuda/slstm.cc:137-254): the host loop BackwardPass::Run (slstm_backward.cu) and
 * SLSTMPointwiseBackward (slstm_pointwise.cu:118-196).  Per step the gate gradients are formed in registers from the
 * cache, written out as dWx, and carried back through the recurrent matrix (held in registers) with a reduce-scatter
 * between the CTAs of a cluster.  The stabiliser state m gets no gradient (dstate0[3] = 0), as in the reference.
 * The gradients of R and of the bias are sums over (b,t) of h_{t-1} (x) dWx_t and of dWx_t -- plain matrix products
 * over this kernel's output that the caller's GEMM library forms (the reference does the same after its loop). */
typedef struct xl_slstm_bwd_params {
  const void* cache;        /* written by xl_slstm_forward with train_cache set, same B,S,NH,DH */
  const void* R;            /* (NH, DH_in, 4, DH_out), dtype `dtype` */
  const void* dh;           /* (B, NH, S, DH) gradient of the forward's h_out, dtype `dtype` */
  const float* dstate_out;  /* (4, B, NH*DH) gradient of the forward's final state (entry 3, m, is ignored), or NULL */
  const float* state0;      /* the forward's initial state, or NULL = zeros */
  void* dwx;                /* out (B, S, 4, NH, DH), dtype `dtype`: gradient of wx (= of the gate pre-activations) */
  float* dstate0;           /* out (4, B, NH*DH): gradient of the initial state */
  int32_t* status;
  int32_t B, S, NH, DH;
  int32_t dtype;
} xl_slstm_bwd_params;

/* Requires DH in {64,128,256}, dtype XL_BF16; no document offsets. */
int xl_slstm_backward(const xl_slstm_bwd_params* p, void* cuda_stream);

/* ------------------------------------------------------------------------------------------------
 * Operators next to the mLSTM cell in the reference's layer (xlstm/xlstm_large/model.py:379-452), each one pass
 * over its data.  Rounding follows the reference's eager sequence: reductions in fp32, the normalised value is
 * rounded to `dtype`, multiplied by the weight and rounded again (components.py:58-63, 86-97, 171-185); the gate is rounded after
 * the sigmoid and after the product (model.py:445-449).
 * ---------------------------------------------------------------------------------------------- */

/* x_out = x + y (rounded to dtype; skipped when y is NULL), normed = RMSNorm(x_out) * weight.
 * Replaces `x = x + block_out` followed by RMSNorm.forward (components.py:70-97; model.py:499-510). */
typedef struct xl_add_rmsnorm_params {
  const void* x;       /* (rows, D), row stride x_sr elements */
  const void* y;       /* (rows, D) contiguous rows with stride y_sr, or NULL */
  const void* weight;  /* (D) */
  void* x_out;         /* (rows, D) stride xo_sr; may alias x; NULL allowed when y is NULL */
  void* normed;        /* (rows, D) stride n_sr */
  int64_t rows; int32_t D;
  int64_t x_sr, y_sr, xo_sr, n_sr;
  float eps;
  int32_t dtype;
} xl_add_rmsnorm_params;

/* Requires D a multiple of the 16-byte vector (8 bf16 / 4 fp32) and D <= 8192 (bf16) / 4096 (fp32). */
int xl_add_rmsnorm(const xl_add_rmsnorm_params* p, void* cuda_stream);

/* out[b, s, head*DH + d] = sigmoid(o[b, s, head*DH + d]) * (LayerNorm_d(h[b, head, s, :]) * weight[head*DH + d]).
 * Replaces MultiHeadLayerNorm.forward on the transposed cell output (components.py:188-242; model.py:435-444) and the
 * output gate (model.py:445-449); h is read through its strides, so the cell's (B, NH, S, DH) output needs no
 * transpose copy. */
typedef struct xl_headnorm_gate_params {
  const void* h;       /* (B, NH, S, DH) through h_sb, h_sh, h_st (elements); DH contiguous */
  const void* o;       /* gate pre-activations (B, S, NH*DH) through o_sb, o_st; NH*DH contiguous.  NULL = no gate: the
                          kernel then is the group norm behind the sLSTM cell, out = (h - mean) * rstd * weight rounded
                          once (MultiHeadLayerNorm.forward, xlstm/components/ln.py:52-68, called at
                          xlstm/blocks/slstm/layer.py:157; pass weight = 1 + the module's residual weight) */
  const void* weight;  /* (NH*DH) */
  void* out;           /* (B, S, NH*DH) contiguous */
  int32_t B, NH, S, DH;
  int64_t h_sb, h_sh, h_st, o_sb, o_st;
  float eps;
  int32_t dtype;
} xl_headnorm_gate_params;

/* Requires DH a multiple of the 16-byte vector and DH <= 1024 (bf16) / 512 (fp32). */
int xl_headnorm_gate(const xl_headnorm_gate_params* p, void* cuda_stream);

/* out[i] = cap * tanh(x[i] / cap) with the quotient, the tanh and the product each rounded to `dtype`, as the
 * reference's eager soft_cap does (xlstm/xlstm_large/components.py:5-22; gate pre-activations model.py:389-394,
 * 407-409, logits model.py:149-151).  out_f32 = 1 writes the (dtype-rounded) result as fp32, which is what the
 * cell kernels take for the gates; out_f32 = 2 writes fp32 computed in fp32 from the `dtype` input without the
 * intermediate roundings (for callers that keep the gates in fp32 although the model runs in bf16). */
typedef struct xl_soft_cap_params {
  const void* x;   /* n elements, contiguous -- or, with cols > 0, n / cols rows of cols elements x_row_stride apart */
  void* out;       /* n elements (contiguous) of `dtype`, or of fp32 when out_f32 is 1 or 2; may alias x when the types
                      and the layouts agree */
  int64_t n;
  float cap;
  int32_t dtype;
  int32_t out_f32;
  int64_t cols;          /* 0 = x is contiguous */
  int64_t x_row_stride;  /* elements; used with cols > 0: x may be a column slice of a wider projection output */
  const void* bias;      /* (cols) of `dtype` or NULL: added to x first and rounded to `dtype`, as a Linear layer's bias
                            is (the gate projections of model.py:389-394 carry one); needs cols > 0 */
} xl_soft_cap_params;

int xl_soft_cap(const xl_soft_cap_params* p, void* cuda_stream);

/* Depthwise causal convolution over time with optional SiLU, as in front of the sLSTM cell:
 * out[b,t,f] = act(bias[f] + sum_j weight[f][j] * x[b, t - (K-1) + j, f]), taps in front of the first token read zero
 * (CausalConv1d.forward, xlstm/components/conv.py:110-129, with conv_act_fn of xlstm/blocks/slstm/layer.py:133-142).
 * The reference pads per batch row only, so with several documents packed into a row its convolution reaches across
 * their boundaries although the cell behind it restarts there; with cu_seqlens a tap never reaches in front of the
 * first token of its own document.  The convolution is accumulated in fp32 and rounded to `dtype` before the activation,
 * as the reference's two modules do. */
typedef struct xl_conv1d_params {
  const void* x;        /* (B, S, F) through x_sb, x_st (elements); F contiguous */
  const void* weight;   /* (F, K) contiguous: nn.Conv1d(groups=F).weight[:, 0, :] */
  const void* bias;     /* (F) or NULL */
  void* out;            /* (B, S, F) through o_sb, o_st; must not alias x */
  const int32_t* cu_seqlens;  /* device, num_docs + 1 offsets on the flattened (B*S) axis, or NULL */
  int32_t B, S, F, K;   /* K <= 8 */
  int32_t num_docs;
  int32_t act;          /* 0 = none, 1 = SiLU */
  int64_t x_sb, x_st, o_sb, o_st;
  int32_t dtype;
} xl_conv1d_params;

/* Requires F a multiple of the 16-byte vector (8 bf16 / 4 fp32). */
int xl_causal_conv1d(const xl_conv1d_params* p, void* cuda_stream);

/* out[r, j] = silu(gz[r, j]) * gz[r, F + j], the sigmoid-linear unit rounded to `dtype` before the product as the
 * reference's eager `act_fn(proj_up_gate(x)) * proj_up(x)` rounds it (xlstm/xlstm_large/model.py:268-277), on the output
 * of ONE projection that stacks proj_up_gate on proj_up. */
typedef struct xl_swiglu_params {
  const void* gz;        /* (rows, 2F) through gz_row_stride (elements) */
  void* out;             /* (rows, F) contiguous */
  int64_t rows; int32_t F;
  int64_t gz_row_stride;
  int32_t dtype;
} xl_swiglu_params;

int xl_swiglu(const xl_swiglu_params* p, void* cuda_stream);

/* Headwise (block-diagonal) projections of the sLSTM layer, up to four in one launch, written into the cell's input layout:
 *   out[r, s, h, :] = W_s[h] x_{in_sel[s]}[r, h*DH : (h+1)*DH]          W_s: (NH, DH, DH) = LinearHeadwiseExpand.weight
 * replaces `self.fgate(x_conv), self.igate(x_conv), self.zgate(x), self.ogate(x)` and the `torch.cat` behind them
 * (xlstm/blocks/slstm/layer.py:145-154; xlstm/components/linear_headwise.py:75-82, bias=False as the layer builds them).
 * bf16 operands, fp32 accumulation on the tensor cores, one rounding to bf16. */
typedef struct xl_headwise_params {
  const void* x[2];        /* two inputs (rows, NH*DH), row strides x_row_stride[] (elements); x[1] may be NULL if unused */
  const void* w[4];        /* per slot (NH, DH, DH) contiguous, [head][out][in] */
  void* out;               /* (rows, n_slots, NH, DH) through out_row_stride */
  int32_t* status;         /* device word or NULL: set to 1 if a bounded wait inside the kernel expired */
  int32_t in_sel[4];       /* which input slot s reads: 0 or 1 */
  int64_t rows;
  int32_t NH, DH;          /* DH in {64, 128, 256} */
  int32_t n_slots;         /* 1..4 */
  int32_t dtype;           /* XL_BF16 */
  int64_t x_row_stride[2], out_row_stride;   /* multiples of 8 elements */
} xl_headwise_params;

int xl_headwise_proj(const xl_headwise_params* p, void* cuda_stream);

/* ------------------------------------------------------------------------------------------------
 * Tensor-parallel decode: x_out = x + sum over ranks of partial, normed = RMSNorm(x_out) * weight, in ONE kernel over peer
 * memory.  (The reference has no tensor parallelism; this fuses what follows its row-parallel projections
 * out_proj / proj_down, model.py:373-377, 268-277, 499-510, when heads are split over GPUs: the all-reduce of their partial
 * sums, the residual add and the next RMSNorm.)  One thread block per row pushes its rank's partial row into every
 * rank's receive area with plain peer stores, publishes a flag, waits (bounded) for all ranks' flags in its own area and
 * reduces from LOCAL memory in rank order.  Every rank must make the same sequence of calls with the same `rows`.
 * Receive areas and flags must be mapped on every rank (peer access / symmetric memory) and zero-initialised once; no
 * multicast and no library operates on the peer pointers, only this kernel's loads and stores.
 * ---------------------------------------------------------------------------------------------- */
typedef struct xl_peer_reduce_params {
  const void* partial;          /* (rows, D) this rank's partial sums, row stride partial_sr */
  void* const* peer_recv;       /* device array [world]: rank r's receive area as seen from this rank */
  const void* recv_local;       /* this rank's own receive area: [2][world][rows_max][D] elements of `dtype` */
  uint32_t* const* peer_flags;  /* device array [world]: rank r's flag area [2][world][rows_max] */
  const uint32_t* flags_local;
  uint32_t* epoch;              /* (rows_max) per-row call counters in this rank's memory, zero-initialised once */
  const void* x;                /* (rows, D) residual stream, row stride x_sr */
  const void* weight;           /* (D) */
  void* x_out;                  /* (rows, D), stride xo_sr; may alias x */
  void* normed;                 /* (rows, D), stride n_sr */
  int32_t* status;              /* device word or NULL: set to 3 when a peer's rows did not arrive in time */
  int32_t rank, world, rows, D, rows_max;
  int64_t partial_sr, x_sr, xo_sr, n_sr;
  float eps;
  int32_t dtype;
} xl_peer_reduce_params;

/* Requires world <= 8, rows <= rows_max, D a multiple of the 16-byte vector and D <= 8192 (bf16) / 4096 (fp32). */
int xl_peer_reduce_add_rmsnorm(const xl_peer_reduce_params* p, void* cuda_stream);

/* ------------------------------------------------------------------------------------------------
 * Greedy sampling head: tokens[r] = argmax_v soft_cap(logits[r, v]).
 * Replaces the tail of the reference's decode step: the soft cap of the logits (xlstm/xlstm_large/model.py:149-151,
 * components.py:5-22, each operator rounded to `dtype`) and greedy_sampling = torch.argmax of the last position
 * (xlstm/xlstm_large/generate.py:13-15; ties go to the lower index).  Every row is reduced by several thread blocks that
 * meet in `scratch` memory (candidates and a ticket counter per row).
 * ---------------------------------------------------------------------------------------------- */
typedef struct xl_greedy_params {
  const void* logits;     /* (rows, V) un-capped logits, dtype `dtype`, row stride row_stride elements */
  int64_t* tokens;        /* out (rows) */
  void* scratch;          /* device memory, 8-byte aligned, at least xl_softcap_argmax_scratch_bytes(rows) bytes, ZEROED ONCE
                             by the caller; the entry leaves its counters at zero again.  Calls that may overlap on the
                             device need scratch areas of their own. */
  int64_t scratch_bytes;
  int32_t rows, V;
  int64_t row_stride;
  float cap;              /* 30 for the logits of xLSTM-Large */
  int32_t dtype;
} xl_greedy_params;

int64_t xl_softcap_argmax_scratch_bytes(int32_t rows);
int xl_softcap_argmax(const xl_greedy_params* p, void* cuda_stream);

/* The greedy head for callers that cannot hand it scratch memory.  (No counterpart in the reference: its decode loop
 * leaves all device memory to PyTorch's allocator.)
 *
 * xl_softcap_argmax needs a scratch area from its caller.  A caller that runs under a fixed device-memory plan -- a C or
 * C++ serving loop whose buffers were all placed at start-up, a plugin inside a host that owns the GPU's memory, code on
 * a latency path where an allocation (which may synchronise the whole device) is not allowed -- has none to give and may
 * not call cudaMalloc for one.  This entry computes the same tokens from the same `logits` into the same `tokens` and
 * takes its scratch from an array built into the library instead: 270 336 bytes of device memory on every GPU that loads
 * the library, held until the process exits.  `scratch` and `scratch_bytes` of the parameter block are ignored.  It calls
 * no allocating routine (no cudaMalloc / cudaFree, no library that allocates).
 *
 * Limits and rules:
 *   - at most xl_softcap_argmax_noalloc_max_rows() = 1024 rows per call; more returns XL_ERR_TOO_LARGE and launches
 *     nothing (xl_strerror: "request exceeds a fixed capacity of this entry point");
 *   - the device that is current at the call is the one whose array is used; the first call on a device looks the
 *     array's address up (a CUDA runtime query).  Make that first call once during start-up, before any stream capture;
 *   - all calls on one device share the one array.  Calls issued to the same stream, or otherwise ordered on the device,
 *     are safe back to back (each clears the rows it uses first); calls that may OVERLAP on the device race on it --
 *     use xl_softcap_argmax with separate scratch areas for those. */
int32_t xl_softcap_argmax_noalloc_max_rows(void);
int xl_softcap_argmax_noalloc(const xl_greedy_params* p, void* cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* XLSTM_B200_H */
