// mLSTM chunkwise-parallel forward on tcgen05 tensor cores (sm_100a), bf16 operands, fp32 state.
//
// One CTA owns a 128-column slice (of DHV) of one (document, head) and walks that document's 64-token
// chunks in order.  Its slice of the matrix state lives TRANSPOSED in tensor memory for the whole
// document, T[dv, dqk] (128 lanes x DHQK fp32 columns), and is never written to HBM between chunks.
//
// Math per chunk (equivalent to xlstm/blocks/mlstm/backends.py:173-258).  With b_j the in-chunk cumulative
// log forget gate, a'_j = i_j - b_j, mu_j = max(m_prev, max_{l<=j} a'_l), mu* = mu_63, g = b_63:
//   S    = Q K^T                                    P_jl = S_jl/sqrt(DHQK) * exp(a'_l - mu_j)   (l <= j)
//   H_j  = r_j q~_j C_prev + sum_l P_jl v_l          r_j  = exp(m_prev - mu_j)
//   C    = exp(m_prev - mu*) C_prev + sum_l w_l k_l v_l^T ,  n likewise ,   w_l = exp(a'_l - mu*)
//   h_j  = H_j / (max(|r_j q~_j.n_prev + sum_l P_jl|, exp(-(b_j + mu_j))) + eps) ,   m_new = g + mu*
// The decay of C is applied lazily: tensor memory holds T with C = exp(rho) T; rho accumulates the log decay
// and is folded into r_j and w_l, and T is rescaled in place only when rho drops below -30.
//
// Tensor-core work per chunk (all operands bf16, fp32 accumulation in tensor memory):
//   [qn|S] [64 x 72]   = Q [n_hi n_lo 0.. | K]^T    M=64  N=72   K=DHQK  S and the normaliser product q.n in one product:
//                                                                        eight more B rows in front of every k box
//   H^T  [128 x 64]    = Tb q^T                 M=128 N=64   K=DHQK  A = bf16 copy of T in tensor memory
//   H^T               += V^T P^T                M=128 N=64   K=64    A = V tile used MN-major, B = P tile
//   T    [128 x DHQK] += (w V)^T K              M=128 N=DHQK K=64    both MN-major
//   nu   [DHQK x 8]    = K^T [w_hi w_lo]^T      M=64  N=8    K=64    n update, per 64-feature block
// nu lands on the odd 16-lane halves of the S columns (an M=64 accumulator only occupies the even halves).  The 512
// tensor-memory columns are: T 256 | H^T 64 | Tb 128 | S 64, and the eight q.n columns in front of S are the last eight
// columns of Tb, which the two take in turns (see CwLayout).  Every UMMA of these shapes costs the pipe 33-40 cycles
// whatever its N (the four N=256 ones 132): 64 of them per chunk.
//
// Warp roles: warp 14 carries the gate recurrence (scans, r, w, frame) one to two chunks ahead; warps 0-3 gate group
// (q.n and S out of tensor memory with one 16x256b fragment load, P, n and its hi/lo rows, the denominators); warps 4-7
// state group (all but the last block of the T -> bf16 conversion / lazy rescale, w-scaled v, in the exact frame
// r-scaled q in place in its TMA stage); warps 8-11 epilogue group (the last block of the conversion, H^T out as 16x256b
// fragments -> scaled by 1/denominator -> stmatrix.trans into a [token][column] tile -> 16-byte global stores); warp 12
// issues every UMMA; warp 13 issues the TMA loads.  Per chunk the tensor pipe runs phase A (H^T inter), phase B (H^T
// intra interleaved with the T update) and phase C: [qn|S] and nu of the NEXT chunk, which need neither T nor its bf16
// copy and so fill the time the conversion of T takes -- the one long dependency of the loop.  Groups hand work to each
// other through mbarriers only; every wait is bounded, and no waiter is ever more than one phase behind its producer.
//
// Three things about code generation decide the speed of this kernel as much as the schedule does:
//   * the compiler issues an UMMA as ~4 instructions only where it can PROVE warp-uniform control flow: the role
//     dispatch uses a shuffled warp index, the issuing warp calls no non-inlined function (waits are inline) and
//     has no branch inside an issue loop; otherwise every UMMA becomes ~35 instructions and the warp sets the pace;
//   * all roles' per-chunk code together must stay small (rolled loops over pieces, one shared copy of the
//     conversion): unrolled, every pass ran mostly on instruction-fetch misses;
//   * polling warps take issue slots from working ones: waits back off at once;
//   * a load inside a branch waits out its latency there: operands of unrolled, branchy code are fetched up front.
// What the kernel is bound by at the xLSTM-7B head shape is the shared-memory data pipe, which UMMA operand fetches
// (~200 KB per chunk), TMA writes (80 KB) and the groups' own loads and stores share; every step that took bytes off it
// (q.n folded into S, stmatrix instead of 2-byte stores) showed in the time, moving work between groups did not.
//
// q, k, v tiles arrive by TMA (128-byte swizzle) straight from the caller's strided (B, NH, S, D) views;
// documents are chunked from their own first token, so a chunk never straddles a document boundary and the
// tail chunk is masked (i = -inf, log f = 0) instead of padded.
#include <cuda.h>

#include "common.cuh"

namespace xl {

constexpr int CW_L = 64;         // tokens per chunk
constexpr int CW_DV = 128;       // value columns per CTA (UMMA M)
constexpr int CW_THREADS = 480;  // 15 warps, see roles above
constexpr int CW_STAGES = 2;
constexpr int CW_BOX_BYTES = 64 * 128;  // one TMA box: 64 rows x 64 bf16
constexpr uint32_t CW_TMEM_COLS = 512;
constexpr float CW_RESCALE_BELOW = -30.f;  // lazy-decay frame limit (natural log)
constexpr float CW_LOG2E = 1.4426950408889634f;
constexpr float CW_FAST_SPREAD = 30.f;     // largest in-chunk spread of the stabiliser the common-frame path accepts

// Per-chunk gate data published by the scan warp (float offsets into one parity's slot).  Every row j of a chunk
// is computed in a frame exp(-phi_j); h_j = H_j / den_j does not depend on the choice.
//   exact frame  phi_j = mu_j        : q is scaled by r_j in place, P_jl = S_jl e^{a'_l - mu_j}, H^T += V^T P^T
//   common frame phi_j = mu* + rho'  : q stays as loaded, the bf16 copy of T carries the scalar,
//                                      P_jl = S_jl w_l (no exponential per element, no per-row factor)
// The common frame is used whenever mu* - mu_0 <= CW_FAST_SPREAD (rows then differ by at most e^-30 in scale,
// which fp32 accumulators and bf16 operands carry without loss); the exact frame covers chunks in which the
// stabiliser jumps further.  Exact: P_jl = S_jl/sqrt(d) 2^(x_l - y_j); common: P_jl = S_jl z_l; rowsum_j = sum_l P_jl.
enum GateSlot {
  G_LOWER = 0 * CW_L,  // exp(-(b_j + phi_j)): lower bound of the denominator (x sqrt(d) in the common frame)
  G_X = 1 * CW_L,      // x_l (log2 units; -inf for tokens past the end of the document)
  G_Y = 2 * CW_L,      // y_j (log2 units)
  G_R = 3 * CW_L,      // r_j exp(rho) / sqrt(d) (exact frame only)
  G_W = 4 * CW_L,      // w_l = exp(a'_l - mu* - rho')
  G_Z = 5 * CW_L,      // z_l = w_l (common frame)
  G_EPS = 6 * CW_L,    // exp(mu_j - phi_j): eps of the denominator in the row's frame (x sqrt(d) in the common frame)
  G_MULT = 7 * CW_L,   // rescale multiplier of T (1 unless the lazy frame ran out)
  G_RHO = G_MULT + 1,  // rho'
  G_EXACT = G_MULT + 2,  // 1.0 = exact frame
  G_CB = G_MULT + 3,     // scale of the bf16 copy of T
  G_QN = G_MULT + 4,     // scale of the normaliser product
};

enum CwWarp { W_GATE_GROUP = 0, W_STATE_GROUP = 4, W_EPI_GROUP = 8, W_UMMA = 12, W_TMA = 13, W_SCAN = 14 };

enum CwBar {  // mbarrier indices.  Barriers whose producer may run two chunks ahead of a waiter come in pairs
              // indexed by chunk parity (a parity wait is only meaningful one phase back).  A satisfied wait
              // still costs the UMMA warp ~35 cycles and a commit ~40, so everything one phase of UMMAs needs
              // arrives on ONE barrier, whatever group it comes from.
  BAR_FULL0 = 0, BAR_FULL1, BAR_EMPTY0, BAR_EMPTY1,   // TMA stage of q,k,v: landed / consumed
  BAR_GFULL0, BAR_GFULL1, BAR_GEMPTY0, BAR_GEMPTY1,   // gate data of a chunk: published / consumed
  BAR_A,     // phase A may issue: bf16 copy of T (state group's blocks), q final (state group), H^T drained
             // (epilogue group), the last block of the bf16 copy (epilogue group): 4 x 128 arrivals
  BAR_B,     // phase B may issue: P (gate group), w-scaled v (state group): 2 x 128 arrivals
  BAR_C2,    // phase C may issue (gate group): n rows of the next chunk published, nu columns read, gate data of the
             // next chunk visible.  Completion k+1 comes from the gate group's iteration k.
  BAR_HC,    // commit after phase B: H^T and T complete
  BAR_S,     // commit inside phase C: [qn|S] of the next chunk complete (completion k = S(k))
  BAR_NU,    // commit after phase C: nu of the next chunk complete (completion k = nu(k))
  BAR_INV,   // gate group -> epilogue group: 1/denominator published
  BAR_EGDONE,  // epilogue group -> gate group: 1/denominator consumed
  BAR_QNREAD,  // gate group -> epilogue group: q.n of a chunk is in registers (its columns may take the bf16 copy again)
  BAR_TINIT,   // state group -> epilogue group: the initial state is in tensor memory
  BAR_COUNT
};

template <int DHQK>
struct CwLayout {
  static constexpr int NKB = DHQK / 64;                       // 64-wide boxes along DHQK
  static constexpr int Q_BYTES = NKB * CW_BOX_BYTES;
  // k: 1 KiB in FRONT of every 64-feature box holds eight more rows for the S product, [n_hi; n_lo; 0 x 6] of that
  // feature block: S and the normaliser product q.n come out of ONE UMMA with N = 72 (an N = 8 UMMA of its own costs
  // the pipe as much as the N = 64 one)
  static constexpr int K_STRIDE = CW_BOX_BYTES + 1024;
  static constexpr int K_BYTES = NKB * K_STRIDE;
  static constexpr int V_BYTES = 2 * CW_BOX_BYTES;
  static constexpr int OFF_K = Q_BYTES, OFF_V = Q_BYTES + K_BYTES;   // within a stage
  static constexpr int STAGE_BYTES = Q_BYTES + K_BYTES + V_BYTES;    // q, k (+ n rows), v of one chunk
  static constexpr int TX_BYTES = 2 * Q_BYTES + V_BYTES;             // what TMA delivers per stage
  static constexpr int OFF_STAGE = 0;
  static constexpr int OFF_VH = CW_STAGES * STAGE_BYTES;       // w_l-scaled v
  static constexpr int OFF_P = OFF_VH + V_BYTES;               // P tile
  static constexpr int OFF_WMAT = OFF_P + CW_BOX_BYTES;        // 2 x [8 x 64] bf16: rows w_hi, w_lo, zeros
  static constexpr int HST_ROW = CW_DV * 2 + 16;               // staged h row: 128 bf16 + 16 B pad
  static constexpr int OFF_HST = OFF_WMAT + 2 * 1024;          // [64][HST_ROW] normalised h of one chunk
  static constexpr int OFF_F32 = OFF_HST + CW_L * HST_ROW;
  static constexpr int GATE_F32 = 7 * CW_L + 8;                // per parity: see GateSlot
  static constexpr int N_F32 = 2 * GATE_F32 + CW_L + DHQK;     // + 1/denominator + n state
  static constexpr int OFF_BAR = OFF_F32 + N_F32 * 4;          // mbarriers (8-byte aligned)
  static constexpr int TOTAL = OFF_BAR + BAR_COUNT * 8 + 16;
  static constexpr int DYN_SMEM = TOTAL + 1024;                // slack to align the base to 1024 B
  // tensor-memory column map (512 columns, all used at DHQK = 256)
  static constexpr uint32_t T_C = 0;            // T (C^T in the lazy frame), fp32   DHQK columns
  static constexpr uint32_t T_H = 256;          // H^T accumulator                   64 columns
  static constexpr uint32_t T_CB = 320;         // bf16 copy of T                    DHQK/2 columns
  static constexpr uint32_t T_S = 448;          // S (even 16-lane halves); nu (odd halves)
  // The S product is 72 columns wide, [q.n | S], and starts eight columns BEFORE T_S.  At DHQK = 256 those eight
  // columns are the last eight of the bf16 copy (features 240..255).  The two uses alternate in time: the copy is read
  // by phase A of a chunk, [q.n | S] of the NEXT chunk is issued behind that phase, the gate group takes q.n out as
  // soon as it is complete, and only then does the epilogue group store the last eight columns of the next copy.
  static constexpr uint32_t T_SX = T_S - 8;
  static constexpr bool TAIL_SHARED = (T_CB + DHQK / 2 > T_SX);
};

struct CwMaps {
  CUtensorMap q, k, v;
  // position (1..3) of the token / head / batch coordinate in each map; the outer dimensions are ordered by
  // ascending stride, which differs between a contiguous (B,NH,S,D) tensor and a transposed (B,S,NH,D) view
  int pos[3][3];  // [q|k|v][token|head|batch]
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fast_log_sigmoid(float x) { return fminf(x, 0.f) - __logf(1.f + __expf(-fabsf(x))); }
__device__ __forceinline__ void gate_group_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ void epilogue_group_sync() { asm volatile("bar.sync 2, 128;" ::: "memory"); }

// 16 bytes of bf16 times a bf16x2 splat, rounded once per product
__device__ __forceinline__ uint4 scale_bf16x8(uint4 raw, __nv_bfloat162 s) {
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&raw);
  p[0] = __hmul2(p[0], s);
  p[1] = __hmul2(p[1], s);
  p[2] = __hmul2(p[2], s);
  p[3] = __hmul2(p[3], s);
  return raw;
}

// byte offset of element (row, col) in an [rows x 64] bf16 box with 128-byte swizzle
__device__ __forceinline__ uint32_t sw128_off(int row, int col) {
  return (uint32_t)(row * 128 + ((((col >> 3) ^ (row & 7)) << 4) | ((col & 7) << 1)));
}

// Wait used by the UMMA-issuing warp: after a first expired wait the later ones return at once.
#define MMA_WAIT_U(idx, parity) (okm ? mbar_wait(bar_u + 8u * (uint32_t)(idx), (uint32_t)(parity)) : false)

#define CW_WAIT(idx, parity)                                   \
  if (!mbar_wait(bar0 + 8u * (uint32_t)(idx), (uint32_t)(parity))) { \
    ok = false;                                                \
    break;                                                     \
  }

// T -> bf16 copy (operand of the inter-chunk product) for 64-column blocks [b0, b1); T itself is rescaled only when
// the lazy frame ran out.  The state group and the gate group each take half of the blocks at the same time.  One
// non-inlined copy on purpose: the kernel's hot loops together must stay small enough for the instruction cache
// (with every role's loop fully unrolled each pass ran mostly on instruction-fetch misses), and two groups running
// the same code at the same moment share its lines.  (Never called from the UMMA-issuing warp: a call there
// defeats the uniform datapath.)
static __device__ __noinline__ void cw_convert_T(uint32_t tC, uint32_t tCb, int b0, int b1, float cb_scale, float mult) {
#pragma unroll 1
  for (int cb = b0; cb < b1; ++cb) {
    uint32_t r0[32], r1[32];
    tmem_ld_x32(tC + cb * 64, r0);
    tmem_ld_x32(tC + cb * 64 + 32, r1);
    tc_wait_ld();
    uint32_t pk[32];
    if (cb_scale == 1.f) {  // the usual case: nothing but the conversion
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        pk[i] = pack_bf16x2(__uint_as_float(r0[2 * i]), __uint_as_float(r0[2 * i + 1]));
        pk[16 + i] = pack_bf16x2(__uint_as_float(r1[2 * i]), __uint_as_float(r1[2 * i + 1]));
      }
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        pk[i] = pack_bf16x2(__uint_as_float(r0[2 * i]) * cb_scale, __uint_as_float(r0[2 * i + 1]) * cb_scale);
        pk[16 + i] = pack_bf16x2(__uint_as_float(r1[2 * i]) * cb_scale, __uint_as_float(r1[2 * i + 1]) * cb_scale);
      }
    }
    tmem_st_x32(tCb + cb * 32, pk);
    if (mult != 1.f) {
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        r0[i] = __float_as_uint(__uint_as_float(r0[i]) * mult);
        r1[i] = __float_as_uint(__uint_as_float(r1[i]) * mult);
      }
      tmem_st_x32(tC + cb * 64, r0);
      tmem_st_x32(tC + cb * 64 + 32, r1);
    }
  }
  tc_wait_st();
}

template <int DHQK>
__global__ void __launch_bounds__(CW_THREADS, 1)
mlstm_chunkwise_kernel(const __grid_constant__ CwMaps maps, const xl_mlstm_seq_params p) {
  using LY = CwLayout<DHQK>;
  constexpr int NKB = LY::NKB;
  constexpr int NB = NKB;  // 64-feature blocks of the normaliser state n
  static_assert(NB == 1 || NB == 2 || NB == 4, "feature blocks");
  extern __shared__ unsigned char cw_smem_raw[];
  // 128-byte-swizzled tiles need 1024-byte aligned bases
  // (pointer arithmetic on the __shared__ array, not an integer round trip, so that every access below is
  // compiled as a shared-memory instruction rather than a generic one)
  unsigned char* smem = cw_smem_raw + ((1024u - (smem_u32(cw_smem_raw) & 1023u)) & 1023u);
  const uint32_t sbase = smem_u32(smem);
  float* s_f = reinterpret_cast<float*>(smem + LY::OFF_F32);
  // gate data of a chunk, double buffered by chunk parity (see GateSlot)
  auto gate_buf = [&](int parity) { return s_f + parity * LY::GATE_F32; };
  float* s_inv = s_f + 2 * LY::GATE_F32;  // 1 / denominator of the chunk in the epilogue
  float* s_n = s_inv + CW_L;              // n state in the lazy frame (DHQK)
  const uint32_t bar0 = sbase + LY::OFF_BAR;
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + LY::OFF_BAR + BAR_COUNT * 8);

  const int tid = threadIdx.x, lane = tid & 31;
  // The warp index is broadcast through a shuffle so that the compiler can PROVE the role branches below are
  // warp-uniform: only then does it issue an UMMA as ~4 instructions on the uniform datapath; behind a branch on
  // plain `threadIdx.x >> 5` every UMMA becomes a ~35-instruction sequence and the issuing warp, not the tensor
  // pipe, sets the pace.
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
  const int slice = blockIdx.x, head = blockIdx.y, doc = blockIdx.z;
  const int col0 = slice * CW_DV;
  const int DHV = p.DHV;

  // ---- document -> (batch row, first token, length)
  long long tok0, len;
  int b;
  if (p.cu_seqlens) {
    const long long s = p.cu_seqlens[doc], e = p.cu_seqlens[doc + 1];
    b = (int)(s / p.S);
    tok0 = s - (long long)b * p.S;
    len = e - s;
  } else {
    b = doc; tok0 = 0; len = p.S;
  }
  const long long sidx = (long long)doc * p.NH + head;

  if (len <= 0) {  // empty document: the state passes through unchanged
    if (tid < CW_DV) {
      const float* c0 = p.c0 ? p.c0 + (sidx * DHQK) * DHV + col0 + tid : nullptr;
      float* c_out = p.c_out + (sidx * DHQK) * DHV + col0 + tid;
      for (int d = 0; d < DHQK; ++d) c_out[(long long)d * DHV] = c0 ? c0[(long long)d * DHV] : 0.f;
    }
    if (slice == 0) {
      for (int d = tid; d < DHQK; d += CW_THREADS) p.n_out[sidx * DHQK + d] = p.n0 ? p.n0[sidx * DHQK + d] : 0.f;
      if (tid == 0) p.m_out[sidx] = p.m0 ? p.m0[sidx] : 0.f;
    }
    return;
  }
  const int nchunks = (int)((len + CW_L - 1) / CW_L);

  // ---- one-time setup: barriers, tensor memory, constant zero rows of the N=8 operands
  if (tid == 0) {
    for (int i = 0; i < BAR_COUNT; ++i) {
      uint32_t cnt = 128;                                                        // one 4-warp group arrives
      if (i == BAR_FULL0 || i == BAR_FULL1 || i == BAR_NU || i == BAR_HC || i == BAR_S) cnt = 1;
      if (i == BAR_EMPTY0 || i == BAR_EMPTY1) cnt = 129;    // state group + UMMA commit
      if (i == BAR_GFULL0 || i == BAR_GFULL1) cnt = 32;     // the scan warp
      if (i == BAR_GEMPTY0 || i == BAR_GEMPTY1) cnt = 256;  // state group + gate group
      if (i == BAR_A) cnt = 512;
      if (i == BAR_B) cnt = 256;
      mbar_init(bar0 + 8u * i, cnt);
    }
    fence_barrier_init();
    tma_prefetch_desc(&maps.q);
    tma_prefetch_desc(&maps.k);
    tma_prefetch_desc(&maps.v);
  }
  // OFF_P .. OFF_HST: the P tile (its blocks right of the diagonal stay zero for ever) and the w operand of nu
  for (int i = tid; i < (LY::OFF_HST - LY::OFF_P) / 16; i += CW_THREADS)
    reinterpret_cast<uint4*>(smem + LY::OFF_P)[i] = make_uint4(0u, 0u, 0u, 0u);
  // the eight extra B rows in front of every k box (rows 2..7 stay zero)
  for (int i = tid; i < CW_STAGES * NKB * (1024 / 16); i += CW_THREADS) {
    const int g = i / (1024 / 16);
    reinterpret_cast<uint4*>(smem + LY::OFF_STAGE + (g / NKB) * LY::STAGE_BYTES + LY::OFF_K + (g % NKB) * LY::K_STRIDE)[i % (1024 / 16)] =
        make_uint4(0u, 0u, 0u, 0u);
  }
  if (warp == W_UMMA) {
    __syncwarp();
    tmem_alloc(smem_u32(s_tmem), CW_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *s_tmem;
  const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;  // tcgen05.ld/st: a warp reaches lanes 32*(warp%4)..+31
  const uint32_t tC = tmem + LY::T_C + lane_base, tCb = tmem + LY::T_CB + lane_base;
  const uint32_t tH = tmem + LY::T_H + lane_base, tS = tmem + LY::T_S + lane_base;
  const float qscale = rsqrtf((float)DHQK);
  bool ok = true;
  auto convert_T = [&](int b0, int b1, float cb_scale, float mult) { cw_convert_T(tC, tCb, b0, b1, cb_scale, mult); };
  // blocks [0, CB_SPLIT) state group, [CB_SPLIT, DHQK/64) epilogue group (one block: it has the slack; the gate
  // group, whose P pass gates phase B, converts nothing).
  constexpr int CB_SPLIT = DHQK / 64 >= 2 ? DHQK / 64 - 1 : 1;

  if (warp == W_SCAN) {
    // =========================================================================================== scan warp
    // Carries the gate recurrence one or two chunks ahead of everybody else: lane L owns tokens 2L and 2L+1.
    const float* ig = p.igate + b * p.g_sb + head * p.g_sh + tok0 * p.g_st;
    const float* fg = p.fgate + b * p.g_sb + head * p.g_sh + tok0 * p.g_st;
    float m_prev = p.m0 ? p.m0[sidx] : 0.f;
    float rho = 0.f;
    // Gate loads are issued one chunk ahead, unconditionally and from clamped addresses; the tail mask is applied
    // when the values are used.
    float gi0, gi1, gf0, gf1;
    {
      const long long t0 = 2 * lane, ta = t0 < len ? t0 : len - 1, tb = t0 + 1 < len ? t0 + 1 : len - 1;
      gi0 = ig[ta * p.g_st]; gf0 = fg[ta * p.g_st];
      gi1 = ig[tb * p.g_st]; gf1 = fg[tb * p.g_st];
    }
#pragma unroll 1
    for (int chunk = 0; chunk < nchunks; ++chunk) {
      const int buf = chunk & 1;
      const long long rem = len - (long long)chunk * CW_L;
      const int len_c = rem < CW_L ? (int)rem : CW_L;
      float* gb = gate_buf(buf);
      CW_WAIT(BAR_GEMPTY0 + buf, ((uint32_t)(chunk >> 1) & 1u) ^ 1u);  // consumers of chunk-2 are done with this buffer
      const float ci0 = gi0, ci1 = gi1, cf0 = gf0, cf1 = gf1;
      {
        const long long tn = (long long)(chunk + 1) * CW_L + 2 * lane;
        const long long ta = tn < len ? tn : len - 1, tb = tn + 1 < len ? tn + 1 : len - 1;
        gi0 = ig[ta * p.g_st]; gf0 = fg[ta * p.g_st];
        gi1 = ig[tb * p.g_st]; gf1 = fg[tb * p.g_st];
      }
      const int t0 = 2 * lane, t1 = t0 + 1;
      const float lf0 = (t0 < len_c) ? fast_log_sigmoid(cf0) : 0.f;
      const float lf1 = (t1 < len_c) ? fast_log_sigmoid(cf1) : 0.f;
      float incl = lf0 + lf1;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
      }
      const float b1 = incl, b0 = incl - lf1;
      const float ap0 = (t0 < len_c) ? ci0 - b0 : -INFINITY;
      const float ap1 = (t1 < len_c) ? ci1 - b1 : -INFINITY;
      float cmx = fmaxf(ap0, ap1);
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, cmx, o);
        if (lane >= o) cmx = fmaxf(cmx, t);
      }
      float prevmax = __shfl_up_sync(0xffffffffu, cmx, 1);
      if (lane == 0) prevmax = -INFINITY;
      const float mu0 = fmaxf(m_prev, fmaxf(prevmax, ap0));
      const float mu1 = fmaxf(m_prev, cmx);
      const float mu_star = __shfl_sync(0xffffffffu, mu1, 31);
      const float gsum = __shfl_sync(0xffffffffu, b1, 31);
      // lazy decay frame: C = exp(rho) T
      const float cand = rho + (m_prev - mu_star);
      const bool rescale = cand < CW_RESCALE_BELOW;
      const float mult = rescale ? __expf(cand) : 1.f;
      const float rho_new = rescale ? 0.f : cand;
      const float mu_first = __shfl_sync(0xffffffffu, mu0, 0);
      const bool exact = (mu_star - mu_first) > CW_FAST_SPREAD;
      const float w0 = __expf(ap0 - mu_star - rho_new), w1 = __expf(ap1 - mu_star - rho_new);
      *reinterpret_cast<float2*>(gb + G_W + t0) = make_float2(w0, w1);
      if (exact) {
        *reinterpret_cast<float2*>(gb + G_LOWER + t0) = make_float2(__expf(-(b0 + mu0)), __expf(-(b1 + mu1)));
        *reinterpret_cast<float2*>(gb + G_X + t0) = make_float2(ap0 * CW_LOG2E, ap1 * CW_LOG2E);
        *reinterpret_cast<float2*>(gb + G_Y + t0) = make_float2(mu0 * CW_LOG2E, mu1 * CW_LOG2E);
        *reinterpret_cast<float2*>(gb + G_R + t0) =
            make_float2(__expf(m_prev - mu0 + rho) * qscale, __expf(m_prev - mu1 + rho) * qscale);
        *reinterpret_cast<float2*>(gb + G_Z + t0) = make_float2(1.f, 1.f);
        *reinterpret_cast<float2*>(gb + G_EPS + t0) = make_float2(1.f, 1.f);
      } else {
        // The common frame leaves the 1/sqrt(d) of q out of BOTH numerator and denominator (h is their ratio): the
        // bf16 copy of T and P then need no multiplication at all; the lower bound and eps take sqrt(d) instead.
        const float phi = mu_star + rho_new, sqrt_d = 1.f / qscale;
        *reinterpret_cast<float2*>(gb + G_LOWER + t0) = make_float2(__expf(-(b0 + phi)) * sqrt_d, __expf(-(b1 + phi)) * sqrt_d);
        *reinterpret_cast<float2*>(gb + G_X + t0) = make_float2(t0 < len_c ? 0.f : -INFINITY, t1 < len_c ? 0.f : -INFINITY);
        *reinterpret_cast<float2*>(gb + G_Y + t0) = make_float2(0.f, 0.f);
        *reinterpret_cast<float2*>(gb + G_Z + t0) = make_float2(w0, w1);
        *reinterpret_cast<float2*>(gb + G_EPS + t0) = make_float2(__expf(mu0 - phi) * sqrt_d, __expf(mu1 - phi) * sqrt_d);
      }
      {
        const __nv_bfloat162 hi = __floats2bfloat162_rn(w0, w1);
        const float2 hif = __bfloat1622float2(hi);
        const __nv_bfloat162 lo = __floats2bfloat162_rn(w0 - hif.x, w1 - hif.y);
        unsigned char* wm = smem + LY::OFF_WMAT + buf * 1024;
        *reinterpret_cast<__nv_bfloat162*>(wm + sw128_off(0, t0)) = hi;
        *reinterpret_cast<__nv_bfloat162*>(wm + sw128_off(1, t0)) = lo;
      }
      if (lane == 0) {
        gb[G_MULT] = mult;
        gb[G_RHO] = rho_new;
        gb[G_EXACT] = exact ? 1.f : 0.f;
        // common frame: T q enters as exp(rho + m_prev - mu* - rho') T q; that exponent is the rescale multiplier
        // itself (1 whenever no rescale happens)
        gb[G_CB] = exact ? 1.f : mult;
        gb[G_QN] = exact ? 1.f : mult;
      }
      m_prev = gsum + mu_star;
      rho = rho_new;
      fence_proxy_async_smem();
      mbar_arrive(bar0 + 8u * (BAR_GFULL0 + buf));
    }
    if (ok && slice == 0 && lane == 0) p.m_out[sidx] = m_prev;
  } else if (warp < W_STATE_GROUP) {
    // =========================================================================================== gate group
    // Iteration j: q.n(j) and S(j) out of tensor memory, P(j); then, with nu(j) (issued one chunk ahead, behind S(j)):
    // n(j) and its hi/lo rows for the S product of chunk j+1, and the denominators of chunk j.
    const int g = tid;  // 0..127
    for (int d = g; d < DHQK; d += 128) s_n[d] = p.n0 ? p.n0[sidx * DHQK + d] : 0.f;
    // hi/lo bf16 split of n[d] into rows 0/1 in front of the k box of feature block d/64 in stage `nbuf`, where the S
    // product of that stage's chunk picks them up as eight more B rows
    auto publish_n = [&](int nbuf, int d, float nv) {
      const __nv_bfloat16 hi = __float2bfloat16_rn(nv);
      const __nv_bfloat16 lo = __float2bfloat16_rn(nv - __bfloat162float(hi));
      unsigned char* box = smem + LY::OFF_STAGE + nbuf * LY::STAGE_BYTES + LY::OFF_K + (d >> 6) * LY::K_STRIDE;
      *reinterpret_cast<__nv_bfloat16*>(box + sw128_off(0, d & 63)) = hi;
      *reinterpret_cast<__nv_bfloat16*>(box + sw128_off(1, d & 63)) = lo;
    };
    for (int d = g; d < DHQK; d += 128) publish_n(0, d, s_n[d]);
    fence_proxy_async_smem();
    if (mbar_wait(bar0 + 8u * BAR_GFULL0, 0u)) mbar_arrive(bar0 + 8u * BAR_C2);  // n rows and gate data of chunk 0
    else ok = false;
    // S fragment of this thread: rows j0 and j0 + 8, column pair cq of every 8-column group (q.n is the group in front
    // of S: the threads with cq == 0 hold its hi and lo part); the nu products sit on lanes 16..31 of the plain
    // (lane = thread) view
    const int j0 = warp * 16 + (lane >> 2), cq = 2 * (lane & 3);
    float back_last = 1.f;
#pragma unroll 1
    for (int chunk = 0; chunk < nchunks; ++chunk) {
      const int buf = chunk & 1;
      const uint32_t par = (uint32_t)chunk & 1u;
      const float* gb = gate_buf(buf);
      CW_WAIT(BAR_GFULL0 + buf, (uint32_t)(chunk >> 1) & 1u);
      const float y0 = gb[G_Y + j0], y1 = gb[G_Y + j0 + 8];
      const float mult = gb[G_MULT];
      const bool exact = gb[G_EXACT] != 0.f;
      // the normaliser product is formed from q as loaded: its scale is the row's r_j in the exact frame
      const int jd = j0 + 8 * (lane & 1);  // the row whose denominator this thread writes (lanes 4i and 4i + 1)
      const float lower = gb[G_LOWER + jd];
      const float eps_j = p.eps * gb[G_EPS + jd];
      const float qn_scale = exact ? gb[G_R + jd] : gb[G_QN];
      if (chunk + 1 == nchunks) back_last = expf(gb[G_RHO]);
      // S of this chunk complete.  The tensor pipe completes in order, so phase B of the previous chunk is complete as
      // well: its UMMAs no longer read the P tile.
      CW_WAIT(BAR_S, par);
      tc_fence_after();
      // ---- P from S.  One fragment load brings this warp's 16 rows x 64 columns of S to all 32 lanes (shape 16x256b:
      // thread t holds rows j0 = 16 warp + t/4 and j0 + 8, columns 8g + 2 (t%4) + {0,1} of every 8-column group g), so
      // the pass is one tensor-memory round trip instead of one per 16-column piece and no lane idles.  Rows 16w..16w+15
      // need groups 0..2w+1 (the last two straddle the diagonal); the groups to their right are zero for ever
      // (written once at set-up).
      float rs0 = 0.f, rs1 = 0.f, dot;
      {
        uint32_t sv[32], dn[4];
        tmem_ld_16x256b_x1(tS - 8, dn);
        tmem_ld_16x256b_x8(tS, sv);
        // the per-column factors of all eight groups are fetched up front, outside any branch: inside the branches below
        // every load would wait out its shared-memory latency on its own, eight times in a row
        float2 zz[8];
#pragma unroll
        for (int g = 0; g < 8; ++g) zz[g] = *reinterpret_cast<const float2*>(gb + (exact ? G_X : G_Z) + 8 * g + cq);
        unsigned char* prow0 = smem + LY::OFF_P + j0 * 128 + 2 * cq;
        unsigned char* prow1 = prow0 + 8 * 128;
        tc_wait_ld();
        tc_fence_before();
        mbar_arrive(bar0 + 8u * BAR_QNREAD);  // the q.n columns may take the tail of the bf16 copy again
        // q.n of rows j0 (registers 0, 1) and j0 + 8 (registers 2, 3) in the threads with cq == 0; the thread next to it
        // takes the second row (jd)
        const float d0 = __uint_as_float(dn[0]) + __uint_as_float(dn[1]), d1 = __uint_as_float(dn[2]) + __uint_as_float(dn[3]);
        const float d1n = __shfl_sync(0xffffffffu, d1, lane & ~3);
        dot = (lane & 1) ? d1n : d0;
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          if (g <= 2 * warp + 1) {  // warp-uniform
            float e00, e01, e10, e11;
            if (exact) {
              e00 = __uint_as_float(sv[4 * g + 0]) * qscale * ex2_approx(zz[g].x - y0);
              e01 = __uint_as_float(sv[4 * g + 1]) * qscale * ex2_approx(zz[g].y - y0);
              e10 = __uint_as_float(sv[4 * g + 2]) * qscale * ex2_approx(zz[g].x - y1);
              e11 = __uint_as_float(sv[4 * g + 3]) * qscale * ex2_approx(zz[g].y - y1);
            } else {
              e00 = __uint_as_float(sv[4 * g + 0]) * zz[g].x;
              e01 = __uint_as_float(sv[4 * g + 1]) * zz[g].y;
              e10 = __uint_as_float(sv[4 * g + 2]) * zz[g].x;
              e11 = __uint_as_float(sv[4 * g + 3]) * zz[g].y;
            }
            // causal mask (only the two groups on the diagonal lose anything to it)
            const int c = 8 * g + cq;
            e00 = (c <= j0) ? e00 : 0.f;
            e01 = (c + 1 <= j0) ? e01 : 0.f;
            e10 = (c <= j0 + 8) ? e10 : 0.f;
            e11 = (c + 1 <= j0 + 8) ? e11 : 0.f;
            // (row sums from the unrounded values: the difference to the bf16 P is below the bf16 rounding of h)
            rs0 += e00 + e01;
            rs1 += e10 + e11;
            const uint32_t sw = (uint32_t)((g ^ (j0 & 7)) << 4);  // (j0 + 8) & 7 == j0 & 7
            *reinterpret_cast<uint32_t*>(prow0 + sw) = pack_bf16x2(e00, e01);
            *reinterpret_cast<uint32_t*>(prow1 + sw) = pack_bf16x2(e10, e11);
          }
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(bar0 + 8u * BAR_B);
      rs0 += __shfl_xor_sync(0xffffffffu, rs0, 1);
      rs0 += __shfl_xor_sync(0xffffffffu, rs0, 2);
      rs1 += __shfl_xor_sync(0xffffffffu, rs1, 1);
      rs1 += __shfl_xor_sync(0xffffffffu, rs1, 2);

      // ---- n of this chunk: n = mult n + nu, published as the hi/lo rows of the next chunk's stage (the S product of
      // the chunk that used that stage before has read its own long ago)
      CW_WAIT(BAR_NU, par);
      tc_fence_after();
      {
        uint32_t r[8 * NB];
        if constexpr (NB == 1) tmem_ld_x8(tS + 8, r);
        else if constexpr (NB == 2) tmem_ld_x16(tS + 8, r);
        else tmem_ld_x32(tS + 8, r);
        tc_wait_ld();
        if (lane >= 16) {
#pragma unroll
          for (int gq = 0; gq < NB; ++gq) {
            const int d = 64 * gq + 16 * warp + (lane - 16);
            const float nv = fmaf(s_n[d], mult, __uint_as_float(r[8 * gq]) + __uint_as_float(r[8 * gq + 1]));
            s_n[d] = nv;
            publish_n(buf ^ 1, d, nv);
          }
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      if (chunk + 1 < nchunks) CW_WAIT(BAR_GFULL0 + (buf ^ 1), (uint32_t)((chunk + 1) >> 1) & 1u);  // w operand of the next chunk
      mbar_arrive(bar0 + 8u * BAR_C2);                // phase C of this chunk may issue
      mbar_arrive(bar0 + 8u * (BAR_GEMPTY0 + buf));  // done with this chunk's gate data (so is nu, which read w)
      // ---- denominators: |rowsum + q.n| against the lower bound (lanes 4i and 4i + 1 write rows j0 and j0 + 8)
      if (chunk >= 1) CW_WAIT(BAR_EGDONE, par ^ 1u);  // the epilogue group has consumed the previous ones
      if ((lane & 2) == 0) s_inv[jd] = __fdividef(1.f, fmaxf(fabsf(fmaf(dot, qn_scale, (lane & 1) ? rs1 : rs0)), lower) + eps_j);
      mbar_arrive(bar0 + 8u * BAR_INV);
    }
    // ---- final n (back in the true frame)
    if (ok && slice == 0 && lane >= 16) {  // the first slice of the head writes n
#pragma unroll
      for (int gq = 0; gq < NB; ++gq) {
        const int d = 64 * gq + 16 * warp + (lane - 16);
        p.n_out[sidx * DHQK + d] = s_n[d] * back_last;
      }
    }
  } else if (warp < W_EPI_GROUP) {
    // =========================================================================================== state group
    const int t = tid - 128;
    const int dv = (warp & 3) * 32 + lane;  // tensor-memory lane = value column within the slice
    const float* c0 = p.c0 ? p.c0 + (sidx * DHQK) * DHV + col0 + dv : nullptr;
    float* c_out = p.c_out + (sidx * DHQK) * DHV + col0 + dv;
#pragma unroll 1
    for (int cb = 0; cb < DHQK / 32; ++cb) {
      uint32_t r[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) r[i] = c0 ? __float_as_uint(c0[(long long)(cb * 32 + i) * DHV]) : 0u;
      tmem_st_x32(tC + cb * 32, r);
    }
    tc_wait_st();
    tc_fence_before();
    mbar_arrive(bar0 + 8u * BAR_TINIT);  // the epilogue group converts its block of the initial state
    float rho_last = 0.f;
#pragma unroll 1
    for (int chunk = 0; chunk < nchunks; ++chunk) {
      const int st = chunk & 1, buf = chunk & 1;
      const uint32_t par = (uint32_t)chunk & 1u, par_full = (uint32_t)(chunk >> 1) & 1u;
      const float* gb = gate_buf(buf);
      CW_WAIT(BAR_GFULL0 + buf, par_full);
      const float mult = gb[G_MULT], cb_scale = gb[G_CB];
      const bool exact = gb[G_EXACT] != 0.f;
      rho_last = gb[G_RHO];
      const __nv_bfloat162 rr = __float2bfloat162_rn(gb[G_R + (t >> 1)]);
      const __nv_bfloat162 ww = __float2bfloat162_rn(gb[G_W + (t >> 1)]);
      if (chunk >= 1) CW_WAIT(BAR_HC, par ^ 1u);  // T holds chunk-1; its UMMAs no longer read Tb or the scaled-v tile
      tc_fence_after();
      // ---- T -> bf16 copy, this group's blocks
      convert_T(0, CB_SPLIT, cb_scale, mult);
      tc_fence_before();
      mbar_arrive(bar0 + 8u * BAR_A);
      if (!exact) mbar_arrive(bar0 + 8u * BAR_A);  // common frame: q is used as loaded
      // ---- w-scaled v (thread: row l = t/2, box = t&1)
      CW_WAIT(BAR_FULL0 + st, par_full);
      {
        const int l = t >> 1, half = t & 1;
        const unsigned char* vt = smem + LY::OFF_STAGE + st * LY::STAGE_BYTES + LY::OFF_V;
        uint4 v[8];
        uint32_t off[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int c = i ^ (half << 2);
          off[i] = half * CW_BOX_BYTES + l * 128 + ((c ^ (l & 7)) << 4);
          v[i] = *reinterpret_cast<const uint4*>(vt + off[i]);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) *reinterpret_cast<uint4*>(smem + LY::OFF_VH + off[i]) = scale_bf16x8(v[i], ww);
      }
      fence_proxy_async_smem();
      mbar_arrive(bar0 + 8u * BAR_B);
      // ---- exact frame only: q <- r_j q IN PLACE in the stage tile (thread: row j = t/2, half of the row).  S of
      // this chunk, the only consumer of the un-scaled q, must have completed.
      if (exact) {
        CW_WAIT(BAR_NU, par);  // [qn|S] and nu of this chunk (issued one chunk ahead) no longer read q as loaded
        const int j = t >> 1, half = t & 1;
        unsigned char* qt = smem + LY::OFF_STAGE + st * LY::STAGE_BYTES;
        constexpr int CH = NKB * 4;              // 16-byte pieces per thread
        constexpr int BATCH = CH < 8 ? CH : 8;   // loads first, then stores
#pragma unroll 1
        for (int i0 = 0; i0 < CH; i0 += BATCH) {
          uint4 v[BATCH];
          uint32_t off[BATCH];
#pragma unroll
          for (int i = 0; i < BATCH; ++i) {
            const int cidx = half * CH + i0 + i;
            const int box = cidx >> 3;
            const int c = (NKB >= 2) ? ((cidx & 7) ^ (half << 2)) : (cidx & 7);
            off[i] = box * CW_BOX_BYTES + j * 128 + ((c ^ (j & 7)) << 4);
            v[i] = *reinterpret_cast<const uint4*>(qt + off[i]);
          }
#pragma unroll
          for (int i = 0; i < BATCH; ++i) *reinterpret_cast<uint4*>(qt + off[i]) = scale_bf16x8(v[i], rr);
        }
        fence_proxy_async_smem();
        mbar_arrive(bar0 + 8u * BAR_A);
      }
      mbar_arrive(bar0 + 8u * (BAR_EMPTY0 + st));
      mbar_arrive(bar0 + 8u * (BAR_GEMPTY0 + buf));
    }
    // ---- final C = exp(rho) T
    if (ok) {
      do {
        CW_WAIT(BAR_HC, (uint32_t)(nchunks - 1) & 1u);
        tc_fence_after();
        const float back = expf(rho_last);
#pragma unroll 1
        for (int cb = 0; cb < DHQK / 32; ++cb) {
          uint32_t r[32];
          tmem_ld_x32(tC + cb * 32, r);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) c_out[(long long)(cb * 32 + i) * DHV] = __uint_as_float(r[i]) * back;
        }
      } while (false);
    }
  } else if (warp < W_UMMA) {
    // =========================================================================================== epilogue group
    // H^T sits in tensor memory with one value column per lane.  The group pulls it into registers (which frees the
    // accumulator for the next chunk at once), scales by 1/denominator, writes bf16 into a [token][column] staging tile
    // in shared memory and streams the tile out with 16-byte stores (a row of the tile is 256 contiguous bytes of h).
    const int t = tid - 256;
    const int cq = 2 * (lane & 3);
    unsigned char* hst = smem + LY::OFF_HST;
    const uint32_t hst_u = smem_u32(hst);
    __nv_bfloat16* hbase = reinterpret_cast<__nv_bfloat16*>(p.h) + b * p.h_sb + head * p.h_sh + tok0 * p.h_st + col0;
    // This group's block of the T -> bf16 copy for chunk `next` (T holds chunk next - 1 or the initial state).  The block
    // is read and converted at once; where its last eight columns double as the q.n columns of [q.n | S](next) they
    // stay in registers (`tail`) until the gate group has taken q.n(next) out (finish_block).
    constexpr bool EG_CONVERTS = DHQK / 64 >= 2;  // with one block only, the state group converts it
    uint32_t tail[8];
    auto convert_block = [&](int next) -> bool {
      if constexpr (EG_CONVERTS) {
        if (!mbar_wait(bar0 + 8u * (BAR_GFULL0 + (next & 1)), (uint32_t)(next >> 1) & 1u)) return false;
        const float* gbn = gate_buf(next & 1);
        const float cb_scale = gbn[G_CB], mult = gbn[G_MULT];
        constexpr int cb = DHQK / 64 - 1;
        uint32_t r0[32], r1[32];
        tmem_ld_x32(tC + cb * 64, r0);
        tmem_ld_x32(tC + cb * 64 + 32, r1);
        tc_wait_ld();
        uint32_t pk[32];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          pk[i] = pack_bf16x2(__uint_as_float(r0[2 * i]) * cb_scale, __uint_as_float(r0[2 * i + 1]) * cb_scale);
          pk[16 + i] = pack_bf16x2(__uint_as_float(r1[2 * i]) * cb_scale, __uint_as_float(r1[2 * i + 1]) * cb_scale);
        }
        if constexpr (LY::TAIL_SHARED) {
          uint32_t lo16[16], mid8[8];
#pragma unroll
          for (int i = 0; i < 16; ++i) lo16[i] = pk[i];
#pragma unroll
          for (int i = 0; i < 8; ++i) { mid8[i] = pk[16 + i]; tail[i] = pk[24 + i]; }
          tmem_st_x16(tCb + cb * 32, lo16);
          tmem_st_x8(tCb + cb * 32 + 16, mid8);
        } else {
          tmem_st_x32(tCb + cb * 32, pk);
        }
        if (mult != 1.f) {  // the lazy frame ran out: rescale T itself
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            r0[i] = __float_as_uint(__uint_as_float(r0[i]) * mult);
            r1[i] = __float_as_uint(__uint_as_float(r1[i]) * mult);
          }
          tmem_st_x32(tC + cb * 64, r0);
          tmem_st_x32(tC + cb * 64 + 32, r1);
        }
      }
      return true;
    };
    auto finish_block = [&](int next) -> bool {
      if constexpr (EG_CONVERTS && LY::TAIL_SHARED) {
        if (!mbar_wait(bar0 + 8u * BAR_QNREAD, (uint32_t)next & 1u)) return false;
        tc_fence_after();
        tmem_st_x8(tCb + DHQK / 2 - 8, tail);
      }
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(bar0 + 8u * BAR_A);  // this group's share of the bf16 copy for chunk `next`
      return true;
    };
    if constexpr (EG_CONVERTS) {
      if (!mbar_wait(bar0 + 8u * BAR_TINIT, 0u)) ok = false;
      tc_fence_after();
    }
    if (ok && !convert_block(0)) ok = false;
    mbar_arrive(bar0 + 8u * BAR_A);  // the accumulator is free for chunk 0
    if (ok && !finish_block(0)) ok = false;
    // Denominators of chunk c: ready long before H^T(c) is (they depend on the previous phase of UMMAs only).
    auto denominators_ready = [&](int c) -> bool {
      if (!mbar_wait(bar0 + 8u * BAR_INV, (uint32_t)c & 1u)) return false;
      return true;
    };
#pragma unroll 1
    for (int chunk = 0; ok && chunk < nchunks; ++chunk) {
      const uint32_t par = (uint32_t)chunk & 1u;
      const long long rem = len - (long long)chunk * CW_L;
      const int len_c = rem < CW_L ? (int)rem : CW_L;
      CW_WAIT(BAR_HC, par);
      tc_fence_after();
      // ---- this group's block of the T -> bf16 copy for the NEXT chunk (T holds this chunk now)
      const bool have_next = chunk + 1 < nchunks;
      if (have_next && !convert_block(chunk + 1)) { ok = false; break; }
      // the denominators of this chunk: published by the gate group about a chunk ago (waited for here and not at the
      // end of the previous iteration, where the wait would hold up the conversion above)
      if (!denominators_ready(chunk)) { ok = false; break; }
      // drain, normalise and stage.  The accumulator comes out as two fragments of 16 value columns x 64 tokens
      // (shape 16x256b: thread t holds columns t/4 and t/4 + 8, tokens 8g + 2 (t%4) + {0,1} of every group g); a pair of
      // tokens packs into one register and stmatrix.trans writes 8 x 8 blocks transposed, so that a token's eight value
      // columns land as 16 contiguous bytes of its row of the staging tile.
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {
        uint32_t hv[32];
        tmem_ld_16x256b_x8(tH + ((uint32_t)(half * 16) << 16), hv);
        // lanes 8m .. 8m+7 address the rows of matrix m: token group (m >> 1), value columns + 8 (m & 1)
        const uint32_t srow = hst_u + (uint32_t)((8 * (lane >> 4) + (lane & 7)) * LY::HST_ROW + ((warp & 3) * 32 + half * 16 + 8 * ((lane >> 3) & 1)) * 2);
        tc_wait_ld();
        if (half == 1) {  // the accumulator is in registers: free for the next chunk
          tc_fence_before();
          mbar_arrive(bar0 + 8u * BAR_A);
          if (have_next && !finish_block(chunk + 1)) ok = false;  // (the loop ends at its top)
        }
#pragma unroll
        for (int gp = 0; gp < 4; ++gp) {
          const float2 i0 = *reinterpret_cast<const float2*>(s_inv + 16 * gp + cq);
          const float2 i1 = *reinterpret_cast<const float2*>(s_inv + 16 * gp + 8 + cq);
          const uint32_t m0 = pack_bf16x2(__uint_as_float(hv[8 * gp + 0]) * i0.x, __uint_as_float(hv[8 * gp + 1]) * i0.y);
          const uint32_t m1 = pack_bf16x2(__uint_as_float(hv[8 * gp + 2]) * i0.x, __uint_as_float(hv[8 * gp + 3]) * i0.y);
          const uint32_t m2 = pack_bf16x2(__uint_as_float(hv[8 * gp + 4]) * i1.x, __uint_as_float(hv[8 * gp + 5]) * i1.y);
          const uint32_t m3 = pack_bf16x2(__uint_as_float(hv[8 * gp + 6]) * i1.x, __uint_as_float(hv[8 * gp + 7]) * i1.y);
          stmatrix_x4_trans(srow + (uint32_t)(16 * gp * LY::HST_ROW), m0, m1, m2, m3);
        }
      }
      mbar_arrive(bar0 + 8u * BAR_EGDONE);  // the denominators of this chunk are consumed
      epilogue_group_sync();
      __nv_bfloat16* ho = hbase + (long long)chunk * CW_L * p.h_st;
      {  // 64 rows of 256 bytes leave as 16-byte pieces, a row per 16 threads: all loads first, then the stores
        uint4 piece[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) piece[i] = *reinterpret_cast<const uint4*>(hst + (i * 8 + (t >> 4)) * LY::HST_ROW + (t & 15) * 16);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int row = i * 8 + (t >> 4);
          if (row < len_c) *reinterpret_cast<uint4*>(ho + (long long)row * p.h_st + (t & 15) * 8) = piece[i];
        }
      }
      epilogue_group_sync();  // the tile is rewritten by the next chunk
    }
  } else if (warp == W_UMMA) {
    // =========================================================================================== UMMA issuer
    // The whole warp runs this code (warp-uniform control flow, waits never branch out of it); one elected lane
    // issues each instruction.  Every descriptor is formed from one runtime base plus compile-time constants so
    // that the address arithmetic stays on the uniform datapath.  A chain of UMMAs accumulating into one tile runs
    // at its latency (about 60 cycles a step), so every phase interleaves two independent products step by step.
    constexpr uint32_t IDESC_S = umma_idesc_bf16(64, 72, 0, 0);  // S and, from eight more B rows, q.n
    constexpr uint32_t IDESC_HI = umma_idesc_bf16(128, 64, 0, 0);
    constexpr uint32_t IDESC_HV = umma_idesc_bf16(128, 64, 1, 0);
    constexpr uint32_t IDESC_C = umma_idesc_bf16(128, DHQK, 1, 1);
    constexpr uint32_t IDESC_NU = umma_idesc_bf16(64, 8, 1, 0);
    // Values that are warp-uniform in fact but not provably so (read from shared or global memory) are broadcast
    // with a shuffle: that is what lets the compiler keep UMMA operands in uniform registers.
    // (shared-memory base for DESCRIPTORS only: the 18-bit offset inside this CTA's window)
    const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem, 0), sbase_u = __shfl_sync(0xffffffffu, sbase, 0) & 0x3FFFFu;
    const uint32_t bar_u = __shfl_sync(0xffffffffu, bar0, 0);
    const int nchunks_u = __shfl_sync(0xffffffffu, nchunks, 0);
    const uint32_t t_odd = tmem_u + LY::T_S + (16u << 16);  // odd 16-lane halves of the S columns
    // lower descriptor words (start address >> 4 | leading offset); K-major tiles use leading offset 16 B, MN-major
    // tiles the distance between their 64-wide boxes (8 KiB; 9 KiB for k, whose boxes have the n rows in front)
    constexpr uint32_t LBO_K = (16u >> 4) << 16, LBO_MN = ((uint32_t)CW_BOX_BYTES >> 4) << 16;
    constexpr uint32_t LBO_MN_K = ((uint32_t)LY::K_STRIDE >> 4) << 16;
    bool okm = true;
    // Phase C of chunk k forms everything of chunk k+1 that does not depend on the state: [q.n | S] and nu.  It runs
    // while T is converted for chunk k+1, so the tensor pipe has work during the one long dependency of the loop.
    auto phase_c = [&](int next) {  // [q.n | S](next), then nu(next)
      const uint32_t nq = sbase_u + LY::OFF_STAGE + (next & 1) * LY::STAGE_BYTES;
      const uint32_t nrow = nq + LY::OFF_K, nk = nrow + 1024;  // n rows in front of the first k box | the k data
      const uint32_t wm = sbase_u + LY::OFF_WMAT + (next & 1) * 1024;
      okm &= MMA_WAIT_U(BAR_FULL0 + (next & 1), (uint32_t)(next >> 1) & 1u);
      okm &= MMA_WAIT_U(BAR_C2, (uint32_t)next & 1u);
      tc_fence_after();
#pragma unroll 1
      for (int kb = 0; kb < NKB; ++kb)
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_ss_lo(tmem_u + LY::T_SX, (LBO_K + ((nq + kb * CW_BOX_BYTES + kk * 32) >> 4)),
                     (LBO_K + ((nrow + kb * LY::K_STRIDE + kk * 32) >> 4)), IDESC_S, (kb | kk) != 0);
      umma_commit_elect(bar_u + 8u * BAR_S);
      // nu of all feature blocks: step (token slice tsl, feature block gq), four independent accumulators in turn
#pragma unroll 1
      for (int tsl = 0; tsl < 4; ++tsl)
#pragma unroll
        for (int gq = 0; gq < NB; ++gq)
          umma_ss_lo(t_odd + 8 + 8 * gq, (LBO_MN_K + ((nk + gq * LY::K_STRIDE + tsl * 2048) >> 4)),
                     (LBO_K + ((wm + tsl * 32) >> 4)), IDESC_NU, tsl != 0);
      umma_commit_elect(bar_u + 8u * BAR_NU);
    };
    phase_c(0);
#pragma unroll 1
    for (int chunk = 0; chunk < nchunks_u; ++chunk) {
      const uint32_t par = (uint32_t)chunk & 1u;
      const uint32_t stg = sbase_u + LY::OFF_STAGE + (chunk & 1) * LY::STAGE_BYTES;  // q | k | v of this chunk
      const uint32_t s_k = stg + LY::OFF_K + 1024, s_v = stg + LY::OFF_V;
      // ---- phase A:  H^T = Tb q^T
      okm &= MMA_WAIT_U(BAR_A, par);
      tc_fence_after();
#pragma unroll 1
      for (int kb = 0; kb < NKB; ++kb)
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_ts_lo(tmem_u + LY::T_H, tmem_u + LY::T_CB + (4 * kb + kk) * 8,
                     (LBO_K + ((stg + kb * CW_BOX_BYTES + kk * 32) >> 4)), IDESC_HI, (kb | kk) != 0);
      // ---- phase B:  H^T += V^T P^T   interleaved with   T += (wV)^T K
      okm &= MMA_WAIT_U(BAR_B, par);
      tc_fence_after();
      {
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          umma_ss_lo(tmem_u + LY::T_H, (LBO_MN + ((s_v >> 4) + ((kk * 2048) >> 4))),
                     (LBO_K + ((sbase_u >> 4) + ((LY::OFF_P + kk * 32) >> 4))), IDESC_HV, 1);
          umma_ss_lo(tmem_u + LY::T_C, (LBO_MN + ((sbase_u >> 4) + ((LY::OFF_VH + kk * 2048) >> 4))),
                     (LBO_MN_K + ((s_k >> 4) + ((kk * 2048) >> 4))), IDESC_C, 1);
        }
      }
      umma_commit_elect(bar_u + 8u * BAR_HC);
      umma_commit_elect(bar_u + 8u * (BAR_EMPTY0 + (chunk & 1)));  // the stage of this chunk is consumed
      // ---- phase C for the next chunk (one branch around the whole phase, none inside the issue loops)
      if (chunk + 1 < nchunks_u) phase_c(chunk + 1);
    }
    ok = okm;
  } else {
    // =========================================================================================== TMA issuer
    if (lane == 0) {
#pragma unroll 1
      for (int chunk = 0; chunk < nchunks; ++chunk) {
        const int st = chunk & 1;
        const uint32_t use = (uint32_t)(chunk >> 1);
        CW_WAIT(BAR_EMPTY0 + st, (use & 1u) ^ 1u);  // passes at once for the first use of a stage
        const uint32_t bar = bar0 + 8u * (BAR_FULL0 + st);
        const uint32_t dst = sbase + LY::OFF_STAGE + st * LY::STAGE_BYTES;
        const int tk = (int)(tok0 + (long long)chunk * CW_L);
        mbar_expect_tx(bar, LY::TX_BYTES);
        int cq[4], ck[4], cv[4];
        cq[maps.pos[0][0]] = tk; cq[maps.pos[0][1]] = head; cq[maps.pos[0][2]] = b;
        ck[maps.pos[1][0]] = tk; ck[maps.pos[1][1]] = head; ck[maps.pos[1][2]] = b;
        cv[maps.pos[2][0]] = tk; cv[maps.pos[2][1]] = head; cv[maps.pos[2][2]] = b;
#pragma unroll
        for (int kb = 0; kb < NKB; ++kb) {
          tma_load_4d(dst + kb * CW_BOX_BYTES, &maps.q, bar, kb * 64, cq[1], cq[2], cq[3]);
          tma_load_4d(dst + LY::OFF_K + kb * LY::K_STRIDE + 1024, &maps.k, bar, kb * 64, ck[1], ck[2], ck[3]);
        }
#pragma unroll
        for (int vb = 0; vb < 2; ++vb)
          tma_load_4d(dst + LY::OFF_V + vb * CW_BOX_BYTES, &maps.v, bar, col0 + vb * 64, cv[1], cv[2], cv[3]);
      }
    }
    __syncwarp();
  }

  if (!ok && p.status) atomicExch(p.status, 1);
  tc_fence_before();
  __syncthreads();
  if (warp == W_UMMA) tmem_dealloc(tmem, CW_TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static encode_tiled_fn get_encode_fn() {
  static encode_tiled_fn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<encode_tiled_fn>(sym);
  }
  return fn;
}

// (B, NH, S, D) bf16 view with element strides -> 4-D tiled map, box = 64 features x 64 tokens, 128-byte swizzle.
// Dimension 0 is D; the other three are ordered by ascending stride (extent-1 dimensions last, with a
// synthetic stride) and `pos` reports where token / head / batch ended up.
static int make_map(CUtensorMap* m, int pos[3], const void* base, int D, int S, int NH, int B, int64_t sb, int64_t sh,
                    int64_t st) {
  encode_tiled_fn enc = get_encode_fn();
  if (!enc) {
    set_last_cuda_error(cudaErrorSymbolNotFound, "cudaGetDriverEntryPoint(cuTensorMapEncodeTiled)");
    return XL_ERR_CUDA;
  }
  struct Dim { int kind; cuuint64_t extent; cuuint64_t stride; };
  Dim ds[3] = {{0, (cuuint64_t)S, (cuuint64_t)st * 2}, {1, (cuuint64_t)NH, (cuuint64_t)sh * 2}, {2, (cuuint64_t)B, (cuuint64_t)sb * 2}};
  // insertion sort: real dimensions by stride, extent-1 dimensions to the back
  for (int i = 1; i < 3; ++i)
    for (int j = i; j > 0; --j) {
      const bool a1 = ds[j - 1].extent == 1, b1 = ds[j].extent == 1;
      const bool swap = (a1 && !b1) || (a1 == b1 && !a1 && ds[j].stride < ds[j - 1].stride);
      if (!swap) break;
      Dim t = ds[j]; ds[j] = ds[j - 1]; ds[j - 1] = t;
    }
  cuuint64_t prev_stride = (cuuint64_t)D * 2, prev_extent = 1;
  for (int i = 0; i < 3; ++i) {
    if (ds[i].extent == 1) ds[i].stride = prev_stride * prev_extent;
    if (ds[i].stride % 16 != 0 || ds[i].stride == 0) return XL_ERR_BAD_STRIDE;
    prev_stride = ds[i].stride; prev_extent = ds[i].extent;
  }
  cuuint64_t dims[4] = {(cuuint64_t)D, ds[0].extent, ds[1].extent, ds[2].extent};
  cuuint64_t strides[3] = {ds[0].stride, ds[1].stride, ds[2].stride};
  cuuint32_t box[4] = {64, 1, 1, 1};
  for (int i = 0; i < 3; ++i) {
    pos[ds[i].kind] = i + 1;
    if (ds[i].kind == 0) box[i + 1] = 64;
  }
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled rejected the tensor layout");
    return XL_ERR_BAD_STRIDE;
  }
  return XL_OK;
}

int validate_seq_common(const xl_mlstm_seq_params* p);

template <int DHQK>
static int launch_chunkwise(const CwMaps& maps, const xl_mlstm_seq_params* p, cudaStream_t st) {
  using LY = CwLayout<DHQK>;
  static_assert(LY::DYN_SMEM <= 227 * 1024, "shared memory budget");
  const int nd = p->cu_seqlens ? p->num_docs : p->B;
  dim3 grid(p->DHV / CW_DV, p->NH, nd);
  auto kern = mlstm_chunkwise_kernel<DHQK>;
  XL_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, LY::DYN_SMEM));
  kern<<<grid, CW_THREADS, LY::DYN_SMEM, st>>>(maps, *p);
  return check_launch("xl_mlstm_chunkwise");
}

}  // namespace xl

extern "C" int xl_mlstm_chunkwise(const xl_mlstm_seq_params* p, void* cuda_stream) {
  using namespace xl;
  int rc = validate_seq_common(p);
  if (rc != XL_OK) return rc;
  if (p->dtype != XL_BF16) return XL_ERR_UNSUPPORTED;
  if (!(p->DHQK == 64 || p->DHQK == 128 || p->DHQK == 256) || p->DHV % CW_DV != 0) return XL_ERR_UNSUPPORTED;
  const int64_t strides[] = {p->q_sb, p->q_sh, p->q_st, p->k_sb, p->k_sh, p->k_st, p->v_sb, p->v_sh, p->v_st};
  for (int64_t s : strides)
    if (s < 0 || s % 8 != 0) return XL_ERR_BAD_STRIDE;  // TMA: strides are multiples of 16 bytes
  if (p->q_st < p->DHQK || p->k_st < p->DHQK || p->v_st < p->DHV) return XL_ERR_BAD_STRIDE;
  if (!aligned16(p->q) || !aligned16(p->k) || !aligned16(p->v) || !aligned16(p->h)) return XL_ERR_BAD_ALIGNMENT;
  if (p->h_sb % 8 || p->h_sh % 8 || p->h_st % 8) return XL_ERR_BAD_STRIDE;  // h leaves in 16-byte pieces
  CwMaps maps;
  if ((rc = make_map(&maps.q, maps.pos[0], p->q, p->DHQK, p->S, p->NH, p->B, p->q_sb, p->q_sh, p->q_st)) != XL_OK) return rc;
  if ((rc = make_map(&maps.k, maps.pos[1], p->k, p->DHQK, p->S, p->NH, p->B, p->k_sb, p->k_sh, p->k_st)) != XL_OK) return rc;
  if ((rc = make_map(&maps.v, maps.pos[2], p->v, p->DHV, p->S, p->NH, p->B, p->v_sb, p->v_sh, p->v_st)) != XL_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  switch (p->DHQK) {
    case 64: return launch_chunkwise<64>(maps, p, st);
    case 128: return launch_chunkwise<128>(maps, p, st);
    default: return launch_chunkwise<256>(maps, p, st);
  }
}
