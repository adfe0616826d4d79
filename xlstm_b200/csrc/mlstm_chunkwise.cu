// mLSTM chunkwise-parallel forward on tcgen05 tensor cores (sm_100a), bf16 operands, fp32 state.
//
// One CTA owns a 128-column slice (of DHV) of one (document, head) and walks that document's 64-token
// chunks in order.  Its slice of the matrix state lives TRANSPOSED in tensor memory for the whole
// document, C^T[dv, dqk] (128 lanes x DHQK fp32 columns), and is never written to HBM between chunks.
// Per chunk, with b_j the in-chunk cumulative log forget gate, a'_j = i_j - b_j, mu_j = max(m_prev,
// max_{l<=j} a'_l), mu* = mu_63 and g = b_63 (equivalent to xlstm/blocks/mlstm/backends.py:173-258):
//
//   S      = Q K^T                               UMMA  M=64  N=64   K=DHQK   (both operands K-major, TMA tiles)
//   P_jl   = S_jl/sqrt(DHQK) * exp(a'_l - mu_j)  (l <= j)   CUDA cores, written as bf16 K-major tile
//   H^T    = Cb^T (r_j q~_j)^T                   UMMA  M=128 N=64   K=DHQK   A = bf16 copy of C^T in TMEM,
//                                                                           r_j = exp(m_prev - mu_j)
//   H^T   += V^T P^T                             UMMA  M=128 N=64   K=64     A = V tile used MN-major
//   C^T    = exp(m_prev - mu*) C^T + (w V)^T K   UMMA  M=128 N=DHQK K=64     w_l = exp(a'_l - mu*), both MN-major
//   h_j    = H_j / (max(|q~_j.n_j|, exp(-(b_j + mu_j))) + eps) ,   m_new = g + mu*
//
// All UMMAs run with M = 128 except S.  q, k, v tiles arrive by TMA (128-byte swizzle) straight from the
// caller's strided (B, NH, S, D) views; documents are chunked from their own first token, so a chunk never
// straddles a document boundary and the tail chunk is masked (i = -inf, log f = 0) instead of padded.
#include <cuda.h>

#include "common.cuh"

namespace xl {

constexpr int CW_L = 64;         // tokens per chunk
constexpr int CW_DV = 128;       // value columns per CTA (UMMA M)
constexpr int CW_THREADS = 128;  // 4 warps; warp w owns TMEM lanes [32w, 32w+32)
constexpr int CW_STAGES = 2;
constexpr int CW_BOX_BYTES = 64 * 128;  // one TMA box: 64 rows x 64 bf16
constexpr uint32_t CW_TMEM_COLS = 512;

template <int DHQK>
struct CwLayout {
  static constexpr int NKB = DHQK / 64;                       // 64-wide boxes along DHQK
  static constexpr int Q_BYTES = NKB * CW_BOX_BYTES;
  static constexpr int V_BYTES = 2 * CW_BOX_BYTES;
  static constexpr int STAGE_BYTES = 2 * Q_BYTES + V_BYTES;    // q, k, v of one chunk
  static constexpr int OFF_STAGE = 0;
  static constexpr int OFF_QS = CW_STAGES * STAGE_BYTES;       // r_j-scaled q
  static constexpr int OFF_VH = OFF_QS + Q_BYTES;              // w_l-scaled v
  static constexpr int OFF_P = OFF_VH + V_BYTES;               // P tile
  static constexpr int OFF_F32 = OFF_P + CW_BOX_BYTES;         // small fp32 arrays
  static constexpr int N_F32 = 7 * CW_L + DHQK + 8;
  static constexpr int OFF_BAR = OFF_F32 + N_F32 * 4;          // mbarriers (8-byte aligned)
  static constexpr int TOTAL = OFF_BAR + 8 * 8;
  static constexpr int DYN_SMEM = TOTAL + 1024;                // slack to align the base to 1024 B
  // tensor-memory column map
  static constexpr uint32_t T_C = 0;            // C^T fp32           DHQK columns
  static constexpr uint32_t T_CB = 256;         // bf16 copy of C^T   DHQK/2 columns
  static constexpr uint32_t T_H = 384;          // H^T accumulator    64 columns
  static constexpr uint32_t T_S = 448;          // S accumulator      64 columns (M=64: lanes 0-15 of each warp)
};

struct CwMaps {
  CUtensorMap q, k, v;
  // position (1..3) of the token / head / batch coordinate in each map; the outer dimensions are ordered by
  // ascending stride, which differs between a contiguous (B,NH,S,D) tensor and a transposed (B,S,NH,D) view
  int pos[3][3];  // [q|k|v][token|head|batch]
};

template <int DHQK>
__global__ void __launch_bounds__(CW_THREADS, 1)
mlstm_chunkwise_kernel(const __grid_constant__ CwMaps maps, const xl_mlstm_seq_params p) {
  using LY = CwLayout<DHQK>;
  constexpr int NKB = LY::NKB;
  extern __shared__ unsigned char cw_smem_raw[];
  // 128-byte-swizzled tiles need 1024-byte aligned bases
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(cw_smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  float* s_f = reinterpret_cast<float*>(smem + LY::OFF_F32);
  float* s_b = s_f;                  // b_j
  float* s_ap = s_f + 1 * CW_L;      // a'_j
  float* s_mu = s_f + 2 * CW_L;      // mu_j
  float* s_r = s_f + 3 * CW_L;       // r_j * 1/sqrt(DHQK)
  float* s_w = s_f + 4 * CW_L;       // w_l
  float* s_qn = s_f + 5 * CW_L;      // q_j . n_prev (raw q)
  float* s_inv = s_f + 6 * CW_L;     // 1 / denominator
  float* s_n = s_f + 7 * CW_L;       // n state, DHQK
  float* s_tmp = s_n + DHQK;         // 8 scratch words
  const uint32_t bar_full0 = sbase + LY::OFF_BAR;        // +8*stage
  const uint32_t bar_s = sbase + LY::OFF_BAR + 16;
  const uint32_t bar_m2 = sbase + LY::OFF_BAR + 24;
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + LY::OFF_BAR + 32);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
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
  const int dv = warp * 32 + lane;                      // this thread's TMEM lane = value column within the slice
  const float* c0 = p.c0 ? p.c0 + (sidx * DHQK) * DHV + col0 + dv : nullptr;
  float* c_out = p.c_out + (sidx * DHQK) * DHV + col0 + dv;

  if (len <= 0) {  // empty document: the state passes through unchanged
    for (int d = 0; d < DHQK; ++d) c_out[(long long)d * DHV] = c0 ? c0[(long long)d * DHV] : 0.f;
    if (slice == 0) {
      for (int d = tid; d < DHQK; d += CW_THREADS) p.n_out[sidx * DHQK + d] = p.n0 ? p.n0[sidx * DHQK + d] : 0.f;
      if (tid == 0) p.m_out[sidx] = p.m0 ? p.m0[sidx] : 0.f;
    }
    return;
  }
  const int nchunks = (int)((len + CW_L - 1) / CW_L);

  // ---- one-time setup: barriers, tensor memory
  if (tid == 0) {
    mbar_init(bar_full0, 1);
    mbar_init(bar_full0 + 8, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_m2, 1);
    fence_barrier_init();
    tma_prefetch_desc(&maps.q);
    tma_prefetch_desc(&maps.k);
    tma_prefetch_desc(&maps.v);
  }
  if (warp == 0) {
    __syncwarp();
    tmem_alloc(smem_u32(s_tmem), CW_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *s_tmem;
  const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
  const uint32_t tC = tmem + LY::T_C + lane_base, tCb = tmem + LY::T_CB + lane_base;
  const uint32_t tH = tmem + LY::T_H + lane_base, tS = tmem + LY::T_S + lane_base;

  auto issue_tma = [&](int chunk) {  // thread 0 only
    const int st = chunk % CW_STAGES;
    const uint32_t bar = bar_full0 + 8 * st;
    const uint32_t dst = sbase + LY::OFF_STAGE + st * LY::STAGE_BYTES;
    const int t = (int)(tok0 + (long long)chunk * CW_L);
    mbar_expect_tx(bar, LY::STAGE_BYTES);
    int cq[4], ck[4], cv[4];
    cq[maps.pos[0][0]] = t; cq[maps.pos[0][1]] = head; cq[maps.pos[0][2]] = b;
    ck[maps.pos[1][0]] = t; ck[maps.pos[1][1]] = head; ck[maps.pos[1][2]] = b;
    cv[maps.pos[2][0]] = t; cv[maps.pos[2][1]] = head; cv[maps.pos[2][2]] = b;
#pragma unroll
    for (int kb = 0; kb < NKB; ++kb) {
      tma_load_4d(dst + kb * CW_BOX_BYTES, &maps.q, bar, kb * 64, cq[1], cq[2], cq[3]);
      tma_load_4d(dst + LY::Q_BYTES + kb * CW_BOX_BYTES, &maps.k, bar, kb * 64, ck[1], ck[2], ck[3]);
    }
#pragma unroll
    for (int vb = 0; vb < 2; ++vb)
      tma_load_4d(dst + 2 * LY::Q_BYTES + vb * CW_BOX_BYTES, &maps.v, bar, col0 + vb * 64, cv[1], cv[2], cv[3]);
  };
  if (tid == 0) {
    issue_tma(0);
    if (nchunks > 1) issue_tma(1);
  }

  // ---- initial state: C^T into tensor memory, n into shared memory
#pragma unroll 1
  for (int cb = 0; cb < DHQK / 32; ++cb) {
    uint32_t r[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) r[i] = c0 ? __float_as_uint(c0[(long long)(cb * 32 + i) * DHV]) : 0u;
    tmem_st_x32(tC + cb * 32, r);
  }
  tc_wait_st();
  for (int d = tid; d < DHQK; d += CW_THREADS) s_n[d] = p.n0 ? p.n0[sidx * DHQK + d] : 0.f;
  float m_prev = p.m0 ? p.m0[sidx] : 0.f;
  const float qscale = rsqrtf((float)DHQK);

  const float* ig = p.igate + b * p.g_sb + head * p.g_sh + tok0 * p.g_st;
  const float* fg = p.fgate + b * p.g_sb + head * p.g_sh + tok0 * p.g_st;
  __nv_bfloat16* hout = reinterpret_cast<__nv_bfloat16*>(p.h) + b * p.h_sb + head * p.h_sh + tok0 * p.h_st + col0 + dv;

  // gate prefetch for chunk 0 (threads 0..63 own token j = tid)
  float g_i = -INFINITY, g_f = 0.f;
  if (tid < CW_L && tid < len) {
    g_i = ig[(long long)tid * p.g_st];
    g_f = fg[(long long)tid * p.g_st];
  }
  tc_fence_before();
  __syncthreads();

  constexpr uint32_t IDESC_S = umma_idesc_bf16(64, 64, 0, 0);
  constexpr uint32_t IDESC_HI = umma_idesc_bf16(128, 64, 0, 0);
  constexpr uint32_t IDESC_HV = umma_idesc_bf16(128, 64, 1, 0);
  constexpr uint32_t IDESC_C = umma_idesc_bf16(128, DHQK, 1, 1);

  bool ok = true;
#pragma unroll 1
  for (int chunk = 0; chunk < nchunks; ++chunk) {
    const int st = chunk % CW_STAGES;
    const uint32_t par_full = (uint32_t)(chunk / CW_STAGES) & 1u, par = (uint32_t)chunk & 1u;
    const uint32_t s_q = sbase + LY::OFF_STAGE + st * LY::STAGE_BYTES, s_k = s_q + LY::Q_BYTES, s_v = s_k + LY::Q_BYTES;
    const long long rem = len - (long long)chunk * CW_L;
    const int len_c = rem < CW_L ? (int)rem : CW_L;

    // this chunk's gates (prefetched), then prefetch the next chunk's
    const float cur_i = g_i, cur_f = g_f;
    {
      const long long jn = (long long)(chunk + 1) * CW_L + tid;
      g_i = -INFINITY; g_f = 0.f;
      if (tid < CW_L && jn < len) {
        g_i = ig[jn * p.g_st];
        g_f = fg[jn * p.g_st];
      }
    }

    // (A) operands of this chunk have landed
    if (!mbar_wait(bar_full0 + 8 * st, par_full)) { ok = false; break; }

    // (B) S = Q K^T
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int kb = 0; kb < NKB; ++kb)
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint64_t ad = umma_desc_sw128(s_q + kb * CW_BOX_BYTES + kk * 32, 16, 1024);
          const uint64_t bd = umma_desc_sw128(s_k + kb * CW_BOX_BYTES + kk * 32, 16, 1024);
          umma_ss(tmem + LY::T_S, ad, bd, IDESC_S, (kb | kk) != 0);
        }
      umma_commit(bar_s);
    }

    // (C) gate scans over the chunk (threads 0..63 carry token j = tid; all threads run the shuffles)
    float lf = (tid < len_c) ? log_sigmoid(cur_f) : 0.f;
    float bj = lf;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float t = __shfl_up_sync(0xffffffffu, bj, o);
      if (lane >= o) bj += t;
    }
    if (tid == 31) s_tmp[0] = bj;
    __syncthreads();
    if (warp == 1) bj += s_tmp[0];
    const float ap = (tid < len_c) ? cur_i - bj : -INFINITY;
    float cm = ap;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float t = __shfl_up_sync(0xffffffffu, cm, o);
      if (lane >= o) cm = fmaxf(cm, t);
    }
    if (tid == 31) s_tmp[1] = cm;
    __syncthreads();
    if (warp == 1) cm = fmaxf(cm, s_tmp[1]);
    const float mu = fmaxf(m_prev, cm);
    if (tid < CW_L) {
      s_b[tid] = bj;
      s_ap[tid] = ap;
      s_mu[tid] = mu;
      s_r[tid] = expf(m_prev - mu) * qscale;
    }
    if (tid == CW_L - 1) { s_tmp[2] = mu; s_tmp[3] = bj; }
    __syncthreads();
    const float mu_star = s_tmp[2], gsum = s_tmp[3];
    if (tid < CW_L) s_w[tid] = expf(ap - mu_star);
    const float decay = expf(m_prev - mu_star);
    const float m_new = gsum + mu_star;
    __syncthreads();

    // (D) r_j-scaled q (bf16, same swizzled layout), q~_j . n_prev, and w_l-scaled v
    {
      const int j = tid >> 1, half = tid & 1;
      const float rj = s_r[j];
      float dot = 0.f;
      constexpr int CH = NKB * 4;  // 16-byte pieces per thread
#pragma unroll 4
      for (int i = 0; i < CH; ++i) {
        const int cidx = half * CH + i;
        const int box = cidx >> 3;
        const int c = (NKB >= 2) ? ((cidx & 7) ^ (half << 2)) : (cidx & 7);
        const uint32_t off = box * CW_BOX_BYTES + j * 128 + ((c ^ (j & 7)) << 4);
        const uint4 raw = *reinterpret_cast<const uint4*>(smem + (s_q - sbase) + off);
        const float4 n0 = *reinterpret_cast<const float4*>(s_n + box * 64 + c * 8);
        const float4 n1 = *reinterpret_cast<const float4*>(s_n + box * 64 + c * 8 + 4);
        const float2 e0 = unpack_bf16x2(raw.x), e1 = unpack_bf16x2(raw.y), e2 = unpack_bf16x2(raw.z), e3 = unpack_bf16x2(raw.w);
        dot += e0.x * n0.x + e0.y * n0.y + e1.x * n0.z + e1.y * n0.w + e2.x * n1.x + e2.y * n1.y + e3.x * n1.z + e3.y * n1.w;
        uint4 o;
        o.x = pack_bf16x2(e0.x * rj, e0.y * rj);
        o.y = pack_bf16x2(e1.x * rj, e1.y * rj);
        o.z = pack_bf16x2(e2.x * rj, e2.y * rj);
        o.w = pack_bf16x2(e3.x * rj, e3.y * rj);
        *reinterpret_cast<uint4*>(smem + LY::OFF_QS + off) = o;
      }
      dot += __shfl_xor_sync(0xffffffffu, dot, 1);
      if (half == 0) s_qn[j] = dot;
      // v tile: row l = j, this thread's box = half
      const float wl = s_w[j];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int c = i ^ (half << 2);
        const uint32_t off = half * CW_BOX_BYTES + j * 128 + ((c ^ (j & 7)) << 4);
        const uint4 raw = *reinterpret_cast<const uint4*>(smem + (s_v - sbase) + off);
        const float2 e0 = unpack_bf16x2(raw.x), e1 = unpack_bf16x2(raw.y), e2 = unpack_bf16x2(raw.z), e3 = unpack_bf16x2(raw.w);
        uint4 o;
        o.x = pack_bf16x2(e0.x * wl, e0.y * wl);
        o.y = pack_bf16x2(e1.x * wl, e1.y * wl);
        o.z = pack_bf16x2(e2.x * wl, e2.y * wl);
        o.w = pack_bf16x2(e3.x * wl, e3.y * wl);
        *reinterpret_cast<uint4*>(smem + LY::OFF_VH + off) = o;
      }
    }
    fence_proxy_async_smem();

    // (E) C^T: bf16 copy for the inter-chunk product, then decay in place
#pragma unroll 1
    for (int cb = 0; cb < DHQK / 32; ++cb) {
      uint32_t r[32];
      tmem_ld_x32(tC + cb * 32, r);
      tc_wait_ld();
      uint32_t pk[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) pk[i] = pack_bf16x2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
      tmem_st_x16(tCb + cb * 16, pk);
#pragma unroll
      for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * decay);
      tmem_st_x32(tC + cb * 32, r);
    }
    tc_wait_st();
    tc_fence_before();
    __syncthreads();

    // (F) H^T = Cb^T (r q~)^T
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < DHQK / 16; ++ks) {
        const uint64_t bd = umma_desc_sw128(sbase + LY::OFF_QS + (ks >> 2) * CW_BOX_BYTES + (ks & 3) * 32, 16, 1024);
        umma_ts(tmem + LY::T_H, tmem + LY::T_CB + ks * 8, bd, IDESC_HI, ks != 0);
      }
    }

    // (G) P from S; denominators
    if (!mbar_wait(bar_s, par)) { ok = false; break; }
    tc_fence_after();
    {
      uint32_t sv[64];
      {
        uint32_t t0[32], t1[32];
        tmem_ld_x32(tS, t0);
        tmem_ld_x32(tS + 32, t1);
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) { sv[i] = t0[i]; sv[32 + i] = t1[i]; }
      }
      if (lane < 16) {
        const int j = warp * 16 + lane;
        const float muj = s_mu[j];
        float rowsum = 0.f;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          float e[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int l = c * 8 + i;
            const float x = __uint_as_float(sv[l]) * qscale * __expf(s_ap[l] - muj);
            e[i] = (l <= j) ? x : 0.f;
          }
          uint4 o;
          o.x = pack_bf16x2(e[0], e[1]);
          o.y = pack_bf16x2(e[2], e[3]);
          o.z = pack_bf16x2(e[4], e[5]);
          o.w = pack_bf16x2(e[6], e[7]);
          const float2 f0 = unpack_bf16x2(o.x), f1 = unpack_bf16x2(o.y), f2 = unpack_bf16x2(o.z), f3 = unpack_bf16x2(o.w);
          rowsum += (f0.x + f0.y) + (f1.x + f1.y) + (f2.x + f2.y) + (f3.x + f3.y);
          *reinterpret_cast<uint4*>(smem + LY::OFF_P + j * 128 + ((c ^ (j & 7)) << 4)) = o;
        }
        const float qn = rowsum + s_r[j] * s_qn[j];  // s_r already carries 1/sqrt(DHQK)
        const float den = fmaxf(fabsf(qn), expf(-(s_b[j] + muj))) + p.eps;
        s_inv[j] = 1.f / den;
      }
    }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();

    // (H) H^T += V^T P^T ;  C^T += (w V)^T K
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const uint64_t ad = umma_desc_sw128(s_v + kk * 2048, CW_BOX_BYTES, 1024);
        const uint64_t bd = umma_desc_sw128(sbase + LY::OFF_P + kk * 32, 16, 1024);
        umma_ss(tmem + LY::T_H, ad, bd, IDESC_HV, 1);
      }
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const uint64_t ad = umma_desc_sw128(sbase + LY::OFF_VH + kk * 2048, CW_BOX_BYTES, 1024);
        const uint64_t bd = umma_desc_sw128(s_k + kk * 2048, CW_BOX_BYTES, 1024);
        umma_ss(tmem + LY::T_C, ad, bd, IDESC_C, 1);
      }
      umma_commit(bar_m2);
    }

    // (I) n = decay n + sum_l w_l k_l   (thread owns two adjacent key features)
    if (2 * tid < DHQK) {
      const int d = 2 * tid, box = d >> 6, c = (d & 63) >> 3, within = (d & 7) * 2;
      const unsigned char* kt = smem + (s_k - sbase) + box * CW_BOX_BYTES + within;
      float a0 = 0.f, a1 = 0.f;
#pragma unroll 8
      for (int l = 0; l < CW_L; ++l) {
        const float2 kv = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(kt + l * 128 + ((c ^ (l & 7)) << 4)));
        const float wl = s_w[l];
        a0 = fmaf(wl, kv.x, a0);
        a1 = fmaf(wl, kv.y, a1);
      }
      s_n[d] = fmaf(decay, s_n[d], a0);
      s_n[d + 1] = fmaf(decay, s_n[d + 1], a1);
    }

    // (J) epilogue: normalise and store this chunk's h (thread = value column, loop over tokens)
    if (!mbar_wait(bar_m2, par)) { ok = false; break; }
    tc_fence_after();
    {
      uint32_t hv[64];
      {
        uint32_t t0[32], t1[32];
        tmem_ld_x32(tH, t0);
        tmem_ld_x32(tH + 32, t1);
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) { hv[i] = t0[i]; hv[32 + i] = t1[i]; }
      }
      __nv_bfloat16* ho = hout + (long long)chunk * CW_L * p.h_st;
#pragma unroll
      for (int j = 0; j < CW_L; ++j)
        if (j < len_c) ho[(long long)j * p.h_st] = __float2bfloat16_rn(__uint_as_float(hv[j]) * s_inv[j]);
    }
    m_prev = m_new;
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && chunk + CW_STAGES < nchunks) issue_tma(chunk + CW_STAGES);
  }

  // ---- final state
  if (ok) {
    tc_fence_after();
#pragma unroll 1
    for (int cb = 0; cb < DHQK / 32; ++cb) {
      uint32_t r[32];
      tmem_ld_x32(tC + cb * 32, r);
      tc_wait_ld();
#pragma unroll
      for (int i = 0; i < 32; ++i) c_out[(long long)(cb * 32 + i) * DHV] = __uint_as_float(r[i]);
    }
    if (slice == 0) {
      for (int d = tid; d < DHQK; d += CW_THREADS) p.n_out[sidx * DHQK + d] = s_n[d];
      if (tid == 0) p.m_out[sidx] = m_prev;
    }
  } else {
    if (p.status && tid == 0) atomicExch(p.status, 1);
    // give copies that may still be in flight a bounded chance to land before the CTA's memory is released
    (void)mbar_wait(bar_full0, 0);
    (void)mbar_wait(bar_full0 + 8, 0);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, CW_TMEM_COLS);
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
  XL_CUDA_TRY(cudaFuncSetAttribute(mlstm_chunkwise_kernel<DHQK>, cudaFuncAttributeMaxDynamicSharedMemorySize, LY::DYN_SMEM));
  const int nd = p->cu_seqlens ? p->num_docs : p->B;
  dim3 grid(p->DHV / CW_DV, p->NH, nd), block(CW_THREADS);
  mlstm_chunkwise_kernel<DHQK><<<grid, block, LY::DYN_SMEM, st>>>(maps, *p);
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
  if (!aligned16(p->q) || !aligned16(p->k) || !aligned16(p->v)) return XL_ERR_BAD_ALIGNMENT;
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
