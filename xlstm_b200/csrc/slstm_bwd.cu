// sLSTM backward through time in ONE persistent kernel (the counterpart of the reference's host loop
// BackwardPass::Run + SLSTMPointwiseBackward: xlstm/blocks/slstm/src/cuda/slstm_backward.cu,
// slstm_pointwise.cu:118-196).
//
// Same mapping as the forward kernel: one thread-block cluster of DH/32 CTAs per (head, 16-row batch group), CTA r
// owns hidden units [32r, 32r+32) with all four gates, a thread owns four (row, unit) pairs and keeps their gradient
// carries dc, dn in fp32 registers for the whole sequence.  Per step, walking t = S-1 .. 0:
//   dy = dh_t (from above) + dh_t (recurrent);  dc += dy o / n';  dn -= dy h' / n'
//   dg_i = i' (z dc + dn);  dg_f = f' (dc c + dn n)(1 - sigmoid(f));  dg_z = dc i' (1 - z^2);  dg_o = (1 - o) h' dy
//   dc <- f' dc;  dn <- f' dn          (the stabiliser m is a constant of the step, as in the reference)
// with i', raw f, z = tanh, o = sigmoid, h', c', n', m' read from the cache the training forward wrote (one 96-byte
// record per thread and step, streamed through a cp.async ring), and
//   dh_{t-1}[b,k] = sum_{g,u} dg_t[b,g,u] R[k,g,u].
// The CTA holds exactly the slice of R the forward holds (all k, its own 32 units, four gates) as mma.sync
// B-fragments in registers, now contracted over (g,u): it forms the PARTIAL sums of dh_{t-1} for all DH columns
// from its own 128 gate gradients (M = 16 rows, N = DH, K = 128), stages them per destination in shared memory and
// sends every 32-column block to the CTA that owns those units with ONE bulk asynchronous copy into that CTA's
// shared memory, which counts its bytes on the receiver's mbarrier (a reduce-scatter: DH/32 copies of 2.3 KB per CTA
// and step; the same exchange as 2 048 eight-byte remote stores per CTA cost 1 200 cycles of issue per step); the
// receiver adds the DH/32 partials in rank order.  Everything of a step's gate arithmetic that does not depend on
// the incoming gradient is computed one step ahead, while the partials are in flight.
// dWx_t = dg_t leaves as bf16 in the layout of Wx.  dR and dbias are sums over (b,t) of h_{t-1} (x) dg_t and of dg_t:
// plain matrix products over the dWx this kernel writes, left to the caller's GEMM library.
#include "common.cuh"
#include "slstm_common.cuh"

namespace xl {

constexpr int SLB_DG_STRIDE = 4 * SL_UNITS + 8;          // bf16 elements per row of the dg tile (+16 B: bank spread)
constexpr int SLB_REC_STEP = SL_THREADS * SL_REC_BYTES;  // cache bytes per CTA and step
constexpr int SLB_PROW = SL_UNITS + 4;                   // floats per row of a partial block (+16 B: rows on distinct banks)
constexpr int SLB_PBLOCK = SL_ROWS * SLB_PROW * 4;       // bytes of one (source, destination) block of partial sums

__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
// bulk copy from this CTA's shared memory into (another) CTA's, counted on an mbarrier of the destination CTA
__device__ __forceinline__ void bulk_copy_to_cta(uint32_t remote_dst, uint32_t local_src, uint32_t bytes, uint32_t remote_bar) {
  asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(remote_dst),
               "r"(local_src), "r"(bytes), "r"(remote_bar)
               : "memory");
}

template <int DH>
__global__ void __launch_bounds__(SL_THREADS, 1) slstm_backward_kernel(const xl_slstm_bwd_params p) {
  constexpr int NCTA = DH / SL_UNITS;
  constexpr int NTW = DH / 32;              // n8 tiles (8 columns of dh_{t-1}) per warp
  constexpr int KS = 4 * SL_UNITS / 16;     // k-steps over the CTA's 128 gate gradients
  constexpr uint32_t RB_BYTES = NCTA * SLB_PBLOCK;   // what one step delivers to a CTA
  extern __shared__ __align__(16) unsigned char slb_smem[];
  __nv_bfloat16* s_dg = reinterpret_cast<__nv_bfloat16*>(slb_smem);                   // [16][SLB_DG_STRIDE]
  float* s_rb = reinterpret_cast<float*>(slb_smem + SL_ROWS * SLB_DG_STRIDE * 2);     // received: [2][source CTA][16][SLB_PROW]
  float* s_st = s_rb + 2 * RB_BYTES / 4;                                              // staged: [2][destination CTA][16][SLB_PROW]
  unsigned char* s_rec = reinterpret_cast<unsigned char*>(s_st) + 2 * RB_BYTES;       // [SL_RING][SLB_REC_STEP]
  uint32_t* s_dh = reinterpret_cast<uint32_t*>(s_rec + SL_RING * SLB_REC_STEP);       // [SL_RING][128][2]
  const uint32_t s_bar = smem_u32(s_dh + SL_RING * SL_THREADS * 2);                   // 2 mbarriers

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t rank = cluster_ctarank();
  const int head = blockIdx.y, bgroup = blockIdx.z;
  const int B = p.B, S = p.S, NH = p.NH, H = NH * DH;
  const int row_a = lane >> 2, row_b = row_a + 8;
  const int unit_l = warp * 8 + (lane & 3) * 2;
  const int unit_h = (int)rank * SL_UNITS + unit_l;
  const int gb_a = bgroup * SL_ROWS + row_a, gb_b = bgroup * SL_ROWS + row_b;
  const bool ok_a = gb_a < B, ok_b = gb_b < B;

  // ---- the CTA's slice of R as B fragments of dh[b,k] = sum_{(g,u)} dg[b,(g,u)] R[k,g,u]:  n = k, contraction index
  // kk = 32 g + (u - 32 rank); a fragment register holds two adjacent u of one (k, g)
  uint32_t bfrag[NTW][KS][2];
  {
    const __nv_bfloat16* R = reinterpret_cast<const __nv_bfloat16*>(p.R) + (size_t)head * DH * 4 * DH;
    const int k0 = (lane & 3) * 2;
#pragma unroll
    for (int j = 0; j < NTW; ++j) {
      const int k_in = (warp * NTW + j) * 8 + (lane >> 2);
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        const int g = ks >> 1, u = (int)rank * SL_UNITS + (ks & 1) * 16 + k0;
        const __nv_bfloat16* base = R + ((size_t)k_in * 4 + g) * DH + u;
        bfrag[j][ks][0] = *reinterpret_cast<const uint32_t*>(base);
        bfrag[j][ks][1] = *reinterpret_cast<const uint32_t*>(base + 8);
      }
    }
  }

  // ---- gradient carries and the recurrent part of dh for the thread's four pairs, from the gradient of the final state
  float dc_[4], dn_[4], dhrec[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gb = (i < 2) ? gb_a : gb_b;
    const bool okr = (i < 2) ? ok_a : ok_b;
    const size_t off = (size_t)gb * H + (size_t)head * DH + unit_h + (i & 1);
    const bool have = p.dstate_out != nullptr && okr;
    dhrec[i] = have ? p.dstate_out[0 * (size_t)B * H + off] : 0.f;
    dc_[i] = have ? p.dstate_out[1 * (size_t)B * H + off] : 0.f;
    dn_[i] = have ? p.dstate_out[2 * (size_t)B * H + off] : 0.f;
  }

  if (tid == 0) {
    mbar_init(s_bar, 1);      // one arrival per phase: the local expect_tx
    mbar_init(s_bar + 8, 1);
    fence_barrier_init();
  }

  // ---- cache and dh rings: every thread fetches ITS record (6 x 16 B) and its two dh words of a step
  const unsigned char* cache = reinterpret_cast<const unsigned char*>(p.cache) +
                               ((((size_t)bgroup * NH + head) * NCTA + rank) * (size_t)S * SL_THREADS + tid) * SL_REC_BYTES;
  const __nv_bfloat16* dh = reinterpret_cast<const __nv_bfloat16*>(p.dh);
  const size_t dh_a = ((size_t)(ok_a ? gb_a : B - 1) * NH + head) * (size_t)S * DH + unit_h;
  const size_t dh_b = ((size_t)(ok_b ? gb_b : B - 1) * NH + head) * (size_t)S * DH + unit_h;
  const uint32_t s_rec_u32 = smem_u32(s_rec) + tid * SL_REC_BYTES, s_dh_u32 = smem_u32(s_dh) + tid * 8;
  auto issue = [&](int t) {
    if (t >= 0) {
      const unsigned char* src = cache + (size_t)t * SLB_REC_STEP;
      const uint32_t dst = s_rec_u32 + (t % SL_RING) * SLB_REC_STEP;
#pragma unroll
      for (int j = 0; j < SL_REC_BYTES / 16; ++j) cp_async16(dst + j * 16, src + j * 16);
      const uint32_t dd = s_dh_u32 + (t % SL_RING) * (SL_THREADS * 8);
      cp_async4(dd, dh + dh_a + (size_t)t * DH);
      cp_async4(dd + 4, dh + dh_b + (size_t)t * DH);
    }
    cp_async_commit();
  };
#pragma unroll
  for (int j = 0; j < SL_RING - 1; ++j) issue(S - 1 - j);
  cluster_barrier();  // every CTA's barriers exist before anything crosses over; also a CTA-wide barrier

  const uint32_t s_dg_u32 = smem_u32(s_dg), s_rb_u32 = smem_u32(s_rb), s_st_u32 = smem_u32(s_st);
  const uint32_t ldm_off = ((lane & 15) * SLB_DG_STRIDE + (lane >> 4) * 8) * 2;
  __nv_bfloat16* dwx = reinterpret_cast<__nv_bfloat16*>(p.dwx);

  // Per pair, everything of a step that does not depend on the incoming gradient (formed one step ahead):
  //   dc = dc_carry + dy pa;  dn = dn_carry - dy pb;  dg_i = pig (pzt dc + dn);  dg_f = pff (dc pcp + dn pnp);
  //   dg_z = dc pz2;  dg_o = po2 dy;  carries <- pfg (dc, dn);  dy = dup + recurrent part
  float pa[4], pb[4], pig[4], pzt[4], pfg[4], pff[4], pcp[4], pnp[4], pz2[4], po2[4], dup[4];
  auto precompute = [&](int t) {
    const unsigned char* rt = s_rec + (t % SL_RING) * SLB_REC_STEP + tid * SL_REC_BYTES;
    const uint4 ga = *reinterpret_cast<const uint4*>(rt), gbw = *reinterpret_cast<const uint4*>(rt + 16);
    const uint2 hw = *reinterpret_cast<const uint2*>(rt + 32);
    const float4 n_new = *reinterpret_cast<const float4*>(rt + 64), m_new = *reinterpret_cast<const float4*>(rt + 80);
    float4 c_prev, n_prev, m_prev;
    if (t > 0) {
      const unsigned char* rp = s_rec + ((t - 1) % SL_RING) * SLB_REC_STEP + tid * SL_REC_BYTES;
      c_prev = *reinterpret_cast<const float4*>(rp + 48);
      n_prev = *reinterpret_cast<const float4*>(rp + 64);
      m_prev = *reinterpret_cast<const float4*>(rp + 80);
    } else {
      float cp[4], np[4], mp[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int gb = (i < 2) ? gb_a : gb_b;
        const bool okr = (i < 2) ? ok_a : ok_b;
        const size_t off = (size_t)gb * H + (size_t)head * DH + unit_h + (i & 1);
        const bool have = p.state0 != nullptr && okr;
        cp[i] = have ? p.state0[1 * (size_t)B * H + off] : 0.f;
        np[i] = have ? p.state0[2 * (size_t)B * H + off] : 0.f;
        mp[i] = have ? p.state0[3 * (size_t)B * H + off] : 0.f;
      }
      c_prev = make_float4(cp[0], cp[1], cp[2], cp[3]);
      n_prev = make_float4(np[0], np[1], np[2], np[3]);
      m_prev = make_float4(mp[0], mp[1], mp[2], mp[3]);
    }
    const uint2 dhw = *reinterpret_cast<const uint2*>(s_dh + (t % SL_RING) * (SL_THREADS * 2) + tid * 2);
    const float2 ia = unpack_bf16x2(ga.x), fa = unpack_bf16x2(ga.y), za = unpack_bf16x2(ga.z), oa = unpack_bf16x2(ga.w);
    const float2 ib = unpack_bf16x2(gbw.x), fb = unpack_bf16x2(gbw.y), zb = unpack_bf16x2(gbw.z), ob = unpack_bf16x2(gbw.w);
    const float2 ya = unpack_bf16x2(hw.x), yb = unpack_bf16x2(hw.y);
    const float2 da = unpack_bf16x2(dhw.x), db = unpack_bf16x2(dhw.y);
    const float ig[4] = {ia.x, ia.y, ib.x, ib.y}, fr[4] = {fa.x, fa.y, fb.x, fb.y};
    const float zt[4] = {za.x, za.y, zb.x, zb.y}, os[4] = {oa.x, oa.y, ob.x, ob.y};
    const float yn[4] = {ya.x, ya.y, yb.x, yb.y};
    const float du[4] = {ok_a ? da.x : 0.f, ok_a ? da.y : 0.f, ok_b ? db.x : 0.f, ok_b ? db.y : 0.f};
    const float nn[4] = {n_new.x, n_new.y, n_new.z, n_new.w}, mn[4] = {m_new.x, m_new.y, m_new.z, m_new.w};
    const float cp[4] = {c_prev.x, c_prev.y, c_prev.z, c_prev.w}, np[4] = {n_prev.x, n_prev.y, n_prev.z, n_prev.w};
    const float mp[4] = {m_prev.x, m_prev.y, m_prev.z, m_prev.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float rn = __fdividef(1.f, nn[i]);
      const float fg = fminf(1.f, __expf(fast_logsigmoid(fr[i]) + mp[i] - mn[i]));
      const float fsig = __fdividef(1.f, 1.f + __expf(-fr[i]));
      pa[i] = os[i] * rn;
      pb[i] = yn[i] * rn;
      pig[i] = ig[i];
      pzt[i] = zt[i];
      pfg[i] = fg;
      pff[i] = fg * (1.f - fsig);
      pcp[i] = cp[i];
      pnp[i] = np[i];
      pz2[i] = ig[i] * (1.f - zt[i] * zt[i]);
      po2[i] = (1.f - os[i]) * yn[i];
      dup[i] = du[i];
    }
  };
  cp_async_wait<SL_RING - 3>();   // the records of the last two steps have landed (this thread's)
  precompute(S - 1);

  bool ok = true;
  for (int it = 0; it < S; ++it) {
    const int t = S - 1 - it;
    const int buf = it & 1;
    issue(t - (SL_RING - 1));
    if (tid == 0) mbar_expect_tx(s_bar + 8u * buf, RB_BYTES);

    // ---- the part of the pointwise backward that depends on the incoming gradient
    float dgi[4], dgf[4], dgz[4], dgo[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float dy = dup[i] + dhrec[i];
      const float dc = fmaf(dy, pa[i], dc_[i]);
      const float dn = fmaf(-dy, pb[i], dn_[i]);
      dgi[i] = pig[i] * fmaf(pzt[i], dc, dn);
      dgf[i] = pff[i] * fmaf(dc, pcp[i], dn * pnp[i]);
      dgz[i] = dc * pz2[i];
      dgo[i] = po2[i] * dy;
      dc_[i] = pfg[i] * dc;
      dn_[i] = pfg[i] * dn;
    }
    // ---- dg_t of this CTA (16 rows x [4 gates x 32 units]) as the A operand of the recurrent product
    {
      uint32_t* ra = reinterpret_cast<uint32_t*>(s_dg + row_a * SLB_DG_STRIDE + unit_l);
      uint32_t* rb = reinterpret_cast<uint32_t*>(s_dg + row_b * SLB_DG_STRIDE + unit_l);
      ra[0 * (SL_UNITS / 2)] = pack_bf16x2(dgi[0], dgi[1]);
      ra[1 * (SL_UNITS / 2)] = pack_bf16x2(dgf[0], dgf[1]);
      ra[2 * (SL_UNITS / 2)] = pack_bf16x2(dgz[0], dgz[1]);
      ra[3 * (SL_UNITS / 2)] = pack_bf16x2(dgo[0], dgo[1]);
      rb[0 * (SL_UNITS / 2)] = pack_bf16x2(dgi[2], dgi[3]);
      rb[1 * (SL_UNITS / 2)] = pack_bf16x2(dgf[2], dgf[3]);
      rb[2 * (SL_UNITS / 2)] = pack_bf16x2(dgz[2], dgz[3]);
      rb[3 * (SL_UNITS / 2)] = pack_bf16x2(dgo[2], dgo[3]);
    }
    __syncthreads();
    // ---- partial dh_{t-1} for all DH columns: 16 x DH = (16 x 128) (128 x DH)
    float acc[NTW][4];
#pragma unroll
    for (int j = 0; j < NTW; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      uint32_t a0, a1, a2, a3;
      ldmatrix_x4(s_dg_u32 + ldm_off + ks * 32, a0, a1, a2, a3);
#pragma unroll
      for (int j = 0; j < NTW; ++j) mma_bf16_16816(acc[j], a0, a1, a2, a3, bfrag[j][ks][0], bfrag[j][ks][1]);
    }
    // ---- stage the partials per destination CTA (columns 32 d .. 32 d + 31 belong to CTA d) ...
#pragma unroll
    for (int j = 0; j < NTW; ++j) {
      const int tile = warp * NTW + j;                 // columns 8 tile .. 8 tile + 7 of the head
      float* blk = s_st + ((size_t)(buf * NCTA + (tile >> 2)) * SL_ROWS) * SLB_PROW + (tile & 3) * 8 + (lane & 3) * 2;
      *reinterpret_cast<float2*>(blk + row_a * SLB_PROW) = make_float2(acc[j][0], acc[j][1]);
      *reinterpret_cast<float2*>(blk + row_b * SLB_PROW) = make_float2(acc[j][2], acc[j][3]);
    }
    fence_proxy_async_smem();
    // ... and send every block with one bulk copy into slot [buf][this CTA] of its owner.  A warp produces whole
    // blocks when it covers at least 32 columns; otherwise the CTA synchronises first.
    if constexpr (NTW >= 4) {
      __syncwarp();
      if (lane < NTW / 4) {
        const uint32_t dst = (uint32_t)(warp * (NTW / 4) + lane);
        bulk_copy_to_cta(map_to_cta(s_rb_u32 + ((uint32_t)buf * NCTA + rank) * SLB_PBLOCK, dst),
                         s_st_u32 + ((uint32_t)buf * NCTA + dst) * SLB_PBLOCK, SLB_PBLOCK, map_to_cta(s_bar + 8u * buf, dst));
      }
    } else {
      __syncthreads();
      if (tid < NCTA)
        bulk_copy_to_cta(map_to_cta(s_rb_u32 + ((uint32_t)buf * NCTA + rank) * SLB_PBLOCK, (uint32_t)tid),
                         s_st_u32 + ((uint32_t)buf * NCTA + tid) * SLB_PBLOCK, SLB_PBLOCK, map_to_cta(s_bar + 8u * buf, (uint32_t)tid));
    }
    // ---- dWx_t = dg_t, (B, S, 4, NH, DH), from the tile: 16-byte pieces, two per thread (off the step-to-step chain)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int pidx = tid + j * SL_THREADS;
      const int r = pidx >> 4, g = (pidx >> 2) & 3, part = pidx & 3;
      const int gb = bgroup * SL_ROWS + r;
      if (gb < B)
        *reinterpret_cast<uint4*>(dwx + (((size_t)gb * S + t) * 4 + g) * H + (size_t)head * DH + rank * SL_UNITS + part * 8) =
            *reinterpret_cast<const uint4*>(s_dg + r * SLB_DG_STRIDE + g * SL_UNITS + part * 8);
    }
    // ---- while the partials are in flight: the gradient-independent part of the next step (t - 1)
    cp_async_wait<SL_RING - 3>();   // the records of steps t-1 and t-2 (this thread's) have landed
    if (t >= 1) precompute(t - 1);
    // ---- the DH/32 partials of this CTA's own columns have landed: add them in rank order
    if (!sl_wait(s_bar + 8u * buf, (uint32_t)(it >> 1) & 1u)) ok = false;
    {
      const float* rb0 = s_rb + (size_t)buf * NCTA * SL_ROWS * SLB_PROW + unit_l;
      float2 sa = make_float2(0.f, 0.f), sb = make_float2(0.f, 0.f);
#pragma unroll
      for (int s = 0; s < NCTA; ++s) {
        const float2 va = *reinterpret_cast<const float2*>(rb0 + (s * SL_ROWS + row_a) * SLB_PROW);
        const float2 vb = *reinterpret_cast<const float2*>(rb0 + (s * SL_ROWS + row_b) * SLB_PROW);
        sa.x += va.x; sa.y += va.y; sb.x += vb.x; sb.y += vb.y;
      }
      dhrec[0] = sa.x; dhrec[1] = sa.y; dhrec[2] = sb.x; dhrec[3] = sb.y;
    }
    // everybody is done with the dg tile and with this receive buffer; the same barrier tells every thread whether
    // any wait expired
    if (__syncthreads_or(ok ? 0 : 1)) { ok = false; break; }
  }
  cp_async_wait<0>();
  if (!ok && p.status) atomicExch(p.status, 1);
  cluster_barrier();  // nobody leaves while a peer may still push into its buffers

  // gradient of the initial state (4, B, H): dh, dc, dn, 0
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gb = (i < 2) ? gb_a : gb_b;
    const bool okr = (i < 2) ? ok_a : ok_b;
    if (!okr) continue;
    const size_t off = (size_t)gb * H + (size_t)head * DH + unit_h + (i & 1);
    p.dstate0[0 * (size_t)B * H + off] = dhrec[i];
    p.dstate0[1 * (size_t)B * H + off] = dc_[i];
    p.dstate0[2 * (size_t)B * H + off] = dn_[i];
    p.dstate0[3 * (size_t)B * H + off] = 0.f;
  }
}

template <int DH>
static int launch_slstm_bwd(const xl_slstm_bwd_params* p, cudaStream_t st) {
  constexpr int NCTA = DH / SL_UNITS;
  const size_t smem = (size_t)SL_ROWS * SLB_DG_STRIDE * 2 + 4 * (size_t)NCTA * SLB_PBLOCK +
                      (size_t)SL_RING * SLB_REC_STEP + (size_t)SL_RING * SL_THREADS * 8 + 16;
  XL_CUDA_TRY(cudaFuncSetAttribute(slstm_backward_kernel<DH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(NCTA, p->NH, (p->B + SL_ROWS - 1) / SL_ROWS);
  cfg.blockDim = dim3(SL_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = NCTA;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  XL_CUDA_TRY(cudaLaunchKernelEx(&cfg, slstm_backward_kernel<DH>, *p));
  return check_launch("xl_slstm_backward");
}

}  // namespace xl

extern "C" int xl_slstm_backward(const xl_slstm_bwd_params* p, void* cuda_stream) {
  using namespace xl;
  if (!p || !p->cache || !p->R || !p->dh || !p->dwx || !p->dstate0) return XL_ERR_NULL_POINTER;
  if (p->B <= 0 || p->S <= 0 || p->NH <= 0) return XL_ERR_BAD_SHAPE;
  if (p->dtype != XL_BF16) return XL_ERR_BAD_DTYPE;
  if (p->NH > 65535 || (p->B + SL_ROWS - 1) / SL_ROWS > 65535) return XL_ERR_TOO_LARGE;
  if (!aligned16(p->cache) || !aligned16(p->dwx) || (reinterpret_cast<uintptr_t>(p->dh) & 3u) || (reinterpret_cast<uintptr_t>(p->R) & 3u))
    return XL_ERR_BAD_ALIGNMENT;
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  switch (p->DH) {
    case 64: return launch_slstm_bwd<64>(p, st);
    case 128: return launch_slstm_bwd<128>(p, st);
    case 256: return launch_slstm_bwd<256>(p, st);
    default: return XL_ERR_UNSUPPORTED;
  }
}
