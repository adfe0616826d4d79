// sLSTM backward through time in ONE persistent kernel (the counterpart of the reference's host loop
// BackwardPass::Run + SLSTMPointwiseBackward: xlstm/blocks/slstm/src/cuda/slstm_backward.cu,
// slstm_pointwise.cu:118-196).
//
// Same decomposition as the forward kernel: one thread-block cluster of DH/32 CTAs per (head, 16-row batch group),
// CTA r owns hidden units [32r, 32r+32) with all four gates.  A CTA has EIGHT warps here (the forward has four): warps
// 2w and 2w+1 share the four (row, unit) pairs of forward thread (w, lane) -- the first takes the pairs of batch row
// lane/4, the second those of row lane/4 + 8 -- and keep their gradient carries dc, dn in fp32 registers for the
// whole sequence.  (With four warps every scheduler of the SM had one warp, whose ~1 000 instructions per step ran at
// one instruction per ~3.7 cycles; two half-as-long instruction streams per scheduler interleave.)  Per step, walking t = S-1 .. 0:
//   dy = dh_t (from above) + dh_t (recurrent);  dc += dy o / n';  dn -= dy h' / n'
//   dg_i = i' (z dc + dn);  dg_f = f' (dc c + dn n)(1 - sigmoid(f));  dg_z = dc i' (1 - z^2);  dg_o = (1 - o) h' dy
//   dc <- f' dc;  dn <- f' dn          (the stabiliser m is a constant of the step, as in the reference)
// with i', raw f, z = tanh, o = sigmoid, h', c', n', m' read from the cache the training forward wrote (one 96-byte
// record per thread and step, streamed through a cp.async ring), and
//   dh_{t-1}[b,k] = sum_{g,u} dg_t[b,g,u] R[k,g,u].
// The CTA holds exactly the slice of R the forward holds (all k, its own 32 units, four gates) as mma.sync
// B-fragments in registers, now contracted over (g,u): it forms the PARTIAL sums of dh_{t-1} for all DH columns
// from its own 128 gate gradients (M = 16 rows, N = DH, K = 128) and sends every 32-column block, as bf16, to the CTA
// that owns those units with asynchronous distributed-shared-memory stores that count their bytes on the receiver's
// mbarrier (a reduce-scatter, 1 KB per CTA pair and step).  A CTA takes in distributed shared memory in 32-byte
// sectors at ~32 B per cycle, so the stores are shaped for whole sectors: a warp regroups its products into 16-byte
// granules (eight columns of one row) and the lanes of one store cover whole rows of the destination block -- two
// 16-byte stores per thread and step (2 048 eight-byte stores per CTA cost 1 200 cycles of issue and twice the sectors;
// staged blocks sent by bulk copies needed a proxy fence of ~250 cycles on the chain).  The receiver adds the DH/32
// partials in fp32 in rank order.  Everything of a step's gate arithmetic that does not depend on the incoming gradient
// is computed one step ahead, while the partials are in flight.
// dWx_t = dg_t leaves as bf16 in the layout of Wx.  dR and dbias are sums over (b,t) of h_{t-1} (x) dg_t and of dg_t:
// plain matrix products over the dWx this kernel writes, left to the caller's GEMM library.
#include "common.cuh"
#include "slstm_common.cuh"

namespace xl {

constexpr int SLB_DG_STRIDE = 4 * SL_UNITS + 8;          // bf16 elements per row of the dg tile (+16 B: bank spread)
constexpr int SLB_THREADS = 256;                         // 8 warps
constexpr int SLB_REC_STEP = SL_THREADS * SL_REC_BYTES;  // cache bytes per CTA and step (records of the forward's 128 threads)
constexpr int SLB_PROW = SL_UNITS;                       // bf16 elements per row of a partial block: 64 B = four 16-byte granules
constexpr int SLB_PBLOCK = SL_ROWS * SLB_PROW * 2;       // bytes of one (source, destination) block of partial sums (bf16: a
                                                         // CTA takes in ~32 B of distributed shared memory per cycle, so the
                                                         // exchange time follows the bytes; the sums are formed in fp32)

__device__ __forceinline__ uint32_t ldg_nc_u32(const void* ptr) {
  uint32_t v;
  asm volatile("ld.global.nc.b32 %0, [%1];" : "=r"(v) : "l"(ptr));
  return v;
}
template <int DH>
__global__ void __launch_bounds__(SLB_THREADS, 1) slstm_backward_kernel(const xl_slstm_bwd_params p) {
  constexpr int NCTA = DH / SL_UNITS;
  constexpr int NTW = DH / 64;              // n8 tiles (8 columns of dh_{t-1}) per warp
  constexpr int KS = 4 * SL_UNITS / 16;     // k-steps over the CTA's 128 gate gradients
  constexpr uint32_t RB_BYTES = NCTA * SLB_PBLOCK;   // what one step delivers to a CTA
  extern __shared__ __align__(16) unsigned char slb_smem[];
  __nv_bfloat16* s_dg = reinterpret_cast<__nv_bfloat16*>(slb_smem);                   // [2][16][SLB_DG_STRIDE]
  __nv_bfloat16* s_rb = reinterpret_cast<__nv_bfloat16*>(slb_smem + 2 * SL_ROWS * SLB_DG_STRIDE * 2);  // received: [2][source CTA][16][SLB_PROW]
  __nv_bfloat16* s_st = s_rb + 2 * RB_BYTES / 2;                                      // per warp: [16 rows][8 NTW columns], its own products
  unsigned char* s_rec = reinterpret_cast<unsigned char*>(s_st) + SL_ROWS * DH * 2;   // [SL_RING][SLB_REC_STEP]
  const uint32_t s_bar = smem_u32(s_rec + SL_RING * SLB_REC_STEP);                    // 2 mbarriers: partials landed

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t rank = cluster_ctarank();
  const int head = blockIdx.y, bgroup = blockIdx.z;
  const int B = p.B, S = p.S, NH = p.NH, H = NH * DH;
  const int fwarp = warp >> 1, half = warp & 1;           // the forward thread whose record this thread shares, and which row of it
  const int ftid = fwarp * 32 + lane;
  const int row = (lane >> 2) + 8 * half;                 // batch row within the group
  const int unit_l = fwarp * 8 + (lane & 3) * 2;          // first of two adjacent units within the CTA
  const int unit_h = (int)rank * SL_UNITS + unit_l;       // ... within the head
  const int gb = bgroup * SL_ROWS + row;                  // global batch row
  const bool ok_r = gb < B;
  const size_t st_off = (size_t)(ok_r ? gb : 0) * H + (size_t)head * DH + unit_h;   // this thread's pair in a (4,B,H) state

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

  // ---- gradient carries and the recurrent part of dh for the thread's two pairs, from the gradient of the final state
  float dc_[2], dn_[2], dhrec[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const bool have = p.dstate_out != nullptr && ok_r;
    dhrec[i] = have ? p.dstate_out[0 * (size_t)B * H + st_off + i] : 0.f;
    dc_[i] = have ? p.dstate_out[1 * (size_t)B * H + st_off + i] : 0.f;
    dn_[i] = have ? p.dstate_out[2 * (size_t)B * H + st_off + i] : 0.f;
  }

  if (tid == 0) {
    mbar_init(s_bar, 1);      // one arrival per phase: the local expect_tx
    mbar_init(s_bar + 8, 1);
    fence_barrier_init();
  }

  // ---- cache ring: the records of one step and CTA are 12 KB of contiguous global memory, fetched SL_RING - 1 steps
  // ahead; every thread copies three 16-byte granules of the block (anybody's: the step's CTA barrier publishes them)
  const unsigned char* cache = reinterpret_cast<const unsigned char*>(p.cache) +
                               (((size_t)bgroup * NH + head) * NCTA + rank) * (size_t)S * SLB_REC_STEP;
  const uint32_t s_rec_u32 = smem_u32(s_rec);
  auto issue = [&](int t) {
    if (t >= 0) {
      const unsigned char* src = cache + (size_t)t * SLB_REC_STEP + tid * 16;
      const uint32_t dst = s_rec_u32 + (uint32_t)(t % SL_RING) * SLB_REC_STEP + tid * 16;
#pragma unroll
      for (int j = 0; j < SLB_REC_STEP / (16 * SLB_THREADS); ++j) cp_async16(dst + j * (16 * SLB_THREADS), src + j * (16 * SLB_THREADS));
    }
    cp_async_commit();
  };
  // the gradient from above, (B, NH, S, DH): one word (two units) per thread and step, loaded one step ahead
  const __nv_bfloat16* dh = reinterpret_cast<const __nv_bfloat16*>(p.dh);
  const size_t dh_off = ((size_t)(ok_r ? gb : B - 1) * NH + head) * (size_t)S * DH + unit_h;
#pragma unroll
  for (int j = 0; j < SL_RING - 1; ++j) issue(S - 1 - j);
  cp_async_wait<SL_RING - 4>();   // this thread's granules of the last three steps' records; everybody's behind the barrier
  cluster_barrier();  // every CTA's barriers exist before anything crosses over; also a CTA-wide barrier

  const uint32_t s_dg_u32 = smem_u32(s_dg), s_rb_u32 = smem_u32(s_rb);
  const uint32_t ldm_off = ((lane & 15) * SLB_DG_STRIDE + (lane >> 4) * 8) * 2;
  __nv_bfloat16* dwx = reinterpret_cast<__nv_bfloat16*>(p.dwx);

  // Per pair, everything of a step that does not depend on the incoming gradient (formed one step ahead):
  //   dc = dc_carry + dy pa;  dn = dn_carry - dy pb;  dg_i = pig (pzt dc + dn);  dg_f = pff (dc pcp + dn pnp);
  //   dg_z = dc pz2;  dg_o = po2 dy;  carries <- pfg (dc, dn);  dy = gradient from above + recurrent part
  float pa[2], pb[2], pig[2], pzt[2], pfg[2], pff[2], pcp[2], pnp[2], pz2[2], po2[2];
  auto precompute = [&](int t) {
    // the forward thread's record: gates of rows a | b (16 B each), h' of rows a | b (4 B each), 8 B pad, then c', n', m'
    // as (row a: u0, u1, row b: u0, u1)
    const unsigned char* rt = s_rec + (t % SL_RING) * SLB_REC_STEP + ftid * SL_REC_BYTES;
    const uint4 gw = *reinterpret_cast<const uint4*>(rt + 16 * half);
    const uint32_t hw = *reinterpret_cast<const uint32_t*>(rt + 32 + 4 * half);
    const float2 n_new = *reinterpret_cast<const float2*>(rt + 64 + 8 * half);
    const float2 m_new = *reinterpret_cast<const float2*>(rt + 80 + 8 * half);
    float2 c_prev, n_prev, m_prev;
    if (t > 0) {
      const unsigned char* rp = s_rec + ((t - 1) % SL_RING) * SLB_REC_STEP + ftid * SL_REC_BYTES;
      c_prev = *reinterpret_cast<const float2*>(rp + 48 + 8 * half);
      n_prev = *reinterpret_cast<const float2*>(rp + 64 + 8 * half);
      m_prev = *reinterpret_cast<const float2*>(rp + 80 + 8 * half);
    } else {
      const bool have = p.state0 != nullptr && ok_r;
      c_prev = make_float2(have ? p.state0[1 * (size_t)B * H + st_off] : 0.f, have ? p.state0[1 * (size_t)B * H + st_off + 1] : 0.f);
      n_prev = make_float2(have ? p.state0[2 * (size_t)B * H + st_off] : 0.f, have ? p.state0[2 * (size_t)B * H + st_off + 1] : 0.f);
      m_prev = make_float2(have ? p.state0[3 * (size_t)B * H + st_off] : 0.f, have ? p.state0[3 * (size_t)B * H + st_off + 1] : 0.f);
    }
    const float2 iw = unpack_bf16x2(gw.x), fw = unpack_bf16x2(gw.y), zw = unpack_bf16x2(gw.z), ow = unpack_bf16x2(gw.w);
    const float2 yw = unpack_bf16x2(hw);
    const float ig[2] = {iw.x, iw.y}, fr[2] = {fw.x, fw.y}, zt[2] = {zw.x, zw.y}, os[2] = {ow.x, ow.y}, yn[2] = {yw.x, yw.y};
    const float nn[2] = {n_new.x, n_new.y}, mn[2] = {m_new.x, m_new.y};
    const float cp[2] = {c_prev.x, c_prev.y}, np[2] = {n_prev.x, n_prev.y}, mp[2] = {m_prev.x, m_prev.y};
#pragma unroll
    for (int i = 0; i < 2; ++i) {
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
    }
  };
  bool ok = true;
  precompute(S - 1);
  uint32_t dh_w = ldg_nc_u32(dh + dh_off + (size_t)(S - 1) * DH);

  for (int it = 0; it < S; ++it) {
    const int t = S - 1 - it;
    const int buf = it & 1;

    // ---- the part of the pointwise backward that depends on the incoming gradient
    float dgi[2], dgf[2], dgz[2], dgo[2];
    const float2 dw = unpack_bf16x2(dh_w);
    const float dup[2] = {ok_r ? dw.x : 0.f, ok_r ? dw.y : 0.f};
#pragma unroll
    for (int i = 0; i < 2; ++i) {
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
      uint32_t* rr = reinterpret_cast<uint32_t*>(s_dg + (buf * SL_ROWS + row) * SLB_DG_STRIDE + unit_l);
      rr[0 * (SL_UNITS / 2)] = pack_bf16x2(dgi[0], dgi[1]);
      rr[1 * (SL_UNITS / 2)] = pack_bf16x2(dgf[0], dgf[1]);
      rr[2 * (SL_UNITS / 2)] = pack_bf16x2(dgz[0], dgz[1]);
      rr[3 * (SL_UNITS / 2)] = pack_bf16x2(dgo[0], dgo[1]);
    }
    // The one CTA-wide barrier of a step.  It also orders the buffers that alternate between steps (dg tile, received
    // partials): whoever passes it has finished the previous step, and nothing of step it+2 can reach this
    // CTA before its own stores of step it+1, which are issued behind this barrier, have arrived at the peers.  The
    // same barrier tells every thread whether any wait expired.
    if (__syncthreads_or(ok ? 0 : 1)) { ok = false; break; }
    // ---- partial dh_{t-1} for all DH columns: 16 x DH = (16 x 128) (128 x DH); this warp's share is NTW 8-column tiles
    float acc[NTW][4];
#pragma unroll
    for (int j = 0; j < NTW; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    uint32_t af[KS][4];
#pragma unroll
    for (int ks = 0; ks < KS; ++ks)
      ldmatrix_x4(s_dg_u32 + buf * (SL_ROWS * SLB_DG_STRIDE * 2) + ldm_off + ks * 32, af[ks][0], af[ks][1], af[ks][2], af[ks][3]);
    // Behind the fragment loads and in front of the products, which keep the warp busy without touching the load/store
    // unit: everything of this step that is off the step-to-step chain but goes through that unit -- the ring fetch, the
    // gradient from above for the next step, dWx_t.  (Issued after the pushes below, these instructions sat in the
    // unit's in-order queue in front of the next step's record loads and held them up for ~800 cycles.)
    if (tid == 0) mbar_expect_tx(s_bar + 8u * buf, RB_BYTES);   // what this step delivers to this CTA: the barrier's phase
                                                                // cannot complete before this arrival, whatever has landed
    issue(t - (SL_RING - 1));
    if (t >= 1) dh_w = ldg_nc_u32(dh + dh_off + (size_t)(t - 1) * DH);
    {  // dWx_t = dg_t, (B, S, 4, NH, DH), from the tile: one 16-byte piece per thread
      const int r = tid >> 4, g = (tid >> 2) & 3, part = tid & 3;
      const int gbr = bgroup * SL_ROWS + r;
      if (gbr < B)
        *reinterpret_cast<uint4*>(dwx + (((size_t)gbr * S + t) * 4 + g) * H + (size_t)head * DH + rank * SL_UNITS + part * 8) =
            *reinterpret_cast<const uint4*>(s_dg + (buf * SL_ROWS + r) * SLB_DG_STRIDE + g * SL_UNITS + part * 8);
    }
#pragma unroll
    for (int ks = 0; ks < KS; ++ks)
#pragma unroll
      for (int j = 0; j < NTW; ++j) mma_bf16_16816(acc[j], af[ks][0], af[ks][1], af[ks][2], af[ks][3], bfrag[j][ks][0], bfrag[j][ks][1]);
    // ---- every 32-column block goes to the CTA that owns those units, slot [buf][this CTA] there.  The warp turns its
    // products (a thread holds two columns of two rows per tile) into 16-byte granules (eight columns of one row) through
    // a buffer of its own, and lane g of store k sends granule 32 k + g = (row, tile): the lanes of a store cover whole rows
    // of the destination block, i.e. full 32-byte sectors.  Which granule of its row a tile takes is XOR-ed with bits 1-2
    // of the row, so that the receiver's loads (eight rows per warp) fall on distinct banks.
    {
      __nv_bfloat16* wb = s_st + warp * (SL_ROWS * NTW * 8);
#pragma unroll
      for (int j = 0; j < NTW; ++j) {
        *reinterpret_cast<uint32_t*>(wb + ((lane >> 2) * NTW + j) * 8 + (lane & 3) * 2) = pack_bf16x2(acc[j][0], acc[j][1]);
        *reinterpret_cast<uint32_t*>(wb + (((lane >> 2) + 8) * NTW + j) * 8 + (lane & 3) * 2) = pack_bf16x2(acc[j][2], acc[j][3]);
      }
      __syncwarp();
      constexpr int NST = (SL_ROWS * NTW + 31) / 32;   // stores per lane
#pragma unroll
      for (int k = 0; k < NST; ++k) {
        const int gidx = 32 * k + lane;
        if (SL_ROWS * NTW >= 32 || gidx < SL_ROWS * NTW) {
          const int prow = gidx / NTW, tile = warp * NTW + gidx % NTW;       // tile: columns 8 tile .. 8 tile + 7 of the head
          const uint4 gr = *reinterpret_cast<const uint4*>(wb + gidx * 8);
          const uint32_t dst = (uint32_t)(tile >> 2);
          const uint32_t off = (((uint32_t)buf * NCTA + rank) * SL_ROWS + prow) * (SLB_PROW * 2) + (uint32_t)(((tile & 3) ^ ((prow >> 1) & 3)) * 16);
          const uint32_t v[4] = {gr.x, gr.y, gr.z, gr.w};
          st_async_v4(map_to_cta(s_rb_u32 + off, dst), v, map_to_cta(s_bar + 8u * buf, dst));
        }
      }
      __syncwarp();   // the buffer is rewritten in the next step
    }
    // ---- while the partials are in flight: the gradient-independent part of the next step (t - 1)
    if (t >= 1) precompute(t - 1);   // records t-1, t-2: waited for a step ago, published by this step's barrier
    cp_async_wait<SL_RING - 4>();    // this thread's granules of records t-2 and t-3, which the next step reads
    // ---- the DH/32 partials of this CTA's own columns have landed: add them in rank order
    if (!sl_wait(s_bar + 8u * buf, (uint32_t)(it >> 1) & 1u)) ok = false;
    {
      const __nv_bfloat16* rb0 = s_rb + ((size_t)buf * NCTA * SL_ROWS + row) * SLB_PROW + ((fwarp ^ ((row >> 1) & 3)) * 8) + (lane & 3) * 2;
      float2 sa = make_float2(0.f, 0.f);
#pragma unroll
      for (int s = 0; s < NCTA; ++s) {
        const float2 va = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(rb0 + s * SL_ROWS * SLB_PROW));
        sa.x += va.x; sa.y += va.y;
      }
      dhrec[0] = sa.x; dhrec[1] = sa.y;
    }
  }
  if (!ok && p.status) atomicExch(p.status, 1);
  cluster_barrier();  // nobody leaves while a peer may still push into its buffers

  // gradient of the initial state (4, B, H): dh, dc, dn, 0
  if (ok_r) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      p.dstate0[0 * (size_t)B * H + st_off + i] = dhrec[i];
      p.dstate0[1 * (size_t)B * H + st_off + i] = dc_[i];
      p.dstate0[2 * (size_t)B * H + st_off + i] = dn_[i];
      p.dstate0[3 * (size_t)B * H + st_off + i] = 0.f;
    }
  }
}

template <int DH>
static int launch_slstm_bwd(const xl_slstm_bwd_params* p, cudaStream_t st) {
  constexpr int NCTA = DH / SL_UNITS;
  const size_t smem = 2 * (size_t)SL_ROWS * SLB_DG_STRIDE * 2 + 2 * (size_t)NCTA * SLB_PBLOCK + (size_t)SL_ROWS * DH * 2 +
                      (size_t)SL_RING * SLB_REC_STEP + 16 + 8 * SL_RING;
  XL_CUDA_TRY(cudaFuncSetAttribute(slstm_backward_kernel<DH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(NCTA, p->NH, (p->B + SL_ROWS - 1) / SL_ROWS);
  cfg.blockDim = dim3(SLB_THREADS);
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
