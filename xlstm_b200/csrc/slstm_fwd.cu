// sLSTM forward over a whole sequence in ONE persistent kernel.
//
// Per time step (reference: slstm_pointwise.cu:60-115 / vanilla/slstm.py:19-37):
//   raw_g = Wx_g + (h_{t-1} R)_g + b_g ,  g in {i,f,z,o}
//   m' = (n == 0) ? i : max(i, m + logsig(f));  i' = min(1, e^{i-m'});  f' = min(1, e^{m + logsig(f) - m'})
//   c' = f' c + i' tanh(z);  n' = f' n + i';  h' = sigmoid(o) c' / n'
//
// Mapping.  One thread-block CLUSTER of DH/32 CTAs serves one (head, 16-row batch group); heads and batch
// groups never exchange data.  CTA r of the cluster owns hidden units [32r, 32r+32) and all four of their
// gates: its slice of the recurrent matrix (DH x 128 bf16) is read once and stays in REGISTERS as
// mma.sync B-fragments (a warp = 8 units x 4 gates = four n8 tiles x DH/16 k-steps).  The batch rows are
// the M=16 side of m16n8k16.  Each thread ends a step holding all four gate pre-activations of its four
// (row, unit) pairs in its accumulators, so the pointwise update runs in registers with c, n, m kept in
// fp32 registers for the whole sequence.  The new h (bf16) is pushed into the double-buffered h tile of
// EVERY CTA of the cluster with asynchronous distributed-shared-memory stores that count their bytes on the
// destination's mbarrier: a CTA starts step t+1 the moment all of h_t has landed in ITS tile -- no cluster-wide
// barrier and no release/acquire fence on the per-step chain (that barrier was 2/3 of the step time).  The data
// dependency itself orders buffer reuse: whoever pushes h_{t+1} into a tile has consumed h_t, which every CTA
// pushed only after its last read of h_{t-1}, the previous content of that buffer.
// A CTA takes in distributed shared memory in 32-byte sectors (~32 B per cycle), so the tile is laid out in 16-byte
// granules -- eight units of one batch row, what one ldmatrix row reads -- with rows r and r+8 of a unit group in one
// sector, and the pushes are whole granules gathered from the quad that computed them: the lanes of one store fill
// full sectors (8 KB of h per step = 256 sectors; 4-byte stores per row pair arrived as 512 half-filled ones).
// Gate arithmetic: one of i', f' is exp(0), the other exp(-|m + logsig(f) - i|); tanh and the sigmoid run on the
// hardware tanh (six special-function instructions per (row, unit) instead of nine).
// Wx is streamed through an 8-step cp.async ring so that HBM latency is off the dependency chain.
// A document boundary (cu_seqlens) zeroes h, c, n, m of that batch row inside the kernel.
//
// Training variant (TRAIN): every thread also writes one 96-byte record per step -- its activated gates
// (i', raw f, tanh z, sigmoid o as bf16 pairs), its h' and its c', n', m' in fp32 -- into a cache that the backward
// kernel (slstm_bwd.cu) reads back by the same (warp, lane) index (the counterpart of the reference's `states` and
// gate caches, slstm.cc:88-101).  The 12 KB of a step are staged in shared memory and leave as one bulk copy.
#include "common.cuh"
#include "slstm_common.cuh"

namespace xl {

constexpr int SL_REC_SLOTS = 3;                          // staging slots of the training cache (one step's records each)
constexpr int SL_REC_STEP = SL_THREADS * SL_REC_BYTES;   // bytes of one step's records of a CTA

// bulk copy of this CTA's shared memory to global memory (bulk-group completion)
__device__ __forceinline__ void bulk_store(void* dst, uint32_t src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait() { asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory"); }

// Advance `idx` past every boundary at or before time index `t_now` of batch row `gb`; return the time index
// of the next boundary inside the row, or INT_MAX.  Repeated offsets (empty documents) are skipped.
__device__ __forceinline__ int next_boundary(const xl_slstm_params& p, int gb, int t_now, int& idx) {
  const long long row0 = (long long)gb * p.S;
  while (idx <= p.num_docs && (long long)p.cu_seqlens[idx] <= row0 + t_now) ++idx;
  if (idx > p.num_docs) return 0x7fffffff;
  const long long pos = p.cu_seqlens[idx];
  return pos < row0 + p.S ? (int)(pos - row0) : 0x7fffffff;
}

template <int DH, bool TRAIN>
__global__ void __launch_bounds__(SL_THREADS, 1) slstm_forward_kernel(const xl_slstm_params p) {
  constexpr int KSTEPS = DH / 16;
  // h tile: 16-byte granules (eight consecutive units of one batch row, what one ldmatrix row reads), laid out so that
  // the granules of rows r and r + 8 of one unit group share a 32-byte sector: a warp's push then fills whole sectors of
  // the destination CTA, which takes in distributed shared memory sector by sector (~32 B per cycle), where separate
  // 4-byte stores per row pair arrived as twice as many half-filled ones.  Which half of its sector a granule takes
  // flips with bit 2 of the row, which keeps the eight rows of an ldmatrix matrix on distinct banks.
  constexpr int H_TILE = SL_ROWS * DH;   // bf16 elements of one tile (dense)
  auto granule_off = [](int row, int kgroup) -> uint32_t {   // byte offset of granule (batch row, unit / 8) in a tile
    return (uint32_t)(kgroup * 256 + (row & 7) * 32 + ((((row >> 3) ^ (row >> 2)) & 1) * 16));
  };
  extern __shared__ __align__(16) unsigned char sl_smem[];
  __nv_bfloat16* s_h = reinterpret_cast<__nv_bfloat16*>(sl_smem);                    // 2 x H_TILE
  unsigned char* s_wx = sl_smem + 2 * H_TILE * sizeof(__nv_bfloat16);                // SL_RING x SL_WX_STEP_BYTES
  const uint32_t s_bar = smem_u32(s_wx + SL_RING * SL_WX_STEP_BYTES);                // 2 mbarriers: h tile 0 / 1 complete
  constexpr uint32_t H_TILE_BYTES = SL_ROWS * DH * 2;                                // what one step delivers to a CTA
  unsigned char* s_recst = s_wx + SL_RING * SL_WX_STEP_BYTES + 16;                   // TRAIN: SL_REC_SLOTS x SL_REC_STEP

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t rank = cluster_ctarank();       // which 32-unit slice of the head
  constexpr int NCTA = DH / SL_UNITS;
  const int head = blockIdx.y, bgroup = blockIdx.z;
  const int B = p.B, S = p.S, NH = p.NH, H = NH * DH;
  const int row_a = lane >> 2, row_b = row_a + 8;             // the two batch rows (within the group) of this thread
  const int unit_l = warp * 8 + (lane & 3) * 2;               // first of two adjacent units within the CTA
  const int unit_h = (int)rank * SL_UNITS + unit_l;           // ... within the head
  const int gb_a = bgroup * SL_ROWS + row_a, gb_b = bgroup * SL_ROWS + row_b;  // global batch rows
  const bool ok_a = gb_a < B, ok_b = gb_b < B;

  // ---- recurrent matrix slice -> registers (B fragments).  R is (NH, DH_in, 4, DH_out).
  uint32_t rfrag[KSTEPS][4][2];
  {
    const __nv_bfloat16* R = reinterpret_cast<const __nv_bfloat16*>(p.R) + (size_t)head * DH * 4 * DH;
    const int n_unit = (int)rank * SL_UNITS + warp * 8 + (lane >> 2);  // column n = lane/4 of every tile
    const int k0 = (lane & 3) * 2;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks)
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const __nv_bfloat16* base = R + ((size_t)(ks * 16 + k0) * 4 + g) * DH + n_unit;
        const uint16_t e0 = *reinterpret_cast<const uint16_t*>(base);
        const uint16_t e1 = *reinterpret_cast<const uint16_t*>(base + 4 * DH);
        const uint16_t e8 = *reinterpret_cast<const uint16_t*>(base + 8 * 4 * DH);
        const uint16_t e9 = *reinterpret_cast<const uint16_t*>(base + 9 * 4 * DH);
        rfrag[ks][g][0] = (uint32_t)e0 | ((uint32_t)e1 << 16);
        rfrag[ks][g][1] = (uint32_t)e8 | ((uint32_t)e9 << 16);
      }
  }
  // ---- bias for this thread's two units, four gates
  float bias[4][2];
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    bias[g][0] = p.bias[((size_t)head * 4 + g) * DH + unit_h];
    bias[g][1] = p.bias[((size_t)head * 4 + g) * DH + unit_h + 1];
  }

  // ---- state registers: [pair] with pair = (row_a,u0), (row_a,u1), (row_b,u0), (row_b,u1)
  float c_[4], n_[4], m_[4], hlast[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gb = (i < 2) ? gb_a : gb_b;
    const bool ok = (i < 2) ? ok_a : ok_b;
    const size_t off = (size_t)gb * H + (size_t)head * DH + unit_h + (i & 1);
    const bool have = p.state0 != nullptr && ok;
    hlast[i] = have ? p.state0[0 * (size_t)B * H + off] : 0.f;
    c_[i] = have ? p.state0[1 * (size_t)B * H + off] : 0.f;
    n_[i] = have ? p.state0[2 * (size_t)B * H + off] : 0.f;
    m_[i] = have ? p.state0[3 * (size_t)B * H + off] : 0.f;
  }

  // ---- next document boundary (as a time index within the row) for the two batch rows
  int nxt_idx[2] = {0, 0};
  int nxt_t[2] = {0x7fffffff, 0x7fffffff};
  if (p.cu_seqlens) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int gb = r == 0 ? gb_a : gb_b;
      const bool ok = r == 0 ? ok_a : ok_b;
      if (!ok) continue;
      // binary search for the first boundary beyond the start of row gb, then the shared helper
      const long long row0 = (long long)gb * S;
      int lo = 0, hi = p.num_docs + 1;
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if ((long long)p.cu_seqlens[mid] > row0) hi = mid; else lo = mid + 1;
      }
      nxt_idx[r] = lo;
      nxt_t[r] = next_boundary(p, gb, 0, nxt_idx[r]);
    }
  }

  // ---- h tile (both buffers) of this CTA: buffer 0 holds h_{-1}; every CTA fills its own copy completely
  for (int i = tid; i < 2 * H_TILE; i += SL_THREADS) s_h[i] = __float2bfloat16_rn(0.f);
  if (tid == 0) {
    mbar_init(s_bar, 1);      // one arrival per phase: the local expect_tx
    mbar_init(s_bar + 8, 1);
    fence_barrier_init();
  }
  __syncthreads();
  if (p.state0) {
    for (int i = tid; i < SL_ROWS * DH; i += SL_THREADS) {
      const int r = i / DH, d = i % DH;
      const int gb = bgroup * SL_ROWS + r;
      if (gb < B) s_h[granule_off(r, d >> 3) / 2 + (d & 7)] = __float2bfloat16_rn(p.state0[(size_t)gb * H + (size_t)head * DH + d]);
    }
  }

  // ---- Wx ring: each thread copies two 16-byte granules per step
  const __nv_bfloat16* wx = reinterpret_cast<const __nv_bfloat16*>(p.wx);
  const uint32_t s_wx_u32 = smem_u32(s_wx);
  auto issue_wx = [&](int t) {
    if (t < S) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int gidx = tid + j * SL_THREADS;            // 0..255
        const int r = gidx >> 4, g = (gidx >> 2) & 3, part = gidx & 3;
        int gb = bgroup * SL_ROWS + r;
        gb = gb < B ? gb : B - 1;                          // padded rows re-read a valid row (result unused)
        const __nv_bfloat16* src = wx + (((size_t)gb * S + t) * 4 + g) * H + (size_t)head * DH + rank * SL_UNITS + part * 8;
        const uint32_t dst = s_wx_u32 + (t % SL_RING) * SL_WX_STEP_BYTES + r * SL_WX_ROW_BYTES + g * (SL_UNITS * 2) + part * 16;
        cp_async16(dst, src);
      }
    }
    cp_async_commit();
  };
#pragma unroll
  for (int t = 0; t < SL_RING - 1; ++t) issue_wx(t);
  cp_async_wait<SL_RING - 2>();   // step 0 has landed (this thread's part)
  cluster_barrier();              // all CTAs of the cluster initialised; also a CTA-wide barrier

  // remote addresses of this thread's four h slots in every CTA of the cluster
  const uint32_t s_h_u32 = smem_u32(s_h);
  // Pushes: lanes 0..15 of a warp send the granule of batch row `lane` (gathered from the quad that computed it) to one
  // CTA, lanes 16..31 the same granules to the next CTA: four 16-byte stores per lane reach all eight CTAs.
  const int prow = lane & 15;
  const uint32_t pslot = granule_off(prow, unit_h >> 3 /* same for the whole warp */);
  const int psrc = 4 * (prow & 7);   // first lane of the quad that holds row prow (in pa if prow < 8, else in pb)
  // ldmatrix source row/column for this lane
  const uint32_t ldm_off = granule_off(lane & 15, lane >> 4);   // + 512 B per k-step (two unit groups)

  __nv_bfloat16* hout = reinterpret_cast<__nv_bfloat16*>(p.h_out);
  // training cache: [cluster][CTA][step][thread] records of SL_REC_BYTES.  The records of a step are staged in shared
  // memory and leave as ONE 12 KB bulk copy (six 16-byte global stores per thread and step cost 350 cycles of a step)
  unsigned char* rec = nullptr;
  if constexpr (TRAIN)
    rec = reinterpret_cast<unsigned char*>(p.train_cache) + (((size_t)bgroup * NH + head) * NCTA + rank) * (size_t)S * SL_REC_STEP;

  bool ok = true;
  for (int t = 0; t < S; ++t) {
    issue_wx(t + SL_RING - 1);
    const int cur = t & 1, nxt = cur ^ 1;
    // this step's h_t will land in tile `nxt` of this CTA: announce its size on that tile's barrier
    if (tid == 0) mbar_expect_tx(s_bar + 8u * nxt, H_TILE_BYTES);
    // h_{t-1} complete in tile `cur` (tile 0 holds the initial state at t = 0: nothing to wait for; its barrier's
    // first phase therefore belongs to t = 2)
    // (an expired wait does not leave the loop here: the decision to stop is taken by the whole CTA at the end of
    // the step, so that no thread is left behind in the barrier there)
    if (t >= 1 && !sl_wait(s_bar + 8u * cur, (uint32_t)((t >> 1) - (cur == 0 ? 1 : 0)) & 1u)) ok = false;

    // accumulators start from Wx + bias
    float acc[4][4];
    {
      const unsigned char* wrow_a = s_wx + (t % SL_RING) * SL_WX_STEP_BYTES + row_a * SL_WX_ROW_BYTES + unit_l * 2;
      const unsigned char* wrow_b = s_wx + (t % SL_RING) * SL_WX_STEP_BYTES + row_b * SL_WX_ROW_BYTES + unit_l * 2;
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const float2 wa = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(wrow_a + g * (SL_UNITS * 2)));
        const float2 wb = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(wrow_b + g * (SL_UNITS * 2)));
        acc[g][0] = wa.x + bias[g][0];
        acc[g][1] = wa.y + bias[g][1];
        acc[g][2] = wb.x + bias[g][0];
        acc[g][3] = wb.y + bias[g][1];
      }
    }
    // h_{t-1} (16 x DH) times the register-resident R slice
    const uint32_t hbase = s_h_u32 + cur * (H_TILE * 2) + ldm_off;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      uint32_t a0, a1, a2, a3;
      ldmatrix_x4(hbase + ks * 512, a0, a1, a2, a3);
#pragma unroll
      for (int g = 0; g < 4; ++g) mma_bf16_16816(acc[g], a0, a1, a2, a3, rfrag[ks][g][0], rfrag[ks][g][1]);
    }
    // pointwise update in registers
    const bool reset_next_a = (t + 1) == nxt_t[0], reset_next_b = (t + 1) == nxt_t[1];
    float hn[4];
    [[maybe_unused]] float gi[4], gz[4], go[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float ir = acc[0][i], fr = acc[1][i], zr = acc[2][i], orr = acc[3][i];
      const float lfm = m_[i] + fast_logsigmoid(fr);
      // One of the two stabilised gates is exp(0): with d = lfm - i, the other one is exp(-|d|) (a fresh unit, n == 0,
      // takes m' = i: its input gate is 1 and its forget gate min(1, e^d)).  One exponential instead of two.
      const bool fresh = n_[i] == 0.f;
      const float d = lfm - ir;
      const float mn = (fresh || d <= 0.f) ? ir : lfm;
      const float e = __expf(-fabsf(d));
      const float ig = (d > 0.f && !fresh) ? e : 1.f;
      const float fg = (d <= 0.f) ? e : 1.f;
      // tanh and the sigmoid (0.5 tanh(x/2) + 0.5) on the hardware tanh: one special-function instruction each
      const float zt = tanh_approx(zr), os = fmaf(0.5f, tanh_approx(0.5f * orr), 0.5f);
      c_[i] = fmaf(fg, c_[i], ig * zt);
      n_[i] = fmaf(fg, n_[i], ig);
      m_[i] = mn;
      hn[i] = __fdividef(c_[i], n_[i]) * os;
      if constexpr (TRAIN) { gi[i] = ig; gz[i] = zt; go[i] = os; }
    }
    const uint32_t pa = pack_bf16x2(hn[0], hn[1]), pb = pack_bf16x2(hn[2], hn[3]);
    // a row whose next token opens a new document restarts from the zero state
    uint32_t push_a = pa, push_b = pb;
    if (reset_next_a) {
      push_a = 0u;
      c_[0] = c_[1] = n_[0] = n_[1] = m_[0] = m_[1] = 0.f;
      nxt_t[0] = next_boundary(p, gb_a, t + 1, nxt_idx[0]);
    }
    if (reset_next_b) {
      push_b = 0u;
      c_[2] = c_[3] = n_[2] = n_[3] = m_[2] = m_[3] = 0.f;
      nxt_t[1] = next_boundary(p, gb_b, t + 1, nxt_idx[1]);
    }
    // broadcast h_t into buffer `nxt` of every CTA in the cluster
    const uint32_t nb = s_h_u32 + nxt * (H_TILE * 2);
    {
      uint32_t gr[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t va = __shfl_sync(0xffffffffu, push_a, psrc + i), vb = __shfl_sync(0xffffffffu, push_b, psrc + i);
        gr[i] = prow < 8 ? va : vb;
      }
      if constexpr (NCTA >= 2) {
#pragma unroll
        for (int r = 0; r < NCTA; r += 2) {
          const uint32_t dst = (uint32_t)(r + (lane >> 4));
          st_async_v4(map_to_cta(nb + pslot, dst), gr, map_to_cta(s_bar + 8u * nxt, dst));
        }
      } else {
        if (lane < 16) st_async_v4(map_to_cta(nb + pslot, 0), gr, map_to_cta(s_bar + 8u * nxt, 0));
      }
    }
    if constexpr (TRAIN) {
      // the record of this step (states after the update; the training path takes no document offsets, so nothing was
      // reset above) into this step's staging slot, behind the pushes like the output below
      uint4* r = reinterpret_cast<uint4*>(s_recst + (t % SL_REC_SLOTS) * SL_REC_STEP + tid * SL_REC_BYTES);
      r[0] = make_uint4(pack_bf16x2(gi[0], gi[1]), pack_bf16x2(acc[1][0], acc[1][1]), pack_bf16x2(gz[0], gz[1]), pack_bf16x2(go[0], go[1]));
      r[1] = make_uint4(pack_bf16x2(gi[2], gi[3]), pack_bf16x2(acc[1][2], acc[1][3]), pack_bf16x2(gz[2], gz[3]), pack_bf16x2(go[2], go[3]));
      r[2] = make_uint4(pa, pb, 0u, 0u);
      r[3] = make_uint4(__float_as_uint(c_[0]), __float_as_uint(c_[1]), __float_as_uint(c_[2]), __float_as_uint(c_[3]));
      r[4] = make_uint4(__float_as_uint(n_[0]), __float_as_uint(n_[1]), __float_as_uint(n_[2]), __float_as_uint(n_[3]));
      r[5] = make_uint4(__float_as_uint(m_[0]), __float_as_uint(m_[1]), __float_as_uint(m_[2]), __float_as_uint(m_[3]));
      fence_proxy_async_smem();
    }
    // output h_t, (B, NH, S, DH) -- after the pushes: they are on the step-to-step chain, this store is not
    if (ok_a) *reinterpret_cast<uint32_t*>(hout + (((size_t)gb_a * NH + head) * S + t) * DH + unit_h) = pa;
    if (ok_b) *reinterpret_cast<uint32_t*>(hout + (((size_t)gb_b * NH + head) * S + t) * DH + unit_h) = pb;
#pragma unroll
    for (int i = 0; i < 4; ++i) hlast[i] = hn[i];
    cp_async_wait<SL_RING - 2>();  // this thread's part of step t+1 has landed
    // ... and everybody else's (CTA-wide only); the same barrier tells every thread whether any wait expired
    if (__syncthreads_or(ok ? 0 : 1)) { ok = false; break; }
    if constexpr (TRAIN) {
      if (tid == 0) {
        bulk_store(rec + (size_t)t * SL_REC_STEP, smem_u32(s_recst) + (t % SL_REC_SLOTS) * SL_REC_STEP, SL_REC_STEP);
        bulk_commit();
        bulk_wait_read<1>();   // the copy of step t-1 has read its slot: step t+2, which reuses it, may stage (behind the next barrier)
      }
    }
  }
  if constexpr (TRAIN) {
    if (tid == 0) bulk_wait<0>();
  }
  // The pushes of h_{S-1} are still on their way into tile S & 1 of every CTA; their completion is signalled on that
  // tile's mbarrier only, so it is waited for (bounded) before anybody may leave: a CTA that exits while a peer's
  // asynchronous store into its shared memory is in flight is undefined behaviour.
  if (ok) {
    const int last = S & 1;
    if (!sl_wait(s_bar + 8u * last, (uint32_t)((S >> 1) - (last == 0 ? 1 : 0)) & 1u)) ok = false;
  }
  if (!ok && p.status) atomicExch(p.status, 1);
  cluster_barrier();  // nobody leaves while a peer may still push into its tile

  // final state (4, B, H): h, c, n, m
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gb = (i < 2) ? gb_a : gb_b;
    const bool ok = (i < 2) ? ok_a : ok_b;
    if (!ok) continue;
    const size_t off = (size_t)gb * H + (size_t)head * DH + unit_h + (i & 1);
    p.state_out[0 * (size_t)B * H + off] = hlast[i];
    p.state_out[1 * (size_t)B * H + off] = c_[i];
    p.state_out[2 * (size_t)B * H + off] = n_[i];
    p.state_out[3 * (size_t)B * H + off] = m_[i];
  }
}

template <int DH, bool TRAIN>
static int launch_slstm(const xl_slstm_params* p, cudaStream_t st) {
  constexpr int NCTA = DH / SL_UNITS;
  const size_t smem = 2 * SL_ROWS * DH * 2 + (size_t)SL_RING * SL_WX_STEP_BYTES + 16 +  // + 2 mbarriers
                      (TRAIN ? (size_t)SL_REC_SLOTS * SL_REC_STEP : 0);
  XL_CUDA_TRY(cudaFuncSetAttribute(slstm_forward_kernel<DH, TRAIN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
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
  XL_CUDA_TRY(cudaLaunchKernelEx(&cfg, slstm_forward_kernel<DH, TRAIN>, *p));
  return check_launch("xl_slstm_forward");
}

}  // namespace xl

extern "C" int xl_slstm_forward(const xl_slstm_params* p, void* cuda_stream) {
  using namespace xl;
  if (!p || !p->wx || !p->R || !p->bias || !p->h_out || !p->state_out) return XL_ERR_NULL_POINTER;
  if (p->B <= 0 || p->S <= 0 || p->NH <= 0) return XL_ERR_BAD_SHAPE;
  if (p->dtype != XL_BF16) return XL_ERR_BAD_DTYPE;
  if (p->cu_seqlens && p->num_docs <= 0) return XL_ERR_BAD_SHAPE;
  if (p->NH > 65535 || (p->B + SL_ROWS - 1) / SL_ROWS > 65535) return XL_ERR_TOO_LARGE;
  if (!aligned16(p->wx) || (reinterpret_cast<uintptr_t>(p->h_out) & 3u)) return XL_ERR_BAD_ALIGNMENT;
  if (p->state0 && p->state0 == p->state_out) return XL_ERR_ALIASING;
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  if (p->train_cache) {
    if (p->cu_seqlens) return XL_ERR_UNSUPPORTED;  // the backward pass takes no document offsets
    if (!aligned16(p->train_cache)) return XL_ERR_BAD_ALIGNMENT;
    switch (p->DH) {
      case 64: return launch_slstm<64, true>(p, st);
      case 128: return launch_slstm<128, true>(p, st);
      case 256: return launch_slstm<256, true>(p, st);
      default: return XL_ERR_UNSUPPORTED;
    }
  }
  switch (p->DH) {
    case 64: return launch_slstm<64, false>(p, st);
    case 128: return launch_slstm<128, false>(p, st);
    case 256: return launch_slstm<256, false>(p, st);
    default: return XL_ERR_UNSUPPORTED;
  }
}

extern "C" int64_t xl_slstm_cache_bytes(int32_t B, int32_t S, int32_t NH, int32_t DH) {
  if (B <= 0 || S <= 0 || NH <= 0 || DH <= 0 || DH % xl::SL_UNITS) return 0;
  const int64_t groups = (B + xl::SL_ROWS - 1) / xl::SL_ROWS;
  return groups * NH * (DH / xl::SL_UNITS) * (int64_t)S * xl::SL_THREADS * xl::SL_REC_BYTES;
}
