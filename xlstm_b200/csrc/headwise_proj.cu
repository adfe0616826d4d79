// Headwise gate projections of the sLSTM layer, all four gates in one launch, written straight into the cell's
// (rows, 4, NH, DH) input layout (xlstm/components/linear_headwise.py:75-82 applied four times and the torch.cat of
// xlstm/blocks/slstm/layer.py:145-154).
//
// out[r, s, h, :] = W_s[h] (DH x DH, [out][in]) * x_{sel(s)}[r, h*DH : (h+1)*DH]        s = 0..3, bf16 in, fp32 accumulation
//
// One CTA owns 128 rows (tokens) of one head and walks the four gates: per gate and 64-feature block of the contraction a
// TMA stage holds a [128 x 64] tile of the gate's input and the [DH x 64] tile of its weight (128-byte swizzle); one
// UMMA per 16 features accumulates the [128 x DH] result in tensor memory (two accumulators in turn, so the next gate's
// products run while this one's result leaves); the epilogue warps round to bf16, stage 64-column boxes in shared memory
// and hand them to TMA stores.  Weights (a few MB) stay L2-resident; the kernel is bound by the output stream.
//
// Warp roles: 0 TMA loads, 1 UMMA issue (+ tensor-memory allocation), 2..5 and 6..9 two epilogue groups (tensor-memory
// lane = row; a group takes every other 64-column box of a result, with its own staging boxes and store queue).
#include <cuda.h>

#include "common.cuh"

namespace xl {

constexpr int HW_ROWS = 128;      // rows per CTA (UMMA M)
constexpr int HW_STAGES = 3;
constexpr int HW_THREADS = 320;    // 10 warps: TMA, UMMA, two epilogue groups of four
constexpr int HW_A_BYTES = HW_ROWS * 128;   // [128 rows x 64 bf16]

struct HwMaps {
  CUtensorMap x[2], w[4], out;
};

template <int DH>
struct HwLayout {
  static constexpr int KB = DH / 64;                 // 64-feature blocks of the contraction (and of the output columns)
  static constexpr int B_BYTES = DH * 128;           // [DH rows x 64 bf16]
  static constexpr int STAGE_BYTES = HW_A_BYTES + B_BYTES;
  static constexpr int OFF_OUT = HW_STAGES * STAGE_BYTES;     // 2 groups x 2 x [128 x 64] bf16 staging boxes of the result
  static constexpr int OFF_BAR = OFF_OUT + 4 * HW_A_BYTES;
  static constexpr int NBAR = 2 * HW_STAGES + 4;     // full, empty per stage; accumulator full / empty x 2
  static constexpr int TOTAL = OFF_BAR + NBAR * 8 + 16;
  static constexpr int DYN_SMEM = TOTAL + 1024;
  static constexpr uint32_t TMEM_COLS = 2 * DH >= 512 ? 512 : (2 * DH >= 256 ? 256 : 128);
};

__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const void* tmap, uint32_t bar, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst_smem),
               "l"(tmap), "r"(bar), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void tma_store_2d(const void* tmap, uint32_t src_smem, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(tmap), "r"(src_smem), "r"(c0),
               "r"(c1)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void epilogue_sync(int group) { asm volatile("bar.sync %0, 128;" ::"r"(1 + group) : "memory"); }

// One [128 rows x 64 columns] box of a result on its way out, called by the 128 threads of an epilogue group: the thread's
// row (64 fp32 values, `v`) is rounded to bf16 and written into the group's staging box with the TMA swizzle, then the
// group's first thread hands the box to a TMA store.  `stage` is the shared-memory address of the staging box; the box the
// group used two boxes ago must have been read by its store before it is overwritten.
__device__ __forceinline__ void hw_store_box(unsigned char* smem_stage, uint32_t stage, const uint32_t (&v)[64], int r, int grp, int te,
                                             const CUtensorMap* out_map, int col, int row0, bool in_range) {
  if (te == 0) tma_store_wait_read<1>();
  epilogue_sync(grp);
  unsigned char* stg = smem_stage + r * 128;
#pragma unroll
  for (int c = 0; c < 8; ++c) {   // 16-byte pieces of the row's 64 columns
    uint4 w;
    w.x = pack_bf16x2(__uint_as_float(v[8 * c + 0]), __uint_as_float(v[8 * c + 1]));
    w.y = pack_bf16x2(__uint_as_float(v[8 * c + 2]), __uint_as_float(v[8 * c + 3]));
    w.z = pack_bf16x2(__uint_as_float(v[8 * c + 4]), __uint_as_float(v[8 * c + 5]));
    w.w = pack_bf16x2(__uint_as_float(v[8 * c + 6]), __uint_as_float(v[8 * c + 7]));
    *reinterpret_cast<uint4*>(stg + ((c ^ (r & 7)) << 4)) = w;
  }
  fence_proxy_async_smem();
  epilogue_sync(grp);
  if (te == 0 && in_range) {
    tma_store_2d(out_map, stage, col, row0);
    tma_store_commit();
  }
}

template <int DH>
__global__ void __launch_bounds__(HW_THREADS, 1) headwise_proj_kernel(const __grid_constant__ HwMaps maps, const xl_headwise_params p) {
  using LY = HwLayout<DH>;
  constexpr int KB = LY::KB;
  extern __shared__ unsigned char hw_smem_raw[];
  unsigned char* smem = hw_smem_raw + ((1024u - (smem_u32(hw_smem_raw) & 1023u)) & 1023u);
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = sbase + LY::OFF_BAR;
  auto bar_full = [&](int s) { return bar0 + 8u * (uint32_t)s; };
  auto bar_empty = [&](int s) { return bar0 + 8u * (uint32_t)(HW_STAGES + s); };
  auto bar_acc_full = [&](int a) { return bar0 + 8u * (uint32_t)(2 * HW_STAGES + a); };
  auto bar_acc_empty = [&](int a) { return bar0 + 8u * (uint32_t)(2 * HW_STAGES + 2 + a); };
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + LY::OFF_BAR + LY::NBAR * 8);

  const int tid = threadIdx.x, lane = tid & 31;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);   // provably warp-uniform role dispatch
  const int row0 = blockIdx.x * HW_ROWS, head = blockIdx.y;
  const int nslots = p.n_slots;
  bool ok = true;

  if (tid == 0) {
    for (int s = 0; s < HW_STAGES; ++s) { mbar_init(bar_full(s), 1); mbar_init(bar_empty(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(bar_acc_full(a), 1); mbar_init(bar_acc_empty(a), 256); }
    fence_barrier_init();
    tma_prefetch_desc(&maps.x[0]); tma_prefetch_desc(&maps.out);
  }
  if (warp == 1) {
    __syncwarp();
    tmem_alloc(smem_u32(s_tmem), LY::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *s_tmem;

  if (warp == 0) {
    // ================================================================================ TMA loads
    if (lane == 0) {
      int it = 0;
      for (int slot = 0; slot < nslots && ok; ++slot) {
        const CUtensorMap* xm = &maps.x[p.in_sel[slot] ? 1 : 0];
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int st = it % HW_STAGES;
          if (!mbar_wait(bar_empty(st), ((uint32_t)(it / HW_STAGES) & 1u) ^ 1u)) { ok = false; break; }
          const uint32_t dst = sbase + st * LY::STAGE_BYTES;
          mbar_expect_tx(bar_full(st), LY::STAGE_BYTES);
          tma_load_2d(dst, xm, bar_full(st), head * DH + kb * 64, row0);
          tma_load_2d(dst + HW_A_BYTES, &maps.w[slot], bar_full(st), kb * 64, head * DH);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ================================================================================ UMMA issue
    constexpr uint32_t IDESC = umma_idesc_bf16(HW_ROWS, DH, 0, 0);
    constexpr uint32_t LBO_K = (16u >> 4) << 16;
    const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem, 0), sbase_u = __shfl_sync(0xffffffffu, sbase, 0) & 0x3FFFFu;
    const int nslots_u = __shfl_sync(0xffffffffu, nslots, 0);
    bool okm = true;
    int it = 0;
#pragma unroll 1
    for (int slot = 0; slot < nslots_u; ++slot) {
      const uint32_t acc = tmem_u + (uint32_t)(slot & 1) * DH;
      okm = okm && mbar_wait(bar_acc_empty(slot & 1), ((uint32_t)(slot >> 1) & 1u) ^ 1u);   // passes at once the first time
      tc_fence_after();
#pragma unroll 1
      for (int kb = 0; kb < KB; ++kb, ++it) {
        const int st = it % HW_STAGES;
        okm = okm && mbar_wait(bar_full(st), (uint32_t)(it / HW_STAGES) & 1u);
        tc_fence_after();
        const uint32_t a = sbase_u + st * LY::STAGE_BYTES, b = a + HW_A_BYTES;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_ss_lo(acc, LBO_K + ((a + kk * 32) >> 4), LBO_K + ((b + kk * 32) >> 4), IDESC, (kb | kk) != 0);
        umma_commit_elect(bar_empty(st));   // the stage may be refilled when these products have read it
      }
      umma_commit_elect(bar_acc_full(slot & 1));
    }
    ok = okm;
  } else {
    // ================================================================================ epilogue
    const int q = warp & 3;                       // tensor-memory lane quarter this warp can read
    const int r = q * 32 + lane;                  // row of the tile
    const int grp = (warp - 2) >> 2;              // epilogue group 0 / 1
    const int te = (tid - 64) & 127;              // thread within the group
    const uint32_t lane_base = (uint32_t)(q * 32) << 16;
    const uint32_t stage0 = LY::OFF_OUT + grp * 2 * HW_A_BYTES;
    int box = 0;
    for (int slot = 0; slot < nslots && ok; ++slot) {
      if (!mbar_wait(bar_acc_full(slot & 1), (uint32_t)(slot >> 1) & 1u)) { ok = false; break; }
      tc_fence_after();
      const uint32_t acc = tmem + lane_base + (uint32_t)(slot & 1) * DH;
#pragma unroll 1
      for (int cb = (KB > 1 ? grp : 0); cb < (KB > 1 || grp == 0 ? KB : 0); cb += (KB > 1 ? 2 : 1), ++box) {
        uint32_t v[64];
        tmem_ld_x32(acc + cb * 64, *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
        tmem_ld_x32(acc + cb * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&v[32]));
        tc_wait_ld();
        const uint32_t off = stage0 + (box & 1) * HW_A_BYTES;
        hw_store_box(smem + off, sbase + off, v, r, grp, te, &maps.out, (slot * p.NH + head) * DH + cb * 64, row0, true);
      }
      tc_fence_before();
      mbar_arrive(bar_acc_empty(slot & 1));
    }
    if (te == 0) tma_store_wait_all();
  }

  if (!ok && p.status) atomicExch(p.status, 1);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, LY::TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------
// Pair variant: two CTAs (two neighbouring 128-row tiles of one head) form a cluster and share every weight tile -- each
// loads only HALF of it (DH/2 rows) and one cta_group::2 UMMA (M = 256, N = DH) of the leader drives both tensor cores,
// each on its own rows.  That takes a third off the L2 -> shared-memory traffic, which bounds this kernel (weights are
// re-read by every row tile).  With N = DH >= 128 the pair instruction runs at the rate of the single-CTA one.
// The other CTA's warp 1 forwards "stage landed" to the leader; accumulator-free arrivals come one per warp.
// ---------------------------------------------------------------------------------------------
constexpr int HWP_STAGES = 4;

template <int DH>
struct HwPairLayout {
  static constexpr int KB = DH / 64;
  static constexpr int B_BYTES = (DH / 2) * 128;     // this CTA's half of the [DH x 64] weight tile
  static constexpr int STAGE_BYTES = HW_A_BYTES + B_BYTES;
  static constexpr int OFF_OUT = HWP_STAGES * STAGE_BYTES;
  static constexpr int OFF_BAR = OFF_OUT + 4 * HW_A_BYTES;
  static constexpr int NBAR = 3 * HWP_STAGES + 4;    // full, empty, peer-full per stage; accumulator full / empty x 2
  static constexpr int TOTAL = OFF_BAR + NBAR * 8 + 16;
  static constexpr int DYN_SMEM = TOTAL + 1024;
  static constexpr uint32_t TMEM_COLS = 2 * DH >= 512 ? 512 : (2 * DH >= 256 ? 256 : 128);
};

template <int DH>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(HW_THREADS, 1)
headwise_proj_pair_kernel(const __grid_constant__ HwMaps maps, const xl_headwise_params p) {
  using LY = HwPairLayout<DH>;
  constexpr int KB = LY::KB;
  extern __shared__ unsigned char hw_smem_raw[];
  unsigned char* smem = hw_smem_raw + ((1024u - (smem_u32(hw_smem_raw) & 1023u)) & 1023u);
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = sbase + LY::OFF_BAR;
  auto bar_full = [&](int s) { return bar0 + 8u * (uint32_t)s; };
  auto bar_empty = [&](int s) { return bar0 + 8u * (uint32_t)(HWP_STAGES + s); };
  auto bar_pfull = [&](int s) { return bar0 + 8u * (uint32_t)(2 * HWP_STAGES + s); };       // leader: the other CTA's stage landed
  auto bar_acc_full = [&](int a) { return bar0 + 8u * (uint32_t)(3 * HWP_STAGES + a); };
  auto bar_acc_empty = [&](int a) { return bar0 + 8u * (uint32_t)(3 * HWP_STAGES + 2 + a); };  // leader: 8 warps of each CTA
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + LY::OFF_BAR + LY::NBAR * 8);

  const int tid = threadIdx.x, lane = tid & 31;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
  const uint32_t rank = cluster_ctarank();
  const int nslots = p.n_slots;
  // persistent: the pair walks work items (pair of row tiles, head); the rings of stages and accumulators run on across
  // items, so loads, products and stores of neighbouring items overlap
  const int n_pairs = (int)((p.rows + 2 * HW_ROWS - 1) / (2 * HW_ROWS));
  const int total_items = n_pairs * p.NH, n_clusters = (int)gridDim.x / 2, first_item = (int)blockIdx.x / 2;
  auto item_row0 = [&](int item) { return ((item / p.NH) * 2 + (int)rank) * HW_ROWS; };
  auto item_head = [&](int item) { return item % p.NH; };
  bool ok = true;

  if (tid == 0) {
    for (int s = 0; s < HWP_STAGES; ++s) { mbar_init(bar_full(s), 1); mbar_init(bar_empty(s), 1); mbar_init(bar_pfull(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(bar_acc_full(a), 1); mbar_init(bar_acc_empty(a), 16); }
    fence_barrier_init();
    tma_prefetch_desc(&maps.x[0]); tma_prefetch_desc(&maps.out);
  }
  if (warp == 1) {
    __syncwarp();
    tmem_alloc(smem_u32(s_tmem), LY::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  cluster_sync_all();   // barriers and tensor memory of BOTH CTAs exist before anything crosses over
  tc_fence_after();
  const uint32_t tmem = *s_tmem;
  const uint32_t lead_bar0 = mapa_u32(bar0, 0);

  if (warp == 0) {
    // ================================================================================ TMA loads (each CTA its own)
    if (lane == 0) {
      int it = 0;
      for (int item = first_item; item < total_items && ok; item += n_clusters) {
        const int row0 = item_row0(item), head = item_head(item);
        for (int slot = 0; slot < nslots && ok; ++slot) {
          const CUtensorMap* xm = &maps.x[p.in_sel[slot] ? 1 : 0];
          for (int kb = 0; kb < KB; ++kb, ++it) {
            const int st = it % HWP_STAGES;
            if (!mbar_wait(bar_empty(st), ((uint32_t)(it / HWP_STAGES) & 1u) ^ 1u)) { ok = false; break; }
            const uint32_t dst = sbase + st * LY::STAGE_BYTES;
            mbar_expect_tx(bar_full(st), LY::STAGE_BYTES);
            tma_load_2d(dst, xm, bar_full(st), head * DH + kb * 64, row0);
            tma_load_2d(dst + HW_A_BYTES, &maps.w[slot], bar_full(st), kb * 64, head * DH + (int)rank * (DH / 2));
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (__shfl_sync(0xffffffffu, rank, 0) == 0) {
      // ============================================================================== UMMA issue (leader of the pair)
      constexpr uint32_t IDESC = umma_idesc_bf16(2 * HW_ROWS, DH, 0, 0);
      constexpr uint32_t LBO_K = (16u >> 4) << 16;
      const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem, 0), sbase_u = __shfl_sync(0xffffffffu, sbase, 0) & 0x3FFFFu;
      int n_items = 0;
      for (int item = first_item; item < total_items; item += n_clusters) ++n_items;
      const int nslots_u = __shfl_sync(0xffffffffu, nslots * n_items, 0);   // accumulator uses of this pair, all items
      bool okm = true;
      int it = 0;
#pragma unroll 1
      for (int slot = 0; slot < nslots_u; ++slot) {
        const uint32_t acc = tmem_u + (uint32_t)(slot & 1) * DH;
        okm = okm && mbar_wait(bar_acc_empty(slot & 1), ((uint32_t)(slot >> 1) & 1u) ^ 1u);
        tc_fence_after();
#pragma unroll 1
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int st = it % HWP_STAGES;
          okm = okm && mbar_wait(bar_full(st), (uint32_t)(it / HWP_STAGES) & 1u);
          okm = okm && mbar_wait(bar_pfull(st), (uint32_t)(it / HWP_STAGES) & 1u);
          tc_fence_after();
          const uint32_t a = sbase_u + st * LY::STAGE_BYTES, b = a + HW_A_BYTES;
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma2_ss_lo(acc, LBO_K + ((a + kk * 32) >> 4), LBO_K + ((b + kk * 32) >> 4), IDESC, (kb | kk) != 0);
          umma2_commit_both(bar_empty(st));   // both CTAs may refill the stage when these products have read it
        }
        umma2_commit_both(bar_acc_full(slot & 1));
      }
      ok = okm;
    } else {
      // ============================================================================== the other CTA: forward "stage landed"
      if (lane == 0) {
        int n_items = 0;
        for (int item = first_item; item < total_items; item += n_clusters) ++n_items;
        const int total_it = nslots * KB * n_items;
        for (int it = 0; it < total_it; ++it) {
          const int st = it % HWP_STAGES;
          if (!mbar_wait(bar_full(st), (uint32_t)(it / HWP_STAGES) & 1u)) { ok = false; break; }
          mbar_arrive_remote(lead_bar0 + 8u * (uint32_t)(2 * HWP_STAGES + st));
        }
      }
      __syncwarp();
    }
  } else {
    // ================================================================================ epilogue (each CTA its own rows)
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const int grp = (warp - 2) >> 2;
    const int te = (tid - 64) & 127;
    const uint32_t lane_base = (uint32_t)(q * 32) << 16;
    const uint32_t stage0 = LY::OFF_OUT + grp * 2 * HW_A_BYTES;
    int box = 0, gs = 0;   // staging boxes and accumulator uses so far, all items
    for (int item = first_item; item < total_items && ok; item += n_clusters) {
    const int row0 = item_row0(item), head = item_head(item);
    for (int slot = 0; slot < nslots && ok; ++slot, ++gs) {
      if (!mbar_wait(bar_acc_full(gs & 1), (uint32_t)(gs >> 1) & 1u)) { ok = false; break; }
      tc_fence_after();
      const uint32_t acc = tmem + lane_base + (uint32_t)(gs & 1) * DH;
      // this group's boxes of the result (every other 64-column box): all of them out of tensor memory first, so that the
      // accumulator goes back to the UMMA issuer before the staging and the stores start
      constexpr int NBX = KB / 2;   // KB >= 2 here (DH >= 128)
      uint32_t v[NBX][64];
#pragma unroll
      for (int i = 0; i < NBX; ++i) {
        tmem_ld_x32(acc + (2 * i + grp) * 64, *reinterpret_cast<uint32_t(*)[32]>(&v[i][0]));
        tmem_ld_x32(acc + (2 * i + grp) * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&v[i][32]));
      }
      tc_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {   // one arrival per warp on the leader's barrier
        if (rank == 0) mbar_arrive(bar_acc_empty(gs & 1));
        else mbar_arrive_remote(lead_bar0 + 8u * (uint32_t)(3 * HWP_STAGES + 2 + (gs & 1)));
      }
#pragma unroll
      for (int i = 0; i < NBX; ++i, ++box) {
        const uint32_t off = stage0 + (box & 1) * HW_A_BYTES;
        hw_store_box(smem + off, sbase + off, v[i], r, grp, te, &maps.out, (slot * p.NH + head) * DH + (2 * i + grp) * 64, row0, row0 < p.rows);
      }
    }
    }
    if (te == 0) tma_store_wait_all();
  }

  if (!ok && p.status) atomicExch(p.status, 1);
  tc_fence_before();
  cluster_sync_all();   // neither CTA leaves (or frees tensor memory) while the other may still reach into it
  if (warp == 1) tmem_dealloc(tmem, LY::TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*hw_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static hw_encode_fn hw_get_encode_fn() {
  static hw_encode_fn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<hw_encode_fn>(sym);
  }
  return fn;
}

// row-major bf16 matrix [rows x cols] with a row stride in elements -> 2-D map, box = 64 columns x box_rows rows
static int hw_make_map(CUtensorMap* m, const void* base, int64_t rows, int64_t cols, int64_t row_stride, int box_rows) {
  hw_encode_fn enc = hw_get_encode_fn();
  if (!enc) {
    set_last_cuda_error(cudaErrorSymbolNotFound, "cudaGetDriverEntryPoint(cuTensorMapEncodeTiled)");
    return XL_ERR_CUDA;
  }
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)row_stride * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled rejected the matrix layout");
    return XL_ERR_BAD_STRIDE;
  }
  return XL_OK;
}

template <int DH>
static int launch_headwise_pair(const HwMaps& maps, const xl_headwise_params* p, cudaStream_t st) {
  using LY = HwPairLayout<DH>;
  static_assert(LY::DYN_SMEM <= 227 * 1024, "shared memory budget");
  auto kern = headwise_proj_pair_kernel<DH>;
  XL_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, LY::DYN_SMEM));
  // persistent pairs: as many clusters as can be resident at once (a tile past the last row loads zeros, stores nothing)
  const long long items = ((p->rows + 2 * HW_ROWS - 1) / (2 * HW_ROWS)) * (long long)p->NH;
  int resident = 0;
  {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * 74);
    cfg.blockDim = dim3(HW_THREADS);
    cfg.dynamicSmemBytes = LY::DYN_SMEM;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    if (cudaOccupancyMaxActiveClusters(&resident, kern, &cfg) != cudaSuccess || resident < 1) {
      (void)cudaGetLastError();
      cfg.attrs = nullptr; cfg.numAttrs = 0;   // (the kernel carries its cluster shape itself)
      if (cudaOccupancyMaxActiveClusters(&resident, kern, &cfg) != cudaSuccess || resident < 1) { (void)cudaGetLastError(); resident = 64; }
    }
    if (resident > 74) resident = 74;
  }
  const unsigned clusters = (unsigned)(items < resident ? items : resident);
  kern<<<dim3(2 * clusters), HW_THREADS, LY::DYN_SMEM, st>>>(maps, *p);
  return check_launch("xl_headwise_proj");
}

template <int DH>
static int launch_headwise(const HwMaps& maps, const xl_headwise_params* p, cudaStream_t st) {
  using LY = HwLayout<DH>;
  static_assert(LY::DYN_SMEM <= 227 * 1024, "shared memory budget");
  auto kern = headwise_proj_kernel<DH>;
  XL_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, LY::DYN_SMEM));
  dim3 grid((unsigned)((p->rows + HW_ROWS - 1) / HW_ROWS), (unsigned)p->NH);
  kern<<<grid, HW_THREADS, LY::DYN_SMEM, st>>>(maps, *p);
  return check_launch("xl_headwise_proj");
}

}  // namespace xl

extern "C" int xl_headwise_proj(const xl_headwise_params* p, void* cuda_stream) {
  using namespace xl;
  if (!p || !p->out || !p->x[0]) return XL_ERR_NULL_POINTER;
  if (p->dtype != XL_BF16) return XL_ERR_BAD_DTYPE;
  if (p->n_slots < 1 || p->n_slots > 4 || p->NH < 1 || p->rows < 0) return XL_ERR_BAD_SHAPE;
  if (!(p->DH == 64 || p->DH == 128 || p->DH == 256)) return XL_ERR_UNSUPPORTED;
  if (p->rows == 0) return XL_OK;
  const int64_t D = (int64_t)p->NH * p->DH;
  bool use[2] = {false, false};
  for (int s = 0; s < p->n_slots; ++s) {
    if (!p->w[s]) return XL_ERR_NULL_POINTER;
    if (!aligned16(p->w[s])) return XL_ERR_BAD_ALIGNMENT;
    if (p->in_sel[s] != 0 && p->in_sel[s] != 1) return XL_ERR_BAD_SHAPE;
    use[p->in_sel[s]] = true;
  }
  if (use[1] && !p->x[1]) return XL_ERR_NULL_POINTER;
  for (int i = 0; i < 2; ++i)
    if (use[i]) {
      if (!aligned16(p->x[i])) return XL_ERR_BAD_ALIGNMENT;
      if (p->x_row_stride[i] < D || p->x_row_stride[i] % 8 != 0) return XL_ERR_BAD_STRIDE;
    }
  if (!aligned16(p->out)) return XL_ERR_BAD_ALIGNMENT;
  if (p->out_row_stride < p->n_slots * D || p->out_row_stride % 8 != 0) return XL_ERR_BAD_STRIDE;
  HwMaps maps;
  int rc;
  for (int i = 0; i < 2; ++i) {
    const int src = use[i] ? i : (use[0] ? 0 : 1);   // an unused input slot gets a valid map of the other one
    if ((rc = hw_make_map(&maps.x[i], p->x[src], p->rows, D, p->x_row_stride[src], HW_ROWS)) != XL_OK) return rc;
  }
  // pairs of row tiles share the weight tiles (each CTA loads half of one) where the pair instruction runs at full rate
  const bool pair = p->DH >= 128 && p->rows > HW_ROWS;
  for (int s = 0; s < 4; ++s) {
    const int src = s < p->n_slots ? s : 0;
    if ((rc = hw_make_map(&maps.w[s], p->w[src], D, p->DH, p->DH, pair ? p->DH / 2 : p->DH)) != XL_OK) return rc;
  }
  if ((rc = hw_make_map(&maps.out, p->out, p->rows, (int64_t)p->n_slots * D, p->out_row_stride, HW_ROWS)) != XL_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  if (pair) return p->DH == 128 ? launch_headwise_pair<128>(maps, p, st) : launch_headwise_pair<256>(maps, p, st);
  switch (p->DH) {
    case 64: return launch_headwise<64>(maps, p, st);
    case 128: return launch_headwise<128>(maps, p, st);
    default: return launch_headwise<256>(maps, p, st);
  }
}
