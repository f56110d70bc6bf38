// CTA-pair variant of the MX-GEMM kernel: two CTAs on neighbouring SMs (a cluster of two) compute one
// 256 x 256 output tile with tcgen05.mma.cta_group::2.
//
// Why: with one CTA per 128 x 256 tile the tensor core re-reads 12 KiB of shared memory per
// 128 x 256 x 32 MMA while TMA refills the same amount, which saturates the SM's shared-memory
// bandwidth before the tensor pipe. As a pair, each CTA stages only its own 128 rows of X and HALF
// of the Y tile (128 of the 256 columns); the MMA unit of each SM reads the other half from the
// peer's shared memory. Per-SM fill traffic drops from 48 to 32 KiB per K block.
//
// The reference gets its operand sharing from TMA cluster multicast
// (mxblas/gemm/generator.py:545-578). Nothing is multicast here: every TMA load targets the
// issuing CTA's own shared memory; only mbarrier signals cross the pair.
//
// Roles per CTA: warp 0 = TMA producer (both CTAs), warp 1 = MMA issuer (leader CTA only; also TMEM
// owner in both), then the epilogue warps (both CTAs, each for its own 128 rows).
//
// Scales that change along K (SCALE_PROMOTE, one scale group per 128-deep K block): every K block's
// partial sum is left in one of the two TMEM buffers and added, scaled, to register sums by eight
// promotion warps per CTA (promote_groups in mxb_kernel.cuh). One tcgen05.commit per K block then
// serves two purposes: it frees the shared-memory stage for the producers and tells the promotion
// warps of both CTAs that the partial sum is complete, so they wait on the stage's empty barrier.
//
// Block-scaled MMA (SCALE_MX): the UE8M0 scale factors do not pass through shared memory. Four
// scale-factor warps per CTA (one per TMEM lane quadrant) read the packed factors from global memory,
// four K blocks ahead, and write them into one of four TMEM column slots with tcgen05.st; their arrival
// on the leader's full barrier tells the MMA thread that the slots of a stage pair are filled.
// (Copying them with tcgen05.cp from the MMA thread put six copies per stage pair in front of the
// MMAs in the tensor pipe's queue: a quarter of the kernel's time.)
// Barriers: full[] lives in the leader, one barrier per two stages, and collects both CTAs' loads;
// empty[s] and tfull[b] exist in both CTAs and are signalled by one tcgen05.commit whose arrival is
// delivered to both CTAs; tempty[b] lives in the leader and collects the epilogue warps of both CTAs.
#pragma once

#include "mxb_kernel.cuh"

namespace mxb {

// BN_ = columns of the pair's tile: 256, or 224 (the block-scaled MMA needs TMEM columns for the scale factors
// next to the two accumulator buffers; with scales constant along K the narrower tile exists as a
// configuration: the MMAs are bound by shared-memory traffic, which shrinks by 6 % only, so saving a wave of
// tiles with it measured no faster). Each CTA stages BN/2 rows of Y.
// SINGLE_Y_ (promotion only): every thread's column slice lies inside one scale block of Y (128 x 128 weight
// blocks): the lean loop promote_groups_single_y replaces the general one.
template <int BN_, int SCALE_MODE_, int OUT_MODE_, int EPI_WARPS_, bool GENERAL_ = false, bool SINGLE_Y_ = false>
struct PairCfg {
  static constexpr bool GENERAL = GENERAL_;  // operands stored along their rows and grouped GEMMs (see KernelCfg)
  static constexpr bool SINGLE_Y = SINGLE_Y_;
  static_assert(!SINGLE_Y_ || SCALE_MODE_ == SCALE_PROMOTE, "single-scale twins exist for promotion only");
  static constexpr int BN = BN_;
  static constexpr int BM_PAIR = 256;      // rows of the pair's tile (each CTA owns 128)
  static constexpr int SCALE_MODE = SCALE_MODE_;
  static constexpr int OUT_MODE = OUT_MODE_;
  static constexpr int EPI_WARPS = EPI_WARPS_;
  // promotion keeps 128 running sums per thread: registers move from the control warpgroup to the
  // promotion warps (setmaxnreg), which needs whole warpgroups on both sides
  static constexpr bool REG_REALLOC = SCALE_MODE == SCALE_PROMOTE;
  static constexpr int CTRL_WARPS = REG_REALLOC ? 4 : 2;
  static constexpr int SF_WARPS = SCALE_MODE == SCALE_MX ? 4 : 0;  // one per TMEM lane quadrant
  static constexpr int FIRST_EPI_WARP = CTRL_WARPS + SF_WARPS;
  static constexpr int THREADS = (FIRST_EPI_WARP + EPI_WARPS) * 32;
  static constexpr int A_BYTES = 128 * 128;
  static constexpr int B_BYTES = (BN / 2) * 128;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  // arrivals on a full barrier (two stages): one expect-tx per stage and CTA, plus, block-scaled, one
  // per scale-factor warp of either CTA
  static constexpr int FULL_ARRIVALS = 4 + 2 * SF_WARPS;
  static constexpr int COL_SPLIT = EPI_WARPS / 4;
  static constexpr int COLS_PER_THREAD = BN / COL_SPLIT;
  static constexpr int CHUNKS = COLS_PER_THREAD / 32;
  static constexpr int PROMOTE_BATCH = 4;  // groups of per-column Y scales staged at a time
  static constexpr int YS_BYTES =
      SCALE_MODE == SCALE_PROMOTE ? EPI_WARPS * PROMOTE_BATCH * COLS_PER_THREAD * 4 : EPI_WARPS * BN * 4;
  static constexpr int XMAX_BYTES = 2 * 2 * 4 * 32 * 4;
  static constexpr int BAR_BYTES = 512;
  static constexpr int AUX_BYTES = YS_BYTES + XMAX_BYTES + BAR_BYTES;
  // 128-column tiles (promotion only): four accumulator buffers of 128 columns, so that a promotion warp may
  // run three K blocks behind the MMAs, and every thread's 64 columns of a partial sum fit in registers at
  // once: the buffer goes back to the MMA thread after ONE TMEM round trip instead of three
  static constexpr int STAGES = BN <= 128 ? 8 : 6;
  static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + AUX_BYTES;
  static constexpr int ACC_STRIDE = BN <= 128 ? 128 : 256;
  static constexpr int NUM_ACC = 512 / ACC_STRIDE;
  // MX: four scale-factor slots of 16 columns (X factors in columns 0..3 of a slot, Y factors in
  // 4..11) in the columns the two 224-wide accumulators leave free: 224..255 and 480..511
  static constexpr int SF_SLOTS = 4, SFB_OFFSET = 4;
  __host__ __device__ static constexpr uint32_t sf_col(uint32_t slot) {
    return slot < 2 ? 224u + 16u * slot : 480u + 16u * (slot - 2);
  }
  static_assert(SMEM_BYTES <= 232448, "shared memory budget");
  static_assert(STAGES % 2 == 0, "full barriers cover stage pairs");
  static_assert(BN == 256 || (BN == 224 && SCALE_MODE != SCALE_PROMOTE) || (BN == 128 && SCALE_MODE != SCALE_MX),
                "tile widths of the pair kernel");
  static_assert(NUM_ACC * ACC_STRIDE <= 512 && STAGES > NUM_ACC, "promotion: a stage's barrier is observed before it turns again");
  static_assert(SCALE_MODE != SCALE_MX || BN == 224, "block-scaled pairs use 224 columns");
  static_assert(COLS_PER_THREAD % 32 == 0, "whole 32-column chunks per epilogue thread");
  static_assert(SCALE_MODE != SCALE_PROMOTE || EPI_WARPS == 8, "promotion: eight warps of 128 columns");
};

// A unit of work of a CTA pair: a whole tile, or one K slice of a tile of the incomplete last wave.
struct PairUnit {
  int t, kb0, kb1;  // tile, K blocks [kb0, kb1)
  int slot;         // K-sliced tiles: index of this unit among all slice units (workspace position)
  int first_slot;   //                 index of the tile's first slice unit
  int tail_tile;    //                 index of the tile among the sliced tiles
  bool whole;
};
__device__ __forceinline__ PairUnit pair_unit(int u, const GemmParams& p) {
  if (u < p.tail_first) return PairUnit{u, 0, p.kblocks, 0, 0, 0, true};
  const int r = u - p.tail_first;
  const int tt = r / p.tail_splits, sp = r - tt * p.tail_splits;
  return PairUnit{p.tail_first + tt,
                  static_cast<int>((static_cast<unsigned>(p.kblocks) * static_cast<unsigned>(sp)) / static_cast<unsigned>(p.tail_splits)),
                  static_cast<int>((static_cast<unsigned>(p.kblocks) * static_cast<unsigned>(sp + 1)) / static_cast<unsigned>(p.tail_splits)),
                  r, tt * p.tail_splits, tt, false};
}

template <class Cfg>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Cfg::THREADS, 1)
mx_gemm_sm100_pair(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_y,
                   const __grid_constant__ GemmParams p) {
  constexpr int BN = Cfg::BN;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int NUM_ACC = Cfg::NUM_ACC;

  // device-side dispatch of a probed call: both CTAs of every pair read the same word, so a pair leaves
  // together, before anything is signalled across it
  if (p.gate != nullptr && *p.gate != p.gate_value) return;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = sA + STAGES * Cfg::A_BYTES;
  uint8_t* aux = sB + STAGES * Cfg::B_BYTES;
  float* sYs = reinterpret_cast<float*>(aux);
  float* sXmax = reinterpret_cast<float*>(aux + Cfg::YS_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(aux + Cfg::YS_BYTES + Cfg::XMAX_BYTES);
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * STAGES;
  const uint32_t bar_tfull = bar_empty + 8 * STAGES;
  const uint32_t bar_tempty = bar_tfull + 8 * NUM_ACC;
  const uint32_t bar_x = bar_tempty + 8 * NUM_ACC;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 2 * NUM_ACC + 2);
  volatile uint32_t* abort_flag = tmem_holder + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();  // 0 = leader

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      // a full barrier covers TWO consecutive stages (the MMA thread waits once per two stages, a
      // wait costs it ~200 cycles): one expect-tx arrival per stage and CTA; only even slots are used
      mbar_init(bar_full + 8 * s, Cfg::FULL_ARRIVALS);
      mbar_init(bar_empty + 8 * s, 1);  // tcgen05.commit of the leader
    }
    for (int b = 0; b < NUM_ACC; ++b) {
      mbar_init(bar_tfull + 8 * b, 1);
      mbar_init(bar_tempty + 8 * b, 2 * Cfg::EPI_WARPS);  // epilogue warps of both CTAs
    }
    mbar_init(bar_x, 4);
    mbar_init(bar_x + 8, 4);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_x);
    tma_prefetch_desc(&tm_y);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_holder), 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything is signalled across the pair
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  const int num_tiles = p.tiles_x * p.tiles_y;
  const int num_units = p.tail_first + (num_tiles - p.tail_first) * p.tail_splits;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  if (warp < Cfg::CTRL_WARPS) {
  // control warpgroup: give registers away (all of its warps execute this together)
  if constexpr (Cfg::REG_REALLOC) reg_dealloc<40>();
  if (warp == 0) {
    // ------------------------------- TMA producer (both CTAs) --------------------------------
    if (lane == 0) {
      uint32_t s = 0, ph = 0;
      bool ok = true;
      const uint32_t fb0 = map_to_cta(bar_full, 0);  // the leader's barriers
      for (int u = pair; u < num_units && ok; u += num_pairs) {
        const PairUnit un = pair_unit(u, p);
        const TileCoord tc = tile_coord(un.t, p);
        const int grp = tile_group<Cfg>(p, tc.tx * 256);  // grouped GEMM: blocks of whole 256-row tiles
        if (grp < 0) continue;
        const int xr = tc.tx * 256 + static_cast<int>(rank) * 128;
        const int yr = (tc.ty + grp * p.group_tiles_y) * BN + static_cast<int>(rank) * (BN / 2);
        for (int kb = un.kb0; kb < un.kb1; ++kb) {
          ok = mbar_wait_cluster(bar_empty + 8 * s, ph ^ 1, abort_flag, p.status, DEV_TIMEOUT_PRODUCER);
          if (!ok) break;
          const uint32_t fb = fb0 + 8 * (s & ~1u);
          mbar_expect_tx_cluster(fb, Cfg::STAGE_BYTES);
          if (x_by_rows<Cfg>(p)) tma_load_2d_pair(smem_u32(sA + s * Cfg::A_BYTES), &tm_x, fb, xr, kb * 128);
          else tma_load_2d_pair(smem_u32(sA + s * Cfg::A_BYTES), &tm_x, fb, kb * 128, xr);
          // (an operand stored along its rows is only planned with 256-wide tiles: this CTA's half is one box)
          if (y_by_rows<Cfg>(p)) tma_load_2d_pair(smem_u32(sB + s * Cfg::B_BYTES), &tm_y, fb, yr, kb * 128);
          else tma_load_2d_pair(smem_u32(sB + s * Cfg::B_BYTES), &tm_y, fb, kb * 128, yr);
          if (++s == STAGES) {
            s = 0;
            ph ^= 1;
          }
        }
      }
      // an odd total leaves the last stage pair half filled: complete it with a plain arrival
      if (ok && (s & 1)) mbar_arrive_cluster(fb0 + 8 * (s & ~1u));
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------- MMA issuer (leader CTA) ---------------------------------
    if (lane == 0 && rank == 0) {
      // one thread feeds both tensor cores: per MMA only additions and compares (see mxb_kernel.cuh)
      uint32_t s = 0, ph = 0, b = 0, aph = 0;
      uint32_t slot = 0;  // block-scaled: TMEM scale-factor slot of the current stage
      bool ok = true;
      const uint32_t idesc = umma_idesc_major(Cfg::SCALE_MODE == SCALE_MX ? umma_idesc_mxf8(256, BN, p.fmt_x, p.fmt_y)
                                                                          : umma_idesc_f8(256, BN, p.fmt_x, p.fmt_y),
                                              x_by_rows<Cfg>(p), y_by_rows<Cfg>(p));
      const uint32_t kstep_a = x_by_rows<Cfg>(p) ? 256u : 2u, kstep_b = y_by_rows<Cfg>(p) ? 256u : 2u;
      // This thread paces the pair's tensor cores (an artificial 100 cycles per K block in this loop cost config 2
      // 12 % and config 4 10 %, measured), so per K block it does as little as it can: the descriptors' high
      // words are constants, their low words (address field in 16-byte units) step from stage to stage by one
      // 32-bit addition, the instruction descriptors of the four K slices are chosen here, and only the first
      // MMA of a unit computes its accumulate predicate.
      const uint64_t hi_a = umma_desc_hi(x_by_rows<Cfg>(p)), hi_b = umma_desc_hi(y_by_rows<Cfg>(p));
      const uint32_t a_hi = static_cast<uint32_t>(hi_a >> 32), b_hi = static_cast<uint32_t>(hi_b >> 32);
      const uint32_t a_lo0 = static_cast<uint32_t>(hi_a) | ((smem_u32(sA) >> 4) & 0x3FFFu);
      const uint32_t b_lo0 = static_cast<uint32_t>(hi_b) | ((smem_u32(sB) >> 4) & 0x3FFFu);
      constexpr uint32_t A_STEP = Cfg::A_BYTES >> 4, B_STEP = Cfg::B_BYTES >> 4;
      uint32_t a_lo = a_lo0, b_lo = b_lo0;  // of stage s
      const uint32_t idesc_k[4] = {umma_idesc_sf_ids(idesc, 0, 0), umma_idesc_sf_ids(idesc, 1, 1),
                                   umma_idesc_sf_ids(idesc, 2, 2), umma_idesc_sf_ids(idesc, 3, 3)};
      for (int u = pair; u < num_units && ok; u += num_pairs) {
        const PairUnit un = pair_unit(u, p);
        if (Cfg::GENERAL && p.x_group != nullptr && tile_group<Cfg>(p, tile_coord(un.t, p).tx * 256) < 0) continue;
        if constexpr (Cfg::SCALE_MODE != SCALE_PROMOTE) {
          ok = mbar_wait_cluster(bar_tempty + 8 * b, aph ^ 1, abort_flag, p.status, DEV_TIMEOUT_MMA_TMEM);
          if (!ok) break;
          tc_fence_after();
        }
        uint32_t d_tmem = tmem_base + b * Cfg::ACC_STRIDE;
        // the four MMAs of the K block staged in `s`, the commit that hands the stage back, and the step to the
        // next stage (without the wrap, which only follows an odd stage)
        auto issue_stage = [&](uint32_t accumulate) {
          if constexpr (Cfg::SCALE_MODE == SCALE_MX) {
            // the stage's scale factors are in TMEM slot `slot` of both CTAs (the full barrier counted
            // the scale-factor warps' arrivals)
            static_assert(Cfg::sf_col(2) == Cfg::sf_col(0) + 32 + 224 && Cfg::sf_col(3) == Cfg::sf_col(1) + 32 + 224, "slots");
            const uint32_t sf = tmem_base + Cfg::sf_col(0) + 16u * slot + 112u * (slot & 2u);
            umma_mxf8_pair(d_tmem, umma_desc_words(a_lo, a_hi), umma_desc_words(b_lo, b_hi), idesc_k[0], accumulate, sf,
                           sf + Cfg::SFB_OFFSET);
#pragma unroll
            for (int kk = 1; kk < 4; ++kk)
              umma_mxf8_pair_acc(d_tmem, umma_desc_words(a_lo + kk * kstep_a, a_hi),
                                 umma_desc_words(b_lo + kk * kstep_b, b_hi), idesc_k[kk], sf, sf + Cfg::SFB_OFFSET);
            slot = (slot + 1) & (Cfg::SF_SLOTS - 1);
          } else {
            umma_f8_pair(d_tmem, umma_desc_words(a_lo, a_hi), umma_desc_words(b_lo, b_hi), idesc, accumulate);
#pragma unroll
            for (int kk = 1; kk < 4; ++kk)
              umma_f8_pair_acc(d_tmem, umma_desc_words(a_lo + kk * kstep_a, a_hi),
                               umma_desc_words(b_lo + kk * kstep_b, b_hi), idesc);
          }
          // the stage is free in both CTAs once these MMAs have read it (promotion: and the partial
          // sum of this K block is complete)
          umma_commit_pair_both(bar_empty + 8 * s, 3);
          a_lo += A_STEP;
          b_lo += B_STEP;
          ++s;
        };
        auto wrap_ring = [&]() {
          if (s == static_cast<uint32_t>(STAGES)) {
            s = 0;
            ph ^= 1;
            a_lo = a_lo0;
            b_lo = b_lo0;
          }
        };
        if constexpr (Cfg::SCALE_MODE == SCALE_PROMOTE) {
          for (int kb = un.kb0; kb < un.kb1; ++kb) {
            if ((s & 1) == 0) {  // both stages of the pair have landed once this barrier completes
              ok = mbar_wait_cluster(bar_full + 8 * s, ph, abort_flag, p.status, DEV_TIMEOUT_MMA_FULL);
              if (!ok) break;
              tc_fence_after();
            }
            // one partial sum per K block, alternating between the TMEM buffers
            ok = mbar_wait_cluster(bar_tempty + 8 * b, aph ^ 1, abort_flag, p.status, DEV_TIMEOUT_MMA_TMEM);
            if (!ok) break;
            tc_fence_after();
            d_tmem = tmem_base + b * Cfg::ACC_STRIDE;
            issue_stage(0u);
            wrap_ring();
            if (++b == NUM_ACC) {
              b = 0;
              aph ^= 1;
            }
          }
        } else {
          // Whole stage pairs per turn (one full barrier covers a pair): one wait, eight MMAs, two commits, one
          // wrap test. A unit may begin on the second stage of a pair (the previous unit passed its barrier) and
          // end on the first (the pair's barrier then also covers the next unit's first K block).
          int kb = un.kb0;
          uint32_t accumulate = 0;
          if ((s & 1) != 0 && kb < un.kb1) {
            issue_stage(accumulate);
            accumulate = 1;
            wrap_ring();
            ++kb;
          }
          for (; kb + 2 <= un.kb1; kb += 2) {
            ok = mbar_wait_cluster(bar_full + 8 * s, ph, abort_flag, p.status, DEV_TIMEOUT_MMA_FULL);
            if (!ok) break;
            tc_fence_after();
            issue_stage(accumulate);
            accumulate = 1;
            issue_stage(1u);
            wrap_ring();
          }
          if (ok && kb < un.kb1) {
            ok = mbar_wait_cluster(bar_full + 8 * s, ph, abort_flag, p.status, DEV_TIMEOUT_MMA_FULL);
            if (ok) {
              tc_fence_after();
              issue_stage(accumulate);
            }
          }
        }
        if (!ok) break;
        if constexpr (Cfg::SCALE_MODE != SCALE_PROMOTE) {
          umma_commit_pair_both(bar_tfull + 8 * b, 3);
          if (++b == NUM_ACC) {
            b = 0;
            aph ^= 1;
          }
        }
      }
    }
    __syncwarp();
  }
  } else if (warp < Cfg::FIRST_EPI_WARP) {
    if constexpr (Cfg::SCALE_MODE == SCALE_MX) {
      // ------------------------------- scale-factor warps (both CTAs) --------------------------
      // Packed factors (pack_scale_factors in mxb_host.cu): X [128-row tile][K block][512 B],
      // Y [tile][K block][2][512 B]; within a 512-byte atom lane l's 16 bytes are the four 32-bit TMEM
      // columns of lane l. Every warp writes the same 12 columns into its own lane quadrant.
      const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
      const uint32_t fb0 = map_to_cta(bar_full, 0);
      // Factors are loaded four K blocks (two stage pairs, ~2 us) before they are stored. The loop runs over
      // this pair's K blocks, all tiles in sequence, unrolled by four so that block i always uses register
      // set i % 4 and TMEM slot i % 4: no register is moved while its load is in flight.
      constexpr int AHEAD = Cfg::SF_SLOTS;
      int lt = pair, lkb = 0;  // load position: tile and K block
      const uint8_t* lx = nullptr;
      const uint8_t* ly = nullptr;
      auto seek = [&]() {
        if (lt < num_tiles) {
          const TileCoord tc = tile_coord(lt, p);
          lx = p.sfx + static_cast<size_t>(tc.tx * 2 + static_cast<int>(rank)) * p.kblocks * 512 + lane * 16;
          ly = p.sfy + static_cast<size_t>(tc.ty) * p.kblocks * 1024 + lane * 16;
        }
      };
      auto load_next = [&](uint4& a, uint4& b0, uint4& b1) {
        if (lt < num_tiles) {
          a = __ldg(reinterpret_cast<const uint4*>(lx));
          b0 = __ldg(reinterpret_cast<const uint4*>(ly));
          b1 = __ldg(reinterpret_cast<const uint4*>(ly + 512));
          lx += 512;
          ly += 1024;
          if (++lkb == p.kblocks) {
            lkb = 0;
            lt += num_pairs;
            seek();
          }
        }
      };
      uint4 qa[AHEAD], qb0[AHEAD], qb1[AHEAD];
      seek();
#pragma unroll
      for (int j = 0; j < AHEAD; ++j) {
        qa[j] = qb0[j] = qb1[j] = make_uint4(0, 0, 0, 0);
        load_next(qa[j], qb0[j], qb1[j]);
      }
      const int my_tiles = pair < num_tiles ? (num_tiles - pair + num_pairs - 1) / num_pairs : 0;
      const uint32_t total = static_cast<uint32_t>(my_tiles) * static_cast<uint32_t>(p.kblocks);
      uint32_t s = 0;            // ring position of block i (i % STAGES)
      uint32_t es = 1, eph = 0;  // empty barrier of the block that used slot (i + 1) % 4 last, and its phase
      bool ok = true;
#pragma unroll 1
      for (uint32_t i0 = 0; i0 < total && ok; i0 += AHEAD) {
        // Two K blocks (one stage pair) per step: their slots j and j + 1 are 32 adjacent TMEM columns, filled by
        // ONE tcgen05.st (half the store instructions and waits of one store per K block; measured within 1 %).
#pragma unroll
        for (int j = 0; j < AHEAD; j += 2) {
          if (i0 + j < total && ok) {
            if (i0 > 0) {
              // slots j and j + 1 were read last by the MMAs of blocks i - 4 and i - 3
              ok = mbar_wait_warp(bar_empty + 8 * es, eph, abort_flag, p.status, DEV_TIMEOUT_SCALES, lane);
              if (ok) {
                tc_fence_after();
                es += 2;
                if (es >= static_cast<uint32_t>(STAGES)) {
                  es -= STAGES;
                  eph ^= 1;
                }
              }
            }
            if (ok) {
              const bool two = i0 + j + 1 < total;  // false only for the last block of an odd total
              const uint32_t r[32] = {qa[j].x,      qa[j].y,      qa[j].z,      qa[j].w,      qb0[j].x,     qb0[j].y,
                                      qb0[j].z,     qb0[j].w,     qb1[j].x,     qb1[j].y,     qb1[j].z,     qb1[j].w,
                                      0u,           0u,           0u,           0u,           qa[j + 1].x,  qa[j + 1].y,
                                      qa[j + 1].z,  qa[j + 1].w,  qb0[j + 1].x, qb0[j + 1].y, qb0[j + 1].z, qb0[j + 1].w,
                                      qb1[j + 1].x, qb1[j + 1].y, qb1[j + 1].z, qb1[j + 1].w, 0u,           0u,
                                      0u,           0u};
              static_assert(Cfg::sf_col(1) == Cfg::sf_col(0) + 16 && Cfg::sf_col(3) == Cfg::sf_col(2) + 16,
                            "slot pairs are adjacent");
              tmem_st_32x32(tmem_base + lane_addr + Cfg::sf_col(j), r);
              load_next(qa[j], qb0[j], qb1[j]);  // blocks i + 4 and i + 5 into the same registers
              if (two) load_next(qa[j + 1], qb0[j + 1], qb1[j + 1]);
              if (two) {
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster_relaxed(fb0 + 8 * s);
                s += 2;
                if (s >= static_cast<uint32_t>(STAGES)) s -= STAGES;
              } else {
                ++s;
              }
            }
          }
        }
      }
      // an odd total leaves the last stage pair half filled: its arrival is still owed
      if (ok && (s & 1)) {
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster_relaxed(fb0 + 8 * (s - 1));
      }
    }
  } else {
    if constexpr (Cfg::REG_REALLOC) reg_alloc<232>();
    // ------------------------------- epilogue warps (both CTAs) ------------------------------
    const int e = warp - Cfg::FIRST_EPI_WARP;
    const int quad = warp & 3;
    const int slice = e >> 2;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    float* my_sy = sYs + e * BN;
    uint32_t acc_it = 0;
    uint32_t xphase = 0;
    bool ok = true;
    const float inv_fp8_max = p.out_dtype == DT_E5M2 ? (1.0f / 57344.0f) : (1.0f / 448.0f);
    const int tail_units = (num_tiles - p.tail_first) * p.tail_splits;
    for (int u = pair; u < num_units && ok; u += num_pairs) {
      const PairUnit un = pair_unit(u, p);
      const TileCoord tc = tile_coord(un.t, p);
      const int grp = tile_group<Cfg>(p, tc.tx * 256);
      if (grp < 0) continue;
      const long long sy_goff = Cfg::GENERAL ? grp * p.sy_group_stride : 0;
      const int xrow = tc.tx * 256 + static_cast<int>(rank) * 128 + quad * 32 + lane;
      const int ycol0 = tc.ty * BN + slice * Cfg::COLS_PER_THREAD;
      // K-sliced tiles: this thread's first value in slice unit `slot` of the workspace,
      // [CTA of the pair][slice unit][BN][128] fp32 (column-major inside a unit: coalesced over the rows)
      auto ws_at = [&](int slot) {
        return p.ws_partial +
               ((static_cast<size_t>(rank) * tail_units + slot) * BN + slice * Cfg::COLS_PER_THREAD) * 128 +
               quad * 32 + lane;
      };
      auto finish = [&](float sxv, const float* sy_ptr) -> bool {
        return arrive_and_finish<Cfg>(
            p, p.ws_count + ((static_cast<size_t>(un.tail_tile) * 2 + rank) * 2 + slice) * 4 + quad, p.tail_splits,
            ws_at(un.first_slot), sxv, sy_ptr, xrow, ycol0, lane, quad, inv_fp8_max, sXmax + slice * 256,
            bar_x + 8 * slice, &xphase, abort_flag);
      };
      if constexpr (Cfg::SCALE_MODE == SCALE_PROMOTE) {
        float acc[Cfg::COLS_PER_THREAD];
#pragma unroll
        for (int j = 0; j < Cfg::COLS_PER_THREAD; ++j) acc[j] = 0.f;
        const uint32_t tempty0 = map_to_cta(bar_tempty, 0);
        // partial sum number `it` of this CTA is complete when the commit of its K block arrives on the stage's
        // empty barrier: stage it % STAGES, turn it / STAGES
        auto wait_fn = [&](uint32_t it) {
          return mbar_wait(bar_empty + 8 * (it % STAGES), (it / STAGES) & 1, abort_flag, p.status,
                           DEV_TIMEOUT_EPILOGUE);
        };
        auto peek_fn = [&](uint32_t it) { return mbar_test_wait(bar_empty + 8 * (it % STAGES), (it / STAGES) & 1); };
        auto release_fn = [&](uint32_t b) {
          if (lane == 0) mbar_arrive_cluster(tempty0 + 8 * b);
        };
        const uint32_t ta0 = tmem_base + lane_addr + slice * Cfg::COLS_PER_THREAD;
        if constexpr (Cfg::SINGLE_Y)
          ok = promote_groups_single_y<Cfg>(p, acc, xrow, ycol0, un.kb0 * 128, un.kb1 * 128, lane, ta0, acc_it,
                                            sy_goff, wait_fn, peek_fn, release_fn);
        else
          ok = promote_groups<Cfg>(p, acc, xrow, ycol0, un.kb0 * 128, un.kb1 * 128, e, lane, ta0, acc_it, sYs,
                                   sy_goff, wait_fn, peek_fn, release_fn);
        if (!ok) break;
        if (un.whole) {
          OutputStage<Cfg, SRC_REGS> os{p, acc, 0u, 1.f, nullptr, xrow, ycol0, lane, quad,
                                        p.out_dtype == DT_E5M2, inv_fp8_max, sXmax + slice * 256,
                                        bar_x + 8 * slice, &xphase, abort_flag};
          ok = os.run();
        } else {
          park_from_regs<Cfg>(ws_at(un.slot), acc);
          ok = finish(1.f, nullptr);
        }
        continue;
      }
      float sxv = 1.f;
      const float* sy_ptr = nullptr;
      if constexpr (Cfg::SCALE_MODE == SCALE_EPILOGUE) {
        sxv = xrow < p.rx ? load_scale(p.sx, (xrow / p.gx) * p.sx_rs, p.scale_dtype) : 0.f;
        __syncwarp();
        for (int j = lane; j < Cfg::COLS_PER_THREAD; j += 32) {
          const int y = ycol0 + j;
          my_sy[j] = y < p.ry ? load_scale(p.sy, sy_goff + (y / p.gy) * p.sy_rs, p.scale_dtype) : 0.f;
        }
        __syncwarp();
        sy_ptr = my_sy;
      }
      const uint32_t b = acc_it % NUM_ACC, aph = (acc_it / NUM_ACC) & 1;
      ok = mbar_wait_warp(bar_tfull + 8 * b, aph, abort_flag, p.status, DEV_TIMEOUT_EPILOGUE, lane);
      if (!ok) break;
      tc_fence_after();
      const uint32_t ta = tmem_base + lane_addr + b * Cfg::ACC_STRIDE + slice * Cfg::COLS_PER_THREAD;
      if (un.whole) {
        OutputStage<Cfg, SRC_TMEM> os{p, nullptr, ta, sxv, sy_ptr, xrow, ycol0, lane, quad,
                                      p.out_dtype == DT_E5M2, inv_fp8_max, sXmax + slice * 256,
                                      bar_x + 8 * slice, &xphase, abort_flag};
        ok = os.run();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(bar_tempty + 8 * b, 0));
      } else {
        // raw partial sums of this K slice -> workspace, accumulator back to the MMA thread, then the exchange
        park_from_tmem<Cfg>(ws_at(un.slot), ta);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(bar_tempty + 8 * b, 0));
        ok = finish(sxv, sy_ptr);
      }
      ++acc_it;
    }
  }

  // ------------------------------- teardown ---------------------------------------------------
  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // no CTA leaves while its peer may still signal it or read its shared memory
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

template <class Cfg>
cudaError_t launch_pair_kernel(const LaunchArgs& a) {
  // Per device: opt in to the large dynamic shared memory and ask how many CTA pairs can be resident
  // at once. A cluster must sit inside one GPC, so a GPC with an odd number of SMs leaves one SM
  // without a partner; a persistent grid larger than the resident count would run in two waves.
  static int max_pairs[64] = {};
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (dev >= 64) return cudaErrorInvalidDevice;
  if (max_pairs[dev] == 0) {
    err = cudaFuncSetAttribute(mx_gemm_sm100_pair<Cfg>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               Cfg::SMEM_BYTES);
    if (err != cudaSuccess) return err;
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(2, 1, 1);
    lc.blockDim = dim3(Cfg::THREADS, 1, 1);
    lc.dynamicSmemBytes = Cfg::SMEM_BYTES;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    lc.attrs = &attr;
    lc.numAttrs = 1;
    int n = 0;
    err = cudaOccupancyMaxActiveClusters(&n, mx_gemm_sm100_pair<Cfg>, &lc);
    if (err != cudaSuccess) return err;
    if (n <= 0) return cudaErrorLaunchOutOfResources;
    max_pairs[dev] = n;
  }
  int pairs = a.grid / 2;
  if (pairs > max_pairs[dev]) pairs = max_pairs[dev];
  if (pairs < 1) pairs = 1;
  mx_gemm_sm100_pair<Cfg><<<2 * pairs, Cfg::THREADS, Cfg::SMEM_BYTES, a.stream>>>(a.tm_x, a.tm_y, a.p);
  return cudaGetLastError();
}

// resident CTA pairs of the last configured device query (diagnostics)
}  // namespace mxb
