// Persistent, warp-specialised FP8 micro-scaled GEMM for sm_100a.
//
//   out(x, y) = sum_k X[x, k] * sX[x / gx, k / gk]  *  Y[y, k] * sY[y / gy, k / gk]
//
// X [rx, K] and Y [ry, K] are K-major FP8 matrices. X rides the 128-row M axis of tcgen05.mma, Y the
// N axis (BN columns). The host maps the public operands onto (X, Y) either as (left, right) or,
// for transposed / skinny outputs, as (right, left); the kernel itself is symmetric.
//
// Roles per CTA: warp 0 = TMA producer, warp 1 = MMA issuer (owns TMEM), warps 2.. = epilogue.
// Pipelines: smem ring (full/empty mbarriers) between producer and MMA, TMEM accumulator ring
// (tfull/tempty) between MMA and epilogue, so the epilogue of one tile overlaps the main loop of the
// next one.
//
// This one kernel family replaces the 28 generated Hopper templates of the reference:
//   main loop + producer        mxblas/gemm/generator.py:517-595, 726-860
//   scale promotion (4 flavours) mxblas/gemm/generator.py:633-718, 862-915 and
//                                mxblas/gemm/mainloop_tma_scales_generator.py:321-443
//   bf16/fp16 store             mxblas/gemm/generator.py:938-964
//   group-quant epilogue        mxblas/gemm/generator.py:966-1144, mxblas/include/mxblas/type_traits.cuh:8-33
//   tile scheduler              mxblas/gemm/generator.py:435-483
#pragma once

#include "mxb_ptx.cuh"

namespace mxb {

enum : int { SCALE_EPILOGUE = 0, SCALE_PROMOTE = 1, SCALE_MX = 2 };
enum : int { OUT_HP = 0, OUT_QUANT_Y = 1, OUT_QUANT_X = 2, OUT_QUANT_2D = 3 };
enum : int { DT_FP32 = 0, DT_BF16 = 1, DT_FP16 = 2, DT_E4M3 = 3, DT_E5M2 = 4 };

struct GemmParams {
  int rx, ry, k;             // rows of X, rows of Y, reduction length
  int tiles_x, tiles_y;      // ceil(rx/128), ceil(ry/BN)
  int raster;                // tile-rows per raster group (L2 reuse)
  int kblocks;               // ceil(k/128)
  // input scales
  const void* sx;
  const void* sy;
  int gx, gy, gk;            // rows of X / rows of Y / K elements that share one scale
  long long sx_rs, sx_ks;    // element strides of sX along the row-block and K-block index
  long long sy_rs, sy_ks;
  int scale_dtype;           // DT_FP32 / DT_BF16 / DT_FP16 (inputs scales and output scales)
  // pre-packed UE8M0 scale factors (SCALE_MX only): [row tile][k block of 128][atom][512 bytes]
  const uint8_t* sfx;
  const uint8_t* sfy;
  // output
  void* out;
  long long out_xs, out_ys;  // element strides of out along x and y
  int out_dtype;             // DT_BF16 / DT_FP16 / DT_E4M3 / DT_E5M2
  int vec_ok;                // 16-byte vector stores allowed: 1 = along y (out_ys == 1, rows 16-byte aligned),
                             // 2 = along x (16-bit results with out_xs == 1, y rows 16-byte aligned),
                             // 3 = along x (FP8 codes with out_xs == 1, y rows 16-byte aligned)
  void* oscale;
  long long os_xs, os_ys;    // QUANT_Y: index (x, y/qn); QUANT_X: index (x/qn, y); QUANT_2D: index (x/qx, y/qy)
  int qn;                    // quantisation group length
  int qx, qy;                // OUT_QUANT_2D: a quantisation block is qx rows of X by qy columns of Y
  int pow2_out;              // round output scales up to a power of two
  int fmt_x, fmt_y;          // 0 = e4m3, 1 = e5m2
  // Operand storage: 0 = K-major ([rows, K], unit stride along K: the reference's only form), 1 = row-major
  // along the rows ([K, rows], unit stride along the operand's rows: a column-major `left`, a row-major `right`).
  // The tensor map of such an operand has the rows as its inner dimension and a 128 x 128 box.
  int x_mn, y_mn;
  // Grouped GEMM (one weight matrix per group, rows of X sorted by group): x_group[b] is the group of block b of
  // 2^group_shift rows of X, or -1 for a block to skip; Y is the stack [groups * ry, K] of the groups' matrices,
  // a tile of group g reads Y tile  ty + g * group_tiles_y  (ry is a multiple of the tile width) and the scales
  // of Y that start  g * sy_group_stride  elements further. nullptr: plain GEMM.
  const int* x_group;
  int group_shift, group_tiles_y;
  long long sy_group_stride;
  unsigned int* status;      // device status word (0 = ok)
  const unsigned int* gate;  // optional: run only if *gate == gate_value (device-side dispatch)
  unsigned int gate_value;
  // split-K (skinny problems): each tile's K range is cut into `splits` pieces, partial sums are
  // exchanged through `ws_partial` ([tile][split][128][BN] fp32) and `ws_count` ([tile]).
  int splits;
  float* ws_partial;
  unsigned int* ws_count;
  // CTA-pair kernels: tiles [0, tail_first) are computed whole; each later tile (the incomplete last wave)
  // is cut into tail_splits K slices whose partial sums meet in ws_partial ([CTA of the pair][slice
  // unit][BN][128] fp32), counted in ws_count. `splits` then equals tail_splits.
  int tail_first, tail_splits;
};

__device__ __forceinline__ float load_scale(const void* p, long long idx, int dt) {
  if (dt == DT_FP32) return __ldg(reinterpret_cast<const float*>(p) + idx);
  if (dt == DT_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[idx]);
  return __half2float(reinterpret_cast<const __half*>(p)[idx]);
}

__device__ __forceinline__ void store_scale(void* p, long long idx, int dt, float v) {
  if (dt == DT_FP32) reinterpret_cast<float*>(p)[idx] = v;
  else if (dt == DT_BF16) reinterpret_cast<__nv_bfloat16*>(p)[idx] = __float2bfloat16_rn(v);
  else reinterpret_cast<__half*>(p)[idx] = __float2half_rn(v);
}

// Group scale from the group's absolute maximum, following the reference epilogue
// (mxblas/gemm/generator.py:1009-1083): amax is floored at 1e-10 and multiplied by the fp32
// constant 1/fp8_max. With pow2 the result is rounded up to the next power of two.
__device__ __forceinline__ float group_scale(float amax, float inv_fp8_max, int pow2) {
  float s = fmaxf(amax, 1e-10f) * inv_fp8_max;
  if (pow2) {
    uint32_t b = __float_as_uint(s);
    uint32_t e = b >> 23;
    if (b & 0x7FFFFFu) e += 1;
    s = __uint_as_float(e << 23);
  }
  return s;
}

// TWO_PER_SM_: a 128-wide tile with scales applied in the epilogue as a "light" CTA, two per SM with three
// shared-memory stages each (narrower tiles are light by themselves, see LIGHT below).
// GENERAL_: the instantiation also handles operands stored along their rows (column-major left, row-major
// right) and grouped GEMMs. The plain instantiations compile those paths out: as run-time branches they cost
// the kernels of the reference's own layout 4 % (same-box A/B on B200: 8192^3 per-tensor 364.5 -> 380 us).
// SINGLE_Y_ (promotion only): every thread's column slice lies inside one scale block of Y, and the lean loop
// promote_groups_single_y replaces the general one.
template <int BN_, int SCALE_MODE_, int OUT_MODE_, int EPI_WARPS_, int TWO_PER_SM_ = 0, bool GENERAL_ = false,
          bool SINGLE_Y_ = false>
struct KernelCfg {
  static constexpr bool GENERAL = GENERAL_;
  static constexpr bool SINGLE_Y = SINGLE_Y_;
  static_assert(!SINGLE_Y_ || SCALE_MODE_ == SCALE_PROMOTE, "single-scale twins exist for promotion only");
  static constexpr int BM = 128, BK = 128;
  static constexpr int BN = BN_;
  static constexpr int SCALE_MODE = SCALE_MODE_;
  static constexpr int OUT_MODE = OUT_MODE_;
  static constexpr int EPI_WARPS = EPI_WARPS_;
  // warp 0 = TMA producer, warp 1 = MMA issuer. With eight epilogue warps the two control warps
  // are padded to a full warpgroup so that registers can be moved from it to the epilogue
  // warpgroups (setmaxnreg); a 320-thread CTA would be capped at 168 registers per thread anyway.
  static constexpr bool REG_REALLOC = EPI_WARPS == 8 && SCALE_MODE == SCALE_PROMOTE;
  static constexpr int CTRL_WARPS = REG_REALLOC ? 4 : 2;
  static constexpr int THREADS = (CTRL_WARPS + EPI_WARPS) * 32;
  static constexpr int A_BYTES = BM * BK;
  static constexpr int B_BYTES = BN * BK;
  static constexpr int Y_ATOMS = (BN + 127) / 128;
  static constexpr int SFA_BYTES = SCALE_MODE == SCALE_MX ? 512 : 0;
  static constexpr int SFB_BYTES = SCALE_MODE == SCALE_MX ? 512 * Y_ATOMS : 0;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
  static constexpr int PROMOTE_BATCH = BN <= 128 ? 8 : 4;  // scale groups fetched ahead (SCALE_PROMOTE)
  // per-warp copy of the tile's Y scales; SCALE_PROMOTE keeps PROMOTE_BATCH groups of them
  static constexpr int YS_BYTES = (SCALE_MODE == SCALE_PROMOTE ? PROMOTE_BATCH : 1) * EPI_WARPS * BN * 4 /
                                  (SCALE_MODE == SCALE_PROMOTE ? EPI_WARPS / 4 : 1);
  static constexpr int XMAX_BYTES = 2 * 2 * 4 * 32 * 4; // cross-warp amax exchange: [slice][phase][quad][32]
  static constexpr int BAR_BYTES = 512;
  static constexpr int AUX_BYTES = YS_BYTES + XMAX_BYTES + BAR_BYTES;
  static constexpr int SMEM_LIMIT = 232448;              // 227 KiB
  static constexpr int STAGES_FIT = (SMEM_LIMIT - 1024 - AUX_BYTES) / STAGE_BYTES;
  // even: one full barrier covers a pair of stages (the MMA thread waits once per two stages)
  // Narrow tiles with scales applied in the epilogue (skinny, HBM-bound problems) run TWO CTAs per SM
  // with four stages each: twice as many tiles stream concurrently, which takes the edge off wave
  // quantisation (224 tiles of config 5 no longer need two rounds on 148 SMs). Such a CTA takes
  // only the 128 TMEM columns it needs, so that two fit.
  static constexpr bool LIGHT = (BN <= 64 || (BN == 128 && TWO_PER_SM_ == 1)) && SCALE_MODE == SCALE_EPILOGUE;
  static_assert(TWO_PER_SM_ == 0 || (TWO_PER_SM_ == 1 && LIGHT), "two CTAs per SM: 128-wide tiles with scales applied in the epilogue");
  static constexpr int CTAS_PER_SM = LIGHT ? 2 : 1;
  static constexpr int STAGES = LIGHT ? (BN == 128 ? 3 : 4) : ((STAGES_FIT > 8 ? 8 : STAGES_FIT) & ~1);
  // one full barrier per PAIR of stages (the MMA thread's wait costs it ~200 cycles), where the stage count is
  // even; the three-stage light CTA, bound by HBM and not by MMA issue, has one per stage
  static constexpr bool PAIRED_FULL = (STAGES % 2) == 0;
  static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + AUX_BYTES;
  // TMEM plan (512 columns allocated): accumulator buffers every ACC_STRIDE columns; the MX scale
  // factors live in columns the accumulators leave free.
  static constexpr int ACC_STRIDE = LIGHT ? (BN == 128 ? 128 : 64) : (BN <= 128 ? 128 : 256);
  static constexpr int NUM_ACC = LIGHT ? 2 : (SCALE_MODE == SCALE_MX ? 2 : 512 / ACC_STRIDE);
  static constexpr int TMEM_COLS = LIGHT ? 2 * ACC_STRIDE : 512;
  static constexpr int SFA_COL = BN <= 128 ? 256 : 224;  // MX only (BN <= 128 or BN == 224)
  static constexpr int SFB_COL = SFA_COL + 4;
  static constexpr int SF_SLOT = 16;                     // column distance of the two scale-factor slots
  static constexpr int COL_SPLIT = EPI_WARPS / 4;        // column slices shared among epilogue warps
  static constexpr int COLS_PER_THREAD = BN / COL_SPLIT;
  static constexpr int CHUNKS = COLS_PER_THREAD / 32;
  static_assert(EPI_WARPS == 4 || EPI_WARPS == 8, "4 or 8 epilogue warps");
  static_assert(BN % 32 == 0 && BN >= 32 && BN <= 256, "BN is a multiple of 32 up to 256");
  static_assert(COLS_PER_THREAD % 32 == 0, "each epilogue thread owns whole 32-column chunks");
  static_assert(SCALE_MODE != SCALE_MX || BN <= 128 || BN == 224, "MX TMEM plan");
  static_assert(STAGES >= 2, "at least two smem stages");
  static_assert(LIGHT ? (2 * SMEM_BYTES <= SMEM_LIMIT && 3 * SMEM_BYTES > SMEM_LIMIT) : SMEM_BYTES > 116 * 1024,
                "CTAs per SM are fixed by shared memory: TMEM is allocated for exactly that many");
};

struct TileCoord {
  int tx, ty;
};

// Grouped raster: `raster` tile-rows are walked column by column so that concurrently running
// CTAs share X rows and Y rows in L2.
__device__ __forceinline__ TileCoord tile_coord(int t, const GemmParams& p) {
  const int per_group = p.raster * p.tiles_y;
  const int g = t / per_group;
  const int first = g * p.raster;
  const int gsz = min(p.raster, p.tiles_x - first);
  const int r = t - g * per_group;
  TileCoord c;
  c.tx = first + r % gsz;
  c.ty = r / gsz;
  return c;
}

// Group of the X rows of a tile whose first row is `row0` (grouped GEMM); 0 for a plain GEMM, negative: skip.
template <class Cfg>
__device__ __forceinline__ int tile_group(const GemmParams& p, int row0) {
  if constexpr (!Cfg::GENERAL) return 0;
  return p.x_group != nullptr ? __ldg(p.x_group + (row0 >> p.group_shift)) : 0;
}
template <class Cfg>
__device__ __forceinline__ bool x_by_rows(const GemmParams& p) { return Cfg::GENERAL && p.x_mn != 0; }
template <class Cfg>
__device__ __forceinline__ bool y_by_rows(const GemmParams& p) { return Cfg::GENERAL && p.y_mn != 0; }

// ---------------------------------------------------------------------------------------------
// Output stage: converts one thread's row slice (CHUNKS * 32 consecutive y columns of x row `xrow`)
// and writes it. Values come from registers (`acc`, SCALE_PROMOTE) or from TMEM (everything else),
// in which case the input scales sxv * sy_s[col] are applied here.
// ---------------------------------------------------------------------------------------------
enum : int { SRC_TMEM = 0, SRC_REGS = 1, SRC_WS = 2 };

template <class Cfg, int SRC>
struct OutputStage {
  static constexpr bool FROM_REGS = SRC == SRC_REGS;
  const GemmParams& p;
  const float* acc;        // SRC_REGS: CHUNKS*32 values; SRC_WS: this thread's first partial sum
  uint32_t taddr;          // SRC_TMEM: TMEM address of this thread's first column (lane in bits 31:16)
  float sxv;               // SRC_TMEM / SRC_WS: X scale of this row
  const float* sy_s;       // SRC_TMEM / SRC_WS: smem, Y scales of this thread's columns (nullptr: all 1)
  int xrow, ycol0, lane, quad;
  bool e5m2_out;
  float inv_fp8_max;
  // cross-warp exchange (QUANT_X with groups longer than a warp)
  float* xmax_s;
  uint32_t xbar;
  uint32_t* xphase;
  volatile uint32_t* abort_flag;

  __device__ __forceinline__ void fetch(int c, float (&v)[32]) const {
    if constexpr (FROM_REGS) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = acc[c * 32 + j];
    } else if constexpr (SRC == SRC_WS) {
      // sum the split-K partial tiles in split order (deterministic); layout [split][BN][128]
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = 0.f;
      // (the decode cases, 16-bit results and narrow swapped tiles with quantised results: two slices' loads in
      // flight at a time, one round trip to L2 per pair of slices; the other kernels, short of registers, take one
      // slice at a time)
      constexpr bool DECODE_OUT = Cfg::OUT_MODE == OUT_HP || (Cfg::OUT_MODE == OUT_QUANT_X && Cfg::BN <= 64);
      constexpr int STEP = (Cfg::SCALE_MODE == SCALE_PROMOTE || !DECODE_OUT) ? 1 : 2;
      for (int sp = 0; sp < p.splits; sp += STEP) {
        const float* w = acc + (static_cast<size_t>(sp) * Cfg::BN + c * 32) * 128;
        const bool two = STEP == 2 && sp + 1 < p.splits;
        float t0[32], t1[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) t0[j] = __ldcg(w + j * 128);
        if (two) {
#pragma unroll
          for (int j = 0; j < 32; ++j) t1[j] = __ldcg(w + (Cfg::BN + j) * 128);
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] += t0[j];
        if (two) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] += t1[j];
        }
      }
      if (sy_s != nullptr) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] *= (sxv * sy_s[c * 32 + j]);
      }
    } else {
      uint32_t r[32];
      __syncwarp();
      tmem_ld_32x32(taddr + c * 32, r);
      tmem_ld_wait();
      if (sy_s != nullptr) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * (sxv * sy_s[c * 32 + j]);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
      }
    }
  }

  // Results stored along x (the lanes): a 32 x 32 block of the warp, lane = x, register = y, would go out as
  // 32 two-byte stores per lane (64 contiguous bytes per warp and store; the load/store unit takes 16-bit
  // stores a lane at a time: 10 us for a 128 x 128 tile, measured). Three butterfly steps over lane bits 0..2
  // trade registers for neighbours' values, so that a lane ends up with eight consecutive x (16 bytes) of the
  // four rows y = (lane & 7) + 8 i: four 16-byte stores per lane. All lanes of the warp must call this.
  __device__ __forceinline__ void store_hp_along_x(int c, const float (&v)[32]) const {
    const bool f16 = p.out_dtype == DT_FP16;
    const bool b0 = (lane & 1) != 0, b1 = (lane & 2) != 0, b2 = (lane & 4) != 0;
    uint32_t w1[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      // even lanes collect the even rows of the pair (x, x + 1), odd lanes the odd rows
      const float recv = __shfl_xor_sync(0xffffffffu, b0 ? v[2 * i] : v[2 * i + 1], 1);
      const float lo = b0 ? recv : v[2 * i], hi = b0 ? v[2 * i + 1] : recv;
      w1[i] = f16 ? pack_f16x2(lo, hi) : pack_bf16x2(lo, hi);
    }
    uint32_t w2[8][2];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t recv = __shfl_xor_sync(0xffffffffu, b1 ? w1[2 * i] : w1[2 * i + 1], 2);
      w2[i][0] = b1 ? recv : w1[2 * i];
      w2[i][1] = b1 ? w1[2 * i + 1] : recv;
    }
    const int y0 = ycol0 + c * 32;
    const int xg = xrow & ~7;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t r0 = __shfl_xor_sync(0xffffffffu, b2 ? w2[2 * i][0] : w2[2 * i + 1][0], 4);
      const uint32_t r1 = __shfl_xor_sync(0xffffffffu, b2 ? w2[2 * i][1] : w2[2 * i + 1][1], 4);
      uint4 w;
      w.x = b2 ? r0 : w2[2 * i][0];
      w.y = b2 ? r1 : w2[2 * i][1];
      w.z = b2 ? w2[2 * i + 1][0] : r0;
      w.w = b2 ? w2[2 * i + 1][1] : r1;
      const int y = y0 + 8 * i + (lane & 7);
      if (y < p.ry && xg < p.rx) {
        uint16_t* dst = reinterpret_cast<uint16_t*>(p.out) + static_cast<long long>(y) * p.out_ys + xg;
        if (xg + 8 <= p.rx) {
          *reinterpret_cast<uint4*>(dst) = w;
        } else {
          const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
          for (int t = 0; t < 8; ++t)
            if (xg + t < p.rx) dst[t] = static_cast<uint16_t>(ws[t >> 1] >> (16 * (t & 1)));
        }
      }
    }
  }

  // store 32 consecutive-y values of 16-bit type
  __device__ __forceinline__ void store_hp(int c, const float (&v)[32]) const {
    if constexpr (!FROM_REGS) {  // (the promotion kernels, short of registers, keep their stores as they are)
      if (p.vec_ok == 2) {       // uniform over the grid: no lane leaves before the shuffles
        store_hp_along_x(c, v);
        return;
      }
    }
    const int y0 = ycol0 + c * 32;
    if (xrow >= p.rx || y0 >= p.ry) return;
    const bool f16 = p.out_dtype == DT_FP16;
    if (p.vec_ok == 1 && y0 + 32 <= p.ry) {
      uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.out) + xrow * p.out_xs + y0);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 w;
        if (f16) {
          w.x = pack_f16x2(v[q * 8 + 0], v[q * 8 + 1]);
          w.y = pack_f16x2(v[q * 8 + 2], v[q * 8 + 3]);
          w.z = pack_f16x2(v[q * 8 + 4], v[q * 8 + 5]);
          w.w = pack_f16x2(v[q * 8 + 6], v[q * 8 + 7]);
        } else {
          w.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
          w.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
          w.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
          w.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
        }
        dst[q] = w;
      }
    } else {
      uint16_t* base = reinterpret_cast<uint16_t*>(p.out) + xrow * p.out_xs;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (y0 + j < p.ry) {
          uint16_t bits;
          if (f16) {
            __half h = __float2half_rn(v[j]);
            bits = *reinterpret_cast<uint16_t*>(&h);
          } else {
            __nv_bfloat16 h = __float2bfloat16_rn(v[j]);
            bits = *reinterpret_cast<uint16_t*>(&h);
          }
          base[(y0 + j) * p.out_ys] = bits;
        }
      }
    }
  }

  // FP8 codes stored along x (the lanes), the byte-sized sibling of store_hp_along_x: one-byte stores go through
  // the load/store unit a lane at a time (32 of them per lane and chunk: ~2 us per chunk with four warps,
  // measured). Four butterfly steps over lane bits 0..3, the first two on bytes (prmt), leave a lane with
  // sixteen consecutive x of the two rows y = (lane & 15) + 16 t: two 16-byte stores per lane.
  // w[i] holds the codes of y = 4 i .. 4 i + 3 of this lane's x. All lanes of the warp must call this.
  __device__ __forceinline__ void store_fp8_along_x(int c, const uint32_t (&w)[8]) const {
    const bool b0 = (lane & 1) != 0, b1 = (lane & 2) != 0, b2 = (lane & 4) != 0, b3 = (lane & 8) != 0;
    uint32_t w1[8];  // w1[2 i + h]: x pair (l & ~1), rows 8 i + 4 h + b0 and that + 2
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t ev = __byte_perm(w[2 * i], w[2 * i + 1], 0x6420), od = __byte_perm(w[2 * i], w[2 * i + 1], 0x7531);
      const uint32_t keep = b0 ? od : ev;
      const uint32_t recv = __shfl_xor_sync(0xffffffffu, b0 ? ev : od, 1);
      const uint32_t lo = b0 ? recv : keep, hi = b0 ? keep : recv;
      w1[2 * i] = __byte_perm(lo, hi, 0x5140);
      w1[2 * i + 1] = __byte_perm(lo, hi, 0x7362);
    }
    uint32_t w2[8];  // w2[2 i + h]: four x at (l & ~3), row 8 i + 4 h + 2 b1 + b0
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t lows = __byte_perm(w1[2 * i], w1[2 * i + 1], 0x5410), highs = __byte_perm(w1[2 * i], w1[2 * i + 1], 0x7632);
      const uint32_t keep = b1 ? highs : lows;
      const uint32_t recv = __shfl_xor_sync(0xffffffffu, b1 ? lows : highs, 2);
      const uint32_t lo = b1 ? recv : keep, hi = b1 ? keep : recv;
      w2[2 * i] = __byte_perm(lo, hi, 0x5410);
      w2[2 * i + 1] = __byte_perm(lo, hi, 0x7632);
    }
    uint32_t d3[4][2];  // eight x at (l & ~7), row 8 i + (l & 7)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t keep = b2 ? w2[2 * i + 1] : w2[2 * i];
      const uint32_t recv = __shfl_xor_sync(0xffffffffu, b2 ? w2[2 * i] : w2[2 * i + 1], 4);
      d3[i][0] = b2 ? recv : keep;
      d3[i][1] = b2 ? keep : recv;
    }
    const int y0 = ycol0 + c * 32;
    const int xg = xrow & ~15;
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      const uint32_t k0 = b3 ? d3[2 * t + 1][0] : d3[2 * t][0], k1 = b3 ? d3[2 * t + 1][1] : d3[2 * t][1];
      const uint32_t r0 = __shfl_xor_sync(0xffffffffu, b3 ? d3[2 * t][0] : d3[2 * t + 1][0], 8);
      const uint32_t r1 = __shfl_xor_sync(0xffffffffu, b3 ? d3[2 * t][1] : d3[2 * t + 1][1], 8);
      const uint4 v16 = b3 ? make_uint4(r0, r1, k0, k1) : make_uint4(k0, k1, r0, r1);
      const int y = y0 + 16 * t + (lane & 15);
      if (y < p.ry && xg < p.rx) {
        uint8_t* dst = reinterpret_cast<uint8_t*>(p.out) + static_cast<long long>(y) * p.out_ys + xg;
        if (xg + 16 <= p.rx) {
          *reinterpret_cast<uint4*>(dst) = v16;
        } else {
          const uint32_t ws[4] = {v16.x, v16.y, v16.z, v16.w};
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (xg + i < p.rx) dst[i] = static_cast<uint8_t>(ws[i >> 2] >> (8 * (i & 3)));
        }
      }
    }
  }

  // store 32 consecutive-y fp8 codes; q[j] = v[j] * inv[j] already applied by the caller
  __device__ __forceinline__ void store_fp8(int c, const float (&q)[32]) const {
    const int y0 = ycol0 + c * 32;
    // (only where quantisation groups run along x: a swapped, decode-sized problem; other kernels keep their
    // register budget)
    if constexpr (!FROM_REGS && Cfg::OUT_MODE == OUT_QUANT_X) {
      if (p.vec_ok == 3) {  // uniform over the grid: no lane leaves before the shuffles
        uint32_t wt[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          wt[i] = e5m2_out ? pack_fp8x4<true>(q[4 * i], q[4 * i + 1], q[4 * i + 2], q[4 * i + 3])
                           : pack_fp8x4<false>(q[4 * i], q[4 * i + 1], q[4 * i + 2], q[4 * i + 3]);
        }
        store_fp8_along_x(c, wt);
        return;
      }
    }
    if (xrow >= p.rx || y0 >= p.ry) return;
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      w[i] = e5m2_out ? pack_fp8x4<true>(q[4 * i], q[4 * i + 1], q[4 * i + 2], q[4 * i + 3])
                      : pack_fp8x4<false>(q[4 * i], q[4 * i + 1], q[4 * i + 2], q[4 * i + 3]);
    }
    uint8_t* base = reinterpret_cast<uint8_t*>(p.out) + xrow * p.out_xs;
    if (p.vec_ok == 1 && y0 + 32 <= p.ry) {
      uint4* dst = reinterpret_cast<uint4*>(base + y0);
      dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
      dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (y0 + j < p.ry) base[(y0 + j) * p.out_ys] = static_cast<uint8_t>(w[j >> 2] >> (8 * (j & 3)));
      }
    }
  }

  // ---- quantisation groups run along y: each group lives inside this thread -------------------
  __device__ __forceinline__ void run_quant_y() const {
    const int qn = p.qn;
    if (qn <= 32) {
#pragma unroll
      for (int c = 0; c < Cfg::CHUNKS; ++c) {
        float v[32];
        fetch(c, v);
        float a0 = 0.f, a1 = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          a0 = fmaxf(a0, fabsf(v[j]));
          a1 = fmaxf(a1, fabsf(v[16 + j]));
        }
        if (qn == 32) a0 = a1 = fmaxf(a0, a1);
        const float s0 = group_scale(a0, inv_fp8_max, p.pow2_out);
        const float s1 = group_scale(a1, inv_fp8_max, p.pow2_out);
        const float i0 = 1.0f / s0, i1 = 1.0f / s1;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          v[j] *= i0;
          v[16 + j] *= i1;
        }
        store_fp8(c, v);
        const int y0 = ycol0 + c * 32;
        if (xrow < p.rx && y0 < p.ry) {
          const long long base = xrow * p.os_xs;
          if (qn == 32) {
            store_scale(p.oscale, base + (y0 / 32) * p.os_ys, p.scale_dtype, s0);
          } else {
            store_scale(p.oscale, base + (y0 / 16) * p.os_ys, p.scale_dtype, s0);
            if (y0 + 16 < p.ry) store_scale(p.oscale, base + (y0 / 16 + 1) * p.os_ys, p.scale_dtype, s1);
          }
        }
      }
    } else {
      const int cpg = qn / 32;  // chunks per group: 2 or 4
#pragma unroll
      for (int c0 = 0; c0 < Cfg::CHUNKS; c0 += 4) {
        // amax of each chunk of this block of (up to) four chunks
        float am[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          if (c0 + cc < Cfg::CHUNKS) {
            float v[32];
            fetch(c0 + cc, v);
#pragma unroll
            for (int j = 0; j < 32; ++j) am[cc] = fmaxf(am[cc], fabsf(v[j]));
          }
        }
        if (cpg == 2) {
          am[0] = am[1] = fmaxf(am[0], am[1]);
          am[2] = am[3] = fmaxf(am[2], am[3]);
        } else {
          am[0] = am[1] = am[2] = am[3] = fmaxf(fmaxf(am[0], am[1]), fmaxf(am[2], am[3]));
        }
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          if (c0 + cc < Cfg::CHUNKS) {
            const float s = group_scale(am[cc], inv_fp8_max, p.pow2_out);
            const float inv = 1.0f / s;
            float v[32];
            fetch(c0 + cc, v);
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] *= inv;
            store_fp8(c0 + cc, v);
            const int y0 = ycol0 + (c0 + cc) * 32;
            if ((cc % cpg) == 0 && xrow < p.rx && y0 < p.ry)
              store_scale(p.oscale, xrow * p.os_xs + (y0 / qn) * p.os_ys, p.scale_dtype, s);
          }
        }
      }
    }
  }

  // ---- quantisation groups run along x: a group is qn consecutive lanes (and warps) -----------
  // Per 32-column chunk the warp holds a 32 x 32 block (lane = row). The column maxima over a
  // group of G = min(qn, 32) lanes come from a butterfly that halves the number of live values per
  // step (31 shuffles for G = 32), leaving lane l of a group with the maximum of column l (G = 32)
  // or of columns 2l and 2l+1 (G = 16). That lane alone computes the group's scale and reciprocal,
  // writes the scale, and the reciprocals are handed back with one shuffle per column.
  // Returns false if a cross-warp wait was abandoned.
  template <int G>
  __device__ __forceinline__ bool quant_x_chunk(int c) const {
    constexpr int NV = 32 / G;  // values a lane ends up owning: 1 or 2
    const int qn = p.qn;
    float v[32], a[32];
    fetch(c, v);
#pragma unroll
    for (int j = 0; j < 32; ++j) a[j] = fabsf(v[j]);
    // rows beyond rx hold zeros (TMA zero fill), so they never raise a group's maximum
    int n = 32;
#pragma unroll
    for (int off = G / 2; off >= 1; off >>= 1) {
      n >>= 1;
      const bool hi = (lane & off) != 0;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        if (j < n) {
          const float send = hi ? a[j] : a[j + n];
          const float keep = hi ? a[j + n] : a[j];
          a[j] = fmaxf(keep, __shfl_xor_sync(0xffffffffu, send, off));
        }
      }
    }
    // a[t], t < NV, now holds the maximum of column t + NV * (lane % G) over this lane's group
    if (qn > 32) {
      // groups span two or four warps: exchange the per-warp maxima through shared memory
      const uint32_t ph = *xphase;
      float* slot = xmax_s + (ph & 1) * 128;
      slot[quad * 32 + lane] = a[0];
      __syncwarp();
      if (lane == 0) mbar_arrive(xbar);
      if (!mbar_wait(xbar, ph & 1, abort_flag, p.status, DEV_TIMEOUT_EPILOGUE)) return false;
      *xphase = ph + 1;
      const int qbase = qn == 64 ? (quad & 2) : 0;
      const int qcnt = qn == 64 ? 2 : 4;
      float m = slot[qbase * 32 + lane];
      for (int t = 1; t < qcnt; ++t) m = fmaxf(m, slot[(qbase + t) * 32 + lane]);
      a[0] = m;
    }
    float inv[NV];
    const bool writer_warp = qn <= 32 || (qn == 64 ? (quad & 1) == 0 : quad == 0);
    const int y0 = ycol0 + c * 32;
    const int xg = xrow - (xrow % qn);  // first row of this lane's group
#pragma unroll
    for (int t = 0; t < NV; ++t) {
      const float sc = group_scale(a[t], inv_fp8_max, p.pow2_out);
      inv[t] = 1.0f / sc;
      const int y = y0 + t + NV * (lane & (G - 1));
      if (writer_warp && xg < p.rx && y < p.ry)
        store_scale(p.oscale, (long long)(xrow / qn) * p.os_xs + (long long)y * p.os_ys, p.scale_dtype, sc);
    }
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      // column j is owned by lane (j / NV) of the group, as its value (j % NV)
      const int src = (lane & ~(G - 1)) | (j / NV);
      v[j] *= __shfl_sync(0xffffffffu, inv[j % NV], src);
    }
    store_fp8(c, v);
    return true;
  }

  __device__ __forceinline__ bool run_quant_x() const {
    if constexpr (FROM_REGS) {
#pragma unroll
      for (int c = 0; c < Cfg::CHUNKS; ++c) {
        const bool ok = p.qn >= 32 ? quant_x_chunk<32>(c) : quant_x_chunk<16>(c);
        if (!ok) return false;
      }
    } else {
#pragma unroll 1
      for (int c = 0; c < Cfg::CHUNKS; ++c) {  // a real loop (instruction cache, see run())
        const bool ok = p.qn >= 32 ? quant_x_chunk<32>(c) : quant_x_chunk<16>(c);
        if (!ok) return false;
      }
    }
    return true;
  }

  // ---- two-dimensional quantisation blocks: qx rows (lanes, then warps) by qy columns (registers) ----------
  // The reference's epilogue refuses them (static_assert(c_q_m == 1), mxblas/gemm/generator.py:971); the
  // arithmetic per block is the one of its [1, QN] groups with the maximum taken over the whole block.
  // Two passes over the thread's row slice: pass 1 leaves the maximum of every 16 columns in a register, the
  // maxima are merged along y up to qy columns and along x over the block's rows (xor butterfly inside the
  // warp, shared memory and a bounded mbarrier wait across the warps of a 64- or 128-row block); pass 2 fetches
  // the values again, scales them and stores codes and scales. Returns false if a cross-warp wait was abandoned.
  template <int SPAN, int NG>
  __device__ __forceinline__ static void merge_y(float (&g)[NG], int qy) {
    if constexpr (NG >= SPAN) {
      if (qy >= 16 * SPAN) {
#pragma unroll
        for (int i = 0; i < NG; i += SPAN) {
          const float m = fmaxf(g[i], g[i + SPAN / 2]);
#pragma unroll
          for (int t = 0; t < SPAN; ++t) g[i + t] = m;
        }
      }
    }
  }

  __device__ __forceinline__ bool run_quant_2d() const {
    constexpr int NG = Cfg::COLS_PER_THREAD / 16;
    const int qx = p.qx, qy = p.qy;
    float g[NG];
#pragma unroll
    for (int c = 0; c < Cfg::CHUNKS; ++c) {
      float v[32];
      fetch(c, v);
      float a0 = 0.f, a1 = 0.f;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        a0 = fmaxf(a0, fabsf(v[j]));
        a1 = fmaxf(a1, fabsf(v[16 + j]));
      }
      g[2 * c] = a0;
      g[2 * c + 1] = a1;
    }
    // along y: every 16-column entry ends up holding the maximum of the qy columns of its block
    merge_y<2>(g, qy);
    merge_y<4>(g, qy);
    merge_y<8>(g, qy);
    // along x inside the warp (rows beyond rx hold zeros and never raise a maximum)
    for (int off = 1; off < 32 && off < qx; off <<= 1) {
#pragma unroll
      for (int i = 0; i < NG; ++i) g[i] = fmaxf(g[i], __shfl_xor_sync(0xffffffffu, g[i], off));
    }
    if (qx > 32) {
      // blocks of 64 or 128 rows span two or four warps: all lanes of a warp now hold the same NG maxima,
      // lane i publishes entry i
      const uint32_t ph = *xphase;
      float* slot = xmax_s + (ph & 1) * 128;
#pragma unroll
      for (int i = 0; i < NG; ++i)
        if (lane == i) slot[quad * 32 + i] = g[i];
      __syncwarp();
      if (lane == 0) mbar_arrive(xbar);
      if (!mbar_wait(xbar, ph & 1, abort_flag, p.status, DEV_TIMEOUT_EPILOGUE)) return false;
      *xphase = ph + 1;
      const int qbase = qx == 64 ? (quad & 2) : 0;
      const int qcnt = qx == 64 ? 2 : 4;
#pragma unroll
      for (int i = 0; i < NG; ++i) {
        float m = slot[qbase * 32 + i];
        for (int t = 1; t < qcnt; ++t) m = fmaxf(m, slot[(qbase + t) * 32 + i]);
        g[i] = m;
      }
    }
    const bool writer = xrow < p.rx && (xrow & (qx - 1)) == 0;
#pragma unroll
    for (int c = 0; c < Cfg::CHUNKS; ++c) {
      const float s0 = group_scale(g[2 * c], inv_fp8_max, p.pow2_out);
      const float s1 = group_scale(g[2 * c + 1], inv_fp8_max, p.pow2_out);
      const float i0 = 1.0f / s0, i1 = 1.0f / s1;
      float v[32];
      fetch(c, v);
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        v[j] *= i0;
        v[16 + j] *= i1;
      }
      store_fp8(c, v);
      const int y0 = ycol0 + c * 32;
      if (writer) {
        const long long base = static_cast<long long>(xrow / qx) * p.os_xs;
        if (y0 < p.ry && (y0 % qy) == 0) store_scale(p.oscale, base + (y0 / qy) * p.os_ys, p.scale_dtype, s0);
        if (qy == 16 && y0 + 16 < p.ry) store_scale(p.oscale, base + (y0 / 16 + 1) * p.os_ys, p.scale_dtype, s1);
      }
    }
    return true;
  }

  __device__ __forceinline__ bool run() const {
    if constexpr (Cfg::OUT_MODE == OUT_QUANT_2D) {
      return run_quant_2d();
    } else if constexpr (Cfg::OUT_MODE == OUT_HP) {
      if constexpr (FROM_REGS) {
#pragma unroll
        for (int c = 0; c < Cfg::CHUNKS; ++c) {
          float v[32];
          fetch(c, v);
          store_hp(c, v);
        }
      } else {
        // a real loop: a CTA with a single tile runs this code once, straight from a cold instruction cache
        // (unrolled four times, the output stage of a 128 x 128 tile took 8 us; measured)
#pragma unroll 1
        for (int c = 0; c < Cfg::CHUNKS; ++c) {
          float v[32];
          fetch(c, v);
          store_hp(c, v);
        }
      }
      return true;
    } else if constexpr (Cfg::OUT_MODE == OUT_QUANT_Y) {
      run_quant_y();
      return true;
    } else {
      return run_quant_x();
    }
  }
};

// ---------------------------------------------------------------------------------------------
// Two-level accumulation, run by every promotion warp for one tile (or one K range of it): the MMA
// warp leaves the partial sum of each scale group in a TMEM buffer; this adds partial * (sX * sY)
// to the warp's running sums in registers (the arithmetic of mxblas/gemm/generator.py:633-718).
//   wait_group(it)   -> lane 0 only: blocks (bounded) until partial sum number `it` is complete
//   peek_group(it)   -> lane 0 only: the same test without blocking
//   release_group(b) -> hands TMEM buffer b back to the MMA warp (called by all lanes, converged)
// ta_base = this thread's TMEM address in buffer 0 (lane quadrant and column slice included).
//
// With two promotion warps per scheduler every dependent instruction of this loop is exposed latency,
// and each warp has to get through every group, so the loop's serial length bounds the kernel as much
// as the arithmetic does: the barrier of the NEXT group is tested right after this group's TMEM buffer
// is handed back (the test's ~200-cycle latency then runs under the FMAs), and the scale addresses
// advance by additions only.
// ---------------------------------------------------------------------------------------------
template <class Cfg, class WaitFn, class PeekFn, class ReleaseFn>
__device__ __forceinline__ bool promote_groups(const GemmParams& p, float (&acc)[Cfg::COLS_PER_THREAD], int xrow,
                                               int ycol0, int kbeg, int kend, int e, int lane, uint32_t ta_base,
                                               uint32_t& acc_it, float* sYs, long long sy_goff, WaitFn wait_group,
                                               PeekFn peek_group, ReleaseFn release_group) {
  bool ok = true;
  const int ngroups = (kend - kbeg + p.gk - 1) / p.gk;
  const int g0 = kbeg / p.gk;
  // groups in the zero-filled K tail have no scale and add nothing
  const int nvalid = min(ngroups, p.k / p.gk - g0);
  const bool y_uniform = (p.gy % 32) == 0;  // one Y scale per 32-column chunk
  constexpr int PB = Cfg::PROMOTE_BATCH;
  const int dt = p.scale_dtype;
  const int esize = dt == DT_FP32 ? 4 : 2;
  auto load_at = [&](const char* q) -> float {
    if (dt == DT_FP32) return __ldg(reinterpret_cast<const float*>(q));
    if (dt == DT_BF16) return __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(q));
    return __half2float(*reinterpret_cast<const __half*>(q));
  };
  // Scales are fetched ahead of their use so that their global-memory latency never sits
  // between two partial sums, and the loop is kept rolled (small code, few registers):
  //  - X scales (one per row and group): two groups ahead, in rotating registers;
  //  - uniform Y scales (same value for the whole warp): lane l fetches group (32*i + l), the
  //    value is broadcast with a shuffle when its group comes up;
  //  - per-column Y scales: PB groups at a time into this warp's shared-memory stage.
  const bool row_ok = xrow < p.rx;
  const long long sx_step = p.sx_ks * esize;
  const char* sx_next = static_cast<const char*>(p.sx) +
                        (row_ok ? ((xrow / p.gx) * p.sx_rs + static_cast<long long>(g0) * p.sx_ks) * esize : 0);
  auto fetch_sx = [&](int gi) -> float {  // called with gi = 0, 1, 2, ... in order
    const float v = (row_ok && gi < nvalid) ? load_at(sx_next) : 0.f;
    sx_next += sx_step;
    return v;
  };
  float sy_lane[Cfg::CHUNKS], sy_lane_nxt[Cfg::CHUNKS];
  auto load_sy_lane = [&](int gb32, float (&dst)[Cfg::CHUNKS]) {
    const int gi = gb32 * 32 + lane;
    const int g = g0 + gi;
#pragma unroll
    for (int c = 0; c < Cfg::CHUNKS; ++c) {
      const int y = ycol0 + c * 32;
      dst[c] = (y < p.ry && gi < nvalid) ? load_scale(p.sy, sy_goff + (y / p.gy) * p.sy_rs + g * p.sy_ks, dt) : 0.f;
    }
  };
  float sx_c = fetch_sx(0), sx_n1 = fetch_sx(1);
#pragma unroll
  for (int c = 0; c < Cfg::CHUNKS; ++c) sy_lane[c] = sy_lane_nxt[c] = 0.f;
  if (y_uniform) load_sy_lane(0, sy_lane);
  float* sy_stage = sYs + e * (PB * Cfg::COLS_PER_THREAD);  // per-column Y scales: [PB][COLS_PER_THREAD]

  // FMA of one 32-column chunk of one group into the running sums
  auto promote_chunk = [&](const uint32_t (&r)[32], int c, int gi, float sxv) {
    if (y_uniform) {
      const float sc = sxv * __shfl_sync(0xffffffffu, sy_lane[c], gi & 31);
#pragma unroll
      for (int i = 0; i < 32; i += 2) fma2(acc[c * 32 + i], acc[c * 32 + i + 1], r[i], r[i + 1], sc, sc);
    } else {
      const float2* syj = reinterpret_cast<const float2*>(sy_stage + (gi % PB) * Cfg::COLS_PER_THREAD + c * 32);
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        const float2 sy2 = syj[i >> 1];
        fma2(acc[c * 32 + i], acc[c * 32 + i + 1], r[i], r[i + 1], sxv * sy2.x, sxv * sy2.y);
      }
    }
  };

  // Per-group scale upkeep, shared by both loop forms below: before group gi's arithmetic the X scale of group
  // gi + 2 is requested and the Y scales are refreshed; after it the X-scale registers rotate.
  float sx_n2 = 0.f;
  auto scales_begin = [&](int gi) {
    sx_n2 = fetch_sx(gi + 2);  // in flight for two groups
    if (y_uniform) {
      if ((gi & 31) == 0 && gi + 32 < ngroups) load_sy_lane(gi / 32 + 1, sy_lane_nxt);
    } else if ((gi % PB) == 0) {
      __syncwarp();
      for (int idx = lane; idx < PB * Cfg::COLS_PER_THREAD; idx += 32) {
        const int j = idx / Cfg::COLS_PER_THREAD, col = idx - j * Cfg::COLS_PER_THREAD;
        const int gj = gi + j, g = g0 + gj, y = ycol0 + col;
        sy_stage[idx] =
            (y < p.ry && gj < nvalid) ? load_scale(p.sy, sy_goff + (y / p.gy) * p.sy_rs + g * p.sy_ks, dt) : 0.f;
      }
      __syncwarp();
    }
  };
  auto scales_end = [&](int gi) {
    if (y_uniform && (gi & 31) == 31) {
#pragma unroll
      for (int c = 0; c < Cfg::CHUNKS; ++c) sy_lane[c] = sy_lane_nxt[c];
    }
    sx_c = sx_n1;
    sx_n1 = sx_n2;
  };

  bool next_ready = false;  // lane 0: the next group's barrier was already seen complete
#pragma unroll 1
  for (int gi = 0; gi < ngroups; ++gi) {
    scales_begin(gi);
    const uint32_t b = acc_it % Cfg::NUM_ACC;
    uint32_t okw = 1u;
    if (lane == 0) okw = (next_ready || wait_group(acc_it)) ? 1u : 0u;
    okw = __shfl_sync(0xffffffffu, okw, 0);
    if (okw == 0u) {
      ok = false;
      break;
    }
    tc_fence_after();
    const uint32_t ta = ta_base + b * Cfg::ACC_STRIDE;
    if constexpr (Cfg::CHUNKS <= 2) {
      // the whole slice fits in registers: read it, hand the TMEM buffer back to the MMA warp at
      // once, then do the arithmetic
      uint32_t r0[32], r1[32];
      __syncwarp();
      tmem_ld_32x32(ta, r0);
      if (Cfg::CHUNKS == 2) tmem_ld_32x32(ta + 32, r1);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      release_group(b);
      if (lane == 0) next_ready = peek_group(acc_it + 1);
      promote_chunk(r0, 0, gi, sx_c);
      if (Cfg::CHUNKS == 2) promote_chunk(r1, Cfg::CHUNKS - 1, gi, sx_c);
    } else {
      // Four chunks through two register buffers: each later chunk's TMEM round trip runs under the
      // arithmetic of the chunk before it, and the buffer goes back to the MMA warp as soon as the last
      // chunk is in registers.
      static_assert(Cfg::CHUNKS == 4, "promotion slices are 32, 64 or 128 columns wide");
      uint32_t r0[32], r1[32];
      __syncwarp();
      tmem_ld_32x32(ta, r0);
      tmem_ld_32x32(ta + 32, r1);
      tmem_ld_wait();
      promote_chunk(r0, 0, gi, sx_c);
      __syncwarp();
      tmem_ld_32x32(ta + 64, r0);
      promote_chunk(r1, 1, gi, sx_c);
      tmem_ld_wait();
      __syncwarp();
      tmem_ld_32x32(ta + 96, r1);
      promote_chunk(r0, 2, gi, sx_c);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      release_group(b);
      if (lane == 0) next_ready = peek_group(acc_it + 1);
      promote_chunk(r1, 3, gi, sx_c);
    }
    ++acc_it;
    scales_end(gi);
  }
  return ok;
}

// The same loop for the common case that ONE Y scale covers a thread's whole column slice (128 x 128 weight
// blocks under 128- or 64-column slices): no per-lane scale batches and shuffles, no shared-memory stage, one
// scale product per group. It exists as instantiations of its own (Cfg::SINGLE_Y), never beside the general
// loop in one kernel: the promotion warps sit at their register limit, this loop reacts to register pressure
// out of proportion, and what counts is the larger of the two. Measured on B200 (4096 x 7168 x 7168, 1x128 .
// 128x128 scales, CTA pairs): 313 us with the general loop, 452 us with both loops in the kernel and this one
// taken, 257 us with this loop alone.
template <class Cfg, class WaitFn, class PeekFn, class ReleaseFn>
__device__ __forceinline__ bool promote_groups_single_y(const GemmParams& p, float (&acc)[Cfg::COLS_PER_THREAD],
                                                        int xrow, int ycol0, int kbeg, int kend, int lane,
                                                        uint32_t ta_base, uint32_t& acc_it, long long sy_goff,
                                                        WaitFn wait_group, PeekFn peek_group, ReleaseFn release_group) {
  bool ok = true;
  const int ngroups = (kend - kbeg + p.gk - 1) / p.gk;
  const int g0 = kbeg / p.gk;
  const int nvalid = min(ngroups, p.k / p.gk - g0);
  const int dt = p.scale_dtype;
  // (32-bit element indices: a scale tensor has far fewer than 2^31 elements, and every register counts here)
  const int sx_row = static_cast<int>((xrow < p.rx ? (xrow / p.gx) * p.sx_rs : 0) + static_cast<long long>(g0) * p.sx_ks);
  const int sy_row = static_cast<int>(sy_goff + (ycol0 < p.ry ? (ycol0 / p.gy) * p.sy_rs : 0) + static_cast<long long>(g0) * p.sy_ks);
  const int sx_ks = static_cast<int>(p.sx_ks), sy_ks = static_cast<int>(p.sy_ks);
  const int last = nvalid - 1;
  auto fetch = [&](int gi, float& sx, float& sy) {
    const int g = min(gi, last);
    sx = load_scale(p.sx, sx_row + g * sx_ks, dt);
    sy = load_scale(p.sy, sy_row + g * sy_ks, dt);
  };
  float sx0, sy0, sx1, sy1, sx2 = 0.f, sy2 = 0.f;
  fetch(0, sx0, sy0);
  fetch(1, sx1, sy1);
  bool next_ready = false;
#pragma unroll 1
  for (int gi = 0; gi < ngroups; ++gi) {
    fetch(gi + 2, sx2, sy2);
    const uint32_t b = acc_it % Cfg::NUM_ACC;
    uint32_t okw = 1u;
    if (lane == 0) okw = (next_ready || wait_group(acc_it)) ? 1u : 0u;
    okw = __shfl_sync(0xffffffffu, okw, 0);
    if (okw == 0u) {
      ok = false;
      break;
    }
    tc_fence_after();
    const uint32_t ta = ta_base + b * Cfg::ACC_STRIDE;
    const float sc = sx0 * sy0;
    auto chunk = [&](const uint32_t (&r)[32], int c) {
#pragma unroll
      for (int i = 0; i < 32; i += 2) fma2(acc[c * 32 + i], acc[c * 32 + i + 1], r[i], r[i + 1], sc, sc);
    };
    uint32_t r0[32], r1[32];
    __syncwarp();
    tmem_ld_32x32(ta, r0);
    tmem_ld_32x32(ta + 32, r1);
    tmem_ld_wait();
    if constexpr (Cfg::CHUNKS == 2) {
      tc_fence_before();
      __syncwarp();
      release_group(b);
      if (lane == 0) next_ready = peek_group(acc_it + 1);
      chunk(r0, 0);
      chunk(r1, 1);
    } else {
      static_assert(Cfg::CHUNKS == 2 || Cfg::CHUNKS == 4, "single-scale promotion: 64- or 128-column slices");
      chunk(r0, 0);
      __syncwarp();
      tmem_ld_32x32(ta + 64, r0);
      chunk(r1, 1);
      tmem_ld_wait();
      __syncwarp();
      tmem_ld_32x32(ta + 96, r1);
      chunk(r0, 2);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      release_group(b);
      if (lane == 0) next_ready = peek_group(acc_it + 1);
      chunk(r1, 3);
    }
    ++acc_it;
    sx0 = sx1;
    sy0 = sy1;
    sx1 = sx2;
    sy1 = sy2;
  }
  return ok;
}

// ---------------------------------------------------------------------------------------------
// Split-K exchange (1-CTA kernels: every tile cut into `splits` K slices; CTA-pair kernels: the tiles of
// an incomplete last wave). A slice unit parks its partial sums in the workspace as [BN][128] fp32,
// column-major, so that the 32 lanes of a warp (32 consecutive rows) write 128 contiguous bytes per
// column; the slice units of a tile are consecutive. The warp that completes a (tile, row quadrant,
// column slice) last adds the slices in slice order (deterministic), applies scales and stores.
// ---------------------------------------------------------------------------------------------
template <class Cfg>
__device__ __forceinline__ void park_from_tmem(float* wp, uint32_t ta) {
#pragma unroll
  for (int c = 0; c < Cfg::CHUNKS; ++c) {
    uint32_t r[32];
    __syncwarp();
    tmem_ld_32x32(ta + c * 32, r);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 32; ++j) __stcg(wp + (c * 32 + j) * 128, __uint_as_float(r[j]));
  }
}

template <class Cfg>
__device__ __forceinline__ void park_from_regs(float* wp, const float (&acc)[Cfg::COLS_PER_THREAD]) {
#pragma unroll
  for (int j = 0; j < Cfg::COLS_PER_THREAD; ++j) __stcg(wp + j * 128, acc[j]);
}

// Counts this warp's slice in *cnt; the warp that brings it to `parts` resets it (the counters are zero
// between calls) and finishes the tile from the workspace, w0 = this thread's first value in the tile's
// first slice. (sxv, sy_s) are applied to raw partial sums; (1, nullptr) for sums that are already scaled.
template <class Cfg>
__device__ __forceinline__ bool arrive_and_finish(const GemmParams& p, unsigned int* cnt, int parts, const float* w0,
                                                  float sxv, const float* sy_s, int xrow, int ycol0, int lane,
                                                  int quad, float inv_fp8_max, float* xmax_s, uint32_t xbar,
                                                  uint32_t* xphase, volatile uint32_t* abort_flag) {
  __threadfence();
  __syncwarp();
  unsigned int old = 0;
  if (lane == 0) old = atomicAdd(cnt, 1u);
  old = __shfl_sync(0xffffffffu, old, 0);
  if (old != static_cast<unsigned int>(parts - 1)) return true;
  __threadfence();
  if (lane == 0) *cnt = 0;
  OutputStage<Cfg, SRC_WS> os{p,    w0,   0u,   sxv,  sy_s, xrow, ycol0, lane, quad, p.out_dtype == DT_E5M2, inv_fp8_max,
                              xmax_s, xbar, xphase, abort_flag};
  return os.run();
}

// ---------------------------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------------------------
template <class Cfg>
__global__ void __launch_bounds__(Cfg::THREADS, Cfg::CTAS_PER_SM)
mx_gemm_sm100(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_y,
              const __grid_constant__ GemmParams p) {
  constexpr int BN = Cfg::BN;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int NUM_ACC = Cfg::NUM_ACC;

  if (p.gate != nullptr && *p.gate != p.gate_value) return;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = sA + STAGES * Cfg::A_BYTES;
  uint8_t* sSFA = sB + STAGES * Cfg::B_BYTES;
  uint8_t* sSFB = sSFA + STAGES * Cfg::SFA_BYTES;
  uint8_t* aux = sSFB + STAGES * Cfg::SFB_BYTES;
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

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      // paired: covers stages s and s+1 (even s only), one arrival per stage
      mbar_init(bar_full + 8 * s, Cfg::PAIRED_FULL ? 2 : 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < NUM_ACC; ++b) {
      mbar_init(bar_tfull + 8 * b, 1);
      mbar_init(bar_tempty + 8 * b, Cfg::EPI_WARPS);
    }
    mbar_init(bar_x, 4);
    mbar_init(bar_x + 8, 4);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_x);
    tma_prefetch_desc(&tm_y);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_holder), Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  const int num_tiles = p.tiles_x * p.tiles_y;
  const int splits = p.splits;
  const int num_units = num_tiles * splits;
  // K blocks of split `sp`: [kb_lo(sp), kb_lo(sp + 1))
  // 32-bit: kblocks * splits stays far below 2^31, and a 64-bit division costs the producer ~300 cycles per tile
  auto kb_lo = [&](int sp) { return static_cast<int>((static_cast<unsigned>(p.kblocks) * static_cast<unsigned>(sp)) / static_cast<unsigned>(splits)); };

  if (warp < Cfg::CTRL_WARPS) {
  // control warpgroup: give registers away (all of its warps execute this together)
  if constexpr (Cfg::REG_REALLOC) reg_dealloc<40>();
  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------------------
    if (lane == 0) {
      uint32_t s = 0, ph = 0;  // smem stage and its phase bit, advanced without divisions
      bool ok = true;
      for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x) {
        const int t = u / splits, sp = u - t * splits;
        const TileCoord tc = tile_coord(t, p);
        const int grp = tile_group<Cfg>(p, tc.tx * 128);
        if (grp < 0) continue;  // every role skips the same tiles
        const int ty_in = tc.ty + grp * p.group_tiles_y;
        const int kb0 = kb_lo(sp), kb1 = kb_lo(sp + 1);
        for (int kb = kb0; kb < kb1; ++kb) {
          ok = mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, p.status, DEV_TIMEOUT_PRODUCER);
          if (!ok) break;
          const uint32_t fb = bar_full + 8 * (Cfg::PAIRED_FULL ? (s & ~1u) : s);
          mbar_expect_tx(fb, Cfg::STAGE_BYTES);
          if (x_by_rows<Cfg>(p)) tma_load_2d(smem_u32(sA + s * Cfg::A_BYTES), &tm_x, fb, tc.tx * 128, kb * 128);
          else tma_load_2d(smem_u32(sA + s * Cfg::A_BYTES), &tm_x, fb, kb * 128, tc.tx * 128);
          if (y_by_rows<Cfg>(p)) {
            // one 128 x 128 box per 128 rows of Y (the host only plans tile widths of 128 and 256 here)
#pragma unroll
            for (int j = 0; j < Cfg::Y_ATOMS; ++j)
              tma_load_2d(smem_u32(sB + s * Cfg::B_BYTES + j * 16384), &tm_y, fb, ty_in * BN + j * 128, kb * 128);
          } else {
            tma_load_2d(smem_u32(sB + s * Cfg::B_BYTES), &tm_y, fb, kb * 128, ty_in * BN);
          }
          if constexpr (Cfg::SCALE_MODE == SCALE_MX) {
            bulk_load_1d(smem_u32(sSFA + s * Cfg::SFA_BYTES),
                         p.sfx + (static_cast<size_t>(tc.tx) * p.kblocks + kb) * 512, 512, fb);
            bulk_load_1d(smem_u32(sSFB + s * Cfg::SFB_BYTES),
                         p.sfy + (static_cast<size_t>(ty_in) * p.kblocks + kb) * Cfg::SFB_BYTES,
                         Cfg::SFB_BYTES, fb);
          }
          if (++s == STAGES) {
            s = 0;
            ph ^= 1;
          }
        }
      }
      // an odd total leaves the last stage pair half filled: complete it with a plain arrival
      if (Cfg::PAIRED_FULL && ok && (s & 1)) mbar_arrive(bar_full + 8 * (s & ~1u));
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------- MMA issuer ---------------------------------------------
    if (lane == 0) {
      // This one thread feeds the tensor pipe, and it runs its instructions back to back with no
      // other work to hide their latency: everything per MMA is kept to additions and compares
      // (no division or modulo; stage, phase, accumulator and scale-group positions are counters).
      uint32_t s = 0, ph = 0;        // smem stage / phase
      uint32_t b = 0, aph = 0;       // accumulator buffer / phase
      bool ok = true;
      const uint32_t idesc = umma_idesc_major(Cfg::SCALE_MODE == SCALE_MX ? umma_idesc_mxf8(128, BN, p.fmt_x, p.fmt_y)
                                                                          : umma_idesc_f8(128, BN, p.fmt_x, p.fmt_y),
                                              x_by_rows<Cfg>(p), y_by_rows<Cfg>(p));
      // descriptor step from one 32-deep K slice to the next: 32 bytes along a K-major row, four 8-row groups
      // (4096 bytes) in an operand staged as K rows
      const uint32_t kstep_a = x_by_rows<Cfg>(p) ? 256u : 2u, kstep_b = y_by_rows<Cfg>(p) ? 256u : 2u;
      // the descriptors' high words are constants; their low words (address field, 16-byte units) step from stage
      // to stage by one 32-bit addition
      const uint64_t hi_a = umma_desc_hi(x_by_rows<Cfg>(p)), hi_b = umma_desc_hi(y_by_rows<Cfg>(p));
      const uint32_t a_hi = static_cast<uint32_t>(hi_a >> 32), b_hi = static_cast<uint32_t>(hi_b >> 32);
      const uint32_t a_lo0 = static_cast<uint32_t>(hi_a) | ((smem_u32(sA) >> 4) & 0x3FFFu);
      const uint32_t b_lo0 = static_cast<uint32_t>(hi_b) | ((smem_u32(sB) >> 4) & 0x3FFFu);
      constexpr uint32_t A_STEP = Cfg::A_BYTES >> 4, B_STEP = Cfg::B_BYTES >> 4;
      uint32_t a_lo = a_lo0, b_lo = b_lo0;  // of stage s
      // K elements accumulated in TMEM before the epilogue warps take the partial sum
      const int group_k = Cfg::SCALE_MODE == SCALE_PROMOTE ? p.gk : 0;
      for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x) {
        const int t = u / splits, sp = u - t * splits;
        if (Cfg::GENERAL && p.x_group != nullptr && tile_group<Cfg>(p, tile_coord(t, p).tx * 128) < 0) continue;
        const int kb0 = kb_lo(sp), kb1 = kb_lo(sp + 1);
        uint32_t d_tmem = 0;
        if constexpr (Cfg::SCALE_MODE != SCALE_PROMOTE && Cfg::PAIRED_FULL) {
          // One accumulator per unit and one full barrier per stage pair: whole pairs per turn (one wait, eight
          // MMAs, two commits, one wrap test), like the CTA-pair kernel. A unit may begin on the second stage of
          // a pair (the previous unit passed its barrier) and end on the first.
          ok = mbar_wait(bar_tempty + 8 * b, aph ^ 1, abort_flag, p.status, DEV_TIMEOUT_MMA_TMEM);
          if (!ok) break;
          tc_fence_after();
          d_tmem = tmem_base + b * Cfg::ACC_STRIDE;
          auto copy_scale_factors = [&]() {  // block-scaled: the factors of both stages of the pair that starts at s
            if constexpr (Cfg::SCALE_MODE == SCALE_MX) {
#pragma unroll
              for (uint32_t j = 0; j < 2; ++j) {
                const uint32_t sj = s + j;
                tmem_cp_32x128b_warpx4(tmem_base + Cfg::SFA_COL + j * Cfg::SF_SLOT,
                                       umma_desc_rows16(smem_u32(sSFA + sj * Cfg::SFA_BYTES)));
#pragma unroll
                for (int a = 0; a < Cfg::Y_ATOMS; ++a)
                  tmem_cp_32x128b_warpx4(tmem_base + Cfg::SFB_COL + j * Cfg::SF_SLOT + 4 * a,
                                         umma_desc_rows16(smem_u32(sSFB + sj * Cfg::SFB_BYTES + a * 512)));
              }
            }
          };
          auto issue_stage = [&](uint32_t accumulate) {
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              const uint64_t da = umma_desc_words(a_lo + kk * kstep_a, a_hi), db = umma_desc_words(b_lo + kk * kstep_b, b_hi);
              if constexpr (Cfg::SCALE_MODE == SCALE_MX) {
                umma_mxf8(d_tmem, da, db, umma_idesc_sf_ids(idesc, kk, kk), kk == 0 ? accumulate : 1u,
                          tmem_base + Cfg::SFA_COL + (s & 1) * Cfg::SF_SLOT, tmem_base + Cfg::SFB_COL + (s & 1) * Cfg::SF_SLOT);
              } else if (kk == 0) {
                umma_f8(d_tmem, da, db, idesc, accumulate);
              } else {
                umma_f8_acc(d_tmem, da, db, idesc);
              }
            }
            umma_commit(bar_empty + 8 * s);
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
          int kb = kb0;
          uint32_t accumulate = 0;
          if ((s & 1) != 0 && kb < kb1) {
            issue_stage(accumulate);
            accumulate = 1;
            wrap_ring();
            ++kb;
          }
          for (; kb + 2 <= kb1; kb += 2) {
            ok = mbar_wait(bar_full + 8 * s, ph, abort_flag, p.status, DEV_TIMEOUT_MMA_FULL);
            if (!ok) break;
            tc_fence_after();
            copy_scale_factors();
            issue_stage(accumulate);
            accumulate = 1;
            issue_stage(1u);
            wrap_ring();
          }
          if (ok && kb < kb1) {
            ok = mbar_wait(bar_full + 8 * s, ph, abort_flag, p.status, DEV_TIMEOUT_MMA_FULL);
            if (ok) {
              tc_fence_after();
              copy_scale_factors();
              issue_stage(accumulate);
            }
          }
          if (!ok) break;
          umma_commit(bar_tfull + 8 * b);
          if (++b == NUM_ACC) {
            b = 0;
            aph ^= 1;
          }
          continue;
        }
        int gpos = 0;       // K elements already in the open scale group (split ranges start on a group)
        bool open = false;  // an accumulator buffer is currently being filled
        for (int kb = kb0; kb < kb1 && ok; ++kb) {
          if (!Cfg::PAIRED_FULL || (s & 1) == 0) {  // paired: both stages have landed once this barrier completes
            ok = mbar_wait(bar_full + 8 * s, ph, abort_flag, p.status, DEV_TIMEOUT_MMA_FULL);
            if (!ok) break;
            tc_fence_after();
          }
          if constexpr (Cfg::SCALE_MODE == SCALE_MX) {
            // Scale factors of BOTH stages of the pair go to TMEM now (two column slots), so that
            // the copy for the second stage runs under the first stage's MMAs instead of in front of
            // its own. tcgen05.cp and tcgen05.mma of one thread execute in issue order, which also
            // protects a slot from being overwritten before the MMAs that read it.
            if ((s & 1) == 0) {
#pragma unroll
              for (uint32_t j = 0; j < 2; ++j) {
                const uint32_t sj = s + j;
                tmem_cp_32x128b_warpx4(tmem_base + Cfg::SFA_COL + j * Cfg::SF_SLOT,
                                       umma_desc_rows16(smem_u32(sSFA + sj * Cfg::SFA_BYTES)));
#pragma unroll
                for (int a = 0; a < Cfg::Y_ATOMS; ++a)
                  tmem_cp_32x128b_warpx4(tmem_base + Cfg::SFB_COL + j * Cfg::SF_SLOT + 4 * a,
                                         umma_desc_rows16(smem_u32(sSFB + sj * Cfg::SFB_BYTES + a * 512)));
              }
            }
          }
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            bool fresh = false;
            if (!open) {
              ok = mbar_wait(bar_tempty + 8 * b, aph ^ 1, abort_flag, p.status, DEV_TIMEOUT_MMA_TMEM);
              if (!ok) break;
              tc_fence_after();
              d_tmem = tmem_base + b * Cfg::ACC_STRIDE;
              open = true;
              fresh = true;
            }
            const uint64_t da = umma_desc_words(a_lo + kk * kstep_a, a_hi), db = umma_desc_words(b_lo + kk * kstep_b, b_hi);
            if constexpr (Cfg::SCALE_MODE == SCALE_MX) {
              umma_mxf8(d_tmem, da, db, umma_idesc_sf_ids(idesc, kk, kk), fresh ? 0u : 1u,
                        tmem_base + Cfg::SFA_COL + (s & 1) * Cfg::SF_SLOT,
                        tmem_base + Cfg::SFB_COL + (s & 1) * Cfg::SF_SLOT);
            } else if (Cfg::SCALE_MODE == SCALE_EPILOGUE && kk != 0) {
              umma_f8_acc(d_tmem, da, db, idesc);  // an accumulator only opens on the first K slice of a K block
            } else {
              umma_f8(d_tmem, da, db, idesc, fresh ? 0u : 1u);
            }
            // close the accumulator at a scale-group boundary (promotion) or at the end of the range
            gpos += 32;
            const bool last = (kb == kb1 - 1) && (kk == 3);
            const bool boundary = group_k > 0 && gpos == group_k;
            if (last || boundary) {
              umma_commit(bar_tfull + 8 * b);
              if (++b == NUM_ACC) {
                b = 0;
                aph ^= 1;
              }
              open = false;
              gpos = 0;
            }
          }
          if (!ok) break;
          umma_commit(bar_empty + 8 * s);
          a_lo += A_STEP;
          b_lo += B_STEP;
          if (++s == STAGES) {
            s = 0;
            ph ^= 1;
            a_lo = a_lo0;
            b_lo = b_lo0;
          }
        }
      }
    }
    __syncwarp();
  }
  } else {
    if constexpr (Cfg::REG_REALLOC) reg_alloc<232>();
    // ------------------------------- epilogue warps -----------------------------------------
    const int e = warp - Cfg::CTRL_WARPS;
    const int quad = warp & 3;              // TMEM lane quadrant this warp may read
    const int slice = e >> 2;               // column slice (0 when there are 4 epilogue warps)
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    float* my_sy = sYs + e * BN;
    uint32_t acc_it = 0;
    uint32_t xphase = 0;
    bool ok = true;
    const float inv_fp8_max = p.out_dtype == DT_E5M2 ? (1.0f / 57344.0f) : (1.0f / 448.0f);

    for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x) {
      const int t = u / splits, sp = u - t * splits;
      const TileCoord tc = tile_coord(t, p);
      const int grp = tile_group<Cfg>(p, tc.tx * 128);
      if (grp < 0) continue;
      const long long sy_goff = Cfg::GENERAL ? grp * p.sy_group_stride : 0;
      const int xrow = tc.tx * 128 + quad * 32 + lane;
      const int ycol0 = tc.ty * BN + slice * Cfg::COLS_PER_THREAD;
      const int kb0 = kb_lo(sp), kb1 = kb_lo(sp + 1);
      (void)kb0;
      (void)kb1;

      if constexpr (Cfg::SCALE_MODE == SCALE_PROMOTE) {
        // -------- two-level accumulation: TMEM partial sums are scaled and added in registers ---
        float acc[Cfg::COLS_PER_THREAD];
#pragma unroll
        for (int j = 0; j < Cfg::COLS_PER_THREAD; ++j) acc[j] = 0.f;
        // K range padded to whole blocks: the MMA warp closes a buffer per group
        auto wait_fn = [&](uint32_t it) {
          return mbar_wait(bar_tfull + 8 * (it % NUM_ACC), (it / NUM_ACC) & 1, abort_flag, p.status,
                           DEV_TIMEOUT_EPILOGUE);
        };
        auto peek_fn = [&](uint32_t it) { return mbar_test_wait(bar_tfull + 8 * (it % NUM_ACC), (it / NUM_ACC) & 1); };
        auto release_fn = [&](uint32_t b) {
          if (lane == 0) mbar_arrive(bar_tempty + 8 * b);
        };
        const uint32_t ta0 = tmem_base + lane_addr + slice * Cfg::COLS_PER_THREAD;
        if constexpr (Cfg::SINGLE_Y)
          ok = promote_groups_single_y<Cfg>(p, acc, xrow, ycol0, kb0 * 128, kb1 * 128, lane, ta0, acc_it, sy_goff,
                                            wait_fn, peek_fn, release_fn);
        else
          ok = promote_groups<Cfg>(p, acc, xrow, ycol0, kb0 * 128, kb1 * 128, e, lane, ta0, acc_it, sYs, sy_goff,
                                   wait_fn, peek_fn, release_fn);
        if (!ok) break;
        if (splits == 1) {
          OutputStage<Cfg, SRC_REGS> os{p, acc, 0u, 1.f, nullptr, xrow, ycol0, lane, quad,
                                        p.out_dtype == DT_E5M2, inv_fp8_max, sXmax + slice * 256,
                                        bar_x + 8 * slice, &xphase, abort_flag};
          ok = os.run();
        } else {
          // split-K: this unit's scaled sums go to the workspace; the last slice's warp finishes the tile
          float* ws0 = p.ws_partial + (slice * Cfg::COLS_PER_THREAD) * 128 + quad * 32 + lane;
          park_from_regs<Cfg>(ws0 + static_cast<size_t>(u) * BN * 128, acc);
          ok = arrive_and_finish<Cfg>(p, p.ws_count + (static_cast<size_t>(t) * 2 + slice) * 4 + quad, splits,
                                      ws0 + static_cast<size_t>(t) * splits * BN * 128, 1.f, nullptr, xrow, ycol0,
                                      lane, quad, inv_fp8_max, sXmax + slice * 256, bar_x + 8 * slice, &xphase,
                                      abort_flag);
        }
      } else {
        // -------- scales applied once, on the TMEM -> register path ----------------------------
        float sxv = 1.f;
        const float* sy_ptr = nullptr;
        if constexpr (Cfg::SCALE_MODE == SCALE_EPILOGUE) {
          sxv = xrow < p.rx ? load_scale(p.sx, (xrow / p.gx) * p.sx_rs, p.scale_dtype) : 0.f;
          __syncwarp();  // the previous tile's readers of my_sy are done
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
        if (splits == 1) {
          OutputStage<Cfg, SRC_TMEM> os{p, nullptr, ta, sxv, sy_ptr, xrow, ycol0, lane, quad,
                                        p.out_dtype == DT_E5M2, inv_fp8_max, sXmax + slice * 256,
                                        bar_x + 8 * slice, &xphase, abort_flag};
          ok = os.run();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_tempty + 8 * b);
        } else {
          // split-K: raw partial sums to the workspace, accumulator back to the MMA warp, then the exchange
          float* ws0 = p.ws_partial + (slice * Cfg::COLS_PER_THREAD) * 128 + quad * 32 + lane;
          park_from_tmem<Cfg>(ws0 + static_cast<size_t>(u) * BN * 128, ta);
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_tempty + 8 * b);
          ok = arrive_and_finish<Cfg>(p, p.ws_count + (static_cast<size_t>(t) * 2 + slice) * 4 + quad, splits,
                                      ws0 + static_cast<size_t>(t) * splits * BN * 128, sxv, sy_ptr, xrow, ycol0, lane,
                                      quad, inv_fp8_max, sXmax + slice * 256, bar_x + 8 * slice, &xphase, abort_flag);
        }
        ++acc_it;
      }
    }
  }

  // ------------------------------- teardown ---------------------------------------------------
  if (*abort_flag) {
    // a wait was abandoned: give copies and MMAs still in flight time to land before smem/TMEM go away
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace mxb
