// Device-side block quantiser: x [M, K] (fp32 / bf16 / fp16) -> e4m3 codes + fp32 scales per
// (bm x bn) block. The step in front of the GEMM, so that activations never leave the GPU to be
// quantised. Follows the reference's host helper block_quant (mxblas/utils.py:66-93) operation by
// operation, including its arithmetic type: torch evaluates amax / 448 and x / scale in the
// tensor's own dtype (computed in fp32, rounded to the dtype after each operation), an all-zero
// block gets scale 1, values are clamped to +-448 before the cast.
//
// HBM-bound: reads sizeof(x) * M * K, writes M * K + 4 * M*K / (bm*bn) bytes.
//   row blocks (bm == 1): one 16-byte vector per lane, amax by shuffles over the lanes of a block; blocks
//                         longer than a warp's 32 vectors take one warp and two passes
//   2-D blocks (any size, up to per-tensor): cut into slabs of ~32K elements, per-CTA partial maxima
//                         merged with one atomicMax each, then a second kernel quantises
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/mxblas_b200.h"

namespace {

template <int DT>
__device__ __forceinline__ float load_elem(const void* p, long long i) {
  if (DT == MXB_FP32) return reinterpret_cast<const float*>(p)[i];
  if (DT == MXB_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(reinterpret_cast<const __half*>(p)[i]);
}
// round an fp32 intermediate to the tensor's dtype, as torch does after every elementwise op
template <int DT>
__device__ __forceinline__ float round_dt(float v) {
  if (DT == MXB_FP32) return v;
  if (DT == MXB_BF16) return __bfloat162float(__float2bfloat16_rn(v));
  return __half2float(__float2half_rn(v));
}
template <int DT>
__device__ __forceinline__ float block_scale(float amax) {
  float s = round_dt<DT>(amax / 448.0f);
  return s == 0.0f ? 1.0f : s;
}
template <int DT>
__device__ __forceinline__ uint8_t quant_elem(float x, float scale) {
  float q = round_dt<DT>(x / scale);
  q = fminf(fmaxf(q, -448.0f), 448.0f);
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(q, __NV_SATFINITE, __NV_E4M3));
}
// The same values without a division per element, for 16-bit inputs: with r = 1 / scale (one division per block),
// q0 = x * r and q1 = fma(fma(-q0, scale, x), r, q0), the quotient rounded to the tensor's dtype equals
// RN_dt(x / scale) for EVERY 16-bit x and EVERY 16-bit scale in [1e-30, 1e30] with |x| <= 1024 * scale (the
// quantiser only divides |x| <= amax ~ 448 * scale): checked exhaustively on the GPU, 0.89 G bf16 pairs and
// 1.55 G fp16 pairs, no difference (signs of zeros included). Outside that range of scales, and for fp32 inputs,
// the division stays.
// Two elements at a time: one conversion to the 16-bit type and one to FP8 per pair.
template <int DT>
__device__ __forceinline__ bool reciprocal_is_exact(float scale) {
  return DT != MXB_FP32 && scale >= 1e-30f && scale <= 1e30f;
}
template <int DT>
__device__ __forceinline__ uint32_t quant_pair_recip(float x0, float x1, float scale, float r) {
  const float p0 = x0 * r, p1 = x1 * r;
  // (a zero keeps its sign: the correction step would turn -0 into +0, and FP8 has both)
  float q0 = p0 == 0.f ? p0 : fmaf(fmaf(-p0, scale, x0), r, p0), q1 = p1 == 0.f ? p1 : fmaf(fmaf(-p1, scale, x1), r, p1);
  if (DT == MXB_BF16) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(q0, q1);
    const uint32_t bits = *reinterpret_cast<const uint32_t*>(&h);
    q0 = __uint_as_float(bits << 16);
    q1 = __uint_as_float(bits & 0xFFFF0000u);
  } else {
    const __half2 h = __floats2half2_rn(q0, q1);
    q0 = __low2float(h);
    q1 = __high2float(h);
  }
  q0 = fminf(fmaxf(q0, -448.0f), 448.0f);
  q1 = fminf(fmaxf(q1, -448.0f), 448.0f);
  return static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(q0, q1), __NV_SATFINITE, __NV_E4M3));  // x in the low byte
}

// 16-byte vector of the input type: VEC elements
template <int DT> struct Vec { static constexpr int N = DT == MXB_FP32 ? 4 : 8; };

template <int DT>
__device__ __forceinline__ void load_vec(const void* x, long long i, float (&v)[Vec<DT>::N]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(static_cast<const char*>(x) + i * (DT == MXB_FP32 ? 4 : 2));
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  if (DT == MXB_FP32) {
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = __uint_as_float(w[j]);
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (DT == MXB_BF16) {
        v[2 * j] = __uint_as_float(w[j] << 16);
        v[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
      } else {
        const __half2 h = *reinterpret_cast<const __half2*>(&w[j]);
        v[2 * j] = __low2float(h);
        v[2 * j + 1] = __high2float(h);
      }
    }
  }
}
template <int DT>
__device__ __forceinline__ void store_codes(uint8_t* dst, const float (&v)[Vec<DT>::N], float s) {
  uint32_t w[2] = {0, 0};
  if (reciprocal_is_exact<DT>(s)) {
    const float r = 1.0f / s;
#pragma unroll
    for (int j = 0; j < Vec<DT>::N; j += 2) w[j >> 2] |= quant_pair_recip<DT>(v[j], v[j + 1], s, r) << (8 * (j & 3));
  } else {
#pragma unroll
    for (int j = 0; j < Vec<DT>::N; ++j) w[j >> 2] |= static_cast<uint32_t>(quant_elem<DT>(v[j], s)) << (8 * (j & 3));
  }
  if (Vec<DT>::N == 8) *reinterpret_cast<uint2*>(dst) = make_uint2(w[0], w[1]);
  else *reinterpret_cast<uint32_t*>(dst) = w[0];
}

// ---- row blocks, vectorised: a block of bn elements is shared by bn/VEC consecutive lanes (<= 32) --
// Each lane owns one 16-byte vector; the amax is reduced over the lanes of the block with xor
// shuffles. Needs bn % VEC == 0, bn / VEC a power of two <= 32, 16-byte aligned rows.
template <int DT>
__global__ void quant_rows_vec(const void* x, long long m, long long k, long long ldx, int bn, uint8_t* codes,
                               long long ldq, float* scales) {
  constexpr int V = Vec<DT>::N;
  const long long vecs_per_row = k / V;
  const long long total = m * vecs_per_row;
  const int lanes = bn / V;
  const long long nblk = k / bn;
  // (row, column vector) of a thread's element advance by a fixed step: one 64-bit division per thread, none per
  // vector. (Two or four vectors per thread and turn, their loads issued together, measured 15-30 % slower:
  // the kernel is not waiting on a single load.)
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long step_rows = stride / vecs_per_row, step_cv = stride - step_rows * vecs_per_row;
  long long i0 = (blockIdx.x * static_cast<long long>(blockDim.x)) + threadIdx.x;
  long long row0 = i0 / vecs_per_row, cv0 = i0 - row0 * vecs_per_row;
  for (; i0 - (threadIdx.x & 31) < total; i0 += stride, row0 += step_rows, cv0 += step_cv) {
    if (cv0 >= vecs_per_row) {
      cv0 -= vecs_per_row;
      ++row0;
    }
    const bool live = i0 < total;
    const long long row = live ? row0 : m - 1, cv = live ? cv0 : vecs_per_row - 1;
    float v[V];
    load_vec<DT>(x, row * ldx + cv * V, v);
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < V; ++j) amax = fmaxf(amax, fabsf(v[j]));
    for (int off = 1; off < lanes; off <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    const float s = block_scale<DT>(amax);
    if (live) {
      store_codes<DT>(codes + row * ldq + cv * V, v, s);
      if ((cv % lanes) == 0) scales[row * nblk + (cv * V) / bn] = s;
    }
  }
}

// ---- long row blocks (bn > 32 vectors): one warp per block, two passes (second one hits L2) -------
template <int DT>
__global__ void quant_rows_long(const void* x, long long m, long long k, long long ldx, int bn, uint8_t* codes,
                                long long ldq, float* scales) {
  constexpr int V = Vec<DT>::N;
  const long long nblk = k / bn;
  const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= m * nblk) return;
  const long long row = warp / nblk, blk = warp - row * nblk;
  const long long base = row * ldx + blk * bn;
  float amax = 0.f;
  for (int j = lane * V; j < bn; j += 32 * V) {
    float v[V];
    load_vec<DT>(x, base + j, v);
#pragma unroll
    for (int t = 0; t < V; ++t) amax = fmaxf(amax, fabsf(v[t]));
  }
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  const float s = block_scale<DT>(amax);
  if (lane == 0) scales[row * nblk + blk] = s;
  uint8_t* out = codes + row * ldq + blk * bn;
  for (int j = lane * V; j < bn; j += 32 * V) {
    float v[V];
    load_vec<DT>(x, base + j, v);
    store_codes<DT>(out + j, v, s);
  }
}

// ---- generic fallback: one warp per (row, block), scalar accesses ---------------------------------
template <int DT>
__global__ void quant_rows(const void* x, long long m, long long k, long long ldx, int bn, uint8_t* codes,
                           long long ldq, float* scales) {
  const long long nblk = k / bn;
  const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= m * nblk) return;
  const long long row = warp / nblk, blk = warp - row * nblk;
  const long long base = row * ldx + blk * bn;
  float amax = 0.f;
  for (int j = lane; j < bn; j += 32) amax = fmaxf(amax, fabsf(load_elem<DT>(x, base + j)));
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  const float s = block_scale<DT>(amax);
  if (lane == 0) scales[row * nblk + blk] = s;
  uint8_t* out = codes + row * ldq + blk * bn;
  for (int j = lane; j < bn; j += 32) out[j] = quant_elem<DT>(load_elem<DT>(x, base + j), s);
}

// ---- 2-D blocks cut into slabs of rows: partial maxima merged with one atomicMax per CTA (the
// float bits of non-negative values order like unsigned integers), then a second kernel quantises.
// `scales` holds the amax bits between the two kernels. `vec` selects 16-byte accesses.
template <int DT>
__global__ void amax_slabs(const void* x, long long k, long long ldx, int bm, int bn, int slab_rows, int slabs,
                           int vec, unsigned int* amax_bits) {
  __shared__ float red[32];
  constexpr int V = Vec<DT>::N;
  const long long nblk_k = k / bn;
  const long long blk = blockIdx.x / slabs;
  const int slab = blockIdx.x - blk * slabs;
  const long long bi = blk / nblk_k, bj = blk - bi * nblk_k;
  const int r_lo = slab * slab_rows, r_hi = min(bm, r_lo + slab_rows);
  const long long r0 = bi * bm, c0 = bj * bn;
  float amax = 0.f;
  if (vec) {
    const int vpr = bn / V;
    const int nvec = (r_hi - r_lo) * vpr;  // a slab holds ~32K elements: 32-bit indices
    for (int e = threadIdx.x; e < nvec; e += blockDim.x) {
      const int rr = e / vpr;
      const int r = r_lo + rr, c = (e - rr * vpr) * V;
      float v[V];
      load_vec<DT>(x, (r0 + r) * ldx + c0 + c, v);
#pragma unroll
      for (int t = 0; t < V; ++t) amax = fmaxf(amax, fabsf(v[t]));
    }
  } else {
    for (long long e = threadIdx.x; e < static_cast<long long>(r_hi - r_lo) * bn; e += blockDim.x) {
      const int r = r_lo + static_cast<int>(e / bn), c = static_cast<int>(e % bn);
      amax = fmaxf(amax, fabsf(load_elem<DT>(x, (r0 + r) * ldx + c0 + c)));
    }
  }
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float a = 0.f;
    for (int w = 0; w < (blockDim.x + 31) / 32; ++w) a = fmaxf(a, red[w]);
    if (a > 0.f) atomicMax(amax_bits + blk, __float_as_uint(a));
  }
}
template <int DT>
__global__ void quant_slabs(const void* x, long long k, long long ldx, int bm, int bn, int slab_rows, int slabs,
                            int vec, uint8_t* codes, long long ldq, const float* amax) {
  constexpr int V = Vec<DT>::N;
  const long long nblk_k = k / bn;
  const long long blk = blockIdx.x / slabs;
  const int slab = blockIdx.x - blk * slabs;
  const long long bi = blk / nblk_k, bj = blk - bi * nblk_k;
  const int r_lo = slab * slab_rows, r_hi = min(bm, r_lo + slab_rows);
  const long long r0 = bi * bm, c0 = bj * bn;
  const float s = block_scale<DT>(amax[blk]);
  if (vec) {
    const int vpr = bn / V;
    const int nvec = (r_hi - r_lo) * vpr;
    for (int e = threadIdx.x; e < nvec; e += blockDim.x) {
      const int rr = e / vpr;
      const int r = r_lo + rr, c = (e - rr * vpr) * V;
      float v[V];
      load_vec<DT>(x, (r0 + r) * ldx + c0 + c, v);
      store_codes<DT>(codes + (r0 + r) * ldq + c0 + c, v, s);
    }
  } else {
    for (long long e = threadIdx.x; e < static_cast<long long>(r_hi - r_lo) * bn; e += blockDim.x) {
      const int r = r_lo + static_cast<int>(e / bn), c = static_cast<int>(e % bn);
      codes[(r0 + r) * ldq + c0 + c] = quant_elem<DT>(load_elem<DT>(x, (r0 + r) * ldx + c0 + c), s);
    }
  }
}
template <int DT>
__global__ void finalize_scales(float* scales, long long n) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i < n) scales[i] = block_scale<DT>(scales[i]);
}

template <int DT>
int launch(const void* x, long long m, long long k, long long ldx, int bm, int bn, uint8_t* codes, long long ldq,
           float* scales, cudaStream_t st) {
  constexpr int V = Vec<DT>::N;
  const long long nblocks = (m / bm) * (k / bn);
  const size_t esz = DT == MXB_FP32 ? 4 : 2;
  const bool aligned = (reinterpret_cast<uintptr_t>(x) % 16) == 0 && (ldx * esz) % 16 == 0 && (bn % V) == 0 &&
                       (reinterpret_cast<uintptr_t>(codes) % 8) == 0 && (ldq % 8) == 0;
  if (bm == 1) {
    const int lanes = bn / V;
    if (aligned && lanes <= 32 && (lanes & (lanes - 1)) == 0) {
      const long long threads = m * (k / V);
      const long long blocks = (threads + 255) / 256;
      quant_rows_vec<DT><<<static_cast<unsigned int>(blocks < 148 * 64 ? blocks : 148 * 64), 256, 0, st>>>(
          x, m, k, ldx, bn, codes, ldq, scales);
    } else if (aligned) {
      quant_rows_long<DT><<<static_cast<unsigned int>((nblocks * 32 + 255) / 256), 256, 0, st>>>(x, m, k, ldx, bn,
                                                                                                codes, ldq, scales);
    } else {
      quant_rows<DT><<<static_cast<unsigned int>((nblocks * 32 + 255) / 256), 256, 0, st>>>(x, m, k, ldx, bn, codes,
                                                                                           ldq, scales);
    }
  } else {
    // slabs of about 32K elements: enough CTAs for any block shape, one atomic per CTA
    int slab_rows = static_cast<int>((32768 + bn - 1) / bn);
    if (slab_rows < 1) slab_rows = 1;
    if (slab_rows > bm) slab_rows = bm;
    const int slabs = (bm + slab_rows - 1) / slab_rows;
    if (nblocks * slabs >= (1ll << 31)) return MXB_ERR_UNSUPPORTED;
    if (cudaMemsetAsync(scales, 0, nblocks * sizeof(float), st) != cudaSuccess) return MXB_ERR_CUDA;
    const unsigned int grid = static_cast<unsigned int>(nblocks * slabs);
    amax_slabs<DT><<<grid, 256, 0, st>>>(x, k, ldx, bm, bn, slab_rows, slabs, aligned ? 1 : 0,
                                         reinterpret_cast<unsigned int*>(scales));
    quant_slabs<DT><<<grid, 256, 0, st>>>(x, k, ldx, bm, bn, slab_rows, slabs, aligned ? 1 : 0, codes, ldq, scales);
    finalize_scales<DT><<<static_cast<unsigned int>((nblocks + 255) / 256), 256, 0, st>>>(scales, nblocks);
  }
  return cudaGetLastError() == cudaSuccess ? MXB_OK : MXB_ERR_CUDA;
}

}  // namespace

extern "C" int mxb_block_quant(const void* x, int x_dtype, long long m, long long k, long long ldx, int bm, int bn,
                               void* codes, long long ldq, float* scales, void* stream) {
  if (!x || !codes || !scales || m <= 0 || k <= 0 || bm <= 0 || bn <= 0) return MXB_ERR_INVALID;
  if (m % bm || k % bn || ldx < k || ldq < k) return MXB_ERR_INVALID;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint8_t* out = static_cast<uint8_t*>(codes);
  switch (x_dtype) {
    case MXB_FP32: return launch<MXB_FP32>(x, m, k, ldx, bm, bn, out, ldq, scales, st);
    case MXB_BF16: return launch<MXB_BF16>(x, m, k, ldx, bm, bn, out, ldq, scales, st);
    case MXB_FP16: return launch<MXB_FP16>(x, m, k, ldx, bm, bn, out, ldq, scales, st);
    default: return MXB_ERR_INVALID;
  }
}
