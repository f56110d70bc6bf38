// Inline-PTX building blocks for the sm_100a MX-GEMM kernels: mbarrier, TMA (no cluster
// multicast anywhere), tcgen05 (TMEM allocation, MMA issue, commit, TMEM loads, smem->TMEM copy).
//
// Replaces, for Blackwell, what the reference keeps in mxblas/include/mxblas/ptx_wrapper.cuh:8-197
// (mbarrier + TMA + wgmma sync wrappers) and mxblas/include/mxblas/wgmma.cuh:11-66 (matrix
// descriptors). Every wait in this file is bounded: it gives up after MXB_WAIT_LIMIT_CYCLES, raises a
// CTA-wide abort flag and records a status code instead of spinning forever on a shared GPU.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>

namespace mxb {

// Upper bound of one wait in SM clock cycles (about one second at 2 GHz, longer at lower clocks);
// after that the kernel bails out. The SM-local cycle counter is used because it is cheap to read:
// reading %globaltimer costs on the order of a microsecond, which would sit on every wait that
// does not succeed at once.
#ifndef MXB_WAIT_LIMIT_CYCLES
#define MXB_WAIT_LIMIT_CYCLES 2000000000ll
#endif

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}


// ---------------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init() {
  // make the initialised barriers visible to the async proxy (TMA, tcgen05.commit)
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Non-blocking form: true if the phase with this parity has completed. (try_wait may suspend the
// thread for a while when it has not; this one returns at once.)
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Status codes written to the device status word (first error wins).
enum : uint32_t {
  DEV_OK = 0,
  DEV_TIMEOUT_PRODUCER = 0x100,  // TMA warp waited too long for a free smem stage
  DEV_TIMEOUT_MMA_FULL = 0x200,  // MMA warp waited too long for a filled smem stage
  DEV_TIMEOUT_MMA_TMEM = 0x300,  // MMA warp waited too long for a drained accumulator
  DEV_TIMEOUT_EPILOGUE = 0x400,  // epilogue warp waited too long for a finished accumulator
  DEV_TIMEOUT_FIXUP = 0x500,     // split-K fix-up waited too long for its peers
  DEV_NOT_POW2 = 0x600,          // scale pre-pack found a scale that is not a power of two
  DEV_TIMEOUT_SELFTEST = 0x700,  // the self-test's wait (which nothing can satisfy) ran out, as designed
  DEV_TIMEOUT_SCALES = 0x800,    // scale-factor warp waited too long for a free TMEM slot
};

// Bounded wait. Returns false if this wait timed out or another role of the CTA already aborted.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                          unsigned int* status, uint32_t code) {
  if (mbar_try_wait(bar, parity)) return true;
  long long t0 = 0;
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 0xFF) == 0) {
      if (*abort_flag) return false;
      const long long now = clock64();
      if (t0 == 0) t0 = now;
      if (now - t0 > MXB_WAIT_LIMIT_CYCLES) {
        *abort_flag = 1;
        atomicCAS(status, 0u, code);
        return false;
      }
    }
  }
  return true;
}

// Warp-wide wait: one lane polls the barrier, the others wait for it at the warp barrier. Thirty-two
// lanes (times eight warps) polling the same mbarrier would keep the shared-memory barrier unit busy
// with requests that compete with the arrivals and waits on the critical path.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                               unsigned int* status, uint32_t code, int lane) {
  uint32_t ok = 1;
  if (lane == 0) ok = mbar_wait(bar, parity, abort_flag, status, code) ? 1u : 0u;
  ok = __shfl_sync(0xffffffffu, ok, 0);
  return ok != 0;
}

// ---------------------------------------------------------------------------------------------
// TMA (bulk tensor copies). Loads are always CTA-local: no .multicast::cluster form is used.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

// 2-D tiled load: c0 = innermost (byte/element) coordinate, c1 = row coordinate.
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const void* tmap, uint32_t bar, int c0,
                                            int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(dst_smem), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}

// Untiled bulk load of `bytes` contiguous bytes (both addresses 16-byte aligned, bytes % 16 == 0).
__device__ __forceinline__ void bulk_load_1d(uint32_t dst_smem, const void* src, uint32_t bytes,
                                             uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      :
      : "r"(dst_smem), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
      : "memory");
}


// ---------------------------------------------------------------------------------------------
// tcgen05: tensor memory + 5th-generation tensor-core MMA
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Shared-memory matrix descriptor for a K-major operand tile whose rows are 128 bytes long and
// stored with the 128-byte TMA swizzle (8-row groups 1024 bytes apart). `addr` is the shared
// address of the (1024-byte aligned) tile plus the byte offset of the K slice to read.
__device__ __forceinline__ uint64_t umma_desc_k128(uint32_t addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr >> 4) & 0x3FFF);  // start address, 16-byte units
  d |= static_cast<uint64_t>(1) << 16;               // leading byte offset (unused with swizzle)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;       // stride byte offset: next 8-row group
  d |= static_cast<uint64_t>(1) << 46;               // descriptor version (Blackwell)
  d |= static_cast<uint64_t>(2) << 61;               // layout: 128-byte swizzle
  return d;
}

// The same for an operand tile that is contiguous along M (or N) instead of K, as a column-major `left` or a
// row-major `right` is: the tile is staged as K rows of 128 bytes (128 consecutive rows of the operand per K
// element) with the 128-byte swizzle; groups of eight K rows lie 1024 bytes apart (stride byte offset) and
// the next 128 operand rows start one whole staged block of `block_bytes` later (leading byte offset). The
// matching instruction-descriptor bit (umma_idesc_major) tells the MMA which form an operand has.
__device__ __forceinline__ uint64_t umma_desc_mn128(uint32_t addr, uint32_t block_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr >> 4) & 0x3FFF);
  d |= static_cast<uint64_t>((block_bytes >> 4) & 0x3FFF) << 16;  // leading byte offset: next 128 rows of the operand
  d |= static_cast<uint64_t>(1024 >> 4) << 32;                    // stride byte offset: next group of eight K rows
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
// The MMA-issuing thread is a serial resource (every instruction between two MMAs is exposed), so the constant
// bits of a descriptor are chosen once, outside the loops (umma_desc_hi, for either operand form), and per stage
// only the address field of the low word steps (umma_desc_words).
__device__ __forceinline__ uint64_t umma_desc_hi(int mn_major) {
  return mn_major ? (umma_desc_mn128(0, 16384)) : (umma_desc_k128(0));
}

// instruction-descriptor bits for operands that are M-/N-major (bit 15: A, bit 16: B); valid for the 8-bit types
__host__ __device__ constexpr uint32_t umma_idesc_major(uint32_t idesc, int a_mn, int b_mn) {
  return idesc | (static_cast<uint32_t>(a_mn ? 1 : 0) << 15) | (static_cast<uint32_t>(b_mn ? 1 : 0) << 16);
}

// Descriptor for an un-swizzled block of rows of 16 bytes each (8-row groups 128 bytes apart),
// the source format of the scale-factor copy tcgen05.cp.32x128b.
__device__ __forceinline__ uint64_t umma_desc_rows16(uint32_t addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr >> 4) & 0x3FFF);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(128 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  return d;
}

// Instruction descriptor, kind::f8f6f4, fp32 accumulate, both operands K-major.
// fmt: 0 = e4m3, 1 = e5m2.
__host__ __device__ constexpr uint32_t umma_idesc_f8(int m, int n, int a_fmt, int b_fmt) {
  return (1u << 4) | (static_cast<uint32_t>(a_fmt) << 7) | (static_cast<uint32_t>(b_fmt) << 10) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}
// Instruction descriptor, kind::mxf8f6f4.block_scale with UE8M0 scale factors. The two scale-id
// fields (which byte of the 32-bit TMEM scale column this MMA uses) are OR-ed in per K slice.
__host__ __device__ constexpr uint32_t umma_idesc_mxf8(int m, int n, int a_fmt, int b_fmt) {
  return (static_cast<uint32_t>(a_fmt) << 7) | (static_cast<uint32_t>(b_fmt) << 10) |
         (static_cast<uint32_t>(n >> 3) << 17) | (1u << 23) | (static_cast<uint32_t>(m >> 4) << 24);
}
__device__ __forceinline__ uint32_t umma_idesc_sf_ids(uint32_t idesc, uint32_t a_id, uint32_t b_id) {
  return idesc | (b_id << 4) | (a_id << 29);
}

// D[tmem] (+)= A[smem] * B[smem]; one thread issues for the CTA.
__device__ __forceinline__ void umma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
      "}\n"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void umma_mxf8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate, uint32_t sfa_tmem, uint32_t sfb_tmem) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n"
      "}\n"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem),
        "r"(sfb_tmem)
      : "memory");
}

// All tcgen05 operations this thread issued so far arrive (once) on `bar` when they complete.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

// 32 rows x 16 bytes of shared memory -> 4 TMEM columns, replicated to all four lane quadrants.
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

// TMEM -> registers: lane i of the warp receives 32 consecutive 32-bit columns of TMEM lane
// (base lane + i). A warp may only touch the lane quadrant 32*(warp_id % 4).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
        "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
        "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// registers -> TMEM: lane i of the warp writes 32 consecutive 32-bit columns of TMEM lane (base lane + i);
// same lane-quadrant rule as the loads
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
        "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]),
        "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// Register re-allocation between warpgroups (all four warps of a warpgroup execute it together).
template <int N>
__device__ __forceinline__ void reg_dealloc() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void reg_alloc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}

// ---------------------------------------------------------------------------------------------
// small numeric helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// Two independent round-to-nearest FMAs in one instruction (sm_100 packed fp32): acc{0,1} += a{0,1} * s{0,1}.
// Same results as two fmaf calls; half the issue slots, which is what bounds the promotion warps.
__device__ __forceinline__ void fma2(float& acc0, float& acc1, uint32_t a0, uint32_t a1, float s0, float s1) {
  uint64_t c, a, s;
  asm("mov.b64 %0, {%1, %2};" : "=l"(c) : "f"(acc0), "f"(acc1));
  asm("mov.b64 %0, {%1, %2};" : "=l"(a) : "r"(a0), "r"(a1));
  asm("mov.b64 %0, {%1, %2};" : "=l"(s) : "f"(s0), "f"(s1));
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(c) : "l"(a), "l"(s));
  asm("mov.b64 {%0, %1}, %2;" : "=f"(acc0), "=f"(acc1) : "l"(c));
}

// four floats -> four fp8 codes (round-to-nearest-even, saturate to the largest finite value)
template <bool E5M2>
__device__ __forceinline__ uint32_t pack_fp8x4(float a, float b, float c, float d) {
  constexpr __nv_fp8_interpretation_t kind = E5M2 ? __NV_E5M2 : __NV_E4M3;
  uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, kind);
  uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, kind);
  return lo | (hi << 16);
}

}  // namespace mxb

// ---------------------------------------------------------------------------------------------
// CTA pairs (cluster of two): tcgen05 cta_group::2 and the cross-CTA barrier traffic it needs.
// No load here is multicast: each CTA fetches its own operand halves; only barrier signals cross.
// ---------------------------------------------------------------------------------------------
namespace mxb {

__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// arrive / expect-tx on a barrier that may live in the peer CTA (shared::cluster address)
__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t bar_cluster, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(bar_cluster),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster) : "memory");
}
// the same with release semantics at cluster scope, for arrivals that publish this thread's own earlier
// work to a waiter in the peer CTA (used off the critical path only: see mbar_try_wait_cluster)
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t bar_cluster) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster) : "memory");
}
// wait on a barrier whose arrivals may come from the peer CTA. Default (CTA-scope) semantics are
// enough: what the arrivals order is asynchronous-proxy traffic (TMA bytes, MMA completion, TMEM
// reads fenced by tcgen05.fence), not generic-proxy memory shared across the pair.
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                                  unsigned int* status, uint32_t code) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  long long t0 = 0;
  uint32_t spins = 0;
  while (!mbar_try_wait_cluster(bar, parity)) {
    if ((++spins & 0xFF) == 0) {
      if (*abort_flag) return false;
      const long long now = clock64();
      if (t0 == 0) t0 = now;
      if (now - t0 > MXB_WAIT_LIMIT_CYCLES) {
        *abort_flag = 1;
        atomicCAS(status, 0u, code);
        return false;
      }
    }
  }
  return true;
}

// TMA load into this CTA's shared memory whose completion bytes are counted on a barrier of the
// pair's leader CTA (cta_group::2 form, not multicast).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst_smem, const void* tmap, uint32_t bar_cluster,
                                                 int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(dst_smem), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar_cluster), "r"(c0), "r"(c1)
      : "memory");
}

__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// 256 x N x 32 MMA across the CTA pair; issued by one thread of the leader CTA.
__device__ __forceinline__ void umma_f8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
      "}\n"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// The same with the accumulate flag fixed at "add to D": no predicate to compute in the issuing thread.
__device__ __forceinline__ void umma_f8_pair_acc(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.eq.u32 p, 1, 1;\n"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
      "}\n"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc)
      : "memory");
}

// Same, but the arrival is delivered to the barrier at this shared-memory offset in every CTA of
// `cta_mask` (bit i = CTA rank i of the cluster): one instruction releases a stage in both CTAs of a
// pair. This multicasts a barrier SIGNAL only; no data load in this library is multicast.
__device__ __forceinline__ void umma_commit_pair_both(uint32_t bar_local, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          bar_local),
      "h"(cta_mask)
      : "memory");
}

// Block-scaled 256 x N x 32 MMA across the CTA pair (UE8M0 scale factors in each CTA's TMEM).
__device__ __forceinline__ void umma_mxf8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                               uint32_t accumulate, uint32_t sfa_tmem, uint32_t sfb_tmem) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n"
      "}\n"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}

__device__ __forceinline__ void umma_mxf8_pair_acc(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                   uint32_t sfa_tmem, uint32_t sfb_tmem) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.eq.u32 p, 1, 1;\n"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%4], [%5], p;\n"
      "}\n"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}

// one-CTA forms with the accumulate flag fixed at "add to D"
__device__ __forceinline__ void umma_f8_acc(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.eq.u32 p, 1, 1;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
      "}\n"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc)
      : "memory");
}

// A 64-bit shared-memory descriptor from its two words (the high word of an operand's descriptors never changes;
// the low word holds the address field, which steps by plain 32-bit additions).
__device__ __forceinline__ uint64_t umma_desc_words(uint32_t lo, uint32_t hi) {
  return (static_cast<uint64_t>(hi) << 32) | lo;
}

}  // namespace mxb
