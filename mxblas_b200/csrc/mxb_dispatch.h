// Glue between the C ABI (mxb_host.cu) and the kernel instantiations (mxb_inst_*.cu).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include "mxb_kernel.cuh"

namespace mxb {

struct LaunchArgs {
  CUtensorMap tm_x, tm_y;
  GemmParams p;
  int grid;
  cudaStream_t stream;
};

typedef cudaError_t (*launch_fn)(const LaunchArgs&);

struct KernelEntry {
  int bn, scale_mode, out_mode, epi_warps;
  launch_fn fn;
  int smem_bytes;
  int stages;
  int ctas_per_sm;
  int two_per_sm;  // 128-wide tile built as a light CTA (two per SM); narrower tiles are light anyway
  int general;     // also handles operands stored along their rows and grouped GEMMs
  int single_y;    // promotion with one Y scale per thread's column slice (lean loop)
};

template <class Cfg>
cudaError_t launch_kernel(const LaunchArgs& a) {
  // the >48 KiB dynamic shared memory opt-in is per device: do it once for each
  static bool configured[64] = {};
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (dev < 64 && !configured[dev]) {
    err = cudaFuncSetAttribute(mx_gemm_sm100<Cfg>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               Cfg::SMEM_BYTES);
    if (err != cudaSuccess) return err;
    configured[dev] = true;
  }
  mx_gemm_sm100<Cfg><<<a.grid, Cfg::THREADS, Cfg::SMEM_BYTES, a.stream>>>(a.tm_x, a.tm_y, a.p);
  return cudaGetLastError();
}

#define MXB_ENTRY(BN, SM, OM, EW)                                                              \
  {                                                                                            \
    BN, SM, OM, EW, &launch_kernel<KernelCfg<BN, SM, OM, EW>>, KernelCfg<BN, SM, OM, EW>::SMEM_BYTES, \
        KernelCfg<BN, SM, OM, EW>::STAGES, KernelCfg<BN, SM, OM, EW>::CTAS_PER_SM, 0, 0, 0       \
  }
#define MXB_ENTRY_GENERAL(BN, SM, OM, EW)                                                                      \
  {                                                                                                            \
    BN, SM, OM, EW, &launch_kernel<KernelCfg<BN, SM, OM, EW, 0, true>>,                                        \
        KernelCfg<BN, SM, OM, EW, 0, true>::SMEM_BYTES, KernelCfg<BN, SM, OM, EW, 0, true>::STAGES,            \
        KernelCfg<BN, SM, OM, EW, 0, true>::CTAS_PER_SM, 0, 1, 0                                               \
  }
#define MXB_ENTRY_SINGLE_Y(BN, SM, OM, EW, GEN)                                                                          \
  {                                                                                                                    \
    BN, SM, OM, EW, &launch_kernel<KernelCfg<BN, SM, OM, EW, 0, GEN, true>>,                                           \
        KernelCfg<BN, SM, OM, EW, 0, GEN, true>::SMEM_BYTES, KernelCfg<BN, SM, OM, EW, 0, GEN, true>::STAGES,          \
        KernelCfg<BN, SM, OM, EW, 0, GEN, true>::CTAS_PER_SM, 0, GEN ? 1 : 0, 1                                        \
  }
#define MXB_ENTRY_TWO_PER_SM(BN, SM, OM, EW)                                                           \
  {                                                                                                    \
    BN, SM, OM, EW, &launch_kernel<KernelCfg<BN, SM, OM, EW, 1>>, KernelCfg<BN, SM, OM, EW, 1>::SMEM_BYTES, \
        KernelCfg<BN, SM, OM, EW, 1>::STAGES, KernelCfg<BN, SM, OM, EW, 1>::CTAS_PER_SM, 1, 0, 0       \
  }

// one table per translation unit
const KernelEntry* epilogue_kernels(int* count);
const KernelEntry* promote_kernels(int* count);
const KernelEntry* mx_kernels(int* count);
const KernelEntry* pair_kernels(int* count);  // CTA-pair (cta_group::2) kernels, bn == 256
const KernelEntry* quant2d_kernels(int* count);       // OUT_QUANT_2D, one CTA per tile, all scale modes
const KernelEntry* quant2d_pair_kernels(int* count);  // OUT_QUANT_2D, CTA pairs
const KernelEntry* general_kernels(int* count);       // GENERAL instantiations, one CTA per tile
const KernelEntry* general_pair_kernels(int* count);  // GENERAL instantiations, CTA pairs

}  // namespace mxb
