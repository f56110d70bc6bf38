// Kernel instantiations: output quantisation in two-dimensional [QM, QN] blocks (OUT_QUANT_2D), which the
// reference refuses (static_assert(c_q_m == 1), mxblas/gemm/generator.py:971). One-CTA kernels on 128- and
// 256-wide tiles for the three ways of applying input scales, and the CTA-pair kernels.
#include "mxb_dispatch.h"
#include "mxb_kernel2.cuh"

namespace mxb {
static const KernelEntry kQuant2d[] = {
    MXB_ENTRY(128, SCALE_EPILOGUE, OUT_QUANT_2D, 4), MXB_ENTRY(256, SCALE_EPILOGUE, OUT_QUANT_2D, 8),
    MXB_ENTRY(128, SCALE_PROMOTE, OUT_QUANT_2D, 4),  MXB_ENTRY(128, SCALE_PROMOTE, OUT_QUANT_2D, 8),
    MXB_ENTRY(256, SCALE_PROMOTE, OUT_QUANT_2D, 8),  MXB_ENTRY(128, SCALE_MX, OUT_QUANT_2D, 4),
};
const KernelEntry* quant2d_kernels(int* count) {
  *count = static_cast<int>(sizeof(kQuant2d) / sizeof(kQuant2d[0]));
  return kQuant2d;
}

#define MXB_PAIR_ENTRY(BN, SM, OM, EW)                                                                    \
  {                                                                                                       \
    BN, SM, OM, EW, &launch_pair_kernel<PairCfg<BN, SM, OM, EW>>, PairCfg<BN, SM, OM, EW>::SMEM_BYTES,    \
        PairCfg<BN, SM, OM, EW>::STAGES, 1, 0, 0, 0                                                       \
  }
static const KernelEntry kQuant2dPair[] = {
    {256, SCALE_PROMOTE, OUT_QUANT_2D, 8, &launch_pair_kernel<PairCfg<256, SCALE_PROMOTE, OUT_QUANT_2D, 8, false, true>>,
     PairCfg<256, SCALE_PROMOTE, OUT_QUANT_2D, 8, false, true>::SMEM_BYTES,
     PairCfg<256, SCALE_PROMOTE, OUT_QUANT_2D, 8, false, true>::STAGES, 1, 0, 0, 1},  // single-scale twin
    MXB_PAIR_ENTRY(256, SCALE_EPILOGUE, OUT_QUANT_2D, 8),
    MXB_PAIR_ENTRY(256, SCALE_PROMOTE, OUT_QUANT_2D, 8),
    MXB_PAIR_ENTRY(224, SCALE_MX, OUT_QUANT_2D, 4),
};
const KernelEntry* quant2d_pair_kernels(int* count) {
  *count = static_cast<int>(sizeof(kQuant2dPair) / sizeof(kQuant2dPair[0]));
  return kQuant2dPair;
}
}  // namespace mxb
