// CTA-pair kernel instantiations that also take operands stored along their rows and grouped GEMMs
// (see mxb_inst_general.cu): 256 x 256 tiles with scales constant along K or promoted per 128-deep K block.
#include "mxb_dispatch.h"
#include "mxb_kernel2.cuh"

namespace mxb {
#define MXB_PAIR_ENTRY_GENERAL(BN, SM, OM, EW)                                                         \
  {                                                                                                    \
    BN, SM, OM, EW, &launch_pair_kernel<PairCfg<BN, SM, OM, EW, true>>,                                \
        PairCfg<BN, SM, OM, EW, true>::SMEM_BYTES, PairCfg<BN, SM, OM, EW, true>::STAGES, 1, 0, 1, 0   \
  }
#define MXB_PAIR_ENTRY_GENERAL_SINGLE_Y(BN, SM, OM, EW)                                                        \
  {                                                                                                           \
    BN, SM, OM, EW, &launch_pair_kernel<PairCfg<BN, SM, OM, EW, true, true>>,                                 \
        PairCfg<BN, SM, OM, EW, true, true>::SMEM_BYTES, PairCfg<BN, SM, OM, EW, true, true>::STAGES, 1, 0, 1, 1 \
  }
static const KernelEntry kGeneralPair[] = {
    MXB_PAIR_ENTRY_GENERAL_SINGLE_Y(256, SCALE_PROMOTE, OUT_HP, 8),
    MXB_PAIR_ENTRY_GENERAL_SINGLE_Y(256, SCALE_PROMOTE, OUT_QUANT_Y, 8),
    MXB_PAIR_ENTRY_GENERAL(256, SCALE_EPILOGUE, OUT_HP, 4),      MXB_PAIR_ENTRY_GENERAL(256, SCALE_EPILOGUE, OUT_QUANT_Y, 4),
    MXB_PAIR_ENTRY_GENERAL(256, SCALE_EPILOGUE, OUT_QUANT_Y, 8), MXB_PAIR_ENTRY_GENERAL(256, SCALE_EPILOGUE, OUT_QUANT_X, 4),
    MXB_PAIR_ENTRY_GENERAL(256, SCALE_EPILOGUE, OUT_QUANT_X, 8), MXB_PAIR_ENTRY_GENERAL(256, SCALE_PROMOTE, OUT_HP, 8),
    MXB_PAIR_ENTRY_GENERAL(256, SCALE_PROMOTE, OUT_QUANT_Y, 8),
};
const KernelEntry* general_pair_kernels(int* count) {
  *count = static_cast<int>(sizeof(kGeneralPair) / sizeof(kGeneralPair[0]));
  return kGeneralPair;
}
}  // namespace mxb
