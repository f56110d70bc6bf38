// Kernel instantiations: CTA-pair (tcgen05 cta_group::2) kernels: 256 x 256 tiles with input scales
// constant along K or changing every 128 elements of K (promotion), and 256 x 224 tiles with 1x32
// power-of-two scales on the block-scaled MMA.
#include "mxb_dispatch.h"
#include "mxb_kernel2.cuh"

namespace mxb {
#define MXB_PAIR_ENTRY(BN, SM, OM, EW)                                                                    \
  {                                                                                                       \
    BN, SM, OM, EW, &launch_pair_kernel<PairCfg<BN, SM, OM, EW>>, PairCfg<BN, SM, OM, EW>::SMEM_BYTES,    \
        PairCfg<BN, SM, OM, EW>::STAGES, 1, 0, 0, 0                                                       \
  }
// single-scale twins of the promotion kernels (one Y scale per thread's column slice)
#define MXB_PAIR_ENTRY_SINGLE_Y(BN, SM, OM, EW)                                                                   \
  {                                                                                                               \
    BN, SM, OM, EW, &launch_pair_kernel<PairCfg<BN, SM, OM, EW, false, true>>,                                    \
        PairCfg<BN, SM, OM, EW, false, true>::SMEM_BYTES, PairCfg<BN, SM, OM, EW, false, true>::STAGES, 1, 0, 0, 1 \
  }
static const KernelEntry kPair[] = {
    MXB_PAIR_ENTRY_SINGLE_Y(256, SCALE_PROMOTE, OUT_HP, 8), MXB_PAIR_ENTRY_SINGLE_Y(256, SCALE_PROMOTE, OUT_QUANT_Y, 8),
    MXB_PAIR_ENTRY_SINGLE_Y(128, SCALE_PROMOTE, OUT_HP, 8), MXB_PAIR_ENTRY_SINGLE_Y(128, SCALE_PROMOTE, OUT_QUANT_Y, 8),
    MXB_PAIR_ENTRY(256, SCALE_EPILOGUE, OUT_HP, 4),      MXB_PAIR_ENTRY(256, SCALE_EPILOGUE, OUT_HP, 8),
    MXB_PAIR_ENTRY(256, SCALE_EPILOGUE, OUT_QUANT_Y, 4), MXB_PAIR_ENTRY(256, SCALE_EPILOGUE, OUT_QUANT_Y, 8),
    MXB_PAIR_ENTRY(256, SCALE_EPILOGUE, OUT_QUANT_X, 4), MXB_PAIR_ENTRY(256, SCALE_EPILOGUE, OUT_QUANT_X, 8),
    MXB_PAIR_ENTRY(224, SCALE_MX, OUT_HP, 4),            MXB_PAIR_ENTRY(224, SCALE_MX, OUT_QUANT_Y, 4),
    MXB_PAIR_ENTRY(224, SCALE_MX, OUT_QUANT_X, 4),
    MXB_PAIR_ENTRY(256, SCALE_PROMOTE, OUT_HP, 8),       MXB_PAIR_ENTRY(256, SCALE_PROMOTE, OUT_QUANT_Y, 8),
    MXB_PAIR_ENTRY(128, SCALE_PROMOTE, OUT_HP, 8),       MXB_PAIR_ENTRY(128, SCALE_PROMOTE, OUT_QUANT_Y, 8),
    MXB_PAIR_ENTRY(224, SCALE_EPILOGUE, OUT_HP, 4),      MXB_PAIR_ENTRY(224, SCALE_EPILOGUE, OUT_QUANT_Y, 4),
    MXB_PAIR_ENTRY(224, SCALE_EPILOGUE, OUT_QUANT_X, 4),
    // 256 x 128 tiles with scales constant along K: a decode-sized left operand (64 < M <= 128) as the Y operand,
    // each CTA staging 128 rows of the weight and 64 rows of left per K block
    MXB_PAIR_ENTRY(128, SCALE_EPILOGUE, OUT_HP, 4),      MXB_PAIR_ENTRY(128, SCALE_EPILOGUE, OUT_QUANT_Y, 4),
    MXB_PAIR_ENTRY(128, SCALE_EPILOGUE, OUT_QUANT_X, 4),
};
const KernelEntry* pair_kernels(int* count) {
  *count = static_cast<int>(sizeof(kPair) / sizeof(kPair[0]));
  return kPair;
}
}  // namespace mxb
