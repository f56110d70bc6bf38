// Kernel instantiations that also take operands stored along their rows (a column-major left, a row-major
// right: the layouts of a backward pass, which the reference's templates do not match,
// mxblas/gemm/template.py:70-73) and grouped GEMMs (one weight per group): one CTA per 128- or 256-wide tile.
#include "mxb_dispatch.h"

namespace mxb {
static const KernelEntry kGeneral[] = {
    MXB_ENTRY_GENERAL(128, SCALE_EPILOGUE, OUT_HP, 4),      MXB_ENTRY_GENERAL(128, SCALE_EPILOGUE, OUT_QUANT_Y, 4),
    MXB_ENTRY_GENERAL(128, SCALE_EPILOGUE, OUT_QUANT_X, 4), MXB_ENTRY_GENERAL(256, SCALE_EPILOGUE, OUT_HP, 4),
    MXB_ENTRY_GENERAL(256, SCALE_EPILOGUE, OUT_QUANT_Y, 4), MXB_ENTRY_GENERAL(256, SCALE_EPILOGUE, OUT_QUANT_Y, 8),
    MXB_ENTRY_GENERAL(256, SCALE_EPILOGUE, OUT_QUANT_X, 4), MXB_ENTRY_GENERAL(256, SCALE_EPILOGUE, OUT_QUANT_X, 8),
    MXB_ENTRY_GENERAL(128, SCALE_PROMOTE, OUT_HP, 4),       MXB_ENTRY_GENERAL(128, SCALE_PROMOTE, OUT_HP, 8),
    MXB_ENTRY_GENERAL(128, SCALE_PROMOTE, OUT_QUANT_Y, 4),  MXB_ENTRY_GENERAL(128, SCALE_PROMOTE, OUT_QUANT_Y, 8),
    MXB_ENTRY_GENERAL(128, SCALE_PROMOTE, OUT_QUANT_X, 4),  MXB_ENTRY_GENERAL(128, SCALE_PROMOTE, OUT_QUANT_X, 8),
    MXB_ENTRY_GENERAL(256, SCALE_PROMOTE, OUT_HP, 8),       MXB_ENTRY_GENERAL(256, SCALE_PROMOTE, OUT_QUANT_Y, 8),
    MXB_ENTRY_GENERAL(128, SCALE_MX, OUT_HP, 4),            MXB_ENTRY_GENERAL(128, SCALE_MX, OUT_QUANT_Y, 4),
    MXB_ENTRY_GENERAL(128, SCALE_MX, OUT_QUANT_X, 4),
    // single-scale twins of the promotion kernels (lean loop)
    MXB_ENTRY_SINGLE_Y(128, SCALE_PROMOTE, OUT_HP, 8, true),       MXB_ENTRY_SINGLE_Y(128, SCALE_PROMOTE, OUT_QUANT_Y, 8, true),
};
const KernelEntry* general_kernels(int* count) {
  *count = static_cast<int>(sizeof(kGeneral) / sizeof(kGeneral[0]));
  return kGeneral;
}
}  // namespace mxb
