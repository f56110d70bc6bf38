// Kernel instantiations: input scales that change along K (1x128 per-token blocks, 128x128 blocks,
// 1x32 blocks with arbitrary values): TMEM partial sums are scaled and accumulated in registers.
#include "mxb_dispatch.h"

namespace mxb {
static const KernelEntry kPromote[] = {
    MXB_ENTRY(32, SCALE_PROMOTE, OUT_HP, 4),       MXB_ENTRY(64, SCALE_PROMOTE, OUT_HP, 4),
    MXB_ENTRY(128, SCALE_PROMOTE, OUT_HP, 4),      MXB_ENTRY(128, SCALE_PROMOTE, OUT_HP, 8),
    MXB_ENTRY(256, SCALE_PROMOTE, OUT_HP, 8),
    MXB_ENTRY(32, SCALE_PROMOTE, OUT_QUANT_Y, 4),  MXB_ENTRY(64, SCALE_PROMOTE, OUT_QUANT_Y, 4),
    MXB_ENTRY(128, SCALE_PROMOTE, OUT_QUANT_Y, 4), MXB_ENTRY(128, SCALE_PROMOTE, OUT_QUANT_Y, 8),
    MXB_ENTRY(256, SCALE_PROMOTE, OUT_QUANT_Y, 8),
    MXB_ENTRY(32, SCALE_PROMOTE, OUT_QUANT_X, 4),  MXB_ENTRY(64, SCALE_PROMOTE, OUT_QUANT_X, 4),
    MXB_ENTRY(128, SCALE_PROMOTE, OUT_QUANT_X, 4), MXB_ENTRY(128, SCALE_PROMOTE, OUT_QUANT_X, 8),
    // single-scale twins: one Y scale covers a thread's whole column slice (lean loop)
    // (128-wide tiles only: on one-CTA 256-wide tiles the lean loop measured slower than the general one)
    MXB_ENTRY_SINGLE_Y(128, SCALE_PROMOTE, OUT_HP, 4, false),      MXB_ENTRY_SINGLE_Y(128, SCALE_PROMOTE, OUT_HP, 8, false),
    MXB_ENTRY_SINGLE_Y(128, SCALE_PROMOTE, OUT_QUANT_Y, 4, false), MXB_ENTRY_SINGLE_Y(128, SCALE_PROMOTE, OUT_QUANT_Y, 8, false),
};
const KernelEntry* promote_kernels(int* count) {
  *count = static_cast<int>(sizeof(kPromote) / sizeof(kPromote[0]));
  return kPromote;
}
}  // namespace mxb

