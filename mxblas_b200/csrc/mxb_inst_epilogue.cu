// Kernel instantiations: input scales constant along K (per-tensor, per-channel, per-token with
// sk == K), applied once on the TMEM -> register path.
#include "mxb_dispatch.h"

namespace mxb {
static const KernelEntry kEpilogue[] = {
    MXB_ENTRY(32, SCALE_EPILOGUE, OUT_HP, 4),       MXB_ENTRY(64, SCALE_EPILOGUE, OUT_HP, 4),
    MXB_ENTRY(128, SCALE_EPILOGUE, OUT_HP, 4),      MXB_ENTRY(256, SCALE_EPILOGUE, OUT_HP, 4),
    MXB_ENTRY(256, SCALE_EPILOGUE, OUT_HP, 8),
    MXB_ENTRY(32, SCALE_EPILOGUE, OUT_QUANT_Y, 4),  MXB_ENTRY(64, SCALE_EPILOGUE, OUT_QUANT_Y, 4),
    MXB_ENTRY(128, SCALE_EPILOGUE, OUT_QUANT_Y, 4), MXB_ENTRY(256, SCALE_EPILOGUE, OUT_QUANT_Y, 4),
    MXB_ENTRY(256, SCALE_EPILOGUE, OUT_QUANT_Y, 8),
    MXB_ENTRY(32, SCALE_EPILOGUE, OUT_QUANT_X, 4),  MXB_ENTRY(64, SCALE_EPILOGUE, OUT_QUANT_X, 4),
    MXB_ENTRY(128, SCALE_EPILOGUE, OUT_QUANT_X, 4), MXB_ENTRY(256, SCALE_EPILOGUE, OUT_QUANT_X, 4),
    MXB_ENTRY(256, SCALE_EPILOGUE, OUT_QUANT_X, 8),
    // 128-wide tiles as light CTAs, two per SM: skinny problems whose tile count falls between one and two waves
    MXB_ENTRY_TWO_PER_SM(128, SCALE_EPILOGUE, OUT_HP, 4),
    MXB_ENTRY_TWO_PER_SM(128, SCALE_EPILOGUE, OUT_QUANT_Y, 4),
    MXB_ENTRY_TWO_PER_SM(128, SCALE_EPILOGUE, OUT_QUANT_X, 4),
};
const KernelEntry* epilogue_kernels(int* count) {
  *count = static_cast<int>(sizeof(kEpilogue) / sizeof(kEpilogue[0]));
  return kEpilogue;
}
}  // namespace mxb
