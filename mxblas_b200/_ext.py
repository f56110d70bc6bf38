"""ctypes binding of libmxblas_b200.so (the C ABI declared in include/mxblas_b200.h).

Stands where the reference loads each JIT-built kernel with ctypes.CDLL and calls its `launch`
symbol (mxblas/jit/runtime.py:10-53). There is no CPU or PyTorch fallback: if the library is
missing the import of this module fails.
"""

from __future__ import annotations

import ctypes
import os
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libmxblas_b200.so"

# mxb_status_t
MXB_OK = 0
MXB_ERR_INVALID = 1
MXB_ERR_UNSUPPORTED = 2
MXB_ERR_WORKSPACE = 3
MXB_ERR_CUDA = 4
MXB_ERR_DEVICE = 5

# mxb_dtype_t
MXB_FP32, MXB_BF16, MXB_FP16, MXB_E4M3, MXB_E5M2 = range(5)

# flags
MXB_OUT_QUANT = 0x1
MXB_OUT_TRANSPOSE = 0x2
MXB_OUT_SCALE_TRANSPOSE = 0x4
MXB_OUT_SCALE_POW2 = 0x8
MXB_IN_SCALES_POW2 = 0x10
MXB_IN_SCALES_PROBE = 0x20
MXB_LEFT_COL_MAJOR = 0x40
MXB_RIGHT_ROW_MAJOR = 0x80

MXB_STATIC_SCRATCH_BYTES = 8 << 20  # scratch built into the library (mxb_gemm_static_scratch)

# every symbol include/mxblas_b200.h declares
EXPORTED_SYMBOLS = (
    "mxb_abi_version",
    "mxb_status_string",
    "mxb_last_cuda_error",
    "mxb_query_workspace",
    "mxb_default_config",
    "mxb_gemm",
    "mxb_gemm_cfg",
    "mxb_grouped_gemm",
    "mxb_grouped_query_workspace",
    "mxb_push_block",
    "mxb_push_block_ex",
    "mxb_push_block_dma",
    "mxb_gemm_host",
    "mxb_gemm_static_scratch",
    "mxb_block_quant",
    "mxb_selftest_wait_timeout",
    "mxb_device_status",
    "mxb_launch_count",
)


class MxbProblem(ctypes.Structure):
    _fields_ = [
        ("m", ctypes.c_int32),
        ("n", ctypes.c_int32),
        ("k", ctypes.c_int32),
        ("sm", ctypes.c_int32),
        ("sn", ctypes.c_int32),
        ("sk", ctypes.c_int32),
        ("qm", ctypes.c_int32),
        ("qn", ctypes.c_int32),
        ("in_dtype", ctypes.c_int32),
        ("out_dtype", ctypes.c_int32),
        ("scale_dtype", ctypes.c_int32),
        ("flags", ctypes.c_uint32),
        ("lda", ctypes.c_int64),
        ("ldb", ctypes.c_int64),
        ("as_rs", ctypes.c_int64),
        ("as_ks", ctypes.c_int64),
        ("bs_rs", ctypes.c_int64),
        ("bs_ks", ctypes.c_int64),
        ("ldc", ctypes.c_int64),
        ("ldcs", ctypes.c_int64),
    ]


class MxbConfig(ctypes.Structure):
    _fields_ = [
        ("bn", ctypes.c_int32),
        ("swap", ctypes.c_int32),
        ("epi_warps", ctypes.c_int32),
        ("raster", ctypes.c_int32),
        ("splits", ctypes.c_int32),
        ("ctas", ctypes.c_int32),
        ("cta_pair", ctypes.c_int32),
    ]

    def key(self):
        return (self.bn, self.swap, self.epi_warps, self.raster, self.splits, self.ctas, self.cta_pair)


def _load() -> ctypes.CDLL:
    path = os.environ.get("MXBLAS_B200_LIB", str(LIB_PATH))
    if not os.path.exists(path):
        raise ImportError(
            f"{path} not found: build it with `python mxblas_b200/build.py` "
            "(there is no fallback implementation)"
        )
    lib = ctypes.CDLL(path)
    vp, sz = ctypes.c_void_p, ctypes.c_size_t
    pp, cp = ctypes.POINTER(MxbProblem), ctypes.POINTER(MxbConfig)
    lib.mxb_abi_version.restype = ctypes.c_int
    lib.mxb_abi_version.argtypes = []
    lib.mxb_status_string.restype = ctypes.c_char_p
    lib.mxb_status_string.argtypes = [ctypes.c_int]
    lib.mxb_last_cuda_error.restype = ctypes.c_char_p
    lib.mxb_last_cuda_error.argtypes = []
    lib.mxb_query_workspace.restype = ctypes.c_int
    lib.mxb_query_workspace.argtypes = [pp, cp, ctypes.POINTER(sz)]
    lib.mxb_default_config.restype = ctypes.c_int
    lib.mxb_default_config.argtypes = [pp, cp]
    lib.mxb_gemm.restype = ctypes.c_int
    lib.mxb_gemm.argtypes = [pp, vp, vp, vp, vp, vp, vp, vp, sz, vp]
    lib.mxb_gemm_cfg.restype = ctypes.c_int
    lib.mxb_gemm_cfg.argtypes = [pp, cp, vp, vp, vp, vp, vp, vp, vp, sz, vp]
    lib.mxb_grouped_gemm.restype = ctypes.c_int
    lib.mxb_grouped_gemm.argtypes = [pp, cp, ctypes.c_int, vp, ctypes.c_int, vp, vp, vp, vp, vp, vp, vp, sz, vp]
    lib.mxb_grouped_query_workspace.restype = ctypes.c_int
    lib.mxb_grouped_query_workspace.argtypes = [pp, cp, ctypes.c_int, ctypes.c_int, ctypes.POINTER(sz)]
    lib.mxb_push_block.restype = ctypes.c_int
    lib.mxb_push_block.argtypes = [vp, ctypes.c_longlong, ctypes.POINTER(vp), ctypes.c_int, ctypes.c_longlong,
                                   ctypes.c_longlong, ctypes.c_longlong, vp]
    lib.mxb_push_block_ex.restype = ctypes.c_int
    lib.mxb_push_block_ex.argtypes = lib.mxb_push_block.argtypes[:-1] + [ctypes.c_int, vp]
    lib.mxb_push_block_dma.restype = ctypes.c_int
    lib.mxb_push_block_dma.argtypes = lib.mxb_push_block.argtypes
    lib.mxb_gemm_host.restype = ctypes.c_int
    lib.mxb_gemm_host.argtypes = [pp, vp, vp, vp, vp, vp, vp]
    lib.mxb_gemm_static_scratch.restype = ctypes.c_int
    lib.mxb_gemm_static_scratch.argtypes = [pp, vp, vp, vp, vp, vp, vp, vp]
    ll = ctypes.c_longlong
    lib.mxb_block_quant.restype = ctypes.c_int
    lib.mxb_block_quant.argtypes = [vp, ctypes.c_int, ll, ll, ll, ctypes.c_int, ctypes.c_int, vp, ll, vp, vp]
    lib.mxb_selftest_wait_timeout.restype = ctypes.c_int
    lib.mxb_selftest_wait_timeout.argtypes = [vp]
    lib.mxb_device_status.restype = ctypes.c_int
    lib.mxb_device_status.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_uint)]
    lib.mxb_launch_count.restype = ctypes.c_ulonglong
    lib.mxb_launch_count.argtypes = []
    if lib.mxb_abi_version() != 1:
        raise ImportError(f"{path}: ABI version {lib.mxb_abi_version()} != 1")
    return lib


lib = _load()


def status_text(status: int) -> str:
    text = lib.mxb_status_string(status).decode()
    if status == MXB_ERR_CUDA:
        text += ": " + lib.mxb_last_cuda_error().decode()
    return text


def device_status(clear: bool = True) -> int:
    """Synchronise the current device and return its status word (0 = no kernel reported an error)."""
    code = ctypes.c_uint(0)
    st = lib.mxb_device_status(1 if clear else 0, ctypes.byref(code))
    if st not in (MXB_OK, MXB_ERR_DEVICE):
        raise RuntimeError("mxb_device_status: " + status_text(st))
    return int(code.value)


def launch_count() -> int:
    return int(lib.mxb_launch_count())
