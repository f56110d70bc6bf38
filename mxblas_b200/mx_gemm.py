"""The public operator: ``mx_gemm_kernel`` and ``register_all_kernels``.

Drop-in for mxblas/jit_kernels/mx_gemm.py:340-457 of the reference: same name, positional order,
defaults, return tuple and ``ValueError`` conditions. Underneath, instead of matching a generated
Hopper template and JIT-compiling it, the call fills an ``mxb_problem_t`` and hands raw device
pointers to the prebuilt sm_100a library through its C ABI (include/mxblas_b200.h).

Extensions (keyword-only, defaults keep the reference's behaviour):
  out_scale_pow2   round every output group scale up to a power of two
  pow2_scales      None: 1x32-scaled problems test their scales on the device and use the native
                   block-scaled MMA when all are powers of two (otherwise the same call falls back,
                   still on the device, to register promotion); True: the caller guarantees it;
                   False: never use the block-scaled MMA
  config           an ``MxbConfig`` to force tile shape / split-K / operand roles (autotuner, tests)
"""

from __future__ import annotations

import ctypes
from functools import lru_cache
from typing import NamedTuple, Optional, Tuple

import torch

from . import _ext
from ._ext import MxbConfig, MxbProblem

supported_fp8_dtypes = (torch.float8_e4m3fn, torch.float8_e5m2)
supported_fp16_dtypes = (torch.float16, torch.bfloat16)
supported_fp32_dtypes = (torch.float32,)
supported_high_precision_dtypes = supported_fp16_dtypes + supported_fp32_dtypes

_DTYPE_CODE = {
    torch.float32: _ext.MXB_FP32,
    torch.bfloat16: _ext.MXB_BF16,
    torch.float16: _ext.MXB_FP16,
    torch.float8_e4m3fn: _ext.MXB_E4M3,
    torch.float8_e5m2: _ext.MXB_E5M2,
}


class _Meta(NamedTuple):
    """Everything derived from dtypes, shapes and strides (cached per distinct call signature)."""

    m: int
    n: int
    k: int
    sm: int
    sn: int
    sk: int
    qm: int
    qn: int
    in_dtype: torch.dtype
    out_dtype: torch.dtype
    scale_dtype: torch.dtype
    quant: bool
    out_transpose: bool
    out_scale_transpose: bool
    lda: int
    ldb: int
    as_rs: int
    as_ks: int
    bs_rs: int
    bs_ks: int
    left_col_major: bool = False
    right_row_major: bool = False


def _is_row_major(stride, size) -> bool:
    return stride[1] == 1 or size[1] == 1


def _is_col_major(stride, size) -> bool:
    return stride[0] == 1 or size[0] == 1


@lru_cache(maxsize=None)
def get_meta_info(
    left_dtype,
    right_dtype,
    left_scale_dtype,
    right_scale_dtype,
    output_quant,
    quant_size,
    out_dtype,
    left_size,
    right_size,
    left_scale_size,
    right_scale_size,
    left_stride,
    right_stride,
    left_scale_stride,
    right_scale_stride,
    out_transpose,
    out_scale_transpose,
) -> _Meta:
    """Validate one call signature; the checks and their order follow mx_gemm.py:60-194."""
    # dtypes (mx_gemm.py:82-92)
    if not (left_dtype == right_dtype and left_dtype in supported_fp8_dtypes):
        raise ValueError(
            f"Unsupported input dtypes {left_dtype} and {right_dtype}. "
            f"Supported dtypes are {supported_fp8_dtypes}."
        )
    if not (left_scale_dtype == right_scale_dtype and left_scale_dtype in supported_high_precision_dtypes):
        raise ValueError(
            f"Unsupported scale dtypes {left_scale_dtype} and {right_scale_dtype}. "
            f"Supported dtypes are {supported_high_precision_dtypes}."
        )
    # output dtype defaulting (mx_gemm.py:97-112)
    if output_quant:
        if out_dtype is None:
            out_dtype = left_dtype
        elif out_dtype not in supported_fp8_dtypes:
            raise ValueError(
                f"Unsupported output dtype {out_dtype}. Supported dtypes are {supported_fp8_dtypes}."
            )
    else:
        if out_dtype is None:
            out_dtype = torch.bfloat16
        elif out_dtype not in supported_fp16_dtypes:
            raise ValueError(
                f"Unsupported output dtype {out_dtype}. Supported dtypes are {supported_fp16_dtypes}."
            )
    # shapes (mx_gemm.py:117-144)
    if len(left_size) != 2 or len(right_size) != 2 or left_size[1] != right_size[0]:
        raise ValueError(
            f"Left tensor shape {left_size} and right tensor shape {right_size} are incompatible "
            "for matrix multiplication."
        )
    m, n, k = left_size[0], right_size[1], left_size[1]
    if len(left_scale_size) != 2 or len(right_scale_size) != 2 or left_scale_size[1] != right_scale_size[0]:
        raise ValueError(
            f"Left scale shape {left_scale_size} and right scale shape {right_scale_size} are incompatible."
        )
    if (
        min(m, n, k) <= 0
        or min(left_scale_size) <= 0
        or min(right_scale_size) <= 0
        or m % left_scale_size[0] != 0
        or n % right_scale_size[1] != 0
        or k % left_scale_size[1] != 0
    ):
        raise ValueError(
            f"Left scale shape {left_scale_size} and right scale shape {right_scale_size} "
            f"do not divide m ({m}) and n ({n})."
        )
    sm, sn, sk = m // left_scale_size[0], n // right_scale_size[1], k // left_scale_size[1]
    # output quantisation (mx_gemm.py:146-158)
    if output_quant:
        if quant_size is None:
            raise ValueError("quant_size must be provided when output_quant is True.")
        if (
            len(quant_size) != 2
            or quant_size[0] <= 0
            or quant_size[1] <= 0
            or m % quant_size[0] != 0
            or n % quant_size[1] != 0
        ):
            raise ValueError(
                f"Invalid quant_size {quant_size}. It must be a tuple of two integers "
                f"that divide m ({m}) and n ({n})."
            )
        qm, qn = int(quant_size[0]), int(quant_size[1])
        # The reference has templates only for 1 x {16, 32, 64, 128} groups and refuses QM > 1 when the kernel
        # is compiled (generator.py:971-974); here QM may also be a power of two up to 128 (two-dimensional
        # blocks, e.g. [128, 128] or [32, 32]).
        if qm > 128 or (qm & (qm - 1)) or qn not in (16, 32, 64, 128):
            raise ValueError(
                f"No matching kernel for quant_size {tuple(quant_size)}: blocks must be [QM, QN] with QN in "
                "(16, 32, 64, 128) and QM a power of two up to 128."
            )
    else:
        qm, qn = 0, 0  # a quant_size passed without output_quant is accepted and ignored
    # Layouts (mx_gemm.py:50-58). The reference's templates match only a row-major left and a column-major right
    # (mxblas/gemm/template.py:70-73, "No matching template" otherwise); here a column-major left (the .T view of
    # a [K, M] tensor) and a row-major right (a [K, N] tensor as stored) are accepted as well: the operand
    # layouts of a backward pass (dX = dY . W, dW = dY^T . X).
    for stride in (left_stride, right_stride, left_scale_stride, right_scale_stride):
        assert stride[0] == 1 or stride[1] == 1, "You should not reach here, stride is not valid."
    left_col_major = not _is_row_major(left_stride, left_size)
    right_row_major = not _is_col_major(right_stride, right_size)
    if left_col_major:
        lda, lda_min = (left_stride[1] if k > 1 else max(left_stride[1], m)), m
    else:
        lda, lda_min = (left_stride[0] if m > 1 else max(left_stride[0], k)), k
    if right_row_major:
        ldb, ldb_min = (right_stride[0] if k > 1 else max(right_stride[0], n)), n
    else:
        ldb, ldb_min = (right_stride[1] if n > 1 else max(right_stride[1], k)), k
    if lda % 16 != 0 or ldb % 16 != 0 or lda < lda_min or ldb < ldb_min or \
            (k % 16 != 0 and not (left_col_major and right_row_major)):
        raise ValueError(
            f"No matching kernel: K ({k}) and the row pitches of left ({lda}) and right ({ldb}) "
            "must be multiples of 16 bytes (TMA)."
        )
    if sk != k and sk % 32 != 0:
        raise ValueError(f"No matching kernel: the K extent of a scale block ({sk}) must be a multiple of 32.")
    return _Meta(
        m, n, k, sm, sn, sk, qm, qn, left_dtype, out_dtype, left_scale_dtype, bool(output_quant),
        bool(out_transpose), bool(out_scale_transpose), lda, ldb,
        left_scale_stride[0], left_scale_stride[1], right_scale_stride[1], right_scale_stride[0],
        left_col_major, right_row_major,
    )  # fmt: skip


def make_problem(meta: _Meta, ldc: int, ldcs: int, out_scale_pow2: bool, pow2_scales: Optional[bool]) -> MxbProblem:
    flags = 0
    if meta.quant:
        flags |= _ext.MXB_OUT_QUANT
    if meta.out_transpose:
        flags |= _ext.MXB_OUT_TRANSPOSE
    if meta.out_scale_transpose:
        flags |= _ext.MXB_OUT_SCALE_TRANSPOSE
    if out_scale_pow2:
        flags |= _ext.MXB_OUT_SCALE_POW2
    if pow2_scales is True:
        flags |= _ext.MXB_IN_SCALES_POW2
    elif pow2_scales is None:
        flags |= _ext.MXB_IN_SCALES_PROBE
    if meta.left_col_major:
        flags |= _ext.MXB_LEFT_COL_MAJOR
    if meta.right_row_major:
        flags |= _ext.MXB_RIGHT_ROW_MAJOR
    return MxbProblem(
        meta.m, meta.n, meta.k, meta.sm, meta.sn, meta.sk, meta.qm, meta.qn,
        _DTYPE_CODE[meta.in_dtype], _DTYPE_CODE[meta.out_dtype], _DTYPE_CODE[meta.scale_dtype], flags,
        meta.lda, meta.ldb, meta.as_rs, meta.as_ks, meta.bs_rs, meta.bs_ks, ldc, ldcs,
    )  # fmt: skip


# Scratch for re-packed scale factors and split-K partial sums, from torch's caching allocator.
# One buffer per (device, stream): launches on one stream are ordered, so they can share it. The
# library keeps the buffer's counters zero between calls, so it is zero-filled once, at creation.
_workspaces: dict = {}


def _workspace(device: torch.device, stream: int, nbytes: int) -> torch.Tensor:
    key = (device.index if device.index is not None else torch.cuda.current_device(), stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


_tune = None


def _tune_module():
    global _tune
    if _tune is None:
        from . import tune as _t

        _tune = _t
    return _tune


def reset_workspaces() -> None:
    """Drop all scratch buffers (after a device-side error they may hold stale split-K counters)."""
    _workspaces.clear()


def mx_gemm_kernel(
    left: torch.Tensor,
    right: torch.Tensor,
    left_scale: torch.Tensor,
    right_scale: torch.Tensor,
    output_quant: bool = False,
    quant_size: Optional[torch.Size] = None,
    out_dtype: Optional[torch.dtype] = None,
    out_transpose: bool = False,
    out_scale_transpose: bool = False,
    *,
    out_scale_pow2: bool = False,
    pow2_scales: Optional[bool] = None,
    config: Optional[MxbConfig] = None,
    _into=None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """FP8 micro-scaled GEMM with optional fused group quantisation of the result.

    Args follow mxblas/jit_kernels/mx_gemm.py:340-378: ``left`` [M, K] fp8 row-major, ``right``
    [K, N] fp8 column-major view (``b.T`` of a [N, K] tensor) -- the one layout pair the reference has kernels
    for -- or, beyond the reference, ``left`` column-major (``a.T`` of a [K, M] tensor) and / or ``right``
    row-major (a [K, N] tensor as stored), ``left_scale`` [M/SM, K/SK],
    ``right_scale`` [K/SK, N/SN] in fp16/bf16/fp32. Returns ``(C, C_scale)``; ``C_scale`` has the
    dtype of the input scales and is a 0-dim empty tensor when ``output_quant`` is False.

    ``quant_size`` [QM, QN]: QM = 1 as in the reference, or a power of two up to 128 for two-dimensional
    blocks (``C_scale`` is then [M/QM, N/QN]).

    ``out_transpose=True`` returns C^T as a contiguous [N, M] tensor and ``out_scale_transpose=True``
    returns C_scale^T as a contiguous [N/QN, M/QM] tensor (the reference declares both flags but has
    no kernel for them: mxblas/gemm/generator.py:933-936, mxblas/gemm/template.py:74).
    """
    if not left.is_cuda:
        raise ValueError("mx_gemm_kernel needs CUDA tensors (there is no CPU implementation).")
    meta = get_meta_info(
        left.dtype, right.dtype, left_scale.dtype, right_scale.dtype, bool(output_quant),
        None if quant_size is None else tuple(quant_size), out_dtype,
        tuple(left.shape), tuple(right.shape), tuple(left_scale.shape), tuple(right_scale.shape),
        tuple(left.stride()), tuple(right.stride()), tuple(left_scale.stride()), tuple(right_scale.stride()),
        bool(out_transpose), bool(out_scale_transpose),
    )  # fmt: skip
    dev = left.device
    m, n = meta.m, meta.n
    if _into is not None:
        # N-sharded runs (mxblas_b200.dist): the caller supplies the views to write, this rank's block of the
        # full result and of its scales
        out, out_scale = _into
        ldcs = out_scale.stride(0) if meta.quant else 0
    else:
        # outputs (mx_gemm.py:301-325)
        out = torch.empty((n, m) if meta.out_transpose else (m, n), dtype=meta.out_dtype, device=dev)
        if meta.quant:
            g, mb = n // meta.qn, m // meta.qm
            out_scale = torch.empty((g, mb) if meta.out_scale_transpose else (mb, g), dtype=meta.scale_dtype,
                                    device=dev)
            ldcs = out_scale.stride(0)
        else:
            out_scale = torch.empty([], dtype=meta.scale_dtype, device=dev)
            ldcs = 0
    problem = make_problem(meta, out.stride(0), ldcs, out_scale_pow2, pow2_scales)
    if config is None:
        # tuned plans (mxblas/gemm/kernel_pool.py:85-89 keeps its winners in memory only; here they persist)
        tune = _tune_module()
        if tune.USE_TABLES:
            config = tune.plan_for(meta, out_scale_pow2, pow2_scales)
            if config is None and tune.ENABLED and not torch.cuda.is_current_stream_capturing():
                key = tune.table_key(meta, out_scale_pow2, pow2_scales)
                if key not in tune._load_table():
                    tune.autotune(
                        left, right, left_scale, right_scale, output_quant, quant_size, out_dtype, out_transpose,
                        out_scale_transpose, out_scale_pow2=out_scale_pow2, pow2_scales=pow2_scales)
                    config = tune.plan_for(meta, out_scale_pow2, pow2_scales)
    cfg_ptr = ctypes.byref(config) if config is not None else None
    # Host time per call matters for the small problems (a decode step's kernel takes 20-40 us): the raw
    # stream handle instead of a Stream object, no device guard when the device is already current, and the
    # stream's scratch buffer handed over as it is; its size is only queried when the library asks for more.
    dev_index = dev.index if dev.index is not None else torch.cuda.current_device()
    stream = torch._C._cuda_getCurrentRawStream(dev_index)
    ws = _workspaces.get((dev_index, stream))
    if ws is None:
        ws = _workspace(dev, stream, 0)
    args = (ctypes.byref(problem), cfg_ptr, left.data_ptr(), right.data_ptr(), out.data_ptr(),
            left_scale.data_ptr(), right_scale.data_ptr(), out_scale.data_ptr() if meta.quant else None)
    launch = _ext.lib.mxb_gemm_cfg
    switch = torch.cuda.current_device() != dev_index
    if switch:
        prev = torch.cuda.current_device()
        torch.cuda.set_device(dev_index)
    try:
        st = launch(*args, ws.data_ptr(), ws.numel(), stream)
        if st == _ext.MXB_ERR_WORKSPACE:
            nbytes = ctypes.c_size_t(0)
            st = _ext.lib.mxb_query_workspace(ctypes.byref(problem), cfg_ptr, ctypes.byref(nbytes))
            if st == _ext.MXB_OK:
                ws = _workspace(dev, stream, nbytes.value)
                st = launch(*args, ws.data_ptr(), ws.numel(), stream)
    finally:
        if switch:
            torch.cuda.set_device(prev)
    if st in (_ext.MXB_ERR_INVALID, _ext.MXB_ERR_UNSUPPORTED):
        raise ValueError(f"No matching kernel ({_ext.status_text(st)}) for {meta}")
    if st != _ext.MXB_OK:
        raise RuntimeError("mx_gemm_kernel: " + _ext.status_text(st))
    return out, out_scale


class _RegisterState:
    def __init__(self):
        self.registered = False

    def is_registered(self) -> bool:
        return self.registered


register_state = _RegisterState()


def register_all_kernels() -> None:
    """Make every kernel available. Idempotent.

    The reference imports its template modules here (mx_gemm.py:449-457) and compiles kernels on
    first use; this build's kernels are compiled ahead of time, so the call only checks that the
    library is loaded and speaks the expected ABI.
    """
    if _ext.lib.mxb_abi_version() != 1:
        raise RuntimeError("libmxblas_b200.so: unexpected ABI version")
    register_state.registered = True
