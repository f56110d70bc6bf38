"""Grouped MX-GEMM: one call for the expert layers of a mixture-of-experts model.

    out[r] = left[r] @ right[g(r)]        g(r) = group_of_block[r // block_rows]

``left`` [M, K] holds the tokens sorted by expert and padded so that every block of ``block_rows`` (128 or 256)
rows belongs to one expert; ``right`` is [G, K, N], the column-major views of G weights stored as [G, N, K]
(``w.transpose(1, 2)``), ``right_scale`` [G, K/SK, N/SN] likewise (``w_scales.transpose(1, 2)``). Scaling
patterns, output quantisation and the extensions are those of ``mx_gemm_kernel``.

The reference has no grouped or batched form (its operator is one dense GEMM,
mxblas/jit_kernels/mx_gemm.py:340-425); the natural caller is the same FP8 layer stack it serves, with
expert weights. One persistent launch covers all groups: a tile looks its group up from the block table and
reads that group's rows of the stacked weight.
"""

from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import _ext
from ._ext import MxbConfig
from .mx_gemm import _workspace, get_meta_info, make_problem


def mx_grouped_gemm(
    left: torch.Tensor,
    right: torch.Tensor,
    left_scale: torch.Tensor,
    right_scale: torch.Tensor,
    group_of_block: torch.Tensor,
    output_quant: bool = False,
    quant_size: Optional[torch.Size] = None,
    out_dtype: Optional[torch.dtype] = None,
    *,
    block_rows: int = 128,
    out_scale_pow2: bool = False,
    pow2_scales: Optional[bool] = None,
    config: Optional[MxbConfig] = None,
    out: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns ``(C [M, N], C_scale)`` as ``mx_gemm_kernel`` does. Rows of blocks whose entry in
    ``group_of_block`` is negative are not computed (they keep the contents of ``out`` if one is passed)."""
    if not left.is_cuda:
        raise ValueError("mx_grouped_gemm needs CUDA tensors (there is no CPU implementation).")
    if right.dim() != 3 or right_scale.dim() != 3 or right.shape[0] != right_scale.shape[0]:
        raise ValueError("right must be [G, K, N] and right_scale [G, K/SK, N/SN]")
    groups = right.shape[0]
    if block_rows not in (128, 256) or left.shape[0] % block_rows:
        raise ValueError(f"block_rows must be 128 or 256 and divide M ({left.shape[0]})")
    if group_of_block.dtype != torch.int32 or group_of_block.numel() != left.shape[0] // block_rows or \
            not group_of_block.is_cuda or not group_of_block.is_contiguous():
        raise ValueError("group_of_block must be a contiguous CUDA int32 tensor with M / block_rows entries")
    meta = get_meta_info(
        left.dtype, right.dtype, left_scale.dtype, right_scale.dtype, bool(output_quant),
        None if quant_size is None else tuple(quant_size), out_dtype,
        tuple(left.shape), tuple(right.shape[1:]), tuple(left_scale.shape), tuple(right_scale.shape[1:]),
        tuple(left.stride()), tuple(right.stride()[1:]), tuple(left_scale.stride()), tuple(right_scale.stride()[1:]),
        False, False,
    )  # fmt: skip
    if meta.left_col_major or meta.right_row_major:
        raise ValueError("No matching kernel: grouped GEMM takes a row-major left and [G, N, K] weights")
    if groups > 1 and (right.stride(0) != meta.n * meta.ldb or
                       right_scale.stride(0) != (meta.n // meta.sn) * meta.bs_rs):
        raise ValueError("the groups' weights and scales must be stacked densely")
    dev = left.device
    m, n = meta.m, meta.n
    if out is None:
        out = torch.empty((m, n), dtype=meta.out_dtype, device=dev)
    if meta.quant:
        out_scale = torch.empty((m // meta.qm, n // meta.qn), dtype=meta.scale_dtype, device=dev)
        ldcs = out_scale.stride(0)
    else:
        out_scale = torch.empty([], dtype=meta.scale_dtype, device=dev)
        ldcs = 0
    problem = make_problem(meta, out.stride(0), ldcs, out_scale_pow2, pow2_scales)
    cfg_ptr = ctypes.byref(config) if config is not None else None
    dev_index = dev.index if dev.index is not None else torch.cuda.current_device()
    stream = torch._C._cuda_getCurrentRawStream(dev_index)
    nbytes = ctypes.c_size_t(0)
    st = _ext.lib.mxb_grouped_query_workspace(ctypes.byref(problem), cfg_ptr, groups, block_rows, ctypes.byref(nbytes))
    if st == _ext.MXB_OK:
        ws = _workspace(dev, stream, nbytes.value)
        with torch.cuda.device(dev_index):
            st = _ext.lib.mxb_grouped_gemm(
                ctypes.byref(problem), cfg_ptr, groups, group_of_block.data_ptr(), block_rows, left.data_ptr(),
                right.data_ptr(), out.data_ptr(), left_scale.data_ptr(), right_scale.data_ptr(),
                out_scale.data_ptr() if meta.quant else None, ws.data_ptr(), ws.numel(), stream)
    if st in (_ext.MXB_ERR_INVALID, _ext.MXB_ERR_UNSUPPORTED):
        raise ValueError(f"No matching kernel ({_ext.status_text(st)}) for grouped {meta}")
    if st != _ext.MXB_OK:
        raise RuntimeError("mx_grouped_gemm: " + _ext.status_text(st))
    return out, out_scale
