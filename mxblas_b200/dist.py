"""N-sharded MX-GEMM over the GPUs of one node: one process per GPU, torch.distributed for plumbing.

The reference is single-GPU (no distributed code anywhere in its tree); this is the multi-GPU
form of the same operator. Output columns are independent, so the problem is cut along N:

    rank r owns   right[:, r*N/g : (r+1)*N/g]   (rows r*N/g.. of the physical [N, K] weight)
                  right_scale[:, matching column blocks]
    every rank has left and left_scale
    rank r computes C[:, r*N/g : (r+1)*N/g] and the matching columns of C_scale

The GEMM itself needs no communication. Only when the caller asks for the gathered result is there
one collective, an NCCL all-gather (NVLink / NVSwitch). With ``out_transpose=True`` the local
results are row blocks of C^T, so the all-gather writes the final tensor in place; row-major C is
gathered as [g, M, N/g] and re-laid out with one device copy.
"""

from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


def shard_bounds(n: int, world: int, rank: int, sn: int = 1, qn: int = 0) -> Tuple[int, int]:
    """Column range [n0, n1) of rank ``rank``. Slices are equal and must hold whole scale blocks
    (``sn`` columns) and whole output quantisation groups (``qn`` columns)."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"invalid rank {rank} of {world}")
    if n % world != 0:
        raise ValueError(f"N ({n}) is not divisible by the number of ranks ({world})")
    per = n // world
    if sn > n:
        raise ValueError(f"a scale block ({sn} columns) is wider than N ({n})")
    if sn < n and per % sn != 0:
        raise ValueError(f"N/ranks ({per}) does not hold whole scale blocks of {sn} columns")
    if qn and per % qn != 0:
        raise ValueError(f"N/ranks ({per}) does not hold whole quantisation groups of {qn} columns")
    if per % 16 != 0:
        raise ValueError(f"N/ranks ({per}) must be a multiple of 16")
    return rank * per, (rank + 1) * per


def shard_right(
    right: torch.Tensor, right_scale: torch.Tensor, world: int, rank: int, qn: int = 0
) -> Tuple[torch.Tensor, torch.Tensor]:
    """This rank's slice of the full ``right`` [K, N] (column-major view) and ``right_scale``
    [K/SK, N/SN]. Views, no copies: a column slice of the column-major view is a block of rows of
    the physical [N, K] tensor. A per-tensor scale ([1, 1]) is shared by all ranks."""
    n = right.shape[1]
    blocks = right_scale.shape[1]
    sn = n // blocks
    n0, n1 = shard_bounds(n, world, rank, sn, qn)
    if blocks == 1:
        return right[:, n0:n1], right_scale
    return right[:, n0:n1], right_scale[:, n0 // sn : n1 // sn]


def gather_columns(
    local: torch.Tensor, transposed: bool, group: Optional[dist.ProcessGroup] = None
) -> torch.Tensor:
    """All-gather per-rank column slices into the full matrix.

    ``transposed=False``: ``local`` is [M, N/g] (a column block of C)  -> returns C [M, N]
    ``transposed=True``:  ``local`` is [N/g, M] (a row block of C^T)   -> returns C^T [N, M]
    """
    world = dist.get_world_size(group)
    local = local.contiguous()
    if world == 1:
        return local
    rows, cols = local.shape
    if transposed:
        full = torch.empty((world * rows, cols), dtype=local.dtype, device=local.device)
        _all_gather_bytes(full, local, group)
        return full
    stacked = torch.empty((world * rows, cols), dtype=local.dtype, device=local.device)
    _all_gather_bytes(stacked, local, group)
    # [g, M, N/g] -> [M, g, N/g] -> [M, N]
    return stacked.view(world, rows, cols).permute(1, 0, 2).reshape(rows, world * cols)


def _all_gather_bytes(full: torch.Tensor, local: torch.Tensor, group) -> None:
    # collectives do not know the fp8 dtypes: move raw bytes
    if local.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
        dist.all_gather_into_tensor(full.view(torch.uint8), local.view(torch.uint8), group=group)
    else:
        dist.all_gather_into_tensor(full, local, group=group)


def sharded_mx_gemm(
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
    group: Optional[dist.ProcessGroup] = None,
    gather=False,
    right_is_local: bool = False,
    compute: Optional[Callable] = None,
    **kwargs,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """``mx_gemm_kernel`` over all ranks of ``group``, sharded along N.

    ``right`` / ``right_scale`` are the full tensors (each rank slices its own columns) unless
    ``right_is_local`` says they already are this rank's shard. Returns this rank's column block of
    the result, or, with ``gather=True``, the full result on every rank (one NCCL all-gather per
    output tensor). ``gather="peer"`` produces the same full result without a collective: the result lives in
    symmetric memory, each rank's GEMM writes its column block of its own copy and the block is then pushed
    into every other rank's copy (plain stores over NVLink from a copy kernel, or the copy engines with
    ``peer_transport="dma"``), at its place in the final layout, followed by one cross-rank barrier on the
    stream. Large row-major results are produced in row chunks (``peer_chunks``), the push of one chunk running
    under the GEMM of the next. Column blocks that are not 16-byte aligned take the all-gather instead. The
    tensors returned are views of buffers that the next ``gather="peer"`` call of the same shape reuses.
    ``compute`` replaces the local GEMM (tests run the host logic on CPU ranks).
    """
    if compute is None:
        from .mx_gemm import mx_gemm_kernel as compute  # the CUDA path; fails without the library
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    qn = int(quant_size[1]) if (output_quant and quant_size is not None) else 0
    if not right_is_local:
        right, right_scale = shard_right(right, right_scale, world, rank, qn)
    if gather == "peer" and world > 1:
        return _peer_gathered(left, right, left_scale, right_scale, output_quant, quant_size, out_dtype,
                              out_transpose, out_scale_transpose, group, world, rank, compute, kwargs)
    out, out_scale = compute(
        left, right, left_scale, right_scale, output_quant, quant_size, out_dtype, out_transpose,
        out_scale_transpose, **kwargs,
    )  # fmt: skip
    if gather and world > 1:
        out = gather_columns(out, out_transpose, group)
        if output_quant:
            out_scale = gather_columns(out_scale, out_scale_transpose, group)
    return out, out_scale


_peer_cache: dict = {}


def _symmetric(shape, dtype, group, tag):
    """A cached symmetric-memory tensor (same size on every rank) and its rendezvous handle."""
    import torch.distributed._symmetric_memory as symm_mem

    key = (tag, tuple(shape), dtype, id(group))
    hit = _peer_cache.get(key)
    if hit is None:
        nbytes = max(1, int(torch.empty((), dtype=dtype).element_size()))
        for d in shape:
            nbytes *= int(d)
        raw = symm_mem.empty(nbytes, dtype=torch.uint8, device=torch.device("cuda", torch.cuda.current_device()))
        hdl = symm_mem.rendezvous(raw, group if group is not None else dist.group.WORLD)
        hit = (raw.view(dtype).view(*shape), hdl)
        _peer_cache[key] = hit
    return hit


def _push(block: torch.Tensor, full: torch.Tensor, hdl, world: int, rank: int, dma: bool = False,
          max_blocks: int = 0) -> None:
    """This rank's block (a view of its symmetric tensor ``full``) into the same place of every peer's copy, on
    the current stream: by a copy kernel (stores over NVLink; ``max_blocks`` bounds its grid) or, with ``dma``,
    by the copy engines."""
    import ctypes

    from . import _ext

    off = block.data_ptr() - full.data_ptr()
    peers = [int(hdl.buffer_ptrs[r]) + off for r in range(world) if r != rank]
    esz = block.element_size()
    ptrs = (ctypes.c_void_p * len(peers))(*peers)
    stream = torch._C._cuda_getCurrentRawStream(block.device.index)
    geom = (block.data_ptr(), block.stride(0) * esz, ptrs, len(peers), block.stride(0) * esz, block.shape[0],
            block.shape[1] * esz)
    if dma:
        st = _ext.lib.mxb_push_block_dma(*geom, stream)
    else:
        st = _ext.lib.mxb_push_block_ex(*geom, max_blocks, stream)
    if st != _ext.MXB_OK:
        raise RuntimeError("mxb_push_block: " + _ext.status_text(st))


def _pushable(block: torch.Tensor) -> bool:
    esz = block.element_size()
    return (block.shape[1] * esz) % 16 == 0 and (block.stride(0) * esz) % 16 == 0 and block.data_ptr() % 16 == 0


_side_streams: dict = {}


def _side_stream(device: torch.device) -> torch.cuda.Stream:
    s = _side_streams.get(device.index)
    if s is None:
        s = _side_streams[device.index] = torch.cuda.Stream(device=device)
    return s


def peer_row_chunks(m: int, sm: int, out_transpose: bool, transposed_scales: bool, want: Optional[int] = None,
                    flops: float = 0.0, push_bytes: float = 0.0) -> int:
    """Into how many row chunks of ``left`` a gather="peer" call is cut so that the push of one chunk's result
    runs under the GEMM of the next. Chunks hold whole 256-row tiles and whole scale blocks; a chunk must keep
    the GPU busy for about 100 us (its GEMM at ~2.5 PFLOP/s or its push at ~600 GB/s, whichever is longer),
    because every chunk costs the host two enqueues and an event: measured on B200, 8192^3 on two GPUs in four
    48-us chunks ran 9 % slower than unchunked, 16384 x 28672 x 8192 in eight 170-us chunks 17 % faster.
    At most 8 chunks; one chunk for transposed results (a row chunk of left is a column strip of C^T, too
    narrow to store or push efficiently)."""
    if out_transpose or transposed_scales:
        return 1
    if want:
        chunks = want
    else:
        busy = max(flops / 2.5e15, push_bytes / 6e11)
        chunks = int(min(8, busy / 100e-6))
    while chunks > 1:
        mc = m // chunks
        if m % chunks == 0 and mc % 256 == 0 and (sm == m or mc % sm == 0):
            break
        chunks -= 1
    return max(chunks, 1)


def _peer_gathered(left, right, left_scale, right_scale, output_quant, quant_size, out_dtype, out_transpose,
                   out_scale_transpose, group, world, rank, compute, kwargs):
    m, nl = left.shape[0], right.shape[1]
    n = nl * world
    odt = out_dtype or (left.dtype if output_quant else torch.bfloat16)
    full, hdl = _symmetric((n, m) if out_transpose else (m, n), odt, group, "out")
    n0 = rank * nl
    mine = full[n0 : n0 + nl] if out_transpose else full[:, n0 : n0 + nl]
    sc_full = sc_hdl = None
    if output_quant:
        g, gl = n // int(quant_size[1]), nl // int(quant_size[1])
        sc_full, sc_hdl = _symmetric((g, m) if out_scale_transpose else (m, g), left_scale.dtype, group, "scale")
        g0 = rank * gl
        sc_mine = sc_full[g0 : g0 + gl] if out_scale_transpose else sc_full[:, g0 : g0 + gl]
    else:
        sc_mine = torch.empty([], dtype=left_scale.dtype, device=left.device)
    # the alignment rule of the push is a property of the shapes: decided before anything is enqueued, the
    # same on every rank, so an unaligned problem takes the all-gather everywhere
    if not (_pushable(mine) and (not output_quant or _pushable(sc_mine))):
        out, out_scale = compute(left, right, left_scale, right_scale, output_quant, quant_size, out_dtype,
                                 out_transpose, out_scale_transpose, **kwargs)
        out = gather_columns(out, out_transpose, group)
        if output_quant:
            out_scale = gather_columns(out_scale, out_scale_transpose, group)
        return out, out_scale
    kwargs = dict(kwargs)
    dma = kwargs.pop("peer_transport", "sm") == "dma"
    sm_rows = m // left_scale.shape[0]
    out_bytes = m * nl * mine.element_size() + (sc_mine.numel() * sc_mine.element_size() if output_quant else 0)
    chunks = peer_row_chunks(m, sm_rows, out_transpose, output_quant and out_scale_transpose,
                             kwargs.pop("peer_chunks", None), 2.0 * m * nl * left.shape[1], (world - 1) * out_bytes)
    hdl.barrier(channel=0)  # every rank is done with the previous contents of the buffers
    if chunks == 1:
        compute(left, right, left_scale, right_scale, output_quant, quant_size, out_dtype, out_transpose,
                out_scale_transpose, _into=(mine, sc_mine), **kwargs)
        _push(mine, full, hdl, world, rank, dma)
        if output_quant:
            _push(sc_mine, sc_full, sc_hdl, world, rank, dma)
    else:
        # Row chunks: the GEMM of chunk i+1 runs on the caller's stream while chunk i's block crosses NVLink on a
        # side stream. The copy kernel needs SMs of its own (a persistent GEMM CTA fills an SM's registers and
        # shared memory), so the GEMMs run on all SMs but `reserve`; the copy engines need none.
        main = torch.cuda.current_stream()
        side = _side_stream(left.device)
        if not dma and "config" not in kwargs:
            from ._ext import MxbConfig

            sms = torch.cuda.get_device_properties(left.device).multi_processor_count
            kwargs["config"] = MxbConfig(0, -1, 0, 0, 0, (sms - PEER_PUSH_SMS) & ~1, 0)
        mc = m // chunks
        for i in range(chunks):
            r0, r1 = i * mc, (i + 1) * mc
            ls_i = left_scale if sm_rows == m else left_scale[r0 // sm_rows : r1 // sm_rows]
            blk = mine[r0:r1]
            sc_blk = sc_mine[r0:r1] if output_quant else sc_mine
            compute(left[r0:r1], right, ls_i, right_scale, output_quant, quant_size, out_dtype, False,
                    False, _into=(blk, sc_blk), **kwargs)
            done = torch.cuda.Event()
            done.record(main)
            side.wait_event(done)
            with torch.cuda.stream(side):
                _push(blk, full, hdl, world, rank, dma, 8 * PEER_PUSH_SMS)
                if output_quant:
                    _push(sc_blk, sc_full, sc_hdl, world, rank, dma, 8 * PEER_PUSH_SMS)
        main.wait_stream(side)
    hdl.barrier(channel=1)  # every rank's block has landed everywhere
    return full, (sc_full if output_quant else sc_mine)


PEER_PUSH_SMS = 20  # SMs left to the copy kernel while a chunked gather="peer" call's GEMMs run


if __name__ == "__main__":
    from .bench_configs import dist_main

    dist_main()
