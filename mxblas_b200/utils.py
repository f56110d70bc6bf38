"""Helpers users of the reference import from ``mxblas.utils``: quantise / dequantise reference
math, the similarity metric, a synthetic-data generator and GPU timers.

Same names and argument meaning as mxblas/utils.py of the reference (block_quant :66-93,
block_dequant :100-116, per_tensor_quant :54-59, calc_diff :39-43, gaussian_with_channel_outlier
:123-144, GPU_bench :325-349, CPU_bench :352-363, check_nan_inf :17-19). These are conveniences for
callers and tests; the GEMM itself never goes through them.
"""

from __future__ import annotations

import contextlib
import os
import sys
import time
import warnings

import torch

FP8_E4M3_MAX = 448.0


def nan_nums(x: torch.Tensor) -> int:
    return int(torch.isnan(x).sum().item())


def inf_nums(x: torch.Tensor) -> int:
    return int(torch.isinf(x).sum().item())


def check_nan_inf(x: torch.Tensor) -> None:
    nans, infs = nan_nums(x), inf_nums(x)
    if nans or infs:
        warnings.warn(f"with {nans} nans and {infs} infs")


def calc_diff(x: torch.Tensor, y: torch.Tensor, dtype=torch.float) -> torch.Tensor:
    """1 - 2<x,y> / (|x|^2 + |y|^2): 0 for identical tensors."""
    x, y = x.to(dtype), y.to(dtype)
    return 1 - 2 * (x * y).sum() / (x * x + y * y).sum()


def relative_error(value: torch.Tensor, real: torch.Tensor, exclude_zeros: bool = True) -> float:
    value, real = value.double().flatten(), real.double().flatten()
    if exclude_zeros:
        keep = ~((real == 0) | real.isinf() | value.isinf())
        value, real = value[keep], real[keep]
        return ((value - real).abs() / real.abs()).mean().item()
    return ((value - real).abs() / (real.abs() + 1e-9)).mean().item()


def round_quant(x: torch.Tensor, lfp_t=torch.float8_e4m3fn) -> torch.Tensor:
    """Plain cast to FP8, no scale (mxblas/utils.py:46-47)."""
    return x.to(lfp_t)


def round_dequant(x: torch.Tensor, hfp_t=torch.float16) -> torch.Tensor:
    return x.to(hfp_t)


def block_quantv1(x: torch.Tensor, blk_shape, lfp_t=torch.float8_e4m3fn) -> torch.Tensor:
    """The reference's first block quantiser (mxblas/utils.py:96-97): a cast that ignores the block shape."""
    return x.to(lfp_t)


def per_tensor_quant(x: torch.Tensor, lfp_t=torch.float8_e4m3fn, scale_fp_t=torch.float32):
    scale = x.abs().max() / FP8_E4M3_MAX
    return (x / scale).to(lfp_t), scale.to(scale_fp_t)


def per_tensor_dequant(x: torch.Tensor, scale: torch.Tensor, hfp_t=torch.float16):
    return x.to(hfp_t) * scale


def _to_blocks(x: torch.Tensor, bm: int, bn: int) -> torch.Tensor:
    """[M, N] -> [M/bm, N/bn, bm*bn]"""
    m, n = x.shape
    return x.reshape(m // bm, bm, n // bn, bn).permute(0, 2, 1, 3).reshape(m // bm, n // bn, bm * bn)


def _from_blocks(xb: torch.Tensor, bm: int, bn: int) -> torch.Tensor:
    qm, qn, _ = xb.shape
    return xb.reshape(qm, qn, bm, bn).permute(0, 2, 1, 3).reshape(qm * bm, qn * bn)


def block_quant(x: torch.Tensor, blk_shape, lfp_t=torch.float8_e4m3fn):
    """Quantise ``x`` in blocks of ``blk_shape``: scale = amax / 448 (1 for an all-zero block),
    values clamped to +-448 before the cast. Returns (fp8 tensor, fp32 scales [M/bm, N/bn])."""
    bm, bn = blk_shape
    assert x.dim() == 2 and x.size(0) % bm == 0 and x.size(1) % bn == 0
    xb = _to_blocks(x, bm, bn)
    scales = xb.abs().amax(dim=2, keepdim=True) / FP8_E4M3_MAX
    scales = torch.where(scales == 0, torch.ones_like(scales), scales)
    q = _from_blocks((xb / scales).clamp(-FP8_E4M3_MAX, FP8_E4M3_MAX), bm, bn).to(lfp_t)
    return q, scales.reshape(scales.shape[0], scales.shape[1]).to(torch.float32)


def block_dequant(x: torch.Tensor, scales: torch.Tensor, blk_shape, hfp_t=torch.float16):
    bm, bn = blk_shape
    qm, qn = scales.shape
    assert x.size(0) == qm * bm and x.size(1) == qn * bn
    return _from_blocks(_to_blocks(x.to(hfp_t), bm, bn) * scales.reshape(qm, qn, 1), bm, bn)


def gaussian(size, mean=0, std=1, dtype=torch.float16, device=None):
    device = device if device is not None else torch.device("cuda:0")
    return torch.normal(mean, std, size=size, device=device, dtype=dtype)


def gaussian_with_channel_outlier(
    size, dim: int, outlier_ratio=0.01, g_mean=0, g_std=1, o_mean=0, o_std=100, dtype=torch.bfloat16, device=None
):
    """Gaussian tensor in which a random ``outlier_ratio`` of the slices along ``dim`` is drawn
    with the (much wider) outlier distribution, the activation statistics FP8 recipes care about."""
    device = device if device is not None else torch.device("cuda:0")
    x = gaussian(size, g_mean, g_std, dtype=dtype, device=device)
    count = int(x.size(dim) * outlier_ratio)
    picks = torch.randperm(x.size(dim), device=device)[:count]
    shape = [count if i == dim else x.size(i) for i in range(x.ndim)]
    x.index_copy_(dim, picks, gaussian(shape, o_mean, o_std, dtype=dtype, device=device))
    return x


class DurationTimer:
    """``with DurationTimer() as t: ...`` then ``t.get_duration()`` in milliseconds (CUDA events on the
    current stream; mxblas/utils.py:147-187). ``cond=False`` turns it into a no-op."""

    def __init__(self, cond: bool = True, device=None, is_sync: bool = True):
        self.cond = cond
        self.device = device if device is not None else torch.cuda.current_device()
        self.is_sync = is_sync
        self.duration = None

    def __enter__(self):
        if self.cond:
            self.start = torch.cuda.Event(enable_timing=True)
            self.end = torch.cuda.Event(enable_timing=True)
            self.start.record()
        return self

    def __exit__(self, *exc):
        if self.cond:
            self.end.record()
            if self.is_sync:
                self.sync()
        return False

    def sync(self):
        if self.cond:
            torch.cuda.synchronize(self.device)
            self.duration = self.start.elapsed_time(self.end)
        return self

    def get_duration(self) -> float:
        if self.duration is None:
            self.sync()
        return self.duration


class empty_suppress(contextlib.nullcontext):
    pass


class suppress_stdout_stderr:
    """Send this process's stdout and stderr (file descriptors included, so native code too) to
    /dev/null inside the block."""

    def __enter__(self):
        sys.stdout.flush()
        sys.stderr.flush()
        self._null = os.open(os.devnull, os.O_WRONLY)
        self._saved = [(fd, os.dup(fd)) for fd in (1, 2)]
        for fd, _ in self._saved:
            os.dup2(self._null, fd)
        return self

    def __exit__(self, *exc):
        sys.stdout.flush()
        sys.stderr.flush()
        for fd, keep in self._saved:
            os.dup2(keep, fd)
            os.close(keep)
        os.close(self._null)
        return False


def bench_kineto(fn, kernel_names, num_tests: int = 30, suppress_kineto_output: bool = False,
                 trace_path: str = None, barrier_comm_profiling: bool = False, flush_l2: bool = False):
    """Mean device time in SECONDS of the kernel(s) whose name contains ``kernel_names`` (a string, or a
    tuple of strings -> tuple of times), taken from the torch profiler's kernel records over ``num_tests``
    calls of ``fn`` (same contract as mxblas/utils.py:233-322, which parses the profiler's text table).
    Each name must match exactly one kernel. ``flush_l2`` rewrites 512 MB before every call."""
    fn()  # first call outside the profile: lazy initialisation, scratch allocation
    names = (kernel_names,) if isinstance(kernel_names, str) else tuple(kernel_names)
    quiet = suppress_stdout_stderr if suppress_kineto_output else empty_suppress
    with quiet():
        with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CUDA]) as prof:
            if barrier_comm_profiling:
                import torch.distributed as dist

                a = torch.randn((8192, 8192), dtype=torch.float, device="cuda")
                a @ a
                dist.all_reduce(torch.ones(1, dtype=torch.float, device="cuda"))
            for _ in range(num_tests):
                if flush_l2:
                    torch.empty(int(512e6 // 4), dtype=torch.int, device="cuda").zero_()
                fn()
            torch.cuda.synchronize()
    if trace_path is not None:
        prof.export_chrome_trace(trace_path)
    rows = prof.key_averages()
    times = []
    for name in names:
        hits = [r for r in rows if name in r.key and getattr(r, "device_time_total", 0) > 0]
        assert len(hits) == 1, f"kernel name {name!r} matches {len(hits)} profiled kernels"
        times.append(hits[0].device_time_total / hits[0].count * 1e-6)
    return times[0] if isinstance(kernel_names, str) else tuple(times)


def GPU_bench(func, iters=100, warmup=30, kernel_name=None, flush_l2: bool = False) -> float:
    """Mean time of ``func`` in milliseconds, CUDA events on the current stream.

    With ``kernel_name`` the time is that of the one kernel whose name contains it, from the torch
    profiler (``bench_kineto``), as in the reference. With ``flush_l2`` a 256 MiB buffer is rewritten before every call and each call is
    timed on its own.
    """
    if kernel_name is not None:
        return bench_kineto(func, kernel_name, num_tests=iters, suppress_kineto_output=True, flush_l2=flush_l2) * 1e3
    for _ in range(warmup):
        func()
    if not flush_l2:
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(iters):
            func()
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end) / iters
    junk = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    total = 0.0
    for _ in range(iters):
        junk.zero_()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        func()
        end.record()
        torch.cuda.synchronize()
        total += start.elapsed_time(end)
    return total / iters


def CPU_bench(func, iters=100, warmup=30) -> float:
    for _ in range(warmup):
        func()
    t0 = time.perf_counter()
    for _ in range(iters):
        func()
    return (time.perf_counter() - t0) * 1e3 / iters


def profiler_enter() -> None:
    """cudaProfilerStart: opens the capture range of an external profiler (mxblas/utils.py:366-369)."""
    torch.cuda.check_error(torch.cuda.cudart().cudaProfilerStart())


def profiler_exit() -> None:
    torch.cuda.check_error(torch.cuda.cudart().cudaProfilerStop())


class Profiler:
    def __enter__(self):
        profiler_enter()
        return self

    def __exit__(self, *exc):
        profiler_exit()
        return False


class WithNVTX:
    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        torch.cuda.nvtx.range_push(self.name)
        return self

    def __exit__(self, *exc):
        torch.cuda.nvtx.range_pop()
        return False
