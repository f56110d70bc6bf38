"""Tile / CTA-pair / split-K autotuner.

Stands where the reference has ``JITTuner.compile_and_tune`` (mxblas/jit/tuner.py:59-182), which
compiles every candidate of a 57 344-point space with nvcc and times it with kineto,
``build_tunning_space`` (mxblas/jit_kernels/mx_gemm.py:197-291) and the in-memory kernel pool
(mxblas/gemm/kernel_pool.py:79-186). Here every kernel variant is already in the library, a candidate
is just an ``MxbConfig``, a few dozen of them are timed with CUDA events, and the winner is persisted
(the reference re-tunes in every process).

Which plan a call without an explicit ``config`` gets:
  1. the entry of the user's table  MXBLAS_CACHE_DIR/autotune_<gpu>.json  for the problem's key
     (dtypes, M bucket, N, K, scale granularity, quantisation, flags), if there is one;
  2. else the entry of the table shipped with the package (mxblas_b200/tuned/<gpu>.json: the BASELINE
     shapes, tuned on a B200);
  3. else, with ``MXBLAS_B200_AUTOTUNE=1`` and outside a stream capture, the problem is tuned on the spot
     and the winner stored in the user's table;
  4. else the library's heuristic plan (choose_plan in csrc/mxb_host.cu).
``MXBLAS_B200_TABLES=0`` skips 1-3. The table is shared by all threads of the process behind one lock;
the file is replaced atomically, so concurrent processes never read a torn table.

``MXBLAS_PRINT_AUTO_TUNE=1`` prints every timed candidate and ``MXBLAS_PROFILING_TIME_PATH`` appends
them to a file, as in the reference. Command lines that time the BASELINE configurations live in
mxblas_b200/bench_configs.py (``python -m mxblas_b200.tune ...`` forwards there).
"""

from __future__ import annotations

import json
import os
import threading
from pathlib import Path
from typing import Callable, Iterable, List, Optional, Tuple

import torch

from . import _ext
from ._ext import MxbConfig
from .const import CACHE_DIR_FLAG, PRINT_AUTOTUNE_FLAG, PROFILING_TIME_PATH

ENABLED = os.environ.get("MXBLAS_B200_AUTOTUNE", "0") not in ("", "0")  # tune unknown problems on first use
USE_TABLES = os.environ.get("MXBLAS_B200_TABLES", "1") not in ("", "0")  # consult the persisted tables
AUTO = (0, -1, 0, 0, 0, 0, 0)  # MxbConfig fields that leave every choice to the library's heuristic
_table: Optional[dict] = None      # user's table (read-write)
_shipped: Optional[dict] = None    # table shipped with the package (read-only)
_lock = threading.RLock()          # guards both tables, the plan cache and the file
_plan_cache: dict = {}             # (meta, flags) -> MxbConfig or None, so a warm call costs one dict lookup
_flush_buf: Optional[torch.Tensor] = None


# -------------------------------------------------------------------------------------------------
# timing
# -------------------------------------------------------------------------------------------------
def time_call(fn: Callable[[], object], iters: int = 10, warmup: int = 3, flush_l2: bool = True) -> Tuple[float, float]:
    """(median, min) seconds of ``fn`` on the current stream, CUDA events, one event pair per call.
    With ``flush_l2`` a 256 MiB buffer is READ before every call, which evicts the operands and leaves
    L2 clean (a write flush leaves dirty lines whose write-back is then charged to the kernel), and
    keeps the GPU busy while the host enqueues the call, so no launch latency lands between the events."""
    global _flush_buf
    if flush_l2 and _flush_buf is None:
        _flush_buf = torch.zeros(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    times = []
    for _ in range(iters):
        if flush_l2:
            _flush_buf.view(torch.int32).sum(dtype=torch.int32)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        end.synchronize()
        times.append(start.elapsed_time(end) * 1e-3)
    times.sort()
    return times[len(times) // 2], times[0]


# -------------------------------------------------------------------------------------------------
# candidates
# -------------------------------------------------------------------------------------------------
def candidates(m: int, n: int, k: int, sk: int, quant: bool, out_transpose: bool, mx: bool) -> List[MxbConfig]:
    """Configurations worth timing for a problem; the library filters out the ones it has no kernel for.
    The first candidate is always the heuristic plan itself, so the winner is never slower than it.
    Fields: (bn, swap, epi_warps, raster, splits, ctas, cta_pair); splits 0 lets CTA-pair plans cut the
    tiles of an incomplete last wave along K, splits 1 forbids it."""
    out: List[MxbConfig] = [MxbConfig(*AUTO)]
    swap_opts = (1,) if out_transpose else ((1,) if m <= 128 else (0,))
    big = m > 256
    if sk == k:  # scales constant along K
        if not big:
            for swap in ((1,) if m <= 32 else (0, 1)):
                for bn in (32, 64, 128, 256):
                    ry = m if swap else n
                    if bn < min(ry, 32) or (bn > 32 and bn >= 2 * max(ry, 16)):
                        continue
                    for splits in (1, 2, 3, 4):
                        out.append(MxbConfig(bn, swap, 4, 8, splits, 0, 1))
            if 64 < m <= 128:  # left as the 128-wide Y operand of a CTA pair, each CTA staging half of it
                for tail in (0, 1):
                    out.append(MxbConfig(128, 1, 4, 16, tail, 0, 2))
        else:
            for swap in swap_opts:
                for ew in ((4, 8) if quant else (4,)):
                    for raster in (4, 8, 16, 32):
                        for tail in (0, 1):
                            out.append(MxbConfig(256, swap, ew, raster, tail, 0, 2))
                    out.append(MxbConfig(256, swap, ew, 8, 1, 0, 1))
                out.append(MxbConfig(224, swap, 4, 16, 1, 0, 2))
                out.append(MxbConfig(128, swap, 4, 8, 1, 0, 1))
    elif mx:  # 1x32 power-of-two scales on the block-scaled MMA
        for swap in swap_opts:
            if big:
                for raster in (4, 8, 16, 32):
                    out.append(MxbConfig(224, swap, 4, raster, 1, 0, 2))
            for bn in (128, 224):
                for raster in (4, 8, 16):
                    out.append(MxbConfig(bn, swap, 4, raster, 1, 0, 1))
    else:  # scales that change along K: promotion in registers
        for swap in swap_opts:
            if big and sk == 128:
                for bn in (256, 128):
                    for raster in (4, 8, 16, 32):
                        for tail in (0, 1):
                            out.append(MxbConfig(bn, swap, 8, raster, tail, 0, 2))
            for bn, ew in ((128, 4), (128, 8), (256, 8), (64, 4)):
                for raster in (4, 8, 16):
                    out.append(MxbConfig(bn, swap, ew, raster, 1, 0, 1))
    return out


# -------------------------------------------------------------------------------------------------
# persisted table
# -------------------------------------------------------------------------------------------------
def _gpu_name() -> str:
    return torch.cuda.get_device_name().replace(" ", "_") if torch.cuda.is_available() else "cpu"


def _table_path() -> Path:
    root = Path(os.environ.get(CACHE_DIR_FLAG, str(Path.home() / ".mxblas_b200")))
    return root / f"autotune_{_gpu_name()}.json"


def _shipped_path() -> Path:
    return Path(__file__).resolve().parent / "tuned" / f"{_gpu_name()}.json"


def _read(path: Path) -> dict:
    try:
        return json.loads(path.read_text())
    except (OSError, ValueError):
        return {}


def _load_table() -> dict:
    global _table
    with _lock:
        if _table is None:
            _table = _read(_table_path())
        return _table


def _load_shipped() -> dict:
    global _shipped
    with _lock:
        if _shipped is None:
            _shipped = _read(_shipped_path())
        return _shipped


def reload_tables() -> None:
    """Forget what was read from disk (a new process-style start; tests, or after another process tuned)."""
    global _table, _shipped
    with _lock:
        _table = _shipped = None
        _plan_cache.clear()


def _save_table() -> None:
    with _lock:
        path = _table_path()
        path.parent.mkdir(parents=True, exist_ok=True)
        # merge what another process stored meanwhile, then replace the file atomically, as the reference's
        # cache writes do (mxblas/jit/compiler.py:113-118)
        merged = _read(path)
        merged.update(_table or {})
        _table.update(merged)
        tmp = path.with_suffix(f".tmp{os.getpid()}.{threading.get_ident()}")
        tmp.write_text(json.dumps(merged, indent=0, sort_keys=True))
        os.replace(tmp, path)


def m_bucket(m: int) -> int:
    """Problems are keyed by M rounded up to a power of two (activations vary, weights do not)."""
    b = 16
    while b < m:
        b *= 2
    return b


def table_key(meta, out_scale_pow2: bool, pow2_scales) -> str:
    if not (meta.sk == 32 and meta.sm == 1 and meta.sn == 1):
        pow2_scales = "-"  # only 1x32 scales can take the block-scaled MMA: the flag changes nothing elsewhere
    return "|".join(str(x) for x in (
        meta.in_dtype, meta.out_dtype, meta.scale_dtype, m_bucket(meta.m), meta.n, meta.k, meta.sm if meta.sm == 1 else
        "M" if meta.sm == meta.m else meta.sm, meta.sn, meta.sk, meta.qm, meta.qn, int(meta.out_transpose),
        int(meta.out_scale_transpose), int(bool(out_scale_pow2)), pow2_scales))


def lookup(meta, out_scale_pow2: bool, pow2_scales) -> Optional[MxbConfig]:
    """The tuned configuration of a problem: user's table first, then the shipped one; None if neither has it
    (or the entry is the heuristic plan itself)."""
    key = table_key(meta, out_scale_pow2, pow2_scales)
    with _lock:
        rec = _load_table().get(key) or _load_shipped().get(key)
    if not rec or tuple(rec["config"]) == AUTO:
        return None
    return MxbConfig(*rec["config"])


def plan_for(meta, out_scale_pow2: bool, pow2_scales) -> Optional[MxbConfig]:
    """``lookup`` behind a per-process cache keyed by the call signature itself (no string formatting on the
    warm path)."""
    ck = (meta, bool(out_scale_pow2), pow2_scales)
    try:
        return _plan_cache[ck]
    except KeyError:
        cfg = lookup(meta, out_scale_pow2, pow2_scales)
        with _lock:
            _plan_cache[ck] = cfg
        return cfg


def autotune(left, right, left_scale, right_scale, output_quant=False, quant_size=None, out_dtype=None,
             out_transpose=False, out_scale_transpose=False, *, out_scale_pow2=False, pow2_scales=None,
             iters: int = 8, persist: bool = True, configs: Optional[Iterable[MxbConfig]] = None):
    """Time the candidate configurations of one problem; returns (best config, [(config key, seconds)])."""
    from .mx_gemm import get_meta_info, mx_gemm_kernel

    meta = get_meta_info(
        left.dtype, right.dtype, left_scale.dtype, right_scale.dtype, bool(output_quant),
        None if quant_size is None else tuple(quant_size), out_dtype, tuple(left.shape), tuple(right.shape),
        tuple(left_scale.shape), tuple(right_scale.shape), tuple(left.stride()), tuple(right.stride()),
        tuple(left_scale.stride()), tuple(right_scale.stride()), bool(out_transpose), bool(out_scale_transpose))
    mx = meta.sk == 32 and meta.sm == 1 and meta.sn == 1 and pow2_scales is not False
    cands = list(configs) if configs is not None else candidates(meta.m, meta.n, meta.k, meta.sk, meta.quant,
                                                                 meta.out_transpose, mx)
    results = []

    def timed(cfg):
        def run():
            return mx_gemm_kernel(left, right, left_scale, right_scale, output_quant, quant_size, out_dtype,
                                  out_transpose, out_scale_transpose, out_scale_pow2=out_scale_pow2,
                                  pow2_scales=pow2_scales, config=cfg)
        med, _ = time_call(run, iters=iters, warmup=2)
        return med

    for cfg in cands:
        try:
            med = timed(cfg)
        except ValueError:
            continue  # the library has no kernel for this candidate
        if _ext.device_status() != 0:
            continue
        results.append((cfg.key(), med))
        if os.environ.get(PRINT_AUTOTUNE_FLAG):
            print(f"[mxblas autotune] {cfg.key()} {med * 1e6:.1f} us")
        if os.environ.get(PROFILING_TIME_PATH):
            with open(os.environ[PROFILING_TIME_PATH], "a") as f:
                f.write(f"{table_key(meta, out_scale_pow2, pow2_scales)} {cfg.key()} {med * 1e6:.2f}\n")
    if not results:
        raise ValueError("autotune: no candidate configuration ran")
    # The first candidate (the heuristic plan) is timed right after the caller produced its operands, with the GPU
    # in whatever clock state that left (measured: 43 us against 20.6 us for the same plan a moment later), so it
    # and the provisional winner are timed once more, back to back, and each keeps its better figure.
    by_key = dict(results)
    first_key = results[0][0]
    provisional = min(results, key=lambda r: r[1])[0]
    for key in dict.fromkeys((first_key, provisional)):
        try:
            by_key[key] = min(by_key[key], timed(MxbConfig(*key)))
        except ValueError:
            pass
    results = [(k, by_key[k]) for k, _ in results]
    best_key, best_t = min(results, key=lambda r: r[1])
    if persist:
        with _lock:
            _load_table()[table_key(meta, out_scale_pow2, pow2_scales)] = {"config": list(best_key), "us": best_t * 1e6}
            _save_table()
            _plan_cache.clear()
    return MxbConfig(*best_key), results


if __name__ == "__main__":
    from .bench_configs import main

    main()
