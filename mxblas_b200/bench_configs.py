"""Timing of the BASELINE configurations (synthetic seeded data of their shapes and value distributions).

Measurement commands, kept apart from the product modules (the operator, the tuner, the N-sharding):

    python -m mxblas_b200.bench_configs --config c2              # default plan of one configuration
    python -m mxblas_b200.bench_configs --config c5 --m 16 --sweep    # every candidate configuration
    python -m mxblas_b200.bench_configs --all                    # one JSON line per configuration
    python -m mxblas_b200.bench_configs --all --write-table      # tune them, write mxblas_b200/tuned/<gpu>.json
    python -m torch.distributed.run --nnodes=1 --nproc-per-node G --master-addr 127.0.0.1 \
        -m mxblas_b200.bench_configs --dist --config c5 --rows 16     # N-sharded over G GPUs (strong scaling)

Times are CUDA events around one call, L2 evicted by a 256 MiB read before it, median of ``--iters``.
The reference times its kernels with kineto inside its tuner (mxblas/jit/tuner.py:118-160) and has no
fixed list of configurations; its sweep over model shapes is mxblas_b200/bench_all.py here.
"""

from __future__ import annotations

import argparse
import json
import os
from typing import Optional

import torch

from . import _ext
from .tune import autotune, time_call

ALL_CONFIGS = [("c1", None, 1), ("c2", None, 1), ("c3", None, 1), ("c4", None, 1), ("c4", None, 8)] + \
    [("c5", mm, 1) for mm in (16, 64, 128, 256, 1024, 4096, 16384)]


def baseline_problem(name: str, m: Optional[int] = None, device="cuda", shard: int = 1):
    """Operands and call arguments of BASELINE config c1..c5; c4 with shard=8 is one GPU's N slice."""
    g = torch.Generator(device="cpu").manual_seed(0)

    def fp8(rows, cols, scale=1.0):
        return (torch.randn(rows, cols, generator=g) * scale).clamp(-448, 448).to(torch.float8_e4m3fn).to(device)

    def uni(rows, cols, lo, hi, dtype=torch.float32):
        return (lo + (hi - lo) * torch.rand(rows, cols, generator=g)).to(dtype).to(device)

    kw = {}
    if name in ("c1", "c2"):
        M = N = K = 256 if name == "c1" else 8192
        N //= shard
        sdt = torch.float32 if name == "c1" else torch.bfloat16
        a, b, sa, sb = fp8(M, K), fp8(N, K), uni(1, 1, 0.5, 2, sdt), uni(1, 1, 0.5, 2, sdt)
        args = (True, torch.Size((1, 16))) if name == "c2" else ()
    elif name == "c3":
        M, N, K = 4096, 7168 // shard, 7168
        a, b = fp8(M, K, 2.0), fp8(N, K, 2.0)
        sa, sb = uni(M, K // 128, 1e-3, 1e-1), uni(N // 128, K // 128, 1e-3, 1e-1)
        args, kw = (), {"pow2_scales": False}
    elif name == "c4":
        M, N, K = 16384, 8192 // shard, 8192
        a, b = fp8(M, K), fp8(N, K)
        sa = torch.pow(2.0, torch.randint(-8, 5, (M, K // 32), generator=g).float()).to(device)
        sb = torch.pow(2.0, torch.randint(-8, 5, (N, K // 32), generator=g).float()).to(device)
        args, kw = (True, torch.Size((1, 32)), None, True), {"out_scale_pow2": True, "pow2_scales": True}
    elif name == "c5":
        M, N, K = m or 16, 28672 // shard, 8192
        a, b, sa, sb = fp8(M, K), fp8(N, K), uni(M, 1, 0.5, 2), uni(N, 1, 0.5, 2)
        args = ()
    else:
        raise ValueError(name)
    quant = bool(args) and args[0] is True
    qn = int(args[1][1]) if quant else 0
    sbytes = sa.element_size()
    nbytes = (M * K + N * K + M * N * (1 if quant else 2) + (M * (N // qn) * sbytes if quant else 0) +
              sa.numel() * sbytes + sb.numel() * sbytes)
    return (a, b.t(), sa, sb.t()) + args, kw, 2.0 * M * N * K, nbytes, (M, N, K)


def bench_config(name: str, m: Optional[int] = None, sweep: bool = False, shard: int = 1, iters: int = 10) -> dict:
    from .mx_gemm import mx_gemm_kernel

    args, kw, flops, nbytes, shape = baseline_problem(name, m, shard=shard)
    rows = []
    if sweep:
        _, results = autotune(*args, **kw, persist=False, iters=iters)
        rows = [{"config": list(key), "us": t * 1e6} for key, t in sorted(results, key=lambda r: r[1])]
        med = rows[0]["us"] * 1e-6
    else:
        med, _ = time_call(lambda: mx_gemm_kernel(*args, **kw), iters=iters)
    status = _ext.device_status()
    return {"config": name, "shape": list(shape), "us": med * 1e6, "tflops": flops / med / 1e12,
            "pct_of_4500": 100 * flops / med / 4.5e15, "gbs": nbytes / med / 1e9, "algorithmic_bytes": nbytes,
            "device_status": status, "candidates": rows}


def main() -> None:
    import sys

    if "--dist" in sys.argv:
        sys.argv.remove("--dist")
        return dist_main()
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--config", choices=["c1", "c2", "c3", "c4", "c5"])
    ap.add_argument("--m", type=int, default=None, help="M of config c5")
    ap.add_argument("--shard", type=int, default=1, help="time one GPU's N slice of an N-sharded run")
    ap.add_argument("--sweep", action="store_true", help="time every candidate configuration")
    ap.add_argument("--all", action="store_true", help="all BASELINE configs with the default plans")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--write-table", action="store_true",
                    help="with --all: tune every configuration and write the winners to mxblas_b200/tuned/<gpu>.json")
    a = ap.parse_args()
    if a.all and a.write_table:
        write_table(a.iters)
    elif a.all:
        for name, m, shard in ALL_CONFIGS:
            print(json.dumps(bench_config(name, m, False, shard, a.iters)), flush=True)
    else:
        print(json.dumps(bench_config(a.config or "c2", a.m, a.sweep, a.shard, a.iters)))




def write_table(iters: int = 10) -> None:
    """Tune every BASELINE configuration (and its 2-, 4- and 8-way N shards) and write the table the package
    ships: winners that beat the heuristic plan by more than 2 %; everything else stays with the heuristic."""
    from pathlib import Path

    from . import tune
    from .mx_gemm import get_meta_info

    table = {}
    jobs = [(n, m, s) for (n, m, _) in ALL_CONFIGS if n != "c1" for s in (1, 2, 4, 8)]
    for name, m, shard in sorted(set(jobs), key=str):
        args, kw, flops, nbytes, shape = baseline_problem(name, m, shard=shard)
        left, right, ls, rs = args[:4]
        rest = list(args[4:]) + [False, None, None, False, False][len(args) - 4:]
        best, results = autotune(*args, **kw, persist=False, iters=iters)
        times = dict(results)
        heur = times.get(tune.AUTO)
        meta = get_meta_info(left.dtype, right.dtype, ls.dtype, rs.dtype, bool(rest[0]),
                             None if rest[1] is None else tuple(rest[1]), rest[2], tuple(left.shape), tuple(right.shape),
                             tuple(ls.shape), tuple(rs.shape), tuple(left.stride()), tuple(right.stride()),
                             tuple(ls.stride()), tuple(rs.stride()), bool(rest[3]), bool(rest[4]))
        key = tune.table_key(meta, kw.get("out_scale_pow2", False), kw.get("pow2_scales"))
        win = times[best.key()]
        line = {"config": name, "shape": list(shape), "heuristic_us": heur and heur * 1e6, "best_us": win * 1e6,
                "best": list(best.key())}
        if heur is not None and win < 0.98 * heur:
            table[key] = {"config": list(best.key()), "us": win * 1e6, "heuristic_us": heur * 1e6}
            line["stored"] = True
        print(json.dumps(line), flush=True)
        del args, left, right, ls, rs
        torch.cuda.empty_cache()
    path = tune._shipped_path()
    path.parent.mkdir(parents=True, exist_ok=True)
    path.write_text(json.dumps(table, indent=0, sort_keys=True))
    out = os.environ.get("MXBLAS_B200_TABLE_COPY")
    if out:
        Path(out).write_text(json.dumps(table, indent=0, sort_keys=True))
    print(f"wrote {len(table)} entries to {path}", flush=True)


# -------------------------------------------------------------------------------------------------
# Strong-scaling measurement of a BASELINE configuration (total N fixed, N/g columns per rank).
# Rank 0 prints one JSON line: GEMM time (max over ranks, CUDA events), GEMM + all-gather, GEMM + peer push.
# -------------------------------------------------------------------------------------------------
def dist_main() -> None:
    import torch.distributed as tdist

    from . import dist as dist_mod

    ap = argparse.ArgumentParser(description="N-sharded timing of one BASELINE configuration")
    ap.add_argument("--config", choices=["c2", "c3", "c4", "c5"], required=True)
    ap.add_argument("--rows", type=int, default=None, help="M of config c5 (torchrun claims every --m… prefix)")
    ap.add_argument("--iters", type=int, default=20)
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    if world > 1:
        tdist.init_process_group("nccl", device_id=torch.device("cuda", local))
    args, kw, flops, nbytes, shape = baseline_problem(a.config, a.rows, device=f"cuda:{local}", shard=world)
    flush = torch.zeros(256 << 20, dtype=torch.uint8, device=f"cuda:{local}")

    def timed(gather, **peer_kw) -> float:
        times = []
        if world > 1:
            tdist.barrier()
        for it in range(a.iters + 3):
            # evict the operands from L2; the read also keeps the GPU busy while the host enqueues the call,
            # so that no launch latency lands between the events
            flush.view(torch.int32).sum(dtype=torch.int32)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            dist_mod.sharded_mx_gemm(*args, gather=gather, right_is_local=True, **kw, **peer_kw)
            e1.record()
            torch.cuda.synchronize()
            if it >= 3:
                times.append(e0.elapsed_time(e1) * 1e-3)
        times.sort()
        t = torch.tensor([times[len(times) // 2]], device=f"cuda:{local}")
        if world > 1:
            tdist.all_reduce(t, op=tdist.ReduceOp.MAX)
        return float(t.item())

    t_gemm = timed(False)
    t_all = timed(True)
    peer = {}
    if world > 1:
        peer["whole_sm"] = timed("peer", peer_chunks=1)
        peer["whole_dma"] = timed("peer", peer_chunks=1, peer_transport="dma")
        peer["auto_chunks_sm"] = timed("peer")
        peer["auto_chunks_dma"] = timed("peer", peer_transport="dma")
    if rank == 0:
        print(json.dumps({"config": a.config, "per_rank_shape": list(shape), "n_gpus": world,
                          "gemm_us": t_gemm * 1e6, "gemm_plus_gather_us": t_all * 1e6,
                          "gemm_plus_peer_push_us": {k: v * 1e6 for k, v in peer.items()},
                          "whole_job_tflops": flops * world / t_gemm / 1e12}), flush=True)
    if world > 1:
        tdist.destroy_process_group()




if __name__ == "__main__":
    main()
