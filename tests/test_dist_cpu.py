"""N-sharding host logic with two gloo ranks on the CPU. The local GEMM is replaced by the CPU
oracle (tests may use it); what is under test is the slicing, the divisibility rules and the
all-gather assembly of mxblas_b200/dist.py."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from conftest import make_inputs

from mxblas_b200.dist import gather_columns, shard_bounds, shard_right, sharded_mx_gemm
from oracle import mx_oracle as orc


def test_shard_bounds_rules():
    assert shard_bounds(8192, 8, 3, sn=128, qn=16) == (3072, 4096)
    assert shard_bounds(28672, 8, 7, sn=1) == (25088, 28672)
    assert shard_bounds(7168, 8, 0, sn=128) == (0, 896)
    assert shard_bounds(8192, 2, 1, sn=8192) == (4096, 8192)  # per-tensor scale is shared
    with pytest.raises(ValueError):
        shard_bounds(8192, 3, 0)
    with pytest.raises(ValueError):
        shard_bounds(1024, 8, 0, sn=256)  # 128 columns per rank cannot hold a 256-wide scale block
    with pytest.raises(ValueError):
        shard_bounds(512, 8, 0, sn=1, qn=128)
    with pytest.raises(ValueError):
        shard_bounds(512, 8, 8)


def test_shard_right_returns_views():
    left, right_phys, ls, rs = make_inputs(32, 256, 128, 1, 128, 128)
    r, s = shard_right(right_phys.t(), rs.t(), 2, 1)
    assert r.shape == (128, 128) and s.shape == (1, 1)
    assert r.data_ptr() == right_phys[128:].data_ptr()
    assert torch.equal(r.t().view(torch.uint8), right_phys[128:].view(torch.uint8))
    assert torch.equal(s, rs.t()[:, 1:2])


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_t, quant):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m, n, k = 48, 256, 128
        left, right_phys, ls, rs = make_inputs(m, n, k, 1, 128, 128, seed=7)
        qs = torch.Size((1, 32))

        def compute(a, b, sa, sb, q, qsz, od, ot, ost, **kw):
            o, s = orc.mx_gemm(a, b, sa, sb, q, qsz, od, ot, ost)
            if o.dtype == torch.float8_e4m3fn:  # gloo has no fp8: carry the codes as bytes
                o = o.view(torch.uint8)
            return o, s

        out, sc = sharded_mx_gemm(left, right_phys.t(), ls, rs.t(), quant, qs, None, out_t, out_t,
                                  gather=True, compute=compute)
        want, want_sc = orc.mx_gemm(left, right_phys.t(), ls, rs.t(), quant, qs, None, out_t, out_t)
        if quant:
            assert torch.equal(out, want.view(torch.uint8)), "gathered codes differ"
            assert torch.equal(sc, want_sc), "gathered scales differ"
        else:
            assert torch.equal(out, want), "gathered output differs"
        # local (un-gathered) result is this rank's column block
        loc, _ = sharded_mx_gemm(left, right_phys.t(), ls, rs.t(), False, None, None, False, False,
                                 gather=False, compute=compute)
        full, _ = orc.mx_gemm(left, right_phys.t(), ls, rs.t())
        per = n // world
        assert torch.equal(loc, full[:, rank * per:(rank + 1) * per])
        # ranks that disagree on divisibility raise the same ValueError everywhere (no collective entered)
        with pytest.raises(ValueError):
            sharded_mx_gemm(left, right_phys[:250].t(), ls, rs.t(), compute=compute)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("out_t,quant", [(False, False), (True, False), (False, True), (True, True)])
def test_two_rank_gather(out_t, quant):
    mp.spawn(_worker, args=(2, _free_port(), out_t, quant), nprocs=2, join=True)


def test_gather_is_identity_for_one_rank():
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(_free_port()))
    dist.init_process_group("gloo", rank=0, world_size=1)
    try:
        x = torch.arange(12.0).reshape(3, 4)
        assert torch.equal(gather_columns(x, False), x)
    finally:
        dist.destroy_process_group()


def test_peer_row_chunks_rule():
    """Row chunks of a gather="peer" call: whole 256-row tiles and scale blocks, about 100 us of GEMM or push per
    chunk, at most 8, none for transposed results."""
    from mxblas_b200.dist import peer_row_chunks

    big = dict(flops=2.0 * 16384 * 14336 * 8192, push_bytes=16384 * 14336 * 2)       # 1.5 ms of GEMM
    assert peer_row_chunks(16384, 1, False, False, **big) == 8
    assert peer_row_chunks(16384, 1, True, False, **big) == 1                          # C^T: column strips
    assert peer_row_chunks(16384, 1, False, True, **big) == 1
    small = dict(flops=2.0 * 8192 * 4096 * 8192, push_bytes=8192 * 4096)              # 0.22 ms: two chunks
    assert peer_row_chunks(8192, 8192, False, False, **small) == 2
    assert peer_row_chunks(8192, 8192, False, False, flops=1e10, push_bytes=1e6) == 1  # too short to chunk
    assert peer_row_chunks(8192 + 256, 1, False, False, **big) in (1, 3)               # only divisors that keep 256-row tiles
    assert peer_row_chunks(16384, 4096, False, False, want=8) == 4                     # chunks hold whole scale blocks
    push_bound = dict(flops=1e9, push_bytes=7 * 16384 * 3584 * 2)                      # 8 ranks: the push dominates
    assert peer_row_chunks(16384, 1, False, False, **push_bound) == 8
