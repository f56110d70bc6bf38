"""N-sharded GEMM on real GPUs with NCCL (needs >= 2 GPUs; skipped otherwise). Child processes, one
per GPU; every rank checks its gathered result against the CPU oracle."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from conftest import make_inputs

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from mxblas_b200 import _ext
        from mxblas_b200.dist import sharded_mx_gemm
        from oracle import mx_oracle as orc

        m, n, k = 256, 1024, 512
        left, right_phys, ls, rs = make_inputs(m, n, k, 1, 1, k, seed=17)
        args = (left.to(dev), right_phys.to(dev).t(), ls.to(dev), rs.to(dev).t())
        c32 = orc.mx_gemm_c32(left, right_phys.t(), ls, rs.t())
        # bf16, gathered row-major
        out, _ = sharded_mx_gemm(*args, gather=True)
        met = orc.compare_hp(out.cpu().float(), c32)
        assert out.shape == (m, n) and met["max_rel"] <= 1e-2 and met["cosine"] >= 0.9999, met
        # quantised + transposed: the all-gather writes C^T in place
        q, qs = sharded_mx_gemm(*args, True, torch.Size((1, 32)), None, True, True, gather=True)
        codes, scales, _ = orc.quantize_groups(c32, 32, torch.float32)
        dist_codes = orc.fp8_code_distance(q.t().contiguous().cpu(), codes)
        assert q.shape == (n, m) and float((dist_codes == 0).float().mean()) >= 0.999 and int(dist_codes.max()) <= 1
        assert ((qs.t().cpu() - scales).abs() / scales).max().item() <= 1e-5
        # local result only: this rank's columns
        loc, _ = sharded_mx_gemm(*args)
        per = n // world
        met = orc.compare_hp(loc.cpu().float(), c32[:, rank * per:(rank + 1) * per])
        assert met["max_rel"] <= 1e-2 and met["cosine"] >= 0.9999
        # the same full result without a collective: each rank's GEMM writes its column block of its own symmetric
        # buffer and a copy kernel (or the copy engines) pushes the block into every other rank's buffer; must equal
        # the NCCL-gathered tensor bit for bit, for bf16 and for quantised results (codes and scales are pushed)
        out_p, _ = sharded_mx_gemm(*args, gather="peer")
        assert torch.equal(out_p.view(torch.int16), out.view(torch.int16))
        q_p, qs_p = sharded_mx_gemm(*args, True, torch.Size((1, 32)), None, True, True, gather="peer")
        assert torch.equal(q_p.view(torch.uint8), q.view(torch.uint8)) and torch.equal(qs_p, qs)
        q_r, qs_r = sharded_mx_gemm(*args, True, torch.Size((1, 32)), gather=True)
        q_rp, qs_rp = sharded_mx_gemm(*args, True, torch.Size((1, 32)), gather="peer")
        assert torch.equal(q_rp.view(torch.uint8), q_r.view(torch.uint8)) and torch.equal(qs_rp, qs_r)
        out_p2, _ = sharded_mx_gemm(*args, gather="peer")  # the buffers are reused: same values again
        assert torch.equal(out_p2.view(torch.int16), out.view(torch.int16))
        out_t, _ = sharded_mx_gemm(*args, False, None, torch.float16, True, gather=True)  # C^T, fp16
        out_tp, _ = sharded_mx_gemm(*args, False, None, torch.float16, True, gather="peer")
        assert out_tp.shape == (n, m) and torch.equal(out_tp.view(torch.int16), out_t.view(torch.int16))
        # row chunks (the push of one chunk under the GEMM of the next, on a side stream) and both transports
        m2 = 1024
        left2, right2, ls2, rs2 = make_inputs(m2, n, k, 1, 1, k, seed=18)
        args2 = (left2.to(dev), right2.to(dev).t(), ls2.to(dev), rs2.to(dev).t())
        want2, _ = sharded_mx_gemm(*args2, gather=True)
        for kw in (dict(peer_chunks=2), dict(peer_chunks=4, peer_transport="dma"), dict(peer_chunks=1, peer_transport="dma")):
            got2, _ = sharded_mx_gemm(*args2, gather="peer", **kw)
            assert torch.equal(got2.view(torch.int16), want2.view(torch.int16)), kw
        q2, qs2 = sharded_mx_gemm(*args2, True, torch.Size((1, 32)), gather=True)
        q2p, qs2p = sharded_mx_gemm(*args2, True, torch.Size((1, 32)), gather="peer", peer_chunks=2)
        assert torch.equal(q2p.view(torch.uint8), q2.view(torch.uint8)) and torch.equal(qs2p, qs2)
        # column blocks that are not 16-byte aligned (N/ranks/QN bf16 scales = 4 bytes per row) take the all-gather
        left3, right3, ls3, rs3 = make_inputs(256, 64, 128, 256, 64, 128, torch.bfloat16, seed=19)
        args3 = (left3.to(dev), right3.to(dev).t(), ls3.to(dev), rs3.to(dev).t(), True, torch.Size((1, 16)))
        q3, qs3 = sharded_mx_gemm(*args3, gather=True)
        q3p, qs3p = sharded_mx_gemm(*args3, gather="peer")
        assert torch.equal(q3p.view(torch.uint8), q3.view(torch.uint8)) and torch.equal(qs3p, qs3)
        assert _ext.device_status() == 0
    finally:
        dist.destroy_process_group()


def test_two_gpu_sharded_gemm_with_nccl_gather():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    mp.spawn(_worker, args=(2, _free_port()), nprocs=2, join=True)
