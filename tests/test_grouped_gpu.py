"""Grouped MX-GEMM (one weight per group, rows sorted by group) against the CPU oracle applied group by group."""

import pytest
import torch

import mxblas_b200 as mxblas
from mxblas_b200 import _ext
from oracle import mx_oracle as orc

pytestmark = pytest.mark.gpu


def _inputs(blocks_per_group, block_rows, n, k, sm, sn, sk, seed, pow2=False, sdt=torch.float32, skip=()):
    """blocks_per_group[g] blocks of block_rows rows for group g, in order; blocks listed in `skip` get -1."""
    g = torch.Generator().manual_seed(seed)
    groups = len(blocks_per_group)
    table = [gi for gi, nb in enumerate(blocks_per_group) for _ in range(nb)]
    m = len(table) * block_rows
    left = torch.randn(m, k, generator=g).to(torch.float8_e4m3fn)
    w = torch.randn(groups, n, k, generator=g).to(torch.float8_e4m3fn)
    sm = m if sm == 0 else sm
    if pow2:
        ls = torch.pow(2.0, torch.randint(-6, 4, (m // sm, k // sk), generator=g).float())
        ws = torch.pow(2.0, torch.randint(-6, 4, (groups, n // sn, k // sk), generator=g).float())
    else:
        ls = 0.25 + 1.5 * torch.rand(m // sm, k // sk, generator=g)
        ws = 0.25 + 1.5 * torch.rand(groups, n // sn, k // sk, generator=g)
    table = [(-1 if i in skip else t) for i, t in enumerate(table)]
    return left, w, ls.to(sdt), ws.to(sdt), torch.tensor(table, dtype=torch.int32)


def _check(left, w, ls, ws, table, block_rows, quant=False, qn=32, qm=1, pow2_scales=False, config=None):
    d = torch.device("cuda:0")
    m, n = left.shape[0], w.shape[1]
    sm = m // ls.shape[0]
    sentinel = torch.full((m, n), 7.0 if not quant else 0.0, device=d).to(torch.float8_e4m3fn if quant else torch.bfloat16)
    out, osc = mxblas.mx_grouped_gemm(
        left.to(d), w.to(d).transpose(1, 2), ls.to(d), ws.to(d).transpose(1, 2), table.to(d), quant,
        torch.Size((qm, qn)), None, block_rows=block_rows, pow2_scales=pow2_scales, config=config, out=sentinel.clone())
    assert _ext.device_status() == 0
    for b, grp in enumerate(table.tolist()):
        r0, r1 = b * block_rows, (b + 1) * block_rows
        got = out[r0:r1].cpu()
        if grp < 0:
            assert torch.equal(got.view(torch.uint8), sentinel[r0:r1].cpu().view(torch.uint8)), "skipped block written"
            continue
        ls_b = ls if sm == m else ls[r0 // sm:r1 // sm]
        c32 = orc.mx_gemm_c32(left[r0:r1], w[grp].t(), ls_b, ws[grp].t())
        if not quant:
            met = orc.compare_hp(got.float(), c32)
            assert met["max_rel"] <= 1e-2 and met["cosine"] >= 0.9999, (b, grp, met)
        else:
            codes, scales, _ = orc.quantize_groups(c32, qn, ls.dtype, qm=qm)
            dist = orc.fp8_code_distance(got, codes)
            assert float((dist == 0).float().mean()) >= 0.999 and int(dist.max()) <= 1, (b, grp)
            gsc = osc[r0 // qm:r1 // qm].cpu().float()
            assert ((gsc - scales.float()).abs() / scales.float()).max().item() <= 2.0**-7


@pytest.mark.parametrize("pattern", ["CC", "TC", "GB", "GG128", "MX"])
def test_grouped_patterns(pattern):
    sm, sn, sk = {"CC": (1, 1, 512), "TC": (0, 1, 512), "GB": (1, 128, 128), "GG128": (1, 1, 128), "MX": (1, 1, 32)}[pattern]
    ins = _inputs([2, 1, 3, 1], 128, 384, 512, sm, sn, sk, seed=11, pow2=pattern == "MX")
    kw = dict(pow2_scales=True) if pattern == "MX" else {}
    _check(*ins, 128, **kw)
    _check(*ins, 128, quant=True, qn=32, **kw)
    if pattern == "MX":
        _check(*ins, 128, pow2_scales=None)  # probed on the device


def test_grouped_skipped_blocks_uneven_groups_and_bf16_scales():
    ins = _inputs([1, 4, 0, 2], 128, 256, 256, 1, 1, 256, seed=12, sdt=torch.bfloat16, skip=(2, 6))
    _check(*ins, 128)
    _check(*ins, 128, quant=True, qn=16)
    with pytest.raises(ValueError):  # two-dimensional quantisation blocks are not built for grouped GEMMs
        _check(*ins, 128, quant=True, qn=32, qm=32)


def test_grouped_on_cta_pairs():
    """Blocks of 256 rows: large problems run on CTA pairs (256 x 256 tiles); forced here on a small one too."""
    ins = _inputs([3, 5, 2, 6], 256, 2560, 256, 1, 1, 256, seed=13)          # 16 x 10 = 160 pair tiles: default
    _check(*ins, 256)
    _check(*ins, 256, quant=True, qn=16)
    gb = _inputs([2, 1, 1], 256, 512, 384, 1, 128, 128, seed=14, skip=(1,))
    _check(*gb, 256, config=mxblas.MxbConfig(256, 0, 8, 2, 1, 0, 2))
    _check(*gb, 256)
    with pytest.raises(ValueError):  # pairs need blocks of whole 256-row tiles
        _check(*_inputs([2, 2], 128, 512, 256, 1, 1, 256, seed=15), 128, config=mxblas.MxbConfig(256, 0, 4, 2, 1, 0, 2))


def test_grouped_rejects_what_it_cannot_do():
    d = torch.device("cuda:0")
    left, w, ls, ws, table = _inputs([1, 1], 128, 256, 256, 1, 1, 256, seed=16)
    args = (left.to(d), w.to(d).transpose(1, 2), ls.to(d), ws.to(d).transpose(1, 2))
    with pytest.raises(ValueError):
        mxblas.mx_grouped_gemm(*args, table.to(d), block_rows=64)
    with pytest.raises(ValueError):
        mxblas.mx_grouped_gemm(*args, table.to(d)[:1])
    with pytest.raises(ValueError):
        mxblas.mx_grouped_gemm(*args, table.to(d).long())
    with pytest.raises(ValueError):  # weights that are not [N, K] per group
        mxblas.mx_grouped_gemm(args[0], w.to(d).transpose(1, 2).contiguous(), args[2], args[3], table.to(d))
