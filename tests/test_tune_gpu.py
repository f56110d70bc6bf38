"""The autotuner on a GPU: it can reach the kernels the heuristic plans use (CTA pairs in all three scale
modes), its winner is no slower than the heuristic plan, and a fresh start finds the winner in the table."""

import pytest
import torch
from conftest import make_inputs

import mxblas_b200 as mxblas
from mxblas_b200 import _ext, tune
from mxblas_b200.mx_gemm import get_meta_info
from oracle import mx_oracle as orc

pytestmark = pytest.mark.gpu

CASES = {
    # name: (make_inputs args, operator args after the scales, keyword args)
    "per_tensor_quant16": ((4096, 4096, 1024, 4096, 4096, 1024, torch.bfloat16), (True, torch.Size((1, 16))), {}),
    "promotion_1x128_128x128": ((4096, 4096, 1024, 1, 128, 128), (), {"pow2_scales": False}),
    "block_scaled_1x32": ((4096, 4096, 1024, 1, 1, 32), (), {"pow2_scales": True}),
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_autotune_winner_is_no_slower_and_survives_a_restart(name, tmp_path, monkeypatch):
    monkeypatch.setenv("MXBLAS_CACHE_DIR", str(tmp_path))
    monkeypatch.setattr(tune, "USE_TABLES", True)
    tune.reload_tables()
    shape, op_args, kw = CASES[name]
    ins = make_inputs(*shape, seed=77, pow2=name.startswith("block_scaled"))
    d = torch.device("cuda:0")
    left, right_phys, ls, rs = (t.to(d) for t in ins)
    args = (left, right_phys.t(), ls, rs.t()) + op_args
    best, results = tune.autotune(*args, **kw, iters=5)
    times = dict(results)
    assert tune.AUTO in times, "the heuristic plan is always a candidate"
    assert any(key[6] == 2 for key in times), "CTA-pair kernels must be among the timed candidates"
    assert times[best.key()] <= times[tune.AUTO]
    # timed again, head to head (the bar allows for run-to-run noise of a ~50 us kernel)
    t_best, _ = tune.time_call(lambda: mxblas.mx_gemm_kernel(*args, **kw, config=best), iters=15)
    t_heur, _ = tune.time_call(lambda: mxblas.mx_gemm_kernel(*args, **kw, config=mxblas.MxbConfig(*tune.AUTO)), iters=15)
    assert t_best <= 1.03 * t_heur + 2e-6, (t_best, t_heur, best.key())
    # a new process would start with nothing in memory and the table on disk
    tune.reload_tables()
    meta = get_meta_info(left.dtype, left.dtype, ls.dtype, rs.dtype, bool(op_args), tuple(op_args[1]) if op_args else None,
                         None, tuple(left.shape), (left.shape[1], right_phys.shape[0]), tuple(ls.shape),
                         tuple(rs.t().shape), tuple(left.stride()), tuple(right_phys.t().stride()), tuple(ls.stride()),
                         tuple(rs.t().stride()), False, False)
    again = tune.plan_for(meta, False, kw.get("pow2_scales"))
    if best.key() == tune.AUTO:
        assert again is None
    else:
        assert again is not None and again.key() == best.key()
    # and the operator, called without a configuration, runs that plan and still agrees with the oracle
    out, osc = mxblas.mx_gemm_kernel(*args, **kw)
    assert _ext.device_status() == 0
    c32 = orc.mx_gemm_c32(ins[0], ins[1].t(), ins[2], ins[3].t())
    if op_args:
        codes, scales, _ = orc.quantize_groups(c32, 16, ls.dtype)
        dist = orc.fp8_code_distance(out.cpu(), codes)
        assert float((dist == 0).float().mean()) >= 0.999 and int(dist.max()) <= 1
    else:
        met = orc.compare_hp(out.cpu().float(), c32)
        assert met["max_rel"] <= 1e-2 and met["cosine"] >= 0.9999, met
    tune.reload_tables()
