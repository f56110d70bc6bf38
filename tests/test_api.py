"""Host logic of the operator on the CPU: argument validation against what the reference's own
get_meta_info derives or raises (tests/golden/meta.json), defaults, and the C ABI surface."""

import ctypes
import json
import re
from pathlib import Path

import pytest
import torch
from conftest import GOLDEN, ROOT

import mxblas_b200
from mxblas_b200 import _ext
from mxblas_b200.mx_gemm import get_meta_info, make_problem

DT = {"e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2, "bf16": torch.bfloat16, "fp16": torch.float16,
      "fp32": torch.float32, None: None}
REF_DT = {"FP8_E4M3": torch.float8_e4m3fn, "FP8_E5M2": torch.float8_e5m2, "BF16": torch.bfloat16,
          "FP16": torch.float16, "FP32": torch.float32}
META = json.loads((GOLDEN / "meta.json").read_text())


def _args(rec):
    a = rec["args"]
    conv = [DT[a[0]], DT[a[1]], DT[a[2]], DT[a[3]], bool(a[4]), None if a[5] is None else tuple(a[5]), DT[a[6]]]
    conv += [tuple(x) for x in a[7:15]] + [bool(a[15]), bool(a[16])]
    return conv


@pytest.mark.parametrize("name", sorted(META))
def test_validation_matches_reference(name):
    rec = META[name]
    if "raises" in rec:
        # the reference raises ValueError for every invalid signature in the list
        assert rec["raises"] == "ValueError"
        with pytest.raises(ValueError):
            get_meta_info(*_args(rec))
        return
    want = rec["result"]
    got = get_meta_info(*_args(rec))
    assert (got.m, got.n, got.k) == (want["m"], want["n"], want["k"])
    assert (got.sm, got.sn, got.sk) == (want["sm"], want["sn"], want["sk"])
    assert got.quant == want["quant"]
    if want["quant"]:
        assert (got.qm, got.qn) == (want["qm"], want["qn"])
    assert got.out_dtype == REF_DT[want["out_dtype"]]
    assert got.scale_dtype == REF_DT[want["scale_dtype"]]


def test_stride_that_is_neither_row_nor_column_major_asserts():
    # the reference hits `assert False` in get_layout (mxblas/jit_kernels/mx_gemm.py:50-58)
    with pytest.raises(AssertionError):
        get_meta_info(torch.float8_e4m3fn, torch.float8_e4m3fn, torch.float32, torch.float32, False, None, None,
                      (64, 64), (64, 64), (1, 1), (1, 1), (128, 2), (1, 64), (1, 1), (1, 1), False, False)


def test_unsupported_layouts_and_alignment_raise_value_error():
    e4, f32 = torch.float8_e4m3fn, torch.float32
    base = dict(ls=(64, 64), rs=(64, 64))
    # right passed row-major instead of as the column-major view: "No matching template" in the reference
    # (mxblas/gemm/template.py:70-73); accepted here and flagged for the library
    meta = get_meta_info(e4, e4, f32, f32, False, None, None, (64, 64), (64, 64), (1, 1), (1, 1), (64, 1), (64, 1),
                         (1, 1), (1, 1), False, False)
    assert meta.right_row_major and not meta.left_col_major and meta.ldb == 64
    meta = get_meta_info(e4, e4, f32, f32, False, None, None, (64, 32), (32, 64), (1, 1), (1, 1), (1, 64), (1, 32),
                         (1, 1), (1, 1), False, False)
    assert meta.left_col_major and not meta.right_row_major and meta.lda == 64
    # a row-major right whose rows are not 16-byte multiples cannot be described to the TMA unit
    with pytest.raises(ValueError):
        get_meta_info(e4, e4, f32, f32, False, None, None, (64, 64), (64, 40), (1, 1), (1, 1), (64, 1), (40, 1),
                      (1, 1), (1, 1), False, False)
    # K not a multiple of 16 bytes: the reference exits the process in its TMA encoder; here ValueError
    with pytest.raises(ValueError):
        get_meta_info(e4, e4, f32, f32, False, None, None, (64, 24), (24, 64), (1, 1), (1, 1), (24, 1), (1, 24),
                      (1, 1), (1, 1), False, False)
    # quantisation groups neither the reference (generator.py:971-974) nor this library has a kernel for;
    # QM > 1 as a power of two up to 128 is an extension here and passes
    get_meta_info(e4, e4, f32, f32, True, (2, 16), None, (64, 64), (64, 64), (1, 1), (1, 1), (64, 1), (1, 64),
                  (1, 1), (1, 1), False, False)
    for qs in ((3, 16), (1, 8), (1, 256)):
        with pytest.raises(ValueError):
            get_meta_info(e4, e4, f32, f32, True, qs, None, (256, 256), (256, 256), (1, 1), (1, 1), (256, 1),
                          (1, 256), (1, 1), (1, 1), False, False)


def test_mx_gemm_kernel_rejects_cpu_tensors_before_touching_the_gpu():
    a = torch.zeros(16, 16).to(torch.float8_e4m3fn)
    s = torch.ones(1, 1)
    with pytest.raises(ValueError):
        mxblas_b200.mx_gemm_kernel(a, a.t(), s, s.t())


def test_register_all_kernels_is_idempotent_and_alias_package_resolves():
    import mxblas
    import mxblas.utils as utils

    mxblas.register_all_kernels()
    mxblas.register_all_kernels()
    assert mxblas_b200.register_state.is_registered()
    assert mxblas.mx_gemm_kernel is mxblas_b200.mx_gemm_kernel
    for name in ("block_quant", "block_dequant", "calc_diff", "GPU_bench", "gaussian_with_channel_outlier",
                 "check_nan_inf", "per_tensor_quant", "CPU_bench"):
        assert hasattr(utils, name)
    assert mxblas.PROJECT_NAME_FULL == "MXBLAS" and mxblas.CACHE_DIR_FLAG == "MXBLAS_CACHE_DIR"


def test_utils_quant_roundtrip_cpu():
    import mxblas_b200.utils as utils

    x = torch.randn(64, 256)
    q, s = utils.block_quant(x, (1, 128))
    assert q.dtype == torch.float8_e4m3fn and s.shape == (64, 2) and s.dtype == torch.float32
    back = utils.block_dequant(q, s, (1, 128), torch.float32)
    assert float(utils.calc_diff(back, x)) < 2e-3
    z, zs = utils.block_quant(torch.zeros(4, 32), (4, 32))
    assert float(zs) == 1.0 and float(z.float().abs().max()) == 0.0


# ---------------------------------------------------------------------------------------------
# C ABI
# ---------------------------------------------------------------------------------------------
def test_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "mxblas_b200.h").read_text()
    declared = set(re.findall(r"\b(mxb_[a-z_0-9]+)\s*\(", header))
    assert declared == set(_ext.EXPORTED_SYMBOLS), declared ^ set(_ext.EXPORTED_SYMBOLS)
    lib = ctypes.CDLL(str(_ext.LIB_PATH))
    for name in declared:
        assert hasattr(lib, name), name
    assert _ext.lib.mxb_abi_version() == 1
    assert _ext.lib.mxb_status_string(_ext.MXB_ERR_WORKSPACE).decode().startswith("workspace")


def test_struct_layout_matches_header():
    # 12 int32/uint32 + 8 int64, no padding surprises
    assert ctypes.sizeof(_ext.MxbProblem) == 12 * 4 + 8 * 8
    assert ctypes.sizeof(_ext.MxbConfig) == 7 * 4


def _problem(m, n, k, sm, sn, sk, quant=False, qn=16, sdt=torch.float32, **kw):
    e4 = torch.float8_e4m3fn
    meta = get_meta_info(e4, e4, sdt, sdt, quant, (1, qn) if quant else None, None, (m, k), (k, n),
                         (m // sm, k // sk), (k // sk, n // sn), (k, 1), (1, k), (k // sk, 1), (1, k // sk),
                         kw.get("out_t", False), False)
    return make_problem(meta, m if kw.get("out_t") else n, n // qn if quant else 0, False, kw.get("pow2"))


def test_plan_selection_without_a_gpu():
    """mxb_default_config / mxb_query_workspace are pure host code."""
    cases = {
        "c1": (_problem(256, 256, 256, 256, 256, 256), dict(bn=128, swap=0, splits=1), False),
        "c2": (_problem(8192, 8192, 8192, 8192, 8192, 8192, True, 16, torch.bfloat16), dict(bn=256, swap=0), False),
        "c3": (_problem(4096, 7168, 7168, 1, 128, 128, pow2=False), dict(swap=0, splits=1), True),  # K-sliced tail tiles
        "c4": (_problem(16384, 8192, 8192, 1, 1, 32, True, 32, out_t=True, pow2=True), dict(swap=1), True),
        "c5_16": (_problem(16, 28672, 8192, 1, 1, 8192), dict(bn=32, swap=1), None),
        "c5_16384": (_problem(16384, 28672, 8192, 1, 1, 8192), dict(bn=256, swap=0, splits=1), False),
        # seven rounds of 256 x 224 CTA-pair tiles instead of seven of 256 x 256
        "c5_1024": (_problem(1024, 28672, 8192, 1, 1, 8192), dict(bn=224, swap=0, cta_pair=2), None),
        # too few tiles for CTA pairs: 112 tiles of 128 x 128 in one round, K not cut
        "c5_256_shard": (_problem(256, 7168, 8192, 1, 1, 8192), dict(bn=128, swap=0, splits=1, cta_pair=1), False),
        # a decode step against a mid-sized weight: 128-wide tiles, K cut in two (cost estimate)
        "decode_128": (_problem(128, 8192, 8192, 128, 8192, 8192), dict(bn=128, swap=1, splits=2), True),
    }
    for name, (p, want, needs_ws) in cases.items():
        cfg = _ext.MxbConfig()
        assert _ext.lib.mxb_default_config(ctypes.byref(p), ctypes.byref(cfg)) == _ext.MXB_OK, name
        for key, val in want.items():
            assert getattr(cfg, key) == val, (name, key, getattr(cfg, key))
        nbytes = ctypes.c_size_t(0)
        assert _ext.lib.mxb_query_workspace(ctypes.byref(p), None, ctypes.byref(nbytes)) == _ext.MXB_OK
        if needs_ws is not None:
            assert (nbytes.value > 0) == needs_ws, (name, nbytes.value)


def test_c_abi_rejects_bad_problems_with_status_codes():
    p = _problem(256, 256, 256, 256, 256, 256)
    nbytes = ctypes.c_size_t(0)
    p.k = 250  # not a multiple of 16
    assert _ext.lib.mxb_query_workspace(ctypes.byref(p), None, ctypes.byref(nbytes)) == _ext.MXB_ERR_INVALID
    p = _problem(256, 256, 256, 256, 256, 256)
    p.sk = 48  # K blocks that are not multiples of 32
    p.k = 240
    assert _ext.lib.mxb_query_workspace(ctypes.byref(p), None, ctypes.byref(nbytes)) in (
        _ext.MXB_ERR_INVALID, _ext.MXB_ERR_UNSUPPORTED)
    p = _problem(256, 256, 256, 256, 256, 256, True, 16)
    p.qm = 3  # rows of a quantisation block: powers of two up to 128
    assert _ext.lib.mxb_query_workspace(ctypes.byref(p), None, ctypes.byref(nbytes)) == _ext.MXB_ERR_UNSUPPORTED
    p.qm = 256
    assert _ext.lib.mxb_query_workspace(ctypes.byref(p), None, ctypes.byref(nbytes)) == _ext.MXB_ERR_UNSUPPORTED
    p.qm = 32
    assert _ext.lib.mxb_query_workspace(ctypes.byref(p), None, ctypes.byref(nbytes)) == _ext.MXB_OK
    assert _ext.lib.mxb_query_workspace(None, None, ctypes.byref(nbytes)) == _ext.MXB_ERR_INVALID
    # null tensors are refused before any CUDA call
    p = _problem(256, 256, 256, 256, 256, 256)
    assert _ext.lib.mxb_gemm(ctypes.byref(p), None, None, None, None, None, None, None, 0, None) == _ext.MXB_ERR_INVALID


def test_grouped_gemm_validates_before_touching_the_gpu():
    """mx_grouped_gemm refuses host tensors and malformed group tables with ValueError (no CPU fallback)."""
    import mxblas_b200 as mxblas

    a = torch.zeros(128, 64).to(torch.float8_e4m3fn)
    w = torch.zeros(2, 32, 64).to(torch.float8_e4m3fn)
    with pytest.raises(ValueError):
        mxblas.mx_grouped_gemm(a, w.transpose(1, 2), torch.ones(128, 1), torch.ones(2, 32, 1).transpose(1, 2),
                               torch.zeros(1, dtype=torch.int32))


def test_c_abi_layout_flags_and_grouped_plans():
    """Planner answers for the extensions, without a GPU: operand-layout flags take 128- / 256-wide tiles, a
    grouped problem refuses what it cannot do."""
    e4, f32 = torch.float8_e4m3fn, torch.float32
    meta = get_meta_info(e4, e4, f32, f32, False, None, None, (512, 1024), (1024, 768), (512, 1), (1, 768),
                         (1024, 1), (768, 1), (1, 1), (768, 1), False, False)
    assert meta.right_row_major
    p = make_problem(meta, 768, 0, False, False)
    cfg = _ext.MxbConfig()
    assert _ext.lib.mxb_default_config(ctypes.byref(p), ctypes.byref(cfg)) == _ext.MXB_OK
    assert cfg.bn in (128, 256)
    nbytes = ctypes.c_size_t(0)
    plain = make_problem(get_meta_info(e4, e4, f32, f32, False, None, None, (512, 1024), (1024, 768), (512, 1),
                                       (1, 768), (1024, 1), (1, 1024), (1, 1), (1, 1), False, False), 768, 0, False, False)
    ok = _ext.lib.mxb_grouped_query_workspace(ctypes.byref(plain), None, 4, 128, ctypes.byref(nbytes))
    assert ok == _ext.MXB_OK
    assert _ext.lib.mxb_grouped_query_workspace(ctypes.byref(plain), None, 4, 64, ctypes.byref(nbytes)) == _ext.MXB_ERR_INVALID
    assert _ext.lib.mxb_grouped_query_workspace(ctypes.byref(plain), None, 0, 128, ctypes.byref(nbytes)) == _ext.MXB_ERR_INVALID
    pair = _ext.MxbConfig(256, 0, 4, 2, 1, 0, 2)
    assert _ext.lib.mxb_grouped_query_workspace(ctypes.byref(plain), ctypes.byref(pair), 4, 128, ctypes.byref(nbytes)) == \
        _ext.MXB_ERR_UNSUPPORTED  # CTA pairs need blocks of whole 256-row tiles
    assert _ext.lib.mxb_grouped_query_workspace(ctypes.byref(plain), ctypes.byref(pair), 2, 256, ctypes.byref(nbytes)) == _ext.MXB_OK


def test_every_plan_of_a_problem_grid_has_a_kernel():
    """Planner sweep without a GPU: every valid problem of a grid over M, N, K, the four scaling patterns, the
    quantisation group lengths and both output orientations gets a plan for which a kernel exists (the width
    rules, the skinny cost estimate and the CTA-pair decisions never pick a combination that was not built)."""
    import itertools

    checked = 0
    for m, n, k in itertools.product((1, 16, 48, 64, 100, 128, 200, 256, 512, 1024, 4096, 16384),
                                     (128, 256, 1024, 3584, 7168, 8192, 28672), (128, 512, 8192)):
        patterns = {"TT": (m, n, k), "CC": (1, 1, k), "GB": (1, 128, 128), "MX": (1, 1, 32)}
        for name, (sm, sn, sk) in patterns.items():
            for qn, out_t in itertools.product((0, 16, 32, 64, 128), (False, True)):
                p = _problem(m, n, k, sm, sn, sk, bool(qn), qn or 16, out_t=out_t, pow2=True if name == "MX" else None)
                cfg, nbytes = _ext.MxbConfig(), ctypes.c_size_t(0)
                assert _ext.lib.mxb_default_config(ctypes.byref(p), ctypes.byref(cfg)) == _ext.MXB_OK, (m, n, k, name, qn, out_t)
                assert _ext.lib.mxb_query_workspace(ctypes.byref(p), None, ctypes.byref(nbytes)) == _ext.MXB_OK
                assert cfg.bn in (32, 64, 128, 224, 256) and cfg.splits >= 1
                checked += 1
    assert checked == 12 * 7 * 3 * 4 * 10

