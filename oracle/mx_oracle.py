"""CPU oracle for the MX-GEMM path. TEST INFRASTRUCTURE ONLY.

This file restates, with plain torch tensor arithmetic on the CPU, what the reference's
``mxblas.mx_gemm_kernel`` computes. Only tests/, ``__graft_entry__.smoke()`` and the CPU-baseline
legs of ``bench.py`` may import it; the product (mxblas_b200/) never does.

Parity status: PINNED. tests/golden/ holds vectors generated in the build container by importing
the reference itself from its source tree (tests/golden/make_golden.py): the reference's own
``block_dequant`` + ``torch.mm`` for the un-quantised result and its ``block_quant`` /
``block_dequant`` helpers as cross-checks; tests/test_oracle.py compares this restatement with them
bit for bit. The reference's GPU kernels cannot run anywhere in this project (sm_90a-only WGMMA),
so for the fused quantisation epilogue the oracle follows the arithmetic written in the reference's
kernel generator, line by line (cited below), and is cross-checked against a second, independent C
restatement (oracle/mx_oracle_c.c).

Semantics (all in fp32):
  1. dequantise    A32 = left  * left_scale  broadcast over (SM, SK) blocks
                   B32 = right * right_scale broadcast over (SK, SN) blocks
                   -- mxblas/utils.py:100-116 (block_dequant), as called by tests/test_mxgemm.py:32-38
  2. multiply      C32 = A32 @ B32           -- torch.mm, tests/test_mxgemm.py:14, bench/bench_all.py:22
  3. not quantised C = C32.to(out_dtype)     -- round-to-nearest-even, mxblas/gemm/generator.py:257-275
  4. quantised, per group of QN consecutive columns of a row
                   amax  = max(1e-10, max |C32|)            -- generator.py:1009-1077, type_traits.cuh:8
                   s32   = amax * fp32(1/448)               -- generator.py:1079-1083, type_traits.cuh:14-33
                   scale = s32.to(scale_dtype)  (RNE)       -- generator.py:1085-1092
                   code  = e4m3_satfinite_rne(C32 * (1/s32)) -- generator.py:1094-1133 (__NV_SATFINITE :394)
     The codes are computed with the fp32 scale *before* it is rounded to the scale dtype.
  5. out_transpose / out_scale_transpose return the transposes of the tensors above, contiguous.
     The reference declares the flags but ships no kernel for them (generator.py:933-936,
     mxblas/gemm/template.py:74); the definition follows its allocation code (mx_gemm.py:301-325).
  6. out_scale_pow2 (extension, not in the reference): s32 is rounded up to the next power of two
     before use, so the stored scale is exact in every scale dtype and codes never saturate.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

FP8_MAX = {torch.float8_e4m3fn: 448.0, torch.float8_e5m2: 57344.0}
SCALE_MIN_THRES = 1e-10  # mxblas/include/mxblas/type_traits.cuh:8


def dequant(x: torch.Tensor, scales: torch.Tensor, block: Tuple[int, int]) -> torch.Tensor:
    """fp32 ``x * scales`` with every scale broadcast over a ``block`` of elements.

    Same result as mxblas/utils.py:100-116 (``block_dequant`` with hfp_t=float32); written with
    repeat_interleave instead of the reference's view/permute so that the restatement is independent.
    """
    bm, bn = block
    assert x.shape[0] == scales.shape[0] * bm and x.shape[1] == scales.shape[1] * bn
    s = scales.to(torch.float32).repeat_interleave(bm, dim=0).repeat_interleave(bn, dim=1)
    return x.to(torch.float32) * s


def pow2_ceil(s: torch.Tensor) -> torch.Tensor:
    """Smallest power of two >= s (s fp32, positive, normal)."""
    mant, exp = torch.frexp(s)  # s = mant * 2**exp, mant in [0.5, 1)
    exp = torch.where(mant == 0.5, exp - 1, exp)
    return torch.ldexp(torch.ones_like(s), exp)


def quantize_groups(
    c32: torch.Tensor, qn: int, scale_dtype: torch.dtype, out_dtype: torch.dtype = torch.float8_e4m3fn,
    pow2: bool = False, qm: int = 1,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:  # fmt: skip
    """Step 4 above. Returns (codes [M, N] fp8, scales [M/qm, N/qn] in scale_dtype, s32 [M/qm, N/qn]).

    ``qm`` > 1 (an extension: the reference's epilogue asserts qm == 1, generator.py:971) takes the maximum
    over a [qm, qn] block instead of a [1, qn] group; everything else is the same arithmetic."""
    m, n = c32.shape
    assert n % qn == 0 and m % qm == 0
    g = c32.reshape(m // qm, qm, n // qn, qn)
    amax = g.abs().amax(dim=(1, 3)).clamp_min(SCALE_MIN_THRES)
    inv_max = torch.tensor(1.0 / FP8_MAX[out_dtype], dtype=torch.float32)
    s32 = amax * inv_max
    if pow2:
        s32 = pow2_ceil(s32)
    inv = 1.0 / s32  # IEEE fp32 division, as `one_value / amax` in generator.py:1094-1095
    fmax = FP8_MAX[out_dtype]
    # torch's CPU cast to fp8 rounds to nearest even but does not saturate: clamp first, which is
    # what __NV_SATFINITE does in the kernel (and what mxblas/utils.py:85 does for the same reason)
    codes = (g * inv[:, None, :, None]).clamp(-fmax, fmax).reshape(m, n).to(out_dtype)
    return codes, s32.to(scale_dtype), s32


def mx_gemm_c32(
    left: torch.Tensor, right: torch.Tensor, left_scale: torch.Tensor, right_scale: torch.Tensor
) -> torch.Tensor:
    """Steps 1-2: the fp32 result before any output conversion. Arguments as the public operator:
    ``right`` is the [K, N] view, ``right_scale`` is [K/SK, N/SN]."""
    m, k = left.shape
    k2, n = right.shape
    assert k == k2
    sm, sk = m // left_scale.shape[0], k // left_scale.shape[1]
    sn = n // right_scale.shape[1]
    assert right_scale.shape[0] == left_scale.shape[1]
    a32 = dequant(left, left_scale, (sm, sk))
    b32 = dequant(right.t(), right_scale.t(), (sn, sk))  # physical [N, K]
    return a32 @ b32.t()


def mx_gemm(
    left: torch.Tensor,
    right: torch.Tensor,
    left_scale: torch.Tensor,
    right_scale: torch.Tensor,
    output_quant: bool = False,
    quant_size: Optional[Tuple[int, int]] = None,
    out_dtype: Optional[torch.dtype] = None,
    out_transpose: bool = False,
    out_scale_transpose: bool = False,
    out_scale_pow2: bool = False,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Oracle of ``mxblas.mx_gemm_kernel`` (mxblas/jit_kernels/mx_gemm.py:340-425); same arguments,
    same return tuple."""
    c32 = mx_gemm_c32(left, right, left_scale, right_scale)
    scale_dtype = left_scale.dtype
    if output_quant:
        assert quant_size is not None
        out_dtype = out_dtype or left.dtype
        out, out_scale, _ = quantize_groups(c32, int(quant_size[1]), scale_dtype, out_dtype, out_scale_pow2,
                                            int(quant_size[0]))
    else:
        out = c32.to(out_dtype or torch.bfloat16)
        out_scale = torch.empty([], dtype=scale_dtype)
    if out_transpose:
        out = out.t().contiguous()
    if out_scale_transpose and output_quant:
        out_scale = out_scale.t().contiguous()
    return out, out_scale


# -------------------------------------------------------------------------------------------------
# comparison metrics used by the parity tests
# -------------------------------------------------------------------------------------------------
def fp8_code_distance(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Distance in representable values between two fp8 tensors of the same dtype (0 = identical).
    Codes are mapped to a monotone integer line (sign-magnitude -> two's-complement order)."""

    def line(t):
        u = t.view(torch.uint8).to(torch.int16)
        mag = u & 0x7F
        return torch.where(u >= 0x80, -mag, mag)

    return (line(a) - line(b)).abs()


def ulp_distance(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Distance in units in the last place between two same-dtype float tensors (positive values)."""
    if a.dtype == torch.float32:
        return (a.view(torch.int32).to(torch.int64) - b.view(torch.int32).to(torch.int64)).abs()
    return (a.view(torch.int16).to(torch.int32) - b.view(torch.int16).to(torch.int32)).abs()


def compare_hp(got: torch.Tensor, want32: torch.Tensor) -> dict:
    """Tolerance metrics for un-quantised outputs: max relative error normalised by the largest
    reference magnitude of each row block, and cosine similarity (1 - calc_diff)."""
    g, w = got.to(torch.float64), want32.to(torch.float64)
    denom = w.abs().amax().clamp_min(1e-30)
    cos = 2 * (g * w).sum() / ((g * g).sum() + (w * w).sum()).clamp_min(1e-300)
    return {
        "max_rel": float(((g - w).abs() / denom).amax()),
        "cosine": float(cos),
    }
