"""mxblas_b200: FP8 micro-scaled GEMM for NVIDIA B200 behind the MXBLAS operator API.

    import mxblas_b200 as mxblas          # or: import mxblas  (thin alias package)
    mxblas.register_all_kernels()
    c, c_scale = mxblas.mx_gemm_kernel(a_fp8, b_fp8.T, a_scales, b_scales.T, True, torch.Size((1, 16)))

Public surface of the reference kept: mxblas/__init__.py:1-2 re-exports mxblas/jit_kernels (the
operator) and mxblas/project (the constants).
"""

from .const import *  # noqa: F401,F403
from .mx_gemm import (  # noqa: F401
    MxbConfig,
    get_meta_info,
    mx_gemm_kernel,
    register_all_kernels,
    register_state,
    reset_workspaces,
)

from .grouped import mx_grouped_gemm  # noqa: F401,E402

__all__ = ["mx_gemm_kernel", "mx_grouped_gemm", "register_all_kernels", "MxbConfig"]
