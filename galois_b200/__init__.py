"""galois_b200 — B200 (sm_100a) implementation of galois's Q4_0 mat-mul and
attention-chain GPU ops behind the reference's own ``galois_*`` op API.

Importing the package loads ``libgalois_b200.so``; there is no CPU fallback.
"""
from ._lib import LIB_PATH, lib  # noqa: F401  (raises if the library is missing)
from .op import (  # noqa: F401
    RopeCustomOption,
    UnaryOp,
    galois_add,
    galois_cont,
    galois_cpy,
    galois_cpy_pair,
    galois_get_rows,
    galois_matmul,
    galois_matmul_add,
    galois_matmul_fused,
    galois_matmul_swiglu,
    galois_mul,
    galois_rms_norm,
    galois_rms_norm_mul,
    galois_rope_custom,
    galois_scale,
    galois_silu_mul,
    galois_soft_max,
    galois_soft_max_ext,
    galois_unary,
    quantize_q8_0,
)
from .tensor import CudaDevice, Device, Dim, GError, GGmlType, Tensor  # noqa: F401
