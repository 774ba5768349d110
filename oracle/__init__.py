"""ctypes/numpy front-end of the CPU oracle (``galois_oracle.cpp``).

TEST INFRASTRUCTURE ONLY.  The oracle is a CPU restatement of the galois CPU
ops that define the numerics of the Q4_0 mat-mul / attention-chain path.  It is
the checker for the CUDA kernels and the CPU baseline the bench times; the
shipped package never imports it.

PARITY UNPINNED: the reference holds no golden vector for any of these
functions and cannot be compiled in this image; see the header of
``galois_oracle.cpp`` for what pins the restatement instead.

Arrays follow ggml order: a numpy array of shape ``(n3, n2, n1, n0)`` (C order)
is a galois tensor with ``ne = [n0, n1, n2, n3]``; strides are in elements
(blocks for Q4_0).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libgalois_oracle.so")

QK = 32
Q4_0_BYTES = 18
Q8_0_BYTES = 34


class Dim(C.Structure):
    """Mirror of galois ``Dim`` (src/shape.rs:29-34): ggml order, element strides."""

    _fields_ = [("n_dims", C.c_int32), ("ne", C.c_int64 * 4), ("nb", C.c_int64 * 4)]

    @staticmethod
    def contiguous(ne, block=1):
        """ggml strides (src/shape.rs:422-430): nb0 = 1, nb1 = ne0 / block, ..."""
        ne = list(ne) + [1] * (4 - len(ne))
        d = Dim()
        nb = [1, ne[0] // block, 0, 0]
        nb[2] = nb[1] * ne[1]
        nb[3] = nb[2] * ne[2]
        for i in range(4):
            d.ne[i] = ne[i]
            d.nb[i] = nb[i]
        d.n_dims = 4
        return d

    @staticmethod
    def make(ne, nb):
        ne = list(ne) + [1] * (4 - len(ne))
        nb = list(nb)
        assert len(nb) == 4
        d = Dim()
        d.n_dims = 4
        for i in range(4):
            d.ne[i] = ne[i]
            d.nb[i] = nb[i]
        return d


def build(force: bool = False) -> str:
    """Compile the oracle with the committed Makefile; returns the .so path."""
    src = os.path.join(_HERE, "galois_oracle.cpp")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "libgalois_oracle.so"], check=True, capture_output=True)
    return _SO


def use_native_build() -> str:
    """For TIMING the CPU baseline only: rebuild the oracle with -march=native on the host this runs on
    (the analogue of the reference README's -Ctarget-cpu=native, README.md:33) and switch this module to it.
    Returns "native", or "portable" when that build fails and the portable library stays in use."""
    global _lib, _SO
    try:
        subprocess.run(["make", "-C", _HERE, "-B", "libgalois_oracle_native.so"], check=True, capture_output=True)
    except Exception:
        return "portable"
    _SO = os.path.join(_HERE, "libgalois_oracle_native.so")
    _lib = None
    try:
        lib()
    except Exception:
        _SO = os.path.join(_HERE, "libgalois_oracle.so")
        _lib = None
        return "portable"
    return "native"


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        L = C.CDLL(_SO)
        P, F, I, I64, U64, U16 = C.c_void_p, C.c_float, C.c_int, C.c_int64, C.c_uint64, C.c_uint16
        DP = C.POINTER(Dim)
        sig = {
            "orc_f32_to_f16": ([F], U16),
            "orc_f16_to_f32": ([U16], F),
            "orc_f32_to_f16_soft": ([F], U16),
            "orc_f32_to_f16_row": ([P, P, I64], None),
            "orc_f16_to_f32_row": ([P, P, I64], None),
            "orc_fill_normal": ([P, I64, U64, F, F], None),
            "orc_quantize_row_q4_0": ([P, P, I64], None),
            "orc_dequantize_row_q4_0": ([P, P, I64], None),
            "orc_quantize_row_q8_0": ([P, P, I64], None),
            "orc_vec_dot_q4_0_q8_0_avx": ([P, P, I64], F),
            "orc_vec_dot_q4_0_q8_0_scalar": ([P, P, I64], F),
            "orc_block_isums_q4_0_q8_0": ([P, P, I64, P, I], None),
            "orc_vec_dot_f16": ([P, P, I64, I], F),
            "orc_mul_mat_q4_0_f32": ([P, DP, P, DP, P, DP, I, I], I),
            "orc_mul_mat_f16_f32": ([P, DP, P, DP, P, DP, I, I], I),
            "orc_mul_mat_q6k_f32": ([P, DP, P, DP, P, DP, I, I], I),
            "orc_quantize_row_q8k": ([P, P, I64], None),
            "orc_quantize_row_q6k": ([P, P, I64], None),
            "orc_dequantize_row_q6k": ([P, P, I64], None),
            "orc_vec_dot_q6k_q8k_avx": ([P, P, I64], F),
            "orc_block_isums_q6k_q8k": ([P, P, I64, P, I], None),
            "orc_rms_norm_f32": ([P, DP, P, DP, F], I),
            "orc_rope_f32": ([P, DP, P, DP, P, DP, I, I, I, F, F, F, I], I),
            "orc_exp_f16_table": ([], P),
            "orc_silu_f16_table": ([], P),
            "orc_soft_max_f32": ([P, DP, P, DP], I),
            "orc_soft_max_ext_f32": ([P, DP, P, DP, F, P], I),
            "orc_silu_f32": ([P, DP, P, DP], I),
            "orc_add_f32": ([P, DP, P, DP, P, DP], I),
            "orc_mul_f32": ([P, DP, P, DP, P, DP], I),
            "orc_scale_f32": ([P, DP, F, P, DP], I),
            "orc_cpy_f32": ([P, DP, P, DP, I], I),
            "orc_has_avx2": ([], I),
        }
        for name, (args, res) in sig.items():
            fn = getattr(L, name)
            fn.argtypes = args
            fn.restype = res
        _lib = L
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _dim_of(a: np.ndarray, block: int = 1) -> Dim:
    """Dim of a C-contiguous numpy array viewed in ggml order."""
    shape = list(a.shape)[::-1]
    return Dim.contiguous(shape, block)


class OracleError(RuntimeError):
    pass


def _check(rc, what):
    if rc != 0:
        raise OracleError(f"{what}: the reference would panic here (code {rc})")


# ----------------------------------------------------------------- data
def fill_normal(n: int, seed: int, mean: float = 0.0, std: float = 1.0) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    lib().orc_fill_normal(_p(out), n, seed, mean, std)
    return out


def f32_to_f16(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().orc_f32_to_f16_row(_p(x), _p(out), x.size)
    return out


def f16_to_f32(h: np.ndarray) -> np.ndarray:
    h = np.ascontiguousarray(h, dtype=np.uint16)
    out = np.empty(h.shape, dtype=np.float32)
    lib().orc_f16_to_f32_row(_p(h), _p(out), h.size)
    return out


def quantize_q4_0(x: np.ndarray) -> np.ndarray:
    """f32 [..., K] -> uint8 [..., K/32*18] Q4_0 blocks."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    k = x.shape[-1]
    assert k % QK == 0
    rows = x.size // k
    out = np.empty((rows, k // QK * Q4_0_BYTES), dtype=np.uint8)
    xr = x.reshape(rows, k)
    for r in range(rows):
        lib().orc_quantize_row_q4_0(_p(xr[r]), _p(out[r]), k)
    return out.reshape(*x.shape[:-1], k // QK * Q4_0_BYTES)


def dequantize_q4_0(w: np.ndarray, k: int) -> np.ndarray:
    w = np.ascontiguousarray(w, dtype=np.uint8)
    rows = w.size // (k // QK * Q4_0_BYTES)
    wr = w.reshape(rows, -1)
    out = np.empty((rows, k), dtype=np.float32)
    for r in range(rows):
        lib().orc_dequantize_row_q4_0(_p(wr[r]), _p(out[r]), k)
    return out


def get_rows_q4_0(w: np.ndarray, k: int, idx: np.ndarray) -> np.ndarray:
    """GetRows::f_q_x_f32::<BlockQ4_0> (src/op.rs:2546-2571): row idx[i] of the Q4_0 table `w`
    ([rows][K/32*18] bytes), dequantised with <BlockQ4_0 as QuantType>::to_f32
    (src/ggml_quants.rs:209-228), becomes row i of the f32 result [len(idx)][K]."""
    w = np.ascontiguousarray(w, dtype=np.uint8)
    wr = w.reshape(-1, k // QK * Q4_0_BYTES)
    idx = np.asarray(idx).reshape(-1)
    out = np.empty((idx.size, k), dtype=np.float32)
    for i, r in enumerate(idx):
        if not 0 <= int(r) < wr.shape[0]:
            raise OracleError(f"get_rows: index {int(r)} outside the table of {wr.shape[0]} rows (the reference panics)")
        lib().orc_dequantize_row_q4_0(_p(wr[int(r)]), _p(out[i]), k)
    return out


def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    """f32 [..., K] -> uint8 [..., K/32*34] Q8_0 blocks (quantize_row_q8_0)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    k = x.shape[-1]
    if k % QK != 0:
        raise OracleError(f"{k} is not divisible by {QK}")
    rows = x.size // k if k else 0
    out = np.empty((rows, k // QK * Q8_0_BYTES), dtype=np.uint8)
    xr = x.reshape(rows, k)
    for r in range(rows):
        lib().orc_quantize_row_q8_0(_p(xr[r]), _p(out[r]), k)
    return out.reshape(*x.shape[:-1], k // QK * Q8_0_BYTES)


QK_K = 256
Q6K_BYTES = 210
Q8K_BYTES = 292


def quantize_q6k(x: np.ndarray) -> np.ndarray:
    """f32 [..., k] -> Q6K bytes [..., k/256 * 210] with the oracle's own (simple) quantiser."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    k = x.shape[-1]
    rows = x.reshape(-1, k)
    out = np.empty((rows.shape[0], k // QK_K * Q6K_BYTES), np.uint8)
    for r in range(rows.shape[0]):
        lib().orc_quantize_row_q6k(_p(rows[r]), _p(out[r]), k)
    return out.reshape(*x.shape[:-1], k // QK_K * Q6K_BYTES)


def dequantize_q6k(w: np.ndarray, k: int) -> np.ndarray:
    w = np.ascontiguousarray(w, dtype=np.uint8).reshape(-1, k // QK_K * Q6K_BYTES)
    out = np.empty((w.shape[0], k), np.float32)
    for r in range(w.shape[0]):
        lib().orc_dequantize_row_q6k(_p(w[r]), _p(out[r]), k)
    return out


def quantize_q8k(x: np.ndarray) -> np.ndarray:
    """f32 [..., k] -> BlockQ8K bytes [..., k/256 * 292] (<BlockQ8K as QuantType>::from_f32)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    k = x.shape[-1]
    rows = x.reshape(-1, k)
    out = np.zeros((rows.shape[0], k // QK_K * Q8K_BYTES), np.uint8)
    for r in range(rows.shape[0]):
        lib().orc_quantize_row_q8k(_p(rows[r]), _p(out[r]), k)
    return out.reshape(*x.shape[:-1], k // QK_K * Q8K_BYTES)


def vec_dot_q6k_q8k(w_row: np.ndarray, x_row: np.ndarray) -> float:
    w_row = np.ascontiguousarray(w_row, dtype=np.uint8)
    x_row = np.ascontiguousarray(x_row, dtype=np.uint8)
    return float(lib().orc_vec_dot_q6k_q8k_avx(_p(w_row), _p(x_row), w_row.size // Q6K_BYTES))


def block_isums_q6k(w_row: np.ndarray, x_row: np.ndarray, avx: bool = False) -> np.ndarray:
    w_row = np.ascontiguousarray(w_row, dtype=np.uint8)
    x_row = np.ascontiguousarray(x_row, dtype=np.uint8)
    nb = w_row.size // Q6K_BYTES
    out = np.empty(nb, np.int32)
    lib().orc_block_isums_q6k_q8k(_p(w_row), _p(x_row), nb, _p(out), int(avx))
    return out


def mul_mat_q6k(w: np.ndarray, x: np.ndarray, nth: int = 4) -> np.ndarray:
    """w: Q6K bytes [N][K/256*210]; x: f32 [B][K] -> f32 [B][N] (MatMul::f_q_f32_f32::<BlockQ6K>)."""
    w = np.ascontiguousarray(w, dtype=np.uint8)
    x = np.ascontiguousarray(x, dtype=np.float32)
    n, k = w.shape[0], x.shape[-1]
    b = x.shape[0]
    dst = np.empty((b, n), np.float32)
    wd = Dim.contiguous([k, n], QK_K)
    xd = Dim.contiguous([k, b])
    dd = Dim.contiguous([n, b])
    _check(lib().orc_mul_mat_q6k_f32(_p(w), wd, _p(x), xd, _p(dst), dd, nth, 1), "mul_mat_q6k")
    return dst


def vec_dot_q4_0_q8_0(w_row: np.ndarray, x_row: np.ndarray, avx: bool = True) -> float:
    nb = w_row.size // Q4_0_BYTES
    assert x_row.size // Q8_0_BYTES == nb
    w_row = np.ascontiguousarray(w_row)
    x_row = np.ascontiguousarray(x_row)
    fn = lib().orc_vec_dot_q4_0_q8_0_avx if avx else lib().orc_vec_dot_q4_0_q8_0_scalar
    return float(fn(_p(w_row), _p(x_row), nb))


def block_isums(w_row: np.ndarray, x_row: np.ndarray, avx: bool = False) -> np.ndarray:
    nb = w_row.size // Q4_0_BYTES
    w_row = np.ascontiguousarray(w_row)
    x_row = np.ascontiguousarray(x_row)
    out = np.empty(nb, dtype=np.int32)
    lib().orc_block_isums_q4_0_q8_0(_p(w_row), _p(x_row), nb, _p(out), int(avx))
    return out


def vec_dot_f16(a: np.ndarray, b: np.ndarray, avx: bool = True) -> float:
    a = np.ascontiguousarray(a, dtype=np.uint16)
    b = np.ascontiguousarray(b, dtype=np.uint16)
    return float(lib().orc_vec_dot_f16(_p(a), _p(b), a.size, int(avx)))


# ----------------------------------------------------------------- ops
def mul_mat_q4_0_raw(w, wd: Dim, x, xd: Dim, dst, dd: Dim, nth=4, avx=True):
    _check(lib().orc_mul_mat_q4_0_f32(_p(w), wd, _p(x), xd, _p(dst), dd, nth, int(avx)), "mul_mat_q4_0_f32")


def mul_mat_f16_raw(w, wd: Dim, x, xd: Dim, dst, dd: Dim, nth=4, avx=True):
    _check(lib().orc_mul_mat_f16_f32(_p(w), wd, _p(x), xd, _p(dst), dd, nth, int(avx)), "mul_mat_f16_f32")


def mul_mat_q4_0(w: np.ndarray, x: np.ndarray, nth: int = 4, avx: bool = True) -> np.ndarray:
    """w: uint8 [N, K/32*18]; x: f32 [B, K] -> f32 [B, N] (galois_matmul, Q4_0 x F32)."""
    w = np.ascontiguousarray(w, dtype=np.uint8)
    x = np.ascontiguousarray(x, dtype=np.float32)
    n = w.shape[0]
    b, k = x.shape
    assert w.shape[1] == k // QK * Q4_0_BYTES
    dst = np.empty((b, n), dtype=np.float32)
    mul_mat_q4_0_raw(w, Dim.contiguous([k, n], QK), x, Dim.contiguous([k, b]), dst, Dim.contiguous([n, b]), nth, avx)
    return dst


def mul_mat_f16(a: np.ndarray, x: np.ndarray, nth: int = 4, avx: bool = True) -> np.ndarray:
    """a: uint16 (f16 bits) [H, N, K]; x: f32 [Hx, B, K] -> f32 [Hx, B, N]; a broadcast over heads."""
    a = np.ascontiguousarray(a, dtype=np.uint16)
    x = np.ascontiguousarray(x, dtype=np.float32)
    if a.ndim == 2:
        a = a[None]
    if x.ndim == 2:
        x = x[None]
    h, n, k = a.shape
    hx, b, k2 = x.shape
    assert k == k2
    dst = np.empty((hx, b, n), dtype=np.float32)
    mul_mat_f16_raw(a, Dim.contiguous([k, n, h]), x, Dim.contiguous([k, b, hx]), dst, Dim.contiguous([n, b, hx]), nth, avx)
    return dst


def rms_norm(x: np.ndarray, eps: float) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty_like(x)
    d = _dim_of(x)
    _check(lib().orc_rms_norm_f32(_p(x), d, _p(y), d, eps), "rms_norm")
    return y


def rope(x: np.ndarray, pos: np.ndarray, n_dims: int, mode: int = 0, n_ctx: int = 0, freq_base: float = 10000.0,
         freq_scale: float = 1.0, xpos_base: float = 0.0, xpos_down: bool = False) -> np.ndarray:
    """x: f32 [tokens, heads, head_dim]; pos: i32 [tokens]."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    pos = np.ascontiguousarray(pos, dtype=np.int32)
    y = np.empty_like(x)
    d = _dim_of(x)
    _check(lib().orc_rope_f32(_p(x), d, _p(pos), _dim_of(pos), _p(y), d, n_dims, mode, n_ctx, freq_base, freq_scale,
                              xpos_base, int(xpos_down)), "rope_custom")
    return y


def exp_f16_table() -> np.ndarray:
    ptr = lib().orc_exp_f16_table()
    return np.ctypeslib.as_array(C.cast(ptr, C.POINTER(C.c_uint16)), shape=(65536,)).copy()


def silu_f16_table() -> np.ndarray:
    ptr = lib().orc_silu_f16_table()
    return np.ctypeslib.as_array(C.cast(ptr, C.POINTER(C.c_uint16)), shape=(65536,)).copy()


def soft_max(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty_like(x)
    d = _dim_of(x)
    _check(lib().orc_soft_max_f32(_p(x), d, _p(y), d), "soft_max")
    return y


def soft_max_ext(x: np.ndarray, scale: float, pos: np.ndarray | None) -> np.ndarray:
    """x: f32 [tokens, heads, cols]; scale then causal mask (col > pos[token]) then soft_max."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty_like(x)
    d = _dim_of(x)
    if pos is not None:
        pos = np.ascontiguousarray(pos, dtype=np.int32)
    _check(lib().orc_soft_max_ext_f32(_p(x), d, _p(y), d, scale, _p(pos) if pos is not None else None), "soft_max_ext")
    return y


def silu(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty_like(x)
    d = _dim_of(x)
    _check(lib().orc_silu_f32(_p(x), d, _p(y), d), "silu")
    return y


def _binary(fn, a, b, what):
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    y = np.empty_like(a)
    _check(fn(_p(a), _dim_of(a), _p(b), _dim_of(b), _p(y), _dim_of(a)), what)
    return y


def add(a, b):
    return _binary(lib().orc_add_f32, a, b, "add")


def mul(a, b):
    return _binary(lib().orc_mul_f32, a, b, "mul")


def scale(x: np.ndarray, s: float) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty_like(x)
    d = _dim_of(x)
    _check(lib().orc_scale_f32(_p(x), d, s, _p(y), d), "scale")
    return y


def cpy_f32_raw(x, xd: Dim, y, yd: Dim, to_f16: bool):
    _check(lib().orc_cpy_f32(_p(x), xd, _p(y), yd, int(to_f16)), "cpy")


def cpy_f32_f16(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty(x.shape, dtype=np.uint16)
    cpy_f32_raw(x, _dim_of(x), y, _dim_of(y), True)
    return y
