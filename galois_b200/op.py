"""The ``galois_*`` op API (src/op.rs:3034-3341 of galois) over the B200 C ABI.

Same names, argument order and meaning as the reference's free functions; every
call validates placement the way the reference's ``match`` on storage does and
then forwards to one ``galois_b200_*`` entry point.  Only the GPU arm exists
here: CPU tensors are rejected (the reference's CPU arm is not part of this
package), and placements the reference leaves as ``todo!()`` raise too.
"""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass

from ._lib import lib
from .tensor import Device, GError, GGmlType, Tensor, _check


class UnaryOp(enum.Enum):
    """src/op.rs:113-124"""

    Abs = 0
    Sgn = 1
    Neg = 2
    Step = 3
    Tanh = 4
    Elu = 5
    Relu = 6
    Gelu = 7
    GeluQuick = 8
    Silu = 9


@dataclass
class RopeCustomOption:
    """src/op.rs:3294-3302"""

    n_dims: int
    mode: int = 0
    n_ctx: int = 0
    freq_base: float = 10000.0
    freq_scale: float = 1.0
    xpos_base: float = 0.0
    xpos_down: bool = False


def _gpu_ctx(*tensors: Tensor):
    """All operands on the same GPU -> its context; anything else is what the
    reference's `_ => todo!()` arm covers (or its CPU arm, absent here)."""
    if not all(t.is_gpu for t in tensors):
        if not any(t.is_gpu for t in tensors):
            raise GError("galois_b200 implements the (Gpu, ..., Gpu) arm only; these tensors are on the CPU")
        raise GError("mixed CPU/GPU placement is todo!() in the reference")
    dev = tensors[0].device.gpu
    if any(t.device.gpu is not dev for t in tensors):
        raise GError("operands live on different CudaDevices")
    return dev.ctx


def _p(t: Tensor):
    return C.c_void_p(t.data_ptr())


def _d(t: Tensor):
    return C.byref(t.dim().c_struct())


def _want(t: Tensor, dtype: GGmlType, what: str):
    if t.dtype != dtype:
        raise GError(f"{what}: expected {dtype.name}, got {t.dtype.name}")


def galois_matmul(a: Tensor, b: Tensor, dst: Tensor) -> None:
    """src/op.rs:3093-3111 -> CudaMatMul (src/cuda.rs:476-521): (Q4_0, F32, F32) and (F16, F32, F32); the
    (Q6K, F32, F32) arm exists on the reference's CPU side only (src/op.rs:3454-3456)."""
    ctx = _gpu_ctx(a, b, dst)
    _want(b, GGmlType.F32, "galois_matmul src1")
    _want(dst, GGmlType.F32, "galois_matmul dst")
    if a.dtype == GGmlType.Q4_0:
        rc = lib.galois_b200_mul_mat_q4_0_f32(ctx, _p(a), _d(a), _p(b), _d(b), _p(dst), _d(dst))
    elif a.dtype == GGmlType.Q6K:  # src/op.rs:3454-3456
        rc = lib.galois_b200_mul_mat_q6k_f32(ctx, _p(a), _d(a), _p(b), _d(b), _p(dst), _d(dst))
    elif a.dtype == GGmlType.F16:
        rc = lib.galois_b200_mul_mat_f16_f32(ctx, _p(a), _d(a), _p(b), _d(b), _p(dst), _d(dst))
    else:
        raise GError(f"galois_matmul: src0 dtype {a.dtype.name} is todo!() on the GPU")
    _check(ctx, rc, "galois_matmul")


def galois_rms_norm(src: Tensor, dst: Tensor, eps: float) -> None:
    """src/op.rs:3155-3169"""
    ctx = _gpu_ctx(src, dst)
    _want(src, GGmlType.F32, "galois_rms_norm")
    _want(dst, GGmlType.F32, "galois_rms_norm")
    _check(ctx, lib.galois_b200_rms_norm_f32(ctx, _p(src), _d(src), _p(dst), _d(dst), eps), "galois_rms_norm")


def galois_matmul_add(src0: Tensor, src1: Tensor, res: Tensor, dst: Tensor) -> None:
    """galois_matmul (src/op.rs:3093-3111, Q4_0 x F32) followed by galois_add of `res` (src/op.rs:3073-3091) in one
    call; bit-identical to the two calls.  Not part of the reference API."""
    ctx = _gpu_ctx(src0, src1, res, dst)
    _want(src0, GGmlType.Q4_0, "galois_matmul_add src0")
    for t in (src1, res, dst):
        _want(t, GGmlType.F32, "galois_matmul_add")
    rc = lib.galois_b200_mul_mat_q4_0_f32_add(ctx, _p(src0), _d(src0), _p(src1), _d(src1), _p(res), _d(res), _p(dst), _d(dst))
    _check(ctx, rc, "galois_matmul_add")


def galois_matmul_fused(src0: Tensor, src1: Tensor, dst: Tensor, *, rms_gain: Tensor | None = None, eps: float = 0.0,
                        silu_mul: Tensor | None = None, res: Tensor | None = None) -> None:
    """Up to four reference ops in one call, bit-identical to running them one after the other:
    [galois_rms_norm(src1, eps) then galois_mul by `rms_gain`  |  galois_unary(Silu)(src1) then galois_mul by
    `silu_mul`] -> galois_matmul(src0, .) -> [galois_add(res, .)] (src/op.rs:3155-3169, 3113-3127, 3232-3256,
    3093-3111, 3073-3091).  Not part of the reference API."""
    from ._lib import GaloisPrologue

    if rms_gain is not None and silu_mul is not None:
        raise GError("galois_matmul_fused: one prologue at most")
    ops = [t for t in (src0, src1, dst, rms_gain, silu_mul, res) if t is not None]
    ctx = _gpu_ctx(*ops)
    _want(src0, GGmlType.Q4_0, "galois_matmul_fused src0")
    for t in ops[1:]:
        _want(t, GGmlType.F32, "galois_matmul_fused")
    pro = GaloisPrologue()
    if rms_gain is not None:
        if rms_gain.dim().shape[0] < src1.dim().shape[0]:
            raise GError("galois_matmul_fused: gain row shorter than the activation row")
        pro.kind, pro.aux, pro.eps = 1, rms_gain.data_ptr(), eps
    elif silu_mul is not None:
        if tuple(silu_mul.dim().shape) != tuple(src1.dim().shape) or tuple(silu_mul.dim().stride) != tuple(src1.dim().stride):
            raise GError("galois_matmul_fused: the silu product's second operand must be laid out like src1")
        pro.kind, pro.aux, pro.eps = 2, silu_mul.data_ptr(), 0.0
    import ctypes as C

    rc = lib.galois_b200_mul_mat_q4_0_f32_fused(ctx, _p(src0), _d(src0), _p(src1), _d(src1), C.byref(pro), _p(res) if res is not None else None,
                                                _d(res) if res is not None else None, _p(dst), _d(dst))
    _check(ctx, rc, "galois_matmul_fused")


def galois_matmul_swiglu(src0: Tensor, src1: Tensor, dst: Tensor, *, rms_gain: Tensor | None = None, eps: float = 0.0) -> None:
    """Gate and up projection with their SwiGLU product for a weight whose rows are interleaved at upload
    (row 2i = gate_i, row 2i + 1 = up_i): dst[i] = galois_mul(galois_unary(Silu)(gate_i . t), up_i . t) with
    t = src1 or rms_norm + gain of it; bit-identical to the separate calls (src/op.rs:3093-3111, 3232-3256,
    3113-3127).  dst is {N / 2, batch}.  Not part of the reference API."""
    import ctypes as C

    from ._lib import GaloisPrologue

    ops = [t for t in (src0, src1, dst, rms_gain) if t is not None]
    ctx = _gpu_ctx(*ops)
    _want(src0, GGmlType.Q4_0, "galois_matmul_swiglu src0")
    for t in ops[1:]:
        _want(t, GGmlType.F32, "galois_matmul_swiglu")
    pro = GaloisPrologue()
    if rms_gain is not None:
        if rms_gain.dim().shape[0] < src1.dim().shape[0]:
            raise GError("galois_matmul_swiglu: gain row shorter than the activation row")
        pro.kind, pro.aux, pro.eps = 1, rms_gain.data_ptr(), eps
    rc = lib.galois_b200_mul_mat_q4_0_f32_swiglu(ctx, _p(src0), _d(src0), _p(src1), _d(src1), C.byref(pro), _p(dst), _d(dst))
    _check(ctx, rc, "galois_matmul_swiglu")


def galois_rms_norm_mul(src: Tensor, gain: Tensor, dst: Tensor, eps: float) -> None:
    """galois_rms_norm (src/op.rs:3155-3169) followed by galois_mul with `gain` (src/op.rs:3113-3127) in one
    launch; bit-identical to the two calls.  Not part of the reference API."""
    ctx = _gpu_ctx(src, gain, dst)
    for t in (src, gain, dst):
        _want(t, GGmlType.F32, "galois_rms_norm_mul")
    _check(ctx, lib.galois_b200_rms_norm_mul_f32(ctx, _p(src), _d(src), _p(gain), _d(gain), _p(dst), _d(dst), eps), "galois_rms_norm_mul")


def galois_silu_mul(src: Tensor, other: Tensor, dst: Tensor) -> None:
    """galois_unary(Silu) (src/op.rs:3232-3256) followed by galois_mul with `other` (src/op.rs:3113-3127) in one
    launch; bit-identical to the two calls.  Not part of the reference API."""
    ctx = _gpu_ctx(src, other, dst)
    for t in (src, other, dst):
        _want(t, GGmlType.F32, "galois_silu_mul")
    _check(ctx, lib.galois_b200_silu_mul_f32(ctx, _p(src), _d(src), _p(other), _d(other), _p(dst), _d(dst)), "galois_silu_mul")


def galois_rope_custom(op: RopeCustomOption, src0: Tensor, src1: Tensor, dst: Tensor) -> None:
    """src/op.rs:3304-3341; src1 holds the i32 positions."""
    ctx = _gpu_ctx(src0, src1, dst)
    _want(src0, GGmlType.F32, "galois_rope_custom src0")
    _want(src1, GGmlType.I32, "galois_rope_custom src1")
    _want(dst, GGmlType.F32, "galois_rope_custom dst")
    rc = lib.galois_b200_rope_f32(ctx, _p(src0), _d(src0), _p(src1), _d(src1), _p(dst), _d(dst), op.n_dims, op.mode,
                                  op.n_ctx, op.freq_base, op.freq_scale, op.xpos_base, int(op.xpos_down))
    _check(ctx, rc, "galois_rope_custom")


def galois_soft_max(src: Tensor, dst: Tensor) -> None:
    """src/op.rs:3216-3230"""
    ctx = _gpu_ctx(src, dst)
    _want(src, GGmlType.F32, "galois_soft_max")
    _want(dst, GGmlType.F32, "galois_soft_max")
    _check(ctx, lib.galois_b200_soft_max_f32(ctx, _p(src), _d(src), _p(dst), _d(dst)), "galois_soft_max")


def galois_soft_max_ext(src: Tensor, dst: Tensor, scale: float, pos: Tensor | None) -> None:
    """Fused galois_scale + causal mask (column > pos[token] -> -inf) + galois_soft_max.
    No counterpart in the reference's API; src/dst are {columns, heads, tokens}."""
    ctx = _gpu_ctx(src, dst) if pos is None else _gpu_ctx(src, dst, pos)
    _want(src, GGmlType.F32, "galois_soft_max_ext")
    _want(dst, GGmlType.F32, "galois_soft_max_ext")
    if pos is not None:
        _want(pos, GGmlType.I32, "galois_soft_max_ext pos")
        if pos.dim().shape[0] < src.dim().shape[2]:
            raise GError("galois_soft_max_ext: fewer positions than tokens")
    rc = lib.galois_b200_soft_max_ext_f32(ctx, _p(src), _d(src), _p(dst), _d(dst), scale, _p(pos) if pos is not None else None)
    _check(ctx, rc, "galois_soft_max_ext")


def galois_unary(src: Tensor, dst: Tensor, op: UnaryOp) -> None:
    """src/op.rs:3232-3256: only Silu is implemented (the other arms are todo!())."""
    ctx = _gpu_ctx(src, dst)
    if op != UnaryOp.Silu:
        raise GError(f"galois_unary: {op.name} is todo!() in the reference")
    _want(src, GGmlType.F32, "galois_unary")
    _want(dst, GGmlType.F32, "galois_unary")
    _check(ctx, lib.galois_b200_silu_f32(ctx, _p(src), _d(src), _p(dst), _d(dst)), "galois_unary(Silu)")


def galois_mul(a: Tensor, b: Tensor, dst: Tensor) -> None:
    """src/op.rs:3113-3129"""
    ctx = _gpu_ctx(a, b, dst)
    for t in (a, b, dst):
        _want(t, GGmlType.F32, "galois_mul")
    _check(ctx, lib.galois_b200_mul_f32(ctx, _p(a), _d(a), _p(b), _d(b), _p(dst), _d(dst)), "galois_mul")


def galois_add(a: Tensor, b: Tensor, dst: Tensor) -> None:
    """src/op.rs:3073-3091"""
    ctx = _gpu_ctx(a, b, dst)
    for t in (a, b, dst):
        _want(t, GGmlType.F32, "galois_add")
    _check(ctx, lib.galois_b200_add_f32(ctx, _p(a), _d(a), _p(b), _d(b), _p(dst), _d(dst)), "galois_add")


def galois_scale(src0: Tensor, src1: Tensor, dst: Tensor) -> None:
    """src/op.rs:3258-3279: the (Gpu, Cpu, Gpu) arm — the scalar `src1` is a CPU tensor."""
    ctx = _gpu_ctx(src0, dst)
    if src1.is_gpu:
        # the (Gpu, Gpu, Gpu) arm reads the scalar back first; keep one code path
        src1 = src1.to_cpu_tensor()
    _want(src0, GGmlType.F32, "galois_scale")
    _want(src1, GGmlType.F32, "galois_scale scalar")
    if src1.dim().elem_count() != 1:
        raise GError("galois_scale: src1 must be a scalar (assert!(inp1_d.is_scalar()), src/op.rs:2381)")
    s = float(src1.storage[src1.offset])
    _check(ctx, lib.galois_b200_scale_f32(ctx, _p(src0), _d(src0), s, _p(dst), _d(dst)), "galois_scale")


def galois_cpy(src: Tensor, dst: Tensor) -> None:
    """src/op.rs:3171-3185: f32 -> f32 or f32 -> f16 (the KV-cache append)."""
    ctx = _gpu_ctx(src, dst)
    _want(src, GGmlType.F32, "galois_cpy src")
    if dst.dtype == GGmlType.F32:
        rc = lib.galois_b200_cpy_f32_f32(ctx, _p(src), _d(src), _p(dst), _d(dst))
    elif dst.dtype == GGmlType.F16:
        rc = lib.galois_b200_cpy_f32_f16(ctx, _p(src), _d(src), _p(dst), _d(dst))
    else:
        raise GError(f"galois_cpy: f32 -> {dst.dtype.name} is todo!() in the reference")
    _check(ctx, rc, "galois_cpy")


def galois_cpy_pair(src0: Tensor, dst0: Tensor, src1: Tensor, dst1: Tensor) -> None:
    """Two independent f32 -> f16 galois_cpy calls (src/op.rs:3171-3185) in one launch (the K and the V
    append of a decode step).  Not part of the reference API."""
    ctx = _gpu_ctx(src0, dst0, src1, dst1)
    for t in (src0, src1):
        _want(t, GGmlType.F32, "galois_cpy_pair src")
    for t in (dst0, dst1):
        _want(t, GGmlType.F16, "galois_cpy_pair dst")
    rc = lib.galois_b200_cpy_f32_f16_pair(ctx, _p(src0), _d(src0), _p(dst0), _d(dst0), _p(src1), _d(src1), _p(dst1), _d(dst1))
    _check(ctx, rc, "galois_cpy_pair")


def galois_get_rows(src0: Tensor, src1: Tensor, dst: Tensor) -> None:
    """src/op.rs:3281-3292 (the reference implements the CPU arm only): rows `src1` (i32) of the Q4_0 table
    `src0`, dequantised, into the f32 tensor `dst` {K, number of indices}."""
    ctx = _gpu_ctx(src0, src1, dst)
    _want(src0, GGmlType.Q4_0, "galois_get_rows src0")
    _want(src1, GGmlType.I32, "galois_get_rows src1")
    _want(dst, GGmlType.F32, "galois_get_rows dst")
    _check(ctx, lib.galois_b200_get_rows_q4_0_f32(ctx, _p(src0), _d(src0), _p(src1), _d(src1), _p(dst), _d(dst)), "galois_get_rows")


def galois_cont(src: Tensor, dst: Tensor) -> None:
    """src/op.rs:3187-3201: same kernel as galois_cpy."""
    galois_cpy(src, dst)


def quantize_q8_0(x: Tensor, out_bytes) -> None:
    """``<BlockQ8_0 as QuantType>::from_f32`` per row of a contiguous F32 tensor; `out_bytes` is a
    torch CUDA uint8 buffer of rows * K/32 * 34 bytes."""
    ctx = _gpu_ctx(x)
    _want(x, GGmlType.F32, "quantize_q8_0")
    k = x.dim().shape[0]
    rc = lib.galois_b200_quantize_q8_0(ctx, _p(x), x.dim().stride[1], C.c_void_p(out_bytes.data_ptr()), k, x.dim().nrows())
    _check(ctx, rc, "quantize_q8_0")
