"""The allocation-free mat-mul entry point (collected last on purpose).

`galois_b200_mul_mat_q4_0_f32_static` serves callers that cannot touch the CUDA allocator when
they call (device memory owned by another allocator, fixed memory budgets, real-time loops): its scratch is an array built
into the library instead of a cudaMalloc'ed arena.  Checked here: it gives exactly the numbers of
the regular entry point on two calls in a row (the second smaller, so stale scratch contents
would show), and it refuses problems beyond its 4 MiB scratch with a clear message."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _run_both(gb, dev, oracle, n, k, b, seed):
    G = gb.Device.Gpu(dev)
    w = oracle.quantize_q4_0(oracle.fill_normal(n * k, seed, 0, 0.02).reshape(n, k))
    x = oracle.fill_normal(b * k, seed + 1).reshape(b, k)
    wt = gb.Tensor.from_raw(w, (k, n), gb.GGmlType.Q4_0, G)
    xt = gb.Tensor.from_numpy(x, gb.GGmlType.F32, G)
    ref = gb.Tensor.zeros((n, b), gb.GGmlType.F32, G)
    out = gb.Tensor.zeros((n, b), gb.GGmlType.F32, G)
    dev.set_mul_mat_variant(1)  # the regular entry point on the same kernels
    try:
        gb.galois_matmul(wt, xt, ref)
    finally:
        dev.set_mul_mat_variant(0)
    err = C.create_string_buffer(256)
    rc = gb.lib.galois_b200_mul_mat_q4_0_f32_static(C.c_void_p(dev.stream.cuda_stream), C.c_void_p(wt.data_ptr()),
                                                    C.byref(wt.dim().c_struct()), C.c_void_p(xt.data_ptr()),
                                                    C.byref(xt.dim().c_struct()), C.c_void_p(out.data_ptr()),
                                                    C.byref(out.dim().c_struct()), err, 256)
    assert rc == 0, err.value
    return out.to_numpy(), ref.to_numpy(), oracle.mul_mat_q4_0(w, x)


def test_static_scratch_matches_regular_entry_point(dev, oracle):
    import galois_b200 as gb
    from conftest import assert_close

    for n, k, b in ((300, 4096, 5), (64, 256, 2)):
        got, ref, want = _run_both(gb, dev, oracle, n, k, b, 5150 + n)
        assert np.array_equal(got, ref)  # same kernels, same inputs: identical bits
        assert_close(got, want)


def test_static_scratch_allocates_nothing_and_zero_fills_empty_contraction(dev, oracle):
    """Free device memory is the same before and after two calls (the scratch is part of the library
    image, already resident), and K == 0 zero-fills dst like the regular entry point."""
    import torch

    import galois_b200 as gb

    _run_both(gb, dev, oracle, 64, 256, 2, 5300)  # the device address of the scratch is resolved by now
    G = gb.Device.Gpu(dev)
    n, k, b = 128, 1024, 3
    w = oracle.quantize_q4_0(oracle.fill_normal(n * k, 5301, 0, 0.02).reshape(n, k))
    wt = gb.Tensor.from_raw(w, (k, n), gb.GGmlType.Q4_0, G)
    xt = gb.Tensor.from_numpy(oracle.fill_normal(b * k, 5302).reshape(b, k), gb.GGmlType.F32, G)
    out = gb.Tensor.zeros((n, b), gb.GGmlType.F32, G)
    err = C.create_string_buffer(256)
    args = (C.c_void_p(dev.stream.cuda_stream), C.c_void_p(wt.data_ptr()), C.byref(wt.dim().c_struct()), C.c_void_p(xt.data_ptr()),
            C.byref(xt.dim().c_struct()), C.c_void_p(out.data_ptr()), C.byref(out.dim().c_struct()), err, 256)
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(2):
        assert gb.lib.galois_b200_mul_mat_q4_0_f32_static(*args) == 0, err.value
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0, (free0, free1)

    # K == 0: every output is an empty sum
    o2 = gb.Tensor.from_numpy(np.full((b, n), 7.0, np.float32), gb.GGmlType.F32, G)
    w0 = gb.Dim(2, (0, n, 1, 1), (1, 0, 0, 0)).c_struct()
    x0 = gb.Dim(2, (0, b, 1, 1), (1, 0, 0, 0)).c_struct()
    rc = gb.lib.galois_b200_mul_mat_q4_0_f32_static(C.c_void_p(dev.stream.cuda_stream), C.c_void_p(wt.data_ptr()), C.byref(w0),
                                                    C.c_void_p(xt.data_ptr()), C.byref(x0), C.c_void_p(o2.data_ptr()),
                                                    C.byref(o2.dim().c_struct()), err, 256)
    assert rc == 0, err.value
    assert np.array_equal(o2.to_numpy(), np.zeros((b, n), np.float32))


def test_static_scratch_rejects_oversize(dev):
    import galois_b200 as gb

    G = gb.Device.Gpu(dev)
    k, n, b = 4096, 8, 2000  # 2000 rows * (4096 + 1024) bytes > 4 MiB
    wt = gb.Tensor.zeros((k, n), gb.GGmlType.Q4_0, G)
    xt = gb.Tensor.zeros((k, b), gb.GGmlType.F32, G)
    out = gb.Tensor.zeros((n, b), gb.GGmlType.F32, G)
    err = C.create_string_buffer(256)
    rc = gb.lib.galois_b200_mul_mat_q4_0_f32_static(C.c_void_p(dev.stream.cuda_stream), C.c_void_p(wt.data_ptr()),
                                                    C.byref(wt.dim().c_struct()), C.c_void_p(xt.data_ptr()),
                                                    C.byref(xt.dim().c_struct()), C.c_void_p(out.data_ptr()),
                                                    C.byref(out.dim().c_struct()), err, 256)
    assert rc == -8 and b"scratch" in err.value
