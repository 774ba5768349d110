"""GPU parity tests: every op runs through the C ABI (via the galois_* mirror) and is
compared with the CPU oracle on the same seeded inputs.

Bars: bit-exact for Q8_0 quantisation, per-block integer sums, f32->f16 copies and
the table-driven silu; relative L2 <= 1e-4 and max-abs <= 1e-3 for f32 outputs
whose summation order differs from the CPU's."""
import ctypes as C

import numpy as np
import pytest

from conftest import assert_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gb():
    import galois_b200

    return galois_b200


def _gpu(gb, dev, arr, dtype=None):
    return gb.Tensor.from_numpy(arr, dtype or gb.GGmlType.F32, gb.Device.Gpu(dev))


def _q4(gb, dev, wbytes, n, k):
    return gb.Tensor.from_raw(wbytes, (k, n), gb.GGmlType.Q4_0, gb.Device.Gpu(dev))


# ------------------------------------------------------------------ quantiser
@pytest.mark.parametrize("rows,k", [(1, 32), (1, 4096), (3, 96), (8, 11008), (5, 4096 + 32), (33, 256)])
def test_quantize_q8_0_bit_exact(gb, dev, oracle, rows, k):
    import torch

    x = oracle.fill_normal(rows * k, 1000 + rows + k).reshape(rows, k)
    if rows >= 3:
        x[1, :32] = 0.0          # zero block
        x[2, 32:64] *= 1e-20     # tiny block
        x[0, 5] = 1e30           # huge outlier
    want = oracle.quantize_q8_0(x)
    out = torch.zeros(rows * (k // 32) * 34, dtype=torch.uint8, device=dev.torch_device)
    gb.quantize_q8_0(_gpu(gb, dev, x), out)
    dev.synchronize()
    assert np.array_equal(out.cpu().numpy().reshape(rows, -1), want)


def test_quantize_q8_0_golden_and_edges(gb, dev, oracle, golden):
    import torch

    x = golden["q8_x"]
    out = torch.zeros(golden["q8_bytes"].size, dtype=torch.uint8, device=dev.torch_device)
    gb.quantize_q8_0(_gpu(gb, dev, x), out)
    dev.synchronize()
    assert np.array_equal(out.cpu().numpy().reshape(4, -1), golden["q8_bytes"])
    # subnormal scale: saturating cast, as Rust's `as i8`
    e = np.zeros((1, 32), np.float32)
    e[0, 0], e[0, 1] = 1e-38, -1e-38
    out = torch.zeros(34, dtype=torch.uint8, device=dev.torch_device)
    gb.quantize_q8_0(_gpu(gb, dev, e), out)
    dev.synchronize()
    assert np.array_equal(out.cpu().numpy()[None], oracle.quantize_q8_0(e))
    # K not a multiple of 32: the reference panics; here an error code
    bad = _gpu(gb, dev, np.zeros((1, 40), np.float32))
    with pytest.raises(gb.GError) as ei:
        gb.quantize_q8_0(bad, out)
    assert ei.value.code == -1
    # empty input is a no-op
    rc = gb.lib.galois_b200_quantize_q8_0(dev.ctx, None, 0, None, 0, 0)
    assert rc == 0


# ------------------------------------------------------------------ integer block sums
@pytest.mark.parametrize("k", [32, 96, 4096, 11008])
def test_block_isums_bit_exact(gb, dev, oracle, k):
    import torch

    w = oracle.quantize_q4_0(oracle.fill_normal(k, 50 + k, 0, 0.02)[None])[0]
    xq = oracle.quantize_q8_0(oracle.fill_normal(k, 60 + k)[None])[0]
    want = oracle.block_isums(w, xq)
    wd = torch.from_numpy(w.copy()).to(dev.torch_device)
    xd = torch.from_numpy(xq.copy()).to(dev.torch_device)
    out = torch.zeros(k // 32, dtype=torch.int32, device=dev.torch_device)
    rc = gb.lib.galois_b200_block_isums_q4_0_q8_0(dev.ctx, C.c_void_p(wd.data_ptr()), C.c_void_p(xd.data_ptr()), k // 32,
                                                  C.c_void_p(out.data_ptr()))
    assert rc == 0
    dev.synchronize()
    assert np.array_equal(out.cpu().numpy(), want)


def test_block_isums_golden_extremes(gb, dev, golden):
    import torch

    for xi, xr in enumerate((0, 2)):
        xq = torch.from_numpy(golden["q8_bytes"][xr][: 3 * 34].copy()).to(dev.torch_device)
        for r in range(5):
            w = torch.from_numpy(golden["dot_w"][r].copy()).to(dev.torch_device)
            out = torch.zeros(3, dtype=torch.int32, device=dev.torch_device)
            assert gb.lib.galois_b200_block_isums_q4_0_q8_0(dev.ctx, C.c_void_p(w.data_ptr()), C.c_void_p(xq.data_ptr()), 3,
                                                            C.c_void_p(out.data_ptr())) == 0
            dev.synchronize()
            assert np.array_equal(out.cpu().numpy(), golden["dot_isums"][xi, r])


# ------------------------------------------------------------------ Q4_0 mat-mul
def _mul_mat_case(gb, dev, oracle, n, k, b, seed, variant):
    w = oracle.quantize_q4_0(oracle.fill_normal(n * k, seed, 0, 0.02).reshape(n, k))
    x = oracle.fill_normal(b * k, seed + 1).reshape(b, k)
    want = oracle.mul_mat_q4_0(w, x)
    dst = gb.Tensor.zeros((n, b), gb.GGmlType.F32, gb.Device.Gpu(dev))
    dev.set_mul_mat_variant(variant)
    try:
        gb.galois_matmul(_q4(gb, dev, w, n, k), _gpu(gb, dev, x), dst)
        got = dst.to_numpy()
    finally:
        dev.set_mul_mat_variant(0)
    assert_close(got, want)


# config 1 of the benchmark (4096x4096, B=1) and odd shapes; variant 1 = direct kernel
@pytest.mark.parametrize("n,k,b", [(4096, 4096, 1), (70, 96, 5), (1, 32, 1), (33, 4096 + 32, 3), (257, 352, 8),
                                   (100, 256, 16), (64, 64, 33), (5, 11008, 2)])
def test_mul_mat_q4_0_direct(gb, dev, oracle, n, k, b):
    _mul_mat_case(gb, dev, oracle, n, k, b, 7000 + n + k + b, 1)


# variant 2 = the streaming GEMV (K % 256 == 0, one activation row; in-kernel cluster-cooperative quantiser)
@pytest.mark.parametrize("n,k,b", [(4096, 4096, 1), (11008, 4096, 1), (4096, 11008, 1), (1, 256, 1), (77, 512, 1), (130, 1024, 1),
                                   (301, 5120, 1), (149, 8192, 1), (500, 14336, 1), (32000, 4096, 1), (3, 16384, 1)])
def test_mul_mat_q4_0_streaming(gb, dev, oracle, n, k, b):
    _mul_mat_case(gb, dev, oracle, n, k, b, 8000 + n + k + b, 2)


def test_mul_mat_q4_0_dependent_launch_ordering(gb, dev, oracle):
    """The streaming GEMV starts before the kernel in front of it has finished (programmatic
    dependent launch) and must still see that kernel's output: scale -> mat-mul -> mat-mul chains,
    with and without the overlap, give the oracle's numbers."""
    G = gb.Device.Gpu(dev)
    n, k = 4096, 4096
    w1 = oracle.quantize_q4_0(oracle.fill_normal(n * k, 41, 0, 0.02).reshape(n, k))
    w2 = oracle.quantize_q4_0(oracle.fill_normal(n * k, 42, 0, 0.02).reshape(n, k))
    x0 = oracle.fill_normal(k, 43).reshape(1, k)
    x1 = oracle.scale(x0, 3.0)
    h = oracle.mul_mat_q4_0(w1, x1)
    want = oracle.mul_mat_q4_0(w2, h)
    t1, t2 = _q4(gb, dev, w1, n, k), _q4(gb, dev, w2, n, k)
    three = gb.Tensor.from_numpy(np.array([3.0], np.float32), gb.GGmlType.F32, gb.Device.Cpu())
    for pdl in (1, 0, 1):
        assert gb.lib.galois_b200_set_pdl(dev.ctx, pdl) == 0
        for _ in range(3):
            xs = gb.Tensor.zeros((k, 1), gb.GGmlType.F32, G)
            hid = gb.Tensor.zeros((n, 1), gb.GGmlType.F32, G)
            out = gb.Tensor.zeros((n, 1), gb.GGmlType.F32, G)
            gb.galois_scale(_gpu(gb, dev, x0), three, xs)
            gb.galois_matmul(t1, xs, hid)
            gb.galois_matmul(t2, hid, out)
            assert_close(out.to_numpy(), want)
    gb.lib.galois_b200_set_pdl(dev.ctx, 1)


# variant 3 = tcgen05 int8 tensor-core GEMM (K % 256 == 0); config 3 of the benchmark is 4096 x 4096 x 512
@pytest.mark.parametrize("n,k,b", [(128, 256, 64), (128, 512, 1), (200, 768, 33), (77, 256, 130), (4096, 4096, 512),
                                   (300, 4096, 37), (4096, 4096, 100), (1000, 11008, 65)])
def test_mul_mat_q4_0_tensor_core(gb, dev, oracle, n, k, b):
    _mul_mat_case(gb, dev, oracle, n, k, b, 9500 + n + k + b, 3)


# variant 4 = skinny mma.sync kernel (K % 256 == 0, batch <= 192 in passes of 16): config 2 at batch 4 / 8, config 5 at batch 16
@pytest.mark.parametrize("n,k,b", [(11008, 4096, 4), (4096, 11008, 8), (11008, 4096, 8), (4096, 11008, 4), (32000, 4096, 16),
                                   (16, 256, 2), (1, 256, 1), (17, 512, 3), (1185, 512, 9), (2371, 4096, 16), (149, 8192, 5),
                                   (300, 768, 12), (31, 1024, 7), (4096, 4096, 1), (500, 14336, 6), (15, 2048, 13), (4096, 4096, 37),
                                   (11008, 4096, 2), (4096, 11008, 2), (3, 256, 2), (131, 2048, 2), (2371, 4096, 5), (149, 8192, 3), (32000, 4096, 8),
                                   (200, 768, 96), (1000, 11008, 65), (128, 256, 192), (77, 512, 130)])
def test_mul_mat_q4_0_skinny(gb, dev, oracle, n, k, b):
    _mul_mat_case(gb, dev, oracle, n, k, b, 9700 + n + k + b, 4)


# automatic dispatch over the shapes of the benchmark (configs 2, 3, 5) incl. large batches
@pytest.mark.parametrize("n,k,b", [(11008, 4096, 8), (4096, 11008, 8), (4096, 4096, 512), (32000, 4096, 16), (28672, 8192, 16),
                                   (4096, 4096, 100), (300, 4096, 37)])
def test_mul_mat_q4_0_auto(gb, dev, oracle, n, k, b):
    _mul_mat_case(gb, dev, oracle, n, k, b, 9000 + n + k + b, 0)


def test_mul_mat_q4_0_linearity_full_size(gb, dev, oracle):
    """Size-independent property at config-2 size: doubling the activations (exact in
    f32 and in Q8_0: d doubles, quants unchanged) doubles the output exactly."""
    n, k = 11008, 4096
    w = oracle.quantize_q4_0(oracle.fill_normal(n * k, 123, 0, 0.02).reshape(n, k))
    x = oracle.fill_normal(4 * k, 124).reshape(4, k)
    wt = _q4(gb, dev, w, n, k)
    y1 = gb.Tensor.zeros((n, 4), gb.GGmlType.F32, gb.Device.Gpu(dev))
    y2 = gb.Tensor.zeros((n, 4), gb.GGmlType.F32, gb.Device.Gpu(dev))
    gb.galois_matmul(wt, _gpu(gb, dev, x), y1)
    gb.galois_matmul(wt, _gpu(gb, dev, 2.0 * x), y2)
    assert np.array_equal(2.0 * y1.to_numpy(), y2.to_numpy())


def test_mul_mat_q4_0_broadcast_and_strides(gb, dev, oracle):
    O = oracle
    k, n = 64, 40
    w = O.quantize_q4_0(O.fill_normal(2 * n * k, 31, 0, 0.02).reshape(2 * n, k))  # ne02 = 2
    x = O.fill_normal(4 * 3 * k, 32).reshape(4, 3, k)                            # ne12 = 4, ne11 = 3
    want = np.empty((4, 3, n), np.float32)
    O.mul_mat_q4_0_raw(w, O.Dim.contiguous([k, n, 2], 32), x, O.Dim.contiguous([k, 3, 4]), want, O.Dim.contiguous([n, 3, 4]))
    wt = gb.Tensor.from_raw(w, (k, n, 2), gb.GGmlType.Q4_0, gb.Device.Gpu(dev))
    dst = gb.Tensor.zeros((n, 3, 4), gb.GGmlType.F32, gb.Device.Gpu(dev))
    gb.galois_matmul(wt, _gpu(gb, dev, x), dst)
    assert_close(dst.to_numpy(), want)
    # padded activation rows (nb11 > K) and a padded destination (nb1 > N)
    xp = np.zeros((3, k + 32), np.float32)
    xp[:, :k] = x[0]
    xt = _gpu(gb, dev, xp).view((k, 3), (1, k + 32, 3 * (k + 32), 3 * (k + 32)))
    big = gb.Tensor.zeros((n + 8, 3), gb.GGmlType.F32, gb.Device.Gpu(dev))
    dv = big.view((n, 3), (1, n + 8, 3 * (n + 8), 3 * (n + 8)))
    w0 = gb.Tensor.from_raw(w[:n], (k, n), gb.GGmlType.Q4_0, gb.Device.Gpu(dev))
    gb.galois_matmul(w0, xt, dv)
    got = big.to_numpy()
    assert_close(got[:, :n], want[0])
    assert not got[:, n:].any()


def test_mul_mat_q4_0_errors(gb, dev, oracle):
    G = gb.Device.Gpu(dev)
    w = gb.Tensor.zeros((64, 8), gb.GGmlType.Q4_0, G)
    x = gb.Tensor.zeros((64, 2), gb.GGmlType.F32, G)
    for shape, code in (((8, 3), -2), ((9, 2), -2)):
        with pytest.raises(gb.GError) as ei:
            gb.galois_matmul(w, x, gb.Tensor.zeros(shape, gb.GGmlType.F32, G))
        assert ei.value.code == code
    with pytest.raises(gb.GError) as ei:   # K mismatch
        gb.galois_matmul(w, gb.Tensor.zeros((32, 2), gb.GGmlType.F32, G), gb.Tensor.zeros((8, 2), gb.GGmlType.F32, G))
    assert ei.value.code == -2
    with pytest.raises(gb.GError) as ei:   # transposed destination
        d = gb.Tensor.zeros((8, 2), gb.GGmlType.F32, G).view((8, 2), (2, 1, 16, 16))
        gb.galois_matmul(w, x, d)
    assert ei.value.code == -4
    with pytest.raises(gb.GError) as ei:   # src0 batch does not divide src1 batch
        w3 = gb.Tensor.zeros((64, 8, 3), gb.GGmlType.Q4_0, G)
        gb.galois_matmul(w3, gb.Tensor.zeros((64, 2, 4), gb.GGmlType.F32, G), gb.Tensor.zeros((8, 2, 4), gb.GGmlType.F32, G))
    assert ei.value.code == -5
    # forced variants refuse shapes they cannot take
    dev.set_mul_mat_variant(2)
    try:
        with pytest.raises(gb.GError) as ei:
            gb.galois_matmul(w, x, gb.Tensor.zeros((8, 2), gb.GGmlType.F32, G))
        assert ei.value.code == -3
    finally:
        dev.set_mul_mat_variant(0)
    # empty batch is a no-op
    gb.galois_matmul(w, gb.Tensor.zeros((64, 0), gb.GGmlType.F32, G), gb.Tensor.zeros((8, 0), gb.GGmlType.F32, G))


def test_mul_mat_q4_0_host_entry(gb, dev, oracle):
    n, k, b = 4096, 4096, 4
    w = oracle.quantize_q4_0(oracle.fill_normal(n * k, 77, 0, 0.02).reshape(n, k))
    x = oracle.fill_normal(b * k, 78).reshape(b, k)
    wt = _q4(gb, dev, w, n, k)
    out = np.zeros((b, n), np.float32)
    xd = gb.Dim.ggml((k, b), gb.GGmlType.F32).c_struct()
    dd = gb.Dim.ggml((n, b), gb.GGmlType.F32).c_struct()
    for _ in range(2):
        rc = gb.lib.galois_b200_mul_mat_q4_0_f32_host(dev.ctx, C.c_void_p(wt.data_ptr()), C.byref(wt.dim().c_struct()),
                                                      x.ctypes.data_as(C.c_void_p), C.byref(xd),
                                                      out.ctypes.data_as(C.c_void_p), C.byref(dd))
        assert rc == 0, gb.lib.galois_b200_last_error(dev.ctx)
        assert_close(out, oracle.mul_mat_q4_0(w, x))
    # pinned (device-mapped) host buffers: the kernel writes the result into host memory itself
    import torch

    xp = torch.from_numpy(x).pin_memory()
    op = torch.zeros(b, n, dtype=torch.float32).pin_memory()
    for _ in range(2):
        rc = gb.lib.galois_b200_mul_mat_q4_0_f32_host(dev.ctx, C.c_void_p(wt.data_ptr()), C.byref(wt.dim().c_struct()),
                                                      C.c_void_p(xp.data_ptr()), C.byref(xd), C.c_void_p(op.data_ptr()), C.byref(dd))
        assert rc == 0, gb.lib.galois_b200_last_error(dev.ctx)
        assert_close(op.numpy().copy(), oracle.mul_mat_q4_0(w, x))
        op.zero_()


# ------------------------------------------------------------------ F16 mat-mul
@pytest.mark.parametrize("h,hx,n,k,b", [(32, 32, 2048, 128, 1), (32, 32, 128, 2048, 1), (2, 4, 6, 75, 3), (1, 1, 300, 40, 5),
                                        (4, 8, 64, 16, 2), (1, 1, 9, 8, 1)])
def test_mul_mat_f16(gb, dev, oracle, h, hx, n, k, b):
    rng = np.random.default_rng(h * 1000 + n + k)
    a = rng.standard_normal((h, n, k)).astype(np.float16)
    x = oracle.fill_normal(hx * b * k, 900 + n + k).reshape(hx, b, k)
    want = oracle.mul_mat_f16(a.view(np.uint16), x)
    at = _gpu(gb, dev, a, gb.GGmlType.F16)
    dst = gb.Tensor.zeros((n, b, hx), gb.GGmlType.F32, gb.Device.Gpu(dev))
    gb.galois_matmul(at, _gpu(gb, dev, x), dst)
    assert_close(dst.to_numpy().reshape(hx, b, n), want)


# ------------------------------------------------------------------ row ops
@pytest.mark.parametrize("rows,k", [(1, 4096), (3, 70), (2, 20), (4, 11008), (1, 32), (5, 1000)])
def test_rms_norm(gb, dev, oracle, rows, k):
    x = oracle.fill_normal(rows * k, 300 + k).reshape(rows, k)
    y = gb.Tensor.zeros((k, rows), gb.GGmlType.F32, gb.Device.Gpu(dev))
    gb.galois_rms_norm(_gpu(gb, dev, x), y, 1e-6)
    assert_close(y.to_numpy(), oracle.rms_norm(x, 1e-6))


def test_rms_norm_golden_and_inplace(gb, dev, golden):
    for key, eps in (("rms_a", 1e-6), ("rms_b", 1e-5)):
        x = golden[key + "_x"][None]
        t = _gpu(gb, dev, x)
        gb.galois_rms_norm(t, t, eps)
        assert_close(t.to_numpy()[0], golden[key + "_y"], rel_l2=1e-6, max_abs=1e-6)


@pytest.mark.parametrize("toks,heads,hd,pos0", [(1, 32, 128, 2047), (3, 2, 8, 0), (5, 4, 64, 100), (2, 1, 256, 4000)])
def test_rope(gb, dev, oracle, toks, heads, hd, pos0):
    x = oracle.fill_normal(toks * heads * hd, 400 + hd).reshape(toks, heads, hd)
    pos = (pos0 + np.arange(toks) * 7).astype(np.int32)
    want = oracle.rope(x, pos, hd)
    y = gb.Tensor.zeros((hd, heads, toks), gb.GGmlType.F32, gb.Device.Gpu(dev))
    gb.galois_rope_custom(gb.RopeCustomOption(n_dims=hd), _gpu(gb, dev, x), _gpu(gb, dev, pos, gb.GGmlType.I32), y)
    assert_close(y.to_numpy(), want, rel_l2=1e-5, max_abs=1e-5)


def test_rope_options_and_errors(gb, dev, oracle, golden):
    G = gb.Device.Gpu(dev)
    x, pos = golden["rope_x"], golden["rope_pos"]
    y = gb.Tensor.zeros((8, 2, 3), gb.GGmlType.F32, G)
    gb.galois_rope_custom(gb.RopeCustomOption(n_dims=8), _gpu(gb, dev, x), _gpu(gb, dev, pos, gb.GGmlType.I32), y)
    assert_close(y.to_numpy(), golden["rope_y"], rel_l2=1e-6, max_abs=1e-6)
    # freq_scale, a different base, xpos
    for kw in (dict(freq_scale=0.5), dict(freq_base=500000.0), dict(xpos_base=512.0), dict(xpos_base=512.0, xpos_down=True)):
        want = oracle.rope(x, pos, 8, **kw)
        gb.galois_rope_custom(gb.RopeCustomOption(n_dims=8, **kw), _gpu(gb, dev, x), _gpu(gb, dev, pos, gb.GGmlType.I32), y)
        assert_close(y.to_numpy(), want, rel_l2=2e-5, max_abs=2e-5)
    for mode in (2, 4):   # todo!() in the reference
        with pytest.raises(gb.GError) as ei:
            gb.galois_rope_custom(gb.RopeCustomOption(n_dims=8, mode=mode), _gpu(gb, dev, x), _gpu(gb, dev, pos, gb.GGmlType.I32), y)
        assert ei.value.code == -6
    with pytest.raises(gb.GError):   # n_dims odd
        gb.galois_rope_custom(gb.RopeCustomOption(n_dims=7), _gpu(gb, dev, x), _gpu(gb, dev, pos, gb.GGmlType.I32), y)


@pytest.mark.parametrize("rows,nc", [(32, 2048), (3, 37), (1, 1), (2, 5000), (7, 1024)])
def test_soft_max(gb, dev, oracle, rows, nc):
    x = (oracle.fill_normal(rows * nc, 500 + nc) * 3).reshape(rows, nc)
    if nc > 5:
        x[0, 3] = -np.inf
        x[-1, nc - 1] = -np.inf
    want = oracle.soft_max(x)
    y = gb.Tensor.zeros((nc, rows), gb.GGmlType.F32, gb.Device.Gpu(dev))
    gb.galois_soft_max(_gpu(gb, dev, x), y)
    got = y.to_numpy()
    assert_close(got, want, rel_l2=1e-5, max_abs=1e-6)
    assert np.array_equal(got == 0, want == 0)


def test_soft_max_golden(gb, dev, golden):
    x = golden["softmax_x"]
    y = gb.Tensor.zeros((37, 3), gb.GGmlType.F32, gb.Device.Gpu(dev))
    gb.galois_soft_max(_gpu(gb, dev, x), y)
    assert_close(y.to_numpy(), golden["softmax_y"], rel_l2=1e-6, max_abs=1e-7)


@pytest.mark.parametrize("toks,heads,nc", [(1, 32, 2048), (3, 4, 64), (2, 2, 37)])
def test_soft_max_ext(gb, dev, oracle, toks, heads, nc):
    x = (oracle.fill_normal(toks * heads * nc, 600 + nc) * 4).reshape(toks, heads, nc)
    pos = np.array([nc - 1 - 5 * t for t in range(toks)], np.int32)
    scale = float(1.0 / np.sqrt(np.float32(128)))
    want = oracle.soft_max_ext(x, scale, pos)
    y = gb.Tensor.zeros((nc, heads, toks), gb.GGmlType.F32, gb.Device.Gpu(dev))
    gb.galois_soft_max_ext(_gpu(gb, dev, x), y, scale, _gpu(gb, dev, pos, gb.GGmlType.I32))
    got = y.to_numpy()
    assert_close(got, want, rel_l2=1e-5, max_abs=1e-6)
    for t in range(toks):
        assert not got[t, :, pos[t] + 1:].any()
    # without a mask it is scale + soft_max
    gb.galois_soft_max_ext(_gpu(gb, dev, x), y, scale, None)
    assert_close(y.to_numpy(), oracle.soft_max(oracle.scale(x, scale)), rel_l2=1e-5, max_abs=1e-6)


@pytest.mark.parametrize("rows,nc", [(1, 11008), (3, 50), (2, 1)])
def test_silu_bit_exact(gb, dev, oracle, rows, nc):
    x = (oracle.fill_normal(rows * nc, 700 + nc) * 4).reshape(rows, nc)
    y = gb.Tensor.zeros((nc, rows), gb.GGmlType.F32, gb.Device.Gpu(dev))
    gb.galois_unary(_gpu(gb, dev, x), y, gb.UnaryOp.Silu)
    assert np.array_equal(y.to_numpy(), oracle.silu(x))
    with pytest.raises(gb.GError):
        gb.galois_unary(_gpu(gb, dev, x), y, gb.UnaryOp.Gelu)


def test_silu_golden(gb, dev, golden):
    y = gb.Tensor.zeros((50,), gb.GGmlType.F32, gb.Device.Gpu(dev))
    gb.galois_unary(_gpu(gb, dev, golden["silu_x"]), y, gb.UnaryOp.Silu)
    assert np.array_equal(y.to_numpy(), golden["silu_y"])


def test_add_mul_scale_bit_exact(gb, dev, oracle):
    G = gb.Device.Gpu(dev)
    a = oracle.fill_normal(3 * 4 * 4096, 801).reshape(3, 4, 4096)
    for bshape in ((1, 1, 4096), (1, 2, 4096), (3, 4, 4096)):
        b = oracle.fill_normal(int(np.prod(bshape)), 802).reshape(bshape)
        for fn, ofn in ((gb.galois_add, oracle.add), (gb.galois_mul, oracle.mul)):
            dst = gb.Tensor.zeros((4096, 4, 3), gb.GGmlType.F32, G)
            fn(_gpu(gb, dev, a), _gpu(gb, dev, b), dst)
            assert np.array_equal(dst.to_numpy(), ofn(a, b))
    s = gb.Tensor.from_numpy(np.array([0.08838835], np.float32), gb.GGmlType.F32, gb.Device.Cpu())
    dst = gb.Tensor.zeros((4096, 4, 3), gb.GGmlType.F32, G)
    gb.galois_scale(_gpu(gb, dev, a), s, dst)
    assert np.array_equal(dst.to_numpy(), oracle.scale(a, 0.08838835))
    with pytest.raises(gb.GError):   # shape mismatch
        gb.galois_add(_gpu(gb, dev, a), _gpu(gb, dev, a), gb.Tensor.zeros((4096, 4, 2), gb.GGmlType.F32, G))


def test_cpy_bit_exact(gb, dev, oracle):
    G = gb.Device.Gpu(dev)
    x = oracle.fill_normal(2 * 5 * 64, 811).reshape(2, 5, 64) * 100
    # contiguous f32 -> f16
    d16 = gb.Tensor.zeros((64, 5, 2), gb.GGmlType.F16, G)
    gb.galois_cpy(_gpu(gb, dev, x), d16)
    assert np.array_equal(d16.to_numpy().view(np.uint16), oracle.cpy_f32_f16(x))
    # KV-cache append: one token's [heads][head_dim] row into row `p` of a [heads][ctx][head_dim] f16 cache
    heads, hd, ctxlen, p = 4, 16, 10, 7
    k_new = oracle.fill_normal(heads * hd, 812).reshape(heads, hd)
    cache = gb.Tensor.zeros((hd, ctxlen, heads), gb.GGmlType.F16, G)
    row = cache.view((hd, 1, heads), (1, hd, hd * ctxlen, hd * ctxlen * heads), offset=p * hd)
    src = _gpu(gb, dev, k_new).view((hd, 1, heads), (1, hd, hd, hd * heads))
    gb.galois_cpy(src, row)
    got = cache.to_numpy().view(np.uint16)
    want = np.zeros((heads, ctxlen, hd), np.uint16)
    want[:, p, :] = oracle.f32_to_f16(k_new)
    assert np.array_equal(got, want)
    # transposed source -> contiguous f32 (galois_cont)
    xt = _gpu(gb, dev, x[0]).view((5, 64), (64, 1, 320, 320))
    dst = gb.Tensor.zeros((5, 64), gb.GGmlType.F32, G)
    gb.galois_cont(xt, dst)
    assert np.array_equal(dst.to_numpy(), x[0].T)
    with pytest.raises(gb.GError):   # element counts differ
        gb.galois_cpy(_gpu(gb, dev, x), gb.Tensor.zeros((64, 5), gb.GGmlType.F32, G))


def test_two_op_fusions_are_bit_identical(gb, dev, oracle):
    """rms_norm_mul == rms_norm then mul; silu_mul == silu then mul: on the GPU bit for bit, and
    against the oracle's two-op sequence."""
    O = oracle
    G = gb.Device.Gpu(dev)
    for (k, rows, seed) in [(4096, 1, 1), (70, 5, 2), (11008, 3, 3)]:
        x = O.fill_normal(rows * k, 600 + seed).reshape(rows, k)
        w = 1.0 + 0.1 * O.fill_normal(k, 700 + seed).reshape(1, k)
        u = O.fill_normal(rows * k, 800 + seed).reshape(rows, k)
        xt, wt, ut = _gpu(gb, dev, x), _gpu(gb, dev, w), _gpu(gb, dev, u)
        y1, y2, t = (gb.Tensor.zeros((k, rows), gb.GGmlType.F32, G) for _ in range(3))
        gb.galois_rms_norm(xt, t, 1e-6)
        gb.galois_mul(t, wt, y1)
        gb.galois_rms_norm_mul(xt, wt, y2, 1e-6)
        assert np.array_equal(y1.to_numpy(), y2.to_numpy())
        assert_close(y2.to_numpy(), O.mul(O.rms_norm(x, 1e-6), w))
        gb.galois_unary(xt, t, gb.UnaryOp.Silu)
        gb.galois_mul(t, ut, y1)
        gb.galois_silu_mul(xt, ut, y2)
        assert np.array_equal(y1.to_numpy(), y2.to_numpy())
        assert np.array_equal(y2.to_numpy(), O.mul(O.silu(x), u))
    # mat-mul + residual: inside the GEMV at one activation row, two launches otherwise
    for (n, k, b, seed) in [(4096, 4096, 1, 11), (4096, 11008, 1, 12), (1185, 512, 1, 13), (11008, 4096, 4, 14), (70, 96, 2, 15)]:
        wq = O.quantize_q4_0(O.fill_normal(n * k, 900 + seed, 0, 0.02).reshape(n, k))
        x = O.fill_normal(b * k, 910 + seed).reshape(b, k)
        r = O.fill_normal(b * n, 920 + seed).reshape(b, n)
        wt, xt, rt = _q4(gb, dev, wq, n, k), _gpu(gb, dev, x), _gpu(gb, dev, r)
        y1, y2, t = (gb.Tensor.zeros((n, b), gb.GGmlType.F32, G) for _ in range(3))
        gb.galois_matmul(wt, xt, t)
        gb.galois_add(rt, t, y1)
        gb.galois_matmul_add(wt, xt, rt, y2)
        assert np.array_equal(y1.to_numpy(), y2.to_numpy())
        assert_close(y2.to_numpy(), O.add(r, O.mul_mat_q4_0(wq, x)))
    # prologue + mat-mul + residual in one call: one launch at one activation row, separate ops otherwise
    for (n, k, b, seed) in [(4096, 4096, 1, 21), (4096, 11008, 1, 22), (1185, 512, 1, 23), (2048, 1024, 3, 24), (70, 96, 1, 25)]:
        wq = O.quantize_q4_0(O.fill_normal(n * k, 1000 + seed, 0, 0.02).reshape(n, k))
        x = O.fill_normal(b * k, 1010 + seed).reshape(b, k)
        u = O.fill_normal(b * k, 1020 + seed).reshape(b, k)
        gain = 1.0 + 0.1 * O.fill_normal(k, 1030 + seed).reshape(1, k)
        r = O.fill_normal(b * n, 1040 + seed).reshape(b, n)
        wt, xt, ut, gt, rt = _q4(gb, dev, wq, n, k), _gpu(gb, dev, x), _gpu(gb, dev, u), _gpu(gb, dev, gain), _gpu(gb, dev, r)
        t = gb.Tensor.zeros((k, b), gb.GGmlType.F32, G)
        y1, y2, y3 = (gb.Tensor.zeros((n, b), gb.GGmlType.F32, G) for _ in range(3))
        l0 = dev.launch_count()
        gb.galois_matmul_fused(wt, xt, y2, rms_gain=gt, eps=1e-6, res=rt)
        launches = dev.launch_count() - l0
        gb.galois_rms_norm(xt, t, 1e-6)
        gb.galois_mul(t, gt, t)
        gb.galois_matmul(wt, t, y3)
        gb.galois_add(rt, y3, y1)
        assert np.array_equal(y1.to_numpy(), y2.to_numpy()), (n, k, b)
        if b == 1 and k % 256 == 0:
            assert launches == 1
        assert_close(y2.to_numpy(), O.add(r, O.mul_mat_q4_0(wq, O.mul(O.rms_norm(x, 1e-6), gain))))
        gb.galois_matmul_fused(wt, xt, y2, silu_mul=ut)
        gb.galois_unary(xt, t, gb.UnaryOp.Silu)
        gb.galois_mul(t, ut, t)
        gb.galois_matmul(wt, t, y1)
        assert np.array_equal(y1.to_numpy(), y2.to_numpy()), (n, k, b)
        assert_close(y2.to_numpy(), O.mul_mat_q4_0(wq, O.mul(O.silu(x), u)))
    # argument errors of the fused call
    from galois_b200._lib import GaloisPrologue
    wt, xt = _q4(gb, dev, O.quantize_q4_0(O.fill_normal(8 * 256, 5, 0, 0.02).reshape(8, 256)), 8, 256), _gpu(gb, dev, O.fill_normal(256, 6).reshape(1, 256))
    yt = gb.Tensor.zeros((8, 1), gb.GGmlType.F32, G)
    fused = lambda pro, res, rd: gb.lib.galois_b200_mul_mat_q4_0_f32_fused(  # noqa: E731
        dev.ctx, C.c_void_p(wt.data_ptr()), C.byref(wt.dim().c_struct()), C.c_void_p(xt.data_ptr()), C.byref(xt.dim().c_struct()), pro, res, rd,
        C.c_void_p(yt.data_ptr()), C.byref(yt.dim().c_struct()))
    pro = GaloisPrologue()
    pro.kind = 7
    assert fused(C.byref(pro), None, None) == -1          # unknown prologue
    pro.kind, pro.aux = 1, None
    assert fused(C.byref(pro), None, None) == -1          # rms_norm without its gain row
    wrong = gb.Tensor.zeros((9, 1), gb.GGmlType.F32, G)
    assert fused(None, C.c_void_p(wrong.data_ptr()), C.byref(wrong.dim().c_struct())) == -2  # residual of another shape
    assert fused(None, None, None) == 0                   # no prologue, no residual: the plain mat-mul
    # shape errors
    bad = gb.Tensor.zeros((8, 2), gb.GGmlType.F32, G)
    with pytest.raises(gb.GError) as ei:
        gb.galois_silu_mul(_gpu(gb, dev, np.zeros((2, 16), np.float32)), bad, gb.Tensor.zeros((16, 2), gb.GGmlType.F32, G))
    assert ei.value.code == -2
    with pytest.raises(gb.GError) as ei:
        gb.galois_rms_norm_mul(_gpu(gb, dev, np.zeros((2, 16), np.float32)), bad, gb.Tensor.zeros((16, 2), gb.GGmlType.F32, G), 1e-6)
    assert ei.value.code == -2


def test_cpy_pair_equals_two_copies(gb, dev, oracle):
    """The paired f32 -> f16 copy (K and V cache appends in one launch) writes what two galois_cpy calls write."""
    G = gb.Device.Gpu(dev)
    hd, nh, ctx, pos = 64, 4, 32, 7
    k = oracle.fill_normal(hd * nh, 51).reshape(nh, 1, hd)
    v = oracle.fill_normal(hd * nh, 52).reshape(nh, hd, 1)
    kt, vt = _gpu(gb, dev, k), _gpu(gb, dev, v)
    caches = []
    for paired in (False, True):
        kc = gb.Tensor.zeros((hd, ctx, nh), gb.GGmlType.F16, G)
        vc = gb.Tensor.zeros((ctx, hd, nh), gb.GGmlType.F16, G)
        k_dst = kc.view((hd, 1, nh), (1, hd, hd * ctx, hd * ctx * nh), offset=pos * hd)
        v_dst = vc.view((1, hd, nh), (1, ctx, hd * ctx, hd * ctx * nh), offset=pos)
        if paired:
            gb.galois_cpy_pair(kt, k_dst, vt, v_dst)
        else:
            gb.galois_cpy(kt, k_dst)
            gb.galois_cpy(vt, v_dst)
        caches.append((kc.to_numpy().view(np.uint16), vc.to_numpy().view(np.uint16)))
    assert np.array_equal(caches[0][0], caches[1][0]) and np.array_equal(caches[0][1], caches[1][1])
    assert caches[1][0].any() and caches[1][1].any()
    with pytest.raises(gb.GError) as ei:
        gb.galois_cpy_pair(kt, gb.Tensor.zeros((hd, 1, nh + 1), gb.GGmlType.F16, G), vt, gb.Tensor.zeros((1, hd, nh), gb.GGmlType.F16, G))
    assert ei.value.code == -2


@pytest.mark.parametrize("n,k,idx", [(32000, 4096, [0, 31999, 17, 17, 4096, 1]), (37, 256, [5, 0, 36]), (3, 32, [2]), (100, 11008, list(range(0, 100, 7)))])
def test_get_rows_q4_0(gb, dev, oracle, n, k, idx):
    """galois_get_rows over a Q4_0 table (the embedding look-up): bit-exact against the oracle, contiguous and strided dst."""
    O = oracle
    G = gb.Device.Gpu(dev)
    w = O.quantize_q4_0(O.fill_normal(n * k, 3000 + n + k, 0, 0.02).reshape(n, k))
    idx = np.array(idx, np.int32)
    want = O.get_rows_q4_0(w, k, idx)
    wt = _q4(gb, dev, w, n, k)
    it = gb.Tensor.from_numpy(idx, gb.GGmlType.I32, G)
    dst = gb.Tensor.zeros((k, len(idx)), gb.GGmlType.F32, G)
    gb.galois_get_rows(wt, it, dst)
    assert np.array_equal(dst.to_numpy(), want)
    wide = gb.Tensor.zeros((k + 32, len(idx)), gb.GGmlType.F32, G)  # rows of a wider buffer
    view = wide.view((k, len(idx)), (1, k + 32, (k + 32) * len(idx), (k + 32) * len(idx)))
    gb.galois_get_rows(wt, it, view)
    got = wide.to_numpy()
    assert np.array_equal(got[:, :k], want) and not got[:, k:].any()


def test_get_rows_q4_0_errors(gb, dev, oracle):
    G = gb.Device.Gpu(dev)
    w = oracle.quantize_q4_0(oracle.fill_normal(4 * 64, 9, 0, 0.02).reshape(4, 64))
    wt = _q4(gb, dev, w, 4, 64)
    it = gb.Tensor.from_numpy(np.array([1, 4], np.int32), gb.GGmlType.I32, G)  # 4 is outside the table
    dst = gb.Tensor.zeros((64, 2), gb.GGmlType.F32, G)
    gb.galois_get_rows(wt, it, dst)
    with pytest.raises(gb.GError) as ei:
        dev.synchronize()
    assert ei.value.code == -1
    got = dst.to_numpy()
    assert np.array_equal(got[0], oracle.get_rows_q4_0(w, 64, np.array([1], np.int32))[0]) and not got[1].any()
    with pytest.raises(gb.GError) as ei:  # dst of the wrong shape
        gb.galois_get_rows(wt, it, gb.Tensor.zeros((64, 3), gb.GGmlType.F32, G))
    assert ei.value.code == -2
    gb.galois_get_rows(wt, gb.Tensor.from_numpy(np.array([3], np.int32), gb.GGmlType.I32, G), gb.Tensor.zeros((64, 1), gb.GGmlType.F32, G))
    dev.synchronize()  # the context is fine
