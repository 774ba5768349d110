"""Q6K weights x Q8K activations (src/ggml_quants.rs:484-719 of galois): the oracle's restatement checked
against itself on the CPU, and the GPU path (galois_b200_mul_mat_q6k_f32 and its hooks) against the oracle."""
import ctypes as C

import numpy as np
import pytest

from conftest import assert_close


def _random_q6k(rng, n, k):
    """Arbitrary valid Q6K bytes: every nibble / bit pattern, scales over the whole int8 range."""
    nb = n * (k // 256)
    raw = rng.integers(0, 256, size=(nb, 210), dtype=np.uint8)
    raw[:, 192:208] = rng.integers(-128, 128, size=(nb, 16)).astype(np.int8).view(np.uint8)
    raw[:, 208:210] = (rng.standard_normal(nb) * 1e-3).astype(np.float16).view(np.uint8).reshape(nb, 2)
    return raw.reshape(n, -1)


# ------------------------------------------------------------------ CPU: the oracle against itself
def test_q8k_quantiser_properties(oracle):
    rng = np.random.default_rng(5)
    x = rng.standard_normal((3, 1024)).astype(np.float32)
    x[1, 256:512] = 0.0            # an all-zero block
    x[2, 7] = -9.0                 # the element of largest magnitude always maps to -128, whatever its sign
    x[2, 300], x[2, 400] = 5.0, -5.0  # a tie in magnitude: the FIRST one gives the sign, the other one saturates at 127
    blocks = oracle.quantize_q8k(x).reshape(3, 4, 292)
    d = blocks[:, :, :4].copy().view(np.float32).reshape(3, 4)
    qs = blocks[:, :, 4:260].view(np.int8)
    bs = blocks[:, :, 260:].copy().view(np.int16).reshape(3, 4, 16)
    assert d[1, 1] == 0.0 and not qs[1, 1].any()
    assert np.array_equal(bs, qs.reshape(3, 4, 16, 16).astype(np.int32).sum(-1))
    assert qs[2, 0, 7] == -128 and d[2, 0] == np.float32(1.0) / (np.float32(-128.0) / np.float32(-9.0))
    assert qs[2, 1, 300 - 256] == -128 and qs[2, 1, 400 - 256] == 127
    # dequantised values are close to the input
    assert np.abs(qs[0].astype(np.float32) * d[0][:, None] - x[0].reshape(4, 256)).max() <= np.abs(d[0]).max() * 0.5 + 1e-6


def test_q6k_dot_avx_lanes_add_up_to_the_plain_integer_sum(oracle):
    rng = np.random.default_rng(6)
    w = _random_q6k(rng, 4, 2048)
    xq = oracle.quantize_q8k(rng.standard_normal((4, 2048)).astype(np.float32) * 3)
    for r in range(4):
        assert np.array_equal(oracle.block_isums_q6k(w[r], xq[r], avx=True), oracle.block_isums_q6k(w[r], xq[r], avx=False))
    # extremes: every quant 63 (value +31), every scale 127, every activation quant -128 / 127
    blk = np.zeros(210, np.uint8)
    blk[:192] = 0xFF
    blk[192:208] = 127
    for q8, want in ((-128, 256 * 31 * 127 * -128), (127, 256 * 31 * 127 * 127)):
        y = np.zeros(292, np.uint8)
        y[4:260] = np.uint8(q8 & 0xFF)
        assert list(oracle.block_isums_q6k(blk, y, avx=False)) == [want]


def test_q6k_mat_mul_against_a_float64_dot_of_the_dequantised_values(oracle):
    n, k, b = 24, 1024, 3
    w = oracle.quantize_q6k(oracle.fill_normal(n * k, 610, 0, 0.02).reshape(n, k))
    x = oracle.fill_normal(b * k, 611).reshape(b, k)
    got = oracle.mul_mat_q6k(w, x)
    # same quantised operands, products and sums in float64
    xq = oracle.quantize_q8k(x).reshape(b, k // 256, 292)
    xdq = (xq[:, :, 4:260].view(np.int8).astype(np.float64) * xq[:, :, :4].copy().view(np.float32).astype(np.float64)).reshape(b, k)
    want = xdq @ oracle.dequantize_q6k(w, k).astype(np.float64).T
    assert_close(got, want)
    src = oracle.fill_normal(n * k, 610, 0, 0.02).reshape(n, k)
    assert np.linalg.norm(oracle.dequantize_q6k(w, k) - src) / np.linalg.norm(src) < 0.05  # the synthetic-weight quantiser is sane


# ------------------------------------------------------------------ GPU parity
@pytest.mark.gpu
@pytest.mark.parametrize("rows,k", [(1, 256), (3, 1024), (5, 4096), (2, 11008 // 256 * 256)])
def test_gpu_q8k_quantiser_bit_exact(dev, oracle, rows, k):
    import torch

    import galois_b200 as gb

    x = oracle.fill_normal(rows * k, 620 + rows).reshape(rows, k) * 2
    x[0, :256] = 0.0
    if k >= 512:
        x[-1, 300], x[-1, 301] = -7.5, 7.5
    xt = torch.from_numpy(x).to(dev.torch_device)
    out = torch.zeros(rows * (k // 256) * 292, dtype=torch.uint8, device=dev.torch_device)
    rc = gb.lib.galois_b200_quantize_q8_k(dev.ctx, C.c_void_p(xt.data_ptr()), k, C.c_void_p(out.data_ptr()), k, rows)
    assert rc == 0, gb.lib.galois_b200_last_error(dev.ctx)
    dev.synchronize()
    assert np.array_equal(out.cpu().numpy().reshape(rows, -1), oracle.quantize_q8k(x))
    assert gb.lib.galois_b200_quantize_q8_k(dev.ctx, C.c_void_p(xt.data_ptr()), k, C.c_void_p(out.data_ptr()), 100, 1) == -1


@pytest.mark.gpu
def test_gpu_q6k_block_isums_bit_exact(dev, oracle):
    import torch

    import galois_b200 as gb

    rng = np.random.default_rng(7)
    k = 4096
    w = _random_q6k(rng, 1, k)[0]
    xq = oracle.quantize_q8k(rng.standard_normal((1, k)).astype(np.float32) * 3)[0]
    blk = np.zeros(210, np.uint8)
    blk[:192] = 0xFF
    blk[192:208] = 127
    y = np.zeros(292, np.uint8)
    y[4:260] = np.uint8(-128 & 0xFF)
    for wb, xb in ((w, xq), (blk, y)):
        wt = torch.from_numpy(wb.copy()).to(dev.torch_device)
        xt = torch.from_numpy(xb.copy()).to(dev.torch_device)
        nsb = wb.size // 210
        out = torch.zeros(nsb, dtype=torch.int32, device=dev.torch_device)
        assert gb.lib.galois_b200_block_isums_q6k_q8k(dev.ctx, C.c_void_p(wt.data_ptr()), C.c_void_p(xt.data_ptr()), nsb, C.c_void_p(out.data_ptr())) == 0
        dev.synchronize()
        assert np.array_equal(out.cpu().numpy(), oracle.block_isums_q6k(wb, xb))


@pytest.mark.gpu
@pytest.mark.parametrize("n,k,b", [(4096, 4096, 1), (70, 256, 5), (1, 512, 1), (33, 1024, 3), (257, 2048, 8), (11008, 4096, 2), (4096, 11008 // 256 * 256, 1)])
def test_gpu_mul_mat_q6k(dev, oracle, n, k, b):
    import galois_b200 as gb

    G = gb.Device.Gpu(dev)
    w = oracle.quantize_q6k(oracle.fill_normal(n * k, 630 + n, 0, 0.02).reshape(n, k))
    x = oracle.fill_normal(b * k, 631 + b).reshape(b, k)
    wt = gb.Tensor.from_raw(w, (k, n), gb.GGmlType.Q6K, G)
    dst = gb.Tensor.zeros((n, b), gb.GGmlType.F32, G)
    gb.galois_matmul(wt, gb.Tensor.from_numpy(x, gb.GGmlType.F32, G), dst)
    assert_close(dst.to_numpy(), oracle.mul_mat_q6k(w, x))


@pytest.mark.gpu
def test_gpu_mul_mat_q6k_random_bytes_broadcast_and_errors(dev, oracle):
    import galois_b200 as gb

    G = gb.Device.Gpu(dev)
    rng = np.random.default_rng(8)
    n, k, b = 48, 512, 3
    w = _random_q6k(rng, n, k)
    x = rng.standard_normal((2, b, k)).astype(np.float32)  # two batched matrices sharing one weight (dims-2 broadcast)
    wt = gb.Tensor.from_raw(w, (k, n), gb.GGmlType.Q6K, G)
    dst = gb.Tensor.zeros((n, b, 2), gb.GGmlType.F32, G)
    gb.galois_matmul(wt, gb.Tensor.from_numpy(x, gb.GGmlType.F32, G), dst)
    want = np.stack([oracle.mul_mat_q6k(w, x[i]) for i in range(2)])
    assert_close(dst.to_numpy(), want, rel_l2=1e-4, max_abs=max(1e-3, 1e-4 * np.abs(want).max()))
    bad = gb.Tensor.from_numpy(np.zeros((1, 256), np.float32), gb.GGmlType.F32, G)
    with pytest.raises(gb.GError) as e:
        gb.galois_matmul(wt, bad, gb.Tensor.zeros((n, 1), gb.GGmlType.F32, G))
    assert e.value.code == -2  # K mismatch
