"""CPU tests of the oracle: against the committed golden vectors (an independent
pure-Python restatement, tests/golden/make_golden.py), AVX path against scalar
path, hand-computable cases and quantiser invariants."""
import struct

import numpy as np
import pytest
from hypothesis import given, settings
from hypothesis import strategies as st
from hypothesis.extra import numpy as hnp


def _nan_index_mask():
    idx = np.arange(65536)
    return ((idx & 0x7C00) == 0x7C00) & ((idx & 0x3FF) != 0)


def test_f16_conversion_soft_matches_f16c(oracle):
    L = oracle.lib()
    rng = np.random.default_rng(1)
    vals = np.concatenate([
        rng.standard_normal(5000).astype(np.float32) * 10.0 ** rng.integers(-8, 6, 5000).astype(np.float32),
        np.array([0.0, -0.0, 65504.0, 65519.99, 65520.0, 1e-8, 5.96e-8, 2.98e-8, 2.9802322e-8, 6.1e-5, np.inf, -np.inf], dtype=np.float32),
    ])
    for v in vals:
        assert L.orc_f32_to_f16(float(v)) == L.orc_f32_to_f16_soft(float(v)), v
    # and numpy's own RNE conversion agrees
    assert np.array_equal(oracle.f32_to_f16(vals), vals.astype(np.float16).view(np.uint16))


def test_q8_0_golden(oracle, golden):
    assert np.array_equal(oracle.quantize_q8_0(golden["q8_x"]), golden["q8_bytes"])


def test_q8_0_hand_cases(oracle):
    # zero block -> d = 0, all q = 0
    z = oracle.quantize_q8_0(np.zeros((1, 32), np.float32))[0]
    assert bytes(z) == b"\x00" * 34
    # amax = 127 -> d = 1 exactly; .5 ties round away from zero
    x = np.zeros((1, 32), np.float32)
    x[0, :6] = [127.0, 0.5, -0.5, 1.5, -2.5, 126.49]
    b = bytes(oracle.quantize_q8_0(x)[0])
    assert struct.unpack("<H", b[:2])[0] == 0x3C00
    assert list(struct.unpack("<32b", b[2:]))[:6] == [127, 1, -1, 2, -3, 126]
    # single non-zero, negative: maps to -127
    x = np.zeros((1, 32), np.float32)
    x[0, 9] = -3.0
    b = bytes(oracle.quantize_q8_0(x)[0])
    q = struct.unpack("<32b", b[2:])
    assert q[9] == -127 and sum(abs(v) for v in q) == 127


def test_q8_0_subnormal_scale_saturates(oracle):
    # amax so small that d = amax / 127 is subnormal and 1 / d overflows to +inf:
    # x * id is +-inf (or NaN for x == 0) and Rust's `as i8` saturates / maps NaN to 0
    x = np.zeros((1, 32), np.float32)
    x[0, 0], x[0, 1] = 1e-38, -1e-38
    q = struct.unpack("<32b", bytes(oracle.quantize_q8_0(x)[0])[2:])
    assert q[0] == 127 and q[1] == -128 and not any(q[2:])


def test_q8_0_rejects_ragged(oracle):
    with pytest.raises(oracle.OracleError):
        oracle.quantize_q8_0(np.zeros((1, 40), np.float32))


@settings(max_examples=60, deadline=None)
@given(hnp.arrays(np.float32, (2, 64), elements=st.floats(-1e4, 1e4, width=32).filter(lambda v: v == 0 or abs(v) > 1e-30)))
def test_q8_0_invariants(x):
    import oracle

    b = oracle.quantize_q8_0(x)
    for r in range(2):
        for i in range(2):
            blk = bytes(b[r, i * 34:(i + 1) * 34])
            q = np.array(struct.unpack("<32b", blk[2:]), dtype=np.int32)
            xs = x[r, i * 32:(i + 1) * 32]
            amax = np.abs(xs).max()
            assert np.abs(q).max() <= 127
            d = np.float32(amax) / np.float32(127)
            if d == 0:
                assert not q.any()
                continue
            idv = np.float32(1) / d
            want = np.sign(xs * idv) * np.floor(np.abs(xs * idv) + np.float32(0.5))
            assert np.array_equal(q, want.astype(np.int32))
            assert struct.unpack("<H", blk[:2])[0] == int(np.array([d]).astype(np.float16).view(np.uint16)[0])


def test_dot_golden(oracle, golden):
    nb = 3
    for xi, xr in enumerate((0, 2)):
        xq = golden["q8_bytes"][xr][: nb * 34]
        for r in range(5):
            w = golden["dot_w"][r]
            assert np.array_equal(oracle.block_isums(w, xq, avx=False), golden["dot_isums"][xi, r])
            assert np.array_equal(oracle.block_isums(w, xq, avx=True), golden["dot_isums"][xi, r])
            assert np.float32(oracle.vec_dot_q4_0_q8_0(w, xq, avx=True)) == golden["dot_avx"][xi, r]
            assert np.float32(oracle.vec_dot_q4_0_q8_0(w, xq, avx=False)) == golden["dot_scalar"][xi, r]


def test_dot_extremes_hand(oracle):
    # one block: every nibble 0 (-8), every q8 = -127, d = 1 both: 32 * (-8) * (-127) = 32512
    w = struct.pack("<H", 0x3C00) + bytes([0x00] * 16)
    xq = struct.pack("<H", 0x3C00) + struct.pack("<32b", *([-127] * 32))
    wa, xa = np.frombuffer(w, np.uint8), np.frombuffer(xq, np.uint8)
    assert oracle.block_isums(wa, xa)[0] == 32512
    assert oracle.vec_dot_q4_0_q8_0(wa, xa, True) == 32512.0
    assert oracle.vec_dot_q4_0_q8_0(wa, xa, False) == 32512.0
    # nibbles 15 (+7) against +127: 32 * 7 * 127 = 28448
    w = struct.pack("<H", 0x3C00) + bytes([0xFF] * 16)
    xq = struct.pack("<H", 0x3C00) + struct.pack("<32b", *([127] * 32))
    assert oracle.block_isums(np.frombuffer(w, np.uint8), np.frombuffer(xq, np.uint8))[0] == 28448
    # low nibble = element j, high nibble = element j + 16
    qs = bytearray(16)
    qs[3] = 0x0F | (0x00 << 4)  # element 3 -> +7, element 19 -> -8; all others 0 -> -8
    y = [0] * 32
    y[3], y[19] = 10, 3
    w = struct.pack("<H", 0x3C00) + bytes(qs)
    xq = struct.pack("<H", 0x3C00) + struct.pack("<32b", *y)
    assert oracle.block_isums(np.frombuffer(w, np.uint8), np.frombuffer(xq, np.uint8))[0] == 7 * 10 - 8 * 3


def test_dot_avx_vs_scalar_random(oracle):
    rng = np.random.default_rng(7)
    for k in (32, 256, 4096, 11008):
        w = oracle.quantize_q4_0(oracle.fill_normal(k, 100 + k, 0, 0.02)[None])[0]
        xq = oracle.quantize_q8_0(oracle.fill_normal(k, 200 + k)[None])[0]
        assert np.array_equal(oracle.block_isums(w, xq, True), oracle.block_isums(w, xq, False))
        a, s = oracle.vec_dot_q4_0_q8_0(w, xq, True), oracle.vec_dot_q4_0_q8_0(w, xq, False)
        assert abs(a - s) <= 1e-5 * max(1.0, abs(s))
        # independent cross-check: dequantise both sides, dot in f64
        wd = oracle.dequantize_q4_0(w, k)[0].astype(np.float64)
        xb = bytes(xq)
        xd = np.concatenate([
            np.array(struct.unpack("<32b", xb[i * 34 + 2:(i + 1) * 34]), np.float64)
            * float(np.frombuffer(xb[i * 34:i * 34 + 2], np.float16)[0]) for i in range(k // 32)])
        assert abs(a - wd @ xd) <= 1e-4 * np.linalg.norm(wd) * np.linalg.norm(xd) / np.sqrt(k) + 1e-6


def test_q4_0_roundtrip_layout(oracle):
    x = oracle.fill_normal(64, 5, 0, 0.02)[None]
    w = oracle.quantize_q4_0(x)
    back = oracle.dequantize_q4_0(w, 64)[0]
    # |error| <= d per element, and the element of largest magnitude maps to nibble 0 (-8) exactly
    for b in range(2):
        d = abs(float(np.frombuffer(bytes(w[0, b * 18:b * 18 + 2]), np.float16)[0]))
        assert np.all(np.abs(back[b * 32:(b + 1) * 32] - x[0, b * 32:(b + 1) * 32]) <= d * 1.01 + 1e-7)


def test_tables_golden(oracle, golden):
    nanmask = _nan_index_mask()
    for name, tab in (("exp_table", oracle.exp_f16_table()), ("silu_table", oracle.silu_f16_table())):
        want = golden[name]
        assert np.array_equal(tab[~nanmask], want[~nanmask])
        assert np.all(np.isnan(tab[nanmask].view(np.float16)))


def test_softmax_silu_golden(oracle, golden):
    assert np.array_equal(oracle.soft_max(golden["softmax_x"]), golden["softmax_y"])
    assert np.array_equal(oracle.silu(golden["silu_x"][None])[0], golden["silu_y"])
    y = oracle.soft_max(golden["softmax_x"])
    assert y[1, 5] == 0.0 and y[1, 36] == 0.0
    assert np.allclose(y.sum(axis=1), 1.0, atol=1e-6)


def test_softmax_all_masked_panics(oracle):
    with pytest.raises(oracle.OracleError):
        oracle.soft_max(np.full((1, 8), -np.inf, np.float32))


def test_softmax_ext_equals_scale_mask_softmax(oracle):
    x = oracle.fill_normal(2 * 3 * 16, 9).reshape(2, 3, 16)
    pos = np.array([4, 15], np.int32)
    got = oracle.soft_max_ext(x, 0.25, pos)
    ref = oracle.scale(x, 0.25)
    for t in range(2):
        ref[t, :, pos[t] + 1:] = -np.inf
    assert np.array_equal(got, oracle.soft_max(ref))


def test_rms_norm_golden(oracle, golden):
    assert np.array_equal(oracle.rms_norm(golden["rms_a_x"][None], 1e-6)[0], golden["rms_a_y"])
    assert np.array_equal(oracle.rms_norm(golden["rms_b_x"][None], 1e-5)[0], golden["rms_b_y"])


def test_rope_golden(oracle, golden):
    y = oracle.rope(golden["rope_x"], golden["rope_pos"], 8)
    assert np.abs(y - golden["rope_y"]).max() <= 1e-6
    # position 0 is the identity
    assert np.array_equal(y[0], golden["rope_x"][0])


def test_rope_unsupported_modes(oracle):
    x = np.zeros((1, 1, 8), np.float32)
    for mode in (2, 4):
        with pytest.raises(oracle.OracleError):
            oracle.rope(x, np.zeros(1, np.int32), 8, mode=mode)


def test_f16_dot_golden(oracle, golden):
    assert np.float32(oracle.vec_dot_f16(golden["f16_a"], golden["f16_b"], True)) == golden["f16_dot_avx"][0]
    a = oracle.vec_dot_f16(golden["f16_a"], golden["f16_b"], True)
    s = oracle.vec_dot_f16(golden["f16_a"], golden["f16_b"], False)
    assert abs(a - s) < 1e-5


def test_mul_mat_driver_matches_row_dots(oracle):
    n, k, b = 70, 96, 5  # ragged against the 16x16 tiling and the 4-way split
    w = oracle.quantize_q4_0(oracle.fill_normal(n * k, 11, 0, 0.02).reshape(n, k))
    x = oracle.fill_normal(b * k, 12).reshape(b, k)
    xq = oracle.quantize_q8_0(x)
    want = np.array([[oracle.vec_dot_q4_0_q8_0(w[i], xq[j], True) for i in range(n)] for j in range(b)], np.float32)
    for nth in (1, 2, 4, 7):
        assert np.array_equal(oracle.mul_mat_q4_0(w, x, nth=nth), want)
    # more activation rows than weight rows: the split runs over src1 rows instead
    x2 = oracle.fill_normal(80 * k, 13).reshape(80, k)
    y1 = oracle.mul_mat_q4_0(w, x2, nth=4)
    y2 = oracle.mul_mat_q4_0(w, x2, nth=1)
    assert np.array_equal(y1, y2)


def test_mul_mat_broadcast_and_errors(oracle):
    O = oracle
    k, n = 64, 8
    w = O.quantize_q4_0(O.fill_normal(n * k, 21, 0, 0.02).reshape(n, k))
    x = O.fill_normal(4 * 2 * k, 22).reshape(4, 2, k)  # ne12 = 4 broadcast over ne02 = 1
    dst = np.empty((4, 2, n), np.float32)
    O.mul_mat_q4_0_raw(w, O.Dim.contiguous([k, n], 32), x, O.Dim.contiguous([k, 2, 4]), dst, O.Dim.contiguous([n, 2, 4]))
    for h in range(4):
        assert np.array_equal(dst[h], O.mul_mat_q4_0(w, x[h]))
    with pytest.raises(O.OracleError):  # dst shape mismatch
        O.mul_mat_q4_0_raw(w, O.Dim.contiguous([k, n], 32), x, O.Dim.contiguous([k, 2, 4]), dst, O.Dim.contiguous([n, 4, 2]))
    with pytest.raises(O.OracleError):  # broadcast does not divide
        O.mul_mat_q4_0_raw(np.concatenate([w, w, w]), O.Dim.contiguous([k, n, 3], 32), x, O.Dim.contiguous([k, 2, 4]), dst, O.Dim.contiguous([n, 2, 4]))


def test_mul_mat_f16(oracle):
    rng = np.random.default_rng(3)
    a = rng.standard_normal((2, 6, 75)).astype(np.float16).view(np.uint16)
    x = rng.standard_normal((4, 3, 75)).astype(np.float32)
    y = oracle.mul_mat_f16(a, x)
    xr = oracle.f32_to_f16(x)
    for h in range(4):
        for b in range(3):
            for n in range(6):
                assert y[h, b, n] == np.float32(oracle.vec_dot_f16(a[h // 2, n], xr[h, b], True))
    ref = np.einsum("hnk,hbk->hbn", a.view(np.float16).astype(np.float64)[[0, 0, 1, 1]], xr.view(np.float16).astype(np.float64))
    assert np.abs(y - ref).max() < 1e-4


def test_add_mul_scale_cpy(oracle):
    a = oracle.fill_normal(3 * 4 * 10, 31).reshape(3, 4, 10)
    b = oracle.fill_normal(10, 32).reshape(1, 1, 10)
    assert np.array_equal(oracle.add(a, b), a + b)
    assert np.array_equal(oracle.mul(a, b), a * b)
    b2 = oracle.fill_normal(2 * 10, 33).reshape(1, 2, 10)  # modulo broadcast over rows
    assert np.array_equal(oracle.mul(a, b2), a * np.tile(b2, (3, 2, 1)))
    assert np.array_equal(oracle.scale(a, 0.125), a * np.float32(0.125))
    assert np.array_equal(oracle.cpy_f32_f16(a), a.astype(np.float16).view(np.uint16))
    # strided destination: one row written into a [rows][cols] cache at row 2
    cache = np.zeros((5, 10), np.uint16)
    src = a[0, 1]
    view = cache[2:3]
    oracle.cpy_f32_raw(src, oracle.Dim.contiguous([10]), view, oracle.Dim.make([10, 1, 1, 1], [1, 10, 10, 10]), True)
    assert np.array_equal(cache[2], src.astype(np.float16).view(np.uint16)) and not cache[[0, 1, 3, 4]].any()


def test_fill_normal_is_deterministic(oracle):
    a = oracle.fill_normal(1001, 42, 0, 0.02)
    assert np.array_equal(a, oracle.fill_normal(1001, 42, 0, 0.02))
    assert abs(a.std() - 0.02) < 2e-3 and abs(a.mean()) < 3e-3
    assert not np.array_equal(a, oracle.fill_normal(1001, 43, 0, 0.02))


def test_get_rows_q4_0(oracle):
    """GetRows over a Q4_0 table (src/op.rs:2546-2571 of galois): a hand-built block, an independent numpy
    restatement of to_f32 (src/ggml_quants.rs:209-228), repeated indices, and the out-of-range panic."""
    O = oracle
    # one block by hand: d = 0.5, byte j = j | ((15 - j) << 4)  ->  element j = (j - 8) / 2, element 16 + j = (7 - j) / 2
    blk = np.zeros(18, np.uint8)
    blk[0:2] = np.array([0.5], np.float16).view(np.uint8)
    blk[2:] = [j | ((15 - j) << 4) for j in range(16)]
    got = O.get_rows_q4_0(blk.reshape(1, 18), 32, np.array([0, 0], np.int32))
    want = np.array([(j - 8) / 2 for j in range(16)] + [(7 - j) / 2 for j in range(16)], np.float32)
    assert np.array_equal(got[0], want) and np.array_equal(got[1], want)
    # random table against a vectorised numpy restatement
    n, k = 37, 256
    w = O.quantize_q4_0(O.fill_normal(n * k, 77, 0, 0.02).reshape(n, k)).reshape(n, k // 32, 18)
    d = w[:, :, 0:2].copy().view(np.float16).astype(np.float32)            # [n][nblk][1]
    qs = w[:, :, 2:].astype(np.int32)
    lo, hi = (qs & 0x0F) - 8, (qs >> 4) - 8
    table = np.concatenate([lo.astype(np.float32) * d, hi.astype(np.float32) * d], axis=2).reshape(n, k)
    idx = np.array([5, 0, 36, 5, 17], np.int32)
    assert np.array_equal(O.get_rows_q4_0(w, k, idx), table[idx])
    with pytest.raises(O.OracleError):
        O.get_rows_q4_0(w, k, np.array([37], np.int32))
