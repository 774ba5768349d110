"""Generates ``golden_small.npz``: small known-answer vectors for the CPU oracle.

The galois reference holds no golden vectors for this path and cannot be built
in this image, so these vectors come from a SECOND, independent restatement of
the reference's arithmetic written here in plain Python / numpy scalar float32
operations (no SIMD, no C): they pin the C++ oracle against a differently
written implementation of the same source lines, not against a run of the
reference itself.

Run:  python tests/golden/make_golden.py   (writes next to this file)

Citations are paths inside the galois repository.
"""
from __future__ import annotations

import math
import os
import struct

import numpy as np

F = np.float32
HERE = os.path.dirname(os.path.abspath(__file__))


def f16_bits(x: float) -> int:
    """IEEE binary32 -> binary16 bits, round to nearest even (numpy's conversion is RNE)."""
    return int(np.array([x], dtype=np.float32).astype(np.float16).view(np.uint16)[0])


def f16_val(bits: int) -> np.float32:
    return F(np.array([bits], dtype=np.uint16).view(np.float16)[0])


def round_half_away(x: np.float32) -> int:
    """Rust f32::round."""
    x = float(x)
    return int(math.floor(abs(x) + 0.5)) * (1 if x >= 0 else -1)


def quantize_q8_0(row: np.ndarray) -> bytes:
    """src/ggml_quants.rs:736-764"""
    out = b""
    for i in range(len(row) // 32):
        xs = row[i * 32 : (i + 1) * 32].astype(np.float32)
        amax = F(0)
        for v in xs:
            amax = max(amax, abs(v))
        d = F(amax) / F(127)
        idv = F(1) / d if d != 0 else F(0)
        q = [round_half_away(F(v) * idv) for v in xs]
        out += struct.pack("<H", f16_bits(d)) + struct.pack("<32b", *q)
    return out


def block_isums(w: bytes, xq: bytes):
    """Integer part of src/ggml_quants.rs:174-191."""
    nb = len(w) // 18
    res = []
    for i in range(nb):
        qs = w[i * 18 + 2 : i * 18 + 18]
        ys = struct.unpack("<32b", xq[i * 34 + 2 : i * 34 + 34])
        s = 0
        for j in range(16):
            s += ((qs[j] & 0x0F) - 8) * ys[j] + ((qs[j] >> 4) - 8) * ys[j + 16]
        res.append(s)
    return res


def dot_scalar(w: bytes, xq: bytes) -> np.float32:
    """vec_dot_unopt, src/ggml_quants.rs:174-191: sumf += sum_i as f32 * dw * dx."""
    sumf = F(0)
    for i, s in enumerate(block_isums(w, xq)):
        dw = f16_val(struct.unpack("<H", w[i * 18 : i * 18 + 2])[0])
        dx = f16_val(struct.unpack("<H", xq[i * 34 : i * 34 + 2])[0])
        sumf = F(sumf + F(F(F(s) * dw) * dx))
    return sumf


def fma32(a, b, c) -> np.float32:
    return F(float(a) * float(b) + float(c))


def dot_avx(w: bytes, xq: bytes) -> np.float32:
    """vec_dot_q8_0, src/ggml_quants.rs:156-172 + helpers :55-90: lane l of 8 sums the four
    products 4l..4l+3 (maddubs pairs, madd pairs); acc = fma(dw*dx, lane, acc); hsum_float_8."""
    acc = [F(0)] * 8
    for i in range(len(w) // 18):
        qs = w[i * 18 + 2 : i * 18 + 18]
        ys = struct.unpack("<32b", xq[i * 34 + 2 : i * 34 + 34])
        dw = f16_val(struct.unpack("<H", w[i * 18 : i * 18 + 2])[0])
        dx = f16_val(struct.unpack("<H", xq[i * 34 : i * 34 + 2])[0])
        d = F(dw * dx)
        el = [(qs[j] & 0x0F) - 8 for j in range(16)] + [(qs[j] >> 4) - 8 for j in range(16)]
        for l in range(8):
            lane = sum(el[4 * l + t] * ys[4 * l + t] for t in range(4))
            acc[l] = fma32(d, F(lane), acc[l])
    r = [F(acc[l] + acc[l + 4]) for l in range(4)]  # high half + low half
    r2 = [F(r[0] + r[2]), F(r[1] + r[3])]          # movehl
    return F(r2[0] + r2[1])                         # movehdup


def exp_table():
    """src/op.rs:245-252: entry i = f16(exp(f32(f16::from_bits(i)))); exp taken in double."""
    t = np.zeros(65536, dtype=np.uint16)
    for i in range(65536):
        v = float(f16_val(i))
        if math.isnan(v):
            t[i] = f16_bits(float("nan"))
            continue
        try:
            e = math.exp(v)
        except OverflowError:
            e = float("inf")
        with np.errstate(over="ignore"):
            t[i] = f16_bits(np.float32(e))
    return t


def silu_table():
    """src/op.rs:227-234 with compute_silu (src/op.rs:88-90): x / (1 + exp(-x)), f32 steps."""
    t = np.zeros(65536, dtype=np.uint16)
    for i in range(65536):
        v = f16_val(i)
        if math.isnan(float(v)):
            t[i] = f16_bits(float("nan"))
            continue
        try:
            e = math.exp(-float(v))
        except OverflowError:
            e = float("inf")
        with np.errstate(over="ignore", invalid="ignore"):
            t[i] = f16_bits(F(v) / F(F(1) + F(e)))
    return t


def softmax_row(row: np.ndarray, tab: np.ndarray) -> np.ndarray:
    """src/lib.rs:564-592"""
    mx = F(-np.inf)
    for v in row:
        mx = max(mx, F(v))
    out = np.zeros(len(row), dtype=np.float32)
    s = F(0)
    for i, v in enumerate(row):
        if v == -np.inf:
            out[i] = 0
        else:
            val = f16_val(int(tab[f16_bits(F(v) - mx)]))
            s = F(s + val)
            out[i] = val
    inv = F(1) / s
    return (out * inv).astype(np.float32)


def rms_norm_row(x: np.ndarray, eps: float) -> np.ndarray:
    """src/lib.rs:594-604: squares summed over the first len & !31 elements only."""
    n32 = len(x) & ~31
    mean = F(0)
    for c in range(0, n32, 32):
        s = F(0)
        for v in x[c : c + 32]:
            s = F(s + F(F(v) * F(v)))
        mean = F(mean + s)
    mean = F(mean / F(len(x)))
    scale = F(F(1) / F(np.sqrt(F(mean + F(eps)))))
    return (x.astype(np.float32) * scale).astype(np.float32)


def rope_rows(x: np.ndarray, pos, n_dims: int, freq_base: float, freq_scale: float) -> np.ndarray:
    """src/op.rs:2697-2749, mode 0.  cos/sin are taken in double and rounded to f32
    (compare with a small tolerance: libm cosf/sinf are not correctly rounded)."""
    toks, heads, ne0 = x.shape
    theta_scale = F(math.pow(float(F(freq_base)), float(F(-2.0) / F(n_dims))))
    y = np.zeros_like(x)
    for t in range(toks):
        p = F(pos[t])
        for h in range(heads):
            theta = F(F(freq_scale) * p)
            for i0 in range(0, ne0, 2):
                c, s = F(math.cos(float(theta))), F(math.sin(float(theta)))
                theta = F(theta * theta_scale)
                x0, x1 = F(x[t, h, i0]), F(x[t, h, i0 + 1])
                y[t, h, i0] = F(F(x0 * c) - F(x1 * s))
                y[t, h, i0 + 1] = F(F(x0 * s) + F(x1 * c))
    return y


def dot_f16_avx(a_bits: np.ndarray, b_bits: np.ndarray) -> np.float32:
    """src/op.rs:137-196: four accumulators of 8 lanes (mul then add), ((s0+s1)+(s2+s3)),
    halves, movehl, movehdup, scalar tail."""
    k = len(a_bits)
    n32 = k & ~31
    sums = [[F(0)] * 8 for _ in range(4)]
    for i in range(0, n32, 32):
        for j in range(4):
            for l in range(8):
                prod = F(f16_val(int(a_bits[i + 8 * j + l])) * f16_val(int(b_bits[i + 8 * j + l])))
                sums[j][l] = F(prod + sums[j][l])
    s01 = [F(sums[0][l] + sums[1][l]) for l in range(8)]
    s23 = [F(sums[2][l] + sums[3][l]) for l in range(8)]
    s = [F(s01[l] + s23[l]) for l in range(8)]
    r4 = [F(s[l] + s[l + 4]) for l in range(4)]
    r2 = [F(r4[0] + r4[2]), F(r4[1] + r4[3])]
    sumf = F(r2[0] + r2[1])
    for i in range(n32, k):
        sumf = F(sumf + F(f16_val(int(a_bits[i])) * f16_val(int(b_bits[i]))))
    return sumf


def main():
    rng = np.random.default_rng(20261125)
    g = {}
    # ---- Q8_0 quantiser: random rows, an all-zero block, exact .5 ties, one non-zero
    q8_x = rng.standard_normal((4, 96)).astype(np.float32)
    q8_x[1, 32:64] = 0.0
    q8_x[2, :32] = np.arange(-16, 16, dtype=np.float32) * 0.5  # amax 8 -> d = 8/127
    q8_x[2, 0] = -127.0  # amax 127 -> d = 1, id = 1: values k + 0.5 hit the tie rule
    q8_x[3, 64:96] = 0.0
    q8_x[3, 70] = -3.25
    g["q8_x"] = q8_x
    g["q8_bytes"] = np.frombuffer(b"".join(quantize_q8_0(r) for r in q8_x), dtype=np.uint8).reshape(4, -1)
    # ---- Q4_0 x Q8_0 dots: 5 weight rows of 4 blocks against row 0 and row 2 of the above
    nb = 3
    w = bytearray()
    for r in range(5):
        for b in range(nb):
            scale = F(rng.uniform(-0.05, 0.05))
            w += struct.pack("<H", f16_bits(scale)) + bytes(rng.integers(0, 256, 16, dtype=np.uint8))
    # extremes: all nibbles 0 (-8) and all 15 (+7) against the -127 block
    w[2:18] = bytes([0x00] * 16)
    w[20:36] = bytes([0xFF] * 16)
    wq = np.frombuffer(bytes(w), dtype=np.uint8).reshape(5, nb * 18)
    g["dot_w"] = wq
    isums, scal, avx = [], [], []
    for xr in (0, 2):
        xb = g["q8_bytes"][xr].tobytes()
        for r in range(5):
            wb = wq[r].tobytes()
            isums.append(block_isums(wb, xb))
            scal.append(dot_scalar(wb, xb))
            avx.append(dot_avx(wb, xb))
    g["dot_isums"] = np.array(isums, dtype=np.int32).reshape(2, 5, nb)
    g["dot_scalar"] = np.array(scal, dtype=np.float32).reshape(2, 5)
    g["dot_avx"] = np.array(avx, dtype=np.float32).reshape(2, 5)
    # ---- f16 tables
    et, st = exp_table(), silu_table()
    g["exp_table"], g["silu_table"] = et, st
    # ---- softmax (with -inf entries), silu
    sm_x = (rng.standard_normal((3, 37)) * 3).astype(np.float32)
    sm_x[1, 5] = -np.inf
    sm_x[1, 36] = -np.inf
    g["softmax_x"] = sm_x
    g["softmax_y"] = np.stack([softmax_row(r, et) for r in sm_x])
    silu_x = (rng.standard_normal(50) * 4).astype(np.float32)
    g["silu_x"] = silu_x
    g["silu_y"] = np.array([f16_val(int(st[f16_bits(v)])) for v in silu_x], dtype=np.float32)
    # ---- rms_norm: K = 70 (only the first 64 enter the sum), K = 20 (sum is empty)
    rn_a = rng.standard_normal(70).astype(np.float32)
    rn_b = rng.standard_normal(20).astype(np.float32)
    g["rms_a_x"], g["rms_a_y"] = rn_a, rms_norm_row(rn_a, 1e-6)
    g["rms_b_x"], g["rms_b_y"] = rn_b, rms_norm_row(rn_b, 1e-5)
    # ---- rope: 3 tokens x 2 heads x 8 dims
    rp_x = rng.standard_normal((3, 2, 8)).astype(np.float32)
    rp_pos = np.array([0, 1, 37], dtype=np.int32)
    g["rope_x"], g["rope_pos"] = rp_x, rp_pos
    g["rope_y"] = rope_rows(rp_x, rp_pos, 8, 10000.0, 1.0)
    # ---- f16 dot, K = 75 (two full 32-chunks + tail of 11)
    fa = rng.standard_normal(75).astype(np.float16).view(np.uint16)
    fb = rng.standard_normal(75).astype(np.float16).view(np.uint16)
    g["f16_a"], g["f16_b"] = fa, fb
    g["f16_dot_avx"] = np.array([dot_f16_avx(fa, fb)], dtype=np.float32)
    np.savez_compressed(os.path.join(HERE, "golden_small.npz"), **g)
    print("wrote", os.path.join(HERE, "golden_small.npz"), {k: v.shape for k, v in g.items()})


if __name__ == "__main__":
    main()
