"""The op sequence of one LLaMA-shaped decode-layer step on the CPU oracle (test infrastructure and
the CPU baseline the bench times for the decode-layer configuration).

`O` is the oracle package itself (passed in so that this module imports nothing); `s` is any object with
the fields hidden, heads, head_dim, ffn, ctx, eps, rope_theta.  Mirrors the op sequence a galois caller
writes for a decoder layer (src/op.rs:3034-3341: rms_norm, mul, matmul, rope_custom, cpy, soft_max, unary,
add) op for op; `avx` selects which of the reference's two
block-dot builds evaluates the mat-muls (BlockQ4_0::vec_dot_q8_0 with +avx, vec_dot_unopt without;
src/ggml_quants.rs:202-207) and the f16 dot (src/op.rs:128-196).  Every intermediate is returned so
that a test can feed the GPU op the oracle's own input ("teacher forcing")."""
import math

import numpy as np


def make_layer_inputs(O, s, seed):
    """Seeded synthetic weights (N(0, 0.02) -> Q4_0), gains, f16 caches (N(0, 1)) and input row."""
    h, f = s.hidden, s.ffn
    shapes = {"wq": (h, h), "wk": (h, h), "wv": (h, h), "wo": (h, h), "w_gate": (f, h), "w_up": (f, h), "w_down": (h, f)}  # (N, K)
    wq4 = {name: O.quantize_q4_0(O.fill_normal(n * k, seed + i, 0, 0.02).reshape(n, k)) for i, (name, (n, k)) in enumerate(shapes.items())}
    attn_norm = 1.0 + 0.1 * O.fill_normal(s.hidden, seed + 100)
    ffn_norm = 1.0 + 0.1 * O.fill_normal(s.hidden, seed + 101)
    k_cache = O.f32_to_f16(O.fill_normal(s.heads * s.ctx * s.head_dim, seed + 102).reshape(s.heads, s.ctx, s.head_dim))
    v_cache = O.f32_to_f16(O.fill_normal(s.heads * s.ctx * s.head_dim, seed + 103).reshape(s.heads, s.head_dim, s.ctx))
    x = O.fill_normal(s.hidden, seed + 104).reshape(1, s.hidden)
    return wq4, attn_norm, ffn_norm, k_cache, v_cache, x


def oracle_layer_trace(O, s, wq4, attn_norm, ffn_norm, k_cache, v_cache, x, position, avx=True):
    """Runs the layer and returns every intermediate by name.  Caches are f16 bit patterns (uint16)
    and are updated in place."""
    hd, nh, ctx = s.head_dim, s.heads, s.ctx
    pos = np.array([position], np.int32)
    t = {"x": x}
    t["h_norm"] = O.rms_norm(x, s.eps)
    t["h"] = O.mul(t["h_norm"], attn_norm[None])
    t["q"] = O.mul_mat_q4_0(wq4["wq"], t["h"], avx=avx)
    t["k"] = O.mul_mat_q4_0(wq4["wk"], t["h"], avx=avx)
    t["v"] = O.mul_mat_q4_0(wq4["wv"], t["h"], avx=avx)
    t["qr"] = O.rope(t["q"].reshape(1, nh, hd), pos, hd, freq_base=s.rope_theta)
    t["kr"] = O.rope(t["k"].reshape(1, nh, hd), pos, hd, freq_base=s.rope_theta)
    k_cache[:, position, :] = O.f32_to_f16(t["kr"][0])
    v_cache[:, :, position] = O.f32_to_f16(t["v"].reshape(nh, hd))
    t["scores"] = O.mul_mat_f16(k_cache, t["qr"].reshape(nh, 1, hd), avx=avx)            # [nh, 1, ctx]
    t["probs"] = O.soft_max_ext(t["scores"].reshape(1, nh, ctx), 1.0 / math.sqrt(hd), pos)
    t["ctxv"] = O.mul_mat_f16(v_cache, t["probs"].reshape(nh, 1, ctx), avx=avx)           # [nh, 1, hd]
    t["o"] = O.mul_mat_q4_0(wq4["wo"], t["ctxv"].reshape(1, nh * hd), avx=avx)
    t["x2"] = O.add(x, t["o"])
    t["h2_norm"] = O.rms_norm(t["x2"], s.eps)
    t["h2"] = O.mul(t["h2_norm"], ffn_norm[None])
    t["g"] = O.mul_mat_q4_0(wq4["w_gate"], t["h2"], avx=avx)
    t["u"] = O.mul_mat_q4_0(wq4["w_up"], t["h2"], avx=avx)
    t["a_silu"] = O.silu(t["g"])
    t["a"] = O.mul(t["a_silu"], t["u"])
    t["d"] = O.mul_mat_q4_0(wq4["w_down"], t["a"], avx=avx)
    t["out"] = O.add(t["x2"], t["d"])
    return t


def oracle_layer_step(O, s, wq4, attn_norm, ffn_norm, k_cache, v_cache, x, position, avx=True):
    return oracle_layer_trace(O, s, wq4, attn_norm, ffn_norm, k_cache, v_cache, x, position, avx)["out"]


def disagreement(a, b):
    """(relative L2, max abs) of a against b."""
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    den = np.linalg.norm(b)
    return (float(np.linalg.norm(a - b) / den) if den > 0 else float(np.linalg.norm(a - b))), float(np.abs(a - b).max())
