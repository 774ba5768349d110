"""One decode step of a LLaMA-shaped decoder layer built from ``galois_*`` ops only.

galois itself holds no model code: a caller crate composes a layer from the free functions
``galois_rms_norm / mul / matmul / rope_custom / cpy / soft_max / unary / add``
(src/op.rs:3034-3341).  This module is that caller for the decode-layer configuration of the benchmark (config 4): hidden 4096,
32 heads x 128, FFN 11008, Q4_0 projections, f16 KV cache, batch 1.

KV-cache layout (both present the contraction dimension contiguously, as
``galois_matmul`` requires of its first operand, src/op.rs:1428):
  K cache  [heads][ctx][head_dim] f16     scores = matmul(K, q)      -> [heads][1][ctx]
  V cache  [heads][head_dim][ctx] f16     context = matmul(V, probs) -> [heads][1][head_dim]
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np

from .op import (RopeCustomOption, UnaryOp, galois_add, galois_cpy, galois_cpy_pair, galois_matmul, galois_matmul_add, galois_matmul_fused, galois_matmul_swiglu, galois_mul, galois_rms_norm,
                 galois_rms_norm_mul, galois_rope_custom, galois_silu_mul, galois_soft_max_ext, galois_unary)
from .tensor import Device, GGmlType, Tensor


@dataclass
class LayerShape:
    hidden: int = 4096
    heads: int = 32
    head_dim: int = 128
    ffn: int = 11008
    ctx: int = 2048
    eps: float = 1e-6
    rope_theta: float = 10000.0


WEIGHT_NAMES = ("wq", "wk", "wv", "wo", "w_gate", "w_up", "w_down")


def weight_shapes(s: LayerShape):
    """name -> (N rows, K columns) of each Q4_0 projection."""
    h, f = s.hidden, s.ffn
    return {"wq": (h, h), "wk": (h, h), "wv": (h, h), "wo": (h, h), "w_gate": (f, h), "w_up": (f, h), "w_down": (h, f)}


class DecodeLayer:
    """Weights (Q4_0 bytes, host numpy), norm gains and the two caches live on one GPU; `step`
    enqueues the kernels of one token on the device's stream and returns the output tensor.

    ``fused=False``: the op-by-op sequence a galois caller writes, 22 kernels.
    ``fused=True`` : the same arithmetic in 9 kernels.  The rows of Wq, Wk, Wv (and of W_gate,
    W_up) are stacked into one Q4_0 weight at upload, so the three (two) projections of the same
    input are one mat-mul whose result is split by views; rope runs once over the 2 x heads rows of
    q and k; rms_norm + gain and silu + gate product run inside the mat-mul that consumes them, the
    residual sums inside the mat-mul that produces their other operand (``galois_matmul_fused``).  Rows
    of a mat-mul are independent and the fusions round like the op pairs, so both variants give
    the same numbers bit for bit.
    ``fused=True, attention_kernel=True``: 6 kernels.  Rope, the two cache appends and the scores run as one
    launch, the masked soft_max and the context product as a second (``galois_b200_decode_attention_f32``, the
    attention phases of the persistent decode kernel as plain kernels); the rows of W_gate and W_up are
    interleaved at upload so that silu(gate) * up leaves the mat-vec that forms both (``galois_matmul_swiglu``)
    and the down projection quantises it directly; again the same numbers bit for bit."""

    def __init__(self, dev, shape: LayerShape, weights: dict, attn_norm: np.ndarray, ffn_norm: np.ndarray,
                 k_cache: np.ndarray, v_cache: np.ndarray, fused: bool = False, attention_kernel: bool = False):
        s, G = shape, Device.Gpu(dev)
        if attention_kernel and not fused:
            raise ValueError("attention_kernel needs fused=True")
        self.shape, self.dev, self.fused, self.attention_kernel = s, dev, fused, attention_kernel
        self.w = {}
        for name, (n, k) in weight_shapes(s).items():
            if fused and name in ("wq", "wk", "wv", "w_gate", "w_up"):
                continue
            self.w[name] = Tensor.from_raw(weights[name], (k, n), GGmlType.Q4_0, G)
        if fused:
            raw = lambda name: np.ascontiguousarray(weights[name]).view(np.uint8).reshape(-1)
            self.w["wqkv"] = Tensor.from_raw(np.concatenate([raw("wq"), raw("wk"), raw("wv")]), (s.hidden, 3 * s.hidden), GGmlType.Q4_0, G)
            if attention_kernel:
                # rows interleaved (gate_0, up_0, gate_1, up_1, ...): the SwiGLU product leaves the mat-vec that forms both
                rb = s.hidden // 32 * 18
                gu = np.stack([raw("w_gate").reshape(s.ffn, rb), raw("w_up").reshape(s.ffn, rb)], axis=1).reshape(-1)
                self.w["w_gate_up"] = Tensor.from_raw(gu, (s.hidden, 2 * s.ffn), GGmlType.Q4_0, G)
            else:
                self.w["w_gate_up"] = Tensor.from_raw(np.concatenate([raw("w_gate"), raw("w_up")]), (s.hidden, 2 * s.ffn), GGmlType.Q4_0, G)
            self.qkv = Tensor.zeros((3 * s.hidden, 1), GGmlType.F32, G)
            self.qkr = Tensor.zeros((s.head_dim, 2 * s.heads, 1), GGmlType.F32, G)
            self.gu = Tensor.zeros((2 * s.ffn, 1), GGmlType.F32, G)
        self.attn_norm = Tensor.from_numpy(attn_norm.reshape(1, s.hidden), GGmlType.F32, G)
        self.ffn_norm = Tensor.from_numpy(ffn_norm.reshape(1, s.hidden), GGmlType.F32, G)
        # caches arrive as f16 arrays [heads][ctx][head_dim] and [heads][head_dim][ctx]
        self.k_cache = Tensor.from_numpy(k_cache, GGmlType.F16, G)
        self.v_cache = Tensor.from_numpy(v_cache, GGmlType.F16, G)
        z = lambda *ne: Tensor.zeros(ne, GGmlType.F32, G)
        self.h = z(s.hidden, 1)
        self.q, self.k, self.v = z(s.hidden, 1), z(s.hidden, 1), z(s.hidden, 1)
        self.qr, self.kr = z(s.head_dim, s.heads, 1), z(s.head_dim, s.heads, 1)
        self.scores, self.probs = z(s.ctx, 1, s.heads), z(s.ctx, 1, s.heads)
        self.ctxv = z(s.head_dim, 1, s.heads)
        self.o, self.x2, self.h2 = z(s.hidden, 1), z(s.hidden, 1), z(s.hidden, 1)
        self.g, self.u, self.a = z(s.ffn, 1), z(s.ffn, 1), z(s.ffn, 1)
        self.d, self.out = z(s.hidden, 1), z(s.hidden, 1)
        self.rope = RopeCustomOption(n_dims=s.head_dim, mode=0, n_ctx=s.ctx, freq_base=s.rope_theta, freq_scale=1.0)
        self.scale = 1.0 / math.sqrt(s.head_dim)
        if attention_kernel:
            import ctypes as C

            from ._lib import GaloisDecodeLayer, GaloisDecodeShape, lib
            from .tensor import _check

            self.c_shape = GaloisDecodeShape(s.hidden, s.heads, s.head_dim, s.ffn, s.ctx, s.eps, s.rope_theta, 1.0)
            self.c_layer = GaloisDecodeLayer()
            self.c_layer.k_cache, self.c_layer.v_cache = self.k_cache.data_ptr(), self.v_cache.data_ptr()
            need = C.c_size_t()
            _check(dev.ctx, lib.galois_b200_decode_workspace_bytes(dev.ctx, C.byref(self.c_shape), C.byref(need)), "decode_workspace_bytes")
            self.ws_bytes = need.value
            self.ws = Tensor.zeros((need.value // 4,), GGmlType.F32, G)

    def step(self, x: Tensor, pos: Tensor, position: int) -> Tensor:
        """x: f32 {hidden, 1}; pos: i32 {1} holding `position` (the row of the caches to fill)."""
        if self.fused:
            return self._step_fused(x, pos, position)
        s = self.shape
        hd, nh, ctx = s.head_dim, s.heads, s.ctx
        # attention block
        galois_rms_norm(x, self.h, s.eps)
        galois_mul(self.h, self.attn_norm, self.h)
        galois_matmul(self.w["wq"], self.h, self.q)
        galois_matmul(self.w["wk"], self.h, self.k)
        galois_matmul(self.w["wv"], self.h, self.v)
        q3 = self.q.view((hd, nh, 1), (1, hd, hd * nh, hd * nh))
        k3 = self.k.view((hd, nh, 1), (1, hd, hd * nh, hd * nh))
        galois_rope_custom(self.rope, q3, pos, self.qr)
        galois_rope_custom(self.rope, k3, pos, self.kr)
        # KV-cache append: K row `position` of every head; V column `position` of every head
        k_src = self.kr.view((hd, 1, nh), (1, hd, hd, hd * nh))
        k_dst = self.k_cache.view((hd, 1, nh), (1, hd, hd * ctx, hd * ctx * nh), offset=position * hd)
        galois_cpy(k_src, k_dst)
        v_src = self.v.view((1, hd, nh), (1, 1, hd, hd * nh))
        v_dst = self.v_cache.view((1, hd, nh), (1, ctx, hd * ctx, hd * ctx * nh), offset=position)
        galois_cpy(v_src, v_dst)
        # scores over the cache, causal soft-max, context
        qh = self.qr.view((hd, 1, nh), (1, hd, hd, hd * nh))
        galois_matmul(self.k_cache, qh, self.scores)
        sc = self.scores.view((ctx, nh, 1), (1, ctx, ctx * nh, ctx * nh))
        pr = self.probs.view((ctx, nh, 1), (1, ctx, ctx * nh, ctx * nh))
        galois_soft_max_ext(sc, pr, self.scale, pos)
        galois_matmul(self.v_cache, self.probs, self.ctxv)
        ctx_flat = self.ctxv.view((s.hidden, 1), (1, s.hidden, s.hidden, s.hidden))
        galois_matmul(self.w["wo"], ctx_flat, self.o)
        galois_add(x, self.o, self.x2)
        # feed-forward block (SwiGLU)
        galois_rms_norm(self.x2, self.h2, s.eps)
        galois_mul(self.h2, self.ffn_norm, self.h2)
        galois_matmul(self.w["w_gate"], self.h2, self.g)
        galois_matmul(self.w["w_up"], self.h2, self.u)
        galois_unary(self.g, self.a, UnaryOp.Silu)
        galois_mul(self.a, self.u, self.a)
        galois_matmul(self.w["w_down"], self.a, self.d)
        galois_add(self.x2, self.d, self.out)
        return self.out

    def _step_fused(self, x: Tensor, pos: Tensor, position: int) -> Tensor:
        s = self.shape
        hd, nh, ctx, H = s.head_dim, s.heads, s.ctx, s.hidden
        # attention block
        # rms_norm + gain run where the GEMV quantises its input; rows [0, H) = q, [H, 2H) = k, [2H, 3H) = v
        galois_matmul_fused(self.w["wqkv"], x, self.qkv, rms_gain=self.attn_norm, eps=s.eps)
        if self.attention_kernel:
            return self._step_tail(x, self._attention_one_launch(pos))
        qk3 = self.qkv.view((hd, 2 * nh, 1), (1, hd, hd * 2 * nh, hd * 2 * nh))
        galois_rope_custom(self.rope, qk3, pos, self.qkr)  # heads 0..nh-1 of q, then of k
        k_src = self.qkr.view((hd, 1, nh), (1, hd, hd, hd * nh), offset=H)
        k_dst = self.k_cache.view((hd, 1, nh), (1, hd, hd * ctx, hd * ctx * nh), offset=position * hd)
        v_src = self.qkv.view((1, hd, nh), (1, 1, hd, hd * nh), offset=2 * H)
        v_dst = self.v_cache.view((1, hd, nh), (1, ctx, hd * ctx, hd * ctx * nh), offset=position)
        galois_cpy_pair(k_src, k_dst, v_src, v_dst)  # both cache appends in one launch
        qh = self.qkr.view((hd, 1, nh), (1, hd, hd, hd * nh))
        galois_matmul(self.k_cache, qh, self.scores)
        sc = self.scores.view((ctx, nh, 1), (1, ctx, ctx * nh, ctx * nh))
        pr = self.probs.view((ctx, nh, 1), (1, ctx, ctx * nh, ctx * nh))
        galois_soft_max_ext(sc, pr, self.scale, pos)
        galois_matmul(self.v_cache, self.probs, self.ctxv)
        return self._step_tail(x, self.ctxv.view((H, 1), (1, H, H, H)))

    def _attention_one_launch(self, pos: Tensor) -> Tensor:
        import ctypes as C

        from ._lib import lib
        from .tensor import _check

        H = self.shape.hidden
        rc = lib.galois_b200_decode_attention_f32(self.dev.ctx, C.byref(self.c_shape), C.byref(self.c_layer), C.c_void_p(self.qkv.data_ptr()),
                                                  C.c_void_p(pos.data_ptr()), C.c_void_p(self.ctxv.data_ptr()), C.c_void_p(self.ws.data_ptr()),
                                                  self.ws_bytes)
        _check(self.dev.ctx, rc, "galois_b200_decode_attention_f32")
        return self.ctxv.view((H, 1), (1, H, H, H))

    def _step_tail(self, x: Tensor, ctx_flat: Tensor) -> Tensor:
        s = self.shape
        galois_matmul_add(self.w["wo"], ctx_flat, x, self.x2)  # x2 = x + Wo ctx
        # feed-forward block (SwiGLU)
        if self.attention_kernel:
            # gate and up rows interleaved: silu(gate) * up is formed where the two sums meet, down takes it as it is
            galois_matmul_swiglu(self.w["w_gate_up"], self.x2, self.a, rms_gain=self.ffn_norm, eps=s.eps)
            galois_matmul_fused(self.w["w_down"], self.a, self.out, res=self.x2)  # out = x2 + Wdown a
            return self.out
        # rows [0, ffn) = gate, [ffn, 2 ffn) = up
        galois_matmul_fused(self.w["w_gate_up"], self.x2, self.gu, rms_gain=self.ffn_norm, eps=s.eps)
        g = self.gu.view((s.ffn, 1), (1, s.ffn, s.ffn, s.ffn))
        u = self.gu.view((s.ffn, 1), (1, s.ffn, s.ffn, s.ffn), offset=s.ffn)
        galois_matmul_fused(self.w["w_down"], g, self.out, silu_mul=u, res=self.x2)  # out = x2 + Wdown (silu(g) * u)
        return self.out

    def algorithmic_bytes(self) -> int:
        """Q4_0 weights once + both f16 caches once + the f32 activations once."""
        s = self.shape
        wb = sum(n * (k // 32) * 18 for n, k in weight_shapes(s).values())
        kv = 2 * s.heads * s.ctx * s.head_dim * 2
        act = 4 * (12 * s.hidden + 3 * s.ffn + 2 * s.heads * s.ctx)
        return wb + kv + act


class DecodeStack:
    """Consecutive decoder layers stepped by ONE persistent kernel (``galois_b200_decode_layers_f32``):
    the 22-op sequence of ``DecodeLayer.step`` for every layer of the stack, bit-identical to calling
    ``step`` layer after layer, without a kernel boundary between ops or layers.  Takes op-by-op
    ``DecodeLayer`` objects (``fused=False``) and uses their weights and caches in place."""

    def __init__(self, layers):
        import ctypes as C

        from ._lib import GaloisDecodeLayer, GaloisDecodeShape, lib
        from .tensor import _check

        if not layers or any(L.fused for L in layers):
            raise ValueError("DecodeStack takes one or more op-by-op DecodeLayer objects")
        self.layers, self.dev, s = list(layers), layers[0].dev, layers[0].shape
        self.shape = s
        self.c_shape = GaloisDecodeShape(s.hidden, s.heads, s.head_dim, s.ffn, s.ctx, s.eps, s.rope_theta, 1.0)
        self.c_layers = (GaloisDecodeLayer * len(layers))()
        for i, L in enumerate(self.layers):
            d = self.c_layers[i]
            d.wq, d.wk, d.wv, d.wo = (L.w[n].data_ptr() for n in ("wq", "wk", "wv", "wo"))
            d.w_gate, d.w_up, d.w_down = (L.w[n].data_ptr() for n in ("w_gate", "w_up", "w_down"))
            d.attn_norm, d.ffn_norm = L.attn_norm.data_ptr(), L.ffn_norm.data_ptr()
            d.k_cache, d.v_cache = L.k_cache.data_ptr(), L.v_cache.data_ptr()
        need = C.c_size_t()
        _check(self.dev.ctx, lib.galois_b200_decode_workspace_bytes(self.dev.ctx, C.byref(self.c_shape), C.byref(need)), "decode_workspace_bytes")
        self.ws_bytes = need.value
        self.ws = Tensor.zeros((need.value // 4,), GGmlType.F32, Device.Gpu(self.dev))
        self.out = Tensor.zeros((s.hidden, 1), GGmlType.F32, Device.Gpu(self.dev))

    def step(self, x: Tensor, pos: Tensor) -> Tensor:
        """x: f32 {hidden, 1}; pos: i32 {1} on the device (the cache row / column to fill)."""
        import ctypes as C

        from ._lib import lib
        from .tensor import _check

        rc = lib.galois_b200_decode_layers_f32(self.dev.ctx, C.byref(self.c_shape), self.c_layers, len(self.layers), C.c_void_p(x.data_ptr()),
                                               C.c_void_p(pos.data_ptr()), C.c_void_p(self.out.data_ptr()), C.c_void_p(self.ws.data_ptr()),
                                               self.ws_bytes)
        _check(self.dev.ctx, rc, "galois_b200_decode_layers_f32")
        return self.out
