"""A pre-LayerNorm transformer encoder stack driven through the op entry points — the caller
side of the hot path for the Whisper-shaped workload (32 layers, d_model 1280, 20 heads, FFN
5120 with exact GELU, 1500 tokens).

The op sequence per layer is the one the reference's exported fp16 graph runs
(tools/attrib_whisper.jl:52-57, plans/projects/whisper/REPORT.md:62-69): native_layer_norm,
three projections as addmm/addmm/mm (the key projection has no bias), the flash sdpa op on
(E,L,H,B) views of the projections, a clone back to token-major, the output addmm, add.Tensor,
native_layer_norm, addmm with the GELU folded into its store, addmm, add.Tensor and the fp16
clamp; a final native_layer_norm closes the stack.  Every intermediate lives at a fixed offset
of one slab, so the whole pass can be captured once and replayed.
"""
from __future__ import annotations

from dataclasses import dataclass
from math import sqrt
from typing import List, Optional

import numpy as np

from .attention import sdpa
from .context import Ctx, DeviceArray
from .elementwise import add_, clamp_
from .layernorm import add_layernorm_, layernorm_
from .matmul import matmul_

F16_MAX = 65504.0


@dataclass
class EncoderConfig:
    layers: int = 32
    d_model: int = 1280
    heads: int = 20
    ffn: int = 5120
    tokens: int = 1500
    eps: float = 1e-5
    clamp: bool = True
    seed: int = 20260101

    @property
    def head_dim(self) -> int:
        return self.d_model // self.heads

    def flops(self) -> float:
        """Dense-contraction flops of one pass: 2MNK per GEMM + 4 Lq Lk E H per attention."""
        d, f, L = self.d_model, self.ffn, self.tokens
        gemm = 2.0 * L * (4 * d * d + 2 * d * f)
        attn = 4.0 * L * L * self.head_dim * self.heads
        return self.layers * (gemm + attn)

    def gemm_flops(self) -> float:
        d, f, L = self.d_model, self.ffn, self.tokens
        return self.layers * 2.0 * L * (4 * d * d + 2 * d * f)


def init_weights(cfg: EncoderConfig) -> List[dict]:
    """Random-init fp16 weights N(0, 0.02) in torch layout: W (out, in), b (out,)."""
    rng = np.random.default_rng(cfg.seed)
    d, f = cfg.d_model, cfg.ffn

    def w(o, i):
        return (rng.standard_normal((o, i), dtype=np.float32) * 0.02).astype(np.float16)

    def b(o):
        return (rng.standard_normal(o, dtype=np.float32) * 0.02).astype(np.float16)

    layers = []
    for _ in range(cfg.layers):
        layers.append(dict(
            ln1_g=np.ones(d, np.float16), ln1_b=np.zeros(d, np.float16),
            wq=w(d, d), bq=b(d), wk=w(d, d), wv=w(d, d), bv=b(d), wo=w(d, d), bo=b(d),
            ln2_g=np.ones(d, np.float16), ln2_b=np.zeros(d, np.float16),
            w1=w(f, d), b1=b(f), w2=w(d, f), b2=b(d)))
    layers.append(dict(lnf_g=np.ones(d, np.float16), lnf_b=np.zeros(d, np.float16)))
    return layers


class Encoder:
    """Device-resident encoder: weights uploaded once (transposed to the dense (out,K)
    column-major form `hoistpermutes` produces), activations in one preallocated slab."""

    def __init__(self, ctx: Ctx, cfg: EncoderConfig, weights: Optional[List[dict]] = None, fused: bool = True):
        """`fused=False` issues the exported graph's ops one by one.  `fused=True` applies three
        load-time rewrites of the kind the reference's `Model` constructor runs (hoistpermutes,
        foldrelu, fuse): the q/k/v projections share one GEMM over concatenated weights, sdpa
        writes token-major so the clone after it disappears, and each residual add (+ clamp) is
        folded into the layer norm that follows.  Same values either way."""
        self.ctx, self.cfg, self.fused = ctx, cfg, fused
        weights = weights if weights is not None else init_weights(cfg)
        self.layers = []
        for lw in weights[:-1]:
            dev = {}
            for k, v in lw.items():
                # torch W (out,in) -> t(W) made dense: torch (in,out) == reference (out,in) column-major
                dev[k] = ctx.toback(np.ascontiguousarray(v.T) if v.ndim == 2 else v)
            if fused:
                wqkv = np.concatenate([lw["wq"], lw["wk"], lw["wv"]], axis=0)            # torch (3d, d)
                bqkv = np.concatenate([lw["bq"], np.zeros_like(lw["bq"]), lw["bv"]])     # k has no bias
                dev["wqkv"] = ctx.toback(np.ascontiguousarray(wqkv.T))
                dev["bqkv"] = ctx.toback(bqkv)
                for k in ("wq", "wk", "wv", "bq", "bv"):
                    del dev[k]
            self.layers.append(dev)
        self.final = {k: ctx.toback(v) for k, v in weights[-1].items()}
        d, f, L = cfg.d_model, cfg.ffn, cfg.tokens
        al = lambda n: (n + 255) // 256 * 256
        sizes = dict(xin=d * L * 2, x=d * L * 2, h=d * L * 2, q=d * L * 2, k=d * L * 2, v=d * L * 2, att=d * L * 2, att_t=d * L * 2,
                     qkv=3 * d * L * 2,
                     f=f * L * 2, y=d * L * 2, mean=L * 4, rstd=L * 4)
        self.slab = ctx.allocate(np.uint8, sum(al(s) for s in sizes.values()))
        off = 0
        self.off = {}
        for name, s in sizes.items():
            self.off[name] = off
            off += al(s)
        self._graph = None

    def _buf(self, name, dtype, *dims) -> DeviceArray:
        return DeviceArray(self.ctx, self.slab.ptr + self.off[name], dtype, dims, owner=self.slab)

    @property
    def xin(self) -> DeviceArray:
        """Input, (d_model, tokens) == torch (tokens, d_model); left untouched by a pass."""
        return self._buf("xin", np.float16, self.cfg.d_model, self.cfg.tokens)

    @property
    def x(self) -> DeviceArray:
        """Residual stream, updated in place layer by layer."""
        return self._buf("x", np.float16, self.cfg.d_model, self.cfg.tokens)

    @property
    def y(self) -> DeviceArray:
        return self._buf("y", np.float16, self.cfg.d_model, self.cfg.tokens)

    def forward(self) -> DeviceArray:
        """One pass over the sequence held in `self.xin`; the result lands in `self.y`."""
        c, ctx = self.cfg, self.ctx
        d, f, L, H, E = c.d_model, c.ffn, c.tokens, c.heads, c.head_dim
        x = self.x
        h = self._buf("h", np.float16, d, L)
        q, k, v = (self._buf(n, np.float16, d, L) for n in ("q", "k", "v"))
        att = self._buf("att", np.float16, E, L, H, 1)
        att_t = self._buf("att_t", np.float16, d, L)
        ff = self._buf("f", np.float16, f, L)
        mean, rstd = self._buf("mean", np.float32, L), self._buf("rstd", np.float32, L)
        scale = 1.0 / sqrt(E)
        as_heads = lambda t: t.reshape(E, H, L, 1).permute((0, 2, 1, 3))   # (E,L,H,B) view, no copy
        ctx.copy(x, self.xin)
        if self.fused:
            return self._forward_fused(x, h, att_t, ff, mean, rstd, scale)
        for w in self.layers:
            ctx.ws.reset()
            layernorm_(ctx, h, mean, rstd, x, w["ln1_g"], w["ln1_b"], d, c.eps)
            matmul_(ctx, q, w["wq"], h, w["bq"])
            matmul_(ctx, k, w["wk"], h, None)
            matmul_(ctx, v, w["wv"], h, w["bv"])
            sdpa(ctx, as_heads(q), as_heads(k), as_heads(v), None, scale, out=att)
            # clone back to token-major: (E,L,H) -> (E,H,L)
            ctx.contiguous(att.reshape(E, L, H).permute((0, 2, 1)), out=att_t.reshape(E, H, L))
            matmul_(ctx, h, w["wo"], att_t, w["bo"])
            add_(ctx, x, x, h)
            layernorm_(ctx, h, mean, rstd, x, w["ln2_g"], w["ln2_b"], d, c.eps)
            matmul_(ctx, ff, w["w1"], h, w["b1"], epi="gelu")
            matmul_(ctx, h, w["w2"], ff, w["b2"])
            add_(ctx, x, x, h)
            if c.clamp:
                clamp_(ctx, x, x, -F16_MAX, F16_MAX)
        layernorm_(ctx, self.y, mean, rstd, x, self.final["lnf_g"], self.final["lnf_b"], d, c.eps)
        return self.y

    def _forward_fused(self, x, h, att_t, ff, mean, rstd, scale) -> DeviceArray:
        c, ctx = self.cfg, self.ctx
        d, f, L, H, E = c.d_model, c.ffn, c.tokens, c.heads, c.head_dim
        qkv = self._buf("qkv", np.float16, 3 * d, L)
        esz = 2

        def head_view(i):  # rows [i*d, (i+1)*d) of qkv seen as (E, L, H, 1)
            return DeviceArray(ctx, qkv.ptr + i * d * esz, np.float16, (E, L, H, 1), (1, 3 * d, E, 3 * d * L), owner=qkv)

        # token-major destination for sdpa: (E, L, H, 1) view of the (d, L) buffer the o-projection reads
        att_view = DeviceArray(ctx, att_t.ptr, np.float16, (E, L, H, 1), (1, d, E, d * L), owner=att_t)
        clamp = (-F16_MAX, F16_MAX) if c.clamp else None
        first = self.layers[0]
        layernorm_(ctx, h, mean, rstd, x, first["ln1_g"], first["ln1_b"], d, c.eps)
        for i, w in enumerate(self.layers):
            ctx.ws.reset()
            matmul_(ctx, qkv, w["wqkv"], h, w["bqkv"])
            sdpa(ctx, head_view(0), head_view(1), head_view(2), None, scale, out=att_view)
            matmul_(ctx, h, w["wo"], att_t, w["bo"])
            add_layernorm_(ctx, h, mean, rstd, x, h, w["ln2_g"], w["ln2_b"], d, c.eps)          # x += o; h = LN2(x)
            matmul_(ctx, ff, w["w1"], h, w["b1"], epi="gelu")
            matmul_(ctx, h, w["w2"], ff, w["b2"])
            if i + 1 < len(self.layers):
                g, b, dst = self.layers[i + 1]["ln1_g"], self.layers[i + 1]["ln1_b"], h
            else:
                g, b, dst = self.final["lnf_g"], self.final["lnf_b"], self.y
            add_layernorm_(ctx, dst, mean, rstd, x, h, g, b, d, c.eps, clamp=clamp)             # x = clamp(x + g); LN
        return self.y

    def capture(self):
        """Run once eagerly (warms pool and workspace), then record the pass as a graph."""
        self.forward()
        self.ctx.synchronize()
        self._graph = self.ctx.capture(self.forward)
        return self._graph

    def launches_per_pass(self) -> int:
        n0 = self.ctx.launch_count()
        self.forward()
        return self.ctx.launch_count() - n0
