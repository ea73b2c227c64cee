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
from .layernorm import layernorm_
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

    def __init__(self, ctx: Ctx, cfg: EncoderConfig, weights: Optional[List[dict]] = None):
        self.ctx, self.cfg = ctx, cfg
        weights = weights if weights is not None else init_weights(cfg)
        self.layers = []
        for lw in weights[:-1]:
            dev = {}
            for k, v in lw.items():
                # torch W (out,in) -> t(W) made dense: torch (in,out) == reference (out,in) column-major
                dev[k] = ctx.toback(np.ascontiguousarray(v.T) if v.ndim == 2 else v)
            self.layers.append(dev)
        self.final = {k: ctx.toback(v) for k, v in weights[-1].items()}
        d, f, L = cfg.d_model, cfg.ffn, cfg.tokens
        al = lambda n: (n + 255) // 256 * 256
        sizes = dict(xin=d * L * 2, x=d * L * 2, h=d * L * 2, q=d * L * 2, k=d * L * 2, v=d * L * 2, att=d * L * 2, att_t=d * L * 2,
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
