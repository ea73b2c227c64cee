"""A hierarchical ViT image encoder (Hiera-B+-shaped) driven through the op entry points: the
caller side of the hot path for the image workload (1024x1024x3 input, patch stride 4, embed 112
doubling per stage to 896, stage depths 2/3/16/3, 56-wide heads, windowed attention with a few
global blocks, MLP ratio 4, a 2x2 max-pool of the queries at each stage transition).

Per block the ops are the ones the reference's exported SAM 2 image-encoder graphs run
(plans/kernels-to-port.md:63-65, tools/attn_lab.jl:11-14): native_layer_norm, addmm (q/k/v in one
weight), window partition as a permuted clone, the sdpa op per window (or per image for the global
blocks), addmm, add.Tensor, native_layer_norm, addmm with the GELU folded, addmm, add.Tensor; the
first block of stages 2-4 widens the channels with an extra addmm and max_pool2d on both the
shortcut and the queries.

Layout.  A token array is (C, tokens) with the tokens of one attention window adjacent
("window order"): image, then window row, window column, then row and column inside the window.
Layer norm, the projections and the MLP are per token and do not care; windowed attention then
reads (E, L, H, windows) straight out of the q/k/v projection through strides, and global
attention — indifferent to the order of its keys — reads (E, L, H, images) from the same array.
Tokens are re-ordered only where the window geometry changes: after the stem, after each pooling
block, and back to raster order at the end.  The exported graph instead partitions and
un-partitions around every attention (two permuted clones per block).

The window sizes and the global blocks are this build's choice (the Hiera-B+ configuration is not
part of the reference tree): windows of 8x8, 8x8, 16x16, 16x16 tokens in the four stages, a pooling
block attending within the window of the stage it leaves, global attention in blocks 12, 16, 20.
"""
from __future__ import annotations

from dataclasses import dataclass
from math import sqrt
from typing import Dict, List, Optional, Tuple

import numpy as np

from .attention import sdpa
from .context import Ctx, DeviceArray
from .conv import convolution_, convsize
from .elementwise import add_, maxpool2d_
from .layernorm import add_layernorm_, layernorm_
from .matmul import matmul_


@dataclass
class HieraConfig:
    image: int = 1024
    in_ch: int = 3
    embed: int = 112
    depths: Tuple[int, ...] = (2, 3, 16, 3)
    head_dim: int = 56
    windows: Tuple[int, ...] = (8, 8, 16, 16)
    global_blocks: Tuple[int, ...] = (12, 16, 20)
    mlp_ratio: int = 4
    patch: Tuple[int, int, int] = (7, 4, 3)        # stem kernel, stride, padding
    eps: float = 1e-6
    seed: int = 20260104

    def dim(self, stage: int) -> int:
        return self.embed << stage

    def side(self, stage: int) -> int:
        """Tokens per image side in a stage."""
        k, s, p = self.patch
        return convsize(self.image, k, s, p, 1) >> stage

    def blocks(self) -> List[dict]:
        """One record per block: stage, dims, whether it pools, its window (0 = global)."""
        out, i = [], 0
        for st, depth in enumerate(self.depths):
            for j in range(depth):
                pool = st > 0 and j == 0
                out.append(dict(index=i, stage=st, pool=pool, dim_in=self.dim(st - 1) if pool else self.dim(st),
                                dim=self.dim(st), heads=self.dim(st) // self.head_dim,
                                window=0 if i in self.global_blocks else (self.windows[st - 1] if pool else self.windows[st]),
                                side_in=self.side(st - 1) if pool else self.side(st), side=self.side(st)))
                i += 1
        return out

    def check(self) -> None:
        for b in self.blocks():
            assert b["dim"] % self.head_dim == 0 and self.head_dim % 8 == 0
            if b["window"]:
                assert b["side_in"] % b["window"] == 0, "windows must tile the token grid"
            assert not (b["pool"] and b["window"] == 0), "a pooling block attends within windows"
            if b["pool"]:
                assert b["window"] % 2 == 0

    def flops(self, batch: int = 1) -> float:
        """2MNK per GEMM (stem included) + 4 Lq Lk E H per attention."""
        k, s, p = self.patch
        S0 = self.side(0)
        total = 2.0 * S0 * S0 * (self.in_ch * k * k) * self.embed
        for b in self.blocks():
            T_in, T = b["side_in"] ** 2, b["side"] ** 2
            d_in, d = b["dim_in"], b["dim"]
            total += 2.0 * T_in * d_in * 3 * d + 2.0 * T * d * d + 4.0 * T * d * d * self.mlp_ratio
            if b["pool"]:
                total += 2.0 * T_in * d_in * d
            Lk = b["window"] ** 2 if b["window"] else T_in
            Lq = Lk // 4 if b["pool"] else Lk
            nwin = T_in // Lk
            total += 4.0 * Lq * Lk * d * nwin
        return total * batch


def init_weights(cfg: HieraConfig) -> dict:
    """Random-init fp16 weights N(0, 0.02), torch layouts: linear W (out, in), conv W (Cout, Cin, KH, KW)."""
    rng = np.random.default_rng(cfg.seed)
    n = lambda *s: (rng.standard_normal(s, dtype=np.float32) * 0.02).astype(np.float16)
    k = cfg.patch[0]
    S0 = cfg.side(0)
    w = dict(stem_w=n(cfg.embed, cfg.in_ch, k, k), stem_b=n(cfg.embed), pos=n(S0, S0, cfg.embed), blocks=[])
    for b in cfg.blocks():
        d_in, d, f = b["dim_in"], b["dim"], b["dim"] * cfg.mlp_ratio
        bw = dict(ln1_g=np.ones(d_in, np.float16), ln1_b=np.zeros(d_in, np.float16), wqkv=n(3 * d, d_in), bqkv=n(3 * d),
                  wo=n(d, d), bo=n(d), ln2_g=np.ones(d, np.float16), ln2_b=np.zeros(d, np.float16),
                  w1=n(f, d), b1=n(f), w2=n(d, f), b2=n(d))
        if b["pool"]:
            bw.update(wproj=n(d, d_in), bproj=n(d))
        w["blocks"].append(bw)
    return w


class Hiera:
    """Device-resident encoder: weights uploaded once, every intermediate in a buffer allocated at
    construction (fixed addresses, so a pass can be captured and replayed)."""

    def __init__(self, ctx: Ctx, cfg: HieraConfig, weights: Optional[dict] = None, batch: int = 1):
        cfg.check()
        self.ctx, self.cfg, self.batch = ctx, cfg, batch
        weights = weights if weights is not None else init_weights(cfg)
        up = lambda v: ctx.toback(np.ascontiguousarray(v.T) if v.ndim == 2 else v)   # linear W -> dense (out, K) column-major
        # conv weight torch (Cout,Cin,KH,KW) is already the reference's (KW,KH,Cin,Cout) column-major
        self.stem_w, self.stem_b = ctx.toback(weights["stem_w"]), ctx.toback(weights["stem_b"])
        self.blocks = [{k: up(v) for k, v in bw.items()} for bw in weights["blocks"]]
        self.plan = cfg.blocks()
        B, S0 = batch, cfg.side(0)
        # positional embedding, stored in the window order of stage 0 once and for all
        pos = np.broadcast_to(weights["pos"][None], (B, S0, S0, cfg.embed))
        self.pos = ctx.toback(np.ascontiguousarray(self._host_windows(pos, cfg.windows[0])))
        # buffers sized for the largest user
        tok = lambda b: b["side_in"] ** 2 * B
        mx = lambda f: max(f(b) for b in self.plan)
        n_x = max(mx(lambda b: tok(b) * b["dim_in"]), mx(lambda b: b["side"] ** 2 * B * b["dim"]))
        self.image = ctx.allocate(np.float16, cfg.image, cfg.image, cfg.in_ch, B)          # (W,H,Cin,N)
        self.stem_out = ctx.allocate(np.float16, S0, S0, cfg.embed, B)                     # (OW,OH,Cout,N)
        self.xa = ctx.allocate(np.float16, n_x)
        self.xb = ctx.allocate(np.float16, n_x)
        self.h = ctx.allocate(np.float16, n_x)
        self.tmp = ctx.allocate(np.float16, n_x)
        self.att = ctx.allocate(np.float16, n_x)
        self.qkv = ctx.allocate(np.float16, mx(lambda b: tok(b) * 3 * b["dim"]))
        self.ff = ctx.allocate(np.float16, mx(lambda b: b["side"] ** 2 * B * b["dim"] * cfg.mlp_ratio))
        self.sc = ctx.allocate(np.float16, mx(lambda b: tok(b) * b["dim"] if b["pool"] else 1))
        self.qp = ctx.allocate(np.float16, n_x)
        self.mean = ctx.allocate(np.float32, S0 * S0 * B)
        self.rstd = ctx.allocate(np.float32, S0 * S0 * B)
        last = self.plan[-1]
        self.y = ctx.allocate(np.float16, last["dim"], last["side"], last["side"], B)     # (C,W,H,N): torch (N,H,W,C)
        self._graph = None

    # ---- token order
    @staticmethod
    def _host_windows(x: np.ndarray, w: int) -> np.ndarray:
        """torch (B,S,S,C) raster -> (B*nWy*nWx, w*w, C) window order (host side, for constants)."""
        B, S, _, Cn = x.shape
        return x.reshape(B, S // w, w, S // w, w, Cn).transpose(0, 1, 3, 2, 4, 5).reshape(-1, w * w, Cn)

    def _view(self, buf: DeviceArray, *dims: int) -> DeviceArray:
        return DeviceArray(self.ctx, buf.ptr, np.float16, dims, owner=buf)

    def _to_windows(self, dst: DeviceArray, src: DeviceArray, Cn: int, S: int, w: int) -> None:
        """raster (C,S,S,B) -> window order (C, w*w, windows): one permuted copy."""
        n = S // w
        v = DeviceArray(self.ctx, src.ptr, np.float16, (Cn * w, n, w, n * self.batch), (1, Cn * w, Cn * S, Cn * S * w), owner=src)
        self.ctx.contiguous(v.permute((0, 2, 1, 3)), out=self._view(dst, Cn * w, w, n, n * self.batch))

    def _to_raster(self, dst: DeviceArray, src: DeviceArray, Cn: int, S: int, w: int) -> None:
        """window order (C, w*w, windows) -> raster (C,S,S,B)."""
        n = S // w
        v = self._view(src, Cn * w, w, n, n * self.batch)
        self.ctx.contiguous(v.permute((0, 2, 1, 3)), out=self._view(dst, Cn * w, n, w, n * self.batch))

    # ---- one pass
    def gemm_pass(self) -> None:
        """Only the projection / MLP GEMM launches of a pass, in pass order and on the pass's own buffers
        (values are meaningless): what a benchmark replays to time the GEMM family of the pass alone."""
        self._gemm_only = True
        try:
            self.forward()
        finally:
            self._gemm_only = False

    def gemm_flops(self) -> float:
        """2MNK summed over the launches of `gemm_pass` (the stem convolution and attention excluded)."""
        total = 0.0
        for b in self.plan:
            T_in, T = b["side_in"] ** 2, b["side"] ** 2
            d_in, d = b["dim_in"], b["dim"]
            total += 2.0 * T_in * d_in * 3 * d + 2.0 * T * d * d + 4.0 * T * d * d * self.cfg.mlp_ratio
            if b["pool"]:
                total += 2.0 * T_in * d_in * d
        return total * self.batch

    def forward(self) -> DeviceArray:
        """Encode the images in `self.image` ((W,H,Cin,N), i.e. torch NCHW); the result, torch
        (N, H/32, W/32, 896), lands in `self.y`."""
        if getattr(self, "_gemm_only", False):
            x, spare, cur_w = self.xa, self.xb, self.cfg.windows[0]
            for b, w in zip(self.plan, self.blocks):
                self.ctx.ws.reset()
                x, spare, cur_w = self._block(b, w, x, spare, cur_w)
            return self.y
        ctx, cfg, B = self.ctx, self.cfg, self.batch
        k, s, p = cfg.patch
        S0, d0 = cfg.side(0), cfg.embed
        ctx.ws.reset()
        convolution_(ctx, self.stem_out, self.image, self.stem_w, self.stem_b, (s, s), (p, p), (1, 1))
        # planar (OW,OH,Cout,N) -> tokens (C,W,H,N): the permute + clone after the stem
        planar = self.stem_out.reshape(S0 * S0, d0, B)
        ctx.contiguous(planar.permute((1, 0, 2)), out=self._view(self.xb, d0, S0 * S0, B))
        x, spare = self.xa, self.xb
        self._to_windows(x, spare, d0, S0, cfg.windows[0])
        add_(ctx, self._view(x, d0 * S0 * S0 * B), self._view(x, d0 * S0 * S0 * B), self.pos.reshape(d0 * S0 * S0 * B))
        cur_w = cfg.windows[0]
        pending = False        # the MLP output of the previous block still to be added to the stream (in self.tmp)
        for i, (b, w) in enumerate(zip(self.plan, self.blocks)):
            ctx.ws.reset()
            # the residual add that ends a block is folded into the next block's first layer norm, unless
            # the tokens are re-ordered in between (after a pooling block) or there is no next block
            defer = i + 1 < len(self.plan) and not (b["pool"] and cfg.windows[b["stage"]] != cur_w // 2)
            x, spare, cur_w = self._block(b, w, x, spare, cur_w, pending, defer)
            pending = defer
        last = self.plan[-1]
        self._to_raster(self.y, x, last["dim"], last["side"], cur_w)
        return self.y

    def _block(self, b: dict, w: Dict[str, DeviceArray], x: DeviceArray, spare: DeviceArray, cur_w: int,
               pending: bool = False, defer: bool = False):
        ctx, cfg, B = self.ctx, self.cfg, self.batch
        every = not getattr(self, "_gemm_only", False)   # False: only the GEMM launches (see gemm_pass)
        d_in, d, H, E = b["dim_in"], b["dim"], b["heads"], cfg.head_dim
        T_in, T = b["side_in"] ** 2 * B, b["side"] ** 2 * B
        Lk = b["window"] ** 2 if b["window"] else b["side_in"] ** 2
        nwin = T_in // Lk
        if b["window"]:
            assert b["window"] == cur_w, "the token order must match the block's window"
        xv = self._view(x, d_in, T_in)
        h = self._view(self.h, d_in, T_in)
        mean, rstd = DeviceArray(ctx, self.mean.ptr, np.float32, (T_in,), owner=self.mean), \
            DeviceArray(ctx, self.rstd.ptr, np.float32, (T_in,), owner=self.rstd)
        if not every:
            pass
        elif pending:      # x += (previous block's MLP output); h = LN1(x)
            add_layernorm_(ctx, h, mean, rstd, xv, self._view(self.tmp, d_in, T_in), w["ln1_g"], w["ln1_b"], d_in, cfg.eps)
        else:
            layernorm_(ctx, h, mean, rstd, xv, w["ln1_g"], w["ln1_b"], d_in, cfg.eps)
        qkv = self._view(self.qkv, 3 * d, T_in)
        matmul_(ctx, qkv, w["wqkv"], h, w["bqkv"])
        part = lambda i: DeviceArray(ctx, qkv.ptr + i * d * 2, np.float16, (E, Lk, H, nwin), (1, 3 * d, E, 3 * d * Lk), owner=qkv)
        if b["pool"]:
            ww = b["window"]
            Lq = Lk // 4
            # shortcut: widen, then 2x2 max-pool inside each window
            sc = self._view(self.sc, d, T_in)
            matmul_(ctx, sc, w["wproj"], h, w["bproj"])
            pooled = lambda buf: DeviceArray(ctx, buf.ptr, np.float16, (ww // 2, ww // 2, d, nwin),
                                             (d, d * (ww // 2), 1, d * Lq), owner=buf)
            sc_in = DeviceArray(ctx, sc.ptr, np.float16, (ww, ww, d, nwin), (d, d * ww, 1, d * Lk), owner=sc)
            if every:
                maxpool2d_(ctx, pooled(spare), sc_in, (2, 2), (2, 2))
            # queries: the q rows of qkv pooled the same way
            q_in = DeviceArray(ctx, qkv.ptr, np.float16, (ww, ww, d, nwin), (3 * d, 3 * d * ww, 1, 3 * d * Lk), owner=qkv)
            if every:
                maxpool2d_(ctx, pooled(self.qp), q_in, (2, 2), (2, 2))
            q = DeviceArray(ctx, self.qp.ptr, np.float16, (E, Lq, H, nwin), (1, d, E, d * Lq), owner=self.qp)
            x_new, spare_new = spare, x            # the pooled shortcut is the new residual stream
        else:
            Lq = Lk
            q = part(0)
            x_new, spare_new = x, spare
        att = self._view(self.att, d, T)
        att_view = DeviceArray(ctx, att.ptr, np.float16, (E, Lq, H, nwin), (1, d, E, d * Lq), owner=att)
        if every:
            sdpa(ctx, q, part(1), part(2), None, 1.0 / sqrt(E), out=att_view)
        o = self._view(self.tmp, d, T)
        matmul_(ctx, o, w["wo"], att, w["bo"])
        xn = self._view(x_new, d, T)
        h2 = self._view(self.h, d, T)
        mean2, rstd2 = DeviceArray(ctx, self.mean.ptr, np.float32, (T,), owner=self.mean), \
            DeviceArray(ctx, self.rstd.ptr, np.float32, (T,), owner=self.rstd)
        if every:
            add_layernorm_(ctx, h2, mean2, rstd2, xn, o, w["ln2_g"], w["ln2_b"], d, cfg.eps)        # x += o; h = LN2(x)
        ff = self._view(self.ff, d * cfg.mlp_ratio, T)
        matmul_(ctx, ff, w["w1"], h2, w["b1"], epi="gelu")
        matmul_(ctx, o, w["w2"], ff, w["b2"])
        if not defer and every:
            add_(ctx, self._view(x_new, d * T), self._view(x_new, d * T), self._view(self.tmp, d * T))
        new_w = cur_w
        if b["pool"]:
            # tokens now sit in the left stage's windows at half the side; move to this stage's windows
            new_w = cfg.windows[b["stage"]]
            if new_w != cur_w // 2 and every:
                self._to_raster(spare_new, x_new, d, b["side"], cur_w // 2)
                self._to_windows(x_new, spare_new, d, b["side"], new_w)
        return x_new, spare_new, new_w

    # ---- capture
    def capture(self):
        self.forward()
        self.ctx.synchronize()
        self._graph = self.ctx.capture(self.forward)
        return self._graph

    def launches_per_pass(self) -> int:
        n0 = self.ctx.launch_count()
        self.forward()
        return self.ctx.launch_count() - n0
