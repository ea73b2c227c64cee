"""The hierarchical image encoder composed from the CPU oracle's ops (test infrastructure, not
product): the checker for juliavision_b200.hiera.Hiera and the body of its timed CPU baseline.

Written the way the exported graph runs it — raster-order (B,H,W,C) tokens, a window partition
before and an un-partition after every windowed attention, max_pool2d on NCHW permutes — and
therefore independent of the window-ordered token layout the device side keeps.
"""
from math import sqrt

import numpy as np

from . import oracle as ora


def _partition(x, w):
    """(B,S,S,C) -> (B*nW, w*w, C), windows row-major."""
    B, S, _, Cn = x.shape
    return np.ascontiguousarray(x.reshape(B, S // w, w, S // w, w, Cn).transpose(0, 1, 3, 2, 4, 5)).reshape(-1, w * w, Cn)


def _unpartition(xw, w, B, S):
    Cn = xw.shape[-1]
    return np.ascontiguousarray(xw.reshape(B, S // w, S // w, w, w, Cn).transpose(0, 1, 3, 2, 4, 5)).reshape(B, S, S, Cn)


def _pool(x):
    """do_pool: (B,S,S,C) -> NCHW -> max_pool2d 2x2 stride 2 -> back."""
    y = ora.maxpool2d(np.ascontiguousarray(x.transpose(0, 3, 1, 2)), (2, 2), (2, 2))
    return np.ascontiguousarray(y.transpose(0, 2, 3, 1))


def _linear(x, W, b, epi="none"):
    sh = x.shape
    y = ora.linear(np.ascontiguousarray(x.reshape(-1, sh[-1])), np.ascontiguousarray(W.T), b, epi=epi)
    return y.reshape(*sh[:-1], W.shape[0])


def oracle_forward(cfg, weights, image: np.ndarray, blocks=None):
    """image: torch (B, Cin, H, W) fp16.  Returns torch (B, S, S, C) fp16 after `blocks` blocks
    (all of them by default)."""
    k, s, p = cfg.patch
    B = image.shape[0]
    E = cfg.head_dim
    x = ora.conv2d(image, weights["stem_w"], weights["stem_b"], stride=(s, s), padding=(p, p))   # (B,C,S,S) fp16
    x = np.ascontiguousarray(x.transpose(0, 2, 3, 1))
    x = ora.add(x, np.ascontiguousarray(np.broadcast_to(weights["pos"][None], x.shape)))
    plan = cfg.blocks()
    for b, w in list(zip(plan, weights["blocks"]))[: len(plan) if blocks is None else blocks]:
        d, H, S_in, S = b["dim"], b["heads"], b["side_in"], b["side"]
        h, _, _ = ora.layernorm(x, w["ln1_g"], w["ln1_b"], cfg.eps)
        shortcut = x
        if b["pool"]:
            shortcut = _pool(_linear(h, w["wproj"], w["bproj"]))
        win = b["window"]
        hw = _partition(h, win) if win else h.reshape(B, S_in * S_in, -1)
        qkv = _linear(hw, w["wqkv"], w["bqkv"])                       # (nW, L, 3d)
        nW, L = qkv.shape[0], qkv.shape[1]
        q, kk, v = (qkv[..., i * d:(i + 1) * d] for i in range(3))
        if b["pool"]:
            q = _pool(np.ascontiguousarray(q).reshape(nW, win, win, d)).reshape(nW, L // 4, d)
        heads = lambda t: t.reshape(t.shape[0], t.shape[1], H, E).transpose(0, 2, 1, 3)   # (nW,H,L,E) view
        att = ora.attention_ref(heads(q), heads(kk), heads(v), 1.0 / sqrt(E)).astype(np.float16)
        att = np.ascontiguousarray(att.transpose(0, 2, 1, 3)).reshape(nW, -1, d)
        o = _linear(att, w["wo"], w["bo"])
        if win:
            o = _unpartition(o, win // 2 if b["pool"] else win, B, S)
        else:
            o = o.reshape(B, S, S, d)
        x = ora.add(np.ascontiguousarray(shortcut), np.ascontiguousarray(o))
        h, _, _ = ora.layernorm(x, w["ln2_g"], w["ln2_b"], cfg.eps)
        f = _linear(h, w["w1"], w["b1"], epi="gelu")
        x = ora.add(x, _linear(f, w["w2"], w["b2"]))
    return x
