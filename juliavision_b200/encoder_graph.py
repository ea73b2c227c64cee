"""The transformer-encoder workload written out in the exported-graph JSON schema (the shape
torch.export + run_decompositions gives a pre-LayerNorm encoder under fp16 autocast: `linear` is a
`t` view of the weight + `addmm`/`mm`, layer norm is `native_layer_norm` + `getitem`, attention is
`_scaled_dot_product_flash_attention` on transposed views followed by a `clone`, the fp16 export adds
a `clamp` after each block).  No exported model files exist where this repository is built, so the
graph is synthesised from the schema (reference tools/export_graphs.py:111-230, graph.jl:9-149).
"""
from __future__ import annotations

from math import sqrt
from typing import Dict, List, Tuple

import numpy as np

from .encoder import F16_MAX, EncoderConfig


def encoder_graph(cfg: EncoderConfig, weights: List[dict]) -> Tuple[dict, Dict[str, np.ndarray]]:
    """Returns (graph dict in the JSON schema, {weight key: numpy array in torch layout})."""
    d, f, L, H, E = cfg.d_model, cfg.ffn, cfg.tokens, cfg.heads, cfg.head_dim
    buffers, ops, wts = [], [], {}
    n = [0]

    def uid(p):
        n[0] += 1
        return f"{p}_{n[0]}"

    def weight(key, arr):
        wts[key] = arr
        buffers.append(dict(id=key, kind="weight", shape=list(arr.shape), dtype="float16", key=key))
        return key

    def transient(p, shape, dtype="float16", **extra):
        i = uid(p)
        buffers.append(dict(id=i, kind="transient", shape=shape, dtype=dtype, **extra))
        return i

    def view(p, of, op, shape, **attrs):
        i = uid(p)
        buffers.append(dict(id=i, kind="view", of=of, op=op, shape=shape, dtype="float16", attrs=attrs))
        return i

    def emit(aten, ins, out, **attrs):
        ops.append({"id": uid("op"), "aten": aten, "in": ins, "out": out, "attrs": attrs})
        return out

    def layer_norm(x, g, b):
        t = transient("native_layer_norm", [], shapes=[[1, L, d], [1, L, 1], [1, L, 1]],
                      dtypes=["float16", "float32", "float32"])
        emit("native_layer_norm.default", [x, g, b], t, arg1=[d], arg4=cfg.eps)
        return view("getitem", t, "getitem", [1, L, d], arg1=0)

    def linear(x2, w, b, out_f):
        wt = view("t", w, "t.default", [wts[w].shape[1], wts[w].shape[0]])
        y = transient("addmm" if b else "mm", [L, out_f])
        if b:
            emit("addmm.default", [b, x2, wt], y)
        else:
            emit("mm.default", [x2, wt], y)
        return y

    buffers.append(dict(id="x", kind="external", shape=[1, L, d], dtype="float16"))
    x = "x"
    for li, lw in enumerate(weights[:-1]):
        W = {k: weight(f"l{li}.{k}", v) for k, v in lw.items()}
        h = layer_norm(x, W["ln1_g"], W["ln1_b"])
        h2 = view("view", h, "view.default", [L, d])
        q2, k2, v2 = linear(h2, W["wq"], W["bq"], d), linear(h2, W["wk"], None, d), linear(h2, W["wv"], W["bv"], d)
        heads = []
        for t in (q2, k2, v2):
            t4 = view("view", t, "view.default", [1, L, H, E])
            heads.append(view("transpose", t4, "transpose.int", [1, H, L, E], arg1=1, arg2=2))
        sd = transient("sdpa", [], shapes=[[1, H, L, E]] + [None] * 8, dtypes=["float16"] + [None] * 8)
        emit("_scaled_dot_product_flash_attention.default", heads, sd, scale=1.0 / sqrt(E))
        a0 = view("getitem", sd, "getitem", [1, H, L, E], arg1=0)
        aT = view("transpose", a0, "transpose.int", [1, L, H, E], arg1=1, arg2=2)
        ac = emit("clone.default", [aT], transient("clone", [1, L, H, E]))
        a2 = view("view", ac, "view.default", [L, d])
        o3 = view("view", linear(a2, W["wo"], W["bo"], d), "view.default", [1, L, d])
        x = emit("add.Tensor", [x, o3], transient("add", [1, L, d]))
        h2 = view("view", layer_norm(x, W["ln2_g"], W["ln2_b"]), "view.default", [L, d])
        g = emit("gelu.default", [linear(h2, W["w1"], W["b1"], f)], transient("gelu", [L, f]))
        y3 = view("view", linear(g, W["w2"], W["b2"], d), "view.default", [1, L, d])
        x = emit("add.Tensor", [x, y3], transient("add", [1, L, d]))
        if cfg.clamp:
            x = emit("clamp.default", [x], transient("clamp", [1, L, d]), arg1=-F16_MAX, arg2=F16_MAX)
    fin = {k: weight(f"final.{k}", v) for k, v in weights[-1].items()}
    out = layer_norm(x, fin["lnf_g"], fin["lnf_b"])
    graph = dict(name="encoder", symbols=[], inputs=["x"], outputs=[out], buffers=buffers, ops=ops)
    return graph, wts
