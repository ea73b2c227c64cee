"""Load-time graph rewrites that touch weights or fold whole ops away, on the host (numpy):
`hoistcasts` (reference hoistcasts.jl:185-226), `foldbatchnorm` (foldbn.jl:44-143) and the relu half
of `foldrelu` (foldrelu.jl:35-132).  The folds on the attention/MLP path (hoistpermutes, the gelu fold,
foldoutcasts, foldincasts) live beside the op loop in execute.py; these three are the ones convolutional
graphs need before their convolutions reach the GEMM with everything fused into its store.

Each pass edits the graph in place and returns how many ops it removed; weights it creates are added to
the `weights` dict under keys scoped by graph name and op id (one weight table serves every graph).
"""
from __future__ import annotations

from typing import Dict, Optional

import numpy as np

from .graph import Buffer, Graph, Op

_ALIAS = ("alias.default", "detach.default")


def weightsource(graph: Graph, id: str) -> Optional[Buffer]:
    """Follow `_to_copy` / clone / alias chains from `id` back to the weight buffer that feeds it, or
    None when anything computed intervenes (hoistcasts.jl:26-45)."""
    producer = {o.out: o for o in graph.ops}
    for _ in range(16):
        b = graph.buffers.get(id)
        if b is None:
            return None
        if b.kind == "weight":
            return b
        if b.kind == "view" and b.viewop in _ALIAS:
            id = b.of
            continue
        op = producer.get(id)
        if op is None or op.aten not in ("_to_copy.default", "clone.default", "detach.default") or len(op.ins) != 1:
            return None
        id = op.ins[0]
    return None


def resolvealias(graph: Graph, id: str) -> str:
    for _ in range(16):
        b = graph.buffers.get(id)
        if b is None or b.kind != "view" or b.viewop not in _ALIAS:
            break
        id = b.of
    return id


def hoistcasts(graph: Graph, weights: Dict[str, np.ndarray]) -> int:
    """A `_to_copy` of a weight is evaluated now: its result becomes a weight of the declared dtype."""
    drop, n = set(), 0
    for op in graph.ops:
        if op.aten != "_to_copy.default" or len(op.ins) != 1:
            continue
        src = weightsource(graph, op.ins[0])
        ob = graph.buffers.get(op.out)
        if src is None or src.key not in weights or ob is None:
            continue
        key = f"{graph.name}|{op.id}|hoistcast"
        weights[key] = np.asarray(weights[src.key]).astype(ob.dtype)
        graph.buffers[op.out] = Buffer(op.out, "weight", list(ob.shape), ob.dtype, key=key)
        drop.add(op.id)
        n += 1
    if n:
        graph.ops[:] = [o for o in graph.ops if o.id not in drop]
    return n


def foldbatchnorm(graph: Graph, weights: Dict[str, np.ndarray]) -> int:
    """Inference batch norm after a convolution is an affine map with constant coefficients,
    z = (s W) * x + (s b + beta - mu s) with s = gamma / sqrt(var + eps): absorb it into the convolution's
    weight and bias and delete the op.  Scaled in fp32 from the master weight and rounded once to the
    operand's declared dtype.  Only when the convolution feeds nothing else and only element 0 of the
    batch norm's tuple is read."""
    producer = {o.out: o for o in graph.ops}
    uses: Dict[str, int] = {}

    def bump(i):
        uses[i] = uses.get(i, 0) + 1

    for o in graph.ops:
        for i in o.ins:
            bump(i)
    for b in graph.buffers.values():
        if b.of:
            bump(b.of)
    for o in graph.outputs:
        bump(o)
    drop, n = set(), 0
    for bn in list(graph.ops):
        if bn.aten != "_native_batch_norm_legit_no_training.default" or len(bn.ins) < 5:
            continue
        conv = producer.get(bn.ins[0])
        if conv is None or conv.aten != "convolution.default" or uses.get(conv.out, 0) != 1:
            continue
        readers = [b for b in graph.buffers.values() if b.of == bn.out]
        if not all("getitem" in b.viewop and int(b.attrs.get("arg1", 0)) == 0 for b in readers):
            continue
        if uses.get(bn.out, 0) != len(readers):
            continue
        srcs = [weightsource(graph, i) for i in (bn.ins[1], bn.ins[2], bn.ins[3], bn.ins[4], conv.ins[1])]
        if any(s is None or s.key not in weights for s in srcs):
            continue
        gamma, beta, mu, var, w = (np.asarray(weights[s.key], dtype=np.float32) for s in srcs)
        eps = np.float32(bn.attrs["arg6"])
        hasbias = len(conv.ins) >= 3
        bsrc = weightsource(graph, conv.ins[2]) if hasbias else None
        if hasbias and (bsrc is None or bsrc.key not in weights):
            continue
        s = gamma / np.sqrt(var + eps)
        b0 = np.asarray(weights[bsrc.key], dtype=np.float32) if hasbias else np.zeros_like(s)
        wb = graph.buffers[conv.ins[1]]
        new_w = (w * s.reshape(-1, *([1] * (w.ndim - 1)))).astype(wb.dtype)     # torch (Cout, Cin, KH, KW): Cout leads
        bbuf = graph.buffers[conv.ins[2]] if hasbias else graph.buffers[bn.ins[2]]
        new_b = (b0 * s + (beta - mu * s)).astype(bbuf.dtype)
        wkey, bkey = f"{graph.name}|{conv.id}|foldbn_weight", f"{graph.name}|{conv.id}|foldbn_bias"
        weights[wkey], weights[bkey] = new_w, new_b
        wid, bid = f"{conv.id}|foldbn_weight", f"{conv.id}|foldbn_bias"
        graph.buffers[wid] = Buffer(wid, "weight", list(wb.shape), wb.dtype, key=wkey)
        graph.buffers[bid] = Buffer(bid, "weight", list(bbuf.shape), bbuf.dtype, key=bkey)
        graph.order += [wid, bid]
        conv.ins[:] = [conv.ins[0], wid, bid]
        for b in readers:       # the getitem that read bn[0] now aliases the convolution's own output
            graph.buffers[b.id] = Buffer(b.id, "view", list(b.shape), b.dtype, of=conv.out, viewop="alias.default",
                                         attrs=dict(b.attrs))
        drop.add(bn.id)
        n += 1
    if n:
        graph.ops[:] = [o for o in graph.ops if o.id not in drop]
    return n


def foldrelu(graph: Graph) -> int:
    """relu(convolution) and relu(add) with no other reader of the producer: the activation moves into
    the producer's store (`attrs["act"] = "relu"`) and the relu's buffer becomes an alias.  Aliases are
    not uses: whoever reads one has been counted against the buffer it resolves to."""
    producer = {o.out: o for o in graph.ops}
    uses: Dict[str, int] = {}

    def bump(i):
        r = resolvealias(graph, i)
        uses[r] = uses.get(r, 0) + 1

    for o in graph.ops:
        for i in o.ins:
            bump(i)
    for b in graph.buffers.values():
        if b.of and not (b.kind == "view" and b.viewop in _ALIAS):
            bump(b.of)
    for o in graph.outputs:
        bump(o)
    drop, n = set(), 0
    for relu in list(graph.ops):
        if relu.aten != "relu.default" or len(relu.ins) != 1:
            continue
        src = resolvealias(graph, relu.ins[0])
        p = producer.get(src)
        if p is None or p.aten not in ("convolution.default", "add.Tensor") or uses.get(src, 0) != 1 or "act" in p.attrs:
            continue
        ob, cb = graph.buffers[relu.out], graph.buffers[p.out]
        if np.dtype(ob.dtype) != np.dtype(cb.dtype):
            continue
        p.attrs["act"] = "relu"
        graph.buffers[relu.out] = Buffer(relu.out, "view", list(ob.shape), ob.dtype, of=p.out, viewop="alias.default",
                                         attrs=dict(ob.attrs))
        drop.add(relu.id)
        n += 1
    if n:
        graph.ops[:] = [o for o in graph.ops if o.id not in drop]
    return n
