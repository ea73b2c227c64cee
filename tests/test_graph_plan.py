"""Host-side graph format, shape evaluation, slab planning and rewrite passes (no GPU).
Invariants follow the reference's test_plan.jl: no two simultaneously-live buffers share a byte,
the slab stays within 1.6x of the liveness bound, outputs are never planned."""
import json

import numpy as np
import pytest

from juliavision_b200.encoder import EncoderConfig, init_weights
from juliavision_b200.encoder_graph import encoder_graph
from juliavision_b200.execute import foldgelu, hoistpermutes
from juliavision_b200.graph import evalexpr, evalshape, loadgraph
from juliavision_b200.plan import alignup, checkslab, escaping, lifetimes, liveness_bound, planslab


def small():
    cfg = EncoderConfig(layers=3, d_model=128, heads=2, ffn=512, tokens=200)
    w = init_weights(cfg)
    g, wts = encoder_graph(cfg, w)
    return cfg, loadgraph(json.loads(json.dumps(g))), wts       # through real JSON text


def test_shapes_are_reversed_and_symbolic():
    assert evalshape([1, 20, "h*w", 64], dict(h=10, w=15)) == (64, 150, 20, 1)
    assert evalexpr("(h + 2*1 - 3)//2 + 1", dict(h=3000)) == 1500
    assert evalexpr("Max(h, 7)", dict(h=3)) == 7 and evalexpr("floor(h/4)", dict(h=10)) == 2
    assert alignup(1) == 256 and alignup(256) == 256 and alignup(257) == 512


def test_loadgraph_roundtrip():
    cfg, g, wts = small()
    assert g.inputs == ["x"] and len(g.outputs) == 1
    per_layer = 2 + 3 + 1 + 1 + 1 + 1 + 2 + 1 + 1 + 1      # ln, qkv, sdpa, clone, out, add, ffn(2)+gelu, add, clamp
    assert len(g.ops) == cfg.layers * per_layer + 1
    atens = {o.aten for o in g.ops}
    assert {"addmm.default", "mm.default", "_scaled_dot_product_flash_attention.default",
            "native_layer_norm.default", "gelu.default", "clamp.default", "clone.default", "add.Tensor"} <= atens
    tup = next(b for b in g.buffers.values() if b.attrs.get("shapes") and len(b.attrs["shapes"]) == 3)
    assert tup.attrs["dtypes"] == [np.float16, np.float32, np.float32] and tup.shape == []


def test_plan_invariants():
    cfg, g, wts = small()
    slab = planslab(g, {})
    planned, conflicts = checkslab(g, {}, slab)
    assert planned > 0 and conflicts == 0
    assert all(o % 256 == 0 for o in slab.offsets.values())
    assert slab.bytes <= 1.6 * liveness_bound(g, {}, slab)
    esc = escaping(g)
    assert not (set(slab.offsets) & esc)                       # escaping values are never planned
    total = sum(slab.sizes.values())
    assert slab.bytes < total / 4                              # lifetimes are worth a lot of reuse
    lt = lifetimes(g)
    assert all(a <= b for a, b in lt.values())
    # a tuple-valued op is planned per element, under "<id>.<i>"
    assert any(k.endswith(".1") for k in slab.offsets) and any(k.endswith(".2") for k in slab.offsets)


def test_hoistpermutes_and_foldgelu():
    cfg, g, wts = small()
    n_lin = sum(o.aten in ("addmm.default", "mm.default") for o in g.ops)
    assert hoistpermutes(g, wts) == n_lin
    for o in g.ops:
        if o.aten in ("addmm.default", "mm.default"):
            b = g.buffers[o.ins[2 if o.aten == "addmm.default" else 1]]
            assert b.kind == "weight" and b.key.endswith("@t")
            src = wts[b.key[:-2]]
            assert np.array_equal(wts[b.key], src.T) and wts[b.key].flags["C_CONTIGUOUS"]
    before = len(g.ops)
    assert foldgelu(g) == cfg.layers
    assert len(g.ops) == before - cfg.layers and not any(o.aten == "gelu.default" for o in g.ops)
    assert sum(o.attrs.get("act") == "gelu" for o in g.ops) == cfg.layers
    assert checkslab(g, {}, planslab(g, {}))[1] == 0           # still a valid plan after the rewrites


def _write_safetensors(path, tensors, metadata=None):
    import json
    import struct
    names = {np.dtype(np.float16): "F16", np.dtype(np.float32): "F32", np.dtype(np.int64): "I64", np.dtype(np.uint16): "BF16",
             np.dtype(np.bool_): "BOOL"}
    header, blobs, off = {}, [], 0
    if metadata:
        header["__metadata__"] = metadata
    for k, v in tensors.items():
        raw = np.ascontiguousarray(v).tobytes()
        header[k] = {"dtype": names[v.dtype], "shape": list(v.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    head = json.dumps(header).encode()
    head += b" " * (-len(head) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(head)))
        f.write(head)
        for b in blobs:
            f.write(b)


def test_readsafetensors_round_trip(tmp_path):
    """safetensors.jl:14-58: header length, JSON header, raw little-endian data; shapes as stored (the
    upload reverses them), scalars 0-dimensional, bf16 as its bit patterns, metadata skipped."""
    from juliavision_b200.safetensors import readsafetensors, safetensorsnames
    rng = np.random.default_rng(0)
    t = {"enc.w": np.float16(rng.standard_normal((5, 3, 2))), "enc.b": np.float32(rng.standard_normal(7)),
         "step": np.array(41, dtype=np.int64), "bf": np.arange(6, dtype=np.uint16).reshape(2, 3),
         "mask": np.array([True, False, True])}
    path = str(tmp_path / "w.safetensors")
    _write_safetensors(path, t, metadata={"format": "pt"})
    assert sorted(safetensorsnames(path)) == sorted(t)
    got = readsafetensors(path)
    assert sorted(got) == sorted(t)
    for k in t:
        assert got[k].shape == t[k].shape and got[k].dtype == t[k].dtype
        assert np.array_equal(got[k], t[k])
    assert got["step"].ndim == 0 and int(got["step"]) == 41
    with open(path, "r+b") as f:                      # a file cut short is an error, not a short array
        f.truncate(40)
    with pytest.raises(ValueError):
        readsafetensors(path)


def _castgraph():
    """layer norm in fp32 -> getitem -> _to_copy to fp16 -> addmm; plus a widening cast that must stay."""
    from juliavision_b200.graph import loadgraph
    return loadgraph({
        "name": "casts", "symbols": [], "inputs": ["x"], "outputs": ["y", "wide"],
        "buffers": [
            {"id": "x", "kind": "external", "shape": [6, 16], "dtype": "float32"},
            {"id": "g", "kind": "weight", "shape": [16], "dtype": "float32", "key": "g"},
            {"id": "w", "kind": "weight", "shape": [16, 8], "dtype": "float16", "key": "w"},
            {"id": "b", "kind": "weight", "shape": [8], "dtype": "float16", "key": "b"},
            {"id": "ln", "kind": "transient", "shape": [], "dtype": "float32", "live": [1, 2],
             "shapes": [[6, 16], [6, 1], [6, 1]], "dtypes": ["float32", "float32", "float32"]},
            {"id": "ln0", "kind": "view", "shape": [6, 16], "dtype": "float32", "of": "ln", "op": "getitem", "attrs": {"arg1": 0}},
            {"id": "h", "kind": "transient", "shape": [6, 16], "dtype": "float16", "live": [2, 3]},
            {"id": "y", "kind": "transient", "shape": [6, 8], "dtype": "float16", "live": [3, 4]},
            {"id": "wide", "kind": "transient", "shape": [6, 8], "dtype": "float32", "live": [4, 4]},
        ],
        "ops": [
            {"id": "o1", "aten": "native_layer_norm.default", "in": ["x", "g", "g"], "out": "ln", "attrs": {"arg1": [16], "arg4": 1e-5}},
            {"id": "o2", "aten": "_to_copy.default", "in": ["ln0"], "out": "h", "attrs": {}},
            {"id": "o3", "aten": "addmm.default", "in": ["b", "h", "w"], "out": "y", "attrs": {}},
            {"id": "o4", "aten": "_to_copy.default", "in": ["y"], "out": "wide", "attrs": {}},
        ]})


def test_foldoutcasts_retypes_the_producer_and_keeps_widening_casts():
    """foldoutcasts.jl:82-155: the narrowing cast behind the layer norm disappears (its result becomes
    an alias and the tuple element is declared fp16); the widening cast stays."""
    from juliavision_b200.execute import foldoutcasts
    g = _castgraph()
    assert foldoutcasts(g) == 1
    assert [o.id for o in g.ops] == ["o1", "o3", "o4"]
    assert g.buffers["ln"].attrs["dtypes"][0] == np.float16 and g.buffers["ln"].attrs["dtypes"][1] == np.float32
    assert g.buffers["ln0"].dtype == np.float16
    h = g.buffers["h"]
    assert h.kind == "view" and h.of == "ln0" and h.viewop == "alias.default"
    assert foldoutcasts(g) == 0                      # idempotent


def test_foldoutcasts_needs_a_single_reader():
    from juliavision_b200.execute import foldoutcasts
    g = _castgraph()
    g.outputs.append("ln0")                          # someone else reads the wide value
    assert foldoutcasts(g) == 0


def _widegraph():
    """add in fp16 -> _to_copy to fp32 -> layer norm declared fp32; plus a widening cast read by an addmm."""
    from juliavision_b200.graph import loadgraph
    return loadgraph({
        "name": "widen", "symbols": [], "inputs": ["a", "b"], "outputs": ["ln0", "y"],
        "buffers": [
            {"id": "a", "kind": "external", "shape": [6, 16], "dtype": "float16"},
            {"id": "b", "kind": "external", "shape": [6, 16], "dtype": "float16"},
            {"id": "g", "kind": "weight", "shape": [16], "dtype": "float16", "key": "g"},
            {"id": "s", "kind": "transient", "shape": [6, 16], "dtype": "float16", "live": [1, 3]},
            {"id": "w32", "kind": "transient", "shape": [6, 16], "dtype": "float32", "live": [2, 3]},
            {"id": "ln", "kind": "transient", "shape": [], "dtype": "float32", "live": [3, 3],
             "shapes": [[6, 16], [6, 1], [6, 1]], "dtypes": ["float32", "float32", "float32"]},
            {"id": "ln0", "kind": "view", "shape": [6, 16], "dtype": "float32", "of": "ln", "op": "getitem", "attrs": {"arg1": 0}},
            {"id": "y", "kind": "transient", "shape": [6, 16], "dtype": "float32", "live": [4, 4]},
        ],
        "ops": [
            {"id": "o1", "aten": "add.Tensor", "in": ["a", "b"], "out": "s", "attrs": {}},
            {"id": "o2", "aten": "_to_copy.default", "in": ["s"], "out": "w32", "attrs": {}},
            {"id": "o3", "aten": "native_layer_norm.default", "in": ["w32", "g", "g"], "out": "ln", "attrs": {"arg1": [16], "arg4": 1e-5}},
            {"id": "o4", "aten": "_to_copy.default", "in": ["s"], "out": "y", "attrs": {}},
        ]})


def test_foldincasts_drops_the_widening_cast_in_front_of_a_layer_norm():
    """foldincasts.jl:82-124: the cast feeding the layer norm becomes an fp16 alias; a widening cast that
    is a graph output stays."""
    from juliavision_b200.execute import foldincasts
    g = _widegraph()
    assert foldincasts(g) == 1
    assert [o.id for o in g.ops] == ["o1", "o3", "o4"]
    w = g.buffers["w32"]
    assert w.kind == "view" and w.of == "s" and w.dtype == np.float16
    assert g.buffers["ln"].attrs["dtypes"][0] == np.float32       # the result keeps its declared dtype
    assert foldincasts(g) == 0
    wide = _widegraph()
    wide.buffers["g"].dtype = np.float32          # wide gamma: folding would force a rounding, so it is left alone
    assert foldincasts(wide) == 0


def _convnet_graph():
    """x -> convolution(w32 cast to fp16, bias) -> batch norm -> getitem 0 -> relu -> y"""
    from juliavision_b200.graph import loadgraph
    return loadgraph({
        "name": "convnet", "symbols": [], "inputs": ["x"], "outputs": ["y"],
        "buffers": [
            {"id": "x", "kind": "external", "shape": [2, 3, 8, 8], "dtype": "float16"},
            {"id": "w32", "kind": "weight", "shape": [4, 3, 3, 3], "dtype": "float32", "key": "conv.weight"},
            {"id": "w16", "kind": "transient", "shape": [4, 3, 3, 3], "dtype": "float16", "live": [1, 2]},
            {"id": "cb", "kind": "weight", "shape": [4], "dtype": "float16", "key": "conv.bias"},
            {"id": "g", "kind": "weight", "shape": [4], "dtype": "float32", "key": "bn.weight"},
            {"id": "b", "kind": "weight", "shape": [4], "dtype": "float32", "key": "bn.bias"},
            {"id": "m", "kind": "weight", "shape": [4], "dtype": "float32", "key": "bn.mean"},
            {"id": "v", "kind": "weight", "shape": [4], "dtype": "float32", "key": "bn.var"},
            {"id": "c", "kind": "transient", "shape": [2, 4, 8, 8], "dtype": "float16", "live": [2, 3]},
            {"id": "bn", "kind": "transient", "shape": [], "dtype": "float16", "live": [3, 4],
             "shapes": [[2, 4, 8, 8], [0], [0]], "dtypes": ["float16", "float32", "float32"]},
            {"id": "bn0", "kind": "view", "shape": [2, 4, 8, 8], "dtype": "float16", "of": "bn", "op": "getitem", "attrs": {"arg1": 0}},
            {"id": "y", "kind": "transient", "shape": [2, 4, 8, 8], "dtype": "float16", "live": [4, 4]},
        ],
        "ops": [
            {"id": "cast", "aten": "_to_copy.default", "in": ["w32"], "out": "w16", "attrs": {}},
            {"id": "conv", "aten": "convolution.default", "in": ["x", "w16", "cb"], "out": "c",
             "attrs": {"arg3": [1, 1], "arg4": [1, 1], "arg5": [1, 1], "arg6": False, "arg8": 1}},
            {"id": "bnop", "aten": "_native_batch_norm_legit_no_training.default", "in": ["c", "g", "b", "m", "v"], "out": "bn",
             "attrs": {"arg5": 0.1, "arg6": 1e-5}},
            {"id": "relu", "aten": "relu.default", "in": ["bn0"], "out": "y", "attrs": {}},
        ]})


def test_hoistcasts_foldbatchnorm_foldrelu_leave_one_convolution(ora):
    """hoistcasts.jl:185-226, foldbn.jl:44-143, foldrelu.jl:35-132 on conv -> bn -> relu: one convolution with
    a scaled weight, a folded bias and the relu in its store; the values match the op-by-op computation."""
    from juliavision_b200.rewrites import foldbatchnorm, foldrelu, hoistcasts
    rng = np.random.default_rng(0)
    w = {"conv.weight": np.float32(rng.standard_normal((4, 3, 3, 3)) * 0.2), "conv.bias": np.float16(rng.standard_normal(4) * 0.1),
         "bn.weight": np.float32(1 + 0.2 * rng.standard_normal(4)), "bn.bias": np.float32(0.1 * rng.standard_normal(4)),
         "bn.mean": np.float32(0.1 * rng.standard_normal(4)), "bn.var": np.float32(0.5 + rng.random(4))}
    g = _convnet_graph()
    assert hoistcasts(g, w) == 1 and g.buffers["w16"].kind == "weight" and w[g.buffers["w16"].key].dtype == np.float16
    assert foldbatchnorm(g, w) == 1
    assert foldrelu(g) == 1
    assert [o.aten for o in g.ops] == ["convolution.default"] and g.ops[0].attrs["act"] == "relu"
    assert g.buffers["y"].viewop == "alias.default" and g.buffers["bn0"].of == "c"
    wk, bk = g.buffers[g.ops[0].ins[1]].key, g.buffers[g.ops[0].ins[2]].key
    assert w[wk].dtype == np.float16 and w[bk].dtype == np.float16
    # values: folded convolution == relu(bn(conv(x))) up to the fp16 roundings the unfolded chain makes
    x = np.float16(rng.standard_normal((2, 3, 8, 8)))
    folded = ora.conv2d(x, w[wk], w[bk], padding=(1, 1), epi="relu").astype(np.float32)
    c = ora.conv2d(x, w["conv.weight"].astype(np.float16), w["conv.bias"], padding=(1, 1)).astype(np.float32)
    s = w["bn.weight"] / np.sqrt(w["bn.var"] + np.float32(1e-5))
    want = np.maximum(c * s[None, :, None, None] + (w["bn.bias"] - w["bn.mean"] * s)[None, :, None, None], 0)
    assert np.max(np.abs(folded - want)) < 2e-2 * max(1.0, float(np.max(np.abs(want))))
    assert foldbatchnorm(g, w) == 0 and foldrelu(g) == 0 and hoistcasts(g, w) == 0
