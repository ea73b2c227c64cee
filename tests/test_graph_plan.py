"""Host-side graph format, shape evaluation, slab planning and rewrite passes (no GPU).
Invariants follow the reference's test_plan.jl: no two simultaneously-live buffers share a byte,
the slab stays within 1.6x of the liveness bound, outputs are never planned."""
import json

import numpy as np

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
