import numpy as np
import pytest

import juliavision_b200 as jv
from juliavision_b200.encoder import Encoder, EncoderConfig, init_weights

from .conftest import relerr
from .gpu_helpers import describe

pytestmark = pytest.mark.gpu


def _run(ctx, cfg, x, graph=False, fused=True):
    w = init_weights(cfg)
    enc = Encoder(ctx, cfg, w, fused=fused)
    ctx.upload(enc.xin, x)
    if graph:
        g = enc.capture()
        ctx.fill_bytes(enc.y, 0xFF)
        g.replay()
    else:
        enc.forward()
    ctx.synchronize()
    return enc, w, enc.y.to_host()


def test_two_layer_prefix_vs_oracle(ctx):
    """The reference verifies a 2-block prefix on its CPU backend (verify.jl:115-118); so does this."""
    from oracle.encoder_ref import oracle_forward
    cfg = EncoderConfig(layers=2, d_model=256, heads=4, ffn=1024, tokens=300)
    x = np.float16(np.random.default_rng(1).standard_normal((cfg.tokens, cfg.d_model)))
    enc, w, got = _run(ctx, cfg, x)
    ref = oracle_forward(cfg, w, x)
    assert got.shape == (cfg.tokens, cfg.d_model)
    assert relerr(got, ref) < 1e-2, describe(got, ref, 1e-2)


def test_fused_rewrites_change_no_value(ctx):
    """qkv in one GEMM, token-major sdpa store and add(+clamp)+LN in one launch are rewrites, not
    approximations: the pass must give the op-by-op result bit for bit."""
    cfg = EncoderConfig(layers=2, d_model=256, heads=4, ffn=1024, tokens=300)
    x = np.float16(np.random.default_rng(4).standard_normal((cfg.tokens, cfg.d_model)))
    _, _, plain = _run(ctx, cfg, x, fused=False)
    _, _, fused = _run(ctx, cfg, x, fused=True)
    assert np.array_equal(plain, fused)


def test_add_layernorm_equals_the_three_ops(ctx):
    rng = np.random.default_rng(5)
    for groups, C in ((300, 256), (77, 1280), (5, 100), (4097, 112), (1001, 64), (3, 56), (65, 128)):
        x0 = np.float16(rng.standard_normal((groups, C)) * 300)
        h0 = np.float16(rng.standard_normal((groups, C)) * 300)
        g = np.float16(1 + 0.1 * rng.standard_normal(C))
        b = np.float16(0.1 * rng.standard_normal(C))
        dg, db = ctx.toback(g), ctx.toback(b)
        mean, rstd = ctx.allocate(np.float32, groups), ctx.allocate(np.float32, groups)
        xa, ha, oa = ctx.toback(x0), ctx.toback(h0), ctx.allocate(np.float16, C, groups)
        jv.add_(ctx, xa, xa, ha)
        jv.clamp_(ctx, xa, xa, -500.0, 500.0)
        jv.layernorm_(ctx, oa, mean, rstd, xa, dg, db, C, 1e-5)
        xb, hb, ob = ctx.toback(x0), ctx.toback(h0), ctx.allocate(np.float16, C, groups)
        jv.add_layernorm_(ctx, ob, mean, rstd, xb, hb, dg, db, C, 1e-5, clamp=(-500.0, 500.0))
        ctx.synchronize()
        assert np.array_equal(xa.to_host(), xb.to_host())
        assert np.array_equal(oa.to_host(), ob.to_host())


def test_graph_replay_equals_eager(ctx):
    cfg = EncoderConfig(layers=3, d_model=128, heads=2, ffn=512, tokens=200)
    x = np.float16(np.random.default_rng(2).standard_normal((cfg.tokens, cfg.d_model)))
    _, _, eager = _run(ctx, cfg, x, graph=False)
    _, _, replay = _run(ctx, cfg, x, graph=True)
    assert np.array_equal(eager, replay)


def test_config3_shape_one_layer_vs_oracle(ctx):
    """Config-3 geometry (d 1280, 20 heads of 64, FFN 5120, 1500 tokens), one layer of the 32."""
    from oracle.encoder_ref import oracle_forward
    cfg = EncoderConfig(layers=1)
    x = np.float16(np.random.default_rng(3).standard_normal((cfg.tokens, cfg.d_model)))
    enc, w, got = _run(ctx, cfg, x)
    ref = oracle_forward(cfg, w, x)
    assert relerr(got, ref) < 1e-2, describe(got, ref, 1e-2)


def test_config3_four_layer_prefix_at_full_geometry_vs_oracle(ctx):
    """The benchmarked stack deeper than one layer at its real size: the residual stream after 4 of the
    32 layers (d 1280, 20 heads of 64, FFN 5120, 1500 tokens) against the oracle's prefix — the
    reference's own gate is a block prefix on its CPU backend (verify.jl:115-118) — and the closing
    layer norm of a 4-layer stack on top of it."""
    from oracle.encoder_ref import oracle_forward
    full = EncoderConfig()
    cfg = EncoderConfig(layers=4)
    x = np.float16(np.random.default_rng(8).standard_normal((cfg.tokens, cfg.d_model)))
    enc, w, got = _run(ctx, cfg, x, graph=True)
    ref_prefix = oracle_forward(full, w, x, layers=4)            # no closing layer norm: 4 < 32
    stream = enc.x.to_host()
    assert relerr(stream, ref_prefix) < 1e-2, describe(stream, ref_prefix, 1e-2)
    ref = oracle_forward(cfg, w, x)
    assert relerr(got, ref) < 1e-2, describe(got, ref, 1e-2)


def test_exported_graph_through_execute_equals_direct_calls(ctx):
    """The same encoder as an exported-graph JSON, run by Model/execute! with the static slab plan and
    the load-time rewrites, must give the op-by-op pass bit for bit — planned, with no allocation
    outside the plan except the transposed-weight staging it never needs after hoisting."""
    import json

    from juliavision_b200.encoder_graph import encoder_graph
    from juliavision_b200.execute import Model
    from juliavision_b200.graph import loadgraph
    cfg = EncoderConfig(layers=2, d_model=256, heads=4, ffn=1024, tokens=300)
    w = init_weights(cfg)
    x = np.float16(np.random.default_rng(6).standard_normal((cfg.tokens, cfg.d_model)))
    g, wts = encoder_graph(cfg, w)
    graph = loadgraph(json.loads(json.dumps(g)))
    model = Model(ctx, graph, wts)
    assert model.rewrites == dict(hoistpermutes=6 * cfg.layers, foldgelu=cfg.layers, foldoutcasts=0, foldincasts=0)
    (out,) = model(x.reshape(1, cfg.tokens, cfg.d_model))
    ctx.synchronize()
    got = out.to_host().reshape(cfg.tokens, cfg.d_model)
    _, _, plain = _run(ctx, cfg, x, fused=False)
    assert np.array_equal(got, plain)
    from juliavision_b200.plan import escaping
    esc = escaping(model.graph)
    assert all(k.rsplit('.', 1)[0] in esc for k in model.planmisses), model.planmisses   # only the escaping output misses the slab
    # and unrewritten (t(W) views materialised per call, gelu as its own op): same values
    (out2,) = Model(ctx, graph, wts, rewrite=False)(x.reshape(1, cfg.tokens, cfg.d_model))
    ctx.synchronize()
    assert np.array_equal(out2.to_host().reshape(cfg.tokens, cfg.d_model), plain)


def test_streamed_passes_give_each_input_its_own_result(ctx):
    """Uploads and downloads on the copy lane overlapped with the replayed pass: seven different inputs streamed
    through one recorded encoder must each come back as the result of a plain upload -> pass -> download of that
    input (so no staging buffer is overwritten before it has been read, in either direction)."""
    import ctypes as C

    from juliavision_b200 import _lib
    cfg = EncoderConfig(layers=2, d_model=256, heads=4, ffn=1024, tokens=300)
    enc = Encoder(ctx, cfg, init_weights(cfg))
    rng = np.random.default_rng(21)
    n = 7
    xs = [np.float16(rng.standard_normal((cfg.tokens, cfg.d_model))) for _ in range(n)]
    want = []
    for x in xs:
        ctx.upload(enc.xin, x)
        enc.forward()
        ctx.synchronize()
        want.append(enc.y.to_host())
    g = enc.capture()
    nbytes = xs[0].nbytes
    hin, hout = [], []
    for x in xs:
        a, b = C.c_void_p(), C.c_void_p()
        _lib.check(_lib.lib().b200_host_alloc(nbytes, C.byref(a)))
        _lib.check(_lib.lib().b200_host_alloc(nbytes, C.byref(b)))
        C.memmove(a.value, x.ctypes.data, nbytes)
        C.memset(b.value, 0xFF, nbytes)
        hin.append(a.value)
        hout.append(b.value)
    # both forms: an already recorded graph with the staging copies around it, and the launching callable, from
    # which StreamedPass records one graph per staging pair with the copies inside
    for fwd in (g, enc.forward):
        for p_ in hout:
            C.memset(p_, 0xFF, nbytes)
        sp = jv.StreamedPass(ctx, fwd, enc.xin, enc.y)
        sp.run(hin, hout)
        ctx.synchronize()
        for i in range(n):
            got = np.frombuffer((C.c_char * nbytes).from_address(hout[i]), dtype=np.float16).reshape(cfg.tokens, cfg.d_model)
            assert np.array_equal(got, want[i]), f"pass {i}"
    for p_ in hin + hout:
        _lib.lib().b200_host_free(C.c_void_p(p_))


def test_diagnostics_time_ops_without_changing_values(ctx):
    """Per-op times (a serialising measurement), launches per op, and an op run twice in situ: the values of
    the pass do not change, every aten of the graph is in the table, and the counts are the graph's."""
    import json

    from juliavision_b200.encoder_graph import encoder_graph
    from juliavision_b200.execute import Model
    from juliavision_b200.graph import loadgraph
    cfg = EncoderConfig(layers=2, d_model=256, heads=4, ffn=1024, tokens=300)
    w = init_weights(cfg)
    x = np.float16(np.random.default_rng(9).standard_normal((cfg.tokens, cfg.d_model)))
    g, wts = encoder_graph(cfg, w)
    model = Model(ctx, loadgraph(json.loads(json.dumps(g))), wts)
    (plain,) = model(x.reshape(1, cfg.tokens, cfg.d_model))
    ctx.synchronize()
    plain = plain.to_host()
    model.diag.optimes, model.diag.launches = {}, {}
    (timed,) = model(x.reshape(1, cfg.tokens, cfg.d_model))
    ctx.synchronize()
    assert np.array_equal(timed.to_host(), plain)
    atens = {op.aten for op in model.graph.ops}
    assert set(model.diag.optimes) == atens == set(model.diag.launches)
    counts = {a: sum(op.aten == a for op in model.graph.ops) for a in atens}
    assert {a: n for a, (n, _) in model.diag.optimes.items()} == counts
    assert all(ms > 0 for _, _, ms in model.diag.table())
    assert model.diag.launches["addmm.default"][1] >= counts["addmm.default"]
    model.diag.optimes = model.diag.launches = None
    model.diag.opdouble = "addmm.default"
    n0 = ctx.launch_count()
    (doubled,) = model(x.reshape(1, cfg.tokens, cfg.d_model))
    ctx.synchronize()
    assert np.array_equal(doubled.to_host(), plain)
    model.diag.opdouble = ""
    n1 = ctx.launch_count()
    model(x.reshape(1, cfg.tokens, cfg.d_model))
    ctx.synchronize()
    assert (n1 - n0) - (ctx.launch_count() - n1) == counts["addmm.default"]     # one extra launch per doubled op
