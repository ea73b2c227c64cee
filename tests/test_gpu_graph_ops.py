"""Graph-level ops around the hot path, run through Model/execute!: _to_copy (and its fold into the
producer), max_pool2d_with_indices, and the mem-efficient attention op with its additive mask."""
import numpy as np
import pytest

import juliavision_b200 as jv
from juliavision_b200 import _lib
from juliavision_b200.graph import loadgraph

from .conftest import relerr
from .test_graph_plan import _castgraph

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", [1, 7, 8, 1000, 4099, 1 << 20])
def test_to_copy_is_the_numpy_cast(ctx, n):
    rng = np.random.default_rng(n)
    a32 = np.float32(rng.standard_normal(n) * 100)
    a32[0] = 70000.0                                   # beyond fp16: rounds to inf, as convert does
    out16 = ctx.allocate(np.float16, n)
    jv.to_copy_(ctx, out16, ctx.toback(a32))
    with np.errstate(over="ignore"):
        assert np.array_equal(out16.to_host(), a32.astype(np.float16))
    a16 = np.float16(rng.standard_normal(n))
    out32 = ctx.allocate(np.float32, n)
    jv.to_copy_(ctx, out32, ctx.toback(a16))
    assert np.array_equal(out32.to_host(), a16.astype(np.float32))


def test_folded_cast_gives_the_same_values(ctx):
    """foldoutcasts is only allowed to be free: the graph with the narrowing cast folded into the layer
    norm returns bit-for-bit what the op-by-op graph returns."""
    rng = np.random.default_rng(1)
    g = _castgraph()
    w = {"g": np.float32(1 + 0.1 * rng.standard_normal(16)), "w": np.float16(rng.standard_normal((16, 8)) * 0.2),
         "b": np.float16(rng.standard_normal(8) * 0.2)}
    x = np.float32(rng.standard_normal((6, 16)))
    plain = jv.Model(ctx, g, w, rewrite=False)
    folded = jv.Model(ctx, g, w, rewrite=True)
    assert folded.rewrites["foldoutcasts"] == 1 and len(folded.graph.ops) == len(plain.graph.ops) - 1
    a, b = plain(x), folded(x)
    ctx.synchronize()
    for u, v in zip(a, b):
        assert u.dtype == v.dtype and np.array_equal(u.to_host(), v.to_host())
    assert a[1].dtype == np.float32                    # the widening cast survived


def test_maxpool_and_masked_attention_ops(ctx, ora):
    """max_pool2d_with_indices (tuple result, element 0) and _scaled_dot_product_efficient_attention
    with its fourth input, the additive mask, through the op loop."""
    B, H, L, E = 2, 2, 64, 16
    g = loadgraph({
        "name": "ops", "symbols": [], "inputs": ["img", "q", "k", "v", "mask"], "outputs": ["p0", "a0"],
        "buffers": [
            {"id": "img", "kind": "external", "shape": [1, 8, 12, 16], "dtype": "float16"},
            {"id": "q", "kind": "external", "shape": [B, H, L, E], "dtype": "float16"},
            {"id": "k", "kind": "external", "shape": [B, H, L, E], "dtype": "float16"},
            {"id": "v", "kind": "external", "shape": [B, H, L, E], "dtype": "float16"},
            {"id": "mask", "kind": "external", "shape": [B, 1, L, L], "dtype": "float16"},
            {"id": "p", "kind": "transient", "shape": [], "dtype": "float16", "live": [1, 1],
             "shapes": [[1, 8, 6, 8], [1, 8, 6, 8]], "dtypes": ["float16", None]},
            {"id": "p0", "kind": "view", "shape": [1, 8, 6, 8], "dtype": "float16", "of": "p", "op": "getitem", "attrs": {"arg1": 0}},
            {"id": "a", "kind": "transient", "shape": [], "dtype": "float16", "live": [2, 2],
             "shapes": [[B, H, L, E], None, None, None], "dtypes": ["float16", None, None, None]},
            {"id": "a0", "kind": "view", "shape": [B, H, L, E], "dtype": "float16", "of": "a", "op": "getitem", "attrs": {"arg1": 0}},
        ],
        "ops": [
            {"id": "o1", "aten": "max_pool2d_with_indices.default", "in": ["img"], "out": "p", "attrs": {"arg1": [2, 2], "arg2": [2, 2]}},
            {"id": "o2", "aten": "_scaled_dot_product_efficient_attention.default", "in": ["q", "k", "v", "mask"], "out": "a",
             "attrs": {"scale": 0.25}},
        ]})
    rng = np.random.default_rng(2)
    img = np.float16(rng.standard_normal((1, 8, 12, 16)))
    q, k, v = (np.float16(rng.standard_normal((B, H, L, E))) for _ in range(3))
    mask = np.float16(rng.standard_normal((B, 1, L, L)))
    mask[rng.random(mask.shape) < 0.25] = -np.inf
    m = jv.Model(ctx, g, {})
    p0, a0 = m(img, q, k, v, mask)
    ctx.synchronize()
    assert np.array_equal(p0.to_host(), ora.maxpool2d(img, (2, 2), (2, 2)))
    ref = ora.attention_ref(q, k, v, 0.25, bias=mask)
    assert relerr(a0.to_host(), ref) < 5e-3


def test_folded_widening_cast_gives_the_same_values(ctx):
    """foldincasts: the layer norm reading fp16 directly sees the same values (fp16 -> fp32 is exact) and
    accumulates in fp32 as before; its fp16 and fp32 kernels deal elements to lanes differently, so the
    sums may differ in the last bit and nothing more."""
    from .test_graph_plan import _widegraph
    rng = np.random.default_rng(3)
    g = _widegraph()
    w = {"g": np.float16(1 + 0.1 * rng.standard_normal(16))}
    a, b = (np.float16(rng.standard_normal((6, 16))) for _ in range(2))
    plain, folded = jv.Model(ctx, g, w, rewrite=False), jv.Model(ctx, g, w, rewrite=True)
    assert folded.rewrites["foldincasts"] == 1
    u, v = plain(a, b), folded(a, b)
    ctx.synchronize()
    for x, y in zip(u, v):
        assert x.dtype == y.dtype == np.float32
        assert np.max(np.abs(x.to_host() - y.to_host())) <= 4e-7 * max(1.0, float(np.max(np.abs(x.to_host()))))


def test_conv_bn_relu_graph_runs_as_one_convolution(ctx, ora):
    """hoistcasts + foldbatchnorm + foldrelu leave a single convolution whose GEMM store carries the bias
    and the relu; there is no batch-norm kernel here, so the graph only runs folded."""
    from .test_graph_plan import _convnet_graph
    rng = np.random.default_rng(4)
    w = {"conv.weight": np.float32(rng.standard_normal((4, 3, 3, 3)) * 0.2), "conv.bias": np.float16(rng.standard_normal(4) * 0.1),
         "bn.weight": np.float32(1 + 0.2 * rng.standard_normal(4)), "bn.bias": np.float32(0.1 * rng.standard_normal(4)),
         "bn.mean": np.float32(0.1 * rng.standard_normal(4)), "bn.var": np.float32(0.5 + rng.random(4))}
    x = np.float16(rng.standard_normal((2, 3, 8, 8)))
    m = jv.Model(ctx, _convnet_graph(), w)
    assert m.rewrites["foldbatchnorm"] == 1 and m.rewrites["foldrelu"] == 1 and m.rewrites["hoistcasts"] == 1
    assert [o.aten for o in m.graph.ops] == ["convolution.default"]
    (y,) = m(x)
    ctx.synchronize()
    c = ora.conv2d(x, w["conv.weight"].astype(np.float16), w["conv.bias"], padding=(1, 1)).astype(np.float32)
    s = w["bn.weight"] / np.sqrt(w["bn.var"] + np.float32(1e-5))
    want = np.maximum(c * s[None, :, None, None] + (w["bn.bias"] - w["bn.mean"] * s)[None, :, None, None], 0)
    assert relerr(y.to_host(), want) < 2e-2


def test_memory_a_graph_uses_is_not_handed_to_anyone_else(ctx):
    """A recorded graph bakes in the addresses of the workspace block and of any pool block handed out
    while capturing.  Growing the workspace afterwards retires the old block, and freeing a capture-time
    temporary returns it; neither may reach a later allocation while the graph lives, or a replay would
    scribble over someone else's array.  Split matrix-vector products are used because they leave
    partial sums in the workspace on every call."""
    import ctypes as C
    with jv.Ctx(0) as c:
        rng = np.random.default_rng(12)
        M, K = 256, 4096
        Wt = c.toback(np.float16(rng.standard_normal((K, M)) * 0.05))
        xv = c.toback(np.float16(rng.standard_normal((1, K))))
        out = c.allocate(np.float16, M, 1)
        temps = []

        def step():
            c.ws.reset()
            temps.append(c.allocate(np.float16, 1 << 18))     # a pool block taken while capturing
            jv.matmul_(c, out, Wt, xv, None)

        step()                       # warm: pool and workspace have what the capture will need
        temps.clear()
        c.synchronize()
        g = c.capture(step)
        ws_cap = c.ws.stats()[1]
        temps.clear()                # the capture-time block is freed by its owner ...
        c.ws.reset()
        c.ws.scratch(np.uint8, 4 * ws_cap)   # ... and the workspace grows, retiring the block the graph uses
        c.ws.reset()
        # Everything allocated now must be disjoint from what the graph writes: fill a lot of memory of
        # the same size classes with a pattern, replay, and look at the pattern again.
        guards = [c.allocate(np.uint8, n) for n in (1 << 19, ws_cap, 1 << 19, ws_cap, 1 << 20)]
        for a in guards:
            c.fill_bytes(a, 0x5A)
        c.fill_bytes(out, 0)
        for _ in range(3):
            g.replay()
        c.synchronize()
        want = (np.float32(xv.to_host()) @ np.float32(Wt.to_host())).ravel()
        assert relerr(out.to_host().ravel(), want) < 1e-2
        for a in guards:
            assert np.all(a.to_host() == 0x5A), "a replay wrote into memory allocated after the capture"
        del g                        # destroying the graph puts its blocks back into circulation
        use, res = C.c_size_t(), C.c_size_t()
        _lib.check(_lib.lib().b200_pool_stats(c.handle, C.byref(use), C.byref(res)))
        again = c.allocate(np.uint8, ws_cap)
        use2, res2 = C.c_size_t(), C.c_size_t()
        _lib.check(_lib.lib().b200_pool_stats(c.handle, C.byref(use2), C.byref(res2)))
        assert res2.value == res.value, "the released workspace block was not reused"


def test_a_wait_that_cannot_be_satisfied_runs_out_and_the_context_carries_on(ctx):
    """Bounded waits: a one-warp kernel waits 2 ms on a barrier nothing arrives at.  It must return, the
    next sync must report the kernel status once, and the same context must then compute correctly."""
    import ctypes as C
    with jv.Ctx(0) as c:
        flag = c.allocate(np.int32, 1)
        c.fill_bytes(flag, 0)
        _lib.check(_lib.lib().b200_selftest_bounded_wait(c.handle, 2_000_000, flag.ptr))
        with pytest.raises(jv.B200Error) as e:
            c.synchronize()
        assert e.value.code == _lib.EKERNEL and "108" in str(e.value)
        assert int(flag.to_host()[0]) == 1
        c.synchronize()              # the status was cleared by the failing sync
        rng = np.random.default_rng(13)
        X = np.float16(rng.standard_normal((300, 256)) * 0.25)
        Wt = np.float16(rng.standard_normal((256, 512)) * 0.25)
        y = c.allocate(np.float16, 512, 300)
        jv.matmul_(c, y, c.toback(Wt), c.toback(X), None)
        c.synchronize()
        assert relerr(y.to_host(), np.float32(X) @ np.float32(Wt)) < 1e-2
