"""The allocation-free convolution entry point.

`b200_conv2d_f16_noalloc` serves hosts that cannot allocate device memory at call time (their
own allocator already owns the GPU, or their loop may not make device-synchronising calls such
as cudaMalloc): its scratch is a fixed array inside the library instead of the growing
workspace.  It must give what `b200_conv2d_f16` gives.  This file sorts last so that a run
stopping at the first failure has already run every other test; it also passes alone in a fresh
process, because it creates nothing but its own operands.
"""
import ctypes as C

import numpy as np
import pytest

import juliavision_b200 as jv
from juliavision_b200 import _lib

pytestmark = pytest.mark.gpu


def _conv(ctx, fn, x, w, b, geom, out):
    W, H, Cin, N, KW, KH, Cout, s, p = geom
    ctx.fill_bytes(out, 0xFF)
    ctx.ws.reset()
    rc = fn(ctx.handle, W, H, Cin, N, KW, KH, Cout, s, s, p, p, 1, 1, x.ptr, w.ptr, b.ptr, out.ptr, _lib.F16,
            _lib.EPI["relu"])
    return rc


@pytest.mark.parametrize("geom", [(48, 48, 7, 2, 5, 5, 48, 2, 2),      # CRS = 175: padded weight + im2col
                                  (64, 64, 8, 1, 3, 3, 32, 1, 1),       # CRS = 72: im2col only
                                  (32, 32, 24, 2, 1, 1, 40, 1, 0)])     # 1x1: no scratch at all
def test_matches_the_allocating_entry_point_twice_in_a_row(ctx, geom):
    W, H, Cin, N, KW, KH, Cout, s, p = geom
    L = _lib.lib()
    rng = np.random.default_rng(W * 31 + Cin)
    OW, OH = jv.convsize(W, KW, s, p, 1), jv.convsize(H, KH, s, p, 1)
    out_ref = ctx.allocate(np.float16, OW, OH, Cout, N)
    out_new = ctx.allocate(np.float16, OW, OH, Cout, N)
    for round_ in range(2):   # the second call finds the first call's bytes in the shared array
        x = ctx.toback(np.float16(rng.standard_normal((N, Cin, H, W)) * 0.5))
        w = ctx.toback(np.float16(rng.standard_normal((Cout, Cin, KH, KW)) * 0.1))
        b = ctx.toback(np.float16(rng.standard_normal(Cout) * 0.1))
        _lib.check(_conv(ctx, L.b200_conv2d_f16, x, w, b, geom, out_ref))
        _lib.check(_conv(ctx, L.b200_conv2d_f16_noalloc, x, w, b, geom, out_new))
        ctx.synchronize()
        ref, got = out_ref.to_host().astype(np.float64), out_new.to_host().astype(np.float64)
        assert np.all(np.isfinite(got)), f"round {round_}: unwritten output"
        assert np.max(np.abs(ref)) > 1e-3
        # same tolerance as the convolution parity tests (max|d|/max|ref| < 5e-3); in practice equal
        assert np.max(np.abs(got - ref)) / np.max(np.abs(ref)) < 5e-3, f"round {round_}"


def _stats(c):
    import ctypes as C
    L = _lib.lib()
    use, res = C.c_size_t(), C.c_size_t()
    _lib.check(L.b200_pool_stats(c.handle, C.byref(use), C.byref(res)))
    return (use.value, res.value) + c.ws.stats()


@pytest.mark.parametrize("geom", [(16, 16, 576, 1, 3, 3, 256, 1, 1),     # 256 pixels, 81 k-blocks: a GEMM the planner
                                  (32, 32, 512, 1, 3, 3, 2048, 1, 1),    # of the allocating entry point runs as stream-K,
                                  (16, 16, 1024, 1, 3, 3, 1024, 1, 1),   # with fp32 partial tiles in the workspace
                                  (48, 48, 7, 2, 5, 5, 48, 2, 2)])
def test_allocates_nothing_on_a_context_whose_pool_and_workspace_are_cold(ctx, geom):
    """The promise itself: on a context that has never grown its workspace, a call leaves the pool's
    reserved bytes and the workspace capacity exactly as they were, also for the few-pixels-many-channels
    shapes whose GEMM would otherwise take partial-tile scratch; and the values equal the allocating
    entry point's (run afterwards, on the shared context)."""
    W, H, Cin, N, KW, KH, Cout, s, p = geom
    L = _lib.lib()
    rng = np.random.default_rng(Cin + Cout)
    OW, OH = jv.convsize(W, KW, s, p, 1), jv.convsize(H, KH, s, p, 1)
    xh = np.float16(rng.standard_normal((N, Cin, H, W)) * 0.5)
    wh = np.float16(rng.standard_normal((Cout, Cin, KH, KW)) * 0.05)
    bh = np.float16(rng.standard_normal(Cout) * 0.1)
    with jv.Ctx(0) as cold:
        x, w, b = cold.toback(xh), cold.toback(wh), cold.toback(bh)
        out = cold.allocate(np.float16, OW, OH, Cout, N)
        cold.fill_bytes(out, 0xFF)
        cold.synchronize()
        before = _stats(cold)
        assert before[3] == 0, "the cold context already has a workspace"
        for _ in range(2):
            _lib.check(L.b200_conv2d_f16_noalloc(cold.handle, W, H, Cin, N, KW, KH, Cout, s, s, p, p, 1, 1, x.ptr, w.ptr,
                                                 b.ptr, out.ptr, _lib.F16, _lib.EPI["relu"]))
        cold.synchronize()
        assert _stats(cold) == before, "the call changed the pool or the workspace"
        got = out.to_host().astype(np.float64)
    x, w, b = ctx.toback(xh), ctx.toback(wh), ctx.toback(bh)
    out_ref = ctx.allocate(np.float16, OW, OH, Cout, N)
    _lib.check(_conv(ctx, L.b200_conv2d_f16, x, w, b, geom, out_ref))
    ctx.synchronize()
    ref = out_ref.to_host().astype(np.float64)
    assert np.all(np.isfinite(got))
    assert np.max(np.abs(got - ref)) / np.max(np.abs(ref)) < 5e-3


def test_rejects_what_does_not_fit(ctx):
    L = _lib.lib()
    # 2048x2048x3 image, 7x7 stride 1: the im2col matrix alone is 1.2 GB, far above 32 MiB
    d = ctx.allocate(np.float16, 8)
    rc = L.b200_conv2d_f16_noalloc(ctx.handle, 2048, 2048, 3, 1, 7, 7, 16, 1, 1, 3, 3, 1, 1, d.ptr, d.ptr, None, d.ptr,
                                   _lib.F16, 0)
    assert rc == _lib.ENOMEM
    msg = _lib.last_error()
    assert "needs" in msg and "b200_conv2d_f16" in msg
