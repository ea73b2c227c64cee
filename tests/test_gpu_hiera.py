"""The hierarchical image encoder (BASELINE config "Hiera-B+-shaped") and the glue it adds:
max_pool2d, window-ordered tokens, pooled queries — checked against the raster-order oracle."""
import numpy as np
import pytest

import juliavision_b200 as jv
from juliavision_b200.hiera import Hiera, HieraConfig, init_weights

from .conftest import relerr
from .gpu_helpers import describe

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("layout", ["planar", "channels_last"])
@pytest.mark.parametrize("W,H,Cn,N,k,s,p", [(16, 12, 8, 2, (2, 2), (2, 2), (0, 0)), (17, 9, 24, 1, (3, 3), (2, 2), (1, 1)),
                                            (8, 8, 5, 3, (2, 2), (2, 2), (0, 0)), (32, 32, 64, 2, (3, 2), (1, 2), (1, 0))])
def test_maxpool2d_bit_exact(ctx, ora, layout, W, H, Cn, N, k, s, p):
    """resample.jl:121-141 on both layouts the callers use: the reference's planar (W,H,C,N) and a
    permuted view of channels-last tokens.  fp16 max is exact, so the results must match bit for bit."""
    rng = np.random.default_rng(W * H + Cn)
    x = np.float16(rng.standard_normal((N, Cn, H, W)))
    x[0, 0, 0, 0] = -np.inf
    want = ora.maxpool2d(x, k, s, p)
    OH, OW = want.shape[2], want.shape[3]
    if layout == "planar":
        dx = ctx.toback(x)                                    # (W,H,C,N)
        out = ctx.allocate(np.float16, OW, OH, Cn, N)
        jv.maxpool2d_(ctx, out, dx, k, s, p)
        got = out.to_host()
    else:
        dx = ctx.toback(np.ascontiguousarray(x.transpose(0, 2, 3, 1)))      # (C,W,H,N) tokens
        out = ctx.allocate(np.float16, Cn, OW, OH, N)
        jv.maxpool2d_(ctx, out.permute((1, 2, 0, 3)), dx.permute((1, 2, 0, 3)), k, s, p)
        got = out.to_host().transpose(0, 3, 1, 2)
    ctx.synchronize()
    assert np.array_equal(got, want)


SMALL = HieraConfig(image=64, embed=16, depths=(2, 2, 3, 2), head_dim=8, windows=(4, 4, 2, 2), global_blocks=(6,))
MID = HieraConfig(image=128, embed=112, depths=(1, 1, 2, 1), head_dim=56, windows=(8, 8, 4, 4), global_blocks=(3,))


@pytest.mark.parametrize("cfg,batch", [(SMALL, 2), (MID, 1)])
def test_hiera_matches_raster_oracle(ctx, cfg, batch):
    """Every block (plain, pooling with and without a change of window, global) against the oracle
    that partitions and un-partitions around each attention, prefix by prefix so an error is
    pinned to the block that made it."""
    from oracle.hiera_ref import oracle_forward
    w = init_weights(cfg)
    rng = np.random.default_rng(3)
    img = np.float16(rng.random((batch, cfg.in_ch, cfg.image, cfg.image)))
    model = Hiera(ctx, cfg, w, batch=batch)
    ctx.upload(model.image, img)
    y = model.forward()
    ctx.synchronize()
    got = y.to_host()                                         # torch (B, S, S, C)
    ref = oracle_forward(cfg, w, img)
    assert got.shape == ref.shape
    assert np.all(np.isfinite(got))
    assert relerr(got, ref) < 1e-2, describe(got, ref, 1e-2)


def test_hiera_graph_replay_equals_eager(ctx):
    cfg = SMALL
    w = init_weights(cfg)
    img = np.float16(np.random.default_rng(4).random((1, 3, cfg.image, cfg.image)))
    model = Hiera(ctx, cfg, w, batch=1)
    ctx.upload(model.image, img)
    eager = model.forward().to_host()
    g = model.capture()
    ctx.fill_bytes(model.y, 0)
    g.replay()
    ctx.synchronize()
    assert np.array_equal(model.y.to_host(), eager)


def test_hiera_full_size_properties(ctx):
    """Config at full size (1024x1024, 24 blocks): runs, finite, deterministic across two passes, and
    the two images of a batch of two identical inputs give identical outputs."""
    cfg = HieraConfig()
    model = Hiera(ctx, cfg, batch=2)
    one = np.float16(np.random.default_rng(5).random((1, 3, cfg.image, cfg.image)))
    ctx.upload(model.image, np.concatenate([one, one]))
    a = model.forward().to_host()
    b = model.forward().to_host()
    assert a.shape == (2, 32, 32, 896) and np.all(np.isfinite(a))
    assert np.array_equal(a, b)
    assert np.array_equal(a[0], a[1])
    assert float(np.std(a.astype(np.float32))) > 1e-3


def test_hiera_full_size_matches_raster_oracle(ctx):
    """The benchmarked configuration itself — 1024x1024x3 image, all 24 blocks (8x8 and 16x16 windows,
    three global blocks, three pooling blocks), 32x32x896 out — against the raster-order oracle on the
    same seeded image and weights.  The oracle's pass is 0.62 TFLOP of scalar fp32 work: tens of seconds
    on the host cores."""
    from oracle import oracle as ora
    from oracle.hiera_ref import oracle_forward
    ora.use_all_cores()
    cfg = HieraConfig()
    w = init_weights(cfg)
    img = np.float16(np.random.default_rng(6).random((1, cfg.in_ch, cfg.image, cfg.image)))
    model = Hiera(ctx, cfg, w, batch=1)
    ctx.upload(model.image, img)
    got = model.forward().to_host()
    ctx.synchronize()
    ref = oracle_forward(cfg, w, img)
    assert got.shape == ref.shape == (1, 32, 32, 896)
    assert np.all(np.isfinite(got))
    assert relerr(got, ref) < 1e-2, describe(got, ref, 1e-2)
