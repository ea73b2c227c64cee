import os

import numpy as np
import pytest

import juliavision_b200 as jv

from .conftest import relerr
from .gpu_helpers import describe, linear_gpu

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")
TOL = 1e-2  # max relative error on fp16 outputs against the fp32-accumulated oracle


def test_golden(ctx):
    g = np.load(os.path.join(G, "linear.npz"))
    for epi, key in (("identity", "y_none"), ("gelu", "y_gelu"), ("relu", "y_relu")):
        got = linear_gpu(ctx, g["X"], g["Wt"], g["b"], epi=epi)
        assert got.shape == g[key].shape
        assert relerr(got, g[key]) < 2e-3, (epi, describe(got, g[key], 2e-3))


def _case(rng, tokens, out, K, scale=0.05):
    X = (rng.standard_normal((tokens, K)) * scale).astype(np.float16)
    Wt = (rng.standard_normal((K, out)) * scale).astype(np.float16)
    b = (rng.standard_normal(out) * scale).astype(np.float16)
    return X, Wt, b


# (tokens, out features, K): aligned, ragged tokens, ragged features, ragged K, tiny, one tile each way
SHAPES = [(256, 256, 128), (128, 64, 64), (1500, 1280, 1280), (100, 1000, 768), (37, 40, 72), (300, 3072, 768),
          (129, 264, 200), (1, 8, 8), (513, 520, 1032), (2000, 112, 448)]


@pytest.mark.parametrize("tokens,out,K", SHAPES)
def test_vs_oracle(ctx, ora, tokens, out, K):
    rng = np.random.default_rng(tokens * 7 + out * 3 + K)
    X, Wt, b = _case(rng, tokens, out, K, scale=0.25)
    plan = jv.mmplan(ctx, ctx.allocate(np.float16, out, tokens), ctx.toback(Wt), ctx.toback(X))
    assert isinstance(plan, jv.MMGemvPlan if tokens == 1 else jv.MMTilePlan), plan
    for epi, bias in (("identity", b), ("gelu", b), ("relu", None)):
        got = linear_gpu(ctx, X, Wt, bias, epi=epi)
        ref = ora.linear(X, Wt, bias, epi=epi if epi != "identity" else "none")
        assert got.shape == (tokens, out)
        assert relerr(got, ref) < TOL, (epi, describe(got, ref, TOL))
        # tighter: the only differences are fp32 summation order, i.e. a last-bit flip here and there
        d = np.abs(got.astype(np.float64) - ref.astype(np.float64))
        assert np.mean(d > 4 * np.spacing(np.abs(ref)).astype(np.float64) + 1e-6) < 1e-3


def test_config1_linear(ctx, ora):
    """BASELINE config 1: X 4096x768, W 3072x768, b 3072, N(0,1)*0.05, fp16 out."""
    rng = np.random.default_rng(20260101)
    X, Wt, b = _case(rng, 4096, 3072, 768)
    got = linear_gpu(ctx, X, Wt, b)
    ref = ora.linear(X, Wt, b)
    assert relerr(got, ref) < TOL, describe(got, ref, TOL)


def test_fp32_output(ctx, ora):
    rng = np.random.default_rng(5)
    X, Wt, b = _case(rng, 200, 136, 264, scale=0.25)
    got = linear_gpu(ctx, X, Wt, b, epi="gelu", out_dtype=np.float32)
    ref = ora.linear(X, Wt, b, epi="gelu", out_dtype=np.float32)
    assert got.dtype == np.float32
    assert relerr(got, ref) < 1e-4, describe(got, ref, 1e-4)


def test_unaligned_operands_take_the_scalar_kernel_bit_exact(ctx, ora):
    """lda = 37 cannot be a tensor-map stride: the scalar kernel runs mm2's arithmetic, so the
    result equals the oracle bit for bit."""
    rng = np.random.default_rng(6)
    X, Wt, b = _case(rng, 50, 37, 96, scale=0.25)
    plan = jv.mmplan(ctx, ctx.allocate(np.float16, 37, 50), ctx.toback(Wt), ctx.toback(X))
    assert isinstance(plan, jv.MMScalarPlan)
    got = linear_gpu(ctx, X, Wt, b, epi="relu")
    assert np.array_equal(got, ora.linear(X, Wt, b, epi="relu"))


def test_batched(ctx, ora):
    rng = np.random.default_rng(7)
    nb, m, k, n = 6, 70, 64, 136
    a = (rng.standard_normal((nb, m, k)) * 0.25).astype(np.float16)
    b = (rng.standard_normal((nb, k, n)) * 0.25).astype(np.float16)
    A, B = ctx.toback(b), ctx.toback(a)          # reference orientation: A = torch b (n,k,nb), B = torch a (k,m,nb)
    out = ctx.allocate(np.float16, n, m, nb)
    ctx.fill_bytes(out, 0xFF)
    jv.batchedmatmul_(ctx, out, A, B)
    ctx.synchronize()
    got = out.to_host()
    ref = ora.bmm(a, b)
    assert relerr(got, ref) < TOL, describe(got, ref, TOL)


@pytest.mark.parametrize("tile", ["320x2", "256x2s", "128x1"])
def test_batched_under_forced_schedules(ctx, ora, tile, monkeypatch):
    """Several planes through the wide tile, a split along K and single-CTA tiles: the plane index is the third
    coordinate of every tensor map and part of the tile index, whatever the schedule."""
    monkeypatch.setenv("B200_GEMM_TILE", tile)
    rng = np.random.default_rng(17)
    nb, m, k, n = 3, 300, 640, 712
    a = (rng.standard_normal((nb, m, k)) * 0.25).astype(np.float16)
    b = (rng.standard_normal((nb, k, n)) * 0.25).astype(np.float16)
    A, B = ctx.toback(b), ctx.toback(a)
    out = ctx.allocate(np.float16, n, m, nb)
    ctx.fill_bytes(out, 0xFF)
    jv.batchedmatmul_(ctx, out, A, B)
    ctx.synchronize()
    assert relerr(out.to_host(), ora.bmm(a, b)) < TOL


def test_padded_leading_dimensions(ctx, ora):
    """Views into wider buffers (ld > extent): the bytes outside the view stay untouched."""
    rng = np.random.default_rng(8)
    tokens, out, K = 130, 72, 80
    X, Wt, b = _case(rng, tokens, out, K, scale=0.25)
    big = ctx.allocate(np.float16, 96, tokens)
    ctx.fill_bytes(big, 0xFF)
    view = big.slice(0, 0, out)                   # (72, tokens) with ld 96
    jv.matmul_(ctx, view, ctx.toback(Wt), ctx.toback(X), ctx.toback(b))
    ctx.synchronize()
    host = big.to_host()                          # torch (tokens, 96)
    assert relerr(host[:, :out], ora.linear(X, Wt, b)) < TOL
    assert np.all(np.isnan(host[:, out:]))


def test_declines(ctx):
    a32 = ctx.allocate(np.float32, 64, 64)
    a16 = ctx.allocate(np.float16, 64, 64)
    assert jv.mmplan(ctx, a16, a32, a16) == jv.Decline("operands")       # test_batchedmatmul.jl:107-125
    assert jv.mmplan(ctx, a16, a16, ctx.allocate(np.float16, 32, 64)) == jv.Decline("extent")
    with pytest.raises(jv.B200Error):
        jv.matmul_(ctx, a16, a32, a16)
    empty = ctx.allocate(np.float16, 64, 0)
    assert jv.mmplan(ctx, empty, a16, empty) == jv.Decline("extent")


def test_linearity_at_full_size(ctx):
    """Size-independent property at the bench's size: W = [I;0] copies X, and f(X1+X2) = f(X1)+f(X2)
    for operands whose sums are exact in fp16."""
    tokens, K, out = 4096, 768, 3072
    rng = np.random.default_rng(9)
    X = rng.integers(-8, 9, (tokens, K)).astype(np.float16)
    Wt = np.zeros((K, out), np.float16)
    Wt[np.arange(K), np.arange(K)] = 1
    got = linear_gpu(ctx, X, Wt)
    assert np.array_equal(got[:, :K], X) and not got[:, K:].any()
    W2 = rng.integers(-2, 3, (K, out)).astype(np.float16)
    X2 = rng.integers(-2, 3, (tokens, K)).astype(np.float16)
    X1 = rng.integers(-2, 3, (tokens, K)).astype(np.float16)
    y1, y2, y12 = (linear_gpu(ctx, x, W2, out_dtype=np.float32) for x in (X1, X2, X1 + X2))
    assert np.array_equal(y1 + y2, y12)           # integer-valued: every partial sum is exact


@pytest.mark.parametrize("tile", ["256x2", "128x2", "256x1", "128x1", "64x1", "256x2s", "128x2s", "256x1s", "64x1s",
                                  "272x2", "320x2", "384x2", "432x2", "512x2"])
def test_every_tile_shape_and_schedule(ctx, ora, tile, monkeypatch):
    """The planner picks one (tile width, CTAs per tile, schedule) per call; the debugging override
    forces each of them in turn — CTA pairs, single CTAs, whole-tile and stream-K schedules (a
    trailing `s`), the wide single-accumulator tile at several widths (a width above 256) — on shapes
    with ragged tails, several tiles per worker and tiles cut across workers.  All must agree with the oracle like the planner's own choice does."""
    monkeypatch.setenv("B200_GEMM_TILE", tile)
    rng = np.random.default_rng(hash(tile) % 1000)
    for tokens, out, K in ((1500, 1280, 1280), (700, 5120, 640), (300, 1000, 4096), (4096, 3072, 768)):
        X, Wt, b = _case(rng, tokens, out, K, scale=0.25)
        got = linear_gpu(ctx, X, Wt, b, epi="gelu")
        ref = ora.linear(X, Wt, b, epi="gelu")
        assert relerr(got, ref) < TOL, (tile, tokens, out, K, describe(got, ref, TOL))


def test_streamk_is_deterministic(ctx, monkeypatch):
    monkeypatch.setenv("B200_GEMM_TILE", "256x2s")
    rng = np.random.default_rng(77)
    X, Wt, b = _case(rng, 1500, 1280, 5120, scale=0.25)
    a1 = linear_gpu(ctx, X, Wt, b)
    a2 = linear_gpu(ctx, X, Wt, b)
    assert np.array_equal(a1, a2)


@pytest.mark.parametrize("K", [768, 1280])
@pytest.mark.parametrize("out", [1000, 3072, 5120])
@pytest.mark.parametrize("tokens", [256, 4096, 65536])
def test_sweep_rows_sampled_and_row_shards(ctx, ora, tokens, out, K):
    """The scaling sweep's GEMM shapes (tokens 256..65536, out 1000/3072/5120 with 1000 ragged, K 768/1280).
    A sample of rows against the oracle, and the row split the sharding layer makes: each shard computed on
    its own equals the same rows of the whole product."""
    rng = np.random.default_rng(tokens + out + K)
    X = np.float16(rng.standard_normal((tokens, K), dtype=np.float32) * 0.05)
    Wt = np.float16(rng.standard_normal((K, out), dtype=np.float32) * 0.05)
    b = np.float16(rng.standard_normal(out, dtype=np.float32) * 0.05)
    got = linear_gpu(ctx, X, Wt, b)
    rows = np.sort(rng.choice(tokens, 48, replace=False))
    ref = ora.linear(np.ascontiguousarray(X[rows]), Wt, b)
    assert relerr(got[rows], ref) < TOL, describe(got[rows], ref, TOL)
    world = 8
    for rank in (0, 3, world - 1):
        r0, r1 = jv.shard_range(tokens, world, rank, align=256)
        if r1 > r0:
            part = linear_gpu(ctx, np.ascontiguousarray(X[r0:r1]), Wt, b)
            assert relerr(part, got[r0:r1]) < 1e-3
            assert np.mean(part != got[r0:r1]) < 1e-3      # summation order may differ where a tile was split along K


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("M,K", [(1280, 1280), (5120, 1280), (1280, 5120), (51865, 1280), (37, 50), (8, 4096), (1000, 3)])
def test_gemv_one_token(ctx, ora, dtype, M, K):
    """The one-token case (MMGemvPlan, matmul.jl:103-137): fp32 operands as in the reference and fp16
    ones; bias and activation in the store; compared with the oracle's fp32-accumulated product."""
    rng = np.random.default_rng(M + K)
    Wt = (rng.standard_normal((K, M)) * 0.05).astype(dtype)          # torch (in, out): column-major (M, K)
    x = (rng.standard_normal((1, K))).astype(dtype)
    b = (rng.standard_normal(M) * 0.05).astype(dtype)
    A, B, bias = ctx.toback(Wt), ctx.toback(x), ctx.toback(b)
    for epi, bb in (("identity", bias), ("gelu", bias), ("relu", None)):
        out = ctx.allocate(dtype, M, 1)
        ctx.fill_bytes(out, 0xFF)
        assert isinstance(jv.mmplan(ctx, out, A, B, bb), jv.MMGemvPlan)
        ctx.ws.reset()
        jv.matmul_(ctx, out, A, B, bb, epi=epi)
        ctx.synchronize()
        got = out.to_host()
        ctx.fill_bytes(out, 0xFF)
        ctx.ws.reset()
        jv.matmul_(ctx, out, A, B, bb, epi=epi)      # the K split's partial sums are added in a fixed order
        ctx.synchronize()
        assert np.array_equal(got.view(np.uint8), out.to_host().view(np.uint8))
        want = x.astype(np.float64) @ Wt.astype(np.float64) + (b.astype(np.float64) if bb is not None else 0)
        if dtype == np.float16:
            ref = ora.linear(x, Wt, b if bb is not None else None, epi=epi if epi != "identity" else "none")
            assert relerr(got, ref) < TOL, describe(got, ref, TOL)
        else:
            from scipy.special import erf
            ref = {"identity": want, "relu": np.maximum(want, 0), "gelu": 0.5 * want * (1 + erf(want / np.sqrt(2)))}[epi]
            assert relerr(got, ref) < 1e-4, describe(got, ref, 1e-4)


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("M0,lead,rows", [(3, 1000, 251), (1, 264, 1), (5, 4099, 4000), (0, 496, 496), (7, 249, 242)])
def test_gemv_rows_of_a_wider_matrix(ctx, dtype, M0, lead, rows):
    """A is rows M0 .. M0+rows of a (lead, K) matrix: the first element off a 16-byte boundary and a
    leading dimension of any parity, so every column starts at its own offset within an aligned vector.
    The rows outside the view hold huge values, which must not reach the result."""
    K = 300
    rng = np.random.default_rng(lead + rows)
    full = np.full((K, lead), 6.0e4, dtype)                         # torch (in, out): column-major (lead, K)
    full[:, M0:M0 + rows] = (rng.standard_normal((K, rows)) * 0.05).astype(dtype)
    x = rng.standard_normal((1, K)).astype(dtype)
    A = ctx.toback(full).slice(0, M0, M0 + rows)
    B = ctx.toback(x)
    out = ctx.allocate(np.float32, rows, 1)
    ctx.fill_bytes(out, 0xFF)
    assert isinstance(jv.mmplan(ctx, out, A, B, None), jv.MMGemvPlan)
    ctx.ws.reset()
    jv.matmul_(ctx, out, A, B, None)
    ctx.synchronize()
    got = out.to_host().reshape(-1)
    want = (x.astype(np.float64) @ full[:, M0:M0 + rows].astype(np.float64)).reshape(-1)
    assert np.all(np.isfinite(got))
    assert relerr(got, want) < 1e-4, describe(got, want, 1e-4)


def test_gemv_without_a_reduction_axis(ctx):
    """K = 0 through the C ABI: the sum is empty, the result is the bias (or zero)."""
    import ctypes as C
    from juliavision_b200 import _lib
    M = 300
    b = np.float16(np.random.default_rng(3).standard_normal(M))
    bias, out = ctx.toback(b), ctx.allocate(np.float16, M, 1)
    for bp, want in ((bias.ptr, b), (None, np.zeros(M, np.float16))):
        ctx.fill_bytes(out, 0xFF)
        rc = _lib.lib().b200_gemv(ctx.handle, M, 0, None, M, None, bp, _lib.F16, out.ptr, _lib.F16, 0)
        assert rc == _lib.OK
        ctx.synchronize()
        assert np.array_equal(out.to_host().reshape(-1), want)


def test_timeline_records_time_and_cycles(ctx):
    """b200_timeline: worker 0's events in nanoseconds and in SM cycles; their ratio is a plausible clock,
    the events are in order, every worker's exit is recorded, and nothing is written once it is off."""
    import ctypes as C
    from juliavision_b200 import _lib
    rng = np.random.default_rng(1)
    X = ctx.toback(np.float16(rng.standard_normal((2048, 1024), dtype=np.float32) * 0.05))
    W = ctx.toback(np.float16(rng.standard_normal((1024, 2048), dtype=np.float32) * 0.05))
    out = ctx.allocate(np.float16, 2048, 2048)
    tl = ctx.allocate(np.uint64, 256)
    ctx.fill_bytes(tl, 0)
    jv.matmul_(ctx, out, W, X, None)
    ctx.synchronize()
    _lib.check(_lib.lib().b200_timeline(ctx.handle, tl.ptr))
    jv.matmul_(ctx, out, W, X, None)
    ctx.synchronize()
    _lib.check(_lib.lib().b200_timeline(ctx.handle, None))
    t = tl.to_host().astype(np.int64)
    assert 0 < t[0] <= t[1] <= t[3] <= t[4] <= t[8] <= t[12] <= t[16]          # entry .. exit, in order
    ns, clk = t[16] - t[0], t[64 + 16] - t[64 + 0]
    assert ns > 0 and 500 < clk / ns * 1e3 < 2200                               # MHz
    exits = t[128:128 + 120]
    assert 1 <= np.count_nonzero(exits) <= 120 and np.all(exits[exits > 0] >= t[0])   # one per worker
    ctx.fill_bytes(tl, 0)
    jv.matmul_(ctx, out, W, X, None)
    ctx.synchronize()
    assert not tl.to_host().any()


def test_weight_operand_produced_by_the_previous_launch(ctx):
    """Launches overlap their predecessor's tail (programmatic dependent launch) and must not read an operand
    before the dependency wait.  Here the first product is the second one's A operand (as in a batched
    product of two activations) and changes every round, so a read that came too early would show."""
    rng = np.random.default_rng(31)
    M1, K1, N1 = 512, 256, 384          # Y1 (M1, N1) = W1 (M1, K1) . X1 (K1, N1)
    N2 = 300                            # Y2 (M1, N2) = Y1 (M1, N1) . X2 (N1, N2)
    W1 = ctx.toback(np.float16(rng.standard_normal((K1, M1)) * 0.1))      # torch (K, out)
    X2 = ctx.toback(np.float16(rng.standard_normal((N2, N1)) * 0.1))      # torch (tokens, K)
    Y1 = ctx.allocate(np.float16, M1, N1)
    Y2 = ctx.allocate(np.float16, M1, N2)
    for round_ in range(4):
        x1 = np.float16(rng.standard_normal((N1, K1)) * 0.1)
        X1 = ctx.toback(x1)
        jv.matmul_(ctx, Y1, W1, X1, None)
        jv.matmul_(ctx, Y2, Y1, X2, None)     # A = the output of the launch just before
        ctx.synchronize()
        y1 = Y1.to_host()                                        # torch (N1, M1)
        want = np.float32(X2.to_host()) @ np.float32(y1)         # (N2, N1) @ (N1, M1)
        assert relerr(Y2.to_host(), want) < 5e-3, f"round {round_}"
