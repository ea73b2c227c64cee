import os

import numpy as np
import pytest

from .conftest import relerr
from .gpu_helpers import describe, layernorm_gpu

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")


def test_golden(ctx):
    g = np.load(os.path.join(G, "layernorm.npz"))
    out, mean, rstd = layernorm_gpu(ctx, g["a"], g["gamma"], g["beta"], float(g["eps"]), out_dtype=np.float32)
    assert np.max(np.abs(out - g["out"])) < 5e-6
    assert np.max(np.abs(mean - g["mean"])) < 1e-6 and relerr(rstd, g["rstd"]) < 1e-6


@pytest.mark.parametrize("groups,C", [(1500, 1280), (4096, 112), (64, 144), (333, 576), (7, 100), (5, 4104),
                                      (3, 8200), (1, 8), (65536, 112), (999, 112), (1001, 64), (7, 56), (130, 128)])
@pytest.mark.parametrize("dt_in,dt_out", [(np.float16, np.float16), (np.float16, np.float32),
                                          (np.float32, np.float32), (np.float32, np.float16)])
def test_vs_oracle(ctx, ora, groups, C, dt_in, dt_out):
    if groups * C > 2_000_000 and dt_in != np.float16:
        pytest.skip("large case runs once")
    rng = np.random.default_rng(groups * 131 + C)
    a = (rng.standard_normal((groups, C)) * 2 + 0.5).astype(dt_in)
    gam = (1 + 0.1 * rng.standard_normal(C)).astype(dt_in)
    bet = (0.1 * rng.standard_normal(C)).astype(dt_in)
    for g, b in ((gam, bet), (None, None), (gam, None)):
        got, mean, rstd = layernorm_gpu(ctx, a, g, b, 1e-5, out_dtype=dt_out)
        ref, rmean, rrstd = ora.layernorm(a, g, b, 1e-5, out_dtype=dt_out)
        assert got.dtype == dt_out and got.shape == ref.shape
        # fp32 statistics in a different summation order: a few fp32 ulps, at most one output ulp
        tol = 1.5e-3 if dt_out == np.float16 else 2e-6
        assert np.all(np.isfinite(got)), describe(got, ref, tol)          # poison fully overwritten
        assert relerr(got, ref) < tol, describe(got, ref, tol)
        assert np.max(np.abs(mean - rmean)) < 1e-5 and relerr(rstd, rrstd) < 1e-5


def test_mean_dominates_variance(ctx, ora):
    a = (np.float32(1000.0) + np.float32(0.5) * np.sin(np.arange(4 * 256, dtype=np.float32))).reshape(4, 256)
    got, _, _ = layernorm_gpu(ctx, a, eps=1e-5)
    ref, _, _ = ora.layernorm(a, eps=1e-5)
    assert np.max(np.abs(got - ref)) < 2e-3


def test_empty_and_errors(ctx):
    import juliavision_b200 as jv
    a = ctx.allocate(np.float16, 16, 0)
    out = ctx.allocate(np.float16, 16, 0)
    m = ctx.allocate(np.float32, 1)
    jv.layernorm_(ctx, out, m, m, a, None, None, 16, 1e-5)  # zero groups: no launch, no error
    b = ctx.allocate(np.float16, 10, 3)
    with pytest.raises(jv.B200Error):
        jv.layernorm_(ctx, b, m, m, b, None, None, 7, 1e-5)  # 30 is not a multiple of 7
