"""Pins the CPU oracle: against the committed golden fixtures (independent float64 numpy
restatement) and against every known-answer assertion the reference's own tests make for
this path (tolerances, special values, bit-equalities)."""
import os

import numpy as np

from .conftest import relerr

G = os.path.join(os.path.dirname(__file__), "golden")


def relrms(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.sqrt(np.sum((a - b) ** 2) / np.sum(b ** 2)))


# ---- activations: reference test/test_activation_width.jl:69-118
def test_erf_half_grid(ora):
    g = np.load(os.path.join(G, "activation.npz"))
    got = ora.erf(g["x"])
    assert got.dtype == np.float16
    assert relrms(got, g["erf"]) < 3e-4
    assert float(ora.erf(np.float16([-4]))[0]) < -0.999
    assert float(ora.erf(np.float16([4]))[0]) > 0.999


def test_gelu_exact_half_grid(ora):
    g = np.load(os.path.join(G, "activation.npz"))
    got = ora.act(g["x"], "gelu")
    assert relrms(got, g["gelu"]) < 1e-4
    assert float(ora.act(np.float16([-4]), "gelu")[0]) != 0.0  # the narrow evaluation returned 0
    m3 = float(ora.act(np.float16([-3]), "gelu")[0])
    assert abs(m3 - float(g["gelu"][np.where(g["x"] == np.float16(-3))[0][0]])) < 1e-4


def test_gelu_tanh_half_grid(ora):
    g = np.load(os.path.join(G, "activation.npz"))
    assert relrms(ora.act(g["x"], "gelu_tanh"), g["gelu_tanh"]) < 1e-4
    assert np.isfinite(ora.act(np.float16([64]), "gelu_tanh")[0])
    assert ora.act(np.float16([64]), "gelu_tanh")[0] == np.float16(64)
    assert ora.act(np.float16([-64]), "gelu_tanh")[0] == 0


def test_relu_epilogue(ora):
    assert ora.act(np.float16([-1.0]), "relu")[0] == np.float16(0)
    assert ora.act(np.float16([2.5]), "none")[0] == np.float16(2.5)


# ---- GEMM: golden + reference test/test_batchedmatmul.jl:43-69 (tolerance 1e-4*K vs float64)
def test_linear_golden(ora):
    g = np.load(os.path.join(G, "linear.npz"))
    for epi, key in (("none", "y_none"), ("gelu", "y_gelu"), ("relu", "y_relu")):
        got = ora.linear(g["X"], g["Wt"], g["b"], epi=epi)
        # fp32 vs float64 accumulation may flip the last fp16 bit on a handful of elements
        d = np.abs(got.astype(np.float64) - g[key].astype(np.float64))
        ulp = np.spacing(np.abs(g[key]).astype(np.float16)).astype(np.float64)
        assert np.all(d <= ulp), (epi, float(d.max()))
        assert np.mean(d == 0) > 0.99


def test_linear_fp32_vs_float64(ora):
    rng = np.random.default_rng(1)
    K = 320
    X = (rng.standard_normal((33, K))).astype(np.float16)
    Wt = (rng.standard_normal((K, 48))).astype(np.float16)
    got = ora.linear(X, Wt, None, out_dtype=np.float32)
    ref = ora.linear_f64(X, Wt, None)
    assert np.max(np.abs(got - ref)) < 1e-4 * K
    np.testing.assert_allclose(ref, X.astype(np.float64) @ Wt.astype(np.float64), rtol=0, atol=1e-9)


def test_bias_joins_the_accumulator(ora):
    # matmul.jl:219-233: the bias starts the fp32 chain (so a huge bias swallows tiny products)
    X = np.full((1, 4), 2.0 ** -12, dtype=np.float16)
    Wt = np.full((4, 1), 2.0 ** -12, dtype=np.float16)
    b = np.array([1024.0], dtype=np.float16)
    assert ora.linear(X, Wt, b, out_dtype=np.float32)[0, 0] == np.float32(1024.0)
    assert ora.linear(X, Wt, None, out_dtype=np.float32)[0, 0] == np.float32(4 * 2.0 ** -24)


def test_activation_on_rounded_value(ora):
    # matmul.jl:210-214: epi(T(acc)), not T(epi(acc))
    X = np.array([[1.0, 2.0 ** -11]], dtype=np.float16)
    Wt = np.array([[1.0], [1.0]], dtype=np.float16)
    got = ora.linear(X, Wt, None, epi="gelu")
    want = ora.act(np.float16([1.0]), "gelu")  # 1 + 2^-11 rounds to 1 in fp16 first
    assert got[0, 0] == want[0]


def test_bmm_matches_planes(ora):
    rng = np.random.default_rng(2)
    a = rng.standard_normal((3, 5, 7)).astype(np.float16)
    b = rng.standard_normal((3, 7, 4)).astype(np.float16)
    got = ora.bmm(a, b, out_dtype=np.float32)
    ref = np.einsum("bmk,bkn->bmn", a.astype(np.float64), b.astype(np.float64))
    assert np.max(np.abs(got - ref)) < 1e-4 * 7


# ---- attention: golden + reference test/test_flash.jl:13-24,142,204 and test_coopmat_attention.jl
def test_attention_golden(ora):
    g = np.load(os.path.join(G, "attention.npz"))
    ref = ora.attention_ref(g["q"], g["k"], g["v"], float(g["scale"]))
    assert relerr(ref, g["out"]) < 1e-6
    tp = ora.attention_threepass(g["q"], g["k"], g["v"], float(g["scale"]))
    assert relerr(tp, g["out"]) < 5e-3  # the fused-vs-reference gate of the reference's tests


def test_attention_reference_shapes(ora):
    rng = np.random.default_rng(3)
    for (E, L, H, B) in ((72, 64, 1, 1), (72, 128, 2, 1), (64, 128, 4, 1)):
        q, k, v = (np.float16(rng.standard_normal((B, H, L, E)) * 0.2) for _ in range(3))
        sc = 1 / np.sqrt(E)
        ref = ora.attention_ref(q, k, v, sc)
        assert np.max(np.abs(ref)) > 1e-3  # wrote something
        assert relerr(ora.attention_threepass(q, k, v, sc), ref) < 5e-3


def test_attention_strided_operands(ora):
    # heads interleaved inside a token row, as the projections leave them
    rng = np.random.default_rng(4)
    B, L, H, E = 1, 24, 3, 16
    buf = np.float16(rng.standard_normal((B, L, 3, H, E)) * 0.3)
    q, k, v = (buf[:, :, i].transpose(0, 2, 1, 3) for i in range(3))  # (B,H,L,E) strided views
    dense = [np.ascontiguousarray(t) for t in (q, k, v)]
    a = ora.attention_threepass(q, k, v, 0.25)
    b = ora.attention_threepass(*dense, 0.25)
    assert np.array_equal(a, b)


def test_to_le_is_permutedims(ora):
    # reference test/test_transposeLE.jl:24-65: bit-equal to permutedims(host, (2,1,3,4))
    rng = np.random.default_rng(5)
    a = rng.standard_normal((2, 3, 10, 8)).astype(np.float16)  # torch (B,H,L,E)
    assert np.array_equal(ora.to_le(a), a.transpose(0, 1, 3, 2))
    view = np.float16(rng.standard_normal((2, 10, 3, 8))).transpose(0, 2, 1, 3)
    assert np.array_equal(ora.to_le(view), view.transpose(0, 1, 3, 2))


# ---- layer norm: golden (the reference has no unit test; plans/perf-plan.md quotes 1.15e-7 vs fp64)
def test_layernorm_golden(ora):
    g = np.load(os.path.join(G, "layernorm.npz"))
    out, mean, rstd = ora.layernorm(g["a"], g["gamma"], g["beta"], float(g["eps"]), out_dtype=np.float32)
    assert np.max(np.abs(out - g["out"])) < 2e-6
    assert np.max(np.abs(mean - g["mean"])) < 1e-6
    assert relerr(rstd, g["rstd"]) < 1e-6
    out16, _, _ = ora.layernorm(g["a"], g["gamma"], g["beta"], float(g["eps"]))
    assert out16.dtype == np.float16
    assert np.array_equal(out16, out.astype(np.float16))


def test_layernorm_no_cancellation(ora):
    # variance about the mean (layernorm.jl:22-25): a mean far above the spread must not cancel
    a = (np.float32(1000.0) + np.float32(0.5) * np.sin(np.arange(64, dtype=np.float32))).reshape(1, 64)
    out, mean, rstd = ora.layernorm(a, eps=1e-5)
    a64 = a.astype(np.float64)
    ref = (a64 - a64.mean()) / np.sqrt(a64.var() + 1e-5)
    assert np.max(np.abs(out - ref)) < 1e-3


# ---- convolution: golden on the reference's deterministic CRS-padding case
def _conv_case():
    g = np.load(os.path.join(G, "conv.npz"))
    W, H, Cin, Cout, KW, KH, st, pd = (int(t) for t in g["geom"])
    x = np.float16(0.4 * np.sin(np.linspace(0, 9, W * H * Cin))).reshape(1, Cin, H, W)
    w = np.float16(0.3 * np.cos(np.linspace(0, 7, KW * KH * Cin * Cout))).reshape(Cout, Cin, KH, KW)
    return g, x, w, st, pd


def test_conv_golden_and_im2col(ora):
    g, x, w, st, pd = _conv_case()
    got = ora.conv2d(x, w, None, (st, st), (pd, pd), (1, 1), out_dtype=np.float32)
    assert relerr(got[0], g["out"]) < 1e-5
    # im2col + GEMM equals the direct form (reference test: rel < 5e-3; here both are fp32 chains)
    Cout, Cin, KH, KW = w.shape
    OH, OW = got.shape[2:]
    NPQ, CRS = OH * OW, KW * KH * Cin
    MP, CRSP = (NPQ + 15) // 16 * 16, (CRS + 15) // 16 * 16
    col = ora.im2col(x, KH, KW, (st, st), (pd, pd), (1, 1), MP, CRSP)      # (CRSP, MP)
    assert np.all(col[CRS:] == 0) and np.all(col[:, NPQ:] == 0)
    wmat = np.zeros((Cout, CRSP), np.float16)
    wmat[:, :CRS] = w.reshape(Cout, CRS)                                   # (Cout, CRS): CRS fastest
    y = ora.linear(wmat, col, None, out_dtype=np.float32)                  # (Cout, MP)
    assert relerr(y[:, :NPQ].reshape(Cout, OH, OW), got[0]) < 1e-5


def test_convsize(ora):
    assert ora.convsize(1024, 7, 4, 3, 1) == 256
    assert ora.convsize(3000, 3, 2, 1, 1) == 1500


def test_glue_ops(ora):
    a = np.float16([1.5, -2.0, 60000.0, 3.0])
    b = np.float16([0.25, 2.0, 60000.0, -1.0])
    assert np.array_equal(ora.add(a, b), (a.astype(np.float32) + b.astype(np.float32)).astype(np.float16))
    assert np.array_equal(ora.clamp(a, -1.0, 2.0), np.float16([1.5, -1.0, 2.0, 2.0]))


def test_attention_additive_bias_matches_a_float64_restatement(ora):
    """attn_scores adds the mask to the scaled score (attention.jl:55-59); attn_softmax turns a row with
    every key blocked into zeros (attention.jl:73-100).  Checked against plain numpy in float64."""
    rng = np.random.default_rng(0)
    B, H, Lq, Lk, E = 1, 2, 20, 30, 16
    q = np.float16(rng.standard_normal((B, H, Lq, E)))
    k = np.float16(rng.standard_normal((B, H, Lk, E)))
    v = np.float16(rng.standard_normal((B, H, Lk, E)))
    bias = np.float16(rng.standard_normal((1, 1, Lq, Lk)))
    bias[rng.random(bias.shape) < 0.3] = -np.inf
    bias[:, :, 5, :] = -np.inf
    s = np.einsum("bhqe,bhke->bhqk", q.astype(np.float64), k.astype(np.float64)) * 0.25 + bias.astype(np.float64)
    m = s.max(-1, keepdims=True)
    m[~np.isfinite(m)] = 0
    p = np.exp(s - m)
    den = p.sum(-1, keepdims=True)
    den[den == 0] = 1
    want = np.einsum("bhqk,bhke->bhqe", p / den, v.astype(np.float64))
    assert np.max(np.abs(ora.attention_ref(q, k, v, 0.25, bias=bias) - want)) < 1e-6
    tp = ora.attention_threepass(q, k, v, 0.25, bias=bias)
    assert np.max(np.abs(tp - want)) < 5e-3
    assert np.all(tp[:, :, 5] == 0)


def test_maxpool_oracle_matches_the_reference_loop(ora):
    """resample.jl:121-141 restated as explicit loops on a small case (padding, stride != window)."""
    rng = np.random.default_rng(1)
    x = np.float16(rng.standard_normal((2, 3, 7, 9)))
    k, s, p = (3, 2), (2, 1), (1, 0)
    got = ora.maxpool2d(x, k, s, p)
    N, Cn, H, W = x.shape
    OW, OH = (W + 2 * p[0] - k[0]) // s[0] + 1, (H + 2 * p[1] - k[1]) // s[1] + 1
    want = np.empty((N, Cn, OH, OW), np.float16)
    for n in range(N):
        for c in range(Cn):
            for oy in range(OH):
                for ox in range(OW):
                    acc = -np.inf
                    for ky in range(k[1]):
                        for kx in range(k[0]):
                            iy, ix = oy * s[1] - p[1] + ky, ox * s[0] - p[0] + kx
                            if 0 <= iy < H and 0 <= ix < W:
                                acc = max(acc, float(x[n, c, iy, ix]))
                    want[n, c, oy, ox] = acc
    assert np.array_equal(got, want)


def test_hiera_reference_window_round_trip():
    from oracle.hiera_ref import _partition, _unpartition
    x = np.arange(2 * 8 * 8 * 3, dtype=np.float32).reshape(2, 8, 8, 3)
    xw = _partition(x, 4)
    assert xw.shape == (8, 16, 3)
    assert np.array_equal(xw[1, 0], x[0, 0, 4])          # second window of the first row starts at column 4
    assert np.array_equal(_unpartition(xw, 4, 2, 8), x)


def test_grouped_conv_is_the_ungrouped_one_per_group(ora):
    """conv2d with GROUPS (conv.jl:26-51): output channel co reads its own group's inputs — so a grouped convolution
    equals the ungrouped one applied to each group's channel slices, bit for bit (same fma chain)."""
    rng = np.random.default_rng(0)
    x = np.float16(rng.standard_normal((2, 6, 9, 8)))
    w = np.float16(rng.standard_normal((8, 3, 3, 3)) * 0.3)
    b = np.float16(rng.standard_normal(8))
    got = ora.conv2d_grouped(x, w, b, (2, 1), (1, 1), (1, 1), groups=2, out_dtype=np.float32)
    ref = np.concatenate([ora.conv2d(x[:, :3], w[:4], b[:4], (2, 1), (1, 1), (1, 1), out_dtype=np.float32),
                          ora.conv2d(x[:, 3:], w[4:], b[4:], (2, 1), (1, 1), (1, 1), out_dtype=np.float32)], 1)
    assert np.array_equal(got, ref)


def _convtranspose_scatter(x, w, b, s, p, d, op, groups):
    """The scatter reading of a transposed convolution ("each input paints a kernel-sized patch") in float64: an
    independent statement of what the oracle's gather (conv.jl:147-190) must equal."""
    N, Cin, H, W = x.shape
    _, COG, KH, KW = w.shape
    OH = (H - 1) * s[0] - 2 * p[0] + d[0] * (KH - 1) + op[0] + 1
    OW = (W - 1) * s[1] - 2 * p[1] + d[1] * (KW - 1) + op[1] + 1
    out = np.zeros((N, COG * groups, OH, OW))
    CG = Cin // groups
    for n in range(N):
        for ci in range(Cin):
            g = ci // CG
            for iy in range(H):
                for ix in range(W):
                    for ky in range(KH):
                        for kx in range(KW):
                            oy, ox = iy * s[0] - p[0] + ky * d[0], ix * s[1] - p[1] + kx * d[1]
                            if 0 <= oy < OH and 0 <= ox < OW:
                                out[n, g * COG:(g + 1) * COG, oy, ox] += float(x[n, ci, iy, ix]) * w[ci, :, ky, kx].astype(np.float64)
    return out + b.astype(np.float64)[None, :, None, None]


def test_transposed_conv_gather_equals_the_scatter(ora):
    rng = np.random.default_rng(1)
    x = np.float16(rng.standard_normal((2, 4, 5, 6)))
    b = np.float16(rng.standard_normal(6))
    for s, p, d, op, groups in (((2, 2), (0, 0), (1, 1), (0, 0), 1), ((2, 3), (1, 0), (1, 2), (1, 1), 2),
                                ((1, 1), (1, 1), (1, 1), (0, 0), 1)):
        w = np.float16(rng.standard_normal((4, 6 // groups, 3, 2)) * 0.3)
        got = ora.convtranspose2d(x, w, b, s, p, d, op, groups, out_dtype=np.float32)
        ref = _convtranspose_scatter(x, w, b, s, p, d, op, groups)
        assert got.shape == ref.shape
        assert np.max(np.abs(got - ref)) < 1e-5
        assert ora.convtransposesize(5, 3, s[0], p[0], d[0], op[0]) == ref.shape[2]      # conv.jl:194
