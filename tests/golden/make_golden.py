"""Generates tests/golden/*.npz: small seeded inputs with expected outputs from an independent
float64 numpy restatement of each op's published formula.

    python tests/golden/make_golden.py

Why not the reference itself: it is Julia on KernelAbstractions + an un-vendored GPU package and
cannot run where this repository is built, and its own tests draw unseeded random inputs, so it
ships no golden bytes.  What the reference's tests DO fix — deterministic input formulas, shapes
and tolerances — is reused here: the convolution case below takes its inputs and geometry from
test/test_convtranspose_gemm.jl:154-200, the activation grid from test/test_activation_width.jl:44,
the attention shapes/input scale from test/test_flash.jl:36-40.
"""
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def f16(a):
    return np.asarray(a, dtype=np.float64).astype(np.float16)


def erf64(t):
    a = np.abs(t)
    s = np.where(t < 0, -1.0, 1.0)
    u = 1 / (1 + 0.3275911 * a)
    return s * (1 - (((((1.061405429 * u - 1.453152027) * u) + 1.421413741) * u - 0.284496736) * u + 0.254829592)
                * u * np.exp(-a * a))


def gelu64(x):
    x = np.asarray(x, dtype=np.float64)
    return 0.5 * x * (1 + erf64(x / np.sqrt(2.0)))


def gelutanh64(x):
    x = np.asarray(x, dtype=np.float64)
    return 0.5 * x * (1 + np.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3)))


def main():
    rng = np.random.default_rng(20260101)

    # activations on the reference's dense fp16 grid
    xs = np.unique(np.concatenate([f16(np.arange(-8, 8.0001, 0.01)), f16([-4, -3, -2, -1, 0, 1, 2, 3, 4])]))
    x64 = xs.astype(np.float64)
    np.savez_compressed(os.path.join(HERE, "activation.npz"), x=xs, erf=erf64(x64), gelu=gelu64(x64),
                        gelu_tanh=gelutanh64(x64))

    # linear: Y = epi(f16(X Wt + b)); ragged extents on purpose
    X = f16(rng.standard_normal((37, 72)) * 0.05 * 8)
    Wt = f16(rng.standard_normal((72, 40)) * 0.05 * 8)
    b = f16(rng.standard_normal(40) * 0.05 * 8)
    acc = X.astype(np.float64) @ Wt.astype(np.float64) + b.astype(np.float64)
    y_none = f16(acc)
    y_gelu = f16(gelu64(y_none.astype(np.float64)))
    y_relu = np.maximum(y_none, np.float16(0))
    np.savez_compressed(os.path.join(HERE, "linear.npz"), X=X, Wt=Wt, b=b, acc=acc, y_none=y_none, y_gelu=y_gelu,
                        y_relu=y_relu)

    # attention: torch (B,H,L,E), inputs randn*0.2 as the reference's flash tests use
    B, H, Lq, Lk, E = 2, 2, 40, 50, 16
    q = f16(rng.standard_normal((B, H, Lq, E)) * 0.2 * 4)
    k = f16(rng.standard_normal((B, H, Lk, E)) * 0.2 * 4)
    v = f16(rng.standard_normal((B, H, Lk, E)) * 0.2 * 4)
    scale = 1 / np.sqrt(E)
    s = np.einsum("bhqe,bhke->bhqk", q.astype(np.float64), k.astype(np.float64)) * scale
    p = np.exp(s - s.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    o = np.einsum("bhqk,bhke->bhqe", p, v.astype(np.float64))
    np.savez_compressed(os.path.join(HERE, "attention.npz"), q=q, k=k, v=v, scale=np.float64(scale), out=o)

    # layer norm: (groups, C) with affine
    a = f16(rng.standard_normal((9, 48)) * 3 + 1.5)
    g = f16(1 + 0.1 * rng.standard_normal(48))
    be = f16(0.1 * rng.standard_normal(48))
    a64 = a.astype(np.float64)
    mu = a64.mean(-1, keepdims=True)
    var = ((a64 - mu) ** 2).mean(-1, keepdims=True)
    r = 1 / np.sqrt(var + 1e-5)
    y = (a64 - mu) * r * g.astype(np.float64) + be.astype(np.float64)
    np.savez_compressed(os.path.join(HERE, "layernorm.npz"), a=a, gamma=g, beta=be, eps=np.float64(1e-5), out=y,
                        mean=mu[:, 0], rstd=r[:, 0])

    # convolution: the reference's deterministic CRS-padding case (W,H,Cin,Cout,KW,KH,s,p) = (48,48,7,48,5,5,2,2)
    W, Hh, Cin, Cout, KW, KH, st, pd = 48, 48, 7, 48, 5, 5, 2, 2
    nx, nw = W * Hh * Cin, KW * KH * Cin * Cout
    x = f16(0.4 * np.sin(np.linspace(0, 9, nx))).reshape(1, Cin, Hh, W)       # torch (N,Cin,H,W)
    w = f16(0.3 * np.cos(np.linspace(0, 7, nw))).reshape(Cout, Cin, KH, KW)   # torch (Cout,Cin,KH,KW)
    OW = (W + 2 * pd - (KW - 1) - 1) // st + 1
    OH = (Hh + 2 * pd - (KH - 1) - 1) // st + 1
    xp = np.zeros((Cin, Hh + 2 * pd, W + 2 * pd))
    xp[:, pd:pd + Hh, pd:pd + W] = x[0].astype(np.float64)
    out = np.zeros((Cout, OH, OW))
    w64 = w.astype(np.float64)
    for oy in range(OH):
        for ox in range(OW):
            patch = xp[:, oy * st:oy * st + KH, ox * st:ox * st + KW]
            out[:, oy, ox] = np.tensordot(w64, patch, axes=([1, 2, 3], [0, 1, 2]))
    np.savez_compressed(os.path.join(HERE, "conv.npz"), geom=np.array([W, Hh, Cin, Cout, KW, KH, st, pd]),
                        out=out.astype(np.float32))
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
