"""Helpers for the GPU parity tests: every call goes through the package's public API, i.e.
through the C ABI of libb200dnn.so."""
import numpy as np

import juliavision_b200 as jv


def describe(got, ref, tol):
    """A short account of where two arrays differ, for assertion messages."""
    got = np.asarray(got, np.float64)
    ref = np.asarray(ref, np.float64)
    bad = ~(np.abs(got - ref) <= tol * max(np.max(np.abs(ref)), 1e-30))
    bad |= ~np.isfinite(got)
    n = int(bad.sum())
    if n == 0:
        return "ok"
    idx = np.argwhere(bad)
    lo, hi = idx.min(0), idx.max(0)
    first = tuple(idx[0])
    return (f"{n}/{bad.size} bad ({100.0 * n / bad.size:.2f}%), nan={int(np.isnan(got).sum())}, "
            f"bbox {tuple(lo)}..{tuple(hi)}, first {first}: got {got[first]} ref {ref[first]}")


def linear_gpu(ctx, X, Wt, b=None, epi="identity", out_dtype=np.float16, poison=True):
    """Y[tokens,out] = epi(X @ Wt + b) through matmul!: A = Wt as (M,K), B = X as (K,N)."""
    A = ctx.toback(np.ascontiguousarray(Wt, dtype=np.float16))
    B = ctx.toback(np.ascontiguousarray(X, dtype=np.float16))
    bias = None if b is None else ctx.toback(np.ascontiguousarray(b, dtype=np.float16))
    out = ctx.allocate(out_dtype, Wt.shape[1], X.shape[0])
    if poison:
        ctx.fill_bytes(out, 0xFF)
    jv.matmul_(ctx, out, A, B, bias, epi=epi)
    ctx.synchronize()
    return out.to_host()


def qkv_views(ctx, q, k, v):
    """Upload torch (B,H,L,E) arrays (possibly strided numpy views of one buffer) and return
    DeviceArray views with the same strides."""
    outs = []
    for a in (q, k, v):
        base = a
        while base.base is not None and isinstance(base.base, np.ndarray):
            base = base.base
        d = ctx.toback(np.ascontiguousarray(base).reshape(-1))
        off = (a.__array_interface__["data"][0] - base.__array_interface__["data"][0])
        assert base.flags["C_CONTIGUOUS"] and off % a.itemsize == 0
        st = [s // a.itemsize for s in a.strides]
        outs.append(jv.DeviceArray(ctx, d.ptr + off, a.dtype, tuple(reversed(a.shape)), tuple(reversed(st)), owner=d))
    return outs


def attention_gpu(ctx, q, k, v, scale, out_dtype=np.float16, bias=None):
    """bias: torch-order (B|1, H|1, Lq|1, Lk|1) fp16 additive mask, uploaded as the (Lk,Lq,H,B) array."""
    dq, dk, dv = qkv_views(ctx, q, k, v)
    B, H, Lq, E = q.shape
    out = ctx.allocate(out_dtype, E, Lq, H, B)
    ctx.fill_bytes(out, 0xFF)
    db = None if bias is None else ctx.toback(np.ascontiguousarray(bias))
    plan = jv.sdpaplan(ctx, dq, dk, dv, db)
    jv.sdpa_(ctx, plan, out, dq, dk, dv, db, scale)
    ctx.synchronize()
    return out.to_host(), plan


def layernorm_gpu(ctx, a, gamma=None, beta=None, eps=1e-5, out_dtype=None):
    da = ctx.toback(a)
    C = a.shape[-1]
    groups = a.size // C
    out = ctx.allocate(out_dtype or a.dtype, *reversed(a.shape))
    mean = ctx.allocate(np.float32, groups)
    rstd = ctx.allocate(np.float32, groups)
    for t in (out, mean, rstd):
        ctx.fill_bytes(t, 0xFF)
    g = None if gamma is None else ctx.toback(np.asarray(gamma, dtype=a.dtype))
    b = None if beta is None else ctx.toback(np.asarray(beta, dtype=a.dtype))
    jv.layernorm_(ctx, out, mean, rstd, da, g, b, C, eps)
    ctx.synchronize()
    return out.to_host(), mean.to_host(), rstd.to_host()
