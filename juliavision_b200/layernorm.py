"""layernorm! for the B200 backend (reference kernels/layernorm.jl:125-135)."""
from __future__ import annotations

from typing import Optional

import numpy as np

from . import _lib
from ._lib import B200Error, check
from .context import Ctx, DeviceArray, dtcode


def layernorm_(ctx: Ctx, out: DeviceArray, mean: DeviceArray, rstd: DeviceArray, a: DeviceArray,
               gamma: Optional[DeviceArray], beta: Optional[DeviceArray], C: int, eps: float) -> DeviceArray:
    """layernorm!(ctx, out, mean, rstd, a, γ, β, C, eps): `a` dense with the normalised axis
    fastest; `length(a) ÷ C` groups; mean/rstd fp32 per group."""
    if not (a.isdense() and out.isdense() and mean.isdense() and rstd.isdense()):
        raise B200Error(18, "layernorm!: operands must be dense")
    if a.size % C != 0 or out.size != a.size:
        raise B200Error(17, "layernorm!: length(a) is not a multiple of C")
    groups = a.size // C
    if mean.dtype != np.float32 or rstd.dtype != np.float32 or mean.size < groups or rstd.size < groups:
        raise B200Error(20, "layernorm!: mean/rstd must be fp32 (groups,)")
    for g in (gamma, beta):
        if g is not None and (g.dtype != a.dtype or g.size != C or not g.isdense()):
            raise B200Error(16, "layernorm!: gamma/beta must be dense (C,) in the input dtype")
    check(_lib.lib().b200_layernorm(ctx.handle, groups, C, a.ptr, dtcode(a.dtype), out.ptr, dtcode(out.dtype),
                                    mean.ptr, rstd.ptr, gamma.ptr if gamma is not None else None,
                                    beta.ptr if beta is not None else None, float(eps)))
    return out


def add_layernorm_(ctx: Ctx, out: DeviceArray, mean: DeviceArray, rstd: DeviceArray, x: DeviceArray, h: DeviceArray,
                   gamma: Optional[DeviceArray], beta: Optional[DeviceArray], C: int, eps: float,
                   clamp: Optional[tuple] = None) -> DeviceArray:
    """x .= clamp(x .+ h); layernorm!(out, mean, rstd, x, ...) as one launch (fp16). The same values
    as add.Tensor, clamp.default and native_layer_norm run one after another."""
    for a in (x, h, out):
        if not a.isdense() or a.dtype != np.float16 or a.size != x.size:
            raise B200Error(16, "add_layernorm!: x, h, out must be dense fp16 arrays of one size")
    groups = x.size // C
    lo, hi = clamp if clamp is not None else (0.0, 0.0)
    check(_lib.lib().b200_add_layernorm_f16(ctx.handle, groups, C, x.ptr, h.ptr, int(clamp is not None), float(lo),
                                            float(hi), out.ptr, mean.ptr, rstd.ptr,
                                            gamma.ptr if gamma is not None else None,
                                            beta.ptr if beta is not None else None, float(eps)))
    return out


def native_layer_norm(ctx: Ctx, a: DeviceArray, nshape, gamma=None, beta=None, eps: float = 1e-5, out_dtype=None):
    """The fast branch of runop!(native_layer_norm.default) (ops.jl:575-609): normalised dims are
    the leading ones; returns (out, mean, rstd)."""
    n = int(np.prod(nshape))
    out = ctx.allocate(out_dtype or a.dtype, *a.shape)
    groups = a.size // n
    mean = ctx.allocate(np.float32, groups)
    rstd = ctx.allocate(np.float32, groups)
    layernorm_(ctx, out, mean, rstd, a, gamma, beta, n, eps)
    return out, mean, rstd
