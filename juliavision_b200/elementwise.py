"""Encoder glue ops on fp16 storage: add.Tensor, clamp.default, gelu.default, max_pool2d
(reference ops.jl:186-197,323-335,1329-1343,1698-1702)."""
from __future__ import annotations

from . import _lib
from ._lib import B200Error, check
from .context import Ctx, DeviceArray


def _dense_same(*arrs):
    n = arrs[0].size
    for a in arrs:
        if not a.isdense() or a.size != n or a.dtype.itemsize != 2:
            raise B200Error(16, "elementwise: operands must be dense fp16 arrays of one length")
    return n


def add_(ctx: Ctx, out: DeviceArray, a: DeviceArray, b: DeviceArray) -> DeviceArray:
    check(_lib.lib().b200_add_f16(ctx.handle, a.ptr, b.ptr, out.ptr, _dense_same(out, a, b)))
    return out


def clamp_(ctx: Ctx, out: DeviceArray, a: DeviceArray, lo: float, hi: float) -> DeviceArray:
    check(_lib.lib().b200_clamp_f16(ctx.handle, a.ptr, out.ptr, _dense_same(out, a), float(lo), float(hi)))
    return out


def act_(ctx: Ctx, out: DeviceArray, a: DeviceArray, name: str) -> DeviceArray:
    check(_lib.lib().b200_act_f16(ctx.handle, a.ptr, out.ptr, _dense_same(out, a), _lib.EPI[name]))
    return out


def to_copy_(ctx: Ctx, out: DeviceArray, a: DeviceArray) -> DeviceArray:
    """_to_copy.default: out = convert(eltype(out), a) for dense fp16/fp32 arrays (ops.jl:342-358)."""
    from .context import dtcode
    if not (a.isdense() and out.isdense() and a.size == out.size):
        raise B200Error(16, "_to_copy: dense arrays of one length")
    check(_lib.lib().b200_cast(ctx.handle, a.ptr, dtcode(a.dtype), out.ptr, dtcode(out.dtype), a.size))
    return out


def maxpool2d_(ctx: Ctx, out: DeviceArray, x: DeviceArray, k, s, p=(0, 0)) -> DeviceArray:
    """maxpool2d!(ctx, out, x, k, s, p) (kernels/resample.jl:141): x is indexed (x, y, c, n) and out
    (ox, oy, c, n), each through its own strides, so a planar array and a permuted view of a
    channels-last one are both accepted without a copy."""
    import ctypes as C
    if x.ndim != 4 or out.ndim != 4 or x.dtype.itemsize != 2 or out.dtype != x.dtype:
        raise B200Error(16, "maxpool2d!: 4-D fp16 arrays")
    W, H, Cn, N = x.shape
    OW, OH = (W + 2 * p[0] - k[0]) // s[0] + 1, (H + 2 * p[1] - k[1]) // s[1] + 1
    if out.shape != (OW, OH, Cn, N):
        raise B200Error(17, f"maxpool2d!: out is {out.shape}, expected {(OW, OH, Cn, N)}")
    check(_lib.lib().b200_maxpool2d_f16(ctx.handle, W, H, Cn, N, x.ptr, (C.c_int64 * 4)(*x.strides), out.ptr,
                                        (C.c_int64 * 4)(*out.strides), k[0], k[1], s[0], s[1], p[0], p[1]))
    return out
