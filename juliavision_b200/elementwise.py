"""Encoder glue ops on fp16 storage: add.Tensor, clamp.default, gelu.default
(reference ops.jl:186-197,323-335,1698-1702)."""
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
