"""sdpa / sdpaplan / sdpa! for the B200 backend (reference kernels/extern/attention.jl:712-834,
kernels/extern/flash.jl:1322-1484).

q, k, v are (E, L, H, B) views with any strides along L, H, B (E contiguous); out is dense
(E, Lq, H, B).  Non-causal.  `bias` is the additive mask of the mem-efficient variant, fp16 in the
graph's own (Lk, Lq, H, B) order with size-1 axes broadcasting (attention.jl:55-59); the reference
declines it on its fused path and runs three passes, here it is added inside the fused kernel.
"""
from __future__ import annotations

import ctypes as C
from math import sqrt
from typing import Optional

import numpy as np

from . import _lib
from ._lib import B200Error, check
from .context import Ctx, DeviceArray, dtcode
from .kernelplans import AttnScalarPlan, Decline, FlashTCPlan, TwoGemmPlan


def _s4(a: DeviceArray) -> "_lib.Strided4":
    s = _lib.Strided4()
    s.ptr = a.ptr
    for i in range(4):
        s.stride[i] = a.strides[i]
    return s


def sdpaplan(ctx: Ctx, q: DeviceArray, k: DeviceArray, v: DeviceArray, bias=None):
    """One decision before `out` exists: FlashTCPlan, AttnScalarPlan or Decline(reason)."""
    if any(a.dtype != np.float16 for a in (q, k, v)):
        return Decline("eltype")
    if any(a.ndim != 4 for a in (q, k, v)):
        return Decline("operands")
    E, Lq, H, B = q.shape
    Lk = k.shape[1]
    if k.shape != (E, Lk, H, B) or v.shape != (E, Lk, H, B):
        return Decline("extent")
    if bias is not None:
        if bias.dtype != np.float16:
            return Decline("eltype")
        if bias.ndim != 4 or any(have not in (1, want) for have, want in zip(bias.shape, (Lk, Lq, H, B))):
            return Decline("bias")   # not broadcastable to (Lk, Lq, H, B)
    arr = lambda a: (C.c_int64 * 4)(*a.strides)
    rc = _lib.lib().b200_attention_f16_supported(E, Lq, Lk, H, B, arr(q), arr(k), arr(v), 0)
    if rc == _lib.OK and all(a.ptr % 16 == 0 for a in (q, k, v)):
        return FlashTCPlan(EP=64 if E <= 64 else 128)
    if any(a.strides[0] != 1 and a.shape[0] != 1 for a in (q, k, v)):
        return Decline("wrapped")  # E must be contiguous; densify first (attention.jl:734-759)
    if _lib.lib().b200_attention_f16_route(E, Lq, Lk, H, B, arr(q), arr(k), arr(v)) == 1:
        return TwoGemmPlan(nbatch=H * B)
    if rc in (_lib.OK, 18, 21):
        return AttnScalarPlan(_lib.DECLINE.get(rc, "wrapped"))
    return Decline(_lib.DECLINE.get(rc, "extent"))


def sdpa_(ctx: Ctx, plan, out: Optional[DeviceArray], q, k, v, bias, scale: float) -> DeviceArray:
    """sdpa!(ctx, plan, out, q, k, v, bias, scale) (attention.jl:773-776)."""
    if isinstance(plan, Decline):
        raise B200Error(16, f"sdpa!: Decline(:{plan.reason}); there is no CPU path behind this entry point")
    E, Lq, H, B = q.shape
    Lk = k.shape[1]
    if out is None:
        # sdpaout: accum(eltype(q)) = fp32 when the caller gives no destination (attention.jl:761-765)
        out = ctx.allocate(np.float32, E, Lq, H, B)
    if out.shape != (E, Lq, H, B) or (E != 1 and out.strides[0] != 1):
        raise B200Error(17, "sdpa!: out must be an (E, Lq, H, B) array with E contiguous")
    # A dense out is the reference's contract; a strided view (e.g. token-major) folds the
    # permute copy that follows sdpa in the exported graphs into the store.
    qs, ks, vs, os_ = _s4(q), _s4(k), _s4(v), _s4(out)
    bs = None
    if bias is not None:
        bs = _s4(bias)
        for i in range(4):
            if bias.shape[i] == 1:
                bs.stride[i] = 0       # bidx: a size-1 axis broadcasts
    check(_lib.lib().b200_attention_f16_bias(ctx.handle, E, Lq, Lk, H, B, C.byref(qs), C.byref(ks), C.byref(vs),
                                             C.byref(bs) if bs is not None else None, C.byref(os_),
                                             dtcode(out.dtype), float(scale)))
    return out


def sdpa(ctx: Ctx, q, k, v, bias=None, scale: Optional[float] = None, out: Optional[DeviceArray] = None):
    """sdpa(ctx, q, k, v, bias, scale; out) (attention.jl:712-719)."""
    if scale is None:
        scale = 1.0 / sqrt(q.shape[0])
    return sdpa_(ctx, sdpaplan(ctx, q, k, v, bias), out, q, k, v, bias, scale)
