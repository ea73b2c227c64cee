"""matmul!, mmplan, batchedmatmul! for the B200 backend (reference kernels/extern/matmul.jl).

`out[i,j] = epi(T(bias[i] + sum_k A[i,k] B[k,j]))` in the reference's reversed layout: A is
(M,K) with M contiguous (the dense weight), B is (K,N) with K contiguous (the activations).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np

from . import _lib
from ._lib import B200Error, check
from .context import Ctx, DeviceArray, dtcode
from .kernelplans import Decline, MMGemvPlan, MMScalarPlan, MMTilePlan


def _colmajor_2d(a: DeviceArray):
    """(ld) of a 2-D column-major view, or None when axis 0 is not unit-stride."""
    if a.ndim != 2 or (a.shape[0] != 1 and a.strides[0] != 1):
        return None
    ld = a.strides[1] if a.shape[1] != 1 else max(a.shape[0], 1)
    return ld if ld >= a.shape[0] else None


def _gemv_plan(out, A, B, bias):
    """mm_gemv_plan (matmul.jl:122-130): one column of B, dense operands of one float type, a bias of
    length M.  None when this is not a matrix-vector product; a Decline only for an odd bias."""
    if not (A.ndim == B.ndim == out.ndim == 2 and B.shape[1] == 1 and out.shape == (A.shape[0], 1)
            and B.shape[0] == A.shape[1] and min(A.shape) >= 1):
        return None
    if A.dtype != B.dtype or A.dtype not in (np.float16, np.float32):
        return None
    if out.dtype != np.float32 and out.dtype != A.dtype:
        return None
    if _colmajor_2d(A) is None or not B.isdense() or not out.isdense():
        return None
    if bias is not None and (bias.dtype != A.dtype or bias.size != A.shape[0] or not bias.isdense()):
        return Decline("bias") if A.dtype == np.float32 else None
    return MMGemvPlan()


def mmplan(ctx: Ctx, out: DeviceArray, A: DeviceArray, B: DeviceArray, bias: Optional[DeviceArray] = None):
    """Which path this shape takes (matmul.jl:91-95,103-130,172-179): MMTilePlan, MMGemvPlan,
    MMScalarPlan or Decline."""
    g = _gemv_plan(out, A, B, bias)
    if g is not None:
        return g
    if A.dtype != np.float16 or B.dtype != np.float16:
        return Decline("operands")
    if out.dtype not in (np.float16, np.float32):
        return Decline("eltype")
    if A.ndim != 2 or B.ndim != 2 or out.ndim != 2:
        return Decline("operands")
    M, K = A.shape
    K2, N = B.shape
    if K != K2 or out.shape != (M, N):
        return Decline("extent")
    lda, ldb, ldo = _colmajor_2d(A), _colmajor_2d(B), _colmajor_2d(out)
    if lda is None or ldb is None or ldo is None:
        return Decline("wrapped")
    if bias is not None and (bias.dtype != np.float16 or bias.size != M or not bias.isdense()):
        return Decline("bias")
    if min(M, N, K) < 1:
        return Decline("extent")
    rc = _lib.lib().b200_gemm_f16_supported(M, N, K, lda, ldb, ldo, dtcode(out.dtype))
    aligned = all(p % 16 == 0 for p in (A.ptr, B.ptr, out.ptr))
    if rc == _lib.OK and aligned:
        p = _lib.GemmPlan()
        check(_lib.lib().b200_gemm_f16_plan(ctx.handle, M, N, K, 1, C.byref(p)))
        return MMTilePlan(p.block_m, p.block_n, p.block_k, p.stages, p.tiles_m, p.tiles_n, p.ctas, p.smem_bytes)
    if rc in (_lib.OK, 18):
        return MMScalarPlan("wrapped")
    return Decline(_lib.DECLINE.get(rc, "extent"))


def matmul_(ctx: Ctx, out: DeviceArray, A: DeviceArray, B: DeviceArray, bias: Optional[DeviceArray] = None,
            epi: str = "identity") -> DeviceArray:
    """matmul!(ctx, out, A, B, bias; epi) (matmul.jl:78-79). An unsupported operand is an error:
    there is no CPU path behind this entry point."""
    plan = mmplan(ctx, out, A, B, bias)
    if isinstance(plan, Decline):
        raise B200Error(16, f"matmul!: Decline(:{plan.reason}) for A{A.shape}:{A.dtype} B{B.shape}:{B.dtype}")
    M, K = A.shape
    N = B.shape[1]
    if isinstance(plan, MMGemvPlan):
        check(_lib.lib().b200_gemv(ctx.handle, M, K, A.ptr, _colmajor_2d(A), B.ptr, bias.ptr if bias is not None else None,
                                   dtcode(A.dtype), out.ptr, dtcode(out.dtype), _lib.EPI[epi]))
        return out
    check(_lib.lib().b200_gemm_f16(ctx.handle, M, N, K, A.ptr, _colmajor_2d(A), B.ptr, _colmajor_2d(B),
                                   bias.ptr if bias is not None else None, out.ptr, _colmajor_2d(out),
                                   dtcode(out.dtype), _lib.EPI[epi], 1, 0, 0, 0))
    return out


def batchedmatmul_(ctx: Ctx, out: DeviceArray, A: DeviceArray, B: DeviceArray) -> DeviceArray:
    """batchedmatmul!(ctx, out, A, B) (matmul.jl:383-392): out[i,j,b] = sum_k A[i,k,b] B[k,j,b],
    all planes in one launch (the tile scheduler walks the batch axis)."""
    if not (A.ndim == B.ndim == out.ndim == 3 and A.shape[2] == B.shape[2] == out.shape[2]):
        raise B200Error(17, "batchedmatmul!: operands are not three 3-D arrays with a common batch extent")
    for a in (A, B, out):
        if a.shape[0] != 1 and a.strides[0] != 1:
            raise B200Error(18, "batchedmatmul!: Decline(:wrapped)")
    M, K, nb = A.shape
    N = B.shape[1]
    if B.shape[0] != K or out.shape[:2] != (M, N):
        raise B200Error(17, "batchedmatmul!: Decline(:extent)")
    check(_lib.lib().b200_gemm_f16(ctx.handle, M, N, K, A.ptr, A.strides[1], B.ptr, B.strides[1], None, out.ptr,
                                   out.strides[1], dtcode(out.dtype), 0, nb, A.strides[2], B.strides[2],
                                   out.strides[2]))
    return out
