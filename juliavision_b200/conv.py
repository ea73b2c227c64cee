"""convolution! lowered to the tensor-core GEMM (reference kernels/extern/conv.jl:100-145,
kernels/extern/conv_coopmat.jl:30-392).  x (W,H,Cin,N), w (KW,KH,Cin,Cout), out (OW,OH,Cout,N)."""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np

from . import _lib
from ._lib import B200Error, check
from .context import Ctx, DeviceArray, dtcode


def convsize(n: int, k: int, s: int, p: int, d: int) -> int:
    """ATen's output extent (conv.jl:309)."""
    return (n + 2 * p - d * (k - 1) - 1) // s + 1


def onebyone(w: DeviceArray, stride, padding, dilation, groups: int) -> bool:
    """The 1x1 case that is a plain GEMM (conv.jl:53-88)."""
    return (w.shape[0] == 1 and w.shape[1] == 1 and tuple(stride) == (1, 1) and tuple(padding) == (0, 0)
            and tuple(dilation) == (1, 1) and groups == 1)


def convolution_(ctx: Ctx, out: DeviceArray, x: DeviceArray, w: DeviceArray, bias: Optional[DeviceArray],
                 stride: Sequence[int], padding: Sequence[int], dilation: Sequence[int], groups: int = 1,
                 act: str = "identity") -> DeviceArray:
    """convolution!(ctx, out, x, w, bias, stride, padding, dilation, groups; act); stride etc. are
    (x, y) in the reference's reversed order."""
    if x.dtype != np.float16 or w.dtype != np.float16:
        raise B200Error(16, "convolution!: Decline(:operands)")
    if not (x.isdense() and w.isdense() and out.isdense()):
        raise B200Error(18, "convolution!: Decline(:wrapped)")
    W, H, Cin, N = x.shape
    KW, KH, Cin2, Cout = w.shape
    if groups < 1 or Cin2 * groups != Cin or Cout % groups:
        raise B200Error(17, "convolution!: channel mismatch")
    OW = convsize(W, KW, stride[0], padding[0], dilation[0])
    OH = convsize(H, KH, stride[1], padding[1], dilation[1])
    if out.shape != (OW, OH, Cout, N):
        raise B200Error(17, f"convolution!: out is {out.shape}, expected {(OW, OH, Cout, N)}")
    check(_lib.lib().b200_conv2d_grouped_f16(ctx.handle, W, H, Cin, N, KW, KH, Cout, stride[0], stride[1], padding[0],
                                             padding[1], dilation[0], dilation[1], groups, x.ptr, w.ptr,
                                             bias.ptr if bias is not None else None, out.ptr, dtcode(out.dtype),
                                             _lib.EPI[act]))
    return out


def convtransposesize(n: int, k: int, s: int, p: int, d: int, op: int) -> int:
    """Output extent of a transposed convolution (conv.jl:194)."""
    return (n - 1) * s - 2 * p + d * (k - 1) + op + 1


def shufflecase(w: DeviceArray, stride, padding, dilation, outpad, groups: int) -> bool:
    """The non-overlapping transposed convolution that is a GEMM plus a depth-to-space interleave (conv.jl:219-222)."""
    return (groups == 1 and tuple(dilation) == (1, 1) and tuple(padding) == (0, 0) and tuple(outpad) == (0, 0)
            and w.shape[0] == stride[0] and w.shape[1] == stride[1])


def convolutiontranspose_(ctx: Ctx, out: DeviceArray, x: DeviceArray, w: DeviceArray, bias: Optional[DeviceArray],
                          stride: Sequence[int], padding: Sequence[int], dilation: Sequence[int],
                          outpad: Sequence[int] = (0, 0), groups: int = 1) -> DeviceArray:
    """convolutiontranspose!(ctx, out, x, w, bias, stride, padding, dilation, outpad, groups) (conv.jl:247-290):
    x (W,H,Cin,N), w (KW,KH,Cout/groups,Cin), out (OW,OH,Cout,N); stride etc. are (x, y)."""
    if x.dtype != np.float16 or w.dtype != np.float16:
        raise B200Error(16, "convolutiontranspose!: Decline(:operands)")
    if not (x.isdense() and w.isdense() and out.isdense()):
        raise B200Error(18, "convolutiontranspose!: Decline(:wrapped)")
    W, H, Cin, N = x.shape
    KW, KH, COG, Cin2 = w.shape
    if groups < 1 or Cin2 != Cin or Cin % groups:
        raise B200Error(17, "convolutiontranspose!: channel mismatch")
    Cout = COG * groups
    OW = convtransposesize(W, KW, stride[0], padding[0], dilation[0], outpad[0])
    OH = convtransposesize(H, KH, stride[1], padding[1], dilation[1], outpad[1])
    if out.shape != (OW, OH, Cout, N):
        raise B200Error(17, f"convolutiontranspose!: out is {out.shape}, expected {(OW, OH, Cout, N)}")
    check(_lib.lib().b200_convtranspose2d_f16(ctx.handle, W, H, Cin, N, KW, KH, Cout, stride[0], stride[1], padding[0],
                                              padding[1], dilation[0], dilation[1], outpad[0], outpad[1], groups, x.ptr,
                                              w.ptr, bias.ptr if bias is not None else None, out.ptr, dtcode(out.dtype)))
    return out
