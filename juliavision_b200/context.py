"""Run context, device facts and device arrays — the host-side mirror of the reference's
`Ctx` / `caps` / `DeviceCaps` (context.jl:55-68,240-331), `Workspace` / `scratch!` / `reset!`
(workspace.jl:19-106) and `toback` (driver.jl:108-115) for the B200 backend.

Shapes follow the reference: column-major, shape = reversed torch shape.  A numpy array in
torch (row-major) order is byte-identical to the reference's array of the reversed shape, so
`toback` takes torch-order numpy arrays and `Array` gives them back.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from math import prod
from typing import Optional, Sequence, Tuple

import numpy as np

from . import _lib
from ._lib import B200Error, check

_DT = {np.dtype(np.float16): _lib.F16, np.dtype(np.float32): _lib.F32}


def dtcode(dtype) -> int:
    try:
        return _DT[np.dtype(dtype)]
    except KeyError:
        raise B200Error(20, f"dtype {dtype} has no device form (fp16/fp32 only)")


@dataclass(frozen=True)
class DeviceCaps:
    """The reference's DeviceCaps(coopmat, tile, subgroup, coopmatsubgroup, sharedbudget,
    workgrouplimit, cores, warps) answered for a B200."""
    coopmat: bool
    tile: int
    subgroup: int
    coopmatsubgroup: int
    sharedbudget: int
    workgrouplimit: int
    cores: int
    warps: int
    cc: Tuple[int, int] = (10, 0)
    total_mem: int = 0


class DeviceArray:
    """A strided view of device memory: (root pointer + element offset, shape, strides).

    This is what `stridedroot` + `strides()` reduce a wrapper stack to in the reference
    (attention.jl:321-337): permutes, reshapes of dense arrays and slices are all views that
    never launch.  `shape`/`strides` are in the reference's order (fastest axis first),
    strides in elements.
    """

    def __init__(self, ctx: "Ctx", ptr: int, dtype, shape: Sequence[int], strides: Optional[Sequence[int]] = None,
                 owner=None):
        self.ctx = ctx
        self.ptr = int(ptr)
        self.dtype = np.dtype(dtype)
        self.shape = tuple(int(s) for s in shape)
        if strides is None:
            st, acc = [], 1
            for s in self.shape:
                st.append(acc)
                acc *= s
            strides = st
        self.strides = tuple(int(s) for s in strides)
        self.owner = owner  # keeps the pool block (or parent) alive

    # -- facts
    @property
    def ndim(self) -> int:
        return len(self.shape)

    @property
    def size(self) -> int:
        return prod(self.shape)

    @property
    def nbytes(self) -> int:
        return self.size * self.dtype.itemsize

    def isdense(self) -> bool:
        acc = 1
        for s, st in zip(self.shape, self.strides):
            if s != 1 and st != acc:
                return False
            acc *= s
        return True

    # -- views (no launch)
    def permute(self, perm: Sequence[int]) -> "DeviceArray":
        """PermutedDimsArray: axis i of the result is axis perm[i] of self (0-based)."""
        return DeviceArray(self.ctx, self.ptr, self.dtype, [self.shape[p] for p in perm],
                           [self.strides[p] for p in perm], owner=self)

    def reshape(self, *dims: int) -> "DeviceArray":
        dims = tuple(int(d) for d in (dims[0] if len(dims) == 1 and not isinstance(dims[0], int) else dims))
        if prod(dims) != self.size:
            raise ValueError(f"reshape {self.shape} -> {dims}")
        if not self.isdense():
            raise ValueError("reshape of a non-dense view needs a copy (contiguous)")
        return DeviceArray(self.ctx, self.ptr, self.dtype, dims, owner=self)

    def slice(self, axis: int, start: int, stop: int) -> "DeviceArray":
        if not (0 <= start <= stop <= self.shape[axis]):
            raise IndexError("slice out of range")
        shape = list(self.shape)
        shape[axis] = stop - start
        return DeviceArray(self.ctx, self.ptr + start * self.strides[axis] * self.dtype.itemsize, self.dtype, shape,
                           self.strides, owner=self)

    # -- host transfer
    def to_host(self) -> np.ndarray:
        """Dense copy to a numpy array in torch order (reversed shape)."""
        src = self if self.isdense() else self.ctx.contiguous(self)
        out = np.empty(tuple(reversed(src.shape)), dtype=self.dtype)
        if out.size:
            check(_lib.lib().b200_download(self.ctx.handle, out.ctypes.data_as(C.c_void_p), src.ptr, out.nbytes))
        return out

    def __repr__(self) -> str:
        return f"DeviceArray{self.shape}:{self.dtype} strides={self.strides}"


class _Block:
    """A pool block returned to the pool when the last array viewing it goes away."""

    def __init__(self, ctx: "Ctx", ptr: int):
        self.ctx, self.ptr = ctx, ptr

    def __del__(self):
        try:
            if self.ctx.handle:
                _lib.lib().b200_pool_free(self.ctx.handle, self.ptr)
        except Exception:
            pass


class Workspace:
    """Per-op bump scratch, reset at the top of each op (workspace.jl:19-106)."""

    def __init__(self, ctx: "Ctx"):
        self.ctx = ctx

    def reset(self) -> None:
        check(_lib.lib().b200_workspace_reset(self.ctx.handle))

    def scratch(self, dtype, *dims: int) -> DeviceArray:
        p = C.c_void_p()
        n = prod(dims) * np.dtype(dtype).itemsize
        check(_lib.lib().b200_workspace_scratch(self.ctx.handle, n, C.byref(p)))
        return DeviceArray(self.ctx, p.value or 0, dtype, dims, owner=self)

    def stats(self):
        used, cap, ret = C.c_size_t(), C.c_size_t(), C.c_int()
        check(_lib.lib().b200_workspace_stats(self.ctx.handle, C.byref(used), C.byref(cap), C.byref(ret)))
        return used.value, cap.value, ret.value


class Ctx:
    """One context per GPU: a stream, a cudaMalloc pool, a workspace and the device caps.

    Mirrors the fields the kernel entry points read from the reference's `Ctx`:
    `backend` (here: the library handle), `dev` (caps), `ws`, `clampattn`.
    """

    def __init__(self, device: int = 0, clampattn: bool = False):
        L = _lib.lib()
        h = C.c_void_p()
        check(L.b200_ctx_create(device, C.byref(h)))
        self.handle = h.value
        self.device = device
        self.clampattn = clampattn  # accepted for API parity; ragged tails need no clamping here
        c = _lib.Caps()
        check(L.b200_caps(self.handle, C.byref(c)))
        self.dev = DeviceCaps(bool(c.coopmat), c.tile, c.subgroup, c.coopmatsubgroup, c.sharedbudget,
                              c.workgrouplimit, c.cores, c.warps, (c.cc_major, c.cc_minor), c.total_mem)
        self.ws = Workspace(self)

    # -- lifetime
    def close(self) -> None:
        if getattr(self, "handle", None):
            h, self.handle = self.handle, None
            _lib.lib().b200_ctx_destroy(h)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    # -- memory
    def allocate(self, dtype, *dims: int) -> DeviceArray:
        """KernelAbstractions.allocate(backend, T, dims...) from the pool."""
        p = C.c_void_p()
        n = max(prod(dims), 1) * np.dtype(dtype).itemsize
        check(_lib.lib().b200_pool_alloc(self.handle, n, C.byref(p)))
        return DeviceArray(self, p.value, dtype, dims, owner=_Block(self, p.value))

    def toback(self, a: np.ndarray) -> DeviceArray:
        """Upload a torch-order numpy array; the device array has the reversed shape."""
        a = np.ascontiguousarray(a)
        d = self.allocate(a.dtype, *reversed(a.shape))
        if a.size:
            check(_lib.lib().b200_upload(self.handle, d.ptr, a.ctypes.data_as(C.c_void_p), a.nbytes))
        return d

    def copy(self, dst: DeviceArray, src: DeviceArray) -> None:
        """copyto!(dst, src) for two dense arrays of one size, asynchronous on the stream."""
        assert dst.isdense() and src.isdense() and dst.nbytes == src.nbytes
        check(_lib.lib().b200_copy(self.handle, dst.ptr, src.ptr, src.nbytes))

    def upload(self, dst: DeviceArray, host: np.ndarray) -> None:
        assert dst.isdense() and host.flags["C_CONTIGUOUS"] and dst.nbytes == host.nbytes
        check(_lib.lib().b200_upload(self.handle, dst.ptr, host.ctypes.data_as(C.c_void_p), host.nbytes))

    def fill_bytes(self, a: DeviceArray, byte: int) -> None:
        assert a.isdense()
        check(_lib.lib().b200_fill_bytes(self.handle, a.ptr, byte, a.nbytes))

    def contiguous(self, a: DeviceArray, out: Optional[DeviceArray] = None) -> DeviceArray:
        """Materialise a strided view densely (permutedims!/contiguous, execute.jl:257-277)."""
        if a.ndim > 4:
            raise B200Error(17, "contiguous: more than 4 axes")
        shape = list(a.shape) + [1] * (4 - a.ndim)
        strides = list(a.strides) + [0] * (4 - a.ndim)
        if out is None:
            out = self.allocate(a.dtype, *a.shape)
        check(_lib.lib().b200_permute4(self.handle, a.ptr, out.ptr, (C.c_int64 * 4)(*shape),
                                       (C.c_int64 * 4)(*strides), a.dtype.itemsize))
        return out

    # -- stream
    def synchronize(self) -> None:
        check(_lib.lib().b200_sync(self.handle))

    def launch_count(self) -> int:
        return _lib.lib().b200_launch_count(self.handle)

    def timer_start(self) -> None:
        check(_lib.lib().b200_timer_start(self.handle))

    def timer_stop(self) -> float:
        ms = C.c_float()
        check(_lib.lib().b200_timer_stop(self.handle, C.byref(ms)))
        return ms.value

    def scratch(self, dtype, *dims: int) -> DeviceArray:
        """scratch!(ctx, T, dims...) (workspace.jl:105)."""
        return self.ws.scratch(dtype, *dims)

    # -- capture / replay (the reference's Lava capture + replay!, SAM2Runner/src/sam2.jl:90-115)
    def capture(self, fn) -> "Graph":
        """Record everything `fn()` launches on this context into a graph.  Call `fn()` once
        eagerly beforehand so the pool and workspace need no new memory while recording."""
        check(_lib.lib().b200_graph_begin(self.handle))
        try:
            fn()
        except BaseException:
            g = C.c_void_p()
            _lib.lib().b200_graph_end(self.handle, C.byref(g))
            if g.value:
                _lib.lib().b200_graph_destroy(g)
            raise
        g = C.c_void_p()
        check(_lib.lib().b200_graph_end(self.handle, C.byref(g)))
        return Graph(self, g.value)


class Graph:
    def __init__(self, ctx: "Ctx", handle: int):
        self.ctx, self.handle = ctx, handle

    def replay(self) -> None:
        check(_lib.lib().b200_graph_launch(self.ctx.handle, self.handle))

    def __del__(self):
        try:
            if self.handle:
                _lib.lib().b200_graph_destroy(self.handle)
        except Exception:
            pass


def caps(ctx: Ctx) -> DeviceCaps:
    return ctx.dev
