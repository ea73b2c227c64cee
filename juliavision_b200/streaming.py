"""A recorded pass fed from host memory with its copies off the critical path.

The op entry points work on device arrays; a caller that streams inputs from the host (one sequence or image
batch per pass) would otherwise pay upload -> pass -> download in series.  `StreamedPass` overlaps them with the
context's copy lane (b200_copy_lane_* and events in the C ABI): while the compute lane replays pass i, the copy
lane uploads the input of pass i+1 and downloads the result of pass i-1.  Every pass still has its own input
copied up from pinned host memory and its own result copied down; only the waiting is gone.  New surface: the
reference uploads with `toback` and reads with `Array`, both blocking (driver.jl:108-115, execute.jl:529-538).
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import numpy as np

from . import _lib
from ._lib import check
from .context import Ctx, DeviceArray

LANE_COMPUTE, LANE_COPY = 0, 1


class Event:
    def __init__(self, ctx: Ctx):
        h = C.c_void_p()
        check(_lib.lib().b200_event_create(ctx.handle, C.byref(h)))
        self.ctx, self.handle = ctx, h.value

    def record(self, lane: int) -> None:
        check(_lib.lib().b200_event_record(self.ctx.handle, self.handle, lane))

    def wait_on(self, lane: int) -> None:
        """Make `lane` wait for the latest record of this event."""
        check(_lib.lib().b200_lane_wait_event(self.ctx.handle, lane, self.handle))

    def __del__(self):
        try:
            if self.handle:
                _lib.lib().b200_event_destroy(self.handle)
        except Exception:
            pass


class StreamedPass:
    """A pass that reads its input from the dense device array `xin` and leaves its result in `y`, given either as
    the callable that launches it (preferred) or as an already recorded graph.

    Two device staging buffers each way.  Given the callable, two graphs are recorded, one per staging pair, each
    with the copy staging_in[b] -> xin in front of the pass and y -> staging_out[b] behind it as nodes of the graph
    itself, so that a step is one graph launch on the compute lane.  For pass i (b = i mod 2):
      compute lane: wait uploaded[b], wait downloaded[b] (result buffer free); graph b; done[b]
      copy lane:    wait done[1-b] (pass i-1 has read its input); upload input i+1 -> staging_in[1-b]; uploaded[1-b]
                    wait done[b]; download staging_out[b] -> host; downloaded[b]
    The upload of pass i+1 is queued before the wait for pass i, so it runs under pass i.  Given a recorded graph
    instead, the two staging copies are separate copies around each replay (and the input buffer is free again as
    soon as the first of them has run: event taken[b]).
    """

    def __init__(self, ctx: Ctx, forward, xin: DeviceArray, y: DeviceArray):
        assert xin.isdense() and y.isdense()
        self.ctx, self.xin, self.y = ctx, xin, y
        self.sin = [ctx.allocate(np.uint8, xin.nbytes) for _ in range(2)]
        self.sout = [ctx.allocate(np.uint8, y.nbytes) for _ in range(2)]
        self.uploaded = [Event(ctx) for _ in range(2)]
        self.taken = [Event(ctx) for _ in range(2)]
        self.done = [Event(ctx) for _ in range(2)]
        self.downloaded = [Event(ctx) for _ in range(2)]
        if hasattr(forward, "replay"):
            self.graph, self.graphs = forward, None
        else:
            L, h = _lib.lib(), ctx.handle

            def staged(b):
                def go():
                    check(L.b200_copy(h, xin.ptr, self.sin[b].ptr, xin.nbytes))
                    forward()
                    check(L.b200_copy(h, self.sout[b].ptr, y.ptr, y.nbytes))
                return go

            self.graph, self.graphs = None, []
            for b in range(2):
                staged(b)()                 # once eagerly: sizes pool and workspace before the capture
                ctx.synchronize()
                self.graphs.append(ctx.capture(staged(b)))

    def run(self, host_in: Sequence[int], host_out: Sequence[int]) -> None:
        """One pass per entry: host_in[i] / host_out[i] are addresses of pinned host buffers of xin.nbytes /
        y.nbytes (they may repeat).  Returns with all work queued; `ctx.synchronize()` waits for it."""
        L, h = _lib.lib(), self.ctx.handle
        n = len(host_in)
        if n == 0:
            return
        check(L.b200_copy_lane_upload(h, self.sin[0].ptr, host_in[0], self.xin.nbytes))
        self.uploaded[0].record(LANE_COPY)
        for i in range(n):
            b = i & 1
            self.uploaded[b].wait_on(LANE_COMPUTE)
            if i >= 2:
                self.downloaded[b].wait_on(LANE_COMPUTE)
            if self.graphs is not None:
                self.graphs[b].replay()
                self.done[b].record(LANE_COMPUTE)
                free_in = self.done
            else:
                check(L.b200_copy(h, self.xin.ptr, self.sin[b].ptr, self.xin.nbytes))
                self.taken[b].record(LANE_COMPUTE)
                self.graph.replay()
                check(L.b200_copy(h, self.sout[b].ptr, self.y.ptr, self.y.nbytes))
                self.done[b].record(LANE_COMPUTE)
                free_in = self.taken
            if i + 1 < n:
                if i >= 1:
                    free_in[1 - b].wait_on(LANE_COPY)
                check(L.b200_copy_lane_upload(h, self.sin[1 - b].ptr, host_in[i + 1], self.xin.nbytes))
                self.uploaded[1 - b].record(LANE_COPY)
            self.done[b].wait_on(LANE_COPY)
            check(L.b200_copy_lane_download(h, host_out[i], self.sout[b].ptr, self.y.nbytes))
            self.downloaded[b].record(LANE_COPY)
