"""Static buffer planning: every transient of a graph laid into one slab, reusing memory across
non-overlapping lifetimes (reference DNNKernels/src/plan.jl:28-331).  Pure host logic, unchanged in
substance; the offsets it produces index a pool block of the B200 context instead of a Lava buffer.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Set, Tuple

import numpy as np

from .graph import Buffer, Graph, evalshape

SHAPEONLY_VIEWS = ("view.default", "_unsafe_view.default", "unsqueeze.default", "squeeze.dims", "squeeze.dim")


def alignup(n: int, a: int = 256) -> int:
    """Round up to a 256-byte boundary (plan.jl:28-29)."""
    return (n + a - 1) // a * a


@dataclass
class Slab:
    offsets: Dict[str, int] = field(default_factory=dict)  # buffer id -> byte offset into the slab
    sizes: Dict[str, int] = field(default_factory=dict)    # buffer id -> bytes reserved there
    bytes: int = 0


def place(plan: Optional[Slab], slab, id: str, dtype, dims):
    """Storage for buffer `id` out of the plan, or None when the plan does not cover it or the request
    does not fit what was reserved (plan.jl:40-61). `slab` is a dense uint8 DeviceArray."""
    if plan is None or slab is None:
        return None
    off = plan.offsets.get(id)
    n = int(np.prod(dims, dtype=np.int64)) * np.dtype(dtype).itemsize
    if off is None or n > plan.sizes.get(id, 0):
        return None
    from .context import DeviceArray
    return DeviceArray(slab.ctx, slab.ptr + off, dtype, dims, owner=slab)   # slabview (execute.jl:173-179)


def escaping(graph: Graph) -> Set[str]:
    """Buffer ids that outlive the graph: its outputs and what they are views of (plan.jl:63-79)."""
    esc: Set[str] = set()

    def mark(i):
        if i in esc:
            return
        esc.add(i)
        b = graph.buffers.get(i)
        if b is not None and b.of:
            mark(b.of)

    for o in graph.outputs:
        mark(o)
    return esc


def rootbuffer(graph: Graph, id: str, depth: int = 0) -> str:
    """Follow a view chain to the buffer that owns the storage (plan.jl:150-160)."""
    if depth > 64:
        return id
    b = graph.buffers.get(id)
    return id if b is None or not b.of else rootbuffer(graph, b.of, depth + 1)


def lifetimes(graph: Graph) -> Dict[str, Tuple[int, int]]:
    """(first_op, last_op), 1-based, computed from this runtime's own execution rather than from
    `Buffer.live`: views are resolved when read, so a parent stays live as long as any view of it is
    read (plan.jl:82-148; no value stays lazy in this runtime, so the fusion walk is empty)."""
    first: Dict[str, int] = {}
    last: Dict[str, int] = {}
    for i, o in enumerate(graph.ops, start=1):
        r = rootbuffer(graph, o.out)
        first[r] = min(first.get(r, i), i)
        last[r] = max(last.get(r, i), i)
        for inp in o.ins:
            ri = rootbuffer(graph, inp)
            last[ri] = max(last.get(ri, i), i)
    return {k: (first.get(k, 0), last.get(k, 0)) for k in last}


def materialisedview(graph: Graph, b: Buffer) -> bool:
    """Whether reading view `b` forces a copy: a shape-only view of a permute (plan.jl:166-184)."""
    if b.kind != "view" or b.viewop not in SHAPEONLY_VIEWS:
        return False
    p = graph.buffers.get(b.of)
    return p is not None and p.viewop in ("permute.default", "transpose.int", "t.default")


def planslab(graph: Graph, dims: Optional[Dict[str, int]] = None) -> Slab:
    """Greedy by size, largest first, lowest non-conflicting offset (plan.jl:215-297)."""
    produced = {o.out for o in graph.ops}
    esc = escaping(graph)
    lt = lifetimes(graph)
    items: List[Tuple[str, int, int, int]] = []
    for id, b in graph.buffers.items():          # copies forced by `contiguous`
        if not materialisedview(graph, b) or id in esc or not b.shape:
            continue
        r = rootbuffer(graph, id)
        if r not in lt:
            continue
        n = alignup(int(np.prod(evalshape(b.shape, dims), dtype=np.int64)) * np.dtype(b.dtype).itemsize)
        items.append((id, n, lt[r][0], lt[r][1]))
    for id, b in graph.buffers.items():
        if b.kind != "transient" or id not in produced or id in esc or id not in lt:
            continue
        if not b.shape:                           # multi-output op: one slot per element, "<id>.<i>"
            shapes = b.attrs.get("shapes")
            if shapes is None:
                continue
            dts = b.attrs.get("dtypes")
            for i, s in enumerate(shapes):
                if not s or (dts is not None and dts[i] is None):
                    continue
                T = dts[i] if dts is not None else b.dtype
                n = alignup(int(np.prod(evalshape(s, dims), dtype=np.int64)) * np.dtype(T).itemsize)
                items.append((f"{id}.{i}", n, lt[id][0], lt[id][1]))
            continue
        n = alignup(int(np.prod(evalshape(b.shape, dims), dtype=np.int64)) * np.dtype(b.dtype).itemsize)
        items.append((id, n, lt[id][0], lt[id][1]))
    items.sort(key=lambda x: (-x[1], x[0]))

    placed: List[Tuple[int, int, int, int]] = []   # offset, bytes, live-from, live-to
    slab = Slab()
    for id, n, ls, le in items:
        off = 0
        while True:
            bumped = False
            for po, pn, pls, ple in placed:
                if not (le < pls or ls > ple) and not (off + n <= po or off >= po + pn):
                    off = po + pn                  # slide past and rescan
                    bumped = True
                    break
            if not bumped:
                break
        placed.append((off, n, ls, le))
        slab.offsets[id] = off
        slab.sizes[id] = n
        slab.bytes = max(slab.bytes, off + n)
    return slab


def checkslab(graph: Graph, dims, slab: Slab) -> Tuple[int, int]:
    """(planned, conflicts): no two buffers alive at the same time may share a byte (plan.jl:299-331)."""
    ids = list(slab.offsets)
    lt = lifetimes(graph)
    root = lambda i: i.rsplit(".", 1)[0] if "." in i and i.rsplit(".", 1)[1].isdigit() else i
    bad = 0
    for x in range(len(ids)):
        for y in range(x + 1, len(ids)):
            a, b = ids[x], ids[y]
            la, lb = lt.get(rootbuffer(graph, root(a))), lt.get(rootbuffer(graph, root(b)))
            if la is None or lb is None or la[1] < lb[0] or la[0] > lb[1]:
                continue
            oa, ob = slab.offsets[a], slab.offsets[b]
            if not (oa + slab.sizes[a] <= ob or oa >= ob + slab.sizes[b]):
                bad += 1
    return len(ids), bad


def liveness_bound(graph: Graph, dims, slab: Slab) -> int:
    """Peak of concurrently live planned bytes: the lower bound any layout must reach."""
    lt = lifetimes(graph)
    root = lambda i: i.rsplit(".", 1)[0] if "." in i and i.rsplit(".", 1)[1].isdigit() else i
    peak = 0
    for i in range(1, len(graph.ops) + 1):
        live = sum(n for id, n in slab.sizes.items()
                   if (l := lt.get(rootbuffer(graph, root(id)))) is not None and l[0] <= i <= l[1])
        peak = max(peak, live)
    return peak
