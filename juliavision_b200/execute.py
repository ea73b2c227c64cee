"""Graph execution over the B200 op entry points: `Model` (load-time rewrites + upload + slab plan)
and `execute_` (the op loop), for the ATen ops on the dense hot path and the glue around them.

Mirrors the reference's `Model` / `call` / `execute!` / `runop!` / `makeview` / `dest`
(DNNKernels/src/driver.jl:128-223, execute.jl:43-158,257-539, ops.jl:575-647,1114-1399) and two of
its rewrite passes: `hoistpermutes` (hoistcasts.jl:62-112 — a `t`/`permute` view of a weight becomes a
dense weight, which is what puts `addmm` on the tensor-core path) and the gelu half of `foldrelu`
(foldrelu.jl:81-124 — `gelu(addmm(...))` becomes `addmm` with `attrs["act"] = "gelu"`), and
`foldoutcasts` (foldoutcasts.jl:82-155 — a narrowing cast folded into the declared dtype of the layer
norm or clone that feeds it) and `foldincasts` (foldincasts.jl:82-124 — a widening cast in front of a
layer norm dropped, the layer norm reading the fp16 value).
An op outside this set raises, as `runop!`'s fallback does (execute.jl:541-542).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from math import sqrt
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np

from ._lib import B200Error
from .attention import sdpa
from .context import Ctx, DeviceArray
from .conv import convolution_, convolutiontranspose_, convsize, convtransposesize
from .elementwise import act_, add_, clamp_, maxpool2d_, to_copy_
from .graph import Buffer, Graph, Op, evalshape
from .layernorm import layernorm_
from .matmul import _colmajor_2d, batchedmatmul_, matmul_
from .plan import SHAPEONLY_VIEWS, Slab, place, planslab


# ------------------------------------------------------------------------------ rewrites
def _consumers(graph: Graph) -> Dict[str, List[Op]]:
    c: Dict[str, List[Op]] = {}
    for o in graph.ops:
        for i in o.ins:
            c.setdefault(i, []).append(o)
    return c


def hoistpermutes(graph: Graph, weights: Dict[str, np.ndarray]) -> int:
    """Make the `t(W)` operand of every addmm/mm a dense weight of its own (done once, on the host)."""
    n = 0
    for o in graph.ops:
        if o.aten not in ("addmm.default", "mm.default"):
            continue
        slot = 2 if o.aten == "addmm.default" else 1
        b = graph.buffers.get(o.ins[slot])
        if b is None or b.kind != "view" or b.viewop not in ("t.default", "permute.default", "transpose.int"):
            continue
        w = graph.buffers.get(b.of)
        if w is None or w.kind != "weight" or len(w.shape) != 2:
            continue
        if b.viewop == "permute.default" and list(b.attrs.get("arg1", [])) != [1, 0]:
            continue
        nid, nkey = w.id + "@t", w.key + "@t"
        if nid not in graph.buffers:
            graph.buffers[nid] = Buffer(nid, "weight", [w.shape[1], w.shape[0]], w.dtype, key=nkey)
            graph.order.append(nid)
            weights[nkey] = np.ascontiguousarray(weights[w.key].T)
        o.ins[slot] = nid
        n += 1
    return n


def foldgelu(graph: Graph) -> int:
    """gelu(addmm(...)) with no other reader of the addmm -> addmm with the activation in its store."""
    cons = _consumers(graph)
    viewed = {b.of for b in graph.buffers.values() if b.kind == "view"}
    producer = {o.out: o for o in graph.ops}
    keep, n = [], 0
    for o in graph.ops:
        src = producer.get(o.ins[0]) if o.aten == "gelu.default" and o.ins else None
        if (src is not None and src.aten == "addmm.default" and len(cons.get(src.out, [])) == 1
                and src.out not in viewed and src.out not in graph.outputs and "act" not in src.attrs):
            approx = str(o.attrs.get("approximate", o.attrs.get("arg1", "none")))
            src.attrs["act"] = "gelu_tanh" if approx == "tanh" else "gelu"
            src.out = o.out                      # the addmm now writes the gelu's buffer
            n += 1
            continue
        keep.append(o)
    graph.ops[:] = keep
    return n


OUTCAST_PRODUCERS = ("native_layer_norm.default", "clone.default")


def _viewchain(graph: Graph, id: str) -> List[str]:
    """Buffer ids from `id` down to the first non-view buffer, `id` included (foldoutcasts.jl:54-62)."""
    ids = [id]
    for _ in range(16):
        b = graph.buffers.get(ids[-1])
        if b is None or b.kind != "view" or not b.of:
            break
        ids.append(b.of)
    return ids


def foldoutcasts(graph: Graph) -> int:
    """A narrowing `_to_copy` whose input is produced by a layer norm or a clone and read by nothing
    else: declare the producer's result in the narrow dtype and turn the cast's result into an alias
    (foldoutcasts.jl:82-155).  The producer computes in fp32 either way and rounds once at its store,
    so the values are the ones the cast produced.  Readers are counted through views."""
    producer = {o.out: o for o in graph.ops}
    reads: Dict[str, int] = {}
    for o in graph.ops:
        for i in o.ins:
            r = _viewchain(graph, i)[-1]
            reads[r] = reads.get(r, 0) + 1
    for o in graph.outputs:
        r = _viewchain(graph, o)[-1]
        reads[r] = reads.get(r, 0) + 1
    drop, n = set(), 0
    for cast in graph.ops:
        if cast.aten != "_to_copy.default" or len(cast.ins) != 1:
            continue
        chain = _viewchain(graph, cast.ins[0])
        src = chain[-1]
        p = producer.get(src)
        ob, ib = graph.buffers.get(cast.out), graph.buffers.get(cast.ins[0])
        if (p is None or p.aten not in OUTCAST_PRODUCERS or reads.get(src, 0) != 1 or ob is None or ib is None
                or ob.kind != "transient" or list(ob.shape) != list(ib.shape)
                or np.dtype(ob.dtype).itemsize >= np.dtype(ib.dtype).itemsize):
            continue
        ok = True
        for id in chain:
            b = graph.buffers[id]
            if id == src and "dtypes" in b.attrs:
                sel = graph.buffers[chain[max(0, len(chain) - 2)]]
                ti = sel.attrs.get("arg1") if sel.kind == "view" and "getitem" in sel.viewop else None
                if not isinstance(ti, int) or ti >= len(b.attrs["dtypes"]):
                    ok = False
                    break
                b.attrs["dtypes"] = list(b.attrs["dtypes"])
                b.attrs["dtypes"][ti] = ob.dtype
            else:
                b.dtype = ob.dtype
        if not ok:
            continue
        graph.buffers[cast.out] = Buffer(cast.out, "view", list(ob.shape), ob.dtype, of=cast.ins[0], viewop="alias.default",
                                         attrs=dict(ob.attrs))
        drop.add(cast.id)
        n += 1
    if n:
        graph.ops[:] = [o for o in graph.ops if o.id not in drop]
    return n


WIDECAST_READERS = ("native_layer_norm.default",)


def foldincasts(graph: Graph) -> int:
    """A `_to_copy` that widens fp16 to fp32 in front of a layer norm, read by nothing else: the layer
    norm reads the fp16 value directly (foldincasts.jl:82-124).  fp16 -> fp32 is exact and the layer norm
    accumulates in fp32 for either input, so it sees the same values (here the fp16 and fp32 kernels deal
    elements to lanes differently, so a sum may differ in its last bit); its result keeps the dtype the
    graph declares for it.  Readers are counted through views."""
    readers: Dict[str, List[Op]] = {}
    for o in graph.ops:
        for i in o.ins:
            readers.setdefault(_viewchain(graph, i)[-1], []).append(o)
    isoutput = {_viewchain(graph, o)[-1] for o in graph.outputs}
    drop, n = set(), 0
    for cast in graph.ops:
        if cast.aten != "_to_copy.default" or len(cast.ins) != 1:
            continue
        ob, ib = graph.buffers.get(cast.out), graph.buffers.get(cast.ins[0])
        if ob is None or ib is None or ob.kind != "transient" or list(ob.shape) != list(ib.shape):
            continue
        if not (np.dtype(ib.dtype) == np.float16 and np.dtype(ob.dtype) in (np.dtype(np.float32), np.dtype(np.float64))):
            continue
        rs = readers.get(cast.out, [])
        if cast.out in isoutput or len(rs) != 1 or rs[0].aten not in WIDECAST_READERS:
            continue
        # This runtime's layer norm reads gamma and beta in its input's dtype: fold only when they are
        # fp16 already (or absent); wide ones would have to be rounded, which the fold must never do.
        wb = [graph.buffers.get(i) for i in rs[0].ins[1:3]]
        if any(b is None or np.dtype(b.dtype) != np.float16 for b in wb):
            continue
        graph.buffers[cast.out] = Buffer(cast.out, "view", list(ib.shape), ib.dtype, of=cast.ins[0], viewop="alias.default",
                                         attrs=dict(ob.attrs))
        drop.add(cast.id)
        n += 1
    if n:
        graph.ops[:] = [o for o in graph.ops if o.id not in drop]
    return n


# ------------------------------------------------------------------------------ diagnostics
@dataclass
class Diagnostics:
    """Measurements a run writes into, all off by default (context.jl:162-221).

    optimes         aten name -> (count, milliseconds): every op bracketed by CUDA events on the context's
                    stream with a synchronise around it — a serialising measurement, the only kind that
                    attributes device time to a source-level op, so the totals run longer than the pass.
    opdouble        name of an aten op to run twice per pass ("*" = every op, together with opdoublefilter);
                    the pass's time then grows by that op's real cost in situ, with nothing else disturbed.
    opdoublefilter  (op) -> bool narrowing opdouble to one shape or call site.
    planmisses      buffer id -> count of destinations the slab plan could not place (allocated from the pool).
    launches        aten name -> (ops, kernel launches): which source-level op costs how many launches.
    """
    optimes: Optional[Dict[str, Tuple[int, float]]] = None
    opdouble: str = ""
    opdoublefilter: Optional[Callable[[Any], bool]] = None
    planmisses: Optional[Dict[str, int]] = None
    launches: Optional[Dict[str, Tuple[int, int]]] = None

    def table(self) -> List[Tuple[str, int, float]]:
        """optimes as (aten, count, ms), slowest first."""
        return sorted(((k, n, ms) for k, (n, ms) in (self.optimes or {}).items()), key=lambda r: -r[2])


# ------------------------------------------------------------------------------ model
class Model:
    """Model(graph, weights): rewrite, upload, plan (driver.jl:128-182). `weights` maps safetensors
    keys to numpy arrays in torch layout."""

    def __init__(self, ctx: Ctx, graph: Graph, weights: Dict[str, np.ndarray], dims: Optional[Dict[str, int]] = None,
                 rewrite: bool = True, plan: bool = True):
        self.ctx, self.dims = ctx, dims or {}
        self.graph = copy.deepcopy(graph)
        weights = dict(weights)
        self.rewrites = dict(hoistpermutes=0, foldgelu=0, foldoutcasts=0, foldincasts=0)
        if rewrite:
            from .rewrites import foldbatchnorm, foldrelu, hoistcasts
            extra = dict(hoistcasts=hoistcasts(self.graph, weights), foldbatchnorm=foldbatchnorm(self.graph, weights),
                         foldrelu=foldrelu(self.graph))
            self.rewrites.update({k: v for k, v in extra.items() if v})     # listed only when they fired
            self.rewrites["hoistpermutes"] = hoistpermutes(self.graph, weights)
            self.rewrites["foldgelu"] = foldgelu(self.graph)
            self.rewrites["foldoutcasts"] = foldoutcasts(self.graph)
            self.rewrites["foldincasts"] = foldincasts(self.graph)
        self.weights: Dict[str, DeviceArray] = {}
        for b in self.graph.buffers.values():
            if b.kind == "weight":
                self.weights[b.id] = ctx.toback(np.ascontiguousarray(weights[b.key], dtype=b.dtype))   # toback
        self.plan: Optional[Slab] = planslab(self.graph, self.dims) if plan else None
        self.slab = ctx.allocate(np.uint8, max(self.plan.bytes, 256)) if self.plan else None       # scratchfor
        self.planmisses: Dict[str, int] = {}
        self.diag = Diagnostics(planmisses=self.planmisses)     # m.diag.optimes = {} instruments the next calls

    def __call__(self, *inputs):
        """call(m, name, x...) (driver.jl:202-223): returns the graph's outputs as device arrays."""
        ins = {}
        for id, x in zip(self.graph.inputs, inputs):
            ins[id] = x if isinstance(x, DeviceArray) else self.ctx.toback(np.ascontiguousarray(x))
        return execute_(self.ctx, self.graph, ins, self.weights, dims=self.dims, plan=self.plan, slab=self.slab,
                        planmisses=self.planmisses, diag=self.diag)


# ------------------------------------------------------------------------------ execution
class _Run:
    def __init__(self, ctx, graph, env, dims, plan, slab, planmisses):
        self.ctx, self.graph, self.env, self.dims = ctx, graph, env, dims
        self.plan, self.slab, self.planmisses = plan, slab, planmisses
        self.outid = ""

    # dest / alloc / tupledest (execute.jl:135-158,404-445)
    def dest(self, id: str, dtype, dims) -> DeviceArray:
        a = place(self.plan, self.slab, id, dtype, dims)
        if a is not None:
            return a
        if self.planmisses is not None:
            self.planmisses[id] = self.planmisses.get(id, 0) + 1
        return self.ctx.allocate(dtype, *dims)

    def alloc(self, id: str, *dims) -> DeviceArray:
        return self.dest(id, self.graph.buffers[id].dtype, dims)

    def tupledest(self, i: int, dtype, *dims) -> DeviceArray:
        return self.dest(f"{self.outid}.{i}", dtype, dims)

    def tupledtype(self, i: int, default):
        dts = self.graph.buffers[self.outid].attrs.get("dtypes")
        return dts[i] if dts and dts[i] is not None else default

    def contiguous(self, id: str, a: DeviceArray) -> DeviceArray:
        if a.isdense():
            return a
        return self.ctx.contiguous(a, out=self.dest(id, a.dtype, a.shape))

    def value(self, id: str):
        if id in self.env:
            return self.env[id]
        b = self.graph.buffers.get(id)
        if b is None or b.kind != "view":
            raise B200Error(1, f"execute!: no value for buffer {id}")
        v = self.makeview(b)
        self.env[id] = v
        return v

    def makeview(self, b: Buffer):
        parent = self.value(b.of)
        op, a = b.viewop, b.attrs
        if "getitem" in op:
            return parent[int(a["arg1"])]
        if op in SHAPEONLY_VIEWS:
            return self.contiguous(b.id, parent).reshape(evalshape(b.shape, self.dims))
        n = parent.ndim
        jdim = lambda d: n - 1 - (d + n if d < 0 else d)       # torch axis -> column-major axis
        if op == "permute.default":
            perm = [int(x) for x in a["arg1"]]
            return parent.permute([n - 1 - perm[n - 1 - i] for i in range(n)])
        if op in ("t.default", "transpose.int"):
            d1, d2 = (0, 1) if op == "t.default" else (int(a["arg1"]), int(a["arg2"]))
            perm = list(range(n))
            perm[jdim(d1)], perm[jdim(d2)] = perm[jdim(d2)], perm[jdim(d1)]
            return parent.permute(perm)
        if op == "slice.Tensor":
            d = jdim(int(a.get("arg1", 0)))
            lo = int(a.get("arg2", 0))
            lo = min(max(parent.shape[d] + lo, 0), parent.shape[d]) if lo < 0 else min(lo, parent.shape[d])
            ln = evalshape(b.shape, self.dims)[d]
            return parent.slice(d, lo, lo + ln)
        if op == "select.int":
            d = jdim(int(a["arg1"]))
            i = int(a["arg2"])
            i = parent.shape[d] + i if i < 0 else i
            s = parent.slice(d, i, i + 1)
            return DeviceArray(s.ctx, s.ptr, s.dtype, [x for k, x in enumerate(s.shape) if k != d],
                               [x for k, x in enumerate(s.strides) if k != d], owner=s)
        if op in ("alias.default", "detach.default"):
            return parent
        raise B200Error(1, f"unhandled view op {op} for {b.id}")


def _act_name(attrs) -> str:
    return str(attrs.get("act", "identity")) if attrs.get("act") not in (None, "none") else "identity"


def _dense_weight(run: _Run, a: DeviceArray) -> DeviceArray:
    """The (M,K) operand with M contiguous; a transposed view is materialised into scratch (the
    reference's decline path hands such operands to mul! as transposes)."""
    if _colmajor_2d(a) is not None:
        return a
    return run.ctx.contiguous(a, out=run.ctx.scratch(a.dtype, *a.shape))


def _op_addmm(run: _Run, op: Op):
    bias, a, b = (run.value(i) for i in op.ins)            # ops.jl:1347-1356
    out = run.alloc(op.out, b.shape[0], a.shape[1])
    matmul_(run.ctx, out, _dense_weight(run, b), run.contiguous(op.ins[1] + "#c", a), bias, epi=_act_name(op.attrs))
    return out


def _op_mm(run: _Run, op: Op):
    a, b = (run.value(i) for i in op.ins)                  # ops.jl:1358-1363
    out = run.alloc(op.out, b.shape[0], a.shape[1])
    matmul_(run.ctx, out, _dense_weight(run, b), run.contiguous(op.ins[0] + "#c", a), None)
    return out


def _op_bmm(run: _Run, op: Op):
    a, b = (run.value(i) for i in op.ins)                  # ops.jl:1393-1399
    out = run.alloc(op.out, b.shape[0], a.shape[1], a.shape[2])
    batchedmatmul_(run.ctx, out, run.contiguous(op.ins[1] + "#c", b), run.contiguous(op.ins[0] + "#c", a))
    return out


def _op_sdpa(run: _Run, op: Op):
    q, k, v = (run.value(i) for i in op.ins[:3])           # ops.jl:1365-1391
    # the mem-efficient variant's fourth input is the additive mask, (Lk, Lq, H, B) in the graph's order
    bias = run.value(op.ins[3]) if len(op.ins) > 3 and "efficient" in op.aten else None
    if bias is not None and not bias.isdense():
        bias = run.contiguous(op.ins[3] + "#c", bias)
    E, Lq, H, B = q.shape
    scale = float(op.attrs["scale"]) if op.attrs.get("scale") is not None else 1.0 / sqrt(E)
    out = run.tupledest(0, run.tupledtype(0, np.float32 if q.dtype == np.float32 else q.dtype), E, Lq, H, B)
    sdpa(run.ctx, q, k, v, bias, scale, out=out)
    return (out,) + (None,) * 8                             # a 9-tuple of which only element 0 is real


def _op_layernorm(run: _Run, op: Op):
    a = run.value(op.ins[0])                                # ops.jl:575-609
    nshape = [int(x) for x in op.attrs["arg1"]]
    n = int(np.prod(nshape))
    eps = float(op.attrs["arg4"])
    g = run.value(op.ins[1]) if len(op.ins) >= 2 else None
    b = run.value(op.ins[2]) if len(op.ins) >= 3 else None
    a = run.contiguous(op.ins[0] + "#c", a)
    # gamma/beta narrower than the input are widened (exact) into scratch; the kernel reads them in the input's dtype
    widen = lambda t: t if t is None or t.dtype == a.dtype or np.dtype(t.dtype).itemsize > a.dtype.itemsize \
        else to_copy_(run.ctx, run.ctx.scratch(a.dtype, *t.shape), t)
    g, b = widen(g), widen(b)
    out = run.tupledest(0, run.tupledtype(0, a.dtype), *a.shape)
    groups = a.size // n
    mean, rstd = run.tupledest(1, np.float32, groups), run.tupledest(2, np.float32, groups)
    layernorm_(run.ctx, out, mean, rstd, a, g, b, n, eps)
    return (out, mean, rstd)


def _op_gelu(run: _Run, op: Op):
    x = run.value(op.ins[0])                                # ops.jl:1698-1702
    approx = str(op.attrs.get("approximate", op.attrs.get("arg1", "none")))
    out = run.alloc(op.out, *x.shape)
    act_(run.ctx, out, run.contiguous(op.ins[0] + "#c", x), "gelu_tanh" if approx == "tanh" else "gelu")
    return out


def _op_add(run: _Run, op: Op):
    a, b = (run.value(i) for i in op.ins[:2])               # ops.jl:186-197 (same-shape operands only)
    if a.shape != b.shape:
        raise B200Error(17, f"add.Tensor: broadcasting {a.shape} + {b.shape} is outside the hot path")
    out = run.alloc(op.out, *a.shape)
    add_(run.ctx, out, run.contiguous(op.ins[0] + "#c", a), run.contiguous(op.ins[1] + "#c", b))
    if _act_name(op.attrs) != "identity":      # a relu folded into the add that ends a residual block (foldrelu)
        act_(run.ctx, out, out, _act_name(op.attrs))
    return out


def _op_clamp(run: _Run, op: Op):
    x = run.value(op.ins[0])                                # ops.jl:323-335
    lo = float(op.attrs["arg1"]) if op.attrs.get("arg1") is not None else -np.inf
    hi = float(op.attrs["arg2"]) if op.attrs.get("arg2") is not None else np.inf
    out = run.alloc(op.out, *x.shape)
    clamp_(run.ctx, out, run.contiguous(op.ins[0] + "#c", x), lo, hi)
    return out


def _op_clone(run: _Run, op: Op):
    x = run.value(op.ins[0])                                # clone.default: a dense copy in the planned slot
    out = run.alloc(op.out, *x.shape)
    if x.isdense():
        run.ctx.copy(out, x)
    else:
        run.ctx.contiguous(x, out=out)
    return out


def _op_to_copy(run: _Run, op: Op):
    x = run.value(op.ins[0])                                # ops.jl:342-358: the declared dtype of the result
    b = run.graph.buffers.get(op.out)
    out = run.dest(op.out, b.dtype if b is not None else x.dtype, x.shape)
    to_copy_(run.ctx, out, run.contiguous(op.ins[0] + "#c", x))
    return out


def _op_maxpool(run: _Run, op: Op):
    x = run.value(op.ins[0])                                # ops.jl:1329-1343; x is (W, H, C, N)
    rev = lambda v: tuple(int(t) for t in reversed(v))
    k = rev(op.attrs["arg1"])
    s = rev(op.attrs["arg2"]) if op.attrs.get("arg2") else k
    p = rev(op.attrs["arg3"]) if op.attrs.get("arg3") else (0, 0)
    W, H, Cn, N = x.shape
    out = run.tupledest(0, x.dtype, (W + 2 * p[0] - k[0]) // s[0] + 1, (H + 2 * p[1] - k[1]) // s[1] + 1, Cn, N)
    maxpool2d_(run.ctx, out, x, k, s, p)                    # strided views are read in place
    return (out, None)                                      # the indices are never read


def _op_convolution(run: _Run, op: Op):
    x, w = run.value(op.ins[0]), run.value(op.ins[1])       # ops.jl:1114-1222 (2-D)
    bias = run.value(op.ins[2]) if len(op.ins) >= 3 else None
    rev = lambda v: tuple(int(t) for t in reversed(v))      # torch (h, w) -> (x, y)
    stride, padding, dilation = rev(op.attrs["arg3"]), rev(op.attrs["arg4"]), rev(op.attrs["arg5"])
    groups = int(op.attrs.get("arg8", 1))
    if x.ndim != 4:
        raise B200Error(17, "convolution: only 2-D convolutions (callers lift 1-D ones, as the reference does)")
    if bool(op.attrs.get("arg6", False)):                    # transposed: arg7 is output_padding
        outpad = rev(op.attrs.get("arg7", (0, 0)))
        W, H, _, N = x.shape
        KW, KH, COG, _ = w.shape
        OW = convtransposesize(W, KW, stride[0], padding[0], dilation[0], outpad[0])
        OH = convtransposesize(H, KH, stride[1], padding[1], dilation[1], outpad[1])
        out = run.alloc(op.out, OW, OH, COG * groups, N)
        convolutiontranspose_(run.ctx, out, run.contiguous(op.ins[0] + "#c", x), w, bias, stride, padding, dilation,
                              outpad, groups)
        return out
    W, H, _, N = x.shape
    KW, KH, _, Cout = w.shape
    OW = convsize(W, KW, stride[0], padding[0], dilation[0])
    OH = convsize(H, KH, stride[1], padding[1], dilation[1])
    out = run.alloc(op.out, OW, OH, Cout, N)
    convolution_(run.ctx, out, run.contiguous(op.ins[0] + "#c", x), w, bias, stride, padding, dilation, groups,
                 act=_act_name(op.attrs))
    return out


RUNOP = {
    "addmm.default": _op_addmm, "mm.default": _op_mm, "bmm.default": _op_bmm,
    "_scaled_dot_product_flash_attention.default": _op_sdpa,
    "_scaled_dot_product_efficient_attention.default": _op_sdpa,
    "native_layer_norm.default": _op_layernorm, "gelu.default": _op_gelu, "add.Tensor": _op_add,
    "clamp.default": _op_clamp, "clone.default": _op_clone, "convolution.default": _op_convolution,
    "_to_copy.default": _op_to_copy, "max_pool2d_with_indices.default": _op_maxpool,
}


def execute_(ctx: Ctx, graph: Graph, inputs: Dict[str, DeviceArray], weights: Dict[str, DeviceArray],
             dims: Optional[Dict[str, int]] = None, plan: Optional[Slab] = None, slab: Optional[DeviceArray] = None,
             planmisses: Optional[Dict[str, int]] = None, diag: Optional[Diagnostics] = None) -> List[Any]:
    """execute!(graph, inputs, weights; slab, plan, ws, diag) (execute.jl:493-539): run the ops in order,
    resetting the workspace at the top of each; nothing synchronises between ops unless `diag.optimes` asks
    for per-op times (timeop!, execute.jl:550-570)."""
    env: Dict[str, Any] = {}
    env.update(weights)
    env.update(inputs)
    diag = diag or Diagnostics()
    if planmisses is None:
        planmisses = diag.planmisses
    run = _Run(ctx, graph, env, dims or {}, plan, slab, planmisses)
    for op in graph.ops:
        run.outid = op.out
        fn = RUNOP.get(op.aten)
        if fn is None:
            raise B200Error(1, f"no B200 implementation for {op.aten} (op {op.id})")
        n0 = ctx.launch_count() if diag.launches is not None else 0
        if diag.optimes is not None:
            ctx.synchronize()
            ctx.ws.reset()
            ctx.timer_start()
            env[op.out] = fn(run, op)
            ms = ctx.timer_stop()          # records, synchronises, reads
            n, tot = diag.optimes.get(op.aten, (0, 0.0))
            diag.optimes[op.aten] = (n + 1, tot + ms)
        else:
            d = diag.opdouble
            if d and (d == "*" or op.aten == d) and (diag.opdoublefilter is None or diag.opdoublefilter(op)):
                ctx.ws.reset()
                fn(run, op)                # an idempotent op run a second time changes nothing but the pass's time
            ctx.ws.reset()
            env[op.out] = fn(run, op)
        if diag.launches is not None:
            n, k = diag.launches.get(op.aten, (0, 0))
            diag.launches[op.aten] = (n + 1, k + ctx.launch_count() - n0)
    return [run.value(o) for o in graph.outputs]
