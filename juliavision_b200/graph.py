"""Exported-graph format: `Buffer` / `Op` / `Graph`, `loadgraph`, `evalshape` (reference
DNNKernels/src/graph.jl:9-207; the JSON is what tools/export_graphs.py:111-230 emits).

Shapes in the file are in torch order and may be symbolic; `evalshape` resolves them and returns
them REVERSED, i.e. in the column-major order the arrays use.
"""
from __future__ import annotations

import ast
import json
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np

DTYPE_NAMES = {"float32": np.float32, "float64": np.float64, "float16": np.float16, "int64": np.int64,
               "int32": np.int32, "bool": np.bool_, "uint8": np.uint8}     # no bfloat16, as in the reference


@dataclass
class Buffer:
    id: str
    kind: str                      # weight | external | transient | view | host
    shape: List[Any]               # ints and symbolic strings, torch order
    dtype: Any
    key: str = ""                  # weight: name in the weights file
    live: Tuple[int, int] = (0, 0)  # transient: op indices (advisory; the planner recomputes)
    of: str = ""                   # view: parent buffer id
    viewop: str = ""               # view: which aten op produced it
    attrs: Dict[str, Any] = field(default_factory=dict)


@dataclass
class Op:
    id: str
    aten: str
    ins: List[str]
    out: str
    attrs: Dict[str, Any] = field(default_factory=dict)


@dataclass
class Graph:
    name: str
    symbols: List[str]
    inputs: List[str]
    outputs: List[str]
    buffers: Dict[str, Buffer]
    order: List[str]               # buffer ids in declaration order
    ops: List[Op]
    fusion: List[List[str]] = field(default_factory=list)


def _buffer(o: dict) -> Buffer:
    attrs = dict(o.get("attrs", {}))
    if "expr" in o:
        attrs["expr"] = o["expr"]
    if "shapes" in o:
        attrs["shapes"] = [None if s is None else list(s) for s in o["shapes"]]
    if "dtypes" in o:
        attrs["dtypes"] = [None if d is None else DTYPE_NAMES.get(d) for d in o["dtypes"]]
    return Buffer(id=str(o["id"]), kind=str(o["kind"]), shape=list(o.get("shape", [])),
                  dtype=DTYPE_NAMES[o["dtype"]] if "dtype" in o else np.float32, key=str(o.get("key", "")),
                  live=tuple(o["live"]) if "live" in o else (0, 0), of=str(o["of"]) if o.get("of") else "",
                  viewop=str(o.get("op", "")), attrs=attrs)


def loadgraph(src) -> Graph:
    """loadgraph(path) (graph.jl:125-149); also accepts the already-parsed dict."""
    j = src if isinstance(src, dict) else json.load(open(src))
    buffers, order = {}, []
    for o in j["buffers"]:
        b = _buffer(o)
        buffers[b.id] = b
        order.append(b.id)
    ops = [Op(str(o["id"]), str(o["aten"]), [str(x) for x in o["in"]], str(o["out"]), dict(o.get("attrs", {})))
           for o in j["ops"]]
    fusion = [[str(x) for x in g["ops"]] for g in j.get("fusion_groups", [])]
    return Graph(str(j["name"]), [str(s) for s in j.get("symbols", [])], [str(s) for s in j["inputs"]],
                 [str(s) for s in j["outputs"]], buffers, order, ops, fusion)


def evalexpr(e, dims: Dict[str, int]) -> int:
    """Products, quotients and sums of the base symbols (graph.jl:176-207)."""
    if isinstance(e, (int, np.integer)):
        return int(e)
    node = ast.parse(str(e), mode="eval").body

    def ev(n):
        if isinstance(n, ast.Constant):
            return int(n.value)
        if isinstance(n, ast.Name):
            return int(dims[n.id])
        if isinstance(n, ast.UnaryOp) and isinstance(n.op, ast.USub):
            return -ev(n.operand)
        if isinstance(n, ast.BinOp):
            a, b = ev(n.left), ev(n.right)
            if isinstance(n.op, ast.Add):
                return a + b
            if isinstance(n.op, ast.Sub):
                return a - b
            if isinstance(n.op, ast.Mult):
                return a * b
            if isinstance(n.op, (ast.Div, ast.FloorDiv)):
                return a // b
            if isinstance(n.op, ast.Mod):
                return a % b
            if isinstance(n.op, ast.Pow):
                return a ** b
        if isinstance(n, ast.Call) and isinstance(n.func, ast.Name):
            as_ = [ev(a) for a in n.args]
            f = n.func.id
            if f == "Mod":
                return as_[0] % as_[1]
            if f == "Max":
                return max(as_)
            if f == "Min":
                return min(as_)
            if f in ("floor", "floordiv"):
                return as_[0] if len(as_) == 1 else as_[0] // as_[1]
            if f == "ceiling":
                return as_[0] if len(as_) == 1 else -(-as_[0] // as_[1])
            if f == "Pow":
                return as_[0] ** as_[1]
        raise ValueError(f"unsupported shape expression: {e}")

    return ev(node)


def evalshape(shape: Sequence[Any], dims: Optional[Dict[str, int]] = None) -> Tuple[int, ...]:
    """Resolve a symbolic torch-order shape and return it reversed (graph.jl:161-167)."""
    dims = dims or {}
    return tuple(reversed([evalexpr(s, dims) for s in shape]))
