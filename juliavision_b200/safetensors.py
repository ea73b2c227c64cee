"""Minimal safetensors reader (reference DNNKernels/src/safetensors.jl:14-58): a u64 little-endian
header length, a JSON header mapping each name to dtype / shape / byte range, then the raw data.

Arrays come back as numpy arrays in the file's own (torch, row-major) shape; `Ctx.toback` uploads
them with the extents reversed, which is the column-major array the reference's reader returns —
element for element the same bytes, no transpose.  bfloat16 has no numpy form and comes back as
uint16 bit patterns, as in the reference (DTYPES maps "BF16" to UInt16).
"""
from __future__ import annotations

import json
import struct
from typing import Dict, List

import numpy as np

DTYPES = {"F64": np.float64, "F32": np.float32, "F16": np.float16, "BF16": np.uint16, "I64": np.int64, "I32": np.int32,
          "I16": np.int16, "I8": np.int8, "U8": np.uint8, "BOOL": np.bool_, "U64": np.uint64, "U32": np.uint32,
          "U16": np.uint16, "C64": np.complex64, "C128": np.complex128}


def _header(f):
    raw = f.read(8)
    if len(raw) != 8:
        raise ValueError("safetensors: file shorter than its header length")
    (hlen,) = struct.unpack("<Q", raw)
    head = f.read(hlen)
    if len(head) != hlen:
        raise ValueError("safetensors: truncated header")
    return json.loads(head), 8 + hlen


def safetensorsnames(path: str) -> List[str]:
    """Header only, without reading any tensor data (safetensors.jl:52-58)."""
    with open(path, "rb") as f:
        header, _ = _header(f)
    return [k for k in header if k != "__metadata__"]


def readsafetensors(path: str) -> Dict[str, np.ndarray]:
    """readsafetensors(path): name -> array.  A scalar (empty shape) comes back 0-dimensional."""
    out: Dict[str, np.ndarray] = {}
    with open(path, "rb") as f:
        header, base = _header(f)
        for name, spec in header.items():
            if name == "__metadata__":
                continue
            if spec["dtype"] not in DTYPES:
                raise KeyError(f"safetensors: dtype {spec['dtype']} of {name} is not supported")
            dt = np.dtype(DTYPES[spec["dtype"]]).newbyteorder("<")
            lo, hi = spec["data_offsets"]
            n = (hi - lo) // dt.itemsize
            shape = tuple(int(s) for s in spec["shape"])
            if int(np.prod(shape, dtype=np.int64)) != n:
                raise ValueError(f"safetensors: {name} has {n} elements for shape {shape}")
            f.seek(base + lo)
            data = np.fromfile(f, dtype=dt, count=n)
            if data.size != n:
                raise ValueError(f"safetensors: {name} runs past the end of the file")
            out[name] = data.reshape(shape)
    return out
