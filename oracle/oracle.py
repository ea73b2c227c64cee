"""ctypes loader for the CPU oracle (test infrastructure, not product).

Only the test-suite, the smoke check and the benchmark's CPU-baseline / reference arm may
import this module.  Arrays follow the reference's convention: a numpy array in torch
(row-major) order *is* the reference's column-major array with the reversed shape, so the
wrappers take numpy arrays in torch order and pass their buffers straight through.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "liboracle.so")

F16, F32 = 0, 1
EPI = {"none": 0, "identity": 0, "relu": 1, "gelu": 2, "gelu_tanh": 3}


def build(force: bool = False) -> str:
    """Compile oracle.c with the committed Makefile (gcc + OpenMP)."""
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        L = C.CDLL(_SO)
        L.ora_erf_f32.restype = C.c_float
        L.ora_erf_f32.argtypes = [C.c_float]
        L.ora_gelu_exact_f32.restype = C.c_float
        L.ora_gelu_exact_f32.argtypes = [C.c_float]
        L.ora_gelu_tanh_f32.restype = C.c_float
        L.ora_gelu_tanh_f32.argtypes = [C.c_float]
        L.ora_convsize.restype = C.c_int64
        L.ora_convsize.argtypes = [C.c_int64] * 5
        L.ora_num_threads.restype = C.c_int
        _lib = L
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _i64(*v):
    return [C.c_int64(int(x)) for x in v]


def _dt(dtype) -> int:
    return F16 if np.dtype(dtype) == np.float16 else F32


def num_threads() -> int:
    return lib().ora_num_threads()


def set_num_threads(n: int) -> int:
    """Use `n` threads from now on, whatever OMP_NUM_THREADS said at load time; returns the count in force."""
    L = lib()
    L.ora_set_num_threads.restype = C.c_int
    return L.ora_set_num_threads(C.c_int(int(n)))


def use_all_cores() -> int:
    """Use every core this process may run on (its affinity mask)."""
    return set_num_threads(len(os.sched_getaffinity(0)))


def act(x: np.ndarray, name: str) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float16)
    y = np.empty_like(x)
    lib().ora_act_f16(_p(x), _p(y), C.c_int64(x.size), C.c_int(EPI[name]))
    return y


def erf(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float16)
    y = np.empty_like(x)
    lib().ora_erf_f16(_p(x), _p(y), C.c_int64(x.size))
    return y


def linear(x: np.ndarray, wt: np.ndarray, bias=None, epi="none", out_dtype=np.float16):
    """Y[tokens,out] = epi(X[tokens,K] @ Wt[K,out] + bias[out]) (torch order).

    In the reference's orientation this is matmul!(out, A=Wt' (M=out,K), B=X' (K,N=tokens)).
    """
    x = np.ascontiguousarray(x, dtype=np.float16)
    wt = np.ascontiguousarray(wt, dtype=np.float16)
    N, K = x.shape
    K2, M = wt.shape
    assert K == K2
    out = np.empty((N, M), dtype=out_dtype)
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float16)
    lib().ora_gemm_f16(*_i64(M, N, K), _p(wt), C.c_int64(M), _p(x), C.c_int64(K), _p(b), _p(out),
                       C.c_int64(M), C.c_int(_dt(out_dtype)), C.c_int(EPI[epi]))
    return out


def linear_f64(x, wt, bias=None):
    x = np.ascontiguousarray(x, dtype=np.float16)
    wt = np.ascontiguousarray(wt, dtype=np.float16)
    N, K = x.shape
    _, M = wt.shape
    out = np.empty((N, M), dtype=np.float64)
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float16)
    lib().ora_gemm_f64(*_i64(M, N, K), _p(wt), C.c_int64(M), _p(x), C.c_int64(K), _p(b), _p(out),
                       C.c_int64(M))
    return out


def bmm(a: np.ndarray, b: np.ndarray, out_dtype=np.float16):
    """torch bmm: a (nb,m,k) @ b (nb,k,n) -> (nb,m,n)."""
    a = np.ascontiguousarray(a, dtype=np.float16)
    b = np.ascontiguousarray(b, dtype=np.float16)
    nb, m, k = a.shape
    _, _, n = b.shape
    out = np.empty((nb, m, n), dtype=out_dtype)
    # reference orientation: out(M=n, N=m) = A(M=n,K=k) [= torch b] * B(K=k,N=m) [= torch a]
    lib().ora_bmm_f16(*_i64(n, m, k, nb), _p(b), C.c_int64(n), C.c_int64(k * n), _p(a),
                      C.c_int64(k), C.c_int64(m * k), _p(out), C.c_int64(n), C.c_int64(m * n),
                      C.c_int(_dt(out_dtype)))
    return out


def _strides4(a: np.ndarray):
    """Element strides of a torch (B,H,L,E) array in the reference's (E,L,H,B) order."""
    s = [x // a.itemsize for x in a.strides]
    return (C.c_int64 * 4)(s[3], s[2], s[1], s[0])


def _bias_args(bias, B, H, Lq, Lk):
    """bias: torch-order (B|1, H|1, Lq|1, Lk|1) fp16 additive mask or None -> (ptr, strides over Lk,Lq,H,B)."""
    if bias is None:
        return None, None
    assert bias.dtype == np.float16 and bias.ndim == 4
    for have, want in zip(bias.shape, (B, H, Lq, Lk)):
        assert have in (1, want), f"bias shape {bias.shape} does not broadcast to {(B, H, Lq, Lk)}"
    it = bias.itemsize
    st = [0 if bias.shape[ax] == 1 else bias.strides[ax] // it for ax in (3, 2, 1, 0)]
    return _p(bias), (C.c_int64 * 4)(*st)


def attention_threepass(q, k, v, scale, out_dtype=np.float32, bias=None):
    """q,k,v: torch (B,H,L,E) fp16 arrays (any strides). Returns dense (B,H,Lq,E)."""
    B, H, Lq, E = q.shape
    Lk = k.shape[2]
    out = np.empty((B, H, Lq, E), dtype=out_dtype)
    bp, bs = _bias_args(bias, B, H, Lq, Lk)
    lib().ora_attention_threepass(*_i64(E, Lq, Lk, H, B), _p(q), _strides4(q), _p(k), _strides4(k),
                                  _p(v), _strides4(v), _p(out), C.c_int(_dt(out_dtype)),
                                  C.c_float(scale), bp, bs)
    return out


def attention_ref(q, k, v, scale, bias=None):
    B, H, Lq, E = q.shape
    Lk = k.shape[2]
    out = np.empty((B, H, Lq, E), dtype=np.float32)
    bp, bs = _bias_args(bias, B, H, Lq, Lk)
    lib().ora_attention_ref(*_i64(E, Lq, Lk, H, B), _p(q), _strides4(q), _p(k), _strides4(k),
                            _p(v), _strides4(v), _p(out), C.c_float(scale), bp, bs)
    return out


def to_le(a):
    """(B,H,L,E) strided -> dense torch (B,H,E,L) (= reference dense (L,E,H,B))."""
    B, H, L, E = a.shape
    out = np.empty((B, H, E, L), dtype=np.float16)
    lib().ora_to_le_f16(*_i64(E, L, H, B), _p(a), _strides4(a), _p(out))
    return out


def layernorm(a: np.ndarray, gamma=None, beta=None, eps=1e-5, out_dtype=None):
    """a: (..., C) torch order. Returns (out, mean, rstd)."""
    a = np.ascontiguousarray(a)
    Cn = a.shape[-1]
    groups = a.size // Cn
    out_dtype = a.dtype if out_dtype is None else np.dtype(out_dtype)
    out = np.empty(a.shape, dtype=out_dtype)
    mean = np.empty(groups, dtype=np.float32)
    rstd = np.empty(groups, dtype=np.float32)
    g = None if gamma is None else np.ascontiguousarray(gamma, dtype=a.dtype)
    b = None if beta is None else np.ascontiguousarray(beta, dtype=a.dtype)
    lib().ora_layernorm(*_i64(groups, Cn), _p(a), C.c_int(_dt(a.dtype)), _p(out),
                        C.c_int(_dt(out_dtype)), _p(mean), _p(rstd), _p(g), _p(b), C.c_float(eps))
    return out, mean, rstd


def convsize(n, k, s, p, d):
    return lib().ora_convsize(*_i64(n, k, s, p, d))


def conv2d(x, w, bias=None, stride=(1, 1), padding=(0, 0), dilation=(1, 1), epi="none",
           out_dtype=np.float16):
    """x: torch (N,Cin,H,W); w: torch (Cout,Cin,KH,KW); stride etc. in torch (h,w) order."""
    x = np.ascontiguousarray(x, dtype=np.float16)
    w = np.ascontiguousarray(w, dtype=np.float16)
    N, Cin, H, W = x.shape
    Cout, _, KH, KW = w.shape
    (sy, sx), (py, px), (dy, dx) = stride, padding, dilation
    OW, OH = convsize(W, KW, sx, px, dx), convsize(H, KH, sy, py, dy)
    out = np.empty((N, Cout, OH, OW), dtype=out_dtype)
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float16)
    lib().ora_conv2d_f16(*_i64(W, H, Cin, N, KW, KH, Cout, sx, sy, px, py, dx, dy), _p(x), _p(w),
                         _p(b), _p(out), C.c_int(_dt(out_dtype)), C.c_int(EPI[epi]))
    return out


def conv2d_grouped(x, w, bias=None, stride=(1, 1), padding=(0, 0), dilation=(1, 1), groups=1, epi="none",
                   out_dtype=np.float16):
    """x: torch (N,Cin,H,W); w: torch (Cout,Cin/groups,KH,KW)."""
    x = np.ascontiguousarray(x, dtype=np.float16)
    w = np.ascontiguousarray(w, dtype=np.float16)
    N, Cin, H, W = x.shape
    Cout, _, KH, KW = w.shape
    (sy, sx), (py, px), (dy, dx) = stride, padding, dilation
    OW, OH = convsize(W, KW, sx, px, dx), convsize(H, KH, sy, py, dy)
    out = np.empty((N, Cout, OH, OW), dtype=out_dtype)
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float16)
    lib().ora_conv2d_grouped_f16(*_i64(W, H, Cin, N, KW, KH, Cout, sx, sy, px, py, dx, dy, groups), _p(x), _p(w),
                                 _p(b), _p(out), C.c_int(_dt(out_dtype)), C.c_int(EPI[epi]))
    return out


def convtransposesize(n, k, s, p, d, op):
    return (n - 1) * s - 2 * p + d * (k - 1) + op + 1


def convtranspose2d(x, w, bias=None, stride=(1, 1), padding=(0, 0), dilation=(1, 1), output_padding=(0, 0), groups=1,
                    out_dtype=np.float16):
    """x: torch (N,Cin,H,W); w: torch (Cin,Cout/groups,KH,KW); stride etc. in torch (h,w) order."""
    x = np.ascontiguousarray(x, dtype=np.float16)
    w = np.ascontiguousarray(w, dtype=np.float16)
    N, Cin, H, W = x.shape
    _, COG, KH, KW = w.shape
    Cout = COG * groups
    (sy, sx), (py, px), (dy, dx), (opy, opx) = stride, padding, dilation, output_padding
    OW, OH = convtransposesize(W, KW, sx, px, dx, opx), convtransposesize(H, KH, sy, py, dy, opy)
    out = np.empty((N, Cout, OH, OW), dtype=out_dtype)
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float16)
    lib().ora_convtranspose2d_f16(*_i64(W, H, Cin, N, KW, KH, Cout, sx, sy, px, py, dx, dy, opx, opy, groups), _p(x),
                                  _p(w), _p(b), _p(out), C.c_int(_dt(out_dtype)))
    return out


def im2col(x, KH, KW, stride, padding, dilation, MP, CRSP):
    """Returns col as a torch-order (CRSP, MP) array (= reference column-major (MP,CRSP))."""
    x = np.ascontiguousarray(x, dtype=np.float16)
    N, Cin, H, W = x.shape
    (sy, sx), (py, px), (dy, dx) = stride, padding, dilation
    col = np.empty((CRSP, MP), dtype=np.float16)
    lib().ora_im2col_f16(*_i64(W, H, Cin, N, KW, KH, sx, sy, px, py, dx, dy, MP, CRSP), _p(x),
                         _p(col))
    return col


def add(a, b):
    a = np.ascontiguousarray(a, dtype=np.float16)
    b = np.ascontiguousarray(b, dtype=np.float16)
    y = np.empty_like(a)
    lib().ora_add_f16(_p(a), _p(b), _p(y), C.c_int64(a.size))
    return y


def clamp(a, lo, hi):
    a = np.ascontiguousarray(a, dtype=np.float16)
    y = np.empty_like(a)
    lib().ora_clamp_f16(_p(a), _p(y), C.c_int64(a.size), C.c_float(lo), C.c_float(hi))
    return y


def maxpool2d(x: np.ndarray, k, s, p=(0, 0)) -> np.ndarray:
    """kernels/resample.jl:121-141 (maxpool): x torch (N,C,H,W); k, s, p = (x, y) pairs; positions
    outside the image are skipped and the maximum starts from the lowest value of the type."""
    N, Cn, H, W = x.shape
    OW, OH = (W + 2 * p[0] - k[0]) // s[0] + 1, (H + 2 * p[1] - k[1]) // s[1] + 1
    pad = np.full((N, Cn, H + 2 * p[1], W + 2 * p[0]), -np.inf, dtype=x.dtype)
    pad[:, :, p[1]:p[1] + H, p[0]:p[0] + W] = x
    out = np.full((N, Cn, OH, OW), -np.inf, dtype=x.dtype)
    for dy in range(k[1]):
        for dx in range(k[0]):
            out = np.maximum(out, pad[:, :, dy:dy + (OH - 1) * s[1] + 1:s[1], dx:dx + (OW - 1) * s[0] + 1:s[0]])
    return out
