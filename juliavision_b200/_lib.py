"""ctypes binding of libb200dnn.so — the same symbols a Julia `ccall` would bind.

The library is sm_100a-only and there is no fallback: if the shared object is missing or a
symbol cannot be resolved, importing the product fails loudly.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
SO_PATH = os.path.join(HERE, "csrc", "libb200dnn.so")

OK, EINVAL, ECUDA, ENOMEM, EKERNEL = 0, 1, 2, 3, 4
DECLINE = {16: "operands", 17: "extent", 18: "wrapped", 19: "bias", 20: "eltype", 21: "tiling"}
F16, F32 = 0, 1
EPI = {"identity": 0, "none": 0, None: 0, "relu": 1, "gelu": 2, "gelu_tanh": 3}


class B200Error(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"b200dnn status {code}: {msg}")
        self.code = code


class Caps(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("coopmat", "tile", "subgroup", "coopmatsubgroup", "sharedbudget",
                                         "workgrouplimit", "cores", "warps", "cc_major", "cc_minor")] + \
               [("total_mem", C.c_int64)]


class GemmPlan(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("block_m", "block_n", "block_k", "stages", "tiles_m", "tiles_n", "ctas",
                                         "smem_bytes")]


class Strided4(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("stride", C.c_int64 * 4)]


_i64, _i32, _vp, _f32, _sz = C.c_int64, C.c_int, C.c_void_p, C.c_float, C.c_size_t
_pp = C.POINTER(C.c_void_p)

# name -> (restype, argtypes); every symbol include/b200dnn.h declares.
SIGNATURES = {
    "b200_ctx_create": (_i32, [_i32, _pp]),
    "b200_ctx_destroy": (_i32, [_vp]),
    "b200_caps": (_i32, [_vp, C.POINTER(Caps)]),
    "b200_sync": (_i32, [_vp]),
    "b200_last_error": (C.c_char_p, []),
    "b200_version": (C.c_char_p, []),
    "b200_stream": (_vp, [_vp]),
    "b200_launch_count": (_i64, [_vp]),
    "b200_selftest_bounded_wait": (_i32, [_vp, _i64, _vp]),
    "b200_timer_start": (_i32, [_vp]),
    "b200_timer_stop": (_i32, [_vp, C.POINTER(_f32)]),
    "b200_graph_begin": (_i32, [_vp]),
    "b200_graph_end": (_i32, [_vp, _pp]),
    "b200_graph_launch": (_i32, [_vp, _vp]),
    "b200_graph_destroy": (_i32, [_vp]),
    "b200_pool_alloc": (_i32, [_vp, _sz, _pp]),
    "b200_pool_free": (_i32, [_vp, _vp]),
    "b200_pool_stats": (_i32, [_vp, C.POINTER(_sz), C.POINTER(_sz)]),
    "b200_upload": (_i32, [_vp, _vp, _vp, _sz]),
    "b200_download": (_i32, [_vp, _vp, _vp, _sz]),
    "b200_upload_async": (_i32, [_vp, _vp, _vp, _sz]),
    "b200_download_async": (_i32, [_vp, _vp, _vp, _sz]),
    "b200_copy": (_i32, [_vp, _vp, _vp, _sz]),
    "b200_fill_bytes": (_i32, [_vp, _vp, _i32, _sz]),
    "b200_host_alloc": (_i32, [_sz, _pp]),
    "b200_host_free": (_i32, [_vp]),
    "b200_copy_lane_upload": (_i32, [_vp, _vp, _vp, _sz]),
    "b200_copy_lane_download": (_i32, [_vp, _vp, _vp, _sz]),
    "b200_event_create": (_i32, [_vp, _pp]),
    "b200_event_destroy": (_i32, [_vp]),
    "b200_event_record": (_i32, [_vp, _vp, _i32]),
    "b200_lane_wait_event": (_i32, [_vp, _i32, _vp]),
    "b200_workspace_reset": (_i32, [_vp]),
    "b200_workspace_scratch": (_i32, [_vp, _sz, _pp]),
    "b200_workspace_stats": (_i32, [_vp, C.POINTER(_sz), C.POINTER(_sz), C.POINTER(_i32)]),
    "b200_gemm_f16": (_i32, [_vp, _i64, _i64, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _i64, _i32, _i32, _i64, _i64,
                             _i64, _i64]),
    "b200_gemm_f16_supported": (_i32, [_i64, _i64, _i64, _i64, _i64, _i64, _i32]),
    "b200_gemm_f16_plan": (_i32, [_vp, _i64, _i64, _i64, _i64, C.POINTER(GemmPlan)]),
    "b200_timeline": (_i32, [_vp, _vp]),
    "b200_gemv": (_i32, [_vp, _i64, _i64, _vp, _i64, _vp, _vp, _i32, _vp, _i32, _i32]),
    "b200_attention_f16": (_i32, [_vp, _i64, _i64, _i64, _i64, _i64, C.POINTER(Strided4), C.POINTER(Strided4),
                                  C.POINTER(Strided4), _vp, _i32, _f32]),
    "b200_attention_f16_strided": (_i32, [_vp, _i64, _i64, _i64, _i64, _i64, C.POINTER(Strided4), C.POINTER(Strided4),
                                          C.POINTER(Strided4), C.POINTER(Strided4), _i32, _f32]),
    "b200_attention_f16_bias": (_i32, [_vp, _i64, _i64, _i64, _i64, _i64, C.POINTER(Strided4), C.POINTER(Strided4),
                                       C.POINTER(Strided4), C.POINTER(Strided4), C.POINTER(Strided4), _i32, _f32]),
    "b200_attention_f16_supported": (_i32, [_i64, _i64, _i64, _i64, _i64, C.POINTER(_i64), C.POINTER(_i64),
                                            C.POINTER(_i64), _i32]),
    "b200_attention_f16_route": (_i32, [_i64, _i64, _i64, _i64, _i64, C.POINTER(_i64), C.POINTER(_i64), C.POINTER(_i64)]),
    "b200_layernorm": (_i32, [_vp, _i64, _i64, _vp, _i32, _vp, _i32, _vp, _vp, _vp, _vp, _f32]),
    "b200_add_layernorm_f16": (_i32, [_vp, _i64, _i64, _vp, _vp, _i32, _f32, _f32, _vp, _vp, _vp, _vp, _vp, _f32]),
    "b200_im2col_f16": (_i32, [_vp] + [_i64] * 14 + [_vp, _vp]),
    "b200_conv2d_f16": (_i32, [_vp] + [_i64] * 13 + [_vp, _vp, _vp, _vp, _i32, _i32]),
    "b200_conv2d_grouped_f16": (_i32, [_vp] + [_i64] * 14 + [_vp, _vp, _vp, _vp, _i32, _i32]),
    "b200_convtranspose2d_f16": (_i32, [_vp] + [_i64] * 16 + [_vp, _vp, _vp, _vp, _i32]),
    "b200_conv2d_f16_noalloc": (_i32, [_vp] + [_i64] * 13 + [_vp, _vp, _vp, _vp, _i32, _i32]),
    "b200_add_f16": (_i32, [_vp, _vp, _vp, _vp, _i64]),
    "b200_clamp_f16": (_i32, [_vp, _vp, _vp, _i64, _f32, _f32]),
    "b200_act_f16": (_i32, [_vp, _vp, _vp, _i64, _i32]),
    "b200_cast": (_i32, [_vp, _vp, _i32, _vp, _i32, _i64]),
    "b200_maxpool2d_f16": (_i32, [_vp, _i64, _i64, _i64, _i64, _vp, C.POINTER(_i64), _vp, C.POINTER(_i64)] + [_i64] * 6),
    "b200_permute4": (_i32, [_vp, _vp, _vp, C.POINTER(_i64), C.POINTER(_i64), _i32]),
    "b200_shard_range": (_i32, [_i64, _i32, _i32, _i64, C.POINTER(_i64), C.POINTER(_i64)]),
}

_lib = None


def lib() -> C.CDLL:
    """Load the library and bind every declared symbol; raises if anything is missing."""
    global _lib
    if _lib is None:
        if not os.path.exists(SO_PATH):
            raise ImportError(
                f"{SO_PATH} is missing: build it with `python -m juliavision_b200.build` "
                "(nvcc, sm_100a). There is no CPU or other-GPU fallback.")
        L = C.CDLL(SO_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)  # AttributeError if the symbol is not exported
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def last_error() -> str:
    return lib().b200_last_error().decode()


def check(rc: int) -> None:
    if rc != OK:
        raise B200Error(rc, last_error())
