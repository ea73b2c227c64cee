"""The C-ABI library loads without a GPU and exports every symbol include/b200dnn.h declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200dnn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_path():
    names = declared_symbols()
    for must in ("b200_gemm_f16", "b200_attention_f16", "b200_layernorm", "b200_conv2d_f16", "b200_ctx_create",
                 "b200_workspace_scratch", "b200_shard_range"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from juliavision_b200 import _lib
    L = ctypes.CDLL(_lib.SO_PATH)
    missing = [n for n in declared_symbols() if not hasattr(L, n)]
    assert not missing, missing


def test_binding_table_matches_header():
    from juliavision_b200 import _lib
    assert sorted(_lib.SIGNATURES) == declared_symbols()
    _lib.lib()  # binds all of them


def test_calls_without_gpu_fail_with_status_not_crash():
    import juliavision_b200 as jv
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(jv.B200Error):
        jv.Ctx(0)
    assert "CUDA" in jv._lib.last_error()


def test_supported_predicates_need_no_gpu():
    from juliavision_b200 import _lib
    L = _lib.lib()
    assert L.b200_gemm_f16_supported(3072, 4096, 768, 3072, 768, 3072, 0) == 0
    assert L.b200_gemm_f16_supported(1000, 256, 768, 1000, 768, 1000, 0) == 0       # ragged M is fine
    assert _lib.DECLINE[L.b200_gemm_f16_supported(1001, 256, 768, 1001, 768, 1001, 0)] == "wrapped"
    assert _lib.DECLINE[L.b200_gemm_f16_supported(0, 256, 768, 8, 768, 8, 0)] == "extent"
    i4 = lambda *v: (ctypes.c_int64 * 4)(*v)
    dense = lambda E, L_, H: i4(1, E, E * L_, E * L_ * H)
    assert L.b200_attention_f16_supported(64, 4096, 4096, 12, 1, dense(64, 4096, 12), dense(64, 4096, 12),
                                          dense(64, 4096, 12), 0) == 0
    # an additive mask does not decline: the fused kernel takes it (b200_attention_f16_bias)
    assert L.b200_attention_f16_supported(64, 8, 8, 1, 1, dense(64, 8, 1), dense(64, 8, 1), dense(64, 8, 1), 1) == 0
    assert L.b200_attention_f16_supported(72, 8, 8, 1, 1, dense(72, 8, 1), dense(72, 8, 1), dense(72, 8, 1), 0) == 0
    assert _lib.DECLINE[L.b200_attention_f16_supported(136, 8, 8, 1, 1, dense(136, 8, 1), dense(136, 8, 1),
                                                       dense(136, 8, 1), 0)] == "tiling"
