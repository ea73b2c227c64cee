"""The encoder stack composed from the CPU oracle's ops (test infrastructure, not product):
the checker for juliavision_b200.encoder.Encoder and the body of the timed CPU baseline."""
from math import sqrt
from typing import List, Optional

import numpy as np

from . import oracle as ora

F16_MAX = 65504.0


def oracle_forward(cfg, weights: List[dict], x: np.ndarray, layers: Optional[int] = None):
    """The same stack on the CPU oracle (test/bench checker only). x: torch (tokens, d_model) fp16."""
    H, E = cfg.heads, cfg.head_dim
    L = x.shape[0]
    x = x.astype(np.float16)
    n = cfg.layers if layers is None else layers
    for w in weights[:n]:
        h, _, _ = ora.layernorm(x, w["ln1_g"], w["ln1_b"], cfg.eps)
        q = ora.linear(h, np.ascontiguousarray(w["wq"].T), w["bq"])
        k = ora.linear(h, np.ascontiguousarray(w["wk"].T), None)
        v = ora.linear(h, np.ascontiguousarray(w["wv"].T), w["bv"])
        heads = lambda t: t.reshape(1, L, H, E).transpose(0, 2, 1, 3)       # (B,H,L,E) strided view
        att = ora.attention_threepass(heads(q), heads(k), heads(v), 1.0 / sqrt(E), out_dtype=np.float16)
        att_t = np.ascontiguousarray(att.transpose(0, 2, 1, 3)).reshape(L, H * E)
        o = ora.linear(att_t, np.ascontiguousarray(w["wo"].T), w["bo"])
        x = ora.add(x, o)
        h, _, _ = ora.layernorm(x, w["ln2_g"], w["ln2_b"], cfg.eps)
        ff = ora.linear(h, np.ascontiguousarray(w["w1"].T), w["b1"], epi="gelu")
        g = ora.linear(ff, np.ascontiguousarray(w["w2"].T), w["b2"])
        x = ora.add(x, g)
        if cfg.clamp:
            x = ora.clamp(x, -F16_MAX, F16_MAX)
    if n == cfg.layers:
        x, _, _ = ora.layernorm(x, weights[-1]["lnf_g"], weights[-1]["lnf_b"], cfg.eps)
    return x
