"""Single-kernel timing runs of the library's entry points (CUDA events on the context's stream).

    python -m juliavision_b200.microbench gemm --tokens 4096 --features 4096 --k 4096 [--epi gelu] [--reps 20]
    python -m juliavision_b200.microbench attention --batch 1 --heads 12 --seq 4096 --head-dim 64
    python -m juliavision_b200.microbench layernorm --groups 65536 --channels 1280
    python -m juliavision_b200.microbench hiera --batch 1          # whole image-encoder pass, eager launches
    python -m juliavision_b200.microbench gemv --features 51865 --k 1280 [--dtype float32]

Each run warms up, then times `reps` back-to-back calls over `--buffers` rotating operand sets
(so L2 does not keep one set resident) and prints one JSON line.  With `--reps` small this is also
the command the profiler captures are taken on.
"""
from __future__ import annotations

import argparse
import json

import numpy as np

import juliavision_b200 as jv


def _time(ctx, fn, reps, warmup=3):
    for _ in range(warmup):
        fn()
    ctx.synchronize()
    ctx.timer_start()
    for _ in range(reps):
        fn()
    return ctx.timer_stop() / reps


def gemm(ctx, a):
    rng = np.random.default_rng(a.seed)
    sets = []
    for _ in range(a.buffers):
        X = ctx.toback(np.float16(rng.standard_normal((a.tokens, a.k), dtype=np.float32) * 0.05))
        W = ctx.toback(np.float16(rng.standard_normal((a.k, a.features), dtype=np.float32) * 0.05))
        b = ctx.toback(np.float16(rng.standard_normal(a.features, dtype=np.float32) * 0.05)) if a.bias else None
        sets.append((X, W, b, ctx.allocate(np.float16, a.features, a.tokens)))
    i = [0]

    def go():
        X, W, b, o = sets[i[0] % a.buffers]
        i[0] += 1
        ctx.ws.reset()
        jv.matmul_(ctx, o, W, X, b, epi=a.epi)

    ms = _time(ctx, go, a.reps)
    flops = 2.0 * a.tokens * a.features * a.k
    plan = jv.mmplan(ctx, sets[0][3], sets[0][1], sets[0][0], sets[0][2])
    return dict(op="gemm", tokens=a.tokens, features=a.features, k=a.k, epi=a.epi, ms=round(ms, 5),
                tflops=round(flops / ms / 1e9, 1), plan=str(plan))


def attention(ctx, a):
    rng = np.random.default_rng(a.seed)
    shape = (a.batch, a.heads, a.seq, a.head_dim)
    sets = []
    for _ in range(a.buffers):
        q, k, v = (ctx.toback(np.float16(rng.standard_normal(shape, dtype=np.float32))) for _ in range(3))
        sets.append((q, k, v, ctx.allocate(np.float16, a.head_dim, a.seq, a.heads, a.batch)))
    i = [0]

    def go():
        q, k, v, o = sets[i[0] % a.buffers]
        i[0] += 1
        ctx.ws.reset()     # one op per call: a key split's partial results reuse the same scratch
        jv.sdpa(ctx, q, k, v, None, 1.0 / np.sqrt(a.head_dim), out=o)

    ms = _time(ctx, go, a.reps)
    flops = 4.0 * a.seq * a.seq * a.head_dim * a.heads * a.batch
    return dict(op="attention", batch=a.batch, heads=a.heads, seq=a.seq, head_dim=a.head_dim, ms=round(ms, 5),
                tflops=round(flops / ms / 1e9, 1))


def layernorm(ctx, a):
    rng = np.random.default_rng(a.seed)
    x = ctx.toback(np.float16(rng.standard_normal((a.groups, a.channels), dtype=np.float32)))
    o = ctx.allocate(np.float16, a.channels, a.groups)
    mean, rstd = ctx.allocate(np.float32, a.groups), ctx.allocate(np.float32, a.groups)
    g = ctx.toback(np.ones(a.channels, np.float16))
    ms = _time(ctx, lambda: jv.layernorm_(ctx, o, mean, rstd, x, g, g, a.channels, 1e-5), a.reps)
    nbytes = a.groups * a.channels * 4 + 2 * a.channels * 2 + a.groups * 8
    return dict(op="layernorm", groups=a.groups, channels=a.channels, ms=round(ms, 5), gbs=round(nbytes / ms / 1e6, 1))


def gemv(ctx, a):
    rng = np.random.default_rng(a.seed)
    dt = np.dtype(a.dtype).type
    sets = []
    for _ in range(a.buffers):
        W = ctx.toback((rng.standard_normal((a.k, a.features), dtype=np.float32) * 0.05).astype(dt))
        x = ctx.toback(rng.standard_normal((1, a.k), dtype=np.float32).astype(dt))
        sets.append((W, x, ctx.allocate(dt, a.features, 1)))
    def go():          # one call per operand set; recorded and replayed, so the host's call rate is not the figure
        for W, x, o in sets:
            ctx.ws.reset()
            jv.matmul_(ctx, o, W, x, None)

    go()
    graph = ctx.capture(go)
    ms = _time(ctx, graph.replay, max(1, a.reps // a.buffers)) / a.buffers
    nbytes = a.features * a.k * np.dtype(dt).itemsize
    return dict(op="gemv", features=a.features, k=a.k, dtype=a.dtype, ms=round(ms, 5), gbs=round(nbytes / ms / 1e6, 1))


def hiera(ctx, a):
    from .hiera import Hiera, HieraConfig
    cfg = HieraConfig()
    m = Hiera(ctx, cfg, batch=a.batch)
    rng = np.random.default_rng(a.seed)
    ctx.upload(m.image, np.float16(rng.random((a.batch, cfg.in_ch, cfg.image, cfg.image), dtype=np.float32)))
    ms = _time(ctx, m.forward, a.reps, warmup=2)
    return dict(op="hiera", batch=a.batch, ms_per_img=round(ms / a.batch, 4), tflops=round(cfg.flops(a.batch) / ms / 1e9, 1),
                launches_per_pass=m.launches_per_pass())


def main():
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="op", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--tokens", type=int, default=4096)
    g.add_argument("--features", type=int, default=4096)
    g.add_argument("--k", type=int, default=4096)
    g.add_argument("--epi", default="identity")
    g.add_argument("--bias", action="store_true")
    at = sub.add_parser("attention")
    at.add_argument("--batch", type=int, default=1)
    at.add_argument("--heads", type=int, default=12)
    at.add_argument("--seq", type=int, default=4096)
    at.add_argument("--head-dim", type=int, default=64)
    ln = sub.add_parser("layernorm")
    ln.add_argument("--groups", type=int, default=65536)
    ln.add_argument("--channels", type=int, default=1280)
    hi = sub.add_parser("hiera")
    hi.add_argument("--batch", type=int, default=1)
    gv = sub.add_parser("gemv")
    gv.add_argument("--features", type=int, default=51865)
    gv.add_argument("--k", type=int, default=1280)
    gv.add_argument("--dtype", default="float16", choices=["float16", "float32"])
    for s in (g, at, ln, hi, gv):
        s.add_argument("--reps", type=int, default=20)
        s.add_argument("--buffers", type=int, default=3)
        s.add_argument("--seed", type=int, default=0)
        s.add_argument("--device", type=int, default=0)
    a = ap.parse_args()
    with jv.Ctx(a.device) as ctx:
        print(json.dumps({"gemm": gemm, "attention": attention, "layernorm": layernorm, "hiera": hiera, "gemv": gemv}[a.op](ctx, a)), flush=True)


if __name__ == "__main__":
    main()
