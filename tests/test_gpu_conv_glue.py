import os

import numpy as np
import pytest

import juliavision_b200 as jv

from .conftest import relerr
from .gpu_helpers import describe

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")


def conv_gpu(ctx, x, w, b, stride, padding, act="identity", out_dtype=np.float16):
    """x torch (N,Cin,H,W), w torch (Cout,Cin,KH,KW); stride/padding torch (h,w) order."""
    dx, dw = ctx.toback(x), ctx.toback(w)
    db = None if b is None else ctx.toback(b)
    N, Cin, H, W = x.shape
    Cout, _, KH, KW = w.shape
    OW = jv.convsize(W, KW, stride[1], padding[1], 1)
    OH = jv.convsize(H, KH, stride[0], padding[0], 1)
    out = ctx.allocate(out_dtype, OW, OH, Cout, N)
    ctx.fill_bytes(out, 0xFF)
    ctx.ws.reset()
    jv.convolution_(ctx, out, dx, dw, db, (stride[1], stride[0]), (padding[1], padding[0]), (1, 1), 1, act=act)
    ctx.synchronize()
    return out.to_host()


def test_conv_golden(ctx):
    g = np.load(os.path.join(G, "conv.npz"))
    W, H, Cin, Cout, KW, KH, st, pd = (int(t) for t in g["geom"])
    x = np.float16(0.4 * np.sin(np.linspace(0, 9, W * H * Cin))).reshape(1, Cin, H, W)
    w = np.float16(0.3 * np.cos(np.linspace(0, 7, KW * KH * Cin * Cout))).reshape(Cout, Cin, KH, KW)
    got = conv_gpu(ctx, x, w, None, (st, st), (pd, pd), out_dtype=np.float32)
    assert relerr(got[0], g["out"]) < 5e-3, describe(got[0], g["out"], 5e-3)   # test_convtranspose_gemm.jl:154-200


# (W,H,Cin,Cout,KW,KH,s,p): the reference's CRS-padding cases plus the Hiera stem geometry at 256^2
@pytest.mark.parametrize("W,H,Cin,Cout,KW,KH,s,p", [(64, 64, 5, 32, 3, 3, 1, 1), (48, 48, 7, 48, 5, 5, 2, 2),
                                                     (32, 32, 32, 64, 3, 3, 1, 1), (256, 256, 3, 112, 7, 7, 4, 3),
                                                     (30, 22, 4, 24, 3, 3, 1, 1)])
def test_conv_vs_oracle(ctx, ora, W, H, Cin, Cout, KW, KH, s, p):
    rng = np.random.default_rng(W + Cin + Cout)
    x = np.float16(rng.standard_normal((2, Cin, H, W)) * 0.5)
    w = np.float16(rng.standard_normal((Cout, Cin, KH, KW)) * 0.1)
    b = np.float16(rng.standard_normal(Cout) * 0.1)
    got = conv_gpu(ctx, x, w, b, (s, s), (p, p), act="relu")
    ref = ora.conv2d(x, w, b, (s, s), (p, p), (1, 1), epi="relu")
    assert got.shape == ref.shape
    assert relerr(got, ref) < 5e-3, describe(got, ref, 5e-3)


@pytest.mark.parametrize("W,H,Cin,Cout", [(64, 64, 144, 256), (32, 32, 32, 48), (16, 24, 8, 8)])
def test_conv_1x1_is_a_gemm(ctx, ora, W, H, Cin, Cout):
    rng = np.random.default_rng(W * Cin)
    x = np.float16(rng.standard_normal((1, Cin, H, W)) * 0.5)
    w = np.float16(rng.standard_normal((Cout, Cin, 1, 1)) * 0.1)
    b = np.float16(rng.standard_normal(Cout) * 0.1)
    got = conv_gpu(ctx, x, w, b, (1, 1), (0, 0))
    ref = ora.conv2d(x, w, b)
    assert relerr(got, ref) < 5e-3, describe(got, ref, 5e-3)


def test_im2col_bit_exact(ctx, ora):
    import ctypes as C
    from juliavision_b200 import _lib
    rng = np.random.default_rng(3)
    x = np.float16(rng.standard_normal((2, 5, 20, 24)))
    N, Cin, H, W = x.shape
    KH = KW = 3
    OW, OH = jv.convsize(W, KW, 2, 1, 1), jv.convsize(H, KH, 2, 1, 1)
    NPQ, CRS = OW * OH * N, KW * KH * Cin
    MP, CRSP = (NPQ + 15) // 16 * 16, (CRS + 15) // 16 * 16
    col = ctx.allocate(np.float16, MP, CRSP)
    ctx.fill_bytes(col, 0xFF)
    _lib.check(_lib.lib().b200_im2col_f16(ctx.handle, W, H, Cin, N, KW, KH, 2, 2, 1, 1, 1, 1, MP, CRSP,
                                          ctx.toback(x).ptr, col.ptr))
    ctx.synchronize()
    assert np.array_equal(col.to_host(), ora.im2col(x, KH, KW, (2, 2), (1, 1), (1, 1), MP, CRSP))


def test_glue_bit_exact(ctx, ora):
    rng = np.random.default_rng(4)
    for n in (1, 7, 8, 1000, 1500 * 1280 + 3):
        a = np.float16(rng.standard_normal(n) * 4)
        b = np.float16(rng.standard_normal(n) * 4)
        da, db, do = ctx.toback(a), ctx.toback(b), ctx.allocate(np.float16, n)
        jv.add_(ctx, do, da, db)
        assert np.array_equal(do.to_host(), ora.add(a, b))
        jv.clamp_(ctx, do, da, -1.5, 2.25)
        assert np.array_equal(do.to_host(), ora.clamp(a, -1.5, 2.25))
        jv.act_(ctx, do, da, "relu")
        assert np.array_equal(do.to_host(), ora.act(a, "relu"))
        jv.act_(ctx, do, da, "gelu")
        ref = ora.act(a, "gelu")
        d = np.abs(do.to_host().astype(np.float32) - ref.astype(np.float32))
        assert np.all(d <= np.spacing(np.abs(ref)).astype(np.float32) + 1e-7)   # fast exp: one fp16 ulp at most


def test_permute_bit_exact(ctx):
    rng = np.random.default_rng(5)
    a = np.float16(rng.standard_normal((2, 37, 5, 24)))         # torch (B,L,H,E) -> device (E,H,L,B)
    d = ctx.toback(a)
    v = d.permute((0, 2, 1, 3))                                  # (E,L,H,B) view
    assert np.array_equal(ctx.contiguous(v).to_host(), a.transpose(0, 2, 1, 3))
    t = d.permute((2, 0, 1, 3))                                  # (L,E,H,B): source contiguous along output axis 1
    assert np.array_equal(ctx.contiguous(t).to_host(), a.transpose(0, 2, 3, 1))
    f = np.float32(rng.standard_normal((3, 4, 50, 33)))
    df = ctx.toback(f)
    assert np.array_equal(ctx.contiguous(df.permute((1, 0, 3, 2))).to_host(), f.transpose(1, 0, 3, 2))
    # axis 0 kept in front: 16-byte pieces when its extent and the strides allow, element by element when not
    for shape, dt in (((4, 9, 6, 64), np.float16), ((2, 5, 7, 20), np.float16), ((3, 6, 5, 8), np.float32), ((2, 3, 4, 6), np.float32)):
        g = rng.standard_normal(shape).astype(dt)
        dg = ctx.toback(g)
        assert np.array_equal(ctx.contiguous(dg.permute((0, 2, 1, 3))).to_host(), g.transpose(0, 2, 1, 3))
        assert np.array_equal(ctx.contiguous(dg.permute((0, 3, 2, 1))).to_host(), g.transpose(2, 1, 0, 3))


def test_pool_and_workspace(ctx):
    from juliavision_b200 import _lib
    import ctypes as C
    ctx.ws.reset()
    a = ctx.scratch(np.float16, 1000)
    b = ctx.scratch(np.float32, 10)
    assert a.ptr % 256 == 0 and b.ptr % 256 == 0 and b.ptr >= a.ptr + 2000     # workspace.jl:63-66
    used, cap, retired = ctx.ws.stats()
    assert cap >= 1 << 20                                                      # min 1 MiB (workspace.jl:85)
    big = ctx.scratch(np.uint8, cap + 5)                                       # forces a grow: old block retired
    assert ctx.ws.stats()[2] == 1 and ctx.ws.stats()[1] >= int(1.5 * (cap + 5)) - 512
    ctx.ws.reset()
    assert ctx.ws.stats()[0] == 0 and ctx.ws.stats()[2] == 0
    def reserved():
        use, res = C.c_size_t(), C.c_size_t()
        _lib.check(_lib.lib().b200_pool_stats(ctx.handle, C.byref(use), C.byref(res)))
        return res.value
    x = ctx.allocate(np.float32, 1024)
    assert x.ptr % 256 == 0
    before = reserved()
    del x
    y = ctx.allocate(np.float32, 1024)                                         # a freed block of the size class is reused:
    assert reserved() == before                                                # nothing new is taken from the driver
    with pytest.raises(jv.B200Error):
        _lib.check(_lib.lib().b200_pool_free(ctx.handle, C.c_void_p(12345)))


# (N, Cin, H, W, Cout, KH, KW, stride, padding, dilation, groups) in torch order
GROUPED = [(2, 16, 20, 24, 32, 3, 3, (1, 1), (1, 1), (1, 1), 2),     # aligned slices: tensor-core GEMM per group
           (1, 6, 9, 8, 8, 3, 3, (2, 1), (1, 1), (1, 1), 2),         # unaligned slices: the scalar GEMM
           (2, 8, 12, 12, 8, 3, 3, (1, 1), (1, 1), (1, 1), 8),       # depthwise
           (1, 32, 16, 16, 64, 1, 1, (1, 1), (0, 0), (1, 1), 4)]     # grouped 1x1: no gather


@pytest.mark.parametrize("N,Cin,H,W,Cout,KH,KW,stride,padding,dilation,groups", GROUPED)
def test_grouped_conv_vs_oracle(ctx, ora, N, Cin, H, W, Cout, KH, KW, stride, padding, dilation, groups):
    """conv2d with GROUPS > 1 (conv.jl:26-51): every group lowered like the ungrouped convolution."""
    rng = np.random.default_rng(Cin * 13 + groups)
    x = np.float16(rng.standard_normal((N, Cin, H, W)) * 0.5)
    w = np.float16(rng.standard_normal((Cout, Cin // groups, KH, KW)) * 0.2)
    b = np.float16(rng.standard_normal(Cout) * 0.2)
    ref = ora.conv2d_grouped(x, w, b, stride, padding, dilation, groups, epi="relu")
    out = ctx.allocate(np.float16, ref.shape[3], ref.shape[2], Cout, N)
    ctx.fill_bytes(out, 0xFF)
    ctx.ws.reset()
    jv.convolution_(ctx, out, ctx.toback(x), ctx.toback(w), ctx.toback(b), stride[::-1], padding[::-1], dilation[::-1],
                    groups, act="relu")
    ctx.synchronize()
    got = out.to_host()
    assert np.all(np.isfinite(got))
    assert relerr(got, ref) < 5e-3, describe(got, ref, 5e-3)


# (N, Cin, H, W, Cout, KH, KW, stride, padding, dilation, output_padding, groups)
TRANSPOSED = [(1, 64, 16, 16, 32, 2, 2, (2, 2), (0, 0), (1, 1), (0, 0), 1),      # SAM 2's upsampler: shufflecase -> GEMM
              (2, 24, 9, 7, 16, 2, 3, (2, 3), (0, 0), (1, 1), (0, 0), 1),        # shufflecase, odd extents, two images
              (2, 4, 5, 6, 6, 3, 2, (2, 3), (1, 0), (1, 2), (1, 1), 2),          # grouped, padded, dilated, output padding
              (1, 8, 10, 10, 8, 3, 3, (1, 1), (1, 1), (1, 1), (0, 0), 8),        # depthwise (Kokoro's upsampler form)
              (1, 16, 8, 8, 8, 4, 4, (2, 2), (1, 1), (1, 1), (0, 0), 1)]         # overlapping receptive fields: the gather


@pytest.mark.parametrize("N,Cin,H,W,Cout,KH,KW,stride,padding,dilation,outpad,groups", TRANSPOSED)
def test_transposed_conv_vs_oracle(ctx, ora, N, Cin, H, W, Cout, KH, KW, stride, padding, dilation, outpad, groups):
    """convolutiontranspose! (conv.jl:247-290): the GEMM + shuffle route where the receptive fields tile the output,
    the deterministic gather elsewhere; both against the oracle's gather (conv.jl:147-190)."""
    rng = np.random.default_rng(Cin * 7 + Cout)
    x = np.float16(rng.standard_normal((N, Cin, H, W)) * 0.5)
    w = np.float16(rng.standard_normal((Cin, Cout // groups, KH, KW)) * 0.2)
    b = np.float16(rng.standard_normal(Cout) * 0.2)
    for out_dtype in (np.float16, np.float32):
        ref = ora.convtranspose2d(x, w, b, stride, padding, dilation, outpad, groups, out_dtype=np.float32)
        out = ctx.allocate(out_dtype, ref.shape[3], ref.shape[2], Cout, N)
        ctx.fill_bytes(out, 0xFF)
        ctx.ws.reset()
        dw = ctx.toback(w)
        assert jv.shufflecase(dw, stride[::-1], padding[::-1], dilation[::-1], outpad[::-1], groups) == \
            (groups == 1 and (KH, KW) == stride and padding == (0, 0) and outpad == (0, 0) and dilation == (1, 1))
        jv.convolutiontranspose_(ctx, out, ctx.toback(x), dw, ctx.toback(b), stride[::-1], padding[::-1], dilation[::-1],
                                 outpad[::-1], groups)
        ctx.synchronize()
        got = out.to_host()
        assert got.shape == ref.shape and np.all(np.isfinite(got))
        assert relerr(got, ref) < 5e-3, describe(got, ref, 5e-3)
