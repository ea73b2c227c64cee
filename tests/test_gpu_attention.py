import os

import numpy as np
import pytest

import juliavision_b200 as jv

from .conftest import relerr
from .gpu_helpers import attention_gpu, describe

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")
TOL = 5e-3  # the reference's fused-attention gate: max|d|/max|ref| (test_flash.jl:142,204)


def test_golden(ctx):
    g = np.load(os.path.join(G, "attention.npz"))
    got, plan = attention_gpu(ctx, g["q"], g["k"], g["v"], float(g["scale"]), out_dtype=np.float32)
    assert isinstance(plan, jv.FlashTCPlan)
    assert relerr(got, g["out"]) < TOL, describe(got, g["out"], TOL)


# torch (B,H,Lq,Lk,E); covers the reference's test shapes that fit E <= 64 (test_flash.jl:36,189-190),
# the Whisper shape's ragged 1500 and the Hiera head dim 56
SHAPES = [(1, 4, 128, 128, 64), (1, 1, 64, 64, 64), (2, 2, 256, 256, 64), (1, 8, 23, 4096, 16),
          (1, 8, 23, 23, 32), (1, 8, 4096, 23, 16), (1, 4, 23, 17, 16), (1, 3, 1500, 1500, 64),
          (3, 2, 300, 200, 56), (1, 2, 129, 257, 8), (1, 1, 1, 1, 64)]


@pytest.mark.parametrize("B,H,Lq,Lk,E", SHAPES)
@pytest.mark.parametrize("out_dtype", [np.float16, np.float32])
def test_vs_oracle(ctx, ora, B, H, Lq, Lk, E, out_dtype):
    rng = np.random.default_rng(B * 1000 + H * 100 + Lq + Lk + E)
    q = np.float16(rng.standard_normal((B, H, Lq, E)))
    k = np.float16(rng.standard_normal((B, H, Lk, E)))
    v = np.float16(rng.standard_normal((B, H, Lk, E)))
    scale = 1 / np.sqrt(E)
    got, plan = attention_gpu(ctx, q, k, v, scale, out_dtype)
    assert isinstance(plan, jv.FlashTCPlan), plan
    assert got.shape == (B, H, Lq, E) and got.dtype == out_dtype
    ref = ora.attention_ref(q, k, v, scale)
    assert np.max(np.abs(got)) > 1e-3
    assert relerr(got, ref) < TOL, describe(got, ref, TOL)
    # and within the stated tolerance of the runtime's own unfused decomposition
    tp = ora.attention_threepass(q, k, v, scale)
    assert relerr(got, tp) < 1e-2, describe(got, tp, 1e-2)


def test_interleaved_heads(ctx, ora):
    """Operands as the projections leave them: (E,H,L,B) memory viewed as (E,L,H,B); fused qkv."""
    rng = np.random.default_rng(11)
    B, L, H, E = 2, 200, 5, 64
    buf = np.float16(rng.standard_normal((B, L, 3, H, E)))
    q, k, v = (buf[:, :, i].transpose(0, 2, 1, 3) for i in range(3))
    got, plan = attention_gpu(ctx, q, k, v, 0.125)
    assert isinstance(plan, jv.FlashTCPlan)
    ref = ora.attention_ref(q, k, v, 0.125)
    assert relerr(got, ref) < TOL, describe(got, ref, TOL)


def test_token_major_output_view(ctx, ora):
    """out given as an (E,L,H,B) view of a token-major buffer: the permute copy after sdpa is folded
    into the store; values are those of the dense call."""
    from .gpu_helpers import qkv_views
    rng = np.random.default_rng(13)
    B, H, L, E = 2, 5, 200, 64
    q, k, v = (np.float16(rng.standard_normal((B, H, L, E))) for _ in range(3))
    dq, dk, dv = qkv_views(ctx, q, k, v)
    dense, _ = attention_gpu(ctx, q, k, v, 0.125)
    buf = ctx.allocate(np.float16, E * H, L, B)                     # torch (B, L, H*E)
    ctx.fill_bytes(buf, 0xFF)
    view = jv.DeviceArray(ctx, buf.ptr, np.float16, (E, L, H, B), (1, E * H, E, E * H * L), owner=buf)
    jv.sdpa(ctx, dq, dk, dv, None, 0.125, out=view)
    ctx.synchronize()
    got = buf.to_host().reshape(B, L, H, E).transpose(0, 2, 1, 3)
    assert np.array_equal(got, dense)


# (E, Lq, Lk, H, B): the reference's own fused tiling and its tests are at head dim 72 (test_flash.jl:36,
# 189-190, 221; FLASHCM_TILINGS flash.jl:1149-1157), SAM 2's windowed shape is (72,256,256,8,16)
# (tools/attn_lab.jl:11-14); 80/96/104/128 cover the rest of the two-atom range
WIDE = [(72, 64, 64, 1, 1), (72, 128, 128, 2, 1), (72, 256, 256, 2, 1), (72, 128, 256, 2, 2), (72, 64, 4096, 2, 1),
        (72, 256, 256, 8, 16), (72, 1000, 700, 3, 2), (80, 300, 300, 2, 1), (96, 257, 129, 1, 2), (104, 130, 513, 2, 1),
        (128, 384, 384, 2, 1), (128, 23, 4096, 4, 1)]


@pytest.mark.parametrize("E,Lq,Lk,H,B", WIDE)
def test_head_dims_above_one_swizzle_row_run_on_the_tensor_cores(ctx, ora, E, Lq, Lk, H, B):
    """Head dims 72..128: two swizzle atoms along E, one query tile per CTA; same contract and tolerance
    as the narrow kernel, ragged query/key tails and the few-queries key split included."""
    rng = np.random.default_rng(E * 7 + Lq + Lk)
    q = np.float16(rng.standard_normal((B, H, Lq, E)) * 0.2)
    k = np.float16(rng.standard_normal((B, H, Lk, E)) * 0.2)
    v = np.float16(rng.standard_normal((B, H, Lk, E)) * 0.2)
    scale = 1 / np.sqrt(E)
    for out_dtype in (np.float32, np.float16):
        got, plan = attention_gpu(ctx, q, k, v, scale, out_dtype)
        assert isinstance(plan, jv.FlashTCPlan), plan
        assert np.all(np.isfinite(got))
        ref = ora.attention_ref(q, k, v, scale)
        assert np.max(np.abs(got)) > 1e-3
        assert relerr(got, ref) < TOL, describe(got, ref, TOL)


def test_sam2_global_shape_head_dim_72_sampled_rows(ctx, ora):
    """(E72, L4096, H8, B1), the global-attention shape of the reference's flagship encoder
    (tools/attn_lab.jl:11-14), checked on sampled query rows against the fp32 reference."""
    rng = np.random.default_rng(72)
    B, H, L, E = 1, 8, 4096, 72
    q, k, v = (np.float16(rng.standard_normal((B, H, L, E)) * 0.5) for _ in range(3))
    scale = 1 / np.sqrt(E)
    got, plan = attention_gpu(ctx, q, k, v, scale)
    assert isinstance(plan, jv.FlashTCPlan)
    rows = np.unique(np.concatenate([np.arange(0, L, 97), [127, 128, 255, 256, L - 1]]))
    ref = ora.attention_ref(q[:, :, rows], k, v, scale)
    assert relerr(got[:, :, rows], ref) < TOL, describe(got[:, :, rows], ref, TOL)


# (B, H, Lq, Lk, E), mask shape or None: head dims past the fused kernel's run as two batched GEMMs and a softmax
TWO_GEMM = [((1, 2, 300, 264, 256), None), ((2, 3, 128, 512, 136), None), ((1, 2, 100, 77, 160), None),   # Lk = 77: unaligned scores
            ((2, 2, 200, 200, 192), (2, 1, 200, 200)), ((1, 4, 1030, 520, 256), None)]


@pytest.mark.parametrize("shape,bshape", TWO_GEMM)
def test_head_dims_above_128_run_as_two_gemms_and_a_softmax(ctx, ora, shape, bshape):
    """sdpa_coopmat! + attn_softmax_rows! (attention.jl:528-705): S = Kt Q in fp32, P = softmax over the keys in fp16,
    O = V P; against the fp32 reference at the fused kernel's tolerance and the three-pass form at 1e-2; with and
    without the additive mask (whose all-blocked rows come out as zeros)."""
    B, H, Lq, Lk, E = shape
    rng = np.random.default_rng(sum(shape))
    q = np.float16(rng.standard_normal((B, H, Lq, E)) * 0.3)
    k = np.float16(rng.standard_normal((B, H, Lk, E)) * 0.3)
    v = np.float16(rng.standard_normal((B, H, Lk, E)) * 0.3)
    bias = None
    if bshape is not None:
        bias = np.float16(rng.standard_normal(bshape))
        bias[rng.random(bshape) < 0.3] = -np.inf
        bias[:, :, 5, :] = -np.inf
    scale = 1 / np.sqrt(E)
    for out_dtype in (np.float16, np.float32):
        got, plan = attention_gpu(ctx, q, k, v, scale, out_dtype, bias=bias)
        assert isinstance(plan, jv.TwoGemmPlan), plan
        assert np.all(np.isfinite(got))
        ref = ora.attention_ref(q, k, v, scale, bias=bias)
        assert relerr(got, ref) < TOL, describe(got, ref, TOL)
        if bias is not None:
            assert np.all(got[:, :, 5] == 0)


def test_two_gemm_route_with_heads_interleaved_in_the_token_row(ctx, ora):
    """q, k, v as views of one (tokens, 3 d) projection and the result token-major: the head and batch strides do not
    fold into one, so the route runs one batched launch per image; values are those of the dense call."""
    from .gpu_helpers import qkv_views
    rng = np.random.default_rng(77)
    B, H, L, E = 2, 2, 160, 136
    d = H * E
    qkv = np.float16(rng.standard_normal((B, L, 3, H, E)) * 0.3)
    q, k, v = (qkv[:, :, i].transpose(0, 2, 1, 3) for i in range(3))     # (B, H, L, E) strided views
    dq, dk, dv = qkv_views(ctx, q, k, v)
    assert isinstance(jv.sdpaplan(ctx, dq, dk, dv), jv.TwoGemmPlan)
    buf = ctx.allocate(np.float16, d, L, B)
    ctx.fill_bytes(buf, 0xFF)
    view = jv.DeviceArray(ctx, buf.ptr, np.float16, (E, L, H, B), (1, d, E, d * L), owner=buf)
    jv.sdpa(ctx, dq, dk, dv, None, 1 / np.sqrt(E), out=view)
    ctx.synchronize()
    got = buf.to_host().reshape(B, L, H, E).transpose(0, 2, 1, 3)
    ref = ora.attention_ref(np.ascontiguousarray(q), np.ascontiguousarray(k), np.ascontiguousarray(v), 1 / np.sqrt(E))
    assert relerr(got, ref) < TOL, describe(got, ref, TOL)


def test_head_dim_not_a_multiple_of_eight_takes_the_scalar_kernel(ctx, ora):
    rng = np.random.default_rng(12)
    q, k, v = (np.float16(rng.standard_normal((1, 2, 64, 132)) * 0.2) for _ in range(3))
    got, plan = attention_gpu(ctx, q, k, v, 1 / np.sqrt(132), np.float32)
    assert isinstance(plan, jv.AttnScalarPlan)
    assert relerr(got, ora.attention_ref(q, k, v, 1 / np.sqrt(132))) < TOL


# torch (B,H,Lq,Lk,E) and the bias shape as torch (B|1, H|1, Lq|1, Lk|1)
BIAS_CASES = [((2, 3, 256, 384, 64), (2, 3, 256, 384)),    # full mask, rows read 8 keys at a time
              ((2, 3, 300, 200, 56), (2, 3, 300, 200)),    # ragged keys: the guarded scalar reads
              ((2, 4, 256, 256, 64), (2, 1, 1, 256)),      # key-padding mask broadcast over heads and queries
              ((1, 2, 130, 257, 32), (1, 1, 130, 257)),    # broadcast over heads, odd row stride
              ((1, 2, 64, 64, 72), (1, 2, 64, 64)),        # head dim past one swizzle row: two atoms along E
              ((2, 2, 300, 260, 96), (2, 1, 300, 260)),
              ((1, 1, 40, 40, 132), (1, 1, 40, 40))]       # not a multiple of 8: scalar kernel


@pytest.mark.parametrize("shape,bshape", BIAS_CASES)
def test_additive_bias_vs_oracle(ctx, ora, shape, bshape):
    """The additive mask of the mem-efficient variant (attention.jl:55-59), which the reference runs
    unfused: random finite values, -inf on a share of the keys, and some rows blocked entirely."""
    B, H, Lq, Lk, E = shape
    rng = np.random.default_rng(sum(shape) + sum(bshape))
    q = np.float16(rng.standard_normal((B, H, Lq, E)))
    k = np.float16(rng.standard_normal((B, H, Lk, E)))
    v = np.float16(rng.standard_normal((B, H, Lk, E)))
    bias = np.float16(rng.standard_normal(bshape))
    bias[rng.random(bshape) < 0.3] = -np.inf
    if bshape[2] > 1:
        bias[:, :, 5, :] = -np.inf            # a query every key is hidden from
        bias[:, :, bshape[2] - 1, : Lk // 2] = -np.inf
    scale = 1 / np.sqrt(E)
    for out_dtype in (np.float16, np.float32):
        got, plan = attention_gpu(ctx, q, k, v, scale, out_dtype, bias=bias)
        assert isinstance(plan, jv.FlashTCPlan if E <= 128 else jv.AttnScalarPlan), plan
        assert np.all(np.isfinite(got))
        ref = ora.attention_ref(q, k, v, scale, bias=bias)
        assert relerr(got, ref) < TOL, describe(got, ref, TOL)
        if bshape[2] > 1:
            assert np.all(got[:, :, 5] == 0)   # all keys blocked: a zero row (attention.jl:73-100)
        tp = ora.attention_threepass(q, k, v, scale, bias=bias)
        assert relerr(got, tp) < 1e-2, describe(got, tp, 1e-2)


def test_zero_bias_changes_nothing(ctx):
    rng = np.random.default_rng(5)
    q, k, v = (np.float16(rng.standard_normal((1, 2, 256, 64))) for _ in range(3))
    plain, _ = attention_gpu(ctx, q, k, v, 0.125)
    masked, _ = attention_gpu(ctx, q, k, v, 0.125, bias=np.zeros((1, 1, 256, 256), np.float16))
    assert relerr(masked, plain) < 1e-3


def test_declines(ctx):
    q = ctx.allocate(np.float16, 64, 128, 2, 1)
    assert jv.sdpaplan(ctx, q, q, q, bias=q) == jv.Decline("bias")          # a mask that does not broadcast
    q32 = ctx.allocate(np.float32, 64, 128, 2, 1)
    assert jv.sdpaplan(ctx, q32, q32, q32) == jv.Decline("eltype")
    k = ctx.allocate(np.float16, 32, 128, 2, 1)
    assert jv.sdpaplan(ctx, q, k, k) == jv.Decline("extent")
    with pytest.raises(jv.B200Error):
        jv.sdpa(ctx, q, q, q, bias=q)


def test_config2_properties_at_full_size(ctx):
    """BASELINE config 2 (B1 H12 L4096 E64). Size-independent checks: V = 1 gives exactly-normalised
    rows, attention is linear in V, and permuting the keys (with their values) changes nothing
    beyond rounding."""
    rng = np.random.default_rng(20260102)
    B, H, L, E = 1, 12, 4096, 64
    q = np.float16(rng.standard_normal((B, H, L, E)))
    k = np.float16(rng.standard_normal((B, H, L, E)))
    v = np.float16(rng.standard_normal((B, H, L, E)))
    ones = np.ones_like(v)
    o1, _ = attention_gpu(ctx, q, k, ones, 0.125, np.float32)
    assert np.max(np.abs(o1 - 1)) < 2e-3
    ov, _ = attention_gpu(ctx, q, k, v, 0.125, np.float32)
    o2v, _ = attention_gpu(ctx, q, k, np.float16(2) * v, 0.125, np.float32)
    assert np.max(np.abs(o2v - 2 * ov)) < 1e-5 * max(1.0, float(np.max(np.abs(ov))))
    perm = rng.permutation(L)
    op, _ = attention_gpu(ctx, q, k[:, :, perm], v[:, :, perm], 0.125, np.float32)
    assert relerr(op, ov) < TOL


def test_config2_sample_rows_vs_oracle(ctx, ora):
    """Config 2 at full key length, checked against the oracle on a sample of query rows."""
    rng = np.random.default_rng(20260103)
    B, H, L, E = 1, 12, 4096, 64
    q, k, v = (np.float16(rng.standard_normal((B, H, L, E))) for _ in range(3))
    got, _ = attention_gpu(ctx, q, k, v, 0.125)
    rows = np.sort(rng.choice(L, 64, replace=False))
    ref = ora.attention_ref(np.ascontiguousarray(q[:, :, rows]), k, v, 0.125)
    assert relerr(got[:, :, rows], ref) < TOL, describe(got[:, :, rows], ref, TOL)


@pytest.mark.parametrize("B,H,Lq,Lk,E", [(512, 2, 64, 64, 56), (1024, 4, 16, 64, 56), (300, 2, 64, 64, 64), (256, 2, 49, 49, 32),
                                         (200, 3, 100, 40, 8), (400, 1, 1, 64, 16), (310, 1, 23, 1, 24), (150, 2, 129, 64, 48),
                                         (16, 8, 256, 256, 56), (40, 2, 64, 256, 56), (64, 3, 130, 200, 64), (90, 2, 17, 65, 16)])
def test_many_small_windows(ctx, ora, B, H, Lq, Lk, E):
    """Attention windows of a few dozen tokens, token-major with the windows back to back (what the image
    encoder hands over): many of them take the small-tile kernel (64 queries of one window and head per
    CTA).  Values must be those of independent windows: checked against the oracle window by window, and
    a window's result must not change when its neighbours do."""
    from .gpu_helpers import qkv_views
    rng = np.random.default_rng(B + Lq + Lk)
    qb = np.float16(rng.standard_normal((B, Lq, H, E)))
    kb = np.float16(rng.standard_normal((B, Lk, H, E)))
    vb = np.float16(rng.standard_normal((B, Lk, H, E)))
    q, k, v = (t.transpose(0, 2, 1, 3) for t in (qb, kb, vb))            # torch (B,H,L,E) views
    scale = 1 / np.sqrt(E)

    def run(q, k, v):
        dq, dk, dv = qkv_views(ctx, q, k, v)
        buf = ctx.allocate(np.float16, E * H, Lq, B)                      # torch (B, Lq, H*E)
        ctx.fill_bytes(buf, 0xFF)
        view = jv.DeviceArray(ctx, buf.ptr, np.float16, (E, Lq, H, B), (1, E * H, E, E * H * Lq), owner=buf)
        jv.sdpa(ctx, dq, dk, dv, None, scale, out=view)
        ctx.synchronize()
        return buf.to_host().reshape(B, Lq, H, E).transpose(0, 2, 1, 3)

    got = run(q, k, v)
    ref = ora.attention_ref(q, k, v, scale)
    assert np.all(np.isfinite(got))
    assert relerr(got, ref) < TOL, describe(got, ref, TOL)
    kb2, vb2 = kb.copy(), vb.copy()
    kb2[1::2] = np.float16(rng.standard_normal(kb2[1::2].shape) * 3)       # disturb every other window
    vb2[1::2] = 7
    got2 = run(q, kb2.transpose(0, 2, 1, 3), vb2.transpose(0, 2, 1, 3))
    assert np.array_equal(got2[0::2], got[0::2])


@pytest.mark.parametrize("B,H,Lq,Lk,E", [(512, 2, 64, 64, 56), (300, 1, 70, 33, 40)])
def test_many_small_windows_dense_fp32_out(ctx, ora, B, H, Lq, Lk, E):
    """The same windows from dense (B,H,L,E) arrays into an fp32 result (the attn_flash! contract)."""
    from .gpu_helpers import qkv_views
    rng = np.random.default_rng(B + Lq + Lk + 1)
    q = np.float16(rng.standard_normal((B, H, Lq, E)))
    k = np.float16(rng.standard_normal((B, H, Lk, E)))
    v = np.float16(rng.standard_normal((B, H, Lk, E)))
    scale = 1 / np.sqrt(E)
    dq, dk, dv = qkv_views(ctx, q, k, v)
    out = ctx.allocate(np.float32, E, Lq, H, B)
    ctx.fill_bytes(out, 0xFF)
    jv.sdpa(ctx, dq, dk, dv, None, scale, out=out)
    ctx.synchronize()
    got = out.to_host()
    ref = ora.attention_ref(q, k, v, scale)
    assert np.all(np.isfinite(got))
    assert relerr(got, ref) < TOL, describe(got, ref, TOL)


@pytest.mark.parametrize("B,H,Lq,Lk,E", [(1, 8, 23, 4096, 64), (2, 3, 1, 4000, 56), (1, 1, 300, 2048, 32), (1, 20, 130, 1500, 64),
                                         (1, 20, 2000, 2000, 64),     # 160 query pairs: the 12 of the last wave are cut, one of them ragged
                                         (1, 39, 1000, 700, 40)])      # 156 pairs, 8 cut three ways, ragged queries and keys
def test_few_queries_many_keys_split_and_merged(ctx, ora, B, H, Lq, Lk, E):
    """Decode-like shapes (flash.jl:298-323: Lq = 23, Lk = 4096): the keys are split over several CTAs
    per query tile and merged (attn_flash_cm_merge!); the values are those of the unsplit computation."""
    rng = np.random.default_rng(Lq + Lk + E)
    q = np.float16(rng.standard_normal((B, H, Lq, E)))
    k = np.float16(rng.standard_normal((B, H, Lk, E)))
    v = np.float16(rng.standard_normal((B, H, Lk, E)))
    k[:, :, Lk // 2] *= 4          # a late key that moves the running maximum of some rows
    scale = 1 / np.sqrt(E)
    ref = ora.attention_ref(q, k, v, scale)
    for out_dtype in (np.float16, np.float32):
        got, plan = attention_gpu(ctx, q, k, v, scale, out_dtype)
        assert isinstance(plan, jv.FlashTCPlan)
        assert relerr(got, ref) < TOL, describe(got, ref, TOL)
