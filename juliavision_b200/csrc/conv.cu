// Convolution lowered to the tensor-core GEMM: an im2col gather (skipped for 1x1/stride-1/
// unpadded kernels, where the image already is the GEMM operand), then one GEMM per image
// with the per-channel bias and the activation fused in its store, written straight into
// out (OW,OH,Cout,N).  Replaces im2col_kernel! + Lava.coopmat_gemm! into fp32 planes +
// conv_epilogue_kernel! (reference kernels/extern/conv_coopmat.jl:246-392) and the 1x1
// route through matmul! (kernels/extern/conv.jl:122-131).
#include <cuda_fp16.h>

#include "internal.h"

namespace b200 {

// col (MP, CRSP) column-major: a thread produces eight consecutive rows m of one column c (one
// 16-byte store), so the column's (kw, kh, cin) is decomposed once per eight elements and the pixel
// index advances incrementally; neighbouring threads take neighbouring m, so the stores coalesce.
// Index math is 32-bit on purpose: every extent is far inside int32 and 64-bit division
// is emulated (same observation as the reference, conv_coopmat.jl:238-245).  MP is a multiple of 8.
__global__ void __launch_bounds__(256)
im2col_f16_kernel(__half* __restrict__ col, const __half* __restrict__ x, int MP, int CRSP, int KW, int KH,
                  int sx, int sy, int px, int py, int dx, int dy, int Wid, int Hei, int OW, int OH, int NPQ,
                  int Cin, int64_t ntot8) {
    const int MP8 = MP >> 3;
    for (int64_t lin = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; lin < ntot8;
         lin += (int64_t)gridDim.x * blockDim.x) {
        const int m0 = (int)(lin % MP8) * 8;
        const int c = (int)(lin / MP8);
        const int kw = c % KW, t = c / KW;
        const int kh = t % KH, cin = t / KH;
        __align__(16) __half v[8];
        int n = m0 / (OH * OW);
        int r = m0 - n * (OH * OW);
        int oh = r / OW, ow = r - oh * OW;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            __half val = __float2half(0.f);
            if (m0 + e < NPQ && cin < Cin) {
                const int ix = ow * sx - px + kw * dx;
                const int iy = oh * sy - py + kh * dy;
                if (ix >= 0 && ix < Wid && iy >= 0 && iy < Hei)
                    val = x[ix + (int64_t)Wid * (iy + (int64_t)Hei * (cin + (int64_t)Cin * n))];
            }
            v[e] = val;
            if (++ow == OW) {
                ow = 0;
                if (++oh == OH) {
                    oh = 0;
                    ++n;
                }
            }
        }
        *reinterpret_cast<uint4*>(col + (int64_t)c * MP + m0) = *reinterpret_cast<const uint4*>(v);
    }
}

// Copy w (CRS, Cout) into (CRSP, Cout) with zero rows past CRS, so the GEMM's B operand has
// a leading dimension a tensor map accepts.
__global__ void __launch_bounds__(256)
padrows_f16_kernel(__half* __restrict__ dst, const __half* __restrict__ src, int CRS, int CRSP, int64_t ntot) {
    for (int64_t lin = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; lin < ntot;
         lin += (int64_t)gridDim.x * blockDim.x) {
        const int c = (int)(lin % CRSP);
        const int64_t co = lin / CRSP;
        dst[lin] = c < CRS ? src[c + (int64_t)CRS * co] : __float2half(0.f);
    }
}

static unsigned grid_for(b200_ctx* ctx, int64_t n) {
    int64_t blocks = cdiv(n, 256);
    const int64_t cap = (int64_t)ctx->prop.multiProcessorCount * 32;
    return (unsigned)(blocks > cap ? cap : blocks);
}

static int64_t convsize(int64_t n, int64_t k, int64_t s, int64_t p, int64_t d) {
    return (n + 2 * p - d * (k - 1) - 1) / s + 1;
}

} // namespace b200

using namespace b200;

extern "C" {

int b200_im2col_f16(b200_ctx* ctx, int64_t W, int64_t H, int64_t Cin, int64_t N, int64_t KW, int64_t KH,
                    int64_t sx, int64_t sy, int64_t px, int64_t py, int64_t dx, int64_t dy, int64_t MP,
                    int64_t CRSP, const void* x, void* col) {
    B200_REQUIRE(ctx && x && col, B200_EINVAL, "im2col: null argument");
    B200_REQUIRE(W > 0 && H > 0 && Cin > 0 && N > 0 && KW > 0 && KH > 0 && sx > 0 && sy > 0 && dx > 0 && dy > 0 &&
                     px >= 0 && py >= 0,
                 B200_EINVAL, "im2col: bad geometry");
    const int64_t OW = convsize(W, KW, sx, px, dx), OH = convsize(H, KH, sy, py, dy);
    B200_REQUIRE(OW > 0 && OH > 0, B200_DECLINE_EXTENT, "im2col: empty output");
    const int64_t NPQ = OW * OH * N;
    B200_REQUIRE(MP >= NPQ && CRSP >= KW * KH * Cin, B200_EINVAL, "im2col: MP/CRSP below the real extents");
    B200_REQUIRE(MP % 8 == 0 && (reinterpret_cast<uintptr_t>(col) & 15u) == 0, B200_DECLINE_ALIGN,
                 "im2col: MP must be a multiple of 8 and col 16-byte aligned");
    B200_REQUIRE(MP < (1ll << 31) && CRSP < (1ll << 31) && W * H * Cin < (1ll << 31), B200_DECLINE_EXTENT,
                 "im2col: extent beyond int32");
    B200_CUDA(cudaSetDevice(ctx->device));
    const int64_t ntot8 = MP / 8 * CRSP;
    im2col_f16_kernel<<<grid_for(ctx, ntot8), 256, 0, ctx->stream>>>(
        (__half*)col, (const __half*)x, (int)MP, (int)CRSP, (int)KW, (int)KH, (int)sx, (int)sy, (int)px, (int)py,
        (int)dx, (int)dy, (int)W, (int)H, (int)OW, (int)OH, (int)NPQ, (int)Cin, ntot8);
    ctx->launches++;
    B200_CUDA(cudaGetLastError());
    return B200_OK;
}

// One group of a convolution: Cin_g input channels starting at x (image n at x + n * x_img), Cout_g output
// channels starting at out (image n at out + n * out_img elements), weight (KW,KH,Cin_g,Cout_g) dense.
static int conv2d_group(b200_ctx* ctx, int64_t W, int64_t H, int64_t Cin, int64_t N, int64_t KW, int64_t KH,
                        int64_t Cout, int64_t sx, int64_t sy, int64_t px, int64_t py, int64_t dx, int64_t dy,
                        const __half* x, int64_t x_img, const void* w, const void* bias, void* out, int64_t out_img,
                        int out_dtype, int epilogue) {
    const int64_t OW = convsize(W, KW, sx, px, dx), OH = convsize(H, KH, sy, py, dy);
    const int64_t P = OW * OH;       // pixels per image = GEMM M (contiguous in out)
    const int64_t CRS = KW * KH * Cin;
    const size_t osz = out_dtype == B200_F16 ? 2 : 4;
    const bool onebyone = KW == 1 && KH == 1 && sx == 1 && sy == 1 && px == 0 && py == 0;
    int rc;

    // Weight operand: (CRS, Cout) with CRS contiguous; pad its leading dimension to a
    // multiple of 8 elements when it is not one already.
    const void* wB = w;
    int64_t ldw = CRS;
    if (CRS % 8 != 0) {
        ldw = (CRS + 7) / 8 * 8;
        void* wp = nullptr;
        if ((rc = ws_scratch(ctx, (size_t)(ldw * Cout) * 2, &wp))) return rc;
        padrows_f16_kernel<<<grid_for(ctx, ldw * Cout), 256, 0, ctx->stream>>>((__half*)wp, (const __half*)w,
                                                                                (int)CRS, (int)ldw, ldw * Cout);
        ctx->launches++;
        B200_CUDA(cudaGetLastError());
        wB = wp;
    }
    if (onebyone) {
        for (int64_t n = 0; n < N; ++n) {
            const __half* xa = x + n * x_img; // (P, Cin) ld = P
            void* on = (char*)out + (size_t)(n * out_img) * osz;
            if ((rc = gemm_f16_run(ctx, P, Cout, Cin, xa, P, wB, ldw, bias, 1, on, P, out_dtype, epilogue, 1, 0, 0, 0)))
                return rc;
        }
        return B200_OK;
    }
    const int64_t MP = (P + 7) / 8 * 8;
    void* col = nullptr;
    if ((rc = ws_scratch(ctx, (size_t)(MP * CRS) * 2, &col))) return rc;
    for (int64_t n = 0; n < N; ++n) {
        const __half* xn = x + n * x_img;
        if ((rc = b200_im2col_f16(ctx, W, H, Cin, 1, KW, KH, sx, sy, px, py, dx, dy, MP, CRS, xn, col))) return rc;
        void* on = (char*)out + (size_t)(n * out_img) * osz;
        if ((rc = gemm_f16_run(ctx, P, Cout, CRS, col, MP, wB, ldw, bias, 1, on, P, out_dtype, epilogue, 1, 0, 0, 0)))
            return rc;
    }
    return B200_OK;
}

int b200_conv2d_f16(b200_ctx* ctx, int64_t W, int64_t H, int64_t Cin, int64_t N, int64_t KW, int64_t KH,
                    int64_t Cout, int64_t sx, int64_t sy, int64_t px, int64_t py, int64_t dx, int64_t dy,
                    const void* x, const void* w, const void* bias, void* out, int out_dtype, int epilogue) {
    return b200_conv2d_grouped_f16(ctx, W, H, Cin, N, KW, KH, Cout, sx, sy, px, py, dx, dy, 1, x, w, bias, out, out_dtype,
                                   epilogue);
}

int b200_conv2d_grouped_f16(b200_ctx* ctx, int64_t W, int64_t H, int64_t Cin, int64_t N, int64_t KW, int64_t KH,
                            int64_t Cout, int64_t sx, int64_t sy, int64_t px, int64_t py, int64_t dx, int64_t dy,
                            int64_t groups, const void* x, const void* w, const void* bias, void* out, int out_dtype,
                            int epilogue) {
    B200_REQUIRE(ctx && x && w && out, B200_EINVAL, "conv2d: null argument");
    B200_REQUIRE(W > 0 && H > 0 && Cin > 0 && N > 0 && KW > 0 && KH > 0 && Cout > 0 && sx > 0 && sy > 0 &&
                     dx > 0 && dy > 0 && px >= 0 && py >= 0 && groups > 0,
                 B200_EINVAL, "conv2d: bad geometry");
    B200_REQUIRE(Cin % groups == 0 && Cout % groups == 0, B200_DECLINE_EXTENT, "conv2d: %lld groups do not divide the channels",
                 (long long)groups);
    B200_REQUIRE(out_dtype == B200_F16 || out_dtype == B200_F32, B200_DECLINE_ELTYPE, "conv2d: out dtype %d", out_dtype);
    const int64_t OW = convsize(W, KW, sx, px, dx), OH = convsize(H, KH, sy, py, dy);
    B200_REQUIRE(OW > 0 && OH > 0, B200_DECLINE_EXTENT, "conv2d: empty output");
    B200_CUDA(cudaSetDevice(ctx->device));
    const int64_t CG = Cin / groups, COG = Cout / groups, P = OW * OH;
    const size_t osz = out_dtype == B200_F16 ? 2 : 4;
    for (int64_t g = 0; g < groups; ++g) {
        // group g: input channels [g CG, (g+1) CG), output channels [g COG, (g+1) COG), its own slice of the weight
        int rc = conv2d_group(ctx, W, H, CG, N, KW, KH, COG, sx, sy, px, py, dx, dy, (const __half*)x + g * CG * W * H,
                              W * H * Cin, (const __half*)w + g * COG * (KW * KH * CG),
                              bias ? (const __half*)bias + g * COG : nullptr, (char*)out + (size_t)(g * COG * P) * osz,
                              P * Cout, out_dtype, epilogue);
        if (rc) return rc;
    }
    return B200_OK;
}

// ------------------------------------------------------------------ transposed convolution
} // extern "C"

namespace b200 {

// convtranspose2d (conv.jl:147-190), the gather form: one thread per output element, fp32 fma chain from the
// bias over (ci, ky, kx); an input reaches an output where the stride divides.  x (W,H,Cin,N),
// w (KW,KH,Cout/groups,Cin), out (OW,OH,Cout,N).  Deterministic: no atomics.
template <typename OutT>
__global__ void __launch_bounds__(256)
convtranspose2d_f16_kernel(OutT* __restrict__ out, const __half* __restrict__ x, const __half* __restrict__ w,
                           const __half* __restrict__ bias, int Wd, int Hd, int Cin, int KW, int KH, int Cout, int sx,
                           int sy, int px, int py, int dx, int dy, int OW, int OH, int groups, int64_t ntot) {
    const int COG = Cout / groups, CG = Cin / groups;
    for (int64_t lin = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; lin < ntot; lin += (int64_t)gridDim.x * blockDim.x) {
        const int ox = (int)(lin % OW);
        int64_t t = lin / OW;
        const int oy = (int)(t % OH);
        t /= OH;
        const int co = (int)(t % Cout);
        const int64_t n = t / Cout;
        float acc = bias ? __half2float(bias[co]) : 0.f;
        const int cog = co % COG, g = co / COG;
        const int bx = ox + px, by = oy + py;
        for (int ci = g * CG; ci < (g + 1) * CG; ++ci)
            for (int ky = 0; ky < KH; ++ky) {
                const int ty = by - ky * dy;
                if (ty < 0 || ty % sy != 0) continue;
                const int iy = ty / sy;
                if (iy >= Hd) continue;
                for (int kx = 0; kx < KW; ++kx) {
                    const int tx = bx - kx * dx;
                    if (tx < 0 || tx % sx != 0) continue;
                    const int ix = tx / sx;
                    if (ix >= Wd) continue;
                    acc = fmaf(__half2float(x[ix + (int64_t)Wd * (iy + (int64_t)Hd * (ci + (int64_t)Cin * n))]),
                               __half2float(w[kx + KW * (ky + KH * (cog + (int64_t)COG * ci))]), acc);
                }
            }
        if constexpr (sizeof(OutT) == 2) out[lin] = __float2half_rn(acc);
        else out[lin] = acc;
    }
}

// shuffleout (conv.jl:232-246): scatter the GEMM's (W*H, SX*SY*Cout) result into (SX*W, SY*H, Cout), adding the
// bias in the output type.  Consecutive threads write consecutive addresses.
template <typename OutT>
__global__ void __launch_bounds__(256)
shuffleout_kernel(OutT* __restrict__ out, const OutT* __restrict__ P, const __half* __restrict__ bias, int Wd, int Hd, int SX,
                  int SY, int Cout, int64_t ntot) {
    const int OW = Wd * SX, OH = Hd * SY;
    for (int64_t lin = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; lin < ntot; lin += (int64_t)gridDim.x * blockDim.x) {
        const int ox = (int)(lin % OW);
        int64_t t = lin / OW;
        const int oy = (int)(t % OH);
        const int co = (int)(t / OH);
        const int i = ox / SX, ddx = ox - i * SX, j = oy / SY, ddy = oy - j * SY;
        const OutT v = P[(i + (int64_t)j * Wd) + (int64_t)Wd * Hd * (ddx + SX * (ddy + SY * co))];
        if constexpr (sizeof(OutT) == 2)
            out[lin] = bias ? __float2half_rn(__half2float(v) + __half2float(bias[co])) : v;
        else
            out[lin] = bias ? v + __half2float(bias[co]) : v;
    }
}

static int64_t convtransposesize(int64_t n, int64_t k, int64_t s, int64_t p, int64_t d, int64_t op) {
    return (n - 1) * s - 2 * p + d * (k - 1) + op + 1;
}

} // namespace b200

extern "C" {

int b200_convtranspose2d_f16(b200_ctx* ctx, int64_t W, int64_t H, int64_t Cin, int64_t N, int64_t KW, int64_t KH,
                             int64_t Cout, int64_t sx, int64_t sy, int64_t px, int64_t py, int64_t dx, int64_t dy,
                             int64_t opx, int64_t opy, int64_t groups, const void* x, const void* w, const void* bias,
                             void* out, int out_dtype) {
    B200_REQUIRE(ctx && x && w && out, B200_EINVAL, "convtranspose2d: null argument");
    B200_REQUIRE(W > 0 && H > 0 && Cin > 0 && N > 0 && KW > 0 && KH > 0 && Cout > 0 && sx > 0 && sy > 0 && dx > 0 &&
                     dy > 0 && px >= 0 && py >= 0 && opx >= 0 && opy >= 0 && groups > 0,
                 B200_EINVAL, "convtranspose2d: bad geometry");
    B200_REQUIRE(Cin % groups == 0 && Cout % groups == 0, B200_DECLINE_EXTENT,
                 "convtranspose2d: %lld groups do not divide the channels", (long long)groups);
    B200_REQUIRE(out_dtype == B200_F16 || out_dtype == B200_F32, B200_DECLINE_ELTYPE, "convtranspose2d: out dtype %d",
                 out_dtype);
    const int64_t OW = convtransposesize(W, KW, sx, px, dx, opx), OH = convtransposesize(H, KH, sy, py, dy, opy);
    B200_REQUIRE(OW > 0 && OH > 0, B200_DECLINE_EXTENT, "convtranspose2d: empty output");
    B200_REQUIRE(OW < (1ll << 31) && OH < (1ll << 31) && W * H * Cin < (1ll << 31), B200_DECLINE_EXTENT,
                 "convtranspose2d: extent beyond int32");
    B200_CUDA(cudaSetDevice(ctx->device));
    const size_t osz = out_dtype == B200_F16 ? 2 : 4;
    // shufflecase (conv.jl:219-222): stride equal to the kernel, no padding, dilation or output padding, one group —
    // every output pixel is fed by exactly one input pixel and one weight slice, i.e. a GEMM over
    // (W*H) x Cin x (KW*KH*Cout) and a depth-to-space interleave.
    const bool shuffle = groups == 1 && dx == 1 && dy == 1 && px == 0 && py == 0 && opx == 0 && opy == 0 && KW == sx &&
                         KH == sy;
    if (shuffle) {
        int rc;
        const int64_t NC = KW * KH * Cout, P = W * H;
        void *wm = nullptr, *pbuf = nullptr;
        if ((rc = ws_scratch(ctx, (size_t)(Cin * NC) * 2, &wm))) return rc;
        if ((rc = ws_scratch(ctx, (size_t)(P * NC) * osz, &pbuf))) return rc;
        // (kx, ky, co, ci) -> (ci, kx, ky, co): the GEMM's B operand with Cin contiguous (a permute of a weight: load-time
        // work in a planned graph, done per call here as the reference does)
        const int64_t shape[4] = {Cin, KW, KH, Cout};
        const int64_t stride[4] = {KW * KH * Cout, 1, KW, KW * KH};
        if ((rc = b200_permute4(ctx, w, wm, shape, stride, 2))) return rc;
        for (int64_t n = 0; n < N; ++n) {
            const __half* xn = (const __half*)x + n * P * Cin;   // (P, Cin), pixels contiguous
            if ((rc = gemm_f16_run(ctx, P, NC, Cin, xn, P, wm, Cin, nullptr, 0, pbuf, P, out_dtype, B200_EPI_NONE, 1, 0, 0, 0)))
                return rc;
            const int64_t ntot = OW * OH * Cout;
            void* on = (char*)out + (size_t)(n * ntot) * osz;
            if (out_dtype == B200_F16)
                shuffleout_kernel<__half><<<grid_for(ctx, ntot), 256, 0, ctx->stream>>>((__half*)on, (const __half*)pbuf,
                                                                                          (const __half*)bias, (int)W, (int)H,
                                                                                          (int)sx, (int)sy, (int)Cout, ntot);
            else
                shuffleout_kernel<float><<<grid_for(ctx, ntot), 256, 0, ctx->stream>>>((float*)on, (const float*)pbuf,
                                                                                        (const __half*)bias, (int)W, (int)H,
                                                                                        (int)sx, (int)sy, (int)Cout, ntot);
            ctx->launches++;
            B200_CUDA(cudaGetLastError());
        }
        return B200_OK;
    }
    const int64_t ntot = OW * OH * Cout * N;
    if (out_dtype == B200_F16)
        convtranspose2d_f16_kernel<__half><<<grid_for(ctx, ntot), 256, 0, ctx->stream>>>(
            (__half*)out, (const __half*)x, (const __half*)w, (const __half*)bias, (int)W, (int)H, (int)Cin, (int)KW, (int)KH,
            (int)Cout, (int)sx, (int)sy, (int)px, (int)py, (int)dx, (int)dy, (int)OW, (int)OH, (int)groups, ntot);
    else
        convtranspose2d_f16_kernel<float><<<grid_for(ctx, ntot), 256, 0, ctx->stream>>>(
            (float*)out, (const __half*)x, (const __half*)w, (const __half*)bias, (int)W, (int)H, (int)Cin, (int)KW, (int)KH,
            (int)Cout, (int)sx, (int)sy, (int)px, (int)py, (int)dx, (int)dy, (int)OW, (int)OH, (int)groups, ntot);
    ctx->launches++;
    B200_CUDA(cudaGetLastError());
    return B200_OK;
}


// ---------------------------------------------------------------- no-allocation variant
//
// Some hosts of this library may not allocate device memory at call time: a serving process
// whose own allocator claimed the whole GPU at start-up (a cudaMalloc from a plug-in then fails
// or fragments its arena), or a latency-critical loop whose rules forbid calls that synchronise
// the device, which cudaMalloc and cudaFree do.  b200_conv2d_f16 takes its im2col matrix and
// padded weight from the context's workspace, which grows through cudaMalloc.  The variant
// below takes them from a fixed array that is part of the loaded module instead, so it never
// allocates: every GPU that loads the library carries these B200_NOALLOC_SCRATCH_BYTES until the
// process exits.
//
// `g_noalloc_scratch` names a device symbol.  In host code that name is only a handle for the
// runtime, not an address a kernel can use, so the device address is looked up once per device
// with cudaGetSymbolAddress (that device current) and cached; kernels and tensor maps only ever
// see the looked-up pointer.
#define B200_NOALLOC_SCRATCH_BYTES (32u << 20)
static __device__ __align__(256) unsigned char g_noalloc_scratch[B200_NOALLOC_SCRATCH_BYTES];
static void* g_noalloc_addr[64] = {};

static int noalloc_scratch(b200_ctx* ctx, void** out) {
    const int dev = ctx->device;
    if (dev < 0 || dev >= 64) return fail(B200_EINVAL, "conv2d_noalloc: device index %d", dev);
    if (!g_noalloc_addr[dev]) {
        B200_CUDA(cudaSetDevice(dev));
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess) return fail_cuda(e, "cudaGetSymbolAddress(g_noalloc_scratch)");
        if (!p) return fail(B200_ECUDA, "conv2d_noalloc: the scratch symbol has no address on device %d", dev);
        g_noalloc_addr[dev] = p;
    }
    *out = g_noalloc_addr[dev];
    return B200_OK;
}

int b200_conv2d_f16_noalloc(b200_ctx* ctx, int64_t W, int64_t H, int64_t Cin, int64_t N, int64_t KW, int64_t KH,
                            int64_t Cout, int64_t sx, int64_t sy, int64_t px, int64_t py, int64_t dx, int64_t dy,
                            const void* x, const void* w, const void* bias, void* out, int out_dtype,
                            int epilogue) {
    B200_REQUIRE(ctx && x && w && out, B200_EINVAL, "conv2d_noalloc: null argument");
    B200_REQUIRE(W > 0 && H > 0 && Cin > 0 && N > 0 && KW > 0 && KH > 0 && Cout > 0 && sx > 0 && sy > 0 &&
                     dx > 0 && dy > 0 && px >= 0 && py >= 0,
                 B200_EINVAL, "conv2d_noalloc: bad geometry");
    const int64_t OW = convsize(W, KW, sx, px, dx), OH = convsize(H, KH, sy, py, dy);
    B200_REQUIRE(OW > 0 && OH > 0, B200_DECLINE_EXTENT, "conv2d_noalloc: empty output");
    const int64_t P = OW * OH, CRS = KW * KH * Cin;
    const size_t osz = out_dtype == B200_F16 ? 2 : 4;
    const bool onebyone = KW == 1 && KH == 1 && sx == 1 && sy == 1 && px == 0 && py == 0;
    const int64_t ldw = (CRS + 7) / 8 * 8, MP = (P + 7) / 8 * 8;
    // Carve-up of the fixed array: [padded weight | im2col matrix], each 256-byte aligned.
    const size_t wbytes = CRS % 8 != 0 ? ((size_t)(ldw * Cout) * 2 + 255) / 256 * 256 : 0;
    const size_t cbytes = onebyone ? 0 : (size_t)(MP * CRS) * 2;
    if (wbytes + cbytes > B200_NOALLOC_SCRATCH_BYTES)
        return fail(B200_ENOMEM,
                    "conv2d_noalloc: this convolution needs %zu bytes of scratch (padded weight %zu + im2col %zu) "
                    "but the built-in array holds %u; use b200_conv2d_f16, which draws on the workspace",
                    wbytes + cbytes, wbytes, cbytes, (unsigned)B200_NOALLOC_SCRATCH_BYTES);
    B200_CUDA(cudaSetDevice(ctx->device));
    void* base = nullptr;
    int rc = noalloc_scratch(ctx, &base);
    if (rc) return rc;

    const void* wB = w;
    int64_t ldwB = CRS;
    if (wbytes) {
        // Every element of the padded weight is written (the zero rows too), so nothing a
        // previous call left in the array can leak into this one.
        padrows_f16_kernel<<<grid_for(ctx, ldw * Cout), 256, 0, ctx->stream>>>((__half*)base, (const __half*)w,
                                                                                (int)CRS, (int)ldw, ldw * Cout);
        ctx->launches++;
        B200_CUDA(cudaGetLastError());
        wB = base;
        ldwB = ldw;
    }
    void* col = (char*)base + wbytes;
    for (int64_t n = 0; n < N; ++n) {
        void* on = (char*)out + (size_t)(n * P * Cout) * osz;
        if (onebyone) {
            const __half* xa = (const __half*)x + n * P * Cin;
            if ((rc = gemm_f16_run(ctx, P, Cout, Cin, xa, P, wB, ldwB, bias, 1, on, P, out_dtype, epilogue, 1, 0, 0, 0,
                                   /*use_workspace=*/0)))
                return rc;
            continue;
        }
        // The gather writes all MP x CRS entries, zeros included: no clearing pass is needed.
        const __half* xn = (const __half*)x + n * W * H * Cin;
        if ((rc = b200_im2col_f16(ctx, W, H, Cin, 1, KW, KH, sx, sy, px, py, dx, dy, MP, CRS, xn, col))) return rc;
        if ((rc = gemm_f16_run(ctx, P, Cout, CRS, col, MP, wB, ldwB, bias, 1, on, P, out_dtype, epilogue, 1, 0, 0, 0,
                                   /*use_workspace=*/0)))
            return rc;
    }
    return B200_OK;
}

} // extern "C"
