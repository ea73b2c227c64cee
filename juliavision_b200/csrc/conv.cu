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

int b200_conv2d_f16(b200_ctx* ctx, int64_t W, int64_t H, int64_t Cin, int64_t N, int64_t KW, int64_t KH,
                    int64_t Cout, int64_t sx, int64_t sy, int64_t px, int64_t py, int64_t dx, int64_t dy,
                    const void* x, const void* w, const void* bias, void* out, int out_dtype, int epilogue) {
    B200_REQUIRE(ctx && x && w && out, B200_EINVAL, "conv2d: null argument");
    B200_REQUIRE(W > 0 && H > 0 && Cin > 0 && N > 0 && KW > 0 && KH > 0 && Cout > 0 && sx > 0 && sy > 0 &&
                     dx > 0 && dy > 0 && px >= 0 && py >= 0,
                 B200_EINVAL, "conv2d: bad geometry");
    const int64_t OW = convsize(W, KW, sx, px, dx), OH = convsize(H, KH, sy, py, dy);
    B200_REQUIRE(OW > 0 && OH > 0, B200_DECLINE_EXTENT, "conv2d: empty output");
    B200_CUDA(cudaSetDevice(ctx->device));
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
            const __half* xa = (const __half*)x + n * P * Cin; // (P, Cin) ld = P
            void* on = (char*)out + (size_t)(n * P * Cout) * osz;
            if ((rc = gemm_f16_run(ctx, P, Cout, Cin, xa, P, wB, ldw, bias, 1, on, P, out_dtype, epilogue, 1, 0, 0, 0)))
                return rc;
        }
        return B200_OK;
    }
    const int64_t MP = (P + 7) / 8 * 8;
    void* col = nullptr;
    if ((rc = ws_scratch(ctx, (size_t)(MP * CRS) * 2, &col))) return rc;
    for (int64_t n = 0; n < N; ++n) {
        const __half* xn = (const __half*)x + n * W * H * Cin;
        if ((rc = b200_im2col_f16(ctx, W, H, Cin, 1, KW, KH, sx, sy, px, py, dx, dy, MP, CRS, xn, col))) return rc;
        void* on = (char*)out + (size_t)(n * P * Cout) * osz;
        if ((rc = gemm_f16_run(ctx, P, Cout, CRS, col, MP, wB, ldw, bias, 1, on, P, out_dtype, epilogue, 1, 0, 0, 0)))
            return rc;
    }
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
