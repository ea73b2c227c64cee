// Convolution lowered to the tensor-core GEMM: an im2col gather (skipped for 1x1/stride-1/
// unpadded kernels, where the image already is the GEMM operand), then one GEMM per image
// with the per-channel bias and the activation fused in its store, written straight into
// out (OW,OH,Cout,N).  Replaces im2col_kernel! + Lava.coopmat_gemm! into fp32 planes +
// conv_epilogue_kernel! (reference kernels/extern/conv_coopmat.jl:246-392) and the 1x1
// route through matmul! (kernels/extern/conv.jl:122-131).
#include <cuda_fp16.h>

#include "internal.h"

namespace b200 {

// col (MP, CRSP) column-major: thread -> (m, c) with m fastest so the writes coalesce.
// Index math is 32-bit on purpose: every extent is far inside int32 and 64-bit division
// is emulated (same observation as the reference, conv_coopmat.jl:238-245).
__global__ void __launch_bounds__(256)
im2col_f16_kernel(__half* __restrict__ col, const __half* __restrict__ x, int MP, int CRSP, int KW, int KH,
                  int sx, int sy, int px, int py, int dx, int dy, int Wid, int Hei, int OW, int OH, int NPQ,
                  int Cin, int64_t ntot) {
    for (int64_t lin = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; lin < ntot;
         lin += (int64_t)gridDim.x * blockDim.x) {
        const int m = (int)(lin % MP);
        const int c = (int)(lin / MP);
        __half v = __float2half(0.f);
        if (m < NPQ) {
            const int n = m / (OH * OW);
            const int r = m - n * (OH * OW);
            const int oh = r / OW, ow = r - oh * OW;
            const int kw = c % KW, t = c / KW;
            const int kh = t % KH, cin = t / KH;
            if (cin < Cin) {
                const int ix = ow * sx - px + kw * dx;
                const int iy = oh * sy - py + kh * dy;
                if (ix >= 0 && ix < Wid && iy >= 0 && iy < Hei)
                    v = x[ix + (int64_t)Wid * (iy + (int64_t)Hei * (cin + (int64_t)Cin * n))];
            }
        }
        col[lin] = v;
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
    B200_REQUIRE(MP < (1ll << 31) && CRSP < (1ll << 31) && W * H * Cin < (1ll << 31), B200_DECLINE_EXTENT,
                 "im2col: extent beyond int32");
    B200_CUDA(cudaSetDevice(ctx->device));
    const int64_t ntot = MP * CRSP;
    im2col_f16_kernel<<<grid_for(ctx, ntot), 256, 0, ctx->stream>>>(
        (__half*)col, (const __half*)x, (int)MP, (int)CRSP, (int)KW, (int)KH, (int)sx, (int)sy, (int)px, (int)py,
        (int)dx, (int)dy, (int)W, (int)H, (int)OW, (int)OH, (int)NPQ, (int)Cin, ntot);
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

} // extern "C"
