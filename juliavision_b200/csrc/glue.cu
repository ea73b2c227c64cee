// Bandwidth-bound glue ops the encoder graphs run between the dense kernels: residual add,
// clamp, standalone activation and the strided -> dense copy behind permute/contiguous.
// fp16 storage, fp32 arithmetic, one rounding at the store (reference ops.jl:186-197,
// 323-335, 1698-1702; execute.jl:257-277).
#include <cuda_fp16.h>

#include "act.cuh"
#include "internal.h"

namespace b200 {

enum { OP_ADD = 0, OP_CLAMP = 1, OP_ACT = 2 };

template <int OP>
__device__ __forceinline__ float ew(float a, float b, float lo, float hi, int epi) {
    if (OP == OP_ADD) return a + b;
    if (OP == OP_CLAMP) return fminf(fmaxf(a, lo), hi);
    return apply_act(epi, a);
}

// 8 halfs (16 B) per thread per step, grid-stride; the scalar tail is handled by the last
// few threads of the same launch.
template <int OP>
__global__ void __launch_bounds__(256)
ew_f16_kernel(const __half* __restrict__ a, const __half* __restrict__ b, __half* __restrict__ out,
              int64_t n, float lo, float hi, int epi, int vec) {
    const int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
    int64_t done = 0;
    if (vec) {
        const int64_t nv = n / 8;
        for (int64_t i = tid; i < nv; i += nthreads) {
            uint4 ua = __ldg(reinterpret_cast<const uint4*>(a) + i);
            uint4 ub = OP == OP_ADD ? __ldg(reinterpret_cast<const uint4*>(b) + i) : ua;
            uint4 uo;
            const __half2* ha = reinterpret_cast<const __half2*>(&ua);
            const __half2* hb = reinterpret_cast<const __half2*>(&ub);
            __half2* ho = reinterpret_cast<__half2*>(&uo);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                float2 fa = __half22float2(ha[q]), fb = __half22float2(hb[q]);
                ho[q] = __floats2half2_rn(ew<OP>(fa.x, fb.x, lo, hi, epi), ew<OP>(fa.y, fb.y, lo, hi, epi));
            }
            reinterpret_cast<uint4*>(out)[i] = uo;
        }
        done = nv * 8;
    }
    for (int64_t i = done + tid; i < n; i += nthreads) {
        float fa = __half2float(a[i]);
        float fb = OP == OP_ADD ? __half2float(b[i]) : 0.f;
        out[i] = __float2half_rn(ew<OP>(fa, fb, lo, hi, epi));
    }
}

template <int OP>
static int launch_ew(b200_ctx* ctx, const void* a, const void* b, void* out, int64_t n, float lo, float hi,
                     int epi) {
    if (n == 0) return B200_OK;
    auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    const int vec = al(a) && al(out) && (OP != OP_ADD || al(b));
    int64_t work = vec ? cdiv(n, 8) : n;
    int64_t blocks = cdiv(work, 256);
    const int64_t cap = (int64_t)ctx->prop.multiProcessorCount * 16;
    if (blocks > cap) blocks = cap;
    ew_f16_kernel<OP><<<(unsigned)blocks, 256, 0, ctx->stream>>>((const __half*)a, (const __half*)b, (__half*)out,
                                                                  n, lo, hi, epi, vec);
    ctx->launches++;
    B200_CUDA(cudaGetLastError());
    return B200_OK;
}

// _to_copy between fp16 and fp32 (ops.jl:342-358): eight elements per thread when both ends are
// 16-byte aligned, a scalar loop for the tail.
template <typename SrcT, typename DstT>
__global__ void __launch_bounds__(256)
cast_kernel(const SrcT* __restrict__ src, DstT* __restrict__ dst, int64_t n, int vec) {
    const int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
    auto tof = [](SrcT v) -> float {
        if constexpr (sizeof(SrcT) == 2) return __half2float(v);
        else return v;
    };
    auto fromf = [](float v) -> DstT {
        if constexpr (sizeof(DstT) == 2) return __float2half_rn(v);
        else return v;
    };
    int64_t done = 0;
    if (vec) {
        const int64_t nv = n / 8;
        for (int64_t i = tid; i < nv; i += nthreads) {
            SrcT in[8];
            DstT o[8];
            if constexpr (sizeof(SrcT) == 2) {
                *reinterpret_cast<uint4*>(in) = __ldg(reinterpret_cast<const uint4*>(src) + i);
            } else {
                *reinterpret_cast<uint4*>(in) = __ldg(reinterpret_cast<const uint4*>(src) + 2 * i);
                *reinterpret_cast<uint4*>(in + 4) = __ldg(reinterpret_cast<const uint4*>(src) + 2 * i + 1);
            }
#pragma unroll
            for (int q = 0; q < 8; ++q) o[q] = fromf(tof(in[q]));
            if constexpr (sizeof(DstT) == 2) {
                reinterpret_cast<uint4*>(dst)[i] = *reinterpret_cast<const uint4*>(o);
            } else {
                reinterpret_cast<uint4*>(dst)[2 * i] = *reinterpret_cast<const uint4*>(o);
                reinterpret_cast<uint4*>(dst)[2 * i + 1] = *reinterpret_cast<const uint4*>(o + 4);
            }
        }
        done = nv * 8;
    }
    for (int64_t i = done + tid; i < n; i += nthreads) dst[i] = fromf(tof(src[i]));
}

template <typename SrcT, typename DstT>
static int launch_cast(b200_ctx* ctx, const void* src, void* dst, int64_t n) {
    auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    const int vec = al(src) && al(dst);
    int64_t blocks = cdiv(vec ? cdiv(n, 8) : n, 256);
    const int64_t cap = (int64_t)ctx->prop.multiProcessorCount * 16;
    if (blocks > cap) blocks = cap;
    cast_kernel<SrcT, DstT><<<(unsigned)blocks, 256, 0, ctx->stream>>>((const SrcT*)src, (DstT*)dst, n, vec);
    ctx->launches++;
    B200_CUDA(cudaGetLastError());
    return B200_OK;
}

// Strided gather into a dense array: one thread per output element, output-coalesced.
template <typename T>
__global__ void __launch_bounds__(256)
permute4_kernel(const T* __restrict__ src, T* __restrict__ out, int64_t n, int64_t d0, int64_t d1, int64_t d2,
                int64_t s0, int64_t s1, int64_t s2, int64_t s3) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t i0 = i % d0, t = i / d0;
        int64_t i1 = t % d1;
        t /= d1;
        int64_t i2 = t % d2, i3 = t / d2;
        out[i] = src[i0 * s0 + i1 * s1 + i2 * s2 + i3 * s3];
    }
}

// Same gather when the source is contiguous along output axis 1 (a transpose of the two
// fastest axes, the layout change behind permute(0,2,1,3)-style views): 32x32 tiles through
// shared memory so both the reads and the writes coalesce.
template <typename T>
__global__ void __launch_bounds__(256)
transpose01_kernel(const T* __restrict__ src, T* __restrict__ out, int d0, int d1, int64_t d2, int64_t s0,
                   int64_t s2, int64_t s3) {
    __shared__ T tile[32][33];
    const int64_t z = blockIdx.z;
    const int64_t i2 = z % d2, i3 = z / d2;
    const T* sp = src + i2 * s2 + i3 * s3;
    T* op = out + z * (int64_t)d0 * d1;
    const int b0 = blockIdx.x * 32, b1 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (int r = ty; r < 32; r += 8) {
        int i0 = b0 + r, i1 = b1 + tx; // read: i1 fastest in the source
        if (i0 < d0 && i1 < d1) tile[r][tx] = sp[(int64_t)i0 * s0 + i1];
    }
    __syncthreads();
    for (int r = ty; r < 32; r += 8) {
        int i1 = b1 + r, i0 = b0 + tx; // write: i0 fastest in the output
        if (i0 < d0 && i1 < d1) op[i0 + (int64_t)d0 * i1] = tile[tx][r];
    }
}

template <typename T>
static int launch_permute(b200_ctx* ctx, const void* src, void* out, const int64_t* d, const int64_t* s) {
    const int64_t n = d[0] * d[1] * d[2] * d[3];
    if (n == 0) return B200_OK;
    // Axis 0 contiguous on both sides (a window partition moves whole runs of channels): the same gather
    // in 16-byte pieces.
    constexpr int64_t V = 16 / (int64_t)sizeof(T);
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    if (s[0] == 1 && d[0] % V == 0 && s[1] % V == 0 && s[2] % V == 0 && s[3] % V == 0 && al16(src) && al16(out)) {
        const int64_t nv = n / V;
        int64_t blocks = cdiv(nv, 256);
        const int64_t cap = (int64_t)ctx->prop.multiProcessorCount * 32;
        if (blocks > cap) blocks = cap;
        permute4_kernel<uint4><<<(unsigned)blocks, 256, 0, ctx->stream>>>((const uint4*)src, (uint4*)out, nv, d[0] / V, d[1], d[2],
                                                                         1, s[1] / V, s[2] / V, s[3] / V);
        ctx->launches++;
        B200_CUDA(cudaGetLastError());
        return B200_OK;
    }
    if (s[1] == 1 && s[0] != 1 && d[0] < (1ll << 30) && d[1] < (1ll << 30) && d[2] * d[3] < 65536 &&
        cdiv(d[1], 32) < 65536) {
        dim3 grid((unsigned)cdiv(d[0], 32), (unsigned)cdiv(d[1], 32), (unsigned)(d[2] * d[3]));
        transpose01_kernel<T><<<grid, 256, 0, ctx->stream>>>((const T*)src, (T*)out, (int)d[0], (int)d[1], d[2], s[0],
                                                            s[2], s[3]);
    } else {
        int64_t blocks = cdiv(n, 256);
        const int64_t cap = (int64_t)ctx->prop.multiProcessorCount * 32;
        if (blocks > cap) blocks = cap;
        permute4_kernel<T><<<(unsigned)blocks, 256, 0, ctx->stream>>>((const T*)src, (T*)out, n, d[0], d[1], d[2], s[0],
                                                                     s[1], s[2], s[3]);
    }
    ctx->launches++;
    B200_CUDA(cudaGetLastError());
    return B200_OK;
}

// max_pool2d (reference kernels/resample.jl:121-141): out[ox,oy,c,n] = max over the window of
// x[ix,iy,c,n], positions outside the image skipped, the running maximum starting at the type's
// lowest value.  Both arrays are indexed (x, y, c, n) through element strides, so the planar layout
// of the reference's call and a channels-last token array go through the same kernel; VEC = 8 takes
// eight channels per thread when the channel axis is contiguous in both.
template <int VEC>
__global__ void __launch_bounds__(256)
maxpool2d_kernel(const __half* __restrict__ x, __half* __restrict__ out, int W, int H, int C, int OW, int OH, int64_t total,
                 int64_t xs0, int64_t xs1, int64_t xs2, int64_t xs3, int64_t os0, int64_t os1, int64_t os2, int64_t os3,
                 int kx, int ky, int sx, int sy, int px, int py, int c_fast) {
    const int CV = C / VEC;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int ox, oy, c, n;
        int64_t t = i;
        if (c_fast) {   // channel fastest: neighbouring threads touch neighbouring channels
            c = (int)(t % CV) * VEC; t /= CV;
            ox = (int)(t % OW); t /= OW;
            oy = (int)(t % OH); n = (int)(t / OH);
        } else {
            ox = (int)(t % OW); t /= OW;
            oy = (int)(t % OH); t /= OH;
            c = (int)(t % CV) * VEC; n = (int)(t / CV);
        }
        const int bx = ox * sx - px, by = oy * sy - py;
        const __half* xp = x + (int64_t)c * xs2 + (int64_t)n * xs3;
        if constexpr (VEC == 8) {
            __half2 acc[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) acc[u] = __half2half2(__ushort_as_half(0xFC00));   // -inf = typemin(Float16)
            for (int dy = 0; dy < ky; ++dy) {
                const int iy = by + dy;
                if (iy < 0 || iy >= H) continue;
                for (int dx = 0; dx < kx; ++dx) {
                    const int ix = bx + dx;
                    if (ix < 0 || ix >= W) continue;
                    const uint4 w = *reinterpret_cast<const uint4*>(xp + (int64_t)ix * xs0 + (int64_t)iy * xs1);
                    const __half2* hh = reinterpret_cast<const __half2*>(&w);
#pragma unroll
                    for (int u = 0; u < 4; ++u) acc[u] = __hmax2_nan(acc[u], hh[u]);
                }
            }
            *reinterpret_cast<uint4*>(out + (int64_t)ox * os0 + (int64_t)oy * os1 + (int64_t)c * os2 + (int64_t)n * os3) =
                *reinterpret_cast<const uint4*>(acc);
        } else {
            __half acc = __ushort_as_half(0xFC00);
            for (int dy = 0; dy < ky; ++dy) {
                const int iy = by + dy;
                if (iy < 0 || iy >= H) continue;
                for (int dx = 0; dx < kx; ++dx) {
                    const int ix = bx + dx;
                    if (ix < 0 || ix >= W) continue;
                    acc = __hmax_nan(acc, xp[(int64_t)ix * xs0 + (int64_t)iy * xs1]);
                }
            }
            out[(int64_t)ox * os0 + (int64_t)oy * os1 + (int64_t)c * os2 + (int64_t)n * os3] = acc;
        }
    }
}

} // namespace b200

using namespace b200;

extern "C" {

int b200_maxpool2d_f16(b200_ctx* ctx, int64_t W, int64_t H, int64_t Cn, int64_t N, const void* x, const int64_t* xstride,
                       void* out, const int64_t* ostride, int64_t kx, int64_t ky, int64_t sx, int64_t sy, int64_t px,
                       int64_t py) {
    B200_REQUIRE(ctx && xstride && ostride, B200_EINVAL, "maxpool2d: null argument");
    B200_REQUIRE(W >= 0 && H >= 0 && Cn >= 0 && N >= 0, B200_EINVAL, "maxpool2d: negative extent");
    B200_REQUIRE(kx >= 1 && ky >= 1 && sx >= 1 && sy >= 1 && px >= 0 && py >= 0 && 2 * px <= kx && 2 * py <= ky,
                 B200_EINVAL, "maxpool2d: window %lldx%lld stride %lldx%lld pad %lldx%lld", (long long)kx, (long long)ky,
                 (long long)sx, (long long)sy, (long long)px, (long long)py);
    B200_REQUIRE(W < (1ll << 30) && H < (1ll << 30) && Cn < (1ll << 30) && N < (1ll << 30), B200_DECLINE_EXTENT,
                 "maxpool2d: extent");
    if (W + 2 * px < kx || H + 2 * py < ky) return B200_OK;   // no output position
    const int64_t OW = (W + 2 * px - kx) / sx + 1, OH = (H + 2 * py - ky) / sy + 1;
    if (OW * OH * Cn * N == 0) return B200_OK;
    B200_REQUIRE(x && out, B200_EINVAL, "maxpool2d: null array");
    B200_CUDA(cudaSetDevice(ctx->device));
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    bool vec = xstride[2] == 1 && ostride[2] == 1 && Cn % 8 == 0 && al16(x) && al16(out);
    for (int d = 0; d < 4; ++d)
        if (d != 2) vec = vec && xstride[d] % 8 == 0 && ostride[d] % 8 == 0;
    const int c_fast = ostride[2] == 1;
    const int64_t total = OW * OH * (vec ? Cn / 8 : Cn) * N;
    int64_t blocks = cdiv(total, 256);
    const int64_t cap = (int64_t)ctx->prop.multiProcessorCount * 32;
    if (blocks > cap) blocks = cap;
    if (vec)
        maxpool2d_kernel<8><<<(unsigned)blocks, 256, 0, ctx->stream>>>(
            (const __half*)x, (__half*)out, (int)W, (int)H, (int)Cn, (int)OW, (int)OH, total, xstride[0], xstride[1],
            xstride[2], xstride[3], ostride[0], ostride[1], ostride[2], ostride[3], (int)kx, (int)ky, (int)sx, (int)sy,
            (int)px, (int)py, c_fast);
    else
        maxpool2d_kernel<1><<<(unsigned)blocks, 256, 0, ctx->stream>>>(
            (const __half*)x, (__half*)out, (int)W, (int)H, (int)Cn, (int)OW, (int)OH, total, xstride[0], xstride[1],
            xstride[2], xstride[3], ostride[0], ostride[1], ostride[2], ostride[3], (int)kx, (int)ky, (int)sx, (int)sy,
            (int)px, (int)py, c_fast);
    ctx->launches++;
    B200_CUDA(cudaGetLastError());
    return B200_OK;
}

int b200_add_f16(b200_ctx* ctx, const void* a, const void* b, void* out, int64_t n) {
    B200_REQUIRE(ctx && n >= 0 && (n == 0 || (a && b && out)), B200_EINVAL, "add: bad argument");
    B200_CUDA(cudaSetDevice(ctx->device));
    return launch_ew<OP_ADD>(ctx, a, b, out, n, 0.f, 0.f, 0);
}
int b200_clamp_f16(b200_ctx* ctx, const void* a, void* out, int64_t n, float lo, float hi) {
    B200_REQUIRE(ctx && n >= 0 && (n == 0 || (a && out)), B200_EINVAL, "clamp: bad argument");
    B200_CUDA(cudaSetDevice(ctx->device));
    return launch_ew<OP_CLAMP>(ctx, a, nullptr, out, n, lo, hi, 0);
}
int b200_act_f16(b200_ctx* ctx, const void* a, void* out, int64_t n, int epilogue) {
    B200_REQUIRE(ctx && n >= 0 && (n == 0 || (a && out)), B200_EINVAL, "act: bad argument");
    B200_REQUIRE(epilogue >= B200_EPI_NONE && epilogue <= B200_EPI_GELU_TANH, B200_EINVAL, "act: epilogue %d",
                 epilogue);
    B200_CUDA(cudaSetDevice(ctx->device));
    return launch_ew<OP_ACT>(ctx, a, nullptr, out, n, 0.f, 0.f, epilogue);
}
int b200_cast(b200_ctx* ctx, const void* src, int src_dtype, void* dst, int dst_dtype, int64_t n) {
    B200_REQUIRE(ctx && n >= 0 && (n == 0 || (src && dst)), B200_EINVAL, "cast: bad argument");
    B200_REQUIRE((src_dtype == B200_F16 || src_dtype == B200_F32) && (dst_dtype == B200_F16 || dst_dtype == B200_F32),
                 B200_DECLINE_ELTYPE, "cast: dtypes %d -> %d", src_dtype, dst_dtype);
    if (n == 0) return B200_OK;
    B200_CUDA(cudaSetDevice(ctx->device));
    if (src_dtype == dst_dtype) {
        B200_CUDA(cudaMemcpyAsync(dst, src, (size_t)n * (src_dtype == B200_F16 ? 2 : 4), cudaMemcpyDeviceToDevice, ctx->stream));
        return B200_OK;
    }
    return src_dtype == B200_F16 ? launch_cast<__half, float>(ctx, src, dst, n) : launch_cast<float, __half>(ctx, src, dst, n);
}
int b200_permute4(b200_ctx* ctx, const void* src, void* out, const int64_t* shape, const int64_t* stride,
                  int elsize) {
    B200_REQUIRE(ctx && shape && stride, B200_EINVAL, "permute4: null argument");
    for (int i = 0; i < 4; ++i) B200_REQUIRE(shape[i] >= 0, B200_EINVAL, "permute4: negative extent");
    B200_REQUIRE(elsize == 2 || elsize == 4, B200_DECLINE_ELTYPE, "permute4: element size %d", elsize);
    if (shape[0] * shape[1] * shape[2] * shape[3] == 0) return B200_OK;
    B200_REQUIRE(src && out, B200_EINVAL, "permute4: null array");
    B200_CUDA(cudaSetDevice(ctx->device));
    return elsize == 2 ? launch_permute<uint16_t>(ctx, src, out, shape, stride)
                       : launch_permute<uint32_t>(ctx, src, out, shape, stride);
}

} // extern "C"
