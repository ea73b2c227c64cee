// LayerNorm over the leading (contiguous) axis: one read of the input, one write of the
// output.  Bandwidth-bound: 16-byte vector loads, the whole group held in registers, fp32
// statistics reduced with warp shuffles, variance taken about the mean (two passes over
// registers, never E[x^2]-mean^2).
//
// Replaces layernorm_kernel! (reference kernels/layernorm.jl:44-114): 128 threads per
// group, shared-memory tree reductions and three strided passes over the group.
#include <cuda_fp16.h>

#include "internal.h"
#include "ptx.cuh"

namespace b200 {

template <typename T> struct Vec16;
template <> struct Vec16<__half> {
    static constexpr int N = 8;
    uint4 raw;
    __device__ __forceinline__ void to_f32(float* f) const {
        const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 t = __half22float2(h[i]);
            f[2 * i] = t.x;
            f[2 * i + 1] = t.y;
        }
    }
};
template <> struct Vec16<float> {
    static constexpr int N = 4;
    uint4 raw;
    __device__ __forceinline__ void to_f32(float* f) const {
        const float* p = reinterpret_cast<const float*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) f[i] = p[i];
    }
};

template <int N> __device__ __forceinline__ void store_vec(__half* dst, const float* f) {
    static_assert(N == 8 || N == 4, "vector width");
    if constexpr (N == 8) {
        uint4 o;
        __half2* h = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
        *reinterpret_cast<uint4*>(dst) = o;
    } else {
        uint2 o;
        __half2* h = reinterpret_cast<__half2*>(&o);
        h[0] = __floats2half2_rn(f[0], f[1]);
        h[1] = __floats2half2_rn(f[2], f[3]);
        *reinterpret_cast<uint2*>(dst) = o;
    }
}
template <int N> __device__ __forceinline__ void store_vec(float* dst, const float* f) {
#pragma unroll
    for (int i = 0; i < N; i += 4)
        *reinterpret_cast<float4*>(dst + i) = make_float4(f[i], f[i + 1], f[i + 2], f[i + 3]);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Sum over the LPG lanes of a group (LPG a power of two; the butterfly never leaves the aligned span).
template <int LPG>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
    for (int o = LPG / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// One warp per group; lane l owns vectors l, l+32, ... (VPL of them at most).  Narrow groups (at most
// 16 or 8 vectors, VPL = 1) share a warp, LPG lanes each, so that no lane idles; the sums are the same
// butterflies with the empty upper steps left out, hence the same bits.
// LAT: the latency form, for launches small enough that every CTA is resident at once and what the kernel takes
// is a chain of round trips, not bytes (the encoder's 1500 rows): everything the row needs is asked for up front.
// It costs ~40 registers; launches of many waves, which want occupancy, take the lean form.
template <typename InT, typename OutT, int VPL, int LPG = 32, bool LAT = false>
__global__ void __launch_bounds__(128)
ln_warp_kernel(const InT* __restrict__ a, OutT* __restrict__ out, float* __restrict__ mean,
               float* __restrict__ rstd, const InT* __restrict__ gamma,
               const InT* __restrict__ beta, int64_t groups, int C, float eps) {
    constexpr int VN = Vec16<InT>::N;
    static_assert(LPG == 32 || VPL == 1, "only single-vector groups share a warp");
    const int lane = threadIdx.x & (LPG - 1);
    const int64_t g = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / LPG;
    const int nvec = g < groups ? C / VN : 0;   // lanes past the last group idle through the shuffles
    const InT* src = a + g * (int64_t)C;
    // Narrow rows ask for gamma and beta together with the row, so that the normalised row does not wait for
    // them at the end (measured on the encoder pass with the add + layer-norm kernel below: 3.45 -> 3.37 ms).
    // Asking for them above the dependency wait would gain another 0.4 % when they are weights, and read stale
    // values when the previous kernel wrote them; nothing here knows which, so they are read below it.
    constexpr bool HOIST = LAT && VPL <= 6;
    grid_dep_wait();     // the input is the previous kernel's output
    grid_dep_launch();
    uint4 gw[HOIST ? VPL : 1], bw[HOIST ? VPL : 1];
    if constexpr (HOIST) {
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            const int v = lane + 32 * i;
            gw[i] = (gamma && v < nvec) ? __ldg(reinterpret_cast<const uint4*>(gamma) + v) : make_uint4(0u, 0u, 0u, 0u);
            bw[i] = (beta && v < nvec) ? __ldg(reinterpret_cast<const uint4*>(beta) + v) : make_uint4(0u, 0u, 0u, 0u);
        }
    }

    float x[VPL][VN];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        int v = lane + 32 * i;
        if (v < nvec) {
            Vec16<InT> t;
            t.raw = __ldg(reinterpret_cast<const uint4*>(src) + v);
            t.to_f32(x[i]);
#pragma unroll
            for (int j = 0; j < VN; ++j) s += x[i][j];
        }
    }
    const float n = (float)C;
    const float mu = group_sum<LPG>(s) / n;
    float s2 = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        if (lane + 32 * i < nvec) {
#pragma unroll
            for (int j = 0; j < VN; ++j) {
                float d = x[i][j] - mu;
                s2 += d * d;
            }
        }
    }
    const float r = 1.0f / sqrtf(group_sum<LPG>(s2) / n + eps);

    OutT* dst = out + g * (int64_t)C;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        int v = lane + 32 * i;
        if (v < nvec) {
            float y[VN];
#pragma unroll
            for (int j = 0; j < VN; ++j) y[j] = (x[i][j] - mu) * r;
            if (gamma) {
                Vec16<InT> t;
                float gf[VN];
                if constexpr (HOIST) t.raw = gw[i];
                else t.raw = __ldg(reinterpret_cast<const uint4*>(gamma) + v);
                t.to_f32(gf);
#pragma unroll
                for (int j = 0; j < VN; ++j) y[j] *= gf[j];
            }
            if (beta) {
                Vec16<InT> t;
                float bf[VN];
                if constexpr (HOIST) t.raw = bw[i];
                else t.raw = __ldg(reinterpret_cast<const uint4*>(beta) + v);
                t.to_f32(bf);
#pragma unroll
                for (int j = 0; j < VN; ++j) y[j] += bf[j];
            }
            store_vec<VN>(dst + (int64_t)v * VN, y);
        }
    }
    if (lane == 0 && g < groups) {
        mean[g] = mu;
        rstd[g] = r;
    }
}

// Residual add (+ optional clamp) fused in front of the layer norm, fp16 only:
//     x <- clamp(fp16(x + h), lo, hi);   out <- LN(x)
// Bit-identical to running add.Tensor, clamp.default and native_layer_norm one after another
// (each rounds to fp16 where the separate ops would), but x and h are read once and the three
// launches become one.
template <int VPL, int LPG = 32, bool LAT = false>
__global__ void __launch_bounds__(128)
ln_add_warp_kernel(__half* __restrict__ x, const __half* __restrict__ h, __half* __restrict__ out,
                   float* __restrict__ mean, float* __restrict__ rstd, const __half* __restrict__ gamma,
                   const __half* __restrict__ beta, int64_t groups, int C, float eps, int use_clamp, float lo,
                   float hi) {
    constexpr int VN = 8;
    static_assert(LPG == 32 || VPL == 1, "only single-vector groups share a warp");
    const int lane = threadIdx.x & (LPG - 1);
    const int64_t g = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / LPG;
    const int nvec = g < groups ? C / VN : 0;
    // gamma and beta are asked for together with the row (after the dependency wait: the previous kernel may have
    // written them), so that the normalised row does not wait for them at the end.
    // (Rows of up to 1536 elements; wider ones would spill, and read them where they are used.)
    constexpr bool HOIST = LAT && VPL <= 6;
    grid_dep_wait();     // x and h are the previous kernels' outputs
    grid_dep_launch();
    uint4 gw[HOIST ? VPL : 1], bw[HOIST ? VPL : 1];
    if constexpr (HOIST) {
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            const int vi = lane + 32 * i;
            gw[i] = (gamma && vi < nvec) ? __ldg(reinterpret_cast<const uint4*>(gamma) + vi) : make_uint4(0u, 0u, 0u, 0u);
            bw[i] = (beta && vi < nvec) ? __ldg(reinterpret_cast<const uint4*>(beta) + vi) : make_uint4(0u, 0u, 0u, 0u);
        }
    }
    __half* xr = x + g * (int64_t)C;
    const __half* hr = h + g * (int64_t)C;

    float v[VPL][VN];
    float s = 0.f;
    // every load of the row first, then the arithmetic: one round trip for the row whatever the compiler would
    // have made of loads and stores through the same pointer
    // (the latency form; the lean one reads each vector where it uses it)
    uint4 xraw[HOIST ? VPL : 1], hraw[HOIST ? VPL : 1];
    if constexpr (HOIST) {
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            const int vi = lane + 32 * i;
            if (vi < nvec) {
                xraw[i] = *(reinterpret_cast<const uint4*>(xr) + vi);
                hraw[i] = __ldg(reinterpret_cast<const uint4*>(hr) + vi);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int vi = lane + 32 * i;
        if (vi < nvec) {
            Vec16<__half> a, b;
            if constexpr (HOIST) {
                a.raw = xraw[i];
                b.raw = hraw[i];
            } else {
                a.raw = *(reinterpret_cast<const uint4*>(xr) + vi);
                b.raw = __ldg(reinterpret_cast<const uint4*>(hr) + vi);
            }
            float fa[VN], fb[VN];
            a.to_f32(fa);
            b.to_f32(fb);
#pragma unroll
            for (int j = 0; j < VN; ++j) {
                float t = __half2float(__float2half_rn(fa[j] + fb[j]));        // add.Tensor rounds here
                if (use_clamp) t = __half2float(__float2half_rn(fminf(fmaxf(t, lo), hi)));
                v[i][j] = t;
                s += t;
            }
            store_vec<VN>(xr + (int64_t)vi * VN, v[i]);                         // exact: already fp16 values
        }
    }
    const float n = (float)C;
    const float mu = group_sum<LPG>(s) / n;
    float s2 = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i)
        if (lane + 32 * i < nvec) {
#pragma unroll
            for (int j = 0; j < VN; ++j) {
                float d = v[i][j] - mu;
                s2 += d * d;
            }
        }
    const float r = 1.0f / sqrtf(group_sum<LPG>(s2) / n + eps);
    __half* dst = out + g * (int64_t)C;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int vi = lane + 32 * i;
        if (vi < nvec) {
            float y[VN];
#pragma unroll
            for (int j = 0; j < VN; ++j) y[j] = (v[i][j] - mu) * r;
            if (gamma) {
                Vec16<__half> t;
                float gf[VN];
                if constexpr (HOIST) t.raw = gw[i];
                else t.raw = __ldg(reinterpret_cast<const uint4*>(gamma) + vi);
                t.to_f32(gf);
#pragma unroll
                for (int j = 0; j < VN; ++j) y[j] *= gf[j];
            }
            if (beta) {
                Vec16<__half> t;
                float bf[VN];
                if constexpr (HOIST) t.raw = bw[i];
                else t.raw = __ldg(reinterpret_cast<const uint4*>(beta) + vi);
                t.to_f32(bf);
#pragma unroll
                for (int j = 0; j < VN; ++j) y[j] += bf[j];
            }
            store_vec<VN>(dst + (int64_t)vi * VN, y);
        }
    }
    if (lane == 0 && g < groups) {
        mean[g] = mu;
        rstd[g] = r;
    }
}

__device__ __forceinline__ float ldf(const __half* p, int64_t i) { return __half2float(p[i]); }
__device__ __forceinline__ float ldf(const float* p, int64_t i) { return p[i]; }
__device__ __forceinline__ void stf(__half* p, int64_t i, float v) { p[i] = __float2half_rn(v); }
__device__ __forceinline__ void stf(float* p, int64_t i, float v) { p[i] = v; }

__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads();
    if (l == 0) red[w] = v;
    __syncthreads();
    float t = l < nw ? red[l] : 0.f;
    return warp_sum(t);
}

// Any C, any alignment: one block per group, scalar accesses, the group re-read from
// L1/L2 for the second and third pass.
template <typename InT, typename OutT>
__global__ void __launch_bounds__(256)
ln_block_kernel(const InT* __restrict__ a, OutT* __restrict__ out, float* __restrict__ mean,
                float* __restrict__ rstd, const InT* __restrict__ gamma,
                const InT* __restrict__ beta, int64_t C, float eps) {
    __shared__ float red[32];
    const int64_t g = blockIdx.x;
    const InT* src = a + g * C;
    float s = 0.f;
    for (int64_t i = threadIdx.x; i < C; i += blockDim.x) s += ldf(src, i);
    const float n = (float)C;
    const float mu = block_sum(s, red) / n;
    float s2 = 0.f;
    for (int64_t i = threadIdx.x; i < C; i += blockDim.x) {
        float d = ldf(src, i) - mu;
        s2 += d * d;
    }
    const float r = 1.0f / sqrtf(block_sum(s2, red) / n + eps);
    OutT* dst = out + g * C;
    for (int64_t i = threadIdx.x; i < C; i += blockDim.x) {
        float y = (ldf(src, i) - mu) * r;
        if (gamma) y *= ldf(gamma, i);
        if (beta) y += ldf(beta, i);
        stf(dst, i, y);
    }
    if (threadIdx.x == 0) {
        mean[g] = mu;
        rstd[g] = r;
    }
}

template <typename InT, typename OutT>
static int launch_ln(b200_ctx* ctx, int64_t groups, int64_t C, const void* a, void* out, float* mean,
                     float* rstd, const void* gamma, const void* beta, float eps) {
    constexpr int VN = Vec16<InT>::N;
    const InT* ap = static_cast<const InT*>(a);
    OutT* op = static_cast<OutT*>(out);
    const InT* gp = static_cast<const InT*>(gamma);
    const InT* bp = static_cast<const InT*>(beta);
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    const size_t out_vec_bytes = VN * sizeof(OutT);
    bool vec_ok = C % VN == 0 && C / VN <= 32 * 16 && al16(a) && (!gamma || al16(gamma)) &&
                  (!beta || al16(beta)) &&
                  (reinterpret_cast<uintptr_t>(out) % (out_vec_bytes > 16 ? 16 : out_vec_bytes)) == 0;
    if (vec_ok) {
        const int nvec = (int)(C / VN);
        const int vpl = (nvec + 31) / 32;
        const int wpb = 4;
        dim3 grid((unsigned)cdiv(groups, wpb)), block(32 * wpb);
        // few enough rows that every CTA is resident at once: the latency form (see the kernel)
        const bool lat = groups <= (int64_t)4 * wpb * ctx->prop.multiProcessorCount;
#define LN_GO(V)                                                                                            \
    do {                                                                                                    \
        if (lat)                                                                                            \
            B200_CUDA(launch_dep(ln_warp_kernel<InT, OutT, V, 32, true>, grid, block, 0, ctx->stream, 1, ap, op, mean, rstd, gp, \
                                 bp, groups, (int)C, eps));                                                 \
        else                                                                                                \
            B200_CUDA(launch_dep(ln_warp_kernel<InT, OutT, V>, grid, block, 0, ctx->stream, 1, ap, op, mean, rstd, gp, bp, \
                                 groups, (int)C, eps));                                                     \
    } while (0)
#define LN_GO_SHARED(L)                                                                                     \
    B200_CUDA(launch_dep(ln_warp_kernel<InT, OutT, 1, L>, dim3((unsigned)cdiv(groups, wpb * (32 / L))), block, 0,   \
                         ctx->stream, 1, ap, op, mean, rstd, gp, bp, groups, (int)C, eps))
        if (nvec <= 8) LN_GO_SHARED(8);
        else if (nvec <= 16) LN_GO_SHARED(16);
        else if (vpl <= 1) LN_GO(1);
        else if (vpl <= 2) LN_GO(2);
        else if (vpl <= 3) LN_GO(3);
        else if (vpl <= 4) LN_GO(4);
        else if (vpl <= 5) LN_GO(5);
        else if (vpl <= 6) LN_GO(6);
        else if (vpl <= 8) LN_GO(8);
        else if (vpl <= 12) LN_GO(12);
        else LN_GO(16);
#undef LN_GO
#undef LN_GO_SHARED
    } else {
        ln_block_kernel<InT, OutT><<<(unsigned)groups, 256, 0, ctx->stream>>>(ap, op, mean, rstd, gp, bp,
                                                                             C, eps);
    }
    ctx->launches++;
    B200_CUDA(cudaGetLastError());
    return B200_OK;
}

} // namespace b200

using namespace b200;

extern "C" int b200_add_layernorm_f16(b200_ctx* ctx, int64_t groups, int64_t C, void* x, const void* h, int use_clamp,
                                      float lo, float hi, void* out, float* mean, float* rstd, const void* gamma,
                                      const void* beta, float eps) {
    B200_REQUIRE(ctx, B200_EINVAL, "add_layernorm: null ctx");
    B200_REQUIRE(groups >= 0 && C > 0, B200_EINVAL, "add_layernorm: groups=%lld C=%lld", (long long)groups,
                 (long long)C);
    if (groups == 0) return B200_OK;
    B200_REQUIRE(x && h && out && mean && rstd, B200_EINVAL, "add_layernorm: null array");
    B200_REQUIRE(groups < (1ll << 31), B200_DECLINE_EXTENT, "add_layernorm: %lld groups", (long long)groups);
    B200_CUDA(cudaSetDevice(ctx->device));
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    const bool vec = C % 8 == 0 && C / 8 <= 32 * 16 && al16(x) && al16(h) && al16(out) && (!gamma || al16(gamma)) &&
                     (!beta || al16(beta));
    if (!vec) {
        // Shapes the vector kernel does not take: the three ops one after another, same results.
        int rc = b200_add_f16(ctx, x, h, x, groups * C);
        if (rc == B200_OK && use_clamp) rc = b200_clamp_f16(ctx, x, x, groups * C, lo, hi);
        if (rc != B200_OK) return rc;
        return b200_layernorm(ctx, groups, C, x, B200_F16, out, B200_F16, mean, rstd, gamma, beta, eps);
    }
    const int nvec = (int)(C / 8), vpl = (nvec + 31) / 32, wpb = 4;
    dim3 grid((unsigned)cdiv(groups, wpb)), block(32 * wpb);
    const bool lat = groups <= (int64_t)4 * wpb * ctx->prop.multiProcessorCount;   // every CTA resident at once: the latency form
#define LNA_GO(V)                                                                                                 \
    do {                                                                                                          \
        if (lat)                                                                                                  \
            B200_CUDA(launch_dep(ln_add_warp_kernel<V, 32, true>, grid, block, 0, ctx->stream, 1, (__half*)x, (const __half*)h, \
                                 (__half*)out, mean, rstd, (const __half*)gamma, (const __half*)beta, groups, (int)C, eps, \
                                 use_clamp, lo, hi));                                                             \
        else                                                                                                      \
            B200_CUDA(launch_dep(ln_add_warp_kernel<V>, grid, block, 0, ctx->stream, 1, (__half*)x, (const __half*)h,   \
                                 (__half*)out, mean, rstd, (const __half*)gamma, (const __half*)beta, groups, (int)C, eps, \
                                 use_clamp, lo, hi));                                                             \
    } while (0)
#define LNA_GO_SHARED(L)                                                                                          \
    B200_CUDA(launch_dep(ln_add_warp_kernel<1, L>, dim3((unsigned)cdiv(groups, wpb * (32 / L))), block, 0, ctx->stream, 1, \
                         (__half*)x, (const __half*)h, (__half*)out, mean, rstd, (const __half*)gamma,             \
                         (const __half*)beta, groups, (int)C, eps, use_clamp, lo, hi))
    if (nvec <= 8) LNA_GO_SHARED(8);
    else if (nvec <= 16) LNA_GO_SHARED(16);
    else if (vpl <= 1) LNA_GO(1);
    else if (vpl <= 2) LNA_GO(2);
    else if (vpl <= 3) LNA_GO(3);
    else if (vpl <= 4) LNA_GO(4);
    else if (vpl <= 5) LNA_GO(5);
    else if (vpl <= 6) LNA_GO(6);
    else if (vpl <= 8) LNA_GO(8);
    else if (vpl <= 12) LNA_GO(12);
    else LNA_GO(16);
#undef LNA_GO
#undef LNA_GO_SHARED
    ctx->launches++;
    B200_CUDA(cudaGetLastError());
    return B200_OK;
}

extern "C" int b200_layernorm(b200_ctx* ctx, int64_t groups, int64_t C, const void* a, int in_dtype,
                              void* out, int out_dtype, float* mean, float* rstd, const void* gamma,
                              const void* beta, float eps) {
    B200_REQUIRE(ctx, B200_EINVAL, "layernorm: null ctx");
    B200_REQUIRE(groups >= 0 && C > 0, B200_EINVAL, "layernorm: groups=%lld C=%lld", (long long)groups,
                 (long long)C);
    if (groups == 0) return B200_OK;
    B200_REQUIRE(a && out && mean && rstd, B200_EINVAL, "layernorm: null array");
    B200_REQUIRE(groups < (1ll << 31), B200_DECLINE_EXTENT, "layernorm: %lld groups", (long long)groups);
    B200_REQUIRE((in_dtype == B200_F16 || in_dtype == B200_F32) &&
                     (out_dtype == B200_F16 || out_dtype == B200_F32),
                 B200_DECLINE_ELTYPE, "layernorm: dtype %d -> %d", in_dtype, out_dtype);
    B200_CUDA(cudaSetDevice(ctx->device));
    if (in_dtype == B200_F16 && out_dtype == B200_F16)
        return launch_ln<__half, __half>(ctx, groups, C, a, out, mean, rstd, gamma, beta, eps);
    if (in_dtype == B200_F16 && out_dtype == B200_F32)
        return launch_ln<__half, float>(ctx, groups, C, a, out, mean, rstd, gamma, beta, eps);
    if (in_dtype == B200_F32 && out_dtype == B200_F16)
        return launch_ln<float, __half>(ctx, groups, C, a, out, mean, rstd, gamma, beta, eps);
    return launch_ln<float, float>(ctx, groups, C, a, out, mean, rstd, gamma, beta, eps);
}
