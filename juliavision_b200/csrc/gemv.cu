// Matrix-vector product for the one-token case of matmul! (reference kernels/extern/matmul.jl:103-137,
// the MMGemvPlan / Lava.gemv! path): out[m] = epi(T(bias[m] + sum_k A[m,k] x[k])), A (M,K) with M
// contiguous (what hoistpermutes leaves), fp32 accumulation.  Bandwidth-bound: every byte of A is read
// once, 16 bytes per lane along M so a warp covers 512 contiguous bytes of a column, the K axis split
// over the warps of a block and, when M alone cannot fill the GPU, over blocks as well (partials in the
// workspace, summed in a fixed order by a second small kernel, so the result does not depend on timing).
#include <cuda_fp16.h>

#include "act.cuh"
#include "internal.h"

namespace b200 {

template <typename T> __device__ __forceinline__ float gemv_tof(T v);
template <> __device__ __forceinline__ float gemv_tof<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float gemv_tof<float>(float v) { return v; }

// The activation sees the value rounded to the output type (ops.jl:161-169), as in the GEMM's store.
template <typename OutT>
__device__ __forceinline__ void gemv_store(OutT* out, int64_t m, float acc, int epi) {
    if constexpr (sizeof(OutT) == 2) out[m] = __float2half_rn(apply_act(epi, __half2float(__float2half_rn(acc))));
    else out[m] = apply_act(epi, acc);
}

constexpr int GEMV_WARPS = 8;

// grid (m blocks, k splits); block (32, GEMV_WARPS).  VEC rows of M per lane.
template <typename T, typename OutT, int VEC>
__global__ void __launch_bounds__(32 * GEMV_WARPS)
gemv_kernel(const T* __restrict__ A, int64_t lda, const T* __restrict__ x, const T* __restrict__ bias, OutT* __restrict__ out,
            float* __restrict__ partial, int64_t M, int64_t K, int64_t kchunk, int epi) {
    __shared__ float red[GEMV_WARPS][32 * VEC];
    const int lane = threadIdx.x, warp = threadIdx.y;
    const int64_t m0 = ((int64_t)blockIdx.x * 32 + lane) * VEC;
    const int64_t k0 = (int64_t)blockIdx.y * kchunk;
    const int64_t k1 = k0 + kchunk < K ? k0 + kchunk : K;
    float acc[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) acc[v] = 0.f;
    if (m0 < M) {
        // Four columns of A in flight per lane: the loop is otherwise one load deep and latency-bound.
        constexpr int UN = 4;
        int64_t k = k0 + warp;
        for (; k + (UN - 1) * GEMV_WARPS < k1; k += UN * GEMV_WARPS) {
            T a[UN][VEC];
            float xv[UN];
#pragma unroll
            for (int u = 0; u < UN; ++u) {
                const T* col = A + (k + u * GEMV_WARPS) * lda + m0;
                if constexpr (VEC > 1) *reinterpret_cast<uint4*>(a[u]) = __ldg(reinterpret_cast<const uint4*>(col));
                else a[u][0] = col[0];
                xv[u] = gemv_tof<T>(x[k + u * GEMV_WARPS]);
            }
#pragma unroll
            for (int u = 0; u < UN; ++u)
#pragma unroll
                for (int v = 0; v < VEC; ++v) acc[v] = fmaf(gemv_tof<T>(a[u][v]), xv[u], acc[v]);
        }
        for (; k < k1; k += GEMV_WARPS) {
            const float xv = gemv_tof<T>(x[k]);
            const T* col = A + k * lda + m0;
            if constexpr (VEC > 1) {
                T a[VEC];
                *reinterpret_cast<uint4*>(a) = __ldg(reinterpret_cast<const uint4*>(col));
#pragma unroll
                for (int v = 0; v < VEC; ++v) acc[v] = fmaf(gemv_tof<T>(a[v]), xv, acc[v]);
            } else {
                acc[0] = fmaf(gemv_tof<T>(col[0]), xv, acc[0]);
            }
        }
    }
#pragma unroll
    for (int v = 0; v < VEC; ++v) red[warp][lane * VEC + v] = acc[v];
    __syncthreads();
    // warp w finishes rows w, w + GEMV_WARPS, ... of the block's 32 * VEC
    for (int r = warp * 32 + lane; r < 32 * VEC; r += 32 * GEMV_WARPS) {
        const int64_t m = (int64_t)blockIdx.x * 32 * VEC + r;
        if (m >= M) continue;
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < GEMV_WARPS; ++w) s += red[w][r];
        if (partial != nullptr) {
            partial[(int64_t)blockIdx.y * M + m] = s;
        } else {
            if (bias != nullptr) s += gemv_tof<T>(bias[m]);
            gemv_store<OutT>(out, m, s, epi);
        }
    }
}

template <typename T, typename OutT>
__global__ void __launch_bounds__(256)
gemv_finish_kernel(const float* __restrict__ partial, int ksplit, const T* __restrict__ bias, OutT* __restrict__ out, int64_t M,
                   int epi) {
    const int64_t m = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (m >= M) return;
    float s = 0.f;
    for (int j = 0; j < ksplit; ++j) s += partial[(int64_t)j * M + m];
    if (bias != nullptr) s += gemv_tof<T>(bias[m]);
    gemv_store<OutT>(out, m, s, epi);
}

template <typename T, typename OutT>
static int gemv_run(b200_ctx* ctx, int64_t M, int64_t K, const void* A, int64_t lda, const void* x, const void* bias, void* out,
                    int epi) {
    constexpr int VECMAX = 16 / (int)sizeof(T);
    const bool vec = lda % VECMAX == 0 && (reinterpret_cast<uintptr_t>(A) & 15u) == 0;
    const int rows_per_block = 32 * (vec ? VECMAX : 1);
    const int64_t mblocks = cdiv(M, rows_per_block);
    // Enough blocks to keep every SM's memory pipe busy, but at least 16 k-steps per warp each.
    const int64_t want = (int64_t)ctx->prop.multiProcessorCount * 6;
    int64_t ksplit = mblocks >= want ? 1 : cdiv(want, mblocks);
    const int64_t maxsplit = K / (16 * GEMV_WARPS) > 0 ? K / (16 * GEMV_WARPS) : 1;
    if (ksplit > maxsplit) ksplit = maxsplit;
    if (ksplit > 64) ksplit = 64;
    const int64_t kchunk = cdiv(K, ksplit);
    ksplit = cdiv(K, kchunk);
    float* partial = nullptr;
    if (ksplit > 1) {
        void* ws = nullptr;
        int rc = ws_scratch(ctx, (size_t)ksplit * M * sizeof(float), &ws);
        if (rc) return rc;
        partial = static_cast<float*>(ws);
    }
    B200_REQUIRE(mblocks < (1ll << 31), B200_DECLINE_EXTENT, "gemv: M = %lld", (long long)M);
    dim3 grid((unsigned)mblocks, (unsigned)ksplit), block(32, GEMV_WARPS);
    if (vec)
        gemv_kernel<T, OutT, VECMAX><<<grid, block, 0, ctx->stream>>>((const T*)A, lda, (const T*)x, (const T*)bias, (OutT*)out,
                                                                      partial, M, K, kchunk, epi);
    else
        gemv_kernel<T, OutT, 1><<<grid, block, 0, ctx->stream>>>((const T*)A, lda, (const T*)x, (const T*)bias, (OutT*)out,
                                                                 partial, M, K, kchunk, epi);
    ctx->launches++;
    B200_CUDA(cudaGetLastError());
    if (partial != nullptr) {
        gemv_finish_kernel<T, OutT><<<(unsigned)cdiv(M, 256), 256, 0, ctx->stream>>>(partial, (int)ksplit, (const T*)bias,
                                                                                  (OutT*)out, M, epi);
        ctx->launches++;
        B200_CUDA(cudaGetLastError());
    }
    return B200_OK;
}

} // namespace b200

using namespace b200;

extern "C" {

int b200_gemv(b200_ctx* ctx, int64_t M, int64_t K, const void* A, int64_t lda, const void* x, const void* bias, int in_dtype,
              void* out, int out_dtype, int epilogue) {
    B200_REQUIRE(ctx, B200_EINVAL, "gemv: null context");
    B200_REQUIRE(M >= 0 && K >= 0 && lda >= (M > 0 ? M : 1), B200_EINVAL, "gemv: M=%lld K=%lld lda=%lld", (long long)M,
                 (long long)K, (long long)lda);
    B200_REQUIRE(in_dtype == B200_F16 || in_dtype == B200_F32, B200_DECLINE_ELTYPE, "gemv: operand dtype %d", in_dtype);
    B200_REQUIRE(out_dtype == B200_F32 || (out_dtype == B200_F16 && in_dtype == B200_F16), B200_DECLINE_ELTYPE,
                 "gemv: out dtype %d for operand dtype %d", out_dtype, in_dtype);
    B200_REQUIRE(epilogue >= B200_EPI_NONE && epilogue <= B200_EPI_GELU_TANH, B200_EINVAL, "gemv: epilogue %d", epilogue);
    if (M == 0) return B200_OK;
    B200_REQUIRE(out && (K == 0 || (A && x)), B200_EINVAL, "gemv: null array");
    B200_CUDA(cudaSetDevice(ctx->device));
    if (in_dtype == B200_F32) return gemv_run<float, float>(ctx, M, K, A, lda, x, bias, out, epilogue);
    if (out_dtype == B200_F16) return gemv_run<__half, __half>(ctx, M, K, A, lda, x, bias, out, epilogue);
    return gemv_run<__half, float>(ctx, M, K, A, lda, x, bias, out, epilogue);
}

} // extern "C"
