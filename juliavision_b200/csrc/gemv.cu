// Matrix-vector product for the one-token case of matmul! (reference kernels/extern/matmul.jl:103-137,
// the MMGemvPlan / Lava.gemv! path): out[m] = epi(T(bias[m] + sum_k A[m,k] x[k])), A (M,K) with M
// contiguous (what hoistpermutes leaves), fp32 accumulation.  Bandwidth-bound: every byte of A is read
// once, as aligned 16-byte vectors whatever the leading dimension (a vocabulary of 51865 rows gives
// every column its own misalignment), a warp covering 512 contiguous bytes of a column, the K axis
// split over the warps of a block and, when M alone cannot fill the GPU, over blocks as well (partials
// in the workspace, summed in a fixed order by whichever block of a row range finishes last, so the
// result does not depend on timing).
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
constexpr int GEMV_UNROLL = 4;          // columns in flight per lane: 64 bytes (8 measured no faster)
constexpr int GEMV_BLOCKS_PER_SM = 6;   // resident blocks of 256 threads at 40 registers
constexpr int GEMV_MIN_COLS = 16;       // columns per warp below which a further K split only adds launch work
#define GEMV_SPLIT_ROUND(a, b) ((a) / (b))

// grid (m blocks, k splits); block (32, GEMV_WARPS).
//
// Warp w takes columns k0 + w, k0 + w + 8, ...  Their start addresses differ by multiples of
// 8 * lda * sizeof(T), a multiple of 16 bytes, so all of one warp's columns sit at the same offset s
// (in elements) from a 16-byte boundary.  The warp therefore keeps its accumulators aligned to memory,
// not to rows: lane l reads the aligned vector j = 31 * block + l of each column, whose VEC elements
// are rows VEC * j - s ... VEC * j - s + VEC - 1, with no shifting or masking in the loop.  A block owns
// 31 * VEC rows; the 32 vectors its lanes read cover them for every s (the neighbouring blocks read the
// first and last of them again, out of L2).  Elements a vector holds outside [0, M) (the end of the
// previous column, the start of the next, or the rest of an aligned 16-byte block at either end of the
// array) only reach accumulators that are thrown away; every vector read holds at least one element of
// A, so no read leaves the 16-byte blocks the array occupies.
template <typename T, typename OutT>
__global__ void __launch_bounds__(32 * GEMV_WARPS, GEMV_BLOCKS_PER_SM)
gemv_kernel(const T* __restrict__ A, int64_t lda, const T* __restrict__ x, const T* __restrict__ bias, OutT* __restrict__ out,
            float* __restrict__ partial, int* __restrict__ arrived, int64_t M, int64_t K, int64_t kchunk, int epi) {
    constexpr int VEC = 16 / (int)sizeof(T);
    constexpr int ROWS = 31 * VEC;
    __shared__ float red[GEMV_WARPS][ROWS];
    __shared__ int last;
    const int lane = threadIdx.x, warp = threadIdx.y;
    const int64_t k0 = (int64_t)blockIdx.y * kchunk;
    const int64_t k1 = k0 + kchunk < K ? k0 + kchunk : K;
    const int64_t j = (int64_t)blockIdx.x * 31 + lane;
    float acc[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) acc[v] = 0.f;
    int s = 0;
    int64_t k = k0 + warp;
    if (k < k1) {
        s = (int)((reinterpret_cast<uintptr_t>(A + k * lda) & 15u) / sizeof(T));
        if (VEC * j - s < M) {
            // first aligned vector of column k, then + j; columns are 8 * lda elements apart
            const uint4* vp = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(A + k * lda) - s * sizeof(T)) + j;
            const int64_t vstep = GEMV_WARPS * lda * (int64_t)sizeof(T) / 16;
            constexpr int UN = GEMV_UNROLL;
            for (; k + (UN - 1) * GEMV_WARPS < k1; k += UN * GEMV_WARPS, vp += UN * vstep) {
                uint4 a[UN];
                float xv[UN];
#pragma unroll
                for (int u = 0; u < UN; ++u) {
                    a[u] = __ldg(vp + u * vstep);
                    xv[u] = gemv_tof<T>(x[k + u * GEMV_WARPS]);
                }
#pragma unroll
                for (int u = 0; u < UN; ++u) {
                    const T* e = reinterpret_cast<const T*>(&a[u]);
#pragma unroll
                    for (int v = 0; v < VEC; ++v) acc[v] = fmaf(gemv_tof<T>(e[v]), xv[u], acc[v]);
                }
            }
            for (; k < k1; k += GEMV_WARPS, vp += vstep) {
                const uint4 a = __ldg(vp);
                const float xv = gemv_tof<T>(x[k]);
                const T* e = reinterpret_cast<const T*>(&a);
#pragma unroll
                for (int v = 0; v < VEC; ++v) acc[v] = fmaf(gemv_tof<T>(e[v]), xv, acc[v]);
            }
        }
    }
    // accumulator v of lane l is row VEC * l + v - s of the block
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
        const int r = VEC * lane + v - s;
        if (r >= 0 && r < ROWS) red[warp][r] = acc[v];
    }
    __syncthreads();
    for (int r = warp * 32 + lane; r < ROWS; r += 32 * GEMV_WARPS) {
        const int64_t m = (int64_t)blockIdx.x * ROWS + r;
        if (m >= M) continue;
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < GEMV_WARPS; ++w) t += red[w][r];
        if (partial != nullptr) {
            partial[(int64_t)blockIdx.y * M + m] = t;
        } else {
            if (bias != nullptr) t += gemv_tof<T>(bias[m]);
            gemv_store<OutT>(out, m, t, epi);
        }
    }
    if (partial == nullptr || arrived == nullptr) return;
    // K was split over gridDim.y blocks: the one that arrives last adds the partial sums of these rows in
    // split order (so the result does not depend on which block that is) and puts the counter back to zero
    // for the next launch.  Nobody waits on anybody.
    __threadfence();
    __syncthreads();
    if (warp == 0 && lane == 0) last = atomicAdd(arrived + blockIdx.x, 1) == (int)gridDim.y - 1;
    __syncthreads();
    if (!last) return;
    __threadfence();
    for (int r = warp * 32 + lane; r < ROWS; r += 32 * GEMV_WARPS) {
        const int64_t m = (int64_t)blockIdx.x * ROWS + r;
        if (m >= M) continue;
        float t = 0.f;
        for (unsigned y = 0; y < gridDim.y; ++y) t += __ldcg(partial + (int64_t)y * M + m);
        if (bias != nullptr) t += gemv_tof<T>(bias[m]);
        gemv_store<OutT>(out, m, t, epi);
    }
    if (warp == 0 && lane == 0) arrived[blockIdx.x] = 0;
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
    constexpr int ROWS = 31 * (16 / (int)sizeof(T));
    const int64_t mblocks = cdiv(M, ROWS);
    // Split K over blocks until the grid is one resident wave (a second, partial wave would cost a whole
    // extra pass of latency), keeping at least GEMV_MIN_COLS columns per warp in every split.
    const int64_t wave = (int64_t)ctx->prop.multiProcessorCount * GEMV_BLOCKS_PER_SM;
    int64_t ksplit = mblocks >= wave ? 1 : GEMV_SPLIT_ROUND(wave, mblocks);
    const int64_t maxsplit = K / (GEMV_MIN_COLS * GEMV_WARPS) > 0 ? K / (GEMV_MIN_COLS * GEMV_WARPS) : 1;
    if (ksplit > maxsplit) ksplit = maxsplit;
    if (ksplit > 64) ksplit = 64;
    const int64_t kchunk = K > 0 ? cdiv(K, ksplit) : 1;   // K = 0: one block per row range writes the bias
    ksplit = K > 0 ? cdiv(K, kchunk) : 1;
    float* partial = nullptr;
    if (ksplit > 1) {
        void* ws = nullptr;
        int rc = ws_scratch(ctx, (size_t)ksplit * M * sizeof(float), &ws);
        if (rc) return rc;
        partial = static_cast<float*>(ws);
    }
    B200_REQUIRE(mblocks < (1ll << 31), B200_DECLINE_EXTENT, "gemv: M = %lld", (long long)M);
    dim3 grid((unsigned)mblocks, (unsigned)ksplit), block(32, GEMV_WARPS);
    int* arrived = partial != nullptr && mblocks <= GEMV_COUNTER_COUNT && ctx->sk_flags != nullptr ? ctx->sk_flags + SK_FLAG_COUNT : nullptr;
    gemv_kernel<T, OutT><<<grid, block, 0, ctx->stream>>>((const T*)A, lda, (const T*)x, (const T*)bias, (OutT*)out, partial,
                                                          arrived, M, K, kchunk, epi);
    ctx->launches++;
    B200_CUDA(cudaGetLastError());
    if (partial != nullptr && arrived == nullptr) {
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
    B200_REQUIRE(reinterpret_cast<uintptr_t>(A) % (in_dtype == B200_F32 ? 4 : 2) == 0, B200_DECLINE_ALIGN,
                 "gemv: A is not aligned to its element size");
    B200_CUDA(cudaSetDevice(ctx->device));
    if (in_dtype == B200_F32) return gemv_run<float, float>(ctx, M, K, A, lda, x, bias, out, epilogue);
    if (out_dtype == B200_F16) return gemv_run<__half, __half>(ctx, M, K, A, lda, x, bias, out, epilogue);
    return gemv_run<__half, float>(ctx, M, K, A, lda, x, bias, out, epilogue);
}

} // extern "C"
