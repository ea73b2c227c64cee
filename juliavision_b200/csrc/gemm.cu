// fp16 GEMM with fp32 accumulation on the sm_100a tensor cores (tcgen05 / TMEM), operands
// staged by TMA through an mbarrier ring, bias + activation + conversion fused into the
// store, and a tile planner with predicated (TMA-clipped) tails in place of padding.
//
// In the reference's orientation (column-major, reversed torch shapes):
//     out(M,N) = epi(T(bias[i] + sum_k A(M,K)[i,k] * B(K,N)[k,j]))
// A is the dense weight (M = out features, contiguous), B the activations (K contiguous,
// N = tokens).  On the tensor core the token axis rides the 128 TMEM lanes and the feature
// axis the accumulator columns, i.e. per tile
//     D[128 tokens, BN features] += Bt[128 tokens, 64 k] (K-major) * A[64 k, BN features] (MN-major)
//
// Replaces matmul_coopmat! + Lava.coopmat_gemm! + padcols_kernel! + mm_epilogue_kernel!
// (reference kernels/extern/matmul.jl:172-273).
//
// Roles inside one persistent CTA (192 threads):
//   warp 0    TMA producer  (one lane)        global -> shared ring, STAGES deep
//   warp 1    UMMA issuer   (one lane)        shared -> TMEM accumulators (two, ping-pong)
//   warps 2-5 epilogue      (128 threads)     TMEM -> registers -> +bias, round, act ->
//                                             swizzled shared staging -> TMA store
#include <cuda_fp16.h>

#include "internal.h"
#include "ptx.cuh"

namespace b200 {

constexpr int GEMM_BM = 128; // tokens per tile (TMEM lanes)
constexpr int GEMM_BK = 64;  // one 128-byte swizzle row of fp16
constexpr int GEMM_THREADS = 192;
constexpr int SMEM_LIMIT = 232448; // 227 KB

template <int BN, typename OutT> struct GemmCfg {
    static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
    static constexpr int B_CHUNK_BYTES = 64 * GEMM_BK * 2; // one 64-feature slab of the B tile
    static constexpr int B_BYTES = BN * GEMM_BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int OUT_COLS = 128 / (int)sizeof(OutT); // columns per 128-byte staging row
    static constexpr int STG_BYTES = GEMM_BM * 128;
    static constexpr int TAIL_BYTES = 2 * STG_BYTES + BN * 4 + 256;
    static constexpr int STAGES_RAW = (SMEM_LIMIT - 1024 - TAIL_BYTES) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
    static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + TAIL_BYTES;
    static constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
    static_assert(STAGES >= 2, "ring too shallow");
    static_assert(SMEM_BYTES <= SMEM_LIMIT, "shared memory over budget");
    static_assert(TMEM_COLS == 128 || TMEM_COLS == 256 || TMEM_COLS == 512, "TMEM columns");
};

struct GemmParams {
    int64_t M, N, K;       // out features, tokens, reduction
    int tiles_m, tiles_n;  // feature tiles, token tiles
    int64_t total_tiles;   // tiles_m * tiles_n * nbatch
    int num_kb;
    const __half* bias;
    int bias_per_n;        // 0: bias[i] over features (M); 1: bias[j] over tokens (N)
    int epilogue;
    int* d_status;
};

__device__ __forceinline__ float erf_as(float x) {
    // Abramowitz & Stegun 7.1.26 in fp32, the reference's erf (ops.jl:161-169).
    float a = fabsf(x);
    float t = __fdividef(1.0f, 1.0f + 0.3275911f * a);
    float y = 1.0f - (((((1.061405429f * t - 1.453152027f) * t) + 1.421413741f) * t - 0.284496736f) * t +
                      0.254829592f) * t * __expf(-a * a);
    return x < 0.f ? -y : y;
}
__device__ __forceinline__ float apply_act(int epi, float v) {
    switch (epi) {
        case B200_EPI_RELU: return fmaxf(v, 0.f);
        case B200_EPI_GELU: return 0.5f * v * (1.0f + erf_as(v * 0.70710678118654752f));
        case B200_EPI_GELU_TANH: {
            float u = 0.7978845608028654f * (v + 0.044715f * v * v * v);
            return 0.5f * v * (1.0f + tanhf(u));
        }
        default: return v;
    }
}

template <int BN, typename OutT>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_f16_tc_kernel(const __grid_constant__ CUtensorMap tmapX,   // B(K,N): {K, tokens, batch}
                   const __grid_constant__ CUtensorMap tmapW,   // A(M,K): {features, K, batch}
                   const __grid_constant__ CUtensorMap tmapO,   // out(M,N): {features, tokens, batch}
                   const GemmParams p) {
    using Cfg = GemmCfg<BN, OutT>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~uintptr_t(1023));
    uint8_t* stg = smem + Cfg::STAGES * Cfg::STAGE_BYTES;
    float* sbias = reinterpret_cast<float*>(stg + 2 * Cfg::STG_BYTES);
    uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(sbias) + BN * 4);
    uint64_t* full = bars;                     // [STAGES]
    uint64_t* empty = bars + Cfg::STAGES;      // [STAGES]
    uint64_t* tfull = bars + 2 * Cfg::STAGES;  // [2]
    uint64_t* tempty = tfull + 2;              // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&tfull[a], 1);
            mbar_init(&tempty[a], 4);
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tmap(&tmapX);
        prefetch_tmap(&tmapW);
        prefetch_tmap(&tmapO);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int64_t tiles_per_batch = (int64_t)p.tiles_m * p.tiles_n;

    if (warp == 0) {
        // ------------------------------------------------------------- TMA producer
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int64_t tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x) {
                const int batch = (int)(tile / tiles_per_batch);
                const int rem = (int)(tile % tiles_per_batch);
                const int m0 = (rem % p.tiles_m) * BN;
                const int n0 = (rem / p.tiles_m) * GEMM_BM;
                for (int kb = 0; kb < p.num_kb; ++kb) {
                    if (!mbar_wait(&empty[s], ph ^ 1, p.d_status, KST_WAIT_EMPTY, abort_flag)) {
                        ok = false;
                        break;
                    }
                    uint8_t* sa = smem + s * Cfg::STAGE_BYTES;
                    uint8_t* sb = sa + Cfg::A_BYTES;
                    mbar_arrive_expect_tx(&full[s], Cfg::STAGE_BYTES);
                    tma_load_3d(sa, &tmapX, &full[s], kb * GEMM_BK, n0, batch);
#pragma unroll
                    for (int j = 0; j < BN / 64; ++j)
                        tma_load_3d(sb + j * Cfg::B_CHUNK_BYTES, &tmapW, &full[s], m0 + j * 64,
                                    kb * GEMM_BK, batch);
                    if (++s == Cfg::STAGES) { s = 0; ph ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------- UMMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_f16(GEMM_BM, BN, /*a K-major*/ 0, /*b MN-major*/ 1);
            constexpr uint64_t adesc0 = make_smem_desc(16, 1024);
            constexpr uint64_t bdesc0 = make_smem_desc(Cfg::B_CHUNK_BYTES, 1024);
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            int64_t it = 0;
            for (int64_t tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x, ++it) {
                const int acc = (int)(it & 1);
                const uint32_t aph = (uint32_t)((it >> 1) & 1);
                if (!mbar_wait(&tempty[acc], aph ^ 1, p.d_status, KST_WAIT_TMEM_EMPTY, abort_flag)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < p.num_kb; ++kb) {
                    if (!mbar_wait(&full[s], ph, p.d_status, KST_WAIT_FULL, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem + s * Cfg::STAGE_BYTES);
                    const uint32_t b_addr = a_addr + Cfg::A_BYTES;
#pragma unroll
                    for (int k = 0; k < GEMM_BK / 16; ++k) {
                        // K-major A: +16 elements of K = +32 B inside the swizzle row.
                        // MN-major B: +16 k-rows = two 8-row groups = +2048 B.
                        umma_ss(d_tmem, smem_desc_at(adesc0, a_addr + k * 32),
                                smem_desc_at(bdesc0, b_addr + k * 2048), idesc, (kb | k) != 0);
                    }
                    umma_commit(&empty[s]);
                    if (++s == Cfg::STAGES) { s = 0; ph ^= 1; }
                }
                if (ok) umma_commit(&tfull[acc]);
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue
        const int et = threadIdx.x - 64;       // 0..127
        const int quad = warp & 3;             // TMEM lane quadrant this warp may read
        const int row = quad * 32 + lane;      // token row inside the tile
        uint32_t chunk_ctr = 0;
        int64_t it = 0;
        for (int64_t tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, ++it) {
            const int batch = (int)(tile / tiles_per_batch);
            const int rem = (int)(tile % tiles_per_batch);
            const int m0 = (rem % p.tiles_m) * BN;
            const int n0 = (rem / p.tiles_m) * GEMM_BM;
            const int acc = (int)(it & 1);
            const uint32_t aph = (uint32_t)((it >> 1) & 1);

            named_bar_sync(1, 128); // previous tile's bias readers are done
            for (int j = et; j < BN; j += 128)
                sbias[j] = (p.bias != nullptr && !p.bias_per_n && m0 + j < p.M) ? __half2float(p.bias[m0 + j]) : 0.f;
            const float rbias =
                (p.bias != nullptr && p.bias_per_n && n0 + row < p.N) ? __half2float(p.bias[n0 + row]) : 0.f;
            const bool got = mbar_wait(&tfull[acc], aph, p.d_status, KST_WAIT_TMEM_FULL, abort_flag);
            // One answer for all 128 threads: a split decision would strand the rest at the
            // barriers inside the chunk loop.
            if (named_bar_or(1, 128, !got || *abort_flag != 0)) break;
            tc_fence_after();

            constexpr int NCHUNK = BN / Cfg::OUT_COLS;
#pragma unroll 1
            for (int c = 0; c < NCHUNK; ++c) {
                const int col0 = c * Cfg::OUT_COLS;
                float v[Cfg::OUT_COLS];
                {
                    const uint32_t taddr = tmem_base + (uint32_t(quad * 32) << 16) + acc * BN + col0;
                    uint32_t r[32];
                    tmem_ld32(taddr, r);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) + rbias;
                    if constexpr (Cfg::OUT_COLS == 64) {
                        tmem_ld32(taddr + 32, r);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[32 + i] = __uint_as_float(r[i]) + rbias;
                    }
                }
                if (c == NCHUNK - 1) {
                    // Accumulator fully read: hand it back to the UMMA issuer.
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&tempty[acc]);
                }
                if (m0 + col0 >= p.M) continue; // whole chunk past the feature extent

                uint8_t* buf = stg + (chunk_ctr & 1) * Cfg::STG_BYTES;
                ++chunk_ctr;
                if (et == 0) tma_store_wait_read<1>(); // the store that last read `buf` is done
                named_bar_sync(1, 128);

                uint8_t* rowp = buf + row * 128;
                if constexpr (sizeof(OutT) == 2) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        uint4 o;
                        __half2* h = reinterpret_cast<__half2*>(&o);
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const int cidx = j * 8 + q * 2;
                            // Round to fp16 first; the activation sees the rounded value.
                            __half2 t = __floats2half2_rn(v[cidx] + sbias[col0 + cidx],
                                                          v[cidx + 1] + sbias[col0 + cidx + 1]);
                            if (p.epilogue != B200_EPI_NONE) {
                                float2 f = __half22float2(t);
                                t = __floats2half2_rn(apply_act(p.epilogue, f.x), apply_act(p.epilogue, f.y));
                            }
                            h[q] = t;
                        }
                        *reinterpret_cast<uint4*>(rowp + ((j ^ (row & 7)) << 4)) = o;
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        float4 o;
                        o.x = apply_act(p.epilogue, v[j * 4 + 0] + sbias[col0 + j * 4 + 0]);
                        o.y = apply_act(p.epilogue, v[j * 4 + 1] + sbias[col0 + j * 4 + 1]);
                        o.z = apply_act(p.epilogue, v[j * 4 + 2] + sbias[col0 + j * 4 + 2]);
                        o.w = apply_act(p.epilogue, v[j * 4 + 3] + sbias[col0 + j * 4 + 3]);
                        *reinterpret_cast<float4*>(rowp + ((j ^ (row & 7)) << 4)) = o;
                    }
                }
                fence_proxy_async_smem();
                named_bar_sync(1, 128);
                if (et == 0) {
                    tma_store_3d(&tmapO, buf, m0 + col0, n0, batch);
                    tma_store_commit();
                }
            }
        }
        if (et == 0) tma_store_wait_all<0>();
    }

    // Teardown: every role arrives here whether it finished or gave up.
    if (*abort_flag) {
        // Let any TMA copy still in flight into this CTA's shared memory land before exit.
        for (int i = 0; i < 4; ++i) __nanosleep(1000000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

// Scalar path for operands the tensor maps cannot express (unaligned pointers or leading
// dimensions): one thread per output, fp32 fma chain in ascending k from the bias — the
// arithmetic of the reference's mm2 (matmul.jl:17-28), bit for bit.
template <typename OutT>
__global__ void gemm_f16_scalar_kernel(int64_t M, int64_t N, int64_t K, const __half* A, int64_t lda,
                                       const __half* B, int64_t ldb, const __half* bias, int bias_per_n,
                                       OutT* out, int64_t ldo, int epi, int64_t sA, int64_t sB, int64_t sO) {
    const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    const int64_t j = blockIdx.y;
    const int64_t b = blockIdx.z;
    if (i >= M) return;
    const __half* a = A + sA * b + i;
    const __half* bb = B + sB * b + ldb * j;
    float acc = bias ? __half2float(bias[bias_per_n ? j : i]) : 0.f;
    for (int64_t k = 0; k < K; ++k) acc = fmaf(__half2float(a[lda * k]), __half2float(bb[k]), acc);
    if constexpr (sizeof(OutT) == 2) {
        float r = __half2float(__float2half_rn(acc));
        out[sO * b + i + ldo * j] = __float2half_rn(apply_act(epi, r));
    } else {
        out[sO * b + i + ldo * j] = apply_act(epi, acc);
    }
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Tile planner: feature-tile width BN in {256,128,64} minimising (waves x tile cost), the
// cost of a tile taken as proportional to BN plus a fixed per-tile overhead.
static int pick_bn(int64_t M, int64_t N, int64_t nbatch, int sms) {
    int best = 256;
    double best_cost = 1e300;
    const int cands[3] = {256, 128, 64};
    for (int bn : cands) {
        int64_t tiles = cdiv(M, bn) * cdiv(N, GEMM_BM) * nbatch;
        int64_t waves = cdiv(tiles, sms);
        // Narrow tiles re-read the activation tile more often and run the tensor core below
        // its shared-memory feed rate: weight them accordingly.
        double eff = bn == 256 ? 1.0 : (bn == 128 ? 1.1 : 1.5);
        double cost = (double)waves * (bn * eff + 24.0);
        if (cost < best_cost) {
            best_cost = cost;
            best = bn;
        }
    }
    return best;
}

template <int BN, typename OutT>
static int launch_tc(b200_ctx* ctx, int64_t M, int64_t N, int64_t K, const void* A, int64_t lda,
                     const void* B, int64_t ldb, const void* bias, int bias_per_n, void* out, int64_t ldo,
                     int epi, int64_t nbatch, int64_t sA, int64_t sB, int64_t sO) {
    using Cfg = GemmCfg<BN, OutT>;
    static bool attr_done[16] = {};
    auto kern = gemm_f16_tc_kernel<BN, OutT>;
    if (!attr_done[ctx->device & 15]) {
        B200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
        attr_done[ctx->device & 15] = true;
    }
    CUtensorMap tX, tW, tO;
    {
        uint64_t dims[3] = {(uint64_t)K, (uint64_t)N, (uint64_t)nbatch};
        uint64_t str[2] = {(uint64_t)ldb * 2, (uint64_t)(nbatch > 1 ? sB : ldb * N) * 2};
        uint32_t box[3] = {GEMM_BK, GEMM_BM, 1};
        int rc = make_tmap(ctx, &tX, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, B, dims, str, box,
                           CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
    }
    {
        uint64_t dims[3] = {(uint64_t)M, (uint64_t)K, (uint64_t)nbatch};
        uint64_t str[2] = {(uint64_t)lda * 2, (uint64_t)(nbatch > 1 ? sA : lda * K) * 2};
        uint32_t box[3] = {64, GEMM_BK, 1};
        int rc = make_tmap(ctx, &tW, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, A, dims, str, box,
                           CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
    }
    {
        uint64_t dims[3] = {(uint64_t)M, (uint64_t)N, (uint64_t)nbatch};
        uint64_t str[2] = {(uint64_t)ldo * sizeof(OutT), (uint64_t)(nbatch > 1 ? sO : ldo * N) * sizeof(OutT)};
        uint32_t box[3] = {(uint32_t)Cfg::OUT_COLS, GEMM_BM, 1};
        int rc = make_tmap(ctx, &tO, sizeof(OutT) == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                       : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                           3, out, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
    }
    GemmParams p;
    p.M = M; p.N = N; p.K = K;
    p.tiles_m = (int)cdiv(M, BN);
    p.tiles_n = (int)cdiv(N, GEMM_BM);
    p.total_tiles = (int64_t)p.tiles_m * p.tiles_n * nbatch;
    p.num_kb = (int)cdiv(K, GEMM_BK);
    p.bias = static_cast<const __half*>(bias);
    p.bias_per_n = bias_per_n;
    p.epilogue = epi;
    p.d_status = ctx->d_status;
    int grid = (int)(p.total_tiles < ctx->prop.multiProcessorCount ? p.total_tiles
                                                                   : ctx->prop.multiProcessorCount);
    kern<<<grid, GEMM_THREADS, Cfg::SMEM_BYTES, ctx->stream>>>(tX, tW, tO, p);
    ctx->launches++;
    B200_CUDA(cudaGetLastError());
    return B200_OK;
}

static int tc_supported(int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldo,
                        int out_dtype) {
    if (M < 1 || N < 1 || K < 1) return B200_DECLINE_EXTENT;
    if (out_dtype != B200_F16 && out_dtype != B200_F32) return B200_DECLINE_ELTYPE;
    const int64_t oal = out_dtype == B200_F16 ? 8 : 4;
    if (lda % 8 || ldb % 8 || ldo % oal) return B200_DECLINE_ALIGN;
    if (lda < M || ldb < K || ldo < M) return B200_EINVAL;
    if (M >= (1ll << 31) || N >= (1ll << 31) || K >= (1ll << 31)) return B200_DECLINE_EXTENT;
    return B200_OK;
}

} // namespace b200

using namespace b200;

extern "C" {

int b200_gemm_f16_supported(int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldo,
                            int out_dtype) {
    return tc_supported(M, N, K, lda, ldb, ldo, out_dtype);
}

int b200_gemm_f16_plan(b200_ctx* ctx, int64_t M, int64_t N, int64_t K, int64_t nbatch,
                       b200_gemm_plan_t* plan) {
    B200_REQUIRE(ctx && plan, B200_EINVAL, "gemm_plan: null argument");
    B200_REQUIRE(M >= 1 && N >= 1 && K >= 1 && nbatch >= 1, B200_DECLINE_EXTENT, "gemm_plan: empty extent");
    const int sms = ctx->prop.multiProcessorCount;
    int bn = pick_bn(M, N, nbatch, sms);
    plan->block_m = GEMM_BM;
    plan->block_n = bn;
    plan->block_k = GEMM_BK;
    plan->stages = bn == 256 ? GemmCfg<256, __half>::STAGES
                             : (bn == 128 ? GemmCfg<128, __half>::STAGES : GemmCfg<64, __half>::STAGES);
    plan->smem_bytes = bn == 256 ? GemmCfg<256, __half>::SMEM_BYTES
                                 : (bn == 128 ? GemmCfg<128, __half>::SMEM_BYTES : GemmCfg<64, __half>::SMEM_BYTES);
    plan->tiles_m = (int)cdiv(M, bn);
    plan->tiles_n = (int)cdiv(N, GEMM_BM);
    int64_t tiles = (int64_t)plan->tiles_m * plan->tiles_n * nbatch;
    plan->ctas = (int)(tiles < sms ? tiles : sms);
    return B200_OK;
}

int b200_gemm_f16(b200_ctx* ctx, int64_t M, int64_t N, int64_t K, const void* A, int64_t lda,
                  const void* B, int64_t ldb, const void* bias, void* out, int64_t ldo, int out_dtype,
                  int epilogue, int64_t nbatch, int64_t strideA, int64_t strideB, int64_t strideO) {
    return gemm_f16_run(ctx, M, N, K, A, lda, B, ldb, bias, 0, out, ldo, out_dtype, epilogue, nbatch, strideA,
                        strideB, strideO);
}

} // extern "C"

namespace b200 {

int gemm_f16_run(b200_ctx* ctx, int64_t M, int64_t N, int64_t K, const void* A, int64_t lda, const void* B,
                 int64_t ldb, const void* bias, int bias_per_n, void* out, int64_t ldo, int out_dtype,
                 int epilogue, int64_t nbatch, int64_t strideA, int64_t strideB, int64_t strideO) {
    B200_REQUIRE(ctx, B200_EINVAL, "gemm: null ctx");
    B200_REQUIRE(M >= 0 && N >= 0 && K >= 0 && nbatch >= 0, B200_EINVAL, "gemm: negative extent");
    B200_REQUIRE(epilogue >= B200_EPI_NONE && epilogue <= B200_EPI_GELU_TANH, B200_EINVAL,
                 "gemm: epilogue %d", epilogue);
    B200_REQUIRE(out_dtype == B200_F16 || out_dtype == B200_F32, B200_DECLINE_ELTYPE, "gemm: out dtype %d",
                 out_dtype);
    if (M == 0 || N == 0 || nbatch == 0) return B200_OK;
    B200_REQUIRE(K >= 1, B200_DECLINE_EXTENT, "gemm: K = 0");
    B200_REQUIRE(A && B && out, B200_EINVAL, "gemm: null array");
    B200_REQUIRE(lda >= M && ldb >= K && ldo >= M, B200_EINVAL, "gemm: leading dimension below extent");
    B200_REQUIRE(nbatch == 1 || bias == nullptr, B200_DECLINE_BIAS, "gemm: bias with nbatch > 1");
    B200_CUDA(cudaSetDevice(ctx->device));

    const int64_t oal = out_dtype == B200_F16 ? 8 : 4;
    bool tc = tc_supported(M, N, K, lda, ldb, ldo, out_dtype) == B200_OK && aligned16(A) && aligned16(B) &&
              aligned16(out) &&
              (nbatch == 1 || (strideA % 8 == 0 && strideB % 8 == 0 && strideO % oal == 0));
    if (!tc) {
        B200_REQUIRE(N < 65536 && nbatch < 65536, B200_DECLINE_EXTENT,
                     "gemm: unaligned operands with N or nbatch >= 65536");
        dim3 grid((unsigned)cdiv(M, 128), (unsigned)N, (unsigned)nbatch), block(128);
        if (out_dtype == B200_F16)
            gemm_f16_scalar_kernel<__half><<<grid, block, 0, ctx->stream>>>(
                M, N, K, (const __half*)A, lda, (const __half*)B, ldb, (const __half*)bias, bias_per_n, (__half*)out,
                ldo, epilogue, strideA, strideB, strideO);
        else
            gemm_f16_scalar_kernel<float><<<grid, block, 0, ctx->stream>>>(
                M, N, K, (const __half*)A, lda, (const __half*)B, ldb, (const __half*)bias, bias_per_n, (float*)out,
                ldo, epilogue, strideA, strideB, strideO);
        ctx->launches++;
        B200_CUDA(cudaGetLastError());
        return B200_OK;
    }
    const int bn = pick_bn(M, N, nbatch, ctx->prop.multiProcessorCount);
#define GEMM_GO(BN_, T_) \
    return launch_tc<BN_, T_>(ctx, M, N, K, A, lda, B, ldb, bias, bias_per_n, out, ldo, epilogue, nbatch, strideA, \
                              strideB, strideO)
    if (out_dtype == B200_F16) {
        if (bn == 256) GEMM_GO(256, __half);
        if (bn == 128) GEMM_GO(128, __half);
        GEMM_GO(64, __half);
    } else {
        if (bn == 256) GEMM_GO(256, float);
        if (bn == 128) GEMM_GO(128, float);
        GEMM_GO(64, float);
    }
#undef GEMM_GO
}

} // namespace b200
