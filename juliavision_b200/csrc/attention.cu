// Fused non-causal attention for sm_100a: one pass over the keys with an online softmax,
// the query tile resident in shared memory, K/V streamed by TMA straight from the strided
// (E,L,H,B) operands, S = Q K' and O += P V on the tcgen05 tensor cores with S and O in TMEM.
//
// Replaces attn_flash_cm! / attn_flash_cm_merge! / attn_flash! (reference
// kernels/extern/flash.jl:160-271,459-1036,1398-1421) and the layout passes that fed them
// (toLE_tiled_*, densify, padE: kernels/extern/attention.jl:342-396,448-463): the tensor maps
// read the operands through their strides, pad E to the MMA granule with zero fill and
// zero-fill the ragged key/query tails, so no operand is copied, padded or clamped.
//
// Rounding points kept from the reference: the scale multiplies the fp32 scores
// (flash.jl:672-675), the softmax runs in fp32, P is rounded to fp16 before P V
// (flash.jl:725,765), O accumulates in fp32, and a row whose sum is zero divides by one
// (flash.jl:1015).
//
// One CTA owns 128 queries of one (head, batch) and walks the keys in blocks of 128.
//   warp 0    TMA producer: Q once, then K and V tiles through a two-stage ring
//   warp 1    UMMA issuer:  S = Q K'  (128x128x64),  O += P V  (128xEPx128)
//   warps 2-5 softmax: one thread per query row; TMEM -> registers, running max / sum,
//             P as fp16 into swizzled shared memory, O rescaled in TMEM when the max moved,
//             and at the end O / l written to global memory.
// Two CTAs share an SM (256 TMEM columns and ~113 KB of shared memory each), so one CTA's
// softmax overlaps the other's tensor-core work.
#include <cuda_fp16.h>

#include "internal.h"
#include "ptx.cuh"

namespace b200 {

constexpr int ATT_BR = 128;  // queries per CTA (TMEM lanes)
constexpr int ATT_BC = 128;  // keys per block
constexpr int ATT_EP = 64;   // head dim padded to one 128-byte swizzle row
constexpr int ATT_THREADS = 192;
constexpr int ATT_TILE_BYTES = 128 * 128; // every operand tile is 128 rows x 128 B
constexpr int ATT_SMEM_TILES = 1 /*Q*/ + 4 /*K,V x2*/ + 2 /*P*/;
constexpr int ATT_SMEM_BYTES = ATT_SMEM_TILES * ATT_TILE_BYTES + 256 /*barriers*/ + 768 /*align slack*/;
constexpr int ATT_TMEM_COLS = 256;
constexpr int ATT_S_COL = 0;    // S: 128 fp32 columns
constexpr int ATT_O_COL = 128;  // O: EP fp32 columns

struct AttnParams {
    int E, Lq, Lk, H, B;
    float scale_log2;   // scale * log2(e)
    void* out;
    int64_t osL, osH, osB;  // element strides of out along L, H, B (E is contiguous)
    int out_f32;
    int* d_status;
};

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__global__ void __launch_bounds__(ATT_THREADS, 2)
attention_f16_tc_kernel(const __grid_constant__ CUtensorMap tmapQ,
                        const __grid_constant__ CUtensorMap tmapK,
                        const __grid_constant__ CUtensorMap tmapV, const AttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~uintptr_t(1023));
    uint8_t* sQ = smem;
    uint8_t* sKV = smem + ATT_TILE_BYTES;          // [stage][K|V]
    uint8_t* sP = smem + 5 * ATT_TILE_BYTES;       // two 64-key halves
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 7 * ATT_TILE_BYTES);
    uint64_t* q_full = bars + 0;
    uint64_t* k_full = bars + 1;   // [2]
    uint64_t* k_empty = bars + 3;  // [2]
    uint64_t* v_full = bars + 5;   // [2]
    uint64_t* v_empty = bars + 7;  // [2]
    uint64_t* s_full = bars + 9;
    uint64_t* s_empty = bars + 10;
    uint64_t* p_full = bars + 11;
    uint64_t* pv_done = bars + 12;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int q0 = blockIdx.x * ATT_BR;
    const int h = blockIdx.y;
    const int b = blockIdx.z;
    const int nblk = (p.Lk + ATT_BC - 1) / ATT_BC;

    // The carve-up above needs the aligned base to leave room for every tile; the test is
    // uniform across the CTA, so a misplaced base makes every thread leave before any
    // barrier or TMEM allocation exists.
    if (smem + 7 * ATT_TILE_BYTES + 256 > smem_raw + ATT_SMEM_BYTES) {
        if (threadIdx.x == 0) atomicCAS(p.d_status, 0, KST_SMEM_LAYOUT);
        return;
    }
    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&k_full[s], 1);
            mbar_init(&k_empty[s], 1);
            mbar_init(&v_full[s], 1);
            mbar_init(&v_empty[s], 1);
        }
        mbar_init(s_full, 1);
        mbar_init(s_empty, 128);
        mbar_init(p_full, 128);
        mbar_init(pv_done, 1);
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tmap(&tmapQ);
        prefetch_tmap(&tmapK);
        prefetch_tmap(&tmapV);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, ATT_TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------- TMA producer
        if (lane == 0) {
            mbar_arrive_expect_tx(q_full, ATT_TILE_BYTES);
            tma_load_4d(sQ, &tmapQ, q_full, 0, q0, h, b);
            for (int j = 0; j < nblk; ++j) {
                const int s = j & 1;
                const uint32_t ph = (uint32_t)((j >> 1) & 1);
                uint8_t* sk = sKV + (2 * s) * ATT_TILE_BYTES;
                uint8_t* sv = sk + ATT_TILE_BYTES;
                if (!mbar_wait(&k_empty[s], ph ^ 1, p.d_status, KST_WAIT_EMPTY, abort_flag)) break;
                mbar_arrive_expect_tx(&k_full[s], ATT_TILE_BYTES);
                tma_load_4d(sk, &tmapK, &k_full[s], 0, j * ATT_BC, h, b);
                if (!mbar_wait(&v_empty[s], ph ^ 1, p.d_status, KST_WAIT_EMPTY, abort_flag)) break;
                mbar_arrive_expect_tx(&v_full[s], ATT_TILE_BYTES);
                tma_load_4d(sv, &tmapV, &v_full[s], 0, j * ATT_BC, h, b);
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------- UMMA issuer
        if (lane == 0) {
            // S = Q K': both operands K-major (E contiguous).  O += P V: P K-major (keys
            // contiguous per query row), V MN-major (E contiguous per key).
            constexpr uint32_t idesc_s = make_idesc_f16(ATT_BR, ATT_BC, 0, 0);
            constexpr uint32_t idesc_o = make_idesc_f16(ATT_BR, ATT_EP, 0, 1);
            constexpr uint64_t kdesc0 = make_smem_desc(16, 1024);
            constexpr uint64_t vdesc0 = make_smem_desc(ATT_TILE_BYTES, 1024);
            const uint32_t q_addr = smem_u32(sQ);
            const uint32_t p_addr = smem_u32(sP);
            const uint32_t s_tmem = tmem_base + ATT_S_COL;
            const uint32_t o_tmem = tmem_base + ATT_O_COL;

            auto issue_qk = [&](int j) -> bool {
                const int s = j & 1;
                const uint32_t ph = (uint32_t)((j >> 1) & 1);
                if (!mbar_wait(&k_full[s], ph, p.d_status, KST_WAIT_FULL, abort_flag)) return false;
                // S is single-buffered: block j may overwrite it once the softmax of block
                // j-1 has read it out.
                if (j > 0 && !mbar_wait(s_empty, (uint32_t)((j - 1) & 1), p.d_status, KST_WAIT_SOFTMAX, abort_flag))
                    return false;
                tc_fence_after();
                const uint32_t k_addr = smem_u32(sKV + (2 * s) * ATT_TILE_BYTES);
#pragma unroll
                for (int k = 0; k < ATT_EP / 16; ++k)
                    umma_ss(s_tmem, smem_desc_at(kdesc0, q_addr + k * 32), smem_desc_at(kdesc0, k_addr + k * 32),
                            idesc_s, k != 0);
                umma_commit(&k_empty[s]);
                umma_commit(s_full);
                return true;
            };

            bool ok = mbar_wait(q_full, 0, p.d_status, KST_WAIT_FULL, abort_flag);
            if (ok && nblk > 0) ok = issue_qk(0);
            for (int j = 0; ok && j < nblk; ++j) {
                if (j + 1 < nblk) {
                    ok = issue_qk(j + 1);
                    if (!ok) break;
                }
                const int s = j & 1;
                const uint32_t ph = (uint32_t)((j >> 1) & 1);
                if (!mbar_wait(&v_full[s], ph, p.d_status, KST_WAIT_FULL, abort_flag)) break;
                if (!mbar_wait(p_full, (uint32_t)(j & 1), p.d_status, KST_WAIT_SOFTMAX, abort_flag)) break;
                tc_fence_after();
                const uint32_t v_addr = smem_u32(sKV + (2 * s + 1) * ATT_TILE_BYTES);
#pragma unroll
                for (int k = 0; k < ATT_BC / 16; ++k) {
                    // P: 64-key halves are whole tiles apart, 16 keys = 32 B inside a row.
                    // V: 16 key rows = two 8-row groups = 2048 B.
                    const uint32_t pa = p_addr + (k >> 2) * ATT_TILE_BYTES + (k & 3) * 32;
                    umma_ss(o_tmem, smem_desc_at(kdesc0, pa), smem_desc_at(vdesc0, v_addr + k * 2048), idesc_o,
                            (j | k) != 0);
                }
                umma_commit(&v_empty[s]);
                umma_commit(pv_done);
            }
        }
    } else {
        // ------------------------------------------------------- softmax + epilogue
        const int quad = warp & 3;
        const int row = quad * 32 + lane;
        const uint32_t lane_base = uint32_t(quad * 32) << 16;
        const uint32_t s_tmem = tmem_base + lane_base + ATT_S_COL;
        const uint32_t o_tmem = tmem_base + lane_base + ATT_O_COL;
        const float sc = p.scale_log2;
        float m_run = -INFINITY, l_run = 0.f;
        uint8_t* prow = sP + row * 128;
        bool ok = true;

        for (int j = 0; j < nblk; ++j) {
            if (!mbar_wait(s_full, (uint32_t)(j & 1), p.d_status, KST_WAIT_TMEM_FULL, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const int kv0 = j * ATT_BC;
            const int nvalid = p.Lk - kv0; // keys of this block that exist (>= 128 when full)

            // Pass 1: the row maximum of the scaled scores.
            float mx = -INFINITY;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t r[32];
                tmem_ld32(s_tmem + c * 32, r);
                tmem_wait_ld();
                if (nvalid >= ATT_BC) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(r[i]) * sc);
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (c * 32 + i < nvalid) mx = fmaxf(mx, __uint_as_float(r[i]) * sc);
                }
            }
            const float m_new = fmaxf(m_run, mx);
            const float alpha = ex2(m_run - m_new); // 0 on the first block (m_run = -inf)

            // P's shared tile and O are both still in use by the previous block's P V.
            if (j > 0 && !mbar_wait(pv_done, (uint32_t)((j - 1) & 1), p.d_status, KST_WAIT_SOFTMAX, abort_flag)) {
                ok = false;
                break;
            }
            tc_fence_after();

            // Pass 2: exponentials, row sum, P as fp16 into the swizzled K-major tile.
            float rs = 0.f;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t r[32];
                tmem_ld32(s_tmem + c * 32, r);
                tmem_wait_ld();
                float e[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    float v = ex2(fmaf(__uint_as_float(r[i]), sc, -m_new));
                    if (nvalid < ATT_BC && c * 32 + i >= nvalid) v = 0.f;
                    e[i] = v;
                    rs += v;
                }
                uint8_t* half_tile = prow + (c >> 1) * ATT_TILE_BYTES;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint4 o;
                    __half2* hh = reinterpret_cast<__half2*>(&o);
#pragma unroll
                    for (int t = 0; t < 4; ++t) hh[t] = __floats2half2_rn(e[q * 8 + 2 * t], e[q * 8 + 2 * t + 1]);
                    const int chunk = (c & 1) * 4 + q;
                    *reinterpret_cast<uint4*>(half_tile + ((chunk ^ (row & 7)) << 4)) = o;
                }
            }
            // S has been read out: the next Q K' may overwrite it.
            tc_fence_before();
            mbar_arrive(s_empty);

            // Rescale O when this row's maximum moved (skipped warp-wide when none did).
            if (j > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll 1
                for (int c = 0; c < ATT_EP / 32; ++c) {
                    uint32_t r[32];
                    tmem_ld32(o_tmem + c * 32, r);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                    tmem_st32(o_tmem + c * 32, r);
                }
                tmem_wait_st();
            }
            l_run = l_run * alpha + rs;
            m_run = m_new;
            fence_proxy_async_smem();
            tc_fence_before();
            mbar_arrive(p_full);
        }

        // Epilogue: O / l to global, dense (E, Lq, H, B).
        if (ok && nblk > 0) ok = mbar_wait(pv_done, (uint32_t)((nblk - 1) & 1), p.d_status, KST_WAIT_SOFTMAX, abort_flag);
        if (ok) {
            tc_fence_after();
            const float inv = 1.0f / (l_run == 0.f ? 1.0f : l_run);
            const int lq = q0 + row;
            const int64_t obase = lq * p.osL + h * p.osH + b * p.osB;
#pragma unroll 1
            for (int c = 0; c < ATT_EP / 32; ++c) {
                uint32_t r[32];
                if (nblk > 0) {
                    tmem_ld32(o_tmem + c * 32, r);
                    tmem_wait_ld();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = 0u;
                }
                if (lq < p.Lq) {
                    if (p.out_f32) {
                        float* o = static_cast<float*>(p.out) + obase + c * 32;
#pragma unroll
                        for (int i = 0; i < 32; i += 4) {
                            if (c * 32 + i < p.E)
                                *reinterpret_cast<float4*>(o + i) =
                                    make_float4(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv,
                                                __uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv);
                        }
                    } else {
                        __half* o = static_cast<__half*>(p.out) + obase + c * 32;
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            if (c * 32 + i < p.E) {
                                uint4 w;
                                __half2* hh = reinterpret_cast<__half2*>(&w);
#pragma unroll
                                for (int t = 0; t < 4; ++t)
                                    hh[t] = __floats2half2_rn(__uint_as_float(r[i + 2 * t]) * inv,
                                                              __uint_as_float(r[i + 2 * t + 1]) * inv);
                                *reinterpret_cast<uint4*>(o + i) = w;
                            }
                        }
                    }
                }
            }
        }
    }

    if (*abort_flag) {
        for (int i = 0; i < 4; ++i) __nanosleep(1000000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, ATT_TMEM_COLS);
    }
}

// Scalar path for operands a tensor map cannot express (E > 64, E not a multiple of 8,
// unaligned strides): one warp per query row, two passes over the keys.
__global__ void attention_f16_scalar_kernel(int E, int Lq, int Lk, int H, int B, const __half* q, int64_t qsE, int64_t qsL, int64_t qsH, int64_t qsB,
                                            const __half* k, int64_t ksE, int64_t ksL, int64_t ksH, int64_t ksB,
                                            const __half* v, int64_t vsE, int64_t vsL, int64_t vsH, int64_t vsB,
                                            void* out, int64_t osL, int64_t osH, int64_t osB, int out_f32, float scale) {
    const int lane = threadIdx.x & 31;
    const int64_t rowid = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (rowid >= (int64_t)Lq * H * B) return;
    const int lq = (int)(rowid % Lq);
    const int h = (int)((rowid / Lq) % H);
    const int b = (int)(rowid / ((int64_t)Lq * H));
    const __half* qp = q + qsL * lq + qsH * h + qsB * b;
    const __half* kp = k + ksH * h + ksB * b;
    const __half* vp = v + vsH * h + vsB * b;
    float m = -INFINITY;
    for (int lk = lane; lk < Lk; lk += 32) {
        float a = 0.f;
        for (int e = 0; e < E; ++e) a = fmaf(__half2float(qp[qsE * e]), __half2float(kp[ksL * lk + ksE * e]), a);
        m = fmaxf(m, a * scale);
    }
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    // Each lane accumulates its own keys into E partial outputs held two per lane-pass.
    float l = 0.f;
    extern __shared__ float acc_sm[]; // [warps][E]
    float* acc = acc_sm + (threadIdx.x >> 5) * E;
    for (int e = lane; e < E; e += 32) acc[e] = 0.f;
    __syncwarp();
    for (int lk0 = 0; lk0 < Lk; lk0 += 32) {
        const int lk = lk0 + lane;
        float pexp = 0.f;
        if (lk < Lk) {
            float a = 0.f;
            for (int e = 0; e < E; ++e) a = fmaf(__half2float(qp[qsE * e]), __half2float(kp[ksL * lk + ksE * e]), a);
            pexp = __expf(a * scale - m);
            l += pexp;
            pexp = __half2float(__float2half_rn(pexp));
        }
        for (int t = 0; t < 32 && lk0 + t < Lk; ++t) {
            const float pt = __shfl_sync(0xffffffffu, pexp, t);
            for (int e = lane; e < E; e += 32) acc[e] = fmaf(pt, __half2float(vp[vsL * (lk0 + t) + vsE * e]), acc[e]);
        }
    }
    for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
    const float inv = 1.0f / (l == 0.f ? 1.0f : l);
    const int64_t obase = lq * osL + h * osH + b * osB;
    for (int e = lane; e < E; e += 32) {
        if (out_f32) static_cast<float*>(out)[obase + e] = acc[e] * inv;
        else static_cast<__half*>(out)[obase + e] = __float2half_rn(acc[e] * inv);
    }
}

static int tc_reason(int64_t E, int64_t Lq, int64_t Lk, int64_t H, int64_t B, const int64_t* qs,
                     const int64_t* ks, const int64_t* vs) {
    if (E < 1 || Lq < 1 || Lk < 1 || H < 1 || B < 1) return B200_DECLINE_EXTENT;
    if (E > ATT_EP || E % 8 != 0) return B200_DECLINE_TILING;
    if (H > 65535 || B > 65535 || Lq >= (1ll << 31) || Lk >= (1ll << 31)) return B200_DECLINE_EXTENT;
    const int64_t* ss[3] = {qs, ks, vs};
    for (int i = 0; i < 3; ++i) {
        const int64_t ext[4] = {E, i == 0 ? Lq : Lk, H, B};
        if (ss[i][0] != 1) return B200_DECLINE_ALIGN;
        // A tensor map wants every stride a multiple of 16 bytes; an axis of extent one is
        // never stepped along, so its stride is free.
        for (int d = 1; d < 4; ++d)
            if (ext[d] > 1 && (ss[i][d] % 8 != 0 || ss[i][d] <= 0)) return B200_DECLINE_ALIGN;
    }
    return B200_OK;
}

static int make_qkv_map(b200_ctx* ctx, CUtensorMap* m, const b200_strided4* t, int64_t E, int64_t L,
                        int64_t H, int64_t B) {
    uint64_t dims[4] = {(uint64_t)E, (uint64_t)L, (uint64_t)H, (uint64_t)B};
    // A unit-extent axis may carry any stride; give the encoder a legal one.
    auto st = [&](int d, uint64_t fallback) {
        uint64_t s = (uint64_t)t->stride[d] * 2;
        return (dims[d] == 1 || s == 0) ? fallback : s;
    };
    uint64_t s1 = st(1, (uint64_t)E * 2 < 16 ? 16 : (uint64_t)((E * 2 + 15) / 16 * 16));
    uint64_t s2 = st(2, s1 * (uint64_t)L);
    uint64_t s3 = st(3, s2 * (uint64_t)H);
    uint64_t str[3] = {s1, s2, s3};
    uint32_t box[4] = {ATT_EP, 128, 1, 1};
    return make_tmap(ctx, m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, t->ptr, dims, str, box,
                     CU_TENSOR_MAP_SWIZZLE_128B);
}

} // namespace b200

using namespace b200;

extern "C" {

int b200_attention_f16_supported(int64_t E, int64_t Lq, int64_t Lk, int64_t H, int64_t B,
                                 const int64_t* qstride, const int64_t* kstride, const int64_t* vstride,
                                 int has_bias) {
    if (has_bias) return B200_DECLINE_BIAS;
    if (!qstride || !kstride || !vstride) return B200_EINVAL;
    return tc_reason(E, Lq, Lk, H, B, qstride, kstride, vstride);
}

int b200_attention_f16(b200_ctx* ctx, int64_t E, int64_t Lq, int64_t Lk, int64_t H, int64_t B,
                       const b200_strided4* q, const b200_strided4* k, const b200_strided4* v, void* out,
                       int out_dtype, float scale) {
    b200_strided4 o;
    o.ptr = out;
    o.stride[0] = 1;
    o.stride[1] = E;
    o.stride[2] = E * Lq;
    o.stride[3] = E * Lq * H;
    return b200_attention_f16_strided(ctx, E, Lq, Lk, H, B, q, k, v, &o, out_dtype, scale);
}

int b200_attention_f16_strided(b200_ctx* ctx, int64_t E, int64_t Lq, int64_t Lk, int64_t H, int64_t B,
                               const b200_strided4* q, const b200_strided4* k, const b200_strided4* v,
                               const b200_strided4* o, int out_dtype, float scale) {
    B200_REQUIRE(ctx && q && k && v && o, B200_EINVAL, "attention: null argument");
    void* out = const_cast<void*>(o->ptr);
    B200_REQUIRE(E >= 0 && Lq >= 0 && Lk >= 0 && H >= 0 && B >= 0, B200_EINVAL, "attention: negative extent");
    B200_REQUIRE(out_dtype == B200_F16 || out_dtype == B200_F32, B200_DECLINE_ELTYPE, "attention: out dtype %d",
                 out_dtype);
    if (E == 0 || Lq == 0 || H == 0 || B == 0) return B200_OK;
    B200_REQUIRE(out && q->ptr, B200_EINVAL, "attention: null array");
    B200_CUDA(cudaSetDevice(ctx->device));
    const size_t osz = out_dtype == B200_F16 ? 2 : 4;
    const int64_t oal = out_dtype == B200_F16 ? 8 : 4; // elements per 16-byte vector store
    B200_REQUIRE(o->stride[0] == 1, B200_DECLINE_ALIGN, "attention: out must be contiguous along E");
    const bool odense = o->stride[1] == E && (H == 1 || o->stride[2] == E * Lq) && (B == 1 || o->stride[3] == E * Lq * H);
    const bool oaligned = (Lq == 1 || o->stride[1] % oal == 0) && (H == 1 || o->stride[2] % oal == 0) &&
                          (B == 1 || o->stride[3] % oal == 0);
    if (Lk == 0) {
        // Softmax over no keys: every row is the all-blocked case, a zero row divided by one.
        B200_REQUIRE(odense, B200_DECLINE_ALIGN, "attention: Lk = 0 with a strided out");
        B200_CUDA(cudaMemsetAsync(out, 0, (size_t)(E * Lq * H * B) * osz, ctx->stream));
        return B200_OK;
    }
    B200_REQUIRE(k->ptr && v->ptr, B200_EINVAL, "attention: null array");
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    const bool tc = tc_reason(E, Lq, Lk, H, B, q->stride, k->stride, v->stride) == B200_OK && al16(q->ptr) &&
                    al16(k->ptr) && al16(v->ptr) && al16(out) && oaligned;
    if (!tc) {
        B200_REQUIRE(E <= 1024, B200_DECLINE_EXTENT, "attention: E = %lld", (long long)E);
        const int wpb = 4;
        const int64_t rows = Lq * H * B;
        attention_f16_scalar_kernel<<<(unsigned)cdiv(rows, wpb), 32 * wpb, wpb * E * sizeof(float), ctx->stream>>>(
            (int)E, (int)Lq, (int)Lk, (int)H, (int)B, (const __half*)q->ptr, q->stride[0], q->stride[1],
            q->stride[2], q->stride[3], (const __half*)k->ptr, k->stride[0], k->stride[1], k->stride[2],
            k->stride[3], (const __half*)v->ptr, v->stride[0], v->stride[1], v->stride[2], v->stride[3], out,
            o->stride[1], o->stride[2], o->stride[3], out_dtype == B200_F32, scale);
        ctx->launches++;
        B200_CUDA(cudaGetLastError());
        return B200_OK;
    }
    static bool attr_done[16] = {};
    if (!attr_done[ctx->device & 15]) {
        B200_CUDA(cudaFuncSetAttribute(attention_f16_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       ATT_SMEM_BYTES));
        attr_done[ctx->device & 15] = true;
    }
    CUtensorMap tq, tk, tv;
    int rc;
    if ((rc = make_qkv_map(ctx, &tq, q, E, Lq, H, B))) return rc;
    if ((rc = make_qkv_map(ctx, &tk, k, E, Lk, H, B))) return rc;
    if ((rc = make_qkv_map(ctx, &tv, v, E, Lk, H, B))) return rc;
    AttnParams p;
    p.E = (int)E; p.Lq = (int)Lq; p.Lk = (int)Lk; p.H = (int)H; p.B = (int)B;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.out = out;
    p.osL = o->stride[1]; p.osH = o->stride[2]; p.osB = o->stride[3];
    p.out_f32 = out_dtype == B200_F32;
    p.d_status = ctx->d_status;
    dim3 grid((unsigned)cdiv(Lq, ATT_BR), (unsigned)H, (unsigned)B);
    attention_f16_tc_kernel<<<grid, ATT_THREADS, ATT_SMEM_BYTES, ctx->stream>>>(tq, tk, tv, p);
    ctx->launches++;
    B200_CUDA(cudaGetLastError());
    return B200_OK;
}

} // extern "C"
