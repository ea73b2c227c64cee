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
// One CTA owns 256 queries (two tiles of 128) of one (head, batch) and walks the keys in blocks
// of 128; the kernel comment below gives the roles and the pipeline.
#include <cuda_fp16.h>

#include "internal.h"
#include "ptx.cuh"

namespace b200 {

constexpr int ATT_BR = 128;  // queries per tile (TMEM lanes)
constexpr int ATT_BC = 128;  // keys per block
constexpr int ATT_THREADS = 384;  // warps 0-3, 4-7: softmax of tile 0, 1; warp 8: TMA; warps 9, 10: UMMA; 11 idle
constexpr int ATT_TILE_BYTES = 128 * 128; // one swizzle atom of an operand tile: 128 rows x 128 B (64 fp16 of E)
#ifndef ATT_TURN_AT
#define ATT_TURN_AT 2   // after which quarter (0..3) of its exponentials a tile passes the turn
#endif
// Two shapes of CTA, chosen by the head dimension:
//   EP = 64  (E <= 64):        two query tiles of 128 per CTA, K/V rings of 4 stages x 16 KB
//   EP = 128 (64 < E <= 128):  two query tiles of 128 per CTA as well; every operand tile is two swizzle atoms along
//                              E (columns 0-63, 64-127, the second zero-filled past E by the tensor map), S = Q K'
//                              runs over both, O has 128 columns per tile — S 2 x 128 + O 2 x 128 fill the tensor
//                              memory, so P is written over the first 64 columns of its tile's S once the softmax
//                              has pulled S into registers, and a tile's Q K'(j+1) is issued after its P V(j)
//                              (the two tiles' chains interleave on the tensor core); K/V rings of 2 stages x 32 KB
// The reference's own fused tiling is E = 72 padded to 80 (flash.jl:1149-1157, flashepad kernelplans.jl).
template <int EP> struct AttCfg {
    static_assert(EP == 64 || EP == 128, "head dim is padded to one or two swizzle atoms");
    static constexpr int ATOMS = EP / 64;              // 16 KB atoms per operand tile
    static constexpr int NT = 2;                       // query tiles per CTA
    static constexpr int KV_STAGES = EP == 64 ? 4 : 2;
    static constexpr bool P_IN_S = EP == 128;          // P shares its tile's S columns (tensor memory is full otherwise)
    static constexpr int OP_BYTES = ATOMS * ATT_TILE_BYTES;   // one Q, K or V tile
    // shared-memory map, in 16 KB atoms
    static constexpr int T_Q = 0;                              // NT tiles
    static constexpr int T_K = NT * ATOMS;                     // KV_STAGES tiles
    static constexpr int T_V = T_K + KV_STAGES * ATOMS;        // KV_STAGES tiles
    static constexpr int T_END = T_V + KV_STAGES * ATOMS;
    static constexpr int SMEM_BYTES = T_END * ATT_TILE_BYTES + 256;
    static_assert(SMEM_BYTES <= 232448, "shared memory over budget");
};
// tensor-memory map (512 columns): S of tile t, fp32, at [128 t, 128 t + 128); O of tile t, fp32, at
// [256 + EP t, ... + EP); P of tile t, fp16 packed two keys per column, at [384 + 64 t, ... + 64) for EP = 64 and
// over the first 64 columns of S_t for EP = 128
constexpr int ATT_TMEM_COLS = 512;
constexpr int ATT_S_COL = 0;
constexpr int ATT_O_COL = 256;
constexpr int ATT_P_COL = 384;

struct AttnParams {
    int E, Lq, Lk, H, B;
    float scale_log2;   // scale * log2(e)
    void* out;
    int64_t osL, osH, osB;  // element strides of out along L, H, B (E is contiguous)
    int out_f32;
    int qpairs;         // work items per (head, batch): groups of NT query tiles ("pairs" when NT = 2)
    int pair_ctas;      // CTAs [0, pair_ctas) own a whole item; the rest own one tile of a pair, or a key range of an item
    int* d_status;
    unsigned long long* trace;  // optional timeline of CTA (0,0,0) (globaltimer ns), null in normal use
    // Additive mask of the mem-efficient variant (attention.jl:55-59), (Lk,Lq,H,B) fp16 with element
    // strides (0 on a broadcast axis); null when absent.  bias_vec: rows can be read 8 keys at a time.
    const __half* bias;
    int64_t bsK, bsQ, bsH, bsB;
    int bias_vec;
    // Keys split over nsplit CTAs per query pair (few queries, many keys): each writes its unnormalised
    // fp32 O rows to part_o[split][tail pair][256 rows][E] and (reference point, row sum) to part_ml[...][2];
    // attention_merge_kernel combines them (the reference's attn_flash_cm_merge!, flash.jl:1398-1421).
    int nsplit;
    int ntail;          // pairs that are split (the last ntail of them)
    float* part_o;
    float* part_ml;
};

#define ATT_TRACE(slot)                                                                              \
    do {                                                                                             \
        if (p.trace != nullptr && blockIdx.x == 0 && (slot) < 128) \
            p.trace[(slot)] = globaltimer_ns();                                                      \
    } while (0)

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Packed pairs of fp32 (sm_100): one instruction does two lanes' worth, which halves the softmax threads'
// FMA and add streams; the exponentials themselves stay on the MUFU pipe.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ void tmem_st16_raw(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

// One CTA = 256 queries (two tiles of 128) of one (head, batch), one CTA per SM:
//   warps 0-3  softmax of tile 0, warps 4-7 softmax of tile 1: one thread per query row, the whole
//              128-score row in registers (these two warpgroups take registers from the third)
//   warp 8     TMA producer: both Q tiles once, then K and V blocks through 3-stage rings
//   warps 9,10 UMMA issuers, one lane per tile: S_t = Q_t K' and O_t += P_t V per key block;
//              the two chains are independent, so the tensor core works on one tile while the
//              other tile's softmax runs
// P never touches shared memory: the softmax threads write it as packed fp16 into tensor memory and
// the P V product takes its A operand from there, so the shared-memory port only feeds K and V.
// BIAS: the scaled score gets an additive fp16 mask before the softmax; a row whose keys are all
// blocked (-inf everywhere) comes out as zeros, as in attn_softmax (attention.jl:73-100).
template <int EP, bool BIAS>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attention_f16_tc_kernel(const __grid_constant__ CUtensorMap tmapQ,
                        const __grid_constant__ CUtensorMap tmapK,
                        const __grid_constant__ CUtensorMap tmapV, const AttnParams p) {
    using Cfg = AttCfg<EP>;
    constexpr int ATT_KV_STAGES = Cfg::KV_STAGES;
    constexpr int NT = Cfg::NT;
    constexpr int ITEM_ROWS = NT * ATT_BR;   // queries one whole work item covers
    extern __shared__ __align__(1024) uint8_t smem[];
    // Uniform across the grid: a base that is not 1024-aligned makes every thread leave before
    // any barrier or TMEM allocation exists.
    if ((smem_u32(smem) & 1023u) != 0) {
        if (threadIdx.x == 0) atomicCAS(p.d_status, 0, KST_SMEM_LAYOUT);
        return;
    }
    auto tile_ptr = [&](int t) { return smem + t * ATT_TILE_BYTES; };
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::T_END * ATT_TILE_BYTES);
    uint64_t* q_full = bars + 0;                           // [2]
    uint64_t* k_full = bars + 2;                           // [STAGES]
    uint64_t* k_empty = k_full + ATT_KV_STAGES;            // [STAGES]
    uint64_t* v_full = k_empty + ATT_KV_STAGES;            // [STAGES]
    uint64_t* v_empty = v_full + ATT_KV_STAGES;            // [STAGES]
    uint64_t* s_full = v_empty + ATT_KV_STAGES;            // [2]
    uint64_t* s_empty = s_full + 2;                        // [2]
    uint64_t* p_full = s_empty + 2;                        // [2]
    uint64_t* pv_done = p_full + 2;                        // [2]
    uint64_t* exp_turn = pv_done + 2;                      // [2]: whose turn it is to run its exponentials
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(exp_turn + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // Work item of this CTA.  Most CTAs own a pair of query tiles; when the pairs do not fill the
    // last wave of SMs, the pairs of that wave are handed out as single tiles instead (twice as
    // many, half as long), which shortens the tail.
    // CTAs [0, pair_ctas) own a whole pair.  The pairs after those are the tail: either each is cut along
    // the keys into nsplit CTAs whose partial results are merged afterwards (nsplit > 1), or each is
    // handed out as two single tiles.
    int item = blockIdx.x, half = -1, split = 0, nsp = 1;
    if (item >= p.pair_ctas) {
        const int t = item - p.pair_ctas;
        if (p.nsplit > 1) {
            nsp = p.nsplit;
            split = t % nsp;
            item = p.pair_ctas + t / nsp;
        } else {
            half = t & 1;
            item = p.pair_ctas + (t >> 1);
        }
    }
    const int tailpair = item - p.pair_ctas;   // index among the split pairs (when nsp > 1)
    const int qp = item % p.qpairs;
    const int h = (item / p.qpairs) % p.H;
    const int b = item / (p.qpairs * p.H);
    const int q0 = qp * ITEM_ROWS + (half > 0 ? ATT_BR : 0);
    const int nblk_all = (p.Lk + ATT_BC - 1) / ATT_BC;
    const int jb0 = (int)((int64_t)split * nblk_all / nsp);           // first key block of this CTA
    const int nblk = (int)((int64_t)(split + 1) * nblk_all / nsp) - jb0;
    const int ntiles = (NT == 2 && half < 0 && q0 + ATT_BR < p.Lq) ? 2 : 1;   // the second tile may lie wholly past Lq

    if (threadIdx.x == 0) {
        ATT_TRACE(0);
        for (int t = 0; t < 2; ++t) {
            mbar_init(&q_full[t], 1);
            mbar_init(&s_full[t], 1);
            mbar_init(&s_empty[t], 4);   // one arrival per softmax warp
            mbar_init(&p_full[t], 4);
            mbar_init(&pv_done[t], 1);
            mbar_init(&exp_turn[t], 4);
        }
        for (int s = 0; s < ATT_KV_STAGES; ++s) {
            mbar_init(&k_full[s], 1);
            mbar_init(&k_empty[s], ntiles);   // freed when every tile's issuer is done with it
            mbar_init(&v_full[s], 1);
            mbar_init(&v_empty[s], ntiles);
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tmap(&tmapQ);
        prefetch_tmap(&tmapK);
        prefetch_tmap(&tmapV);
    }
    if (warp == 8) {
        tmem_alloc(tmem_slot, ATT_TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Everything above overlapped the previous kernel's tail; from here on its results are needed.
    grid_dep_wait();
    grid_dep_launch();

    // Register budget: the two softmax warpgroups hold a full score row per thread; the third
    // warpgroup (one TMA lane, one UMMA lane, two idle warps) needs almost nothing and hands its
    // share over (setmaxnreg at the head of each role's branch).
    if (warp == 11) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    } else if (warp == 8) {
        // ------------------------------------------------------------- TMA producer
        asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
        if (lane == 0) {
            for (int t = 0; t < ntiles; ++t) {
                mbar_arrive_expect_tx(&q_full[t], Cfg::OP_BYTES);
#pragma unroll
                for (int a = 0; a < Cfg::ATOMS; ++a)
                    tma_load_4d(tile_ptr(Cfg::T_Q + t * Cfg::ATOMS + a), &tmapQ, &q_full[t], a * 64, q0 + t * ATT_BR, h, b);
            }
            for (int j = 0; j < nblk; ++j) {
                const int s = j % ATT_KV_STAGES;
                const uint32_t ph = (uint32_t)((j / ATT_KV_STAGES) & 1);
                if (!mbar_wait(&k_empty[s], ph ^ 1, p.d_status, KST_WAIT_EMPTY, abort_flag)) break;
                mbar_arrive_expect_tx(&k_full[s], Cfg::OP_BYTES);
#pragma unroll
                for (int a = 0; a < Cfg::ATOMS; ++a)
                    tma_load_4d(tile_ptr(Cfg::T_K + s * Cfg::ATOMS + a), &tmapK, &k_full[s], a * 64, (jb0 + j) * ATT_BC, h, b);
                if (!mbar_wait(&v_empty[s], ph ^ 1, p.d_status, KST_WAIT_EMPTY, abort_flag)) break;
                mbar_arrive_expect_tx(&v_full[s], Cfg::OP_BYTES);
#pragma unroll
                for (int a = 0; a < Cfg::ATOMS; ++a)
                    tma_load_4d(tile_ptr(Cfg::T_V + s * Cfg::ATOMS + a), &tmapV, &v_full[s], a * 64, (jb0 + j) * ATT_BC, h, b);
            }
        }
    } else if (warp == 9 || warp == 10) {
        // ------------------------------------------------------------- UMMA issuers
        // One issuing lane per query tile (warp 9: tile 0, warp 10: tile 1).  Each walks its own
        // chain  S_t(j+1) = Q_t K(j+1)'  as soon as the softmax has pulled S_t(j) into registers,
        // then  O_t += P_t(j) V(j)  once P_t(j) is written.  The two chains share only the
        // K/V rings.  (Issuing a UMMA blocks while the tensor pipe is busy, so the issuing lanes
        // are not softmax threads.)
        asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
        const int t = warp - 9;
        if (lane == 0 && t < ntiles) {
            // S = Q K': both operands K-major (E contiguous), from shared memory.  O += P V: P from
            // tensor memory, V MN-major (E contiguous per key) from shared memory.
            constexpr uint32_t idesc_s = make_idesc_f16(ATT_BR, ATT_BC, 0, 0);
            constexpr uint32_t idesc_o = make_idesc_f16(ATT_BR, EP, 0, 1);
            constexpr uint64_t kdesc0 = make_smem_desc(16, 1024);
            constexpr uint64_t vdesc0 = make_smem_desc(ATT_TILE_BYTES, 1024);
            const uint32_t q_addr = smem_u32(tile_ptr(Cfg::T_Q + t * Cfg::ATOMS));
            const uint32_t s_tmem = tmem_base + ATT_S_COL + t * 128;
            const uint32_t o_tmem = tmem_base + ATT_O_COL + t * EP;
            const uint32_t p_tmem = Cfg::P_IN_S ? s_tmem : tmem_base + ATT_P_COL + t * 64;

            auto issue_qk = [&](int j) -> bool {
                const int sk = j % ATT_KV_STAGES;
                if (!mbar_wait(&k_full[sk], (uint32_t)((j / ATT_KV_STAGES) & 1), p.d_status, KST_WAIT_FULL, abort_flag))
                    return false;
                // With P in S's columns this product is issued after P V(j-1), which read P after the softmax had taken
                // S(j-1), and UMMAs of one thread run in issue order: nothing else to wait for.
                if (!Cfg::P_IN_S && j > 0 &&
                    !mbar_wait(&s_empty[t], (uint32_t)((j - 1) & 1), p.d_status, KST_WAIT_SOFTMAX, abort_flag))
                    return false;
                tc_fence_after();
                const uint32_t k_addr = smem_u32(tile_ptr(Cfg::T_K + sk * Cfg::ATOMS));
#pragma unroll
                for (int k = 0; k < EP / 16; ++k) {
                    // 16 elements of E = 32 B inside the swizzle row; every fourth step moves to the next atom
                    const uint32_t off = (uint32_t)(k >> 2) * ATT_TILE_BYTES + (uint32_t)(k & 3) * 32;
                    umma_ss(s_tmem, smem_desc_at(kdesc0, q_addr + off), smem_desc_at(kdesc0, k_addr + off), idesc_s, k != 0);
                }
                umma_commit(&s_full[t]);
                umma_commit(&k_empty[sk]);   // one of `ntiles` arrivals that free this K stage
                if (j >= 1 && j < 7) ATT_TRACE(64 * t + 8 + 8 * (j - 1) + 0);   // Q K'(j) issued, filed under block j-1
                return true;
            };

            bool ok = mbar_wait(&q_full[t], 0, p.d_status, KST_WAIT_FULL, abort_flag);
            if (ok && nblk > 0) ok = issue_qk(0);
            for (int j = 0; ok && j < nblk; ++j) {
                if (!Cfg::P_IN_S && j + 1 < nblk && !issue_qk(j + 1)) break;
                const int sv = j % ATT_KV_STAGES;
                if (!mbar_wait(&v_full[sv], (uint32_t)((j / ATT_KV_STAGES) & 1), p.d_status, KST_WAIT_FULL, abort_flag)) break;
                if (j < 6) ATT_TRACE(64 * t + 8 + 8 * j + 7);   // issuer reaches its wait for P(j)
                if (!mbar_wait(&p_full[t], (uint32_t)(j & 1), p.d_status, KST_WAIT_SOFTMAX, abort_flag)) break;
                tc_fence_after();
                const uint32_t v_addr = smem_u32(tile_ptr(Cfg::T_V + sv * Cfg::ATOMS));
#pragma unroll
                for (int k = 0; k < ATT_BC / 16; ++k) {
                    // P comes from tensor memory: 16 keys = 8 packed columns per step.
                    // V: 16 key rows = two 8-row groups = 2048 B.
                    umma_ts(o_tmem, p_tmem + k * 8, smem_desc_at(vdesc0, v_addr + k * 2048), idesc_o, (j | k) != 0);
                }
                umma_commit(&pv_done[t]);
                umma_commit(&v_empty[sv]);   // one of `ntiles` arrivals that free this V stage
                if (j < 6) ATT_TRACE(64 * t + 8 + 8 * j + 1);   // P V(j) issued
                if (Cfg::P_IN_S && j + 1 < nblk && !issue_qk(j + 1)) break;   // overwrites P(j): after the product that reads it
            }
        }
    } else {
        // ------------------------------------------------------- softmax + epilogue
        asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
        const int t = warp >> 2;               // which query tile this warpgroup owns
        const int quad = warp & 3;             // TMEM lane quadrant
        const int row = quad * 32 + lane;
        if (t < ntiles) {
            const uint32_t lane_base = uint32_t(quad * 32) << 16;
            const uint32_t s_tmem = tmem_base + lane_base + ATT_S_COL + t * 128;
            const uint32_t o_tmem = tmem_base + lane_base + ATT_O_COL + t * EP;
            const uint32_t p_tmem = Cfg::P_IN_S ? s_tmem : tmem_base + lane_base + ATT_P_COL + t * 64;
            const float sc = p.scale_log2;
            const float sce = BIAS ? 1.0f : sc;   // with a bias the scores are rescaled when it is added
            float m_run = -INFINITY, l_run = 0.f;
            bool ok = true;
            // Both tiles take the same time per block, and left alone they fall into step: both
            // want the MUFU pipe in the same half of every period and leave it idle in the other.
            // So the exponential phases take turns (tile 0 block j, tile 1 block j, tile 0 block
            // j+1, ...): while one tile owns the MUFU pipe the other does its max / rescale / waits
            // and its tensor-core work runs.
            const bool pingpong = ntiles == 2 && ATT_TURN_AT >= 0;


            for (int j = 0; ok && j < nblk; ++j) {
                if (!mbar_wait(&s_full[t], (uint32_t)(j & 1), p.d_status, KST_WAIT_TMEM_FULL, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const int nvalid = p.Lk - (jb0 + j) * ATT_BC; // keys of this block that exist (>= 128 when full)
                if (lane == 0 && quad == 0 && j < 6) ATT_TRACE(64 * t + 8 + 8 * j + 2);  // S(0, j) ready

                // The whole row of S (128 fp32) comes into registers in one round trip; S is then
                // free for the next Q K' of this tile.
                uint32_t r[4][32];
#pragma unroll
                for (int c = 0; c < 4; ++c) tmem_ld32(s_tmem + c * 32, r[c]);
                tmem_wait_ld();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&s_empty[t]);
                if (lane == 0 && quad == 0 && j < 6) ATT_TRACE(64 * t + 8 + 8 * j + 3);  // S in registers

                if constexpr (BIAS) {
                    // r <- s * scale * log2(e) (+ bias * log2(e)): from here on the scores are in the
                    // exponent's own units and the scale below is one.
                    const int lq = q0 + t * ATT_BR + row;
                    const float L2E = 1.4426950408889634f;
                    if (p.bias == nullptr) {
#pragma unroll
                        for (int c = 0; c < 4; ++c)
#pragma unroll
                            for (int i = 0; i < 32; ++i) r[c][i] = __float_as_uint(__uint_as_float(r[c][i]) * sc);
                    } else {
                        const __half* brow = p.bias + (int64_t)(lq < p.Lq ? lq : 0) * p.bsQ + (int64_t)h * p.bsH +
                                             (int64_t)b * p.bsB + (int64_t)(jb0 + j) * ATT_BC * p.bsK;
                        if (p.bias_vec && nvalid >= ATT_BC) {
#pragma unroll
                            for (int c = 0; c < 4; ++c)
#pragma unroll
                                for (int g = 0; g < 4; ++g) {
                                    const uint4 w = __ldg(reinterpret_cast<const uint4*>(brow + c * 32 + g * 8));
                                    const __half2* hh = reinterpret_cast<const __half2*>(&w);
#pragma unroll
                                    for (int u = 0; u < 4; ++u) {
                                        const float2 f = __half22float2(hh[u]);
                                        r[c][g * 8 + 2 * u] = __float_as_uint(fmaf(__uint_as_float(r[c][g * 8 + 2 * u]), sc, f.x * L2E));
                                        r[c][g * 8 + 2 * u + 1] = __float_as_uint(fmaf(__uint_as_float(r[c][g * 8 + 2 * u + 1]), sc, f.y * L2E));
                                    }
                                }
                        } else {
#pragma unroll
                            for (int c = 0; c < 4; ++c)
#pragma unroll
                                for (int i = 0; i < 32; ++i) {
                                    const float bv = (c * 32 + i < nvalid) ? __half2float(brow[(int64_t)(c * 32 + i) * p.bsK]) : 0.f;
                                    r[c][i] = __float_as_uint(fmaf(__uint_as_float(r[c][i]), sc, bv * L2E));
                                }
                        }
                    }
                }
                // Row maximum of the raw scores (the scale is positive, so it commutes with max);
                // eight independent chains instead of one 128-long dependent one.
                if (nvalid < ATT_BC) {
#pragma unroll
                    for (int c = 0; c < 4; ++c)
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (c * 32 + i >= nvalid) r[c][i] = 0xff800000u; // -inf: a key that does not exist gives 2^-inf = 0
                }
                float mxa = -INFINITY, mxb = -INFINITY, mxc = -INFINITY, mxd = -INFINITY;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {   // three-input max: two scores per instruction
                        mxa = fmax3(mxa, __uint_as_float(r[c][i]), __uint_as_float(r[c][i + 1]));
                        mxb = fmax3(mxb, __uint_as_float(r[c][i + 2]), __uint_as_float(r[c][i + 3]));
                        mxc = fmax3(mxc, __uint_as_float(r[c][i + 4]), __uint_as_float(r[c][i + 5]));
                        mxd = fmax3(mxd, __uint_as_float(r[c][i + 6]), __uint_as_float(r[c][i + 7]));
                    }
                }
                const float mx = fmaxf(fmaxf(mxa, mxb), fmaxf(mxc, mxd));
                // The reference point of the exponentials only has to keep 2^(x - m) inside fp16:
                // it follows the true maximum lazily, moving (and rescaling O and the running sum)
                // only when the maximum has grown by more than 2^8.  Any reference point gives the
                // same quotient O / l; the lazy one makes rescales rare after the first blocks.
                const float m_blk = mx * sce;
                const float m_new = (m_blk > m_run + 8.0f) ? m_blk : m_run;
                // 0 on the first block (m_run = -inf), else 1 or < 2^-8.  With a mask a row may have seen
                // nothing but -inf so far: then the reference point stays -inf and nothing is rescaled.
                const float alpha = (BIAS && m_run == m_new) ? 1.0f : ex2(m_run - m_new);
                const float m_sub = (BIAS && m_new == -INFINITY) ? 0.f : m_new;

                // P's shared tile and O are both still in use by the previous block's P V.
                if (j > 0 && !mbar_wait(&pv_done[t], (uint32_t)((j - 1) & 1), p.d_status, KST_WAIT_SOFTMAX, abort_flag)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                if (lane == 0 && quad == 0 && j < 6) ATT_TRACE(64 * t + 8 + 8 * j + 4);  // max done, PV(j-1) done
                // Rescale O (and the running sum in its column 64) when this row's maximum moved;
                // skipped warp-wide when no row's did — exact, the factor would be 1.
                if (j > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll 1
                    for (int c = 0; c < EP / 16; ++c) {   // 16 columns at a time: S is live in registers
                        uint32_t o16[16];
                        tmem_ld16(o_tmem + c * 16, o16);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 16; ++i) o16[i] = __float_as_uint(__uint_as_float(o16[i]) * alpha);
                        tmem_st16_raw(o_tmem + c * 16, o16);
                    }
                    tmem_wait_st();
                }

                if (pingpong && (t == 1 || j > 0)) {
                    // tile 0 waits for tile 1's block j-1, tile 1 for tile 0's block j
                    const uint32_t par = (uint32_t)((t == 1 ? j : j - 1) & 1);
                    if (!mbar_wait(&exp_turn[t], par, p.d_status, KST_WAIT_SOFTMAX, abort_flag)) { ok = false; break; }
                }
                if (lane == 0 && quad == 0 && j < 6) ATT_TRACE(64 * t + 8 + 8 * j + 5);  // rescale done, my turn
                // P = 2^(s*scale - m): fp32 exponentials, their fp32 row sum, and P rounded to fp16
                // (two keys per 32-bit column) straight into tensor memory for the P V product.
                const uint64_t sc2 = pack2(sce, sce), nm2 = pack2(-m_sub, -m_sub);
                uint64_t lsa = pack2(0.f, 0.f), lsb = pack2(0.f, 0.f);
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t pk[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        // two scores per FMA and per add (packed fp32 pairs), one ex2 each, one convert for the pair
                        const uint64_t x2 = fma2(pack2(__uint_as_float(r[c][2 * i]), __uint_as_float(r[c][2 * i + 1])), sc2, nm2);
                        float x0, x1;
                        unpack2(x2, x0, x1);
                        const float e0 = ex2(x0), e1 = ex2(x1);
                        if (i & 1) lsb = add2(lsb, pack2(e0, e1));
                        else lsa = add2(lsa, pack2(e0, e1));
                        const __half2 h2 = __floats2half2_rn(e0, e1);
                        pk[i] = *reinterpret_cast<const uint32_t*>(&h2);
                    }
                    tmem_st16_raw(p_tmem + c * 16, pk);
                    // Hand the turn over part way: the other tile's exponentials then overlap the
                    // rest of these, which keeps the MUFU pipe fed without falling in step.
                    if (c == ATT_TURN_AT && pingpong) {
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&exp_turn[1 - t]);
                    }
                }
                tmem_wait_st();
                float ls0, ls1;
                unpack2(add2(lsa, lsb), ls0, ls1);
                l_run = l_run * alpha + (ls0 + ls1);
                m_run = m_new;
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&p_full[t]);
                if (lane == 0 && quad == 0 && j < 6) ATT_TRACE(64 * t + 8 + 8 * j + 6);  // P written
                if (lane == 0 && j == 3) ATT_TRACE(56 + 64 * t + quad);                  // per-warp P written, block 3
            }

            // Epilogue: O / l to global through the caller's output strides.
            if (ok && nblk > 0)
                ok = mbar_wait(&pv_done[t], (uint32_t)((nblk - 1) & 1), p.d_status, KST_WAIT_SOFTMAX, abort_flag);
            if (ok) {
                tc_fence_after();
                const int lq = q0 + t * ATT_BR + row;
                if (nsp > 1) {
                    // Unnormalised rows and their (reference point, sum) for the merge.  tcgen05.ld is a
                    // warp-wide (.sync.aligned) instruction: every lane executes it, whether or not its
                    // row exists; only the stores are predicated.
                    const int64_t prow = ((int64_t)split * p.ntail + tailpair) * ITEM_ROWS + t * ATT_BR + row;
                    float* po = p.part_o + prow * p.E;
#pragma unroll 1
                    for (int c = 0; c < EP / 32; ++c) {
                        uint32_t r[32];
                        tmem_ld32(o_tmem + c * 32, r);
                        tmem_wait_ld();
                        if (lq < p.Lq) {
#pragma unroll
                            for (int i = 0; i < 32; i += 4)
                                if (c * 32 + i < p.E)
                                    *reinterpret_cast<float4*>(po + c * 32 + i) =
                                        make_float4(__uint_as_float(r[i]), __uint_as_float(r[i + 1]), __uint_as_float(r[i + 2]),
                                                    __uint_as_float(r[i + 3]));
                        }
                    }
                    if (lq < p.Lq) {
                        p.part_ml[prow * 2] = m_run;
                        p.part_ml[prow * 2 + 1] = l_run;
                    }
                } else {
                const float inv = 1.0f / (l_run == 0.f ? 1.0f : l_run);
                const int64_t obase = lq * p.osL + h * p.osH + b * p.osB;
#pragma unroll 1
                for (int c = 0; c < EP / 32; ++c) {
                    uint32_t r[32];
                    tmem_ld32(o_tmem + c * 32, r);
                    tmem_wait_ld();
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
                                    for (int u = 0; u < 4; ++u)
                                        hh[u] = __floats2half2_rn(__uint_as_float(r[i + 2 * u]) * inv,
                                                                  __uint_as_float(r[i + 2 * u + 1]) * inv);
                                    *reinterpret_cast<uint4*>(o + i) = w;
                                }
                            }
                        }
                    }
                }
                }   // nsplit == 1
            }
        }
    }

    if (*abort_flag) {
        for (int i = 0; i < 4; ++i) __nanosleep(1000000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 8) {
        tc_fence_after();
        tmem_dealloc(tmem_base, ATT_TMEM_COLS);
    }
}

// Combine the partial results of a key split (attn_flash_cm_merge!, flash.jl:1398-1421): one warp per
// query row; out = sum_s O_s 2^(m_s - M) / sum_s l_s 2^(m_s - M), M the largest reference point.
__global__ void __launch_bounds__(128)
attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, int nsplit, int ntail,
                       int first_pair, int qpairs, int item_rows, int E, int Lq, int H, void* out, int64_t osL, int64_t osH,
                       int64_t osB, int out_f32) {
    grid_dep_wait();
    const int lane = threadIdx.x & 31;
    const int64_t rows = (int64_t)ntail * item_rows;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int pair = first_pair + (int)(row / item_rows);
    const int lq = (pair % qpairs) * item_rows + (int)(row % item_rows);
    if (lq >= Lq) return;
    const int h = (pair / qpairs) % H, b = pair / (qpairs * H);
    float M = -INFINITY;
    for (int s = 0; s < nsplit; ++s) M = fmaxf(M, part_ml[(s * rows + row) * 2]);
    float den = 0.f, num[4] = {0.f, 0.f, 0.f, 0.f};   // E <= 128: up to four elements per lane
    for (int s = 0; s < nsplit; ++s) {
        const float m = part_ml[(s * rows + row) * 2], l = part_ml[(s * rows + row) * 2 + 1];
        const float w = (m == -INFINITY) ? 0.f : exp2f(m - M);
        den = fmaf(l, w, den);
        const float* po = part_o + (s * rows + row) * E;
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (lane + 32 * u < E) num[u] = fmaf(po[lane + 32 * u], w, num[u]);
    }
    const float inv = 1.0f / (den == 0.f ? 1.0f : den);
    const int64_t obase = lq * osL + h * osH + b * osB;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        if (lane + 32 * u >= E) continue;
        if (out_f32) static_cast<float*>(out)[obase + lane + 32 * u] = num[u] * inv;
        else static_cast<__half*>(out)[obase + lane + 32 * u] = __float2half_rn(num[u] * inv);
    }
}

// Scalar path for operands a tensor map cannot express (E > 128, E not a multiple of 8,
// unaligned strides): one warp per query row, two passes over the keys.
__global__ void attention_f16_scalar_kernel(int E, int Lq, int Lk, int H, int B, const __half* q, int64_t qsE, int64_t qsL, int64_t qsH, int64_t qsB,
                                            const __half* k, int64_t ksE, int64_t ksL, int64_t ksH, int64_t ksB,
                                            const __half* v, int64_t vsE, int64_t vsL, int64_t vsH, int64_t vsB,
                                            void* out, int64_t osL, int64_t osH, int64_t osB, int out_f32, float scale,
                                            const __half* bias, int64_t bsK, int64_t bsQ, int64_t bsH, int64_t bsB) {
    const int lane = threadIdx.x & 31;
    const int64_t rowid = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (rowid >= (int64_t)Lq * H * B) return;
    const int lq = (int)(rowid % Lq);
    const int h = (int)((rowid / Lq) % H);
    const int b = (int)(rowid / ((int64_t)Lq * H));
    const __half* qp = q + qsL * lq + qsH * h + qsB * b;
    const __half* kp = k + ksH * h + ksB * b;
    const __half* vp = v + vsH * h + vsB * b;
    const __half* bp = bias ? bias + bsQ * lq + bsH * h + bsB * b : nullptr;
    float m = -INFINITY;
    for (int lk = lane; lk < Lk; lk += 32) {
        float a = 0.f;
        for (int e = 0; e < E; ++e) a = fmaf(__half2float(qp[qsE * e]), __half2float(kp[ksL * lk + ksE * e]), a);
        a *= scale;
        if (bp) a += __half2float(bp[bsK * lk]);
        m = fmaxf(m, a);
    }
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (m == -INFINITY) m = 0.f;   // every key blocked: all exponentials are zero and the row divides by one
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
            a *= scale;
            if (bp) a += __half2float(bp[bsK * lk]);
            pexp = __expf(a - m);
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

// ----------------------------------------------------------------------- the two-GEMM route
// Attention as two batched tensor-core GEMMs with a softmax between them, for head dims the fused kernel's
// tensor memory cannot hold (E > 128): S(Lk, Lq) = Kt(Lk, E) . Q(E, Lq) in fp32, P = softmax over the keys
// (fp16, already divided by the row sum), O(E, Lq) = V(E, Lk) . P(Lk, Lq) written straight into out.  The
// reference's second tier, sdpa_coopmat! + attn_softmax_rows! (attention.jl:528-705), restated for this
// GEMM's orientation: only K is transposed (one permuted copy), Q and V are read through their strides, and
// the scores keep the keys contiguous so that the softmax reads and writes whole rows.
//
// One warp per (query, head*batch) column of S: scale (+ additive mask), maximum, exponentials, sum, P.  A
// column whose keys are all blocked comes out as zeros (attn_softmax, attention.jl:73-100).
__global__ void __launch_bounds__(256)
attn_softmax_cols_kernel(const float* __restrict__ S, __half* __restrict__ P, int Lk, int64_t ldS, int CH, int64_t ncols,
                         float scale, const __half* __restrict__ bias, int64_t bsK, int64_t bsQ, int64_t bsH, int64_t bsB,
                         int q0, int Lq, int H) {
    const int lane = threadIdx.x & 31;
    const int64_t col = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);   // lq_local + CH * hb
    if (col >= ncols) return;
    const int lq = q0 + (int)(col % CH);
    if (lq >= Lq) return;   // a short last chunk: the columns past it hold an earlier chunk's scores and are not used
    const int hb = (int)(col / CH);
    const float* s = S + col * ldS;
    __half* p = P + col * ldS;
    const __half* bp = bias ? bias + (int64_t)lq * bsQ + (int64_t)(hb % H) * bsH + (int64_t)(hb / H) * bsB : nullptr;
    float m = -INFINITY;
    for (int k = lane; k < Lk; k += 32) {
        float a = s[k] * scale;
        if (bp) a += __half2float(bp[(int64_t)k * bsK]);
        m = fmaxf(m, a);
    }
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (m == -INFINITY) m = 0.f;
    float l = 0.f;
    for (int k = lane; k < Lk; k += 32) {
        float a = s[k] * scale;
        if (bp) a += __half2float(bp[(int64_t)k * bsK]);
        l += __expf(a - m);
    }
    for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
    const float inv = 1.0f / (l == 0.f ? 1.0f : l);
    for (int k = lane; k < Lk; k += 32) {
        float a = s[k] * scale;
        if (bp) a += __half2float(bp[(int64_t)k * bsK]);
        p[k] = __float2half_rn(__expf(a - m) * inv);
    }
}

static int attention_two_gemm(b200_ctx* ctx, int64_t E, int64_t Lq, int64_t Lk, int64_t H, int64_t B,
                              const b200_strided4* q, const b200_strided4* k, const b200_strided4* v,
                              const __half* bias, const int64_t* bs, const b200_strided4* o, int out_dtype, float scale) {
    const int64_t HB = H * B;
    const size_t osz = out_dtype == B200_F16 ? 2 : 4;
    int rc;
    // Kt(Lk, E, H, B), dense: the one layout pass of this route (the reference transposes Q and V as well)
    void* kT = nullptr;
    if ((rc = ws_scratch(ctx, (size_t)(Lk * E * HB) * 2, &kT))) return rc;
    {
        const int64_t shape[4] = {Lk, E, H, B};
        const int64_t stride[4] = {k->stride[1], 1, k->stride[2], k->stride[3]};
        if ((rc = b200_permute4(ctx, k->ptr, kT, shape, stride, 2))) return rc;
    }
    // Queries are taken in chunks so that the fp32 scores and the fp16 probabilities stay within ~256 MB.
    int64_t CH = (int64_t)(256ll << 20) / (Lk * HB * 6);
    if (CH > Lq) CH = Lq;
    CH = CH / 8 * 8;
    if (CH < 8) CH = Lq < 8 ? Lq : 8;
    void *S = nullptr, *P = nullptr;
    if ((rc = ws_scratch(ctx, (size_t)(Lk * CH * HB) * 4, &S))) return rc;
    if ((rc = ws_scratch(ctx, (size_t)(Lk * CH * HB) * 2, &P))) return rc;
    // One batched launch over (h, b) when the operands' head and batch strides fold into one, else one per image.
    auto folds = [&](const b200_strided4* t) { return B == 1 || t->stride[3] == H * t->stride[2]; };
    const bool one = folds(q) && folds(v) && folds(o);
    const int64_t nb = one ? HB : H, reps = one ? 1 : B;
    for (int64_t q0 = 0; q0 < Lq; q0 += CH) {
        const int64_t n = Lq - q0 < CH ? Lq - q0 : CH;
        for (int64_t r = 0; r < reps; ++r) {
            const __half* qp = (const __half*)q->ptr + q0 * q->stride[1] + r * q->stride[3];
            if ((rc = gemm_f16_run(ctx, Lk, n, E, (const __half*)kT + r * H * Lk * E, Lk, qp, q->stride[1], nullptr, 0,
                                   (float*)S + r * H * Lk * CH, Lk, B200_F32, B200_EPI_NONE, nb, Lk * E, q->stride[2],
                                   Lk * CH)))
                return rc;
        }
        const int64_t ncols = CH * HB;
        attn_softmax_cols_kernel<<<(unsigned)cdiv(ncols, 8), 256, 0, ctx->stream>>>(
            (const float*)S, (__half*)P, (int)Lk, Lk, (int)CH, ncols, scale, bias, bs[0], bs[1], bs[2], bs[3], (int)q0, (int)Lq,
            (int)H);
        ctx->launches++;
        B200_CUDA(cudaGetLastError());
        for (int64_t r = 0; r < reps; ++r) {
            const __half* vp = (const __half*)v->ptr + r * v->stride[3];
            char* op = (char*)const_cast<void*>(o->ptr) + (size_t)(q0 * o->stride[1] + r * o->stride[3]) * osz;
            if ((rc = gemm_f16_run(ctx, E, n, Lk, vp, v->stride[1], (const __half*)P + r * H * Lk * CH, Lk, nullptr, 0, op,
                                   o->stride[1], out_dtype, B200_EPI_NONE, nb, v->stride[2], Lk * CH, o->stride[2])))
                return rc;
        }
    }
    return B200_OK;
}

static int tc_reason(int64_t E, int64_t Lq, int64_t Lk, int64_t H, int64_t B, const int64_t* qs,
                     const int64_t* ks, const int64_t* vs) {
    if (E < 1 || Lq < 1 || Lk < 1 || H < 1 || B < 1) return B200_DECLINE_EXTENT;
    if (E > 128 || E % 8 != 0) return B200_DECLINE_TILING;
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
    uint32_t box[4] = {64, 128, 1, 1};   // one swizzle atom; a head dim above 64 takes two boxes per tile
    return make_tmap(ctx, m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, t->ptr, dims, str, box,
                     CU_TENSOR_MAP_SWIZZLE_128B);
}

} // namespace b200

using namespace b200;

extern "C" {

int b200_attention_f16_supported(int64_t E, int64_t Lq, int64_t Lk, int64_t H, int64_t B,
                                 const int64_t* qstride, const int64_t* kstride, const int64_t* vstride,
                                 int has_bias) {
    (void)has_bias;   // an additive mask no longer declines: b200_attention_f16_bias takes it
    if (!qstride || !kstride || !vstride) return B200_EINVAL;
    return tc_reason(E, Lq, Lk, H, B, qstride, kstride, vstride);
}

int b200_attention_f16_route(int64_t E, int64_t Lq, int64_t Lk, int64_t H, int64_t B, const int64_t* qstride,
                             const int64_t* kstride, const int64_t* vstride) {
    if (!qstride || !kstride || !vstride) return -1;
    if (tc_reason(E, Lq, Lk, H, B, qstride, kstride, vstride) == B200_OK) return 0;
    // Two batched GEMMs and a softmax: head dims past the fused kernel's, when the GEMM's tensor maps can take the
    // operands as they lie (E contiguous and a multiple of 8) and the problem is worth three launches.
    if (E > 128 && E % 8 == 0 && E <= 4096 && Lq >= 1 && Lk >= 1 && H >= 1 && B >= 1 && Lk < (1ll << 31) && Lq < (1ll << 31) &&
        qstride[0] == 1 && kstride[0] == 1 && vstride[0] == 1 && Lq * Lk >= 64 * 64)
        return 1;
    return 2;
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
    return b200_attention_f16_bias(ctx, E, Lq, Lk, H, B, q, k, v, nullptr, o, out_dtype, scale);
}

int b200_attention_f16_bias(b200_ctx* ctx, int64_t E, int64_t Lq, int64_t Lk, int64_t H, int64_t B,
                            const b200_strided4* q, const b200_strided4* k, const b200_strided4* v,
                            const b200_strided4* bias, const b200_strided4* o, int out_dtype, float scale) {
    B200_REQUIRE(ctx && q && k && v && o, B200_EINVAL, "attention: null argument");
    const __half* bptr = (bias != nullptr) ? static_cast<const __half*>(bias->ptr) : nullptr;
    const int64_t bs[4] = {bptr ? bias->stride[0] : 0, bptr ? bias->stride[1] : 0, bptr ? bias->stride[2] : 0,
                           bptr ? bias->stride[3] : 0};
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
                    al16(k->ptr) && al16(v->ptr) && al16(out) && oaligned && scale > 0.f;
    if (!tc && b200_attention_f16_route(E, Lq, Lk, H, B, q->stride, k->stride, v->stride) == 1 && scale > 0.f &&
        o->stride[1] > 0 && o->stride[2] > 0 && o->stride[3] > 0)
        return attention_two_gemm(ctx, E, Lq, Lk, H, B, q, k, v, bptr, bs, o, out_dtype, scale);
    if (!tc) {
        B200_REQUIRE(E <= 1024, B200_DECLINE_EXTENT, "attention: E = %lld", (long long)E);
        const int wpb = 4;
        const int64_t rows = Lq * H * B;
        attention_f16_scalar_kernel<<<(unsigned)cdiv(rows, wpb), 32 * wpb, wpb * E * sizeof(float), ctx->stream>>>(
            (int)E, (int)Lq, (int)Lk, (int)H, (int)B, (const __half*)q->ptr, q->stride[0], q->stride[1],
            q->stride[2], q->stride[3], (const __half*)k->ptr, k->stride[0], k->stride[1], k->stride[2],
            k->stride[3], (const __half*)v->ptr, v->stride[0], v->stride[1], v->stride[2], v->stride[3], out,
            o->stride[1], o->stride[2], o->stride[3], out_dtype == B200_F32, scale, bptr, bs[0], bs[1], bs[2], bs[3]);
        ctx->launches++;
        B200_CUDA(cudaGetLastError());
        return B200_OK;
    }
    static bool attr_done[16] = {};
    if (!attr_done[ctx->device & 15]) {
        B200_CUDA(cudaFuncSetAttribute(attention_f16_tc_kernel<64, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       AttCfg<64>::SMEM_BYTES));
        B200_CUDA(cudaFuncSetAttribute(attention_f16_tc_kernel<64, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       AttCfg<64>::SMEM_BYTES));
        B200_CUDA(cudaFuncSetAttribute(attention_f16_tc_kernel<128, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       AttCfg<128>::SMEM_BYTES));
        B200_CUDA(cudaFuncSetAttribute(attention_f16_tc_kernel<128, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       AttCfg<128>::SMEM_BYTES));
        attr_done[ctx->device & 15] = true;
    }
    // Many windows of at most 64 keys: bound by HBM and latency, not by the tensor pipe; the small-tile
    // kernel keeps six CTAs per SM in flight where this one's set-up would cost more than the arithmetic.
    if (bptr == nullptr && E <= 64 && Lk <= 64 && B * H * cdiv(Lq, 64) > 2 * ctx->prop.multiProcessorCount)
        return attention_window_launch(ctx, E, Lq, Lk, H, B, q, k, v, o, out_dtype, scale);
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
    p.trace = ctx->gemm_trace;
    p.bias = bptr;
    p.bsK = bs[0]; p.bsQ = bs[1]; p.bsH = bs[2]; p.bsB = bs[3];
    p.bias_vec = bptr && bs[0] == 1 && al16(bptr) && bs[1] % 8 == 0 && bs[2] % 8 == 0 && bs[3] % 8 == 0;
    const bool wide = E > 64;                              // two swizzle atoms along E
    const int64_t item_rows = wide ? AttCfg<128>::NT * ATT_BR : AttCfg<64>::NT * ATT_BR;
    const size_t smem_bytes = wide ? AttCfg<128>::SMEM_BYTES : AttCfg<64>::SMEM_BYTES;
    auto launch = [&](dim3 grid) -> cudaError_t {
        if (wide)
            return bptr ? launch_dep(attention_f16_tc_kernel<128, true>, grid, dim3(ATT_THREADS, 1, 1), smem_bytes, ctx->stream, 1, tq, tk, tv, p)
                        : launch_dep(attention_f16_tc_kernel<128, false>, grid, dim3(ATT_THREADS, 1, 1), smem_bytes, ctx->stream, 1, tq, tk, tv, p);
        return bptr ? launch_dep(attention_f16_tc_kernel<64, true>, grid, dim3(ATT_THREADS, 1, 1), smem_bytes, ctx->stream, 1, tq, tk, tv, p)
                    : launch_dep(attention_f16_tc_kernel<64, false>, grid, dim3(ATT_THREADS, 1, 1), smem_bytes, ctx->stream, 1, tq, tk, tv, p);
    };
    p.qpairs = (int)cdiv(Lq, item_rows);
    const int64_t pairs = (int64_t)p.qpairs * H * B;      // work items: pairs of query tiles, or single tiles when wide
    B200_REQUIRE(pairs < (1ll << 30), B200_DECLINE_EXTENT, "attention: too many query tiles");
    const int64_t sms = ctx->prop.multiProcessorCount;
    // Two cases cut pairs along the keys (at least two key blocks per piece) and merge afterwards:
    // few queries over many keys (a decode step, Lq = 23, Lk = 4096: every pair is cut so that the
    // SMs are all used), and a last wave that would leave most SMs idle (its pairs are cut so that
    // the wave is as short as the cut allows instead of a whole pair long).
    p.nsplit = 1;
    p.ntail = 0;
    p.part_o = p.part_ml = nullptr;
    const int64_t nblk_all = cdiv(Lk, ATT_BC);
    const int64_t rem = pairs % sms;
    if (bptr == nullptr && nblk_all >= 4) {
        int64_t ntail = 0, ns = 1;
        if (2 * pairs <= sms) {
            ntail = pairs;
            ns = sms / pairs;
        } else if (pairs > sms && rem > 0 && 2 * rem <= sms) {
            ntail = rem;
            ns = sms / rem;
        }
        if (ns > nblk_all / 2) ns = nblk_all / 2;
        if (ns > 64) ns = 64;
        if (ntail > 0 && ns >= 2) {
            const int64_t rows = ntail * item_rows;
            void* ws = nullptr;
            rc = ws_scratch(ctx, (size_t)(ns * rows * (E + 2)) * sizeof(float), &ws);
            if (rc) return rc;
            p.nsplit = (int)ns;
            p.ntail = (int)ntail;
            p.part_o = static_cast<float*>(ws);
            p.part_ml = p.part_o + ns * rows * E;
        }
    }
    if (p.nsplit > 1) {
        p.pair_ctas = (int)(pairs - p.ntail);
        const int64_t ctas = p.pair_ctas + (int64_t)p.ntail * p.nsplit;
        B200_CUDA(launch(dim3((unsigned)ctas, 1, 1)));
        const int64_t rows = (int64_t)p.ntail * item_rows;
        B200_CUDA(launch_dep(attention_merge_kernel, dim3((unsigned)cdiv(rows, 4), 1, 1), dim3(128, 1, 1), 0, ctx->stream, 1,
                             (const float*)p.part_o, (const float*)p.part_ml, p.nsplit, p.ntail, p.pair_ctas, p.qpairs, (int)item_rows, (int)E,
                             (int)Lq, (int)H, out, o->stride[1], o->stride[2], o->stride[3], (int)(out_dtype == B200_F32)));
        ctx->launches += 2;
        return B200_OK;
    }
    // Split the pairs of a last wave that would leave more than half of the SMs idle — but not a
    // pair whose second tile does not exist.
    int64_t nsplit = (pairs > sms && rem > 0 && 2 * rem <= sms && Lq % (2 * ATT_BR) == 0) ? rem : 0;
    p.pair_ctas = (int)(pairs - nsplit);
    B200_CUDA(launch(dim3((unsigned)(pairs + nsplit), 1, 1)));
    ctx->launches++;
    return B200_OK;
}

} // extern "C"
