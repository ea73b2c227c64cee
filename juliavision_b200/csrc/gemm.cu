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
// Roles inside one persistent CTA (608 threads):
//   warp 0     TMA producer  (one lane)        global -> shared ring, STAGES deep
//   warp 1     UMMA issuer   (one lane issues) shared -> TMEM accumulators (two, ping-pong)
//   warps 2-17 epilogue      (512 threads)     TMEM -> registers -> +bias, round, act ->
//                                              warp-private shared slab -> bulk tensor store
//   warp 18    relay                           waits for each stage to land and passes that on to the
//                                              issuer through a named barrier (see the issuer's comment)
#include <cuda_fp16.h>
#include <stdio.h>
#include <stdlib.h>

#include "act.cuh"
#include "internal.h"
#include "ptx.cuh"

namespace b200 {

constexpr int GEMM_BM = 128; // tokens per CTA (TMEM lanes)
constexpr int GEMM_BK = 64;  // one 128-byte swizzle row of fp16
constexpr int EPI_WARPS = 16;
constexpr int RELAY_WARP = 2 + EPI_WARPS;
constexpr int GEMM_THREADS = 64 + 32 * EPI_WARPS + 32; // producer warp, UMMA warp, epilogue warps, relay warp
static_assert(GEMM_BK == 64, "the UMMA issuer unrolls four K = 16 steps per k-block");
constexpr int SMEM_LIMIT = 232448; // 227 KB

// NCTA = 1: one CTA per tile of 128 tokens x BN features (tcgen05.mma.cta_group::1).
// NCTA = 2: a cluster of two CTAs per tile of 256 tokens x BN features (cta_group::2, UMMA M = 256):
//           each CTA stages its own 128 token rows and BN/2 of the feature columns, so the shared
//           memory traffic per flop halves and the tensor core is no longer starved by it.
// BN = 512 (pairs only) is the wide tile: one accumulator of up to 512 columns instead of two of BN, two UMMAs
//           per K step (256 columns + the rest), the tile's width a launch parameter (a multiple of 16 in
//           (256, 512]).  It is for launches whose 256-wide tiles would need a second, mostly empty round of
//           the workers: the width is chosen so that every tile is some worker's only one.
template <int BN, typename OutT, int NCTA> struct GemmCfg {
    static constexpr bool WIDE = BN == 512;
    static_assert(!WIDE || NCTA == 2, "the wide tile is built for CTA pairs");
    static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
    static constexpr int B_CHUNK_BYTES = 64 * GEMM_BK * 2; // one 64-feature slab of the B tile
    static constexpr int B_COLS = BN / NCTA;               // feature columns this CTA stages
    static constexpr int B_BYTES = B_COLS * GEMM_BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int OUT_COLS = 128 / (int)sizeof(OutT); // columns per 128-byte staging row
    static constexpr int SUB_COLS = 64 / (int)sizeof(OutT);   // epilogue slab: 64 bytes of output per row
    static constexpr int TAIL_BYTES = EPI_WARPS * (BN / (EPI_WARPS / 4) * 4 + 32 * 16 * (int)sizeof(OutT)) + 256; // per-warp fp32 bias of its own columns and one staged chunk; barriers
    static constexpr int STAGES_RAW = (SMEM_LIMIT - TAIL_BYTES) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + TAIL_BYTES;
    static constexpr int TMEM_COLS = WIDE ? 512 : (2 * BN < 32 ? 32 : 2 * BN);
    static_assert(STAGES >= 2, "ring too shallow");
    static_assert(SMEM_BYTES <= SMEM_LIMIT, "shared memory over budget");
    static_assert(TMEM_COLS == 128 || TMEM_COLS == 256 || TMEM_COLS == 512, "TMEM columns");
    static_assert(B_COLS % 64 == 0, "each CTA stages whole 64-column slabs of B");
    static_assert((EPI_WARPS * (BN / (EPI_WARPS / 4)) * 4) % 512 == 0 && (STAGES * STAGE_BYTES) % 1024 == 0,
                  "the epilogue slabs must start on the swizzle pattern's period");
};

template <typename OutT> struct GemmParams {
    int64_t M, N, K;       // out features, tokens, reduction
    int tiles_m, tiles_n;  // feature tiles, token tiles
    int bn;                // feature columns per tile: BN, or the wide tile's width
    uint32_t total_tiles;  // tiles_m * tiles_n * nbatch (times num_kb below 2^31, checked at launch)
    int num_kb;
    OutT* out;             // out(M,N): element (i,j) of plane b at out[b*strideO + j*ldo + i]
    int64_t ldo, strideO;
    const __half* bias;
    int bias_per_n;        // 0: bias[i] over features (M); 1: bias[j] over tokens (N)
    int epilogue;
    int streamk;           // 0: whole tiles, strided over the workers; 1 + lean: contiguous k-block ranges per worker (see SegIter)
    float* sk_part;        // stream-K: fp32 partial accumulators, one 128 x BN block per (worker, CTA rank)
    int* sk_flag;          // stream-K: one flag per (worker, CTA rank, epilogue warp), zero between launches
    int* d_status;
    unsigned long long* trace;  // optional timeline of worker 0 (globaltimer ns), null in normal use
};

// Timeline slots written by worker 0 when tracing (b200_timeline): globaltimer ns at [slot] and
// the SM's own cycle counter at [64 + slot], so a phase can be read both in time and in cycles (their
// ratio is the clock the SM actually ran at).  Costs one predictable branch per event otherwise.
#define GEMM_TRACE(slot)                                                   \
    do {                                                                   \
        if (p.trace != nullptr && worker == 0 && rank == 0) {              \
            p.trace[(slot)] = globaltimer_ns();                            \
            p.trace[64 + (slot)] = (unsigned long long)clock64();          \
        }                                                                  \
    } while (0)

// The work of one worker (a CTA, or a CTA pair) as a sequence of segments, a segment being the
// k-blocks [kb0, kb1) of one tile.
//   whole-tile mode: worker w takes tiles w, w + W, w + 2W, ... each with all its k-blocks;
//   stream-K mode:   the (tile, k-block) pairs, tile-major, are cut into W equal contiguous ranges,
//                    so every worker does the same number of k-blocks whatever the tile count.  A
//                    tile cut by a range boundary is finished by the worker that holds its first
//                    k-block (that segment comes last in the worker's range); the workers holding
//                    its later k-blocks (their first segment) leave fp32 partials for it.
struct SegIter {
    // 32-bit throughout (the host refuses a launch whose tiles x k-blocks do not fit): every role of every
    // CTA walks this per tile, and what the sixteen epilogue warps issue there is taken from the UMMA
    // issuer's share of the schedulers, so a 64-bit division here costs main-loop time.
    uint32_t tile, u, uend, step;
    int kb0, kb1, nkb, streamk;
    // `lean` (stream-K with exactly two workers per tile) moves that many k-blocks from the second worker of a
    // tile, whose fp32 partial then takes ~6 us to reach the first (write-out + fence + flag), to the first.
    __device__ __forceinline__ static uint32_t range_start(uint32_t units, uint32_t w, uint32_t W, uint32_t lean) {
        const uint32_t r = units / W * w + units % W * w / W;   // floor(units * w / W) without leaving 32 bits (w <= W < 2^16)
        return (w & 1u) && w < W ? r + lean : r;
    }
    __device__ __forceinline__ void set() {
        if (streamk) {
            tile = u / (uint32_t)nkb;
            kb0 = (int)(u - tile * (uint32_t)nkb);
            const uint32_t left = uend - u;
            kb1 = (uint32_t)(nkb - kb0) < left ? nkb : kb0 + (int)left;
        } else {
            tile = u;
            kb0 = 0;
            kb1 = nkb;
        }
    }
    __device__ __forceinline__ void init(uint32_t total_tiles, int nkb_, int streamk_, uint32_t w, uint32_t W) {
        nkb = nkb_;
        streamk = streamk_;
        if (streamk) {
            u = range_start(total_tiles * (uint32_t)nkb, w, W, (uint32_t)streamk - 1u);
            uend = range_start(total_tiles * (uint32_t)nkb, w + 1, W, (uint32_t)streamk - 1u);
            step = 0;
        } else {
            u = w;
            uend = total_tiles;
            step = W;
        }
        set();
    }
    __device__ __forceinline__ bool valid() const { return u < uend; }
    __device__ __forceinline__ void next() {
        // whole-tile mode: the last step may pass total_tiles by up to W, far below 2^32 (total_tiles < 2^31)
        u += streamk ? (uint32_t)(kb1 - kb0) : step;
        set();
    }
};

// Where tile `tile` sits: plane, first feature, first token.  One 32-bit division when there is one plane.
struct TileAt { int batch, tm, tn; };
__device__ __forceinline__ TileAt tile_at(uint32_t tile, uint32_t tiles_m, uint32_t tiles_per_batch, bool one_plane) {
    TileAt t;
    uint32_t rem = tile;
    t.batch = 0;
    if (!one_plane) {
        t.batch = (int)(tile / tiles_per_batch);
        rem = tile - (uint32_t)t.batch * tiles_per_batch;
    }
    t.tn = (int)(rem / tiles_m);
    t.tm = (int)(rem - (uint32_t)t.tn * tiles_m);
    return t;
}

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_gpu(int* p, int v) {
    asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

template <int BN, typename OutT, int NCTA>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_f16_tc_kernel(const __grid_constant__ CUtensorMap tmapX,   // B(K,N): {K, tokens, batch}
                   const __grid_constant__ CUtensorMap tmapW,   // A(M,K): {features, K, batch}
                   const __grid_constant__ CUtensorMap tmapO,   // out(M,N): {features, tokens, batch}, boxes of 16 x 32
                   const GemmParams<OutT> p) {
    using Cfg = GemmCfg<BN, OutT, NCTA>;
    constexpr int TILE_N = GEMM_BM * NCTA; // tokens per tile
    // The swizzled tiles need a 1024-byte aligned base.  The declaration asks for it; should a
    // toolchain not honour that, every thread of the grid sees the same misaligned offset and
    // leaves before any barrier, cluster sync or TMEM allocation exists.
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw;
    if ((smem_u32(smem_raw) & 1023u) != 0) {
        if (threadIdx.x == 0) atomicCAS(p.d_status, 0, KST_SMEM_LAYOUT);
        return;
    }
    __half* sbias = reinterpret_cast<__half*>(smem + Cfg::STAGES * Cfg::STAGE_BYTES);
    uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(sbias) + EPI_WARPS * (BN / (EPI_WARPS / 4) * 4 + 32 * 16 * (int)sizeof(OutT)));
    uint64_t* full = bars;                     // [STAGES]  (pair: only the leader's are used)
    uint64_t* empty = bars + Cfg::STAGES;      // [STAGES]
    uint64_t* tfull = bars + 2 * Cfg::STAGES;  // [2]
    uint64_t* tempty = tfull + 2;              // [2]      (pair: only the leader's are used)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = NCTA == 2 ? cluster_ctarank() : 0u;  // 0 = the CTA that issues the UMMAs
    const uint32_t worker = NCTA == 2 ? (blockIdx.x >> 1) : blockIdx.x;
    const uint32_t nworkers = NCTA == 2 ? (gridDim.x >> 1) : gridDim.x;

    if (threadIdx.x == 0) {
        GEMM_TRACE(0); // kernel entry
        for (int s = 0; s < Cfg::STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&tfull[a], 1);
            mbar_init(&tempty[a], EPI_WARPS * NCTA);
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tmap(&tmapX);
        prefetch_tmap(&tmapW);
        prefetch_tmap(&tmapO);
    }
    if (warp == 1) {
        if constexpr (NCTA == 2) {
            tmem_alloc_pair(tmem_slot, Cfg::TMEM_COLS);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
            tmem_relinquish();
        }
    }
    tc_fence_before();
    if constexpr (NCTA == 2) cluster_sync_all(); // both CTAs' barriers and TMEM exist before any use
    else __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tiles_per_batch = (uint32_t)p.tiles_m * (uint32_t)p.tiles_n;
    const bool one_plane = tiles_per_batch == p.total_tiles;
    // Everything above overlapped the previous kernel's tail; from here on its results are needed.
    // (Starting the weight operand's first stages above this wait, for launches whose predecessor is known
    // not to write the weights, was measured on the 32-layer encoder pass: 1 % slower, so nothing is fetched early.)
    grid_dep_wait();
    grid_dep_launch();

    if (threadIdx.x == 0) GEMM_TRACE(1); // setup done

    if (warp == 0) {
        // ------------------------------------------------------------- TMA producer
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            SegIter seg;
            for (seg.init(p.total_tiles, p.num_kb, p.streamk, worker, nworkers); ok && seg.valid(); seg.next()) {
                const TileAt at = tile_at(seg.tile, (uint32_t)p.tiles_m, tiles_per_batch, one_plane);
                const int batch = at.batch;
                const int m0 = Cfg::WIDE ? at.tm * p.bn : at.tm * BN + (int)rank * Cfg::B_COLS;
                const int n0 = at.tn * TILE_N + (int)rank * GEMM_BM;
                // wide tile: this CTA stages its half of the first 256 columns (slabs 0, 1) and its half of the
                // remaining n2 (slabs 2, 3: whole 64-column boxes, so up to 63 columns more than needed)
                const int n2h = (p.bn - 256) >> 1;
                const int slabs2 = (n2h + 63) >> 6;
                for (int kb = seg.kb0; kb < seg.kb1; ++kb) {
                    if (!mbar_wait(&empty[s], ph ^ 1, p.d_status, KST_WAIT_EMPTY, abort_flag)) {
                        ok = false;
                        break;
                    }
                    uint8_t* sa = smem + s * Cfg::STAGE_BYTES;
                    uint8_t* sb = sa + Cfg::A_BYTES;
                    if constexpr (NCTA == 2) {
                        // Both CTAs' bytes are counted on the leader's barrier; the leader posts
                        // the expectation for the pair.
                        const uint32_t bar = mapa_u32(smem_u32(&full[s]), 0);
                        if constexpr (Cfg::WIDE) {
                            if (rank == 0) mbar_arrive_expect_tx(&full[s], 2 * (Cfg::A_BYTES + (2 + slabs2) * Cfg::B_CHUNK_BYTES));
                            tma_load_3d_pair(sa, &tmapX, bar, kb * GEMM_BK, n0, batch);
#pragma unroll
                            for (int j = 0; j < 2; ++j)
                                tma_load_3d_pair(sb + j * Cfg::B_CHUNK_BYTES, &tmapW, bar, m0 + (int)rank * 128 + j * 64, kb * GEMM_BK, batch);
                            for (int j = 0; j < slabs2; ++j)
                                tma_load_3d_pair(sb + (2 + j) * Cfg::B_CHUNK_BYTES, &tmapW, bar, m0 + 256 + (int)rank * n2h + j * 64, kb * GEMM_BK, batch);
                        } else {
                            if (rank == 0) mbar_arrive_expect_tx(&full[s], 2 * Cfg::STAGE_BYTES);
                            tma_load_3d_pair(sa, &tmapX, bar, kb * GEMM_BK, n0, batch);
#pragma unroll
                            for (int j = 0; j < Cfg::B_COLS / 64; ++j)
                                tma_load_3d_pair(sb + j * Cfg::B_CHUNK_BYTES, &tmapW, bar, m0 + j * 64, kb * GEMM_BK, batch);
                        }
                    } else {
                        mbar_arrive_expect_tx(&full[s], Cfg::STAGE_BYTES);
                        tma_load_3d(sa, &tmapX, &full[s], kb * GEMM_BK, n0, batch);
#pragma unroll
                        for (int j = 0; j < Cfg::B_COLS / 64; ++j)
                            tma_load_3d(sb + j * Cfg::B_CHUNK_BYTES, &tmapW, &full[s], m0 + j * 64, kb * GEMM_BK, batch);
                    }
                    if (++s == Cfg::STAGES) { s = 0; ph ^= 1; }
                }
                GEMM_TRACE(2); // producer: last load of a tile issued (overwritten per tile)
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------- UMMA issuer
        // What one k-block costs the issuing thread, measured with the SM's cycle counter on a stand-alone
        // loop of the same instructions: 64 cycles per tcgen05.mma (whatever N), ~45 for the commit, and
        // ~215 more for the first shared-memory read after them whose value the thread needs — which is what
        // an mbarrier test is.  4 x 64 + 45 + 215 made every k-block take 560-590 cycles for every tile width,
        // above the 512 the tensor pipe needs for a 256-wide pair tile.  So this thread never reads shared
        // memory in its loop: the relay warp watches the stage barriers and hands each "stage has landed"
        // over through a named barrier (a hardware barrier, ~100 cycles here), one per stage of the ring.
        // The whole warp runs the loop so that the barrier instruction is warp-uniform; lane 0 issues.
        if (rank == 0) {
            constexpr uint32_t idesc = make_idesc_f16(TILE_N, Cfg::WIDE ? 256 : BN, /*a K-major*/ 0, /*b MN-major*/ 1);
            const uint32_t idesc2 = make_idesc_f16(TILE_N, p.bn - 256, 0, 1);   // wide tile: the columns past 256
            constexpr uint64_t adesc0 = make_smem_desc(16, 1024);
            constexpr uint64_t bdesc0 = make_smem_desc(Cfg::B_CHUNK_BYTES, 1024);
            int s = 0;
            int it = 0;
            SegIter seg;
            for (seg.init(p.total_tiles, p.num_kb, p.streamk, worker, nworkers); seg.valid(); seg.next(), ++it) {
                const int acc = Cfg::WIDE ? 0 : (int)(it & 1);
                const uint32_t aph = (uint32_t)((Cfg::WIDE ? it : it >> 1) & 1);
                bool got;
                if constexpr (NCTA == 2) got = mbar_wait_cluster(&tempty[acc], aph ^ 1, p.d_status, KST_WAIT_TMEM_EMPTY, abort_flag);
                else got = mbar_wait(&tempty[acc], aph ^ 1, p.d_status, KST_WAIT_TMEM_EMPTY, abort_flag);
                if (__any_sync(0xffffffffu, !got)) break;   // one answer per warp; the relay keeps arriving, which is harmless
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = seg.kb0; kb < seg.kb1; ++kb) {
                    named_bar_sync(1 + s, 64);   // the relay has seen full[s] complete (or has given up: see there)
                    tc_fence_after();
                    if (lane == 0) {
                        if (kb == seg.kb0 && it == 0) GEMM_TRACE(3); // first stage landed
                        const uint32_t a_addr = smem_u32(smem + s * Cfg::STAGE_BYTES);
                        const uint32_t b_addr = a_addr + Cfg::A_BYTES;
                        // low descriptor words: the constant fields | start address >> 4 (the address field cannot
                        // carry: shared memory ends below 2^18)
                        const uint32_t a_lo = (uint32_t)adesc0 | ((a_addr & 0x3FFFFu) >> 4);
                        const uint32_t b_lo = (uint32_t)bdesc0 | ((b_addr & 0x3FFFFu) >> 4);
#pragma unroll
                        for (int k = 0; k < GEMM_BK / 16; ++k) {
                            // K-major A: +16 elements of K = +32 B inside the swizzle row.
                            // MN-major B: +16 k-rows = two 8-row groups = +2048 B.
                            const uint32_t accum = (kb != seg.kb0 || k != 0); // a segment starts a fresh accumulator
                            if constexpr (NCTA == 2) {
                                umma_ss_pair_words(d_tmem, a_lo + k * 2, (uint32_t)(adesc0 >> 32), b_lo + k * 128,
                                                   (uint32_t)(bdesc0 >> 32), idesc, k == 0 ? accum : 1u);
                                if constexpr (Cfg::WIDE)   // slabs 2 and 3 -> accumulator columns 256..
                                    umma_ss_pair_words(d_tmem + 256, a_lo + k * 2, (uint32_t)(adesc0 >> 32),
                                                       b_lo + k * 128 + ((2 * Cfg::B_CHUNK_BYTES) >> 4), (uint32_t)(bdesc0 >> 32),
                                                       idesc2, k == 0 ? accum : 1u);
                            } else {
                                umma_ss(d_tmem, smem_desc_at(adesc0, a_addr + k * 32), smem_desc_at(bdesc0, b_addr + k * 2048),
                                        idesc, accum);
                            }
                        }
                        if constexpr (NCTA == 2) umma_commit_pair(&empty[s], 3); // frees the stage in both CTAs
                        else umma_commit(&empty[s]);
                    }
                    __syncwarp();
                    if (++s == Cfg::STAGES) s = 0;
                }
                if (lane == 0) {
                    if constexpr (NCTA == 2) umma_commit_pair(&tfull[acc], 3);
                    else umma_commit(&tfull[acc]);
                    GEMM_TRACE(4 + (it < 4 ? it : 3)); // all UMMAs of tile `it` issued
                }
                __syncwarp();
            }
        }
    } else if (warp == RELAY_WARP) {
        // -------------------------------------------------------------------- relay
        // Waits (bounded) for each stage's operands to land and arrives on that stage's named barrier, on
        // which the issuer warp syncs.  It can run ahead of the issuer by at most the ring depth, because
        // stage s is refilled only after the issuer's commit for it, so one barrier id per stage suffices.
        // After a wait has run out it stops waiting but keeps arriving, so the issuer is never left
        // blocked: the UMMAs then run on whatever the stages hold, the status word says the result is void.
        if (rank == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            SegIter seg;
            for (seg.init(p.total_tiles, p.num_kb, p.streamk, worker, nworkers); seg.valid(); seg.next()) {
                for (int kb = seg.kb0; kb < seg.kb1; ++kb) {
                    if (ok) {
                        bool got;
                        if constexpr (NCTA == 2) got = mbar_wait_cluster(&full[s], ph, p.d_status, KST_WAIT_FULL, abort_flag);
                        else got = mbar_wait(&full[s], ph, p.d_status, KST_WAIT_FULL, abort_flag);
                        ok = !__any_sync(0xffffffffu, !got);
                    }
                    named_bar_arrive(1 + s, 64);
                    if (++s == Cfg::STAGES) { s = 0; ph ^= 1; }
                }
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue
        // Sixteen warps, four per TMEM lane quadrant, each taking every fourth chunk of 16 columns.
        // Per chunk: tcgen05.ld -> +bias, round, activation -> a warp-private shared slab (32 rows x 16
        // columns, plain rows) -> one bulk tensor store of the 16 x 32 box, clipped at the ragged edges
        // of the output.  Each step is a short dependent chain, so the throughput comes from the four
        // warps per scheduler taking turns; warps never wait for one another.  What bounds a tile's ~4000 cycles
        // here is the SM's way out to L2, ~23 bytes per clock measured (64 KB of fp16 per CTA and tile): wider
        // chunks, two slabs per warp and stores straight from registers were each built and measured slower.
        constexpr int CH = 16;                 // columns per chunk (one tcgen05.ld.32x32b.x16)
        constexpr int NPART = EPI_WARPS / 4;   // warps sharing a lane quadrant
        constexpr int NCH = BN / NPART / CH;   // chunks one warp owns of a tile
        constexpr int RB = CH * (int)sizeof(OutT);  // staged bytes per row and chunk
        const int ew = warp - 2;               // 0..15
        const int quad = warp & 3;             // TMEM lane quadrant this warp may read
        const int part = ew >> 2;              // which chunks of the quadrant's rows
        const int row = quad * 32 + lane;      // token row inside this CTA's half of the tile
        uint8_t* wstg = reinterpret_cast<uint8_t*>(sbias) + EPI_WARPS * (BN / NPART) * 4 + ew * (32 * RB);
        float* wbias = reinterpret_cast<float*>(sbias) + ew * (BN / NPART);   // fp32 bias of this warp's own columns
        auto chunk_col = [&](int c) { return (NPART * c + part) * CH; };
        int it = 0;
        SegIter seg;
        for (seg.init(p.total_tiles, p.num_kb, p.streamk, worker, nworkers); seg.valid(); seg.next(), ++it) {
            const uint32_t tile = seg.tile;
            const TileAt at = tile_at(tile, (uint32_t)p.tiles_m, tiles_per_batch, one_plane);
            const int batch = at.batch;
            const int m0 = at.tm * (Cfg::WIDE ? p.bn : BN);
            const int n0 = at.tn * TILE_N + (int)rank * GEMM_BM;
            const int acc = Cfg::WIDE ? 0 : (int)(it & 1);
            const uint32_t aph = (uint32_t)((Cfg::WIDE ? it : it >> 1) & 1);
            // Stream-K roles of this segment: a contributor holds later k-blocks of a tile some other
            // worker finishes; a finisher holds the tile's first k-block and collects what the
            // following workers left for it.
            const bool contributor = seg.kb0 > 0;
            int ncontrib = 0;
            if (!contributor && seg.kb1 < seg.nkb) {
                const uint32_t units = p.total_tiles * (uint32_t)seg.nkb, tile_end = (tile + 1) * (uint32_t)seg.nkb;
                while (worker + 1 + (uint32_t)ncontrib < nworkers &&
                       SegIter::range_start(units, worker + 1 + (uint32_t)ncontrib, nworkers, (uint32_t)p.streamk - 1u) < tile_end)
                    ++ncontrib;
            }
            constexpr int PART_PER_WARP = (BN / NPART) * 32;             // floats one epilogue warp owns of a tile
            const int64_t my_slot = ((int64_t)worker * NCTA + rank) * EPI_WARPS + ew;
            bool sk_ok = true;
            if (ncontrib > 0) {
                // Wait (bounded) for the matching warp of every contributor; they wrote these at the
                // very start of their ranges, this segment is the last of ours.
                for (int c = 0; c < ncontrib && sk_ok; ++c) {
                    const int* f = p.sk_flag + (((int64_t)(worker + 1 + c) * NCTA + rank) * EPI_WARPS + ew);
                    unsigned long long t0 = 0;
                    uint32_t spins = 0;
                    while (ld_acquire_gpu(f) == 0) {
                        if ((++spins & 255u) == 0) {
                            const unsigned long long now = globaltimer_ns();
                            if (t0 == 0) t0 = now;
                            if (*abort_flag || now - t0 > WAIT_LIMIT_NS) {
                                atomicCAS(p.d_status, 0, KST_WAIT_STREAMK);
                                *abort_flag = 1;
                                sk_ok = false;
                                break;
                            }
                        }
                    }
                }
                sk_ok = !__any_sync(0xffffffffu, !sk_ok);
            }
            const bool collect = ncontrib > 0 && sk_ok;

            __syncwarp(); // the previous tile's readers of wbias are done
            for (int j = lane; j < BN / NPART; j += 32) {   // wbias[c*CH + t] = bias of column chunk_col(c) + t
                const int col = chunk_col(j / CH) + (j % CH);
                wbias[j] = (p.bias != nullptr && !p.bias_per_n && m0 + col < p.M) ? __half2float(p.bias[m0 + col]) : 0.f;
            }
            const bool row_bias = !contributor && p.bias != nullptr && p.bias_per_n;   // the finisher adds the bias
            const float rbias = (row_bias && n0 + row < p.N) ? __half2float(p.bias[n0 + row]) : 0.f;
            const bool got = mbar_wait(&tfull[acc], aph, p.d_status, KST_WAIT_TMEM_FULL, abort_flag);
            if (__any_sync(0xffffffffu, !got)) break; // one answer per warp
            tc_fence_after();
            if (ew == 0 && lane == 0) GEMM_TRACE(8 + (it < 4 ? it : 3)); // accumulator of tile `it` ready

            const int rows_valid = (int)(p.N - (n0 + quad * 32));   // rows of this warp's slab inside the output
            const uint32_t tacc = tmem_base + (uint32_t(quad * 32) << 16) + acc * BN;
            const int act_kind = p.epilogue;
            uint8_t* rowp = wstg + lane * RB;
            // The slab's rows are 32 B (fp16) or 64 B (fp32) apart, so lanes four (two) apart would hit the same
            // banks.  The store map swizzles at that width (16-byte chunk index ^= address bits from 7 up), which
            // spreads a warp's 16-byte stores over all banks: four wavefronts per instruction instead of eight.
            const int swz = RB == 32 ? ((lane >> 2) & 1) : ((lane >> 1) & 3);

#pragma unroll 1
            for (int c = 0; c < NCH; ++c) {
                const int col0 = chunk_col(c);
                float v[CH];
                {
                    uint32_t r[CH];
                    tmem_ld16(tacc + col0, r);
                    tmem_wait_ld();
#pragma unroll
                    for (int t = 0; t < CH; ++t) v[t] = __uint_as_float(r[t]);
                }
                if (c == NCH - 1) {
                    // This warp has read all it needs of the accumulator: hand it back (leader CTA).
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        if constexpr (NCTA == 2) mbar_arrive_cluster_cta_release(mapa_u32(smem_u32(&tempty[acc]), 0));
                        else mbar_arrive(&tempty[acc]);
                    }
                }
                if (row_bias) {
#pragma unroll
                    for (int t = 0; t < CH; ++t) v[t] += rbias;
                }
                if (contributor) {
                    // Leave the raw fp32 accumulator chunk for the finisher: [quarter q][lane] float4,
                    // so each store instruction of the warp writes 512 contiguous bytes.
                    float4* dst = reinterpret_cast<float4*>(p.sk_part + my_slot * PART_PER_WARP + (size_t)c * (CH * 32));
#pragma unroll
                    for (int q = 0; q < CH / 4; ++q)
                        dst[q * 32 + lane] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                    continue;
                }
                if (collect) {
                    for (int k = 0; k < ncontrib; ++k) {
                        const int64_t slot = ((int64_t)(worker + 1 + k) * NCTA + rank) * EPI_WARPS + ew;
                        const float4* src = reinterpret_cast<const float4*>(p.sk_part + slot * PART_PER_WARP + (size_t)c * (CH * 32));
#pragma unroll
                        for (int q = 0; q < CH / 4; ++q) {
                            const float4 f = __ldcg(src + q * 32 + lane);
                            v[4 * q] += f.x;
                            v[4 * q + 1] += f.y;
                            v[4 * q + 2] += f.z;
                            v[4 * q + 3] += f.w;
                        }
                    }
                }
                if (m0 + col0 >= p.M || rows_valid <= 0 || (Cfg::WIDE && col0 >= p.bn)) continue; // nothing to write to the output

                // the engine must have read the previous chunk out of the slab before it is overwritten; that
                // read ran under this chunk's tcgen05.ld and arithmetic
                if (lane == 0) tma_store_wait_read<0>();
                __syncwarp();
                // registers -> shared, lane = row
                const float* bc = wbias + c * CH;
                if constexpr (sizeof(OutT) == 2) {
                    auto emit = [&](auto act) {
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            const float4 b0 = *reinterpret_cast<const float4*>(bc + j * 8);
                            const float4 b1 = *reinterpret_cast<const float4*>(bc + j * 8 + 4);
                            uint4 o;
                            __half2* h = reinterpret_cast<__half2*>(&o);
                            // Round to fp16 first; the activation sees the rounded value.
                            h[0] = act(__floats2half2_rn(v[j * 8 + 0] + b0.x, v[j * 8 + 1] + b0.y));
                            h[1] = act(__floats2half2_rn(v[j * 8 + 2] + b0.z, v[j * 8 + 3] + b0.w));
                            h[2] = act(__floats2half2_rn(v[j * 8 + 4] + b1.x, v[j * 8 + 5] + b1.y));
                            h[3] = act(__floats2half2_rn(v[j * 8 + 6] + b1.z, v[j * 8 + 7] + b1.w));
                            *reinterpret_cast<uint4*>(rowp + ((j ^ swz) << 4)) = o;
                        }
                    };
                    switch (act_kind) {
                        case B200_EPI_RELU: emit([](__half2 t) { return __hmax2(t, __float2half2_rn(0.f)); }); break;
                        case B200_EPI_GELU:
                            emit([](__half2 t) {
                                const float2 g = gelu_exact2(__half22float2(t));
                                return __floats2half2_rn(g.x, g.y);
                            });
                            break;
                        case B200_EPI_GELU_TANH:
                            emit([](__half2 t) {
                                const float2 f = __half22float2(t);
                                return __floats2half2_rn(apply_act(B200_EPI_GELU_TANH, f.x), apply_act(B200_EPI_GELU_TANH, f.y));
                            });
                            break;
                        default: emit([](__half2 t) { return t; }); break;
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float4 b = *reinterpret_cast<const float4*>(bc + j * 4);
                        float4 o;
                        o.x = apply_act(act_kind, v[j * 4 + 0] + b.x);
                        o.y = apply_act(act_kind, v[j * 4 + 1] + b.y);
                        o.z = apply_act(act_kind, v[j * 4 + 2] + b.z);
                        o.w = apply_act(act_kind, v[j * 4 + 3] + b.w);
                        *reinterpret_cast<float4*>(rowp + ((j ^ swz) << 4)) = o;
                    }
                }
                // shared -> global by the bulk-store engine: one instruction for the 16 x 32 box (the engine undoes
                // the slab's swizzle), clipped at the ragged edges of the output.
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    tma_store_3d(&tmapO, wstg, m0 + col0, n0 + quad * 32, batch);
                    tma_store_commit();
                }
            }
            if (contributor) {
                __threadfence();
                __syncwarp();
                if (lane == 0) st_release_gpu(p.sk_flag + my_slot, 1);
            } else if (ncontrib > 0) {
                __syncwarp();
                if (lane == 0)   // consumed: the flags are zero again for the next launch
                    for (int c = 0; c < ncontrib; ++c)
                        p.sk_flag[((int64_t)(worker + 1 + c) * NCTA + rank) * EPI_WARPS + ew] = 0;
            }
            if (ew == 0 && lane == 0) GEMM_TRACE(12 + (it < 4 ? it : 3)); // epilogue of tile `it` done
        }
        // The CTA may leave once the engine has read the slab; the writes themselves complete with the grid.
        if (lane == 0) tma_store_wait_read<0>();
    }

    // Teardown: every role arrives here whether it finished or gave up.
    if (*abort_flag) {
        // Let any TMA copy still in flight into this CTA's shared memory land before exit.
        for (int i = 0; i < 4; ++i) __nanosleep(1000000);
    }
    tc_fence_before();
    if constexpr (NCTA == 2) cluster_sync_all(); // neither CTA leaves while its peer may still signal it
    else __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        if constexpr (NCTA == 2) tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
        else tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
    if (threadIdx.x == 0) GEMM_TRACE(16); // exit
    if (threadIdx.x == 0 && rank == 0 && p.trace != nullptr && worker < 120)
        p.trace[128 + worker] = globaltimer_ns();   // when each worker left, to see how evenly the work was dealt
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

struct TilePick {
    int bn;      // feature columns per tile
    int ncta;    // 1: 128-token tiles, one CTA each; 2: 256-token tiles, one CTA pair each
    int streamk; // 1: equal k-block ranges per worker instead of whole tiles
    int width;   // bn == 512 (the wide tile): feature columns per tile, a multiple of 16 in (256, 512]
};

// Tile planner.  Candidates are (BN, NCTA, whole-tile | stream-K); the estimate for each is
//   whole tiles: waves x (k-blocks x t_kb + t_tile)      stream-K: (tiles x k-blocks / workers) x t_kb + t_tile + t_fix
// with t_kb the time one worker takes per k-block when the whole GPU is pulling operands through
// L2 (measured on B200: it is the L2 -> SM traffic per k-block that sets it, ~83 GB/s per SM), t_tile
// the part of a tile's epilogue nothing hides, and t_fix the stream-K partial hand-off.
// Workers a stream-K launch uses so that no tile is cut more than once (0: not applicable).
static int64_t streamk_workers(int64_t tiles, int64_t workers_max) {
    if (tiles >= workers_max) return workers_max;
    if (2 * tiles <= workers_max) return 2 * tiles;
    return 0;
}

static TilePick pick_tile(int64_t M, int64_t N, int64_t K, int64_t nbatch, int sms, bool allow_streamk = true,
                          int epilogue = B200_EPI_NONE) {
    if (const char* f = getenv("B200_GEMM_TILE")) { // debugging aid: "<bn>x<ncta>[s]", e.g. 256x2 or 256x2s
        int bn = 0, nc = 0;
        char sk = 0;
        const int got = sscanf(f, "%dx%d%c", &bn, &nc, &sk);
        if (got >= 2 && (bn == 256 || bn == 128 || (bn == 64 && nc == 1)) && (nc == 1 || nc == 2))
            return {bn, nc, allow_streamk && got == 3 && sk == 's', 0};
        if (got >= 2 && bn > 256 && bn <= 512 && bn % 16 == 0 && nc == 2) return {512, 2, 0, bn};   // "<width>x2": the wide tile
    }
    struct Cand { int bn, ncta; double t_kb; };
    const Cand cands[5] = {{256, 2, 0.39}, {128, 2, 0.38}, {256, 1, 0.50}, {128, 1, 0.38}, {64, 1, 0.32}};
    const int64_t nkb = cdiv(K, GEMM_BK);
    const double t_tile = 2.0, t_fix = 8.0;  // measured: partial dump + fence + flag + read-back
    TilePick best{256, 1, 0, 0};
    double best_cost = 1e300;
    for (const Cand& c : cands) {   // whole-tile schedules first: stream-K has to beat the best of them clearly
        const int64_t tiles = cdiv(M, c.bn) * cdiv(N, (int64_t)GEMM_BM * c.ncta) * nbatch;
        const int64_t waves = cdiv(tiles, (int64_t)(sms / c.ncta));
        const double dp = (double)waves * ((double)nkb * c.t_kb + t_tile);
        if (dp < best_cost - 1e-9) {
            best_cost = dp;
            best = {c.bn, c.ncta, 0, 0};
        }
    }
    {
        // The wide tile: when 256-wide pair tiles need more than one round of the workers, a width in
        // (256, 512] that makes every tile some worker's only one.  Measured on B200 (1500 tokens, K = 1280,
        // microseconds): 7 + k-blocks x 0.3 x width/256 (two UMMAs per K step; never below 1.25 tile-widths,
        // where issuing them is what takes the time) + 0.25 per 64 columns of epilogue, none of which anything
        // hides (0.85 with GELU).  It has to beat the whole-tile estimate by a margin to be taken.
        const int64_t workers = sms / 2;
        const int64_t token_tiles = cdiv(N, (int64_t)GEMM_BM * 2) * nbatch;
        const int64_t fm = workers / token_tiles;   // feature tiles a single round has room for
        if (fm >= 1 && cdiv(M, 256) * token_tiles > workers) {
            const int64_t width = cdiv(cdiv(M, fm), 16) * 16;
            if (width > 256 && width <= 512) {
                const double rel = (double)width / 256.0;
                const bool gelu = epilogue == B200_EPI_GELU || epilogue == B200_EPI_GELU_TANH;
                const double wide = 7.0 + (double)nkb * 0.3 * (rel < 1.25 ? 1.25 : rel) + (gelu ? 0.85 : 0.25) * (double)width / 64.0;
                if (wide < 0.92 * best_cost) {
                    best_cost = wide;
                    best = {512, 2, 0, (int)width};
                }
            }
        }
    }
    best_cost *= 0.85;
    if (!allow_streamk) return best;
    for (const Cand& c : cands) {
        const int64_t tiles = cdiv(M, c.bn) * cdiv(N, (int64_t)GEMM_BM * c.ncta) * nbatch;
        const int64_t workers = sms / c.ncta;
        const int64_t waves = cdiv(tiles, workers);
        // Stream-K pays when the whole-tile schedule leaves a wave mostly empty.  Only splits
        // that cut a tile at most once are considered (one contributor per finisher keeps the
        // hand-off short): all workers when there is at least a tile each, else two per tile.
        const int64_t skw = streamk_workers(tiles, workers);
        if (skw > 0 && tiles % workers != 0 && waves <= 3 && nkb >= 8) {
            const double sk = (double)(tiles * nkb) / (double)skw * c.t_kb + t_tile + t_fix;
            if (sk < best_cost - 1e-9) {
                best_cost = sk;
                best = {c.bn, c.ncta, 1, 0};
            }
        }
    }
    return best;
}

template <int BN, typename OutT, int NCTA>
static int launch_tc(b200_ctx* ctx, int64_t M, int64_t N, int64_t K, const void* A, int64_t lda,
                     const void* B, int64_t ldb, const void* bias, int bias_per_n, void* out, int64_t ldo,
                     int epi, int64_t nbatch, int64_t sA, int64_t sB, int64_t sO, int streamk, int width) {
    using Cfg = GemmCfg<BN, OutT, NCTA>;
    if (Cfg::WIDE) {
        B200_REQUIRE(width > 256 && width <= 512 && width % 16 == 0, B200_EINVAL, "gemm: wide tile of %d columns", width);
        streamk = 0;
    }
    static bool attr_done[16] = {};
    auto kern = gemm_f16_tc_kernel<BN, OutT, NCTA>;
    if (!attr_done[ctx->device & 15]) {
        B200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
        attr_done[ctx->device & 15] = true;
    }
    CUtensorMap tX, tW;
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
    CUtensorMap tO;
    {
        const uint64_t osz = sizeof(OutT);
        uint64_t dims[3] = {(uint64_t)M, (uint64_t)N, (uint64_t)nbatch};
        uint64_t str[2] = {(uint64_t)ldo * osz, (uint64_t)(nbatch > 1 ? sO : ldo * N) * osz};
        uint32_t box[3] = {16, 32, 1};
        int rc = make_tmap(ctx, &tO, sizeof(OutT) == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, out,
                           dims, str, box, sizeof(OutT) == 2 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_64B);
        if (rc) return rc;
    }
    GemmParams<OutT> p;
    p.M = M; p.N = N; p.K = K;
    p.out = static_cast<OutT*>(out);
    p.ldo = ldo;
    p.strideO = nbatch > 1 ? sO : 0;
    p.bn = Cfg::WIDE ? width : BN;
    p.tiles_m = (int)cdiv(M, p.bn);
    p.tiles_n = (int)cdiv(N, (int64_t)GEMM_BM * NCTA);
    p.num_kb = (int)cdiv(K, GEMM_BK);
    {
        const int64_t tiles = (int64_t)p.tiles_m * p.tiles_n * nbatch;
        B200_REQUIRE(tiles * p.num_kb < ((int64_t)1 << 31), B200_EINVAL,
                     "gemm: %lld tiles of %d k-blocks are more than one launch indexes", (long long)tiles, p.num_kb);
        p.total_tiles = (uint32_t)tiles;
    }
    p.bias = static_cast<const __half*>(bias);
    p.bias_per_n = bias_per_n;
    p.epilogue = epi;
    p.d_status = ctx->d_status;
    p.trace = ctx->gemm_trace;
    // Persistent workers: as many CTAs (or CTA pairs) as can be resident at once.  Pairs must sit
    // in one GPC, so fewer than SMs/2 may fit; ask the runtime once per device.
    static int resident[16] = {};
    int64_t workers_max = ctx->prop.multiProcessorCount / NCTA;
    if (NCTA == 2) {
        if (!resident[ctx->device & 15]) {
            int n = 0;
            cudaLaunchConfig_t cfg = {};
            cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
            cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
            cfg.stream = ctx->stream;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = NCTA;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            cfg.gridDim = dim3((unsigned)(workers_max * NCTA), 1, 1);
            cudaError_t e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
            if (e != cudaSuccess || n <= 0) {
                cudaGetLastError();
                n = (int)workers_max;
            }
            resident[ctx->device & 15] = n;
        }
        if (resident[ctx->device & 15] < workers_max) workers_max = resident[ctx->device & 15];
    }
    int workers = (int)((int64_t)p.total_tiles < workers_max ? (int64_t)p.total_tiles : workers_max);
    p.streamk = 0;
    p.sk_part = nullptr;
    p.sk_flag = ctx->sk_flags;
    const int64_t skw = streamk_workers(p.total_tiles, workers_max);
    if (streamk && skw > 0 && p.num_kb >= 2 && ctx->sk_flags != nullptr) {
        // Every worker gets the same number of k-blocks; partial tiles meet in a workspace block
        // of one fp32 tile per (worker, CTA rank).
        workers = (int)skw;
        void* part = nullptr;
        int rc = ws_scratch(ctx, (size_t)workers * NCTA * GEMM_BM * BN * sizeof(float), &part);
        if (rc) return rc;
        // Two workers per tile: the second one's share is shortened, so that its partial is on its way while the
        // first still multiplies.  Measured on 1280 x 1500 x 5120 (30 tiles of 80 k-blocks): 25.1 us with equal
        // shares, 24.1 / 23.3 / 23.6 / 24.2 / 25.2 with 4 / 8 / 10 / 12 / 16 k-blocks moved.
        int lean = 0;
        if (skw == 2 * (int64_t)p.total_tiles) lean = p.num_kb / 8 < 8 ? p.num_kb / 8 : 8;
        p.streamk = 1 + lean;
        p.sk_part = static_cast<float*>(part);
    }
    B200_CUDA(launch_dep(kern, dim3((unsigned)(workers * NCTA), 1, 1), dim3(GEMM_THREADS, 1, 1), Cfg::SMEM_BYTES,
                         ctx->stream, NCTA, tX, tW, tO, p));
    ctx->launches++;
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
    const TilePick t = pick_tile(M, N, K, nbatch, sms);
    const int bn = t.bn == 512 ? t.width : t.bn;
    plan->block_m = GEMM_BM * t.ncta;
    plan->block_n = bn;
    plan->block_k = GEMM_BK;
    if (t.bn == 512) {
        plan->stages = GemmCfg<512, __half, 2>::STAGES;
        plan->smem_bytes = GemmCfg<512, __half, 2>::SMEM_BYTES;
    } else if (t.ncta == 2) {
        plan->stages = bn == 256 ? GemmCfg<256, __half, 2>::STAGES : GemmCfg<128, __half, 2>::STAGES;
        plan->smem_bytes = bn == 256 ? GemmCfg<256, __half, 2>::SMEM_BYTES : GemmCfg<128, __half, 2>::SMEM_BYTES;
    } else {
        plan->stages = bn == 256 ? GemmCfg<256, __half, 1>::STAGES
                                 : (bn == 128 ? GemmCfg<128, __half, 1>::STAGES : GemmCfg<64, __half, 1>::STAGES);
        plan->smem_bytes = bn == 256 ? GemmCfg<256, __half, 1>::SMEM_BYTES
                                     : (bn == 128 ? GemmCfg<128, __half, 1>::SMEM_BYTES
                                                  : GemmCfg<64, __half, 1>::SMEM_BYTES);
    }
    plan->tiles_m = (int)cdiv(M, bn);
    plan->tiles_n = (int)cdiv(N, (int64_t)GEMM_BM * t.ncta);
    const int64_t tiles = (int64_t)plan->tiles_m * plan->tiles_n * nbatch;
    const int64_t workers = sms / t.ncta;
    plan->ctas = (int)((tiles < workers ? tiles : workers) * t.ncta);
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
                 int epilogue, int64_t nbatch, int64_t strideA, int64_t strideB, int64_t strideO, int use_workspace) {
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
    const TilePick t = pick_tile(M, N, K, nbatch, ctx->prop.multiProcessorCount, use_workspace != 0, epilogue);
#define GEMM_GO(BN_, T_, NC_)                                                                                     \
    return launch_tc<BN_, T_, NC_>(ctx, M, N, K, A, lda, B, ldb, bias, bias_per_n, out, ldo, epilogue, nbatch, strideA, \
                                   strideB, strideO, t.streamk, t.width)
    if (out_dtype == B200_F16) {
        if (t.bn == 512) GEMM_GO(512, __half, 2);
        if (t.ncta == 2 && t.bn == 256) GEMM_GO(256, __half, 2);
        if (t.ncta == 2) GEMM_GO(128, __half, 2);
        if (t.bn == 256) GEMM_GO(256, __half, 1);
        if (t.bn == 128) GEMM_GO(128, __half, 1);
        GEMM_GO(64, __half, 1);
    } else {
        if (t.bn == 512) GEMM_GO(512, float, 2);
        if (t.ncta == 2 && t.bn == 256) GEMM_GO(256, float, 2);
        if (t.ncta == 2) GEMM_GO(128, float, 2);
        if (t.bn == 256) GEMM_GO(256, float, 1);
        if (t.bn == 128) GEMM_GO(128, float, 1);
        GEMM_GO(64, float, 1);
    }
#undef GEMM_GO
}

} // namespace b200
