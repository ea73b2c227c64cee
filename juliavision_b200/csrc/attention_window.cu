// Attention over many short key sequences (windows of at most 64 keys, e.g. the 8x8-token windows of a
// hierarchical image encoder's first stages): out = softmax(scale * Q K^T) V per (window, head), the same
// arithmetic as attention_f16_tc_kernel (fp32 scores and softmax, P rounded to fp16 for the second
// product, fp32 accumulation, reference kernels/extern/flash.jl:459-1036 for the fused form).
//
// At this size the work per window is a megaflop and the operation is bound by HBM and by latency, not by
// the tensor pipe: the 128-row TMEM tiles of the large kernel are mostly empty and its per-CTA set-up
// (TMEM allocation, barriers, tensor maps) costs more than the window's arithmetic, with one CTA resident
// per SM.  So this kernel is small instead: one CTA of four warps per 64 queries of one (window, head),
// 27 KB of shared memory so that eight or more are resident per SM, operands fetched with plain 16-byte
// loads (twelve in flight per thread), and each warp's 16 x 64 scores and 16 x 64 output held in registers
// as warp-level m16n8k16 tiles.
#include <cuda_fp16.h>

#include "internal.h"
#include "ptx.cuh"

namespace b200 {

constexpr int AW_THREADS = 128;
constexpr int AW_BQ = 64;      // queries per CTA (16 per warp)
constexpr int AW_LK = 64;      // keys per window at most
constexpr int AW_PITCH = 72;   // halves per shared row: 144 bytes, rows 4 banks apart, conflict-free fragments

struct WinParams {
    const __half *q, *k, *v;
    void* out;
    int64_t qsL, qsH, qsB, ksL, ksH, ksB, vsL, vsH, vsB, osL, osH, osB;
    int E, Lq, Lk, H, B, qtiles, out_f32;
    float scale_log2;
};

__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const __half* row) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(row);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// rows [0, rows) x E halves of a strided (E, L) slice into a zero-padded [64][AW_PITCH] shared tile
__device__ __forceinline__ void win_fetch(uint4 (&r)[4], const __half* base, int64_t sL, int rows, int E, int tid) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int idx = tid + i * AW_THREADS;          // 512 vectors: 64 rows x 8
        const int row = idx >> 3, vec = idx & 7;
        r[i] = make_uint4(0u, 0u, 0u, 0u);
        if (row < rows && vec * 8 < E) r[i] = __ldg(reinterpret_cast<const uint4*>(base + (int64_t)row * sL) + vec);
    }
}

__device__ __forceinline__ void win_put(__half* tile, const uint4 (&r)[4], int tid) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int idx = tid + i * AW_THREADS;
        *reinterpret_cast<uint4*>(tile + (idx >> 3) * AW_PITCH + (idx & 7) * 8) = r[i];
    }
}

__global__ void __launch_bounds__(AW_THREADS, 6) attention_window_kernel(const WinParams p) {
    __shared__ __align__(16) __half Qs[AW_BQ * AW_PITCH];
    __shared__ __align__(16) __half Ks[AW_LK * AW_PITCH];
    __shared__ __align__(16) __half Vs[AW_LK * AW_PITCH];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    int64_t u = blockIdx.x;
    const int qt = (int)(u % p.qtiles);
    u /= p.qtiles;
    const int h = (int)(u % p.H);
    const int b = (int)(u / p.H);
    const int q0 = qt * AW_BQ;
    const int qrows = min(AW_BQ, p.Lq - q0);

    grid_dep_wait();
    {
        uint4 rq[4], rk[4], rv[4];
        win_fetch(rq, p.q + (int64_t)q0 * p.qsL + (int64_t)h * p.qsH + (int64_t)b * p.qsB, p.qsL, qrows, p.E, tid);
        win_fetch(rk, p.k + (int64_t)h * p.ksH + (int64_t)b * p.ksB, p.ksL, p.Lk, p.E, tid);
        win_fetch(rv, p.v + (int64_t)h * p.vsH + (int64_t)b * p.vsB, p.vsL, p.Lk, p.E, tid);
        win_put(Qs, rq, tid);
        win_put(Ks, rk, tid);
        win_put(Vs, rv, tid);
    }
    __syncthreads();
    grid_dep_launch();
    const int r0 = warp * 16;
    if (r0 >= qrows) return;

    // S = Q K^T: 16 queries x 64 keys as eight n-tiles of 8 keys, four k-steps of 16 along E
    // Fragments come out of the row-major tiles with ldmatrix: four 8 x 8 blocks per instruction.
    uint32_t qa[4][4];
#pragma unroll
    for (int ks = 0; ks < 4; ++ks)      // blocks (rows 0-7 | 8-15) x (dims 16ks.. | 16ks+8..) of the warp's queries
        ldmatrix_x4(qa[ks], Qs + (r0 + (lane & 7) + ((lane >> 3) & 1) * 8) * AW_PITCH + ks * 16 + (lane >> 4) * 8);
    float s[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
    for (int nt = 0; nt < 8; nt += 2) {
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            uint32_t kb[4];             // blocks (keys 8nt.. | 8nt+8..) x (dims 16ks.. | 16ks+8..)
            ldmatrix_x4(kb, Ks + ((nt + (lane >> 4)) * 8 + (lane & 7)) * AW_PITCH + ks * 16 + ((lane >> 3) & 1) * 8);
            mma_16816(s[nt], qa[ks], kb[0], kb[1]);
            mma_16816(s[nt + 1], qa[ks], kb[2], kb[3]);
        }
    }
    // softmax over the keys of rows g (values 0,1) and g + 8 (values 2,3); a quad of lanes shares a row
    float m0 = -INFINITY, m1 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int key = nt * 8 + 2 * t + (c & 1);
            s[nt][c] = key < p.Lk ? s[nt][c] * p.scale_log2 : -INFINITY;
        }
        m0 = fmaxf(m0, fmaxf(s[nt][0], s[nt][1]));
        m1 = fmaxf(m1, fmaxf(s[nt][2], s[nt][3]));
    }
    m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, 1));
    m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, 2));
    m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, 1));
    m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, 2));
    if (m0 == -INFINITY) m0 = 0.f;
    if (m1 == -INFINITY) m1 = 0.f;
    float l0 = 0.f, l1 = 0.f;
    uint32_t pa[4][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
        // the row sum is taken over the fp16-rounded probabilities the second product uses
        const __half2 lo = __floats2half2_rn(exp2f(s[nt][0] - m0), exp2f(s[nt][1] - m0));
        const __half2 hi = __floats2half2_rn(exp2f(s[nt][2] - m1), exp2f(s[nt][3] - m1));
        const float2 flo = __half22float2(lo), fhi = __half22float2(hi);
        l0 += flo.x + flo.y;
        l1 += fhi.x + fhi.y;
        pa[nt >> 1][(nt & 1) * 2 + 0] = *reinterpret_cast<const uint32_t*>(&lo);
        pa[nt >> 1][(nt & 1) * 2 + 1] = *reinterpret_cast<const uint32_t*>(&hi);
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

    // O = P V: 16 queries x 64 dims as eight n-tiles of 8 dims, four k-steps of 16 keys; V's fragments
    // come transposed out of its row-major tile
    float o[8][4];
#pragma unroll
    for (int ne = 0; ne < 8; ++ne) o[ne][0] = o[ne][1] = o[ne][2] = o[ne][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
        for (int ne = 0; ne < 8; ne += 2) {
            uint32_t b0, b1, b2, b3;
            const __half* vrow = Vs + (kk * 16 + (lane & 15)) * AW_PITCH + (ne + (lane >> 4)) * 8;
            const uint32_t addr = (uint32_t)__cvta_generic_to_shared(vrow);
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                         : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3)
                         : "r"(addr));
            mma_16816(o[ne], pa[kk], b0, b1);
            mma_16816(o[ne + 1], pa[kk], b2, b3);
        }
    }
    const float i0 = 1.f / l0, i1 = 1.f / l1;
    const int64_t obase = (int64_t)h * p.osH + (int64_t)b * p.osB;
    if (p.out_f32) {
        float* out = static_cast<float*>(p.out) + obase;
#pragma unroll
        for (int ne = 0; ne < 8; ++ne) {
            const int e = ne * 8 + 2 * t;
            if (e >= p.E) continue;
            if (r0 + g < qrows)
                *reinterpret_cast<float2*>(out + (int64_t)(q0 + r0 + g) * p.osL + e) = make_float2(o[ne][0] * i0, o[ne][1] * i0);
            if (r0 + g + 8 < qrows)
                *reinterpret_cast<float2*>(out + (int64_t)(q0 + r0 + g + 8) * p.osL + e) = make_float2(o[ne][2] * i1, o[ne][3] * i1);
        }
        return;
    }
    // fp16: through the warp's own 16 rows of the Q tile (its fragments are in registers by now), so that
    // a row leaves as whole 16-byte vectors
    __syncwarp();
#pragma unroll
    for (int ne = 0; ne < 8; ++ne) {
        __half* d = Qs + (r0 + g) * AW_PITCH + ne * 8 + 2 * t;
        *reinterpret_cast<uint32_t*>(d) = pack_h2(o[ne][0] * i0, o[ne][1] * i0);
        *reinterpret_cast<uint32_t*>(d + 8 * AW_PITCH) = pack_h2(o[ne][2] * i1, o[ne][3] * i1);
    }
    __syncwarp();
    __half* out = static_cast<__half*>(p.out) + obase;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int idx = lane + i * 32;                  // 128 vectors: 16 rows x 8
        const int row = idx >> 3, vec = idx & 7;
        if (r0 + row < qrows && vec * 8 < p.E)
            *reinterpret_cast<uint4*>(out + (int64_t)(q0 + r0 + row) * p.osL + vec * 8) =
                *reinterpret_cast<const uint4*>(Qs + (r0 + row) * AW_PITCH + vec * 8);
    }
}

int attention_window_launch(b200_ctx* ctx, int64_t E, int64_t Lq, int64_t Lk, int64_t H, int64_t B, const b200_strided4* q,
                            const b200_strided4* k, const b200_strided4* v, const b200_strided4* o, int out_dtype,
                            float scale) {
    WinParams p;
    p.q = static_cast<const __half*>(q->ptr);
    p.k = static_cast<const __half*>(k->ptr);
    p.v = static_cast<const __half*>(v->ptr);
    p.out = const_cast<void*>(o->ptr);
    p.qsL = q->stride[1]; p.qsH = q->stride[2]; p.qsB = q->stride[3];
    p.ksL = k->stride[1]; p.ksH = k->stride[2]; p.ksB = k->stride[3];
    p.vsL = v->stride[1]; p.vsH = v->stride[2]; p.vsB = v->stride[3];
    p.osL = o->stride[1]; p.osH = o->stride[2]; p.osB = o->stride[3];
    p.E = (int)E; p.Lq = (int)Lq; p.Lk = (int)Lk; p.H = (int)H; p.B = (int)B;
    p.qtiles = (int)cdiv(Lq, AW_BQ);
    p.out_f32 = out_dtype == B200_F32;
    p.scale_log2 = scale * 1.4426950408889634f;
    const int64_t ctas = (int64_t)p.qtiles * H * B;
    B200_REQUIRE(ctas < (1ll << 31), B200_DECLINE_EXTENT, "attention: too many windows");
    B200_CUDA(launch_dep(attention_window_kernel, dim3((unsigned)ctas, 1, 1), dim3(AW_THREADS, 1, 1), 0, ctx->stream, 1, p));
    ctx->launches++;
    return B200_OK;
}

} // namespace b200
