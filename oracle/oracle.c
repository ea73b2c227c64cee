/*
 * CPU oracle for the DNNKernels dense hot path.
 *
 * TEST INFRASTRUCTURE, NOT PRODUCT.  This file is a plain-C restatement of the
 * reference's CPU-capable forms of each op.  Only the test-suite, the smoke
 * check and the benchmark's cpu-baseline / reference arm may load it; the
 * product library never links, loads or calls it.
 *
 * The reference is Julia on KernelAbstractions and cannot be executed where this
 * is built (no Julia toolchain, and its Lava/Mantle dependencies are not in the
 * tree), and its tests draw unseeded random inputs, so no golden byte vectors
 * exist: PARITY UNPINNED at the byte level.  What pins this file is the set of
 * known-answer assertions the reference's own tests make (tolerances, special
 * values, bit-equalities), re-asserted in tests/test_oracle_pins.py, and an
 * independent float64 numpy restatement committed under tests/golden/.
 *
 * Layout convention (the reference's): column-major arrays whose shape is the
 * reverse of the torch shape.  fp16 values are passed as uint16_t bit patterns.
 *
 * Each function cites the reference file:line it follows (paths relative to the
 * reference project root, DNNKernels/src/...).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

typedef uint16_t f16bits;

static inline float h2f(f16bits h) {
    _Float16 x;
    memcpy(&x, &h, 2);
    return (float)x;
}
static inline f16bits f2h(float f) {
    _Float16 x = (_Float16)f; /* round-to-nearest-even */
    f16bits h;
    memcpy(&h, &x, 2);
    return h;
}

enum { ORA_F16 = 0, ORA_F32 = 1 };
enum { ORA_EPI_NONE = 0, ORA_EPI_RELU = 1, ORA_EPI_GELU = 2, ORA_EPI_GELU_TANH = 3 };

int ora_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Thread count of the parallel loops below, overriding an inherited OMP_NUM_THREADS (launchers
 * that start one process per GPU export OMP_NUM_THREADS=1).  Returns the count now in force. */
int ora_set_num_threads(int n) {
#ifdef _OPENMP
    if (n >= 1) omp_set_num_threads(n);
    return omp_get_max_threads();
#else
    (void)n;
    return 1;
#endif
}

/* ------------------------------------------------------------------ activations */

/* ops.jl:161-169 — Abramowitz & Stegun 7.1.26, evaluated in fp32 for half input. */
float ora_erf_f32(float x) {
    float a = fabsf(x);
    float t = 1.0f / (1.0f + 0.3275911f * a);
    float y = 1.0f - (((((1.061405429f * t - 1.453152027f) * t) + 1.421413741f) * t -
                       0.284496736f) * t + 0.254829592f) * t * expf(-a * a);
    return x < 0.0f ? -y : y;
}

/* ops.jl:1665-1670 — exact gelu, fp32 evaluation, one rounding at the store. */
float ora_gelu_exact_f32(float x) {
    return 0.5f * x * (1.0f + ora_erf_f32(x / sqrtf(2.0f)));
}

/* ops.jl:1678-1683 — tanh-approximated gelu, fp32 evaluation. */
float ora_gelu_tanh_f32(float x) {
    const float c = 0.7978845608028654f;
    return 0.5f * x * (1.0f + tanhf(c * (x + 0.044715f * x * x * x)));
}

static inline float apply_epi(int epi, float v) {
    switch (epi) {
        case ORA_EPI_RELU: return v > 0.0f ? v : 0.0f;           /* ops.jl:1684 */
        case ORA_EPI_GELU: return ora_gelu_exact_f32(v);
        case ORA_EPI_GELU_TANH: return ora_gelu_tanh_f32(v);
        default: return v;
    }
}

/* Elementwise forms over fp16 storage (value -> fp32 -> f -> fp16). */
void ora_erf_f16(const f16bits* x, f16bits* y, int64_t n) {
    for (int64_t i = 0; i < n; ++i) y[i] = f2h(ora_erf_f32(h2f(x[i])));
}
void ora_act_f16(const f16bits* x, f16bits* y, int64_t n, int epi) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) y[i] = f2h(apply_epi(epi, h2f(x[i])));
}

/* ------------------------------------------------------------------------ GEMM */

/*
 * matmul.jl:17-28 (mm2) + matmul.jl:140-148 / 210-214 (epilogue on the converted
 * value).  out[i,j] = epi(T(bias[i] + sum_k A[i,k] B[k,j])), column-major,
 * A (M,K) ld=lda, B (K,N) ld=ldb, out (M,N) ld=ldo; fp32 fma chain in ascending k
 * starting from the bias.
 */
void ora_gemm_f16(int64_t M, int64_t N, int64_t K, const f16bits* A, int64_t lda,
                  const f16bits* B, int64_t ldb, const f16bits* bias, void* out,
                  int64_t ldo, int out_dtype, int epi) {
#pragma omp parallel
    {
        float* acc = (float*)malloc(sizeof(float) * (size_t)M);
#pragma omp for schedule(static)
        for (int64_t j = 0; j < N; ++j) {
            for (int64_t i = 0; i < M; ++i) acc[i] = bias ? h2f(bias[i]) : 0.0f;
            /* Row-sweep order keeps every element's chain in ascending k. */
            for (int64_t k = 0; k < K; ++k) {
                float b = h2f(B[k + ldb * j]);
                const f16bits* a = A + lda * k;
                for (int64_t i = 0; i < M; ++i) acc[i] = fmaf(h2f(a[i]), b, acc[i]);
            }
            if (out_dtype == ORA_F16) {
                f16bits* o = (f16bits*)out + ldo * j;
                for (int64_t i = 0; i < M; ++i) {
                    float v = h2f(f2h(acc[i]));
                    o[i] = f2h(apply_epi(epi, v));
                }
            } else {
                float* o = (float*)out + ldo * j;
                for (int64_t i = 0; i < M; ++i) o[i] = apply_epi(epi, acc[i]);
            }
        }
        free(acc);
    }
}

/* matmul.jl:30-39 (mm3): batched, no bias, planes strided by sA/sB/sO elements. */
void ora_bmm_f16(int64_t M, int64_t N, int64_t K, int64_t nb, const f16bits* A,
                 int64_t lda, int64_t sA, const f16bits* B, int64_t ldb, int64_t sB,
                 void* out, int64_t ldo, int64_t sO, int out_dtype) {
    for (int64_t b = 0; b < nb; ++b) {
        void* o = out_dtype == ORA_F16 ? (void*)((f16bits*)out + sO * b)
                                       : (void*)((float*)out + sO * b);
        ora_gemm_f16(M, N, K, A + sA * b, lda, B + sB * b, ldb, NULL, o, ldo, out_dtype,
                     ORA_EPI_NONE);
    }
}

/* float64 truth over the same fp16 operands (test_batchedmatmul.jl:43-52 ref3). */
void ora_gemm_f64(int64_t M, int64_t N, int64_t K, const f16bits* A, int64_t lda,
                  const f16bits* B, int64_t ldb, const f16bits* bias, double* out,
                  int64_t ldo) {
#pragma omp parallel for schedule(static)
    for (int64_t j = 0; j < N; ++j)
        for (int64_t i = 0; i < M; ++i) {
            double acc = bias ? (double)h2f(bias[i]) : 0.0;
            for (int64_t k = 0; k < K; ++k)
                acc += (double)h2f(A[i + lda * k]) * (double)h2f(B[k + ldb * j]);
            out[i + ldo * j] = acc;
        }
}

/* ------------------------------------------------------------------- attention */

/*
 * The runtime's unfused path: attention.jl:790-834 (sdpa!(::Decline)) with bodies
 * attn_scores (:46-61), attn_softmax (:73-100) and attn_apply (:102-112).
 * q,k,v are (E,L,H,B) with element strides s[0..3] (s[0] is the E stride);
 * scores are stored in the operands' dtype (fp16) between passes, the exponent is
 * stored as fp16 while the row sum adds the unrounded fp32 value, and the divide
 * happens in the apply pass.  out is dense (E,Lq,H,B).  bias (may be NULL) is the additive
 * mask of the mem-efficient variant, added to the scaled fp32 score before it is stored.
 */
void ora_attention_threepass(int64_t E, int64_t Lq, int64_t Lk, int64_t H, int64_t B,
                             const f16bits* q, const int64_t* qs, const f16bits* k,
                             const int64_t* ks, const f16bits* v, const int64_t* vs,
                             void* out, int out_dtype, float scale, const f16bits* bias,
                             const int64_t* bs) {
#pragma omp parallel
    {
        f16bits* row = (f16bits*)malloc(sizeof(f16bits) * (size_t)Lk);
        float* acc = (float*)malloc(sizeof(float) * (size_t)E);
#pragma omp for collapse(3) schedule(static)
        for (int64_t b = 0; b < B; ++b)
            for (int64_t h = 0; h < H; ++h)
                for (int64_t lq = 0; lq < Lq; ++lq) {
                    const f16bits* qp = q + qs[1] * lq + qs[2] * h + qs[3] * b;
                    float m = -INFINITY;
                    for (int64_t lk = 0; lk < Lk; ++lk) {
                        const f16bits* kp = k + ks[1] * lk + ks[2] * h + ks[3] * b;
                        float a = 0.0f;
                        for (int64_t e = 0; e < E; ++e)
                            a = fmaf(h2f(qp[qs[0] * e]), h2f(kp[ks[0] * e]), a);
                        a *= scale;
                        /* additive mask in the graph's own (Lk,Lq,H,B) order, size-1 axes
                         * broadcast (stride 0): attention.jl:55-59 */
                        if (bias) a += h2f(bias[bs[0] * lk + bs[1] * lq + bs[2] * h + bs[3] * b]);
                        row[lk] = f2h(a);
                        float r = h2f(row[lk]);
                        if (r > m) m = r;
                    }
                    float s = 0.0f;
                    if (!isfinite(m)) { /* every key blocked: zero row, divide by one */
                        for (int64_t lk = 0; lk < Lk; ++lk) row[lk] = 0;
                        s = 1.0f;
                    } else {
                        for (int64_t lk = 0; lk < Lk; ++lk) {
                            float ex = expf(h2f(row[lk]) - m);
                            row[lk] = f2h(ex);
                            s += ex;
                        }
                    }
                    for (int64_t e = 0; e < E; ++e) acc[e] = 0.0f;
                    for (int64_t lk = 0; lk < Lk; ++lk) {
                        float p = h2f(row[lk]);
                        const f16bits* vp = v + vs[1] * lk + vs[2] * h + vs[3] * b;
                        for (int64_t e = 0; e < E; ++e)
                            acc[e] = fmaf(p, h2f(vp[vs[0] * e]), acc[e]);
                    }
                    int64_t o = E * (lq + Lq * (h + H * b));
                    if (out_dtype == ORA_F16)
                        for (int64_t e = 0; e < E; ++e)
                            ((f16bits*)out)[o + e] = f2h(acc[e] / s);
                    else
                        for (int64_t e = 0; e < E; ++e) ((float*)out)[o + e] = acc[e] / s;
                }
        free(row);
        free(acc);
    }
}

/*
 * test/test_flash.jl:13-24 (attnref): plain softmax(QK'·scale)·V over the
 * fp16-rounded operands, here carried in float64 as the tighter truth.
 */
void ora_attention_ref(int64_t E, int64_t Lq, int64_t Lk, int64_t H, int64_t B,
                       const f16bits* q, const int64_t* qs, const f16bits* k,
                       const int64_t* ks, const f16bits* v, const int64_t* vs, float* out,
                       float scale, const f16bits* bias, const int64_t* bs) {
#pragma omp parallel
    {
        double* row = (double*)malloc(sizeof(double) * (size_t)Lk);
        double* acc = (double*)malloc(sizeof(double) * (size_t)E);
#pragma omp for collapse(3) schedule(static)
        for (int64_t b = 0; b < B; ++b)
            for (int64_t h = 0; h < H; ++h)
                for (int64_t lq = 0; lq < Lq; ++lq) {
                    const f16bits* qp = q + qs[1] * lq + qs[2] * h + qs[3] * b;
                    double m = -INFINITY;
                    for (int64_t lk = 0; lk < Lk; ++lk) {
                        const f16bits* kp = k + ks[1] * lk + ks[2] * h + ks[3] * b;
                        double a = 0.0;
                        for (int64_t e = 0; e < E; ++e)
                            a += (double)h2f(qp[qs[0] * e]) * (double)h2f(kp[ks[0] * e]);
                        row[lk] = a * (double)scale;
                        if (bias) row[lk] += (double)h2f(bias[bs[0] * lk + bs[1] * lq + bs[2] * h + bs[3] * b]);
                        if (row[lk] > m) m = row[lk];
                    }
                    double s = 0.0;
                    if (!isfinite(m)) { /* every key blocked: zero row (attention.jl:73-100) */
                        for (int64_t lk = 0; lk < Lk; ++lk) row[lk] = 0.0;
                        s = 1.0;
                    } else
                    for (int64_t lk = 0; lk < Lk; ++lk) {
                        row[lk] = exp(row[lk] - m);
                        s += row[lk];
                    }
                    for (int64_t e = 0; e < E; ++e) acc[e] = 0.0;
                    for (int64_t lk = 0; lk < Lk; ++lk) {
                        const f16bits* vp = v + vs[1] * lk + vs[2] * h + vs[3] * b;
                        double p = row[lk] / s;
                        for (int64_t e = 0; e < E; ++e) acc[e] += p * (double)h2f(vp[vs[0] * e]);
                    }
                    int64_t o = E * (lq + Lq * (h + H * b));
                    for (int64_t e = 0; e < E; ++e) out[o + e] = (float)acc[e];
                }
        free(row);
        free(acc);
    }
}

/* attention.jl:37-40 (toLE): (E,L,H,B) strided -> dense (L,E,H,B). */
void ora_to_le_f16(int64_t E, int64_t L, int64_t H, int64_t B, const f16bits* a,
                   const int64_t* s, f16bits* out) {
    for (int64_t b = 0; b < B; ++b)
        for (int64_t h = 0; h < H; ++h)
            for (int64_t e = 0; e < E; ++e)
                for (int64_t l = 0; l < L; ++l)
                    out[l + L * (e + E * (h + H * b))] =
                        a[s[0] * e + s[1] * l + s[2] * h + s[3] * b];
}

/* ------------------------------------------------------------------ layer norm */

#define LN_WG 128

/* The reference kernel's reduction shape: LN_WG strided partial sums, then a
 * binary tree over them (layernorm.jl:56-75). */
static float ln_tree(float* red) {
    for (int stride = LN_WG / 2; stride > 0; stride /= 2)
        for (int t = 0; t < stride; ++t) red[t] += red[t + stride];
    return red[0];
}

/*
 * layernorm.jl:44-114 (layernorm_kernel!) — same arithmetic as the fallback
 * expression at ops.jl:610-646: fp32 mean, variance about that mean (two passes),
 * rstd = 1/sqrt(var+eps), out = (x-mean)*rstd*gamma+beta rounded once.
 * a is (C, groups) contiguous; in/out dtype fp16 or fp32; gamma/beta share the
 * input dtype and may be NULL; mean/rstd are fp32 (groups,).
 */
void ora_layernorm(int64_t groups, int64_t C, const void* a, int in_dtype, void* out,
                   int out_dtype, float* mean, float* rstd, const void* gamma,
                   const void* beta, float eps) {
#define LD(p, i) (in_dtype == ORA_F16 ? h2f(((const f16bits*)(p))[i]) : ((const float*)(p))[i])
#pragma omp parallel for schedule(static)
    for (int64_t g = 0; g < groups; ++g) {
        float red[LN_WG];
        int64_t base = g * C;
        float n = (float)C;
        for (int t = 0; t < LN_WG; ++t) {
            float s = 0.0f;
            for (int64_t i = t; i < C; i += LN_WG) s += LD(a, base + i);
            red[t] = s;
        }
        float mu = ln_tree(red) / n;
        for (int t = 0; t < LN_WG; ++t) {
            float s2 = 0.0f;
            for (int64_t i = t; i < C; i += LN_WG) {
                float d = LD(a, base + i) - mu;
                s2 += d * d;
            }
            red[t] = s2;
        }
        float r = 1.0f / sqrtf(ln_tree(red) / n + eps);
        for (int64_t i = 0; i < C; ++i) {
            float x = (LD(a, base + i) - mu) * r;
            if (gamma) x *= LD(gamma, i);
            if (beta) x += LD(beta, i);
            if (out_dtype == ORA_F16) ((f16bits*)out)[base + i] = f2h(x);
            else ((float*)out)[base + i] = x;
        }
        mean[g] = mu;
        rstd[g] = r;
    }
#undef LD
}

/* ----------------------------------------------------------------- convolution */

/* conv.jl:309 (convsize). */
int64_t ora_convsize(int64_t n, int64_t k, int64_t s, int64_t p, int64_t d) {
    return (n + 2 * p - d * (k - 1) - 1) / s + 1;
}

/*
 * conv.jl:26-51 (conv2d), groups == 1: x (W,H,Cin,N), w (KW,KH,Cin,Cout),
 * out (OW,OH,Cout,N); fp32 fma chain from the bias over (ci, ky, kx) ascending.
 */
void ora_conv2d_f16(int64_t W, int64_t Hh, int64_t Cin, int64_t Nn, int64_t KW, int64_t KH,
                    int64_t Cout, int64_t sx, int64_t sy, int64_t px, int64_t py,
                    int64_t dx, int64_t dy, const f16bits* x, const f16bits* w,
                    const f16bits* bias, void* out, int out_dtype, int epi) {
    int64_t OW = ora_convsize(W, KW, sx, px, dx), OH = ora_convsize(Hh, KH, sy, py, dy);
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t n = 0; n < Nn; ++n)
        for (int64_t co = 0; co < Cout; ++co)
            for (int64_t oy = 0; oy < OH; ++oy)
                for (int64_t ox = 0; ox < OW; ++ox) {
                    float acc = bias ? h2f(bias[co]) : 0.0f;
                    int64_t bx = ox * sx - px, by = oy * sy - py;
                    for (int64_t ci = 0; ci < Cin; ++ci)
                        for (int64_t ky = 0; ky < KH; ++ky) {
                            int64_t iy = by + ky * dy;
                            if (iy < 0 || iy >= Hh) continue;
                            for (int64_t kx = 0; kx < KW; ++kx) {
                                int64_t ix = bx + kx * dx;
                                if (ix < 0 || ix >= W) continue;
                                acc = fmaf(h2f(x[ix + W * (iy + Hh * (ci + Cin * n))]),
                                           h2f(w[kx + KW * (ky + KH * (ci + Cin * co))]), acc);
                            }
                        }
                    int64_t o = ox + OW * (oy + OH * (co + Cout * n));
                    if (out_dtype == ORA_F16)
                        ((f16bits*)out)[o] = f2h(apply_epi(epi, h2f(f2h(acc))));
                    else
                        ((float*)out)[o] = apply_epi(epi, acc);
                }
}

/*
 * conv.jl:26-51 (conv2d) with GROUPS >= 1: w is (KW,KH,Cin/groups,Cout); output channel co reads the input
 * channels of its own group, g = co / (Cout/groups).
 */
void ora_conv2d_grouped_f16(int64_t W, int64_t Hh, int64_t Cin, int64_t Nn, int64_t KW, int64_t KH,
                            int64_t Cout, int64_t sx, int64_t sy, int64_t px, int64_t py,
                            int64_t dx, int64_t dy, int64_t groups, const f16bits* x, const f16bits* w,
                            const f16bits* bias, void* out, int out_dtype, int epi) {
    int64_t OW = ora_convsize(W, KW, sx, px, dx), OH = ora_convsize(Hh, KH, sy, py, dy);
    int64_t CG = Cin / groups, COG = Cout / groups;
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t n = 0; n < Nn; ++n)
        for (int64_t co = 0; co < Cout; ++co)
            for (int64_t oy = 0; oy < OH; ++oy)
                for (int64_t ox = 0; ox < OW; ++ox) {
                    float acc = bias ? h2f(bias[co]) : 0.0f;
                    int64_t g = co / COG;
                    int64_t bx = ox * sx - px, by = oy * sy - py;
                    for (int64_t ci = 0; ci < CG; ++ci) {
                        int64_t xc = g * CG + ci;
                        for (int64_t ky = 0; ky < KH; ++ky) {
                            int64_t iy = by + ky * dy;
                            if (iy < 0 || iy >= Hh) continue;
                            for (int64_t kx = 0; kx < KW; ++kx) {
                                int64_t ix = bx + kx * dx;
                                if (ix < 0 || ix >= W) continue;
                                acc = fmaf(h2f(x[ix + W * (iy + Hh * (xc + Cin * n))]),
                                           h2f(w[kx + KW * (ky + KH * (ci + CG * co))]), acc);
                            }
                        }
                    }
                    int64_t o = ox + OW * (oy + OH * (co + Cout * n));
                    if (out_dtype == ORA_F16)
                        ((f16bits*)out)[o] = f2h(apply_epi(epi, h2f(f2h(acc))));
                    else
                        ((float*)out)[o] = apply_epi(epi, acc);
                }
}

/* conv.jl:194 (convtransposesize) */
int64_t ora_convtransposesize(int64_t n, int64_t k, int64_t s, int64_t p, int64_t d, int64_t op) {
    return (n - 1) * s - 2 * p + d * (k - 1) + op + 1;
}

/*
 * conv.jl:147-190 (convtranspose2d), the gather form: x (W,H,Cin,N), w (KW,KH,Cout/groups,Cin) — the transposed
 * weight has its two channel axes the other way round — out (OW,OH,Cout,N); fp32 fma chain from the bias over
 * (ci, ky, kx) ascending; an input reaches an output where the stride divides.
 */
void ora_convtranspose2d_f16(int64_t W, int64_t Hh, int64_t Cin, int64_t Nn, int64_t KW, int64_t KH,
                             int64_t Cout, int64_t sx, int64_t sy, int64_t px, int64_t py, int64_t dx,
                             int64_t dy, int64_t opx, int64_t opy, int64_t groups, const f16bits* x,
                             const f16bits* w, const f16bits* bias, void* out, int out_dtype) {
    int64_t OW = ora_convtransposesize(W, KW, sx, px, dx, opx), OH = ora_convtransposesize(Hh, KH, sy, py, dy, opy);
    int64_t COG = Cout / groups, CG = Cin / groups;
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t n = 0; n < Nn; ++n)
        for (int64_t co = 0; co < Cout; ++co)
            for (int64_t oy = 0; oy < OH; ++oy)
                for (int64_t ox = 0; ox < OW; ++ox) {
                    float acc = bias ? h2f(bias[co]) : 0.0f;
                    int64_t cog = co % COG, g = co / COG;
                    int64_t bx = ox + px, by = oy + py;
                    for (int64_t ci = g * CG; ci < (g + 1) * CG; ++ci)
                        for (int64_t ky = 0; ky < KH; ++ky) {
                            int64_t ty = by - ky * dy;
                            if (ty < 0 || ty % sy != 0) continue;
                            int64_t iy = ty / sy;
                            if (iy >= Hh) continue;
                            for (int64_t kx = 0; kx < KW; ++kx) {
                                int64_t tx = bx - kx * dx;
                                if (tx < 0 || tx % sx != 0) continue;
                                int64_t ix = tx / sx;
                                if (ix >= W) continue;
                                acc = fmaf(h2f(x[ix + W * (iy + Hh * (ci + Cin * n))]),
                                           h2f(w[kx + KW * (ky + KH * (cog + COG * ci))]), acc);
                            }
                        }
                    int64_t o = ox + OW * (oy + OH * (co + Cout * n));
                    if (out_dtype == ORA_F16) ((f16bits*)out)[o] = f2h(acc);
                    else ((float*)out)[o] = acc;
                }
}

/*
 * conv_coopmat.jl:246-289 (im2col_kernel!): col is (MP, CRSP) column-major,
 * row m = pixel (ow + OW*(oh + OH*n)), column crs = kw + KW*(kh + KH*cin);
 * rows >= NPQ, columns >= CRS and taps outside the image are zero.
 */
void ora_im2col_f16(int64_t W, int64_t Hh, int64_t Cin, int64_t Nn, int64_t KW, int64_t KH,
                    int64_t sx, int64_t sy, int64_t px, int64_t py, int64_t dx, int64_t dy,
                    int64_t MP, int64_t CRSP, const f16bits* x, f16bits* col) {
    int64_t OW = ora_convsize(W, KW, sx, px, dx), OH = ora_convsize(Hh, KH, sy, py, dy);
    int64_t NPQ = OW * OH * Nn;
#pragma omp parallel for schedule(static)
    for (int64_t c = 0; c < CRSP; ++c) {
        int64_t kw = c % KW, t = c / KW, kh = t % KH, cin = t / KH;
        for (int64_t m = 0; m < MP; ++m) {
            f16bits v = 0;
            if (m < NPQ && cin < Cin) {
                int64_t n = m / (OH * OW), r = m - n * OH * OW, oh = r / OW, ow = r - oh * OW;
                int64_t ix = ow * sx - px + kw * dx, iy = oh * sy - py + kh * dy;
                if (ix >= 0 && ix < W && iy >= 0 && iy < Hh)
                    v = x[ix + W * (iy + Hh * (cin + Cin * n))];
            }
            col[m + MP * c] = v;
        }
    }
}

/* ------------------------------------------------------- elementwise glue ops */

/* ops.jl add.Tensor / clamp.default on fp16 storage: fp32 arithmetic, one rounding. */
void ora_add_f16(const f16bits* a, const f16bits* b, f16bits* y, int64_t n) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) y[i] = f2h(h2f(a[i]) + h2f(b[i]));
}
void ora_clamp_f16(const f16bits* a, f16bits* y, int64_t n, float lo, float hi) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        float v = h2f(a[i]);
        v = v < lo ? lo : (v > hi ? hi : v);
        y[i] = f2h(v);
    }
}
