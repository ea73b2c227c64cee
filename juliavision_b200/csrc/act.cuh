// The epilogue activations shared by the GEMM store, the matrix-vector store and the stand-alone
// activation op (reference ops.jl:161-169,1665-1685): one definition, so a folded activation and the op it
// replaced give the same bits.
#pragma once
#include <cuda_fp16.h>

#include "../../include/b200dnn.h"

namespace b200 {

// geluexact on the fp16-rounded value: 0.5 x (1 + erf(x/sqrt2)) with the reference's erf, Abramowitz &
// Stegun 7.1.26 in fp32 (ops.jl:161-169,1665-1670); the reciprocal and the exponential are the approximate
// hardware forms.
// Every multiply, add and fused multiply-add is spelled out, so that the packed form below, which the GEMM
// store uses, performs the same roundings and gives the same bits.
__device__ __forceinline__ float gelu_exact(float x) {
    const float z = __fmul_rn(x, 0.70710678118654752f);
    const float a = fabsf(z);
    float t;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(__fmaf_rn(0.3275911f, a, 1.0f)));
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(__fmul_rn(__fmul_rn(a, a), -1.4426950408889634f)));
    float poly = __fmaf_rn(1.061405429f, t, -1.453152027f);
    poly = __fmaf_rn(poly, t, 1.421413741f);
    poly = __fmaf_rn(poly, t, -0.284496736f);
    poly = __fmaf_rn(poly, t, 0.254829592f);
    poly = __fmul_rn(poly, t);
    const float y = __fmaf_rn(-poly, e, 1.0f);          // erf(|z|)
    const float hx = __fmul_rn(0.5f, x);
    return __fmaf_rn(hx, copysignf(y, z), hx);
}

// The same function on a pair, with the multiplies and FMAs as packed fp32-pair instructions (sm_100): half
// the instructions per element in the GEMM store, where the activation is what a short-K tile waits for.
namespace act_detail {
__device__ __forceinline__ unsigned long long pk(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void upk(unsigned long long v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ unsigned long long mul2(unsigned long long a, unsigned long long b) {
    unsigned long long d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ unsigned long long dup(float c) { return pk(c, c); }
} // namespace act_detail

__device__ __forceinline__ float2 gelu_exact2(float2 x) {
    using namespace act_detail;
    const unsigned long long x2 = pk(x.x, x.y);
    float z0, z1;
    upk(mul2(x2, dup(0.70710678118654752f)), z0, z1);
    const float a0 = fabsf(z0), a1 = fabsf(z1);
    const unsigned long long a2 = pk(a0, a1);
    float d0, d1, t0, t1, u0, u1, e0, e1;
    upk(fma2(dup(0.3275911f), a2, dup(1.0f)), d0, d1);
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t0) : "f"(d0));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t1) : "f"(d1));
    upk(mul2(mul2(a2, a2), dup(-1.4426950408889634f)), u0, u1);
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e0) : "f"(u0));
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e1) : "f"(u1));
    const unsigned long long t2 = pk(t0, t1);
    unsigned long long poly = fma2(dup(1.061405429f), t2, dup(-1.453152027f));
    poly = fma2(poly, t2, dup(1.421413741f));
    poly = fma2(poly, t2, dup(-0.284496736f));
    poly = fma2(poly, t2, dup(0.254829592f));
    poly = mul2(poly, t2);
    float p0, p1, y0, y1;
    upk(poly, p0, p1);
    upk(fma2(pk(-p0, -p1), pk(e0, e1), dup(1.0f)), y0, y1);
    const unsigned long long hx = mul2(dup(0.5f), x2);
    float r0, r1;
    upk(fma2(hx, pk(copysignf(y0, z0), copysignf(y1, z1)), hx), r0, r1);
    return make_float2(r0, r1);
}
__device__ __forceinline__ float apply_act(int epi, float v) {
    switch (epi) {
        case B200_EPI_RELU: return fmaxf(v, 0.f);
        case B200_EPI_GELU: return gelu_exact(v);
        case B200_EPI_GELU_TANH: {
            float u = 0.7978845608028654f * (v + 0.044715f * v * v * v);
            return 0.5f * v * (1.0f + tanhf(u));
        }
        default: return v;
    }
}

} // namespace b200
