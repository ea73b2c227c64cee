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
__device__ __forceinline__ float gelu_exact(float x) {
    const float z = x * 0.70710678118654752f;
    const float a = fabsf(z);
    float t;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(fmaf(0.3275911f, a, 1.0f)));
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-a * a * 1.4426950408889634f));
    const float poly = ((((1.061405429f * t - 1.453152027f) * t + 1.421413741f) * t - 0.284496736f) * t + 0.254829592f) * t;
    const float y = fmaf(-poly, e, 1.0f);          // erf(|z|)
    const float hx = 0.5f * x;
    return fmaf(hx, copysignf(y, z), hx);
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
