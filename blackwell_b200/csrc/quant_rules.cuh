// Block-16 activation quantization rules of the reference, shared by the
// stand-alone quantizers and the fused GEMV prologues so that both produce the
// same bits.
#pragma once
#include <cuda_runtime.h>

namespace bw {

// Reference rule for int8 activations: sc = absmax/127 (1 when < 1e-10),
// q = clamp(roundf(v/sc), +-127).
__device__ __forceinline__ float quant_scale_i8(float absmax) {
    float sc = absmax / 127.0f;
    return sc < 1e-10f ? 1.0f : sc;
}
__device__ __forceinline__ int quant_i8(float v, float sc) {
    float q = roundf(v / sc);
    q = fminf(127.0f, fmaxf(-127.0f, q));
    return (int)q;
}
// Reference rule for int4 activations: sc = absmax > 1e-10 ? absmax/7 : 1/7,
// q = clamp((int)roundf(v/sc), -8, 7).
__device__ __forceinline__ float quant_scale_i4(float absmax) {
    return absmax > 1e-10f ? absmax / 7.0f : 1.0f / 7.0f;
}
__device__ __forceinline__ int quant_i4(float v, float sc) {
    int q = (int)roundf(v / sc);
    return max(-8, min(7, q));
}

// silu(g) * u in the form of the stand-alone SwiGLU kernel.
__device__ __forceinline__ float silu_mul(float g, float u) { return (g / (1.0f + expf(-g))) * u; }

}  // namespace bw
