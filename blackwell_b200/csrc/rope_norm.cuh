// Per-head RMSNorm followed by RoPE for one 128-wide head held by a warp, four consecutive elements per lane
// (the reference's caller-side head_norm_kernel and apply_rope_kernel, server/inference_server_int4_batched.cu:49-70).
// RoPE rotates interleaved pairs (2i, 2i+1) by theta = pos * base^(-2i/128).
#pragma once
#include "common.cuh"

namespace bw {

__device__ __forceinline__ float4 head_norm_rope(float4 v, const float* norm_w, float eps, int pos, float rope_base,
                                                 int lane) {
    float ss = v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    ss = warp_sum(ss);
    const float is = rsqrtf(ss / 128.0f + eps);
    const float4 w = *reinterpret_cast<const float4*>(norm_w + 4 * lane);
    v.x = v.x * is * w.x; v.y = v.y * is * w.y; v.z = v.z * is * w.z; v.w = v.w * is * w.w;
    const float t0 = (float)pos * powf(rope_base, -2.0f * (float)(2 * lane) / 128.0f);
    const float t1 = (float)pos * powf(rope_base, -2.0f * (float)(2 * lane + 1) / 128.0f);
    const float c0 = cosf(t0), s0 = sinf(t0), c1 = cosf(t1), s1 = sinf(t1);
    return make_float4(v.x * c0 - v.y * s0, v.x * s0 + v.y * c0, v.z * c1 - v.w * s1, v.z * s1 + v.w * c1);
}

// Four floats -> four binary16 values, one 8-byte store.
__device__ __forceinline__ void store_half4(__half* dst, float4 v) {
    const __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<const uint32_t*>(&a);
    u.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>(dst) = u;
}

}  // namespace bw
