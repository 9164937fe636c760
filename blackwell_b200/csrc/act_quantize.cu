// Stand-alone block-16 activation quantizers (INT4 and INT8 rules of the
// reference) and the two fused "op + INT4 quantize" kernels.  One thread owns
// one 16-element block: 64 bytes in (four float4 loads), 8 or 16 bytes out.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../../include/blackwell_b200.h"
#include "common.cuh"
#include "quant_rules.cuh"
#include "host_util.h"

namespace bw {

__device__ __forceinline__ void load16(const float* p, float (&v)[16]) {
    const float4* q = reinterpret_cast<const float4*>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float4 f = __ldg(q + i);
        v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
    }
}
__device__ __forceinline__ void load16(const __half* p, float (&v)[16]) {
    const uint4* q = reinterpret_cast<const uint4*>(p);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const uint4 u = __ldg(q + i);
        const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __half22float2(h[j]);
            v[8 * i + 2 * j] = f.x;
            v[8 * i + 2 * j + 1] = f.y;
        }
    }
}

// 16 values -> 8 packed bytes (nibble = q + 8, even element low) + scale.
// kFusedRule selects sc = fmaxf(absmax/7, 1e-9), clamp +-7; otherwise
// sc = absmax > 1e-10 ? absmax/7 : 1/7, clamp [-8, 7].
template <bool kFusedRule>
__device__ __forceinline__ void pack_block_i4(const float (&v)[16], uint8_t* out8, float* sc_out) {
    float am = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) am = fmaxf(am, fabsf(v[i]));
    const float sc = kFusedRule ? fmaxf(am / 7.0f, 1e-9f) : quant_scale_i4(am);
    *sc_out = sc;
    uint32_t w[2] = {0, 0};
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        int q;
        if (kFusedRule) q = (int)fminf(7.0f, fmaxf(-7.0f, roundf(v[i] / sc)));
        else q = quant_i4(v[i], sc);
        w[i >> 3] |= (uint32_t)((q + 8) & 0xF) << (4 * (i & 7));
    }
    *reinterpret_cast<uint2*>(out8) = make_uint2(w[0], w[1]);
}

__global__ void __launch_bounds__(256) quantize_int4_kernel_b200(uint8_t* out, float* sc, const float* in,
                                                                 long total_blocks) {
    const long b = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= total_blocks) return;
    float v[16];
    load16(in + 16 * b, v);
    pack_block_i4<false>(v, out + 8 * b, sc + b);
}

template <typename T>
__global__ void __launch_bounds__(256) quantize_int8_kernel_b200(int8_t* out, float* sc, const T* in,
                                                                 long total_blocks) {
    const long b = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= total_blocks) return;
    float v[16];
    load16(in + 16 * b, v);
    float am = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) am = fmaxf(am, fabsf(v[i]));
    const float s = quant_scale_i8(am);
    sc[b] = s;
    uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
    for (int i = 0; i < 16; ++i) w[i >> 2] |= (uint32_t)(quant_i8(v[i], s) & 0xFF) << (8 * (i & 3));
    *reinterpret_cast<uint4*>(out + 16 * b) = make_uint4(w[0], w[1], w[2], w[3]);
}

// silu(gate) * up -> INT4 (fused rule).
__global__ void __launch_bounds__(256) swiglu_quant_int4_kernel(uint8_t* out, float* sc, const float* gate,
                                                                const float* up, long total_blocks) {
    const long b = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= total_blocks) return;
    float g[16], u[16];
    load16(gate + 16 * b, g);
    load16(up + 16 * b, u);
#pragma unroll
    for (int i = 0; i < 16; ++i) g[i] = g[i] * (1.0f / (1.0f + expf(-g[i]))) * u[i];  // form used by the fused reference kernel
    pack_block_i4<true>(g, out + 8 * b, sc + b);
}

// RMSNorm over one row of N elements, then INT4 (fused rule).  One CTA.
__global__ void __launch_bounds__(1024) rmsnorm_quant_int4_kernel(uint8_t* out, float* sc, const float* x,
                                                                  const float* w, int N, float eps) {
    __shared__ float part[32];
    __shared__ float rstd_s;
    const int t = threadIdx.x;
    float ss = 0.f;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    for (int i = t; i < N / 4; i += blockDim.x) {
        const float4 f = __ldg(x4 + i);
        ss = fmaf(f.x, f.x, ss); ss = fmaf(f.y, f.y, ss); ss = fmaf(f.z, f.z, ss); ss = fmaf(f.w, f.w, ss);
    }
    ss = warp_sum(ss);
    if ((t & 31) == 0) part[t >> 5] = ss;
    __syncthreads();
    if (t < 32) {
        float v = t < (int)(blockDim.x >> 5) ? part[t] : 0.f;
        v = warp_sum(v);
        if (t == 0) rstd_s = rsqrtf(v / (float)N + eps);
    }
    __syncthreads();
    const float rstd = rstd_s;
    for (int b = t; b < N / 16; b += blockDim.x) {
        float v[16], g[16];
        load16(x + 16 * b, v);
        load16(w + 16 * b, g);
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = v[i] * g[i] * rstd;
        pack_block_i4<true>(v, out + 8 * (size_t)b, sc + b);
    }
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace bw

using namespace bw;

extern "C" int bw_quantize_int4_batched(void* x_out_packed, float* x_out_sc, const float* in_fp32, int K, int M,
                                        void* stream) {
    if (!x_out_packed || !x_out_sc || !in_fp32 || K <= 0 || K % 16 != 0 || M < 1) return cudaErrorInvalidValue;
    if (!aligned16(in_fp32) || (reinterpret_cast<uintptr_t>(x_out_packed) & 7)) return cudaErrorInvalidValue;
    const long total = (long)M * (K / 16);
    quantize_int4_kernel_b200<<<(unsigned)((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<uint8_t*>(x_out_packed), x_out_sc, in_fp32, total);
    count_launch(1);
    return cudaPeekAtLastError();
}

extern "C" int bw_quantize_int4(void* x_out_packed, float* x_out_sc, const float* in_fp32, int K, void* stream) {
    return bw_quantize_int4_batched(x_out_packed, x_out_sc, in_fp32, K, 1, stream);
}

extern "C" int bw_quantize_int8(void* out_int8, float* out_scale, const float* in_fp32, int num_elements,
                                void* stream) {
    if (!out_int8 || !out_scale || !in_fp32 || num_elements <= 0 || num_elements % 16 != 0)
        return cudaErrorInvalidValue;
    if (!aligned16(in_fp32) || !aligned16(out_int8)) return cudaErrorInvalidValue;
    const long total = num_elements / 16;
    quantize_int8_kernel_b200<float><<<(unsigned)((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<int8_t*>(out_int8), out_scale, in_fp32, total);
    count_launch(1);
    return cudaPeekAtLastError();
}

extern "C" int bw_quantize_int8_f16(void* out_int8, float* out_scale, const uint16_t* in_f16, int num_elements,
                                    void* stream) {
    if (!out_int8 || !out_scale || !in_f16 || num_elements <= 0 || num_elements % 16 != 0)
        return cudaErrorInvalidValue;
    if (!aligned16(in_f16) || !aligned16(out_int8)) return cudaErrorInvalidValue;
    const long total = num_elements / 16;
    quantize_int8_kernel_b200<__half><<<(unsigned)((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<int8_t*>(out_int8), out_scale, reinterpret_cast<const __half*>(in_f16), total);
    count_launch(1);
    return cudaPeekAtLastError();
}

extern "C" int bw_fused_rmsnorm_quant_int4(uint8_t* x_out_packed, float* x_out_scale, const float* proj,
                                           const float* weight, int N, float eps, void* stream) {
    if (!x_out_packed || !x_out_scale || !proj || !weight || N <= 0 || N % 32 != 0) return cudaErrorInvalidValue;
    if (!aligned16(proj) || !aligned16(weight) || (reinterpret_cast<uintptr_t>(x_out_packed) & 7))
        return cudaErrorInvalidValue;
    rmsnorm_quant_int4_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(x_out_packed, x_out_scale, proj,
                                                                                weight, N, eps);
    count_launch(1);
    return cudaPeekAtLastError();
}

extern "C" int bw_fused_swiglu_quant_int4(uint8_t* out_packed, float* out_scale, const float* gate, const float* up,
                                          int N, void* stream) {
    if (!out_packed || !out_scale || !gate || !up || N <= 0 || N % 32 != 0) return cudaErrorInvalidValue;
    if (!aligned16(gate) || !aligned16(up) || (reinterpret_cast<uintptr_t>(out_packed) & 7))
        return cudaErrorInvalidValue;
    const long total = N / 16;
    swiglu_quant_int4_kernel<<<(unsigned)((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        out_packed, out_scale, gate, up, total);
    count_launch(1);
    return cudaPeekAtLastError();
}
