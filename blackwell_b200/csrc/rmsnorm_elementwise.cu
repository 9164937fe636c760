// RMSNorm, SwiGLU, residual add and decode-time RoPE: the small fp32 glue
// kernels between the GEMVs.  All are bandwidth-trivial; they are written with
// 16-byte accesses and one CTA per sequence (norm) or a flat grid (elementwise).
#include <cuda_runtime.h>

#include "../../include/blackwell_b200.h"
#include "common.cuh"
#include "host_util.h"

namespace bw {

// out = x * w * rsqrt(mean(x^2) + eps), one CTA per sequence, every element of
// the row takes part.  kVec = rows and pointers allow float4 access.
template <bool kVec>
__global__ void __launch_bounds__(512) rmsnorm_rows_kernel(float* out, const float* inp, const float* weight, int H,
                                                           float eps) {
    __shared__ float part[16];
    __shared__ float rstd_s;
    const int t = threadIdx.x;
    const float* x = inp + (size_t)blockIdx.x * H;
    float* o = out + (size_t)blockIdx.x * H;
    float ss = 0.f;
    if (kVec) {
        const float4* x4 = reinterpret_cast<const float4*>(x);
        for (int i = t; i < H / 4; i += blockDim.x) {
            const float4 f = x4[i];
            ss = fmaf(f.x, f.x, ss); ss = fmaf(f.y, f.y, ss); ss = fmaf(f.z, f.z, ss); ss = fmaf(f.w, f.w, ss);
        }
    } else {
        for (int i = t; i < H; i += blockDim.x) ss = fmaf(x[i], x[i], ss);
    }
    ss = warp_sum(ss);
    if ((t & 31) == 0) part[t >> 5] = ss;
    __syncthreads();
    if (t < 32) {
        float v = t < (int)(blockDim.x >> 5) ? part[t] : 0.f;
        v = warp_sum(v);
        if (t == 0) rstd_s = rsqrtf(v / (float)H + eps);
    }
    __syncthreads();
    const float rstd = rstd_s;
    if (kVec) {
        const float4* x4 = reinterpret_cast<const float4*>(x);
        const float4* w4 = reinterpret_cast<const float4*>(weight);
        float4* o4 = reinterpret_cast<float4*>(o);
        for (int i = t; i < H / 4; i += blockDim.x) {
            const float4 f = x4[i], g = __ldg(w4 + i);
            o4[i] = make_float4(f.x * g.x * rstd, f.y * g.y * rstd, f.z * g.z * rstd, f.w * g.w * rstd);
        }
    } else {
        for (int i = t; i < H; i += blockDim.x) o[i] = x[i] * weight[i] * rstd;
    }
}

__global__ void __launch_bounds__(256) swiglu_kernel_b200(float* out, const float* gate, const float* up, int n) {
    const int i4 = blockIdx.x * blockDim.x + threadIdx.x;
    const int base = i4 * 4;
    if (base + 3 < n && ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(gate) |
                          reinterpret_cast<uintptr_t>(up)) & 15) == 0) {
        const float4 g = reinterpret_cast<const float4*>(gate)[i4];
        const float4 u = reinterpret_cast<const float4*>(up)[i4];
        float4 r;
        r.x = (g.x / (1.0f + expf(-g.x))) * u.x;
        r.y = (g.y / (1.0f + expf(-g.y))) * u.y;
        r.z = (g.z / (1.0f + expf(-g.z))) * u.z;
        r.w = (g.w / (1.0f + expf(-g.w))) * u.w;
        reinterpret_cast<float4*>(out)[i4] = r;
    } else {
        for (int i = base; i < n && i < base + 4; ++i) out[i] = (gate[i] / (1.0f + expf(-gate[i]))) * up[i];
    }
}

__global__ void __launch_bounds__(256) vector_add_kernel_b200(float* out, const float* a, const float* b, int n) {
    const int i4 = blockIdx.x * blockDim.x + threadIdx.x;
    const int base = i4 * 4;
    if (base + 3 < n && ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(a) |
                          reinterpret_cast<uintptr_t>(b)) & 15) == 0) {
        const float4 x = reinterpret_cast<const float4*>(a)[i4];
        const float4 y = reinterpret_cast<const float4*>(b)[i4];
        reinterpret_cast<float4*>(out)[i4] = make_float4(x.x + y.x, x.y + y.y, x.z + y.z, x.w + y.w);
    } else {
        for (int i = base; i < n && i < base + 4; ++i) out[i] = a[i] + b[i];
    }
}

// In-place rotation of interleaved pairs (2i, 2i+1) of every head by the
// cos/sin table row of the position read from device memory.
__global__ void __launch_bounds__(128) rope_decode_kernel_b200(float* data, const float* cos_cache,
                                                               const float* sin_cache, const int* seq_pos_ptr,
                                                               int heads, int head_dim) {
    const int pairs = head_dim / 2;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= heads * pairs) return;
    const int h = idx / pairs, i = idx - h * pairs;
    const int pos = *seq_pos_ptr;
    const float c = cos_cache[(size_t)pos * pairs + i], s = sin_cache[(size_t)pos * pairs + i];
    float2* p = reinterpret_cast<float2*>(data + (size_t)h * head_dim) + i;
    const float2 v = *p;
    *p = make_float2(v.x * c - v.y * s, v.x * s + v.y * c);
}

}  // namespace bw

using namespace bw;

extern "C" int bw_fused_rmsnorm_batched(float* out, const float* inp, const float* weight, int H, float eps, int M,
                                        void* stream) {
    if (!out || !inp || !weight || H <= 0 || M < 1) return cudaErrorInvalidValue;
    const bool vec = (H % 4 == 0) && ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(inp) |
                                       reinterpret_cast<uintptr_t>(weight)) & 15) == 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (vec) rmsnorm_rows_kernel<true><<<M, 512, 0, st>>>(out, inp, weight, H, eps);
    else rmsnorm_rows_kernel<false><<<M, 512, 0, st>>>(out, inp, weight, H, eps);
    count_launch(1);
    return cudaPeekAtLastError();
}

extern "C" int bw_fused_rmsnorm(float* out, const float* inp, const float* weight, int num_elements, float eps,
                                void* stream) {
    return bw_fused_rmsnorm_batched(out, inp, weight, num_elements, eps, 1, stream);
}

extern "C" int bw_apply_swiglu(float* out, const float* gate, const float* up, int num_elements, void* stream) {
    if (!out || !gate || !up || num_elements < 0) return cudaErrorInvalidValue;
    if (num_elements == 0) return cudaSuccess;
    const int n4 = (num_elements + 3) / 4;
    swiglu_kernel_b200<<<(n4 + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(out, gate, up, num_elements);
    count_launch(1);
    return cudaPeekAtLastError();
}

extern "C" int bw_vector_add_fp32(float* out, const float* a, const float* b, int num_elements, void* stream) {
    if (!out || !a || !b || num_elements < 0) return cudaErrorInvalidValue;
    if (num_elements == 0) return cudaSuccess;
    const int n4 = (num_elements + 3) / 4;
    vector_add_kernel_b200<<<(n4 + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(out, a, b, num_elements);
    count_launch(1);
    return cudaPeekAtLastError();
}

extern "C" int bw_fused_rope_decode(float* out_inplace, const float* cos_cache, const float* sin_cache,
                                    const int* seq_pos_ptr, int heads, int head_dim, int max_seq_len, void* stream) {
    (void)max_seq_len;
    if (!out_inplace || !cos_cache || !sin_cache || !seq_pos_ptr || heads < 1 || head_dim < 2 || head_dim % 2)
        return cudaErrorInvalidValue;
    const int total = heads * (head_dim / 2);
    rope_decode_kernel_b200<<<(total + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        out_inplace, cos_cache, sin_cache, seq_pos_ptr, heads, head_dim);
    count_launch(1);
    return cudaPeekAtLastError();
}
