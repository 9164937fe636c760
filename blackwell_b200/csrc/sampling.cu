// Token sampling on the device: greedy argmax over the vocabulary (many CTAs,
// last-arriver finish), repetition penalty, and softmax / top-k sampling.
#include <cuda_runtime.h>

#include "../../include/blackwell_b200.h"
#include "common.cuh"
#include "host_util.h"

namespace bw {

constexpr int kArgmaxMaxBlocks = 1024;
// Per-device static scratch of the argmax: one packed candidate per CTA and the
// arrival ticket.  Calls that overlap on one GPU (different streams) would race on it.
__device__ unsigned long long g_argmax_part[kArgmaxMaxBlocks];
__device__ unsigned int g_argmax_ticket = 0;

// Total order on floats as unsigned keys; the index is stored inverted so that a
// 64-bit max prefers the larger value and then the smaller index.
__device__ __forceinline__ unsigned int float_key(float f) {
    const unsigned int b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ unsigned long long pack_cand(float v, int idx) {
    return ((unsigned long long)float_key(v) << 32) | (unsigned int)(0xFFFFFFFFu - (unsigned int)idx);
}
__device__ __forceinline__ unsigned long long warp_max_u64(unsigned long long v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, v, o);
        v = other > v ? other : v;
    }
    return v;
}
__device__ __forceinline__ unsigned long long block_max_u64(unsigned long long v, unsigned long long* sh) {
    const int t = threadIdx.x;
    v = warp_max_u64(v);
    if ((t & 31) == 0) sh[t >> 5] = v;
    __syncthreads();
    if (t < 32) {
        unsigned long long w = t < (int)(blockDim.x >> 5) ? sh[t] : 0ull;
        w = warp_max_u64(w);
        if (t == 0) sh[0] = w;
    }
    __syncthreads();
    return sh[0];
}

// Candidates start at (-1e38, index 0) and only values strictly greater replace
// them, as in the reference's scan.
__global__ void __launch_bounds__(256) argmax_kernel_b200(const float* logits, int vocab, int* out_id) {
    __shared__ unsigned long long sh[32];
    __shared__ bool last;
    unsigned long long best = pack_cand(-1e38f, 0);
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < vocab; i += gridDim.x * blockDim.x) {
        const float v = logits[i];
        if (v > -1e38f) {
            const unsigned long long c = pack_cand(v, i);
            best = c > best ? c : best;
        }
    }
    best = block_max_u64(best, sh);
    if (threadIdx.x == 0) {
        g_argmax_part[blockIdx.x] = best;
        __threadfence();
        const unsigned int ticket = atomicAdd(&g_argmax_ticket, 1u);
        last = (ticket == gridDim.x - 1);
    }
    __syncthreads();
    if (!last) return;
    __threadfence();
    unsigned long long b2 = pack_cand(-1e38f, 0);
    for (int i = threadIdx.x; i < (int)gridDim.x; i += blockDim.x) {
        const unsigned long long c = *((volatile unsigned long long*)&g_argmax_part[i]);
        b2 = c > b2 ? c : b2;
    }
    b2 = block_max_u64(b2, sh);
    if (threadIdx.x == 0) {
        *out_id = (int)(0xFFFFFFFFu - (unsigned int)(b2 & 0xFFFFFFFFull));
        g_argmax_ticket = 0;
    }
}

__global__ void __launch_bounds__(256) repetition_penalty_kernel_b200(float* logits, const int* recent,
                                                                      int num_recent, float penalty, int vocab) {
    // one thread per listed id; an id listed several times is penalised once (the first listing acts)
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= num_recent) return;
    const int id = recent[i];
    if (id < 0 || id >= vocab) return;
    for (int j = 0; j < i; ++j)
        if (recent[j] == id) return;
    const float l = logits[id];
    logits[id] = l > 0 ? l / penalty : l * penalty;
}

// splitmix64 -> uniform in (0, 1]
__device__ __forceinline__ float uniform01(unsigned long long seed, int step) {
    unsigned long long z = seed + 0x9E3779B97F4A7C15ull * (unsigned long long)(step + 1);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z = z ^ (z >> 31);
    return ((float)(z >> 40) + 1.0f) * (1.0f / 16777216.0f);
}

__device__ __forceinline__ float block_sum_f(float v, float* sh) {
    const int t = threadIdx.x;
    v = warp_sum(v);
    __syncthreads();
    if ((t & 31) == 0) sh[t >> 5] = v;
    __syncthreads();
    if (t < 32) {
        float w = t < (int)(blockDim.x >> 5) ? sh[t] : 0.f;
        w = warp_sum(w);
        if (t == 0) sh[0] = w;
    }
    __syncthreads();
    return sh[0];
}

// Softmax over the raw logits, optional top-k filter (keep the k largest, ties
// at the threshold kept), renormalise, draw one token by inverse CDF.  One CTA.
__global__ void __launch_bounds__(1024) sample_kernel_b200(const float* logits, int vocab, int top_k, int* out_id,
                                                           unsigned long long seed, int step) {
    __shared__ float shf[32];
    __shared__ unsigned int hist[256];
    __shared__ unsigned int sel_prefix, sel_remaining;
    __shared__ float chunk_sum[1024];
    const int t = threadIdx.x, T = blockDim.x;

    float mx = -3.0e38f;
    for (int i = t; i < vocab; i += T) mx = fmaxf(mx, logits[i]);
    mx = warp_max(mx);
    if ((t & 31) == 0) shf[t >> 5] = mx;
    __syncthreads();
    if (t < 32) {
        float w = t < (T >> 5) ? shf[t] : -3.0e38f;
        w = warp_max(w);
        if (t == 0) shf[0] = w;
    }
    __syncthreads();
    mx = shf[0];
    __syncthreads();

    // radix select of the k-th largest key, 8 bits per pass from the top
    unsigned int thr_key = 0;
    if (top_k > 0 && top_k < vocab) {
        if (t == 0) { sel_prefix = 0; sel_remaining = (unsigned int)top_k; }
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            for (int i = t; i < 256; i += T) hist[i] = 0;
            __syncthreads();
            const unsigned int prefix = sel_prefix;
            const unsigned int mask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
            for (int i = t; i < vocab; i += T) {
                const unsigned int k = float_key(logits[i]);
                if ((k & mask) == prefix) atomicAdd(&hist[(k >> shift) & 0xFF], 1u);
            }
            __syncthreads();
            if (t == 0) {
                unsigned int rem = sel_remaining;
                int b = 255;
                for (; b > 0; --b) {
                    if (hist[b] >= rem) break;
                    rem -= hist[b];
                }
                sel_prefix = prefix | ((unsigned int)b << shift);
                sel_remaining = rem;
            }
            __syncthreads();
        }
        thr_key = sel_prefix;
    }

    // contiguous chunk per thread so that the CDF runs in index order
    const int per = (vocab + T - 1) / T;
    const int i0 = min(t * per, vocab), i1 = min(i0 + per, vocab);
    float local = 0.f;
    for (int i = i0; i < i1; ++i) {
        const float v = logits[i];
        if (float_key(v) >= thr_key) local += expf(v - mx);
    }
    chunk_sum[t] = local;
    const float total = block_sum_f(local, shf);
    if (t == 0) {
        const float r = uniform01(seed, step) * total;
        float cum = 0.f;
        int pick = vocab - 1;
        int c = 0;
        for (; c < T; ++c) {
            if (cum + chunk_sum[c] >= r) break;
            cum += chunk_sum[c];
        }
        if (c < T) {
            const int a0 = min(c * per, vocab), a1 = min(a0 + per, vocab);
            for (int i = a0; i < a1; ++i) {
                const float v = logits[i];
                if (float_key(v) >= thr_key) {
                    cum += expf(v - mx);
                    pick = i;
                    if (cum >= r) break;
                }
            }
        }
        *out_id = pick;
    }
}

}  // namespace bw

using namespace bw;

extern "C" int bw_sample_argmax_gpu(const float* logits, int vocab, int* out_id, void* stream) {
    if (!logits || !out_id || vocab < 1) return cudaErrorInvalidValue;
    int blocks = (vocab + 256 * 4 - 1) / (256 * 4);
    const int cap = 2 * sm_count(current_device());
    if (blocks > cap) blocks = cap;
    if (blocks > kArgmaxMaxBlocks) blocks = kArgmaxMaxBlocks;
    if (blocks < 1) blocks = 1;
    argmax_kernel_b200<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(logits, vocab, out_id);
    count_launch(1);
    return cudaPeekAtLastError();
}

extern "C" int bw_sample_gpu(const float* logits, int vocab, float temperature, int top_k, int* out_id,
                             unsigned long long rng_seed, int step, void* stream) {
    if (temperature < 0.01f) return bw_sample_argmax_gpu(logits, vocab, out_id, stream);
    if (!logits || !out_id || vocab < 1) return cudaErrorInvalidValue;
    sample_kernel_b200<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(logits, vocab, top_k, out_id, rng_seed,
                                                                         step);
    count_launch(1);
    return cudaPeekAtLastError();
}

extern "C" int bw_apply_repetition_penalty(float* logits, const int* recent, int num_recent, float penalty, int vocab,
                                           void* stream) {
    if (penalty <= 1.0f || num_recent == 0) return cudaSuccess;
    if (!logits || !recent || num_recent < 0 || vocab < 1) return cudaErrorInvalidValue;
    repetition_penalty_kernel_b200<<<(num_recent + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        logits, recent, num_recent, penalty, vocab);
    count_launch(1);
    return cudaPeekAtLastError();
}
