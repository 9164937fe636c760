// Glue kernels of the batched decode step that the reference runs as separate per-sequence launches from its
// caller (head norm, RoPE, KV update: server/inference_server_int4_batched.cu:49-70,262-266) or on the host
// (embedding lookup, :251): here one launch each for the whole batch, with per-sequence positions in device memory
// and a binary16 KV cache, so that a decode step can live in one CUDA graph.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../../include/blackwell_b200.h"
#include "common.cuh"
#include "host_util.h"
#include "rope_norm.cuh"

namespace bw {

constexpr int kHeadDim = 128;

// One warp per (sequence, head) of the fused QKV projection output [M][(nqh + 2 nkv) * 128]:
//   q heads: per-head RMSNorm (q_norm_w) then RoPE            -> q_out f32 [M][nqh * 128]
//   k heads: per-head RMSNorm (k_norm_w) then RoPE, to half   -> K cache row at the sequence's position
//   v heads: to half                                          -> V cache row at the sequence's position
// RoPE rotates interleaved pairs (2i, 2i+1) by theta = pos * base^(-2i/128).
__global__ void __launch_bounds__(128) qk_norm_rope_kv_kernel(float* q_out, __half* k_cache, __half* v_cache,
                                                              const float* qkv, const float* q_norm_w,
                                                              const float* k_norm_w, const int* d_seq_pos, int nqh,
                                                              int nkv, int max_seq, int M, size_t kv_batch_elems,
                                                              size_t kv_layer_elems, float eps, float rope_base) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int heads = nqh + 2 * nkv;
    const int gw = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (gw >= M * heads) return;
    const int m = gw / heads, h = gw - m * heads;
    const int pos = d_seq_pos[m];
    float4 v = *reinterpret_cast<const float4*>(qkv + ((size_t)m * heads + h) * kHeadDim + 4 * lane);
    const bool is_q = h < nqh, is_k = !is_q && h < nqh + nkv;
    if (is_q || is_k) v = head_norm_rope(v, is_q ? q_norm_w : k_norm_w, eps, pos, rope_base, lane);
    if (is_q) {
        *reinterpret_cast<float4*>(q_out + ((size_t)m * nqh + h) * kHeadDim + 4 * lane) = v;
    } else {
        // A position outside the cache (a sequence that has run past max_seq) is never written.
        if ((unsigned)pos >= (unsigned)max_seq) return;
        const int kvh = is_k ? h - nqh : h - nqh - nkv;
        __half* dst = (is_k ? k_cache : v_cache) + (size_t)m * kv_batch_elems + kv_layer_elems +
                      ((size_t)kvh * max_seq + pos) * kHeadDim + 4 * lane;
        store_half4(dst, v);
    }
}

// x[m][:] = float(table[token[m]][:]) -- the embedding lookup with token ids in device memory.
__global__ void __launch_bounds__(256) embed_gather_kernel(float* x, const __half* table, const int* tokens, int H,
                                                           int vocab) {
    const int m = blockIdx.y;
    int tok = tokens[m];
    tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (i >= H) return;
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(table + (size_t)tok * H + i));
    const __half2* h = reinterpret_cast<const __half2*>(&u);
    float4 a, b;
    float2 f;
    f = __half22float2(h[0]); a.x = f.x; a.y = f.y;
    f = __half22float2(h[1]); a.z = f.x; a.w = f.y;
    f = __half22float2(h[2]); b.x = f.x; b.y = f.y;
    f = __half22float2(h[3]); b.z = f.x; b.w = f.y;
    float4* o = reinterpret_cast<float4*>(x + (size_t)m * H + i);
    o[0] = a;
    o[1] = b;
}

// x[m][:] = table[token[m]][:] for an fp32 table (the reference dequantizes its INT4 embedding to fp32 once at start-up:
// server/inference_server_int4_batched.cu:196-217).
__global__ void __launch_bounds__(256) embed_gather_f32_kernel(float* x, const float* table, const int* tokens, int H,
                                                               int vocab) {
    const int m = blockIdx.y;
    int tok = tokens[m];
    tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= H) return;
    *reinterpret_cast<float4*>(x + (size_t)m * H + i) = __ldg(reinterpret_cast<const float4*>(table + (size_t)tok * H + i));
}

// Token bookkeeping of a batched generation that never leaves the GPU.  Sequence m has a prompt of prompt_len[m] ids
// in prompt[m][0 .. max_prompt) and stands at position pos[m] (the index of the token it consumes in this step).
//   select: the step's input id = the prompt's id at that position while the prompt lasts, else the id sampled by
//           the previous step;
//   record: after sampling (pos already advanced to the new token's index p), a token beyond the prompt is the
//           sequence's generated token number p - prompt_len[m], stored in gen[m][..] if it is one of the first max_new.
__global__ void select_input_tokens_kernel(int* tokens_in, const int* sampled, const int* prompt, const int* prompt_len,
                                           const int* pos, int M, int max_prompt) {
    const int m = blockIdx.x * blockDim.x + threadIdx.x;
    if (m >= M) return;
    const int p = pos[m];
    tokens_in[m] = (p >= 0 && p < prompt_len[m] && p < max_prompt) ? prompt[(size_t)m * max_prompt + p] : sampled[m];
}
__global__ void record_generated_kernel(int* gen, const int* sampled, const int* prompt_len, const int* pos, int M,
                                        int max_new) {
    const int m = blockIdx.x * blockDim.x + threadIdx.x;
    if (m >= M) return;
    const int j = pos[m] - prompt_len[m];
    if (j >= 0 && j < max_new) gen[(size_t)m * max_new + j] = sampled[m];
}

// Greedy argmax of every row of logits [M][stride], with the candidate rule of the single-row kernel (start at
// (-1e38, 0), strict '>', lowest index on ties).  Optionally advances the per-sequence positions by one, which
// closes the decode step inside a CUDA graph.
constexpr int kBatchArgmaxBlocks = 64;
constexpr int kBatchArgmaxRows = 256;
__device__ unsigned long long g_bargmax_part[kBatchArgmaxRows][kBatchArgmaxBlocks];
__device__ unsigned int g_bargmax_ticket[kBatchArgmaxRows];

__device__ __forceinline__ unsigned int fkey(float f) {
    const unsigned int b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ unsigned long long cand(float v, int idx) {
    return ((unsigned long long)fkey(v) << 32) | (unsigned int)(0xFFFFFFFFu - (unsigned int)idx);
}
__device__ __forceinline__ unsigned long long bmax64(unsigned long long v, unsigned long long* sh) {
    const int t = threadIdx.x;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, v, o);
        v = other > v ? other : v;
    }
    __syncthreads();
    if ((t & 31) == 0) sh[t >> 5] = v;
    __syncthreads();
    if (t < 32) {
        unsigned long long w = t < (int)(blockDim.x >> 5) ? sh[t] : 0ull;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xffffffffu, w, o);
            w = other > w ? other : w;
        }
        if (t == 0) sh[0] = w;
    }
    __syncthreads();
    return sh[0];
}

__device__ __forceinline__ float fkey_inverse(unsigned int k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k);
}

// out_ids (may be null) receives the winning index; cand_out (may be null) the pair {value bits, index + index_offset}
// that a tensor-parallel caller exchanges instead of its slice of the logits.
__global__ void __launch_bounds__(256) argmax_batched_kernel(const float* logits, long stride, int vocab,
                                                             int* out_ids, int* seq_pos_to_advance, int pos_limit,
                                                             int2* cand_out, int index_offset) {
    __shared__ unsigned long long sh[32];
    __shared__ bool last;
    const int m = blockIdx.y;
    const float* row = logits + (size_t)m * stride;
    unsigned long long best = cand(-1e38f, 0);
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < vocab; i += gridDim.x * blockDim.x) {
        const float v = row[i];
        if (v > -1e38f) {
            const unsigned long long c = cand(v, i);
            best = c > best ? c : best;
        }
    }
    best = bmax64(best, sh);
    if (threadIdx.x == 0) {
        g_bargmax_part[m][blockIdx.x] = best;
        __threadfence();
        last = (atomicAdd(&g_bargmax_ticket[m], 1u) == gridDim.x - 1);
    }
    __syncthreads();
    if (!last) return;
    __threadfence();
    unsigned long long b2 = cand(-1e38f, 0);
    for (int i = threadIdx.x; i < (int)gridDim.x; i += blockDim.x) {
        const unsigned long long c = *((volatile unsigned long long*)&g_bargmax_part[m][i]);
        b2 = c > b2 ? c : b2;
    }
    b2 = bmax64(b2, sh);
    if (threadIdx.x == 0) {
        const int best_idx = (int)(0xFFFFFFFFu - (unsigned int)(b2 & 0xFFFFFFFFull));
        if (out_ids) out_ids[m] = best_idx;
        if (cand_out)
            cand_out[m] = make_int2(__float_as_int(fkey_inverse((unsigned int)(b2 >> 32))), best_idx + index_offset);
        g_bargmax_ticket[m] = 0;
        // positions stop at pos_limit (the last row of the cache), so a replayed step can never index past it
        if (seq_pos_to_advance && (pos_limit <= 0 || seq_pos_to_advance[m] < pos_limit)) seq_pos_to_advance[m] += 1;
    }
}

// Picks, for every sequence, the best of `world` candidates {value bits, global index} (largest value, lowest index on
// ties: the rule of the single-GPU argmax), writes the token id and advances the positions as the batched argmax does.
__global__ void __launch_bounds__(256) argmax_merge_kernel(const int2* cand_all, int world, int M, int* out_ids,
                                                           int* seq_pos_to_advance, int pos_limit) {
    const int m = blockIdx.x * blockDim.x + threadIdx.x;
    if (m >= M) return;
    unsigned long long best = 0ull;
    for (int r = 0; r < world; ++r) {
        const int2 c = cand_all[(size_t)r * M + m];
        const unsigned long long key = cand(__int_as_float(c.x), c.y);
        best = key > best ? key : best;
    }
    out_ids[m] = (int)(0xFFFFFFFFu - (unsigned int)(best & 0xFFFFFFFFull));
    if (seq_pos_to_advance && (pos_limit <= 0 || seq_pos_to_advance[m] < pos_limit)) seq_pos_to_advance[m] += 1;
}

}  // namespace bw

using namespace bw;

extern "C" int bw_qk_norm_rope_kv_f16(float* q_out, uint16_t* k_cache, uint16_t* v_cache, const float* qkv,
                                      const float* q_norm_w, const float* k_norm_w, const int* d_seq_pos,
                                      int num_q_heads, int num_kv_heads, int head_dim, int max_seq_len, int M,
                                      size_t kv_batch_elems, size_t kv_layer_elems, float eps, float rope_base,
                                      void* stream) {
    if (!q_out || !k_cache || !v_cache || !qkv || !q_norm_w || !k_norm_w || !d_seq_pos) return cudaErrorInvalidValue;
    if (head_dim != kHeadDim || num_q_heads < 1 || num_kv_heads < 1 || M < 1 || max_seq_len < 1)
        return cudaErrorInvalidValue;
    const int warps = M * (num_q_heads + 2 * num_kv_heads);
    cudaError_t le = launch_pdl(qk_norm_rope_kv_kernel, dim3((warps + 3) / 4), dim3(128), 0,
                                static_cast<cudaStream_t>(stream), q_out, reinterpret_cast<__half*>(k_cache),
                                reinterpret_cast<__half*>(v_cache), qkv, q_norm_w, k_norm_w, d_seq_pos, num_q_heads,
                                num_kv_heads, max_seq_len, M, kv_batch_elems, kv_layer_elems, eps, rope_base);
    count_launch(1);
    return le != cudaSuccess ? le : cudaPeekAtLastError();
}

extern "C" int bw_embed_gather_f16(float* x_out, const uint16_t* table_f16, const int* d_tokens, int H, int vocab,
                                   int M, void* stream) {
    if (!x_out || !table_f16 || !d_tokens || H < 8 || H % 8 != 0 || vocab < 1 || M < 1) return cudaErrorInvalidValue;
    const dim3 grid((H / 8 + 255) / 256, M);
    embed_gather_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        x_out, reinterpret_cast<const __half*>(table_f16), d_tokens, H, vocab);
    count_launch(1);
    return cudaPeekAtLastError();
}

extern "C" int bw_embed_gather_f32(float* x_out, const float* table_f32, const int* d_tokens, int H, int vocab, int M,
                                   void* stream) {
    if (!x_out || !table_f32 || !d_tokens || H < 4 || H % 4 != 0 || vocab < 1 || M < 1) return cudaErrorInvalidValue;
    const dim3 grid((H / 4 + 255) / 256, M);
    embed_gather_f32_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(x_out, table_f32, d_tokens, H, vocab);
    count_launch(1);
    return cudaPeekAtLastError();
}

extern "C" int bw_select_input_tokens(int* tokens_in, const int* sampled, const int* prompt, const int* prompt_len,
                                      const int* d_seq_pos, int M, int max_prompt, void* stream) {
    if (!tokens_in || !sampled || !prompt || !prompt_len || !d_seq_pos || M < 1 || max_prompt < 1)
        return cudaErrorInvalidValue;
    select_input_tokens_kernel<<<(M + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        tokens_in, sampled, prompt, prompt_len, d_seq_pos, M, max_prompt);
    count_launch(1);
    return cudaPeekAtLastError();
}

extern "C" int bw_record_generated(int* gen, const int* sampled, const int* prompt_len, const int* d_seq_pos, int M,
                                   int max_new, void* stream) {
    if (!gen || !sampled || !prompt_len || !d_seq_pos || M < 1 || max_new < 1) return cudaErrorInvalidValue;
    record_generated_kernel<<<(M + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(gen, sampled, prompt_len,
                                                                                           d_seq_pos, M, max_new);
    count_launch(1);
    return cudaPeekAtLastError();
}

extern "C" int bw_sample_argmax_batched(const float* logits, long row_stride, int vocab, int M, int* out_ids,
                                        int* seq_pos_to_advance_or_null, int pos_limit, void* stream) {
    if (!logits || !out_ids || vocab < 1 || M < 1 || M > kBatchArgmaxRows || row_stride < vocab)
        return cudaErrorInvalidValue;
    int blocks = (vocab + 256 * 8 - 1) / (256 * 8);
    if (blocks > kBatchArgmaxBlocks) blocks = kBatchArgmaxBlocks;
    const dim3 grid(blocks, M);
    argmax_batched_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(logits, row_stride, vocab, out_ids,
                                                                              seq_pos_to_advance_or_null, pos_limit,
                                                                              nullptr, 0);
    count_launch(1);
    return cudaPeekAtLastError();
}

extern "C" int bw_sample_argmax_candidates(const float* logits, long row_stride, int vocab, int M, int index_offset,
                                           int* cand_out_pairs, void* stream) {
    if (!logits || !cand_out_pairs || vocab < 1 || M < 1 || M > kBatchArgmaxRows || row_stride < vocab)
        return cudaErrorInvalidValue;
    int blocks = (vocab + 256 * 8 - 1) / (256 * 8);
    if (blocks > kBatchArgmaxBlocks) blocks = kBatchArgmaxBlocks;
    argmax_batched_kernel<<<dim3(blocks, M), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        logits, row_stride, vocab, nullptr, nullptr, 0, reinterpret_cast<int2*>(cand_out_pairs), index_offset);
    count_launch(1);
    return cudaPeekAtLastError();
}

extern "C" int bw_sample_argmax_merge(const int* cand_all_pairs, int world, int M, int* out_ids,
                                      int* seq_pos_to_advance_or_null, int pos_limit, void* stream) {
    if (!cand_all_pairs || !out_ids || world < 1 || M < 1) return cudaErrorInvalidValue;
    argmax_merge_kernel<<<(M + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const int2*>(cand_all_pairs), world, M, out_ids, seq_pos_to_advance_or_null, pos_limit);
    count_launch(1);
    return cudaPeekAtLastError();
}
