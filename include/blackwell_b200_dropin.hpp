// C++ face of libblackwell_kernels for callers written against the reference's
// include/blackwell/kernels.h: the same functions, in the same namespace, with
// the same parameter lists, so that objects compiled against that header link
// against this library without change (the link-level contract is the
// Itanium-mangled name).  Only the decode-path functions are provided; each is a
// thin forwarder to the C entry point of the same name in blackwell_b200.h.
//
// Differences a caller can observe: argument checks are a superset of the
// reference's (M > 16 and N % 16 != 0 are accepted by the GEMV); no call
// enqueues a host-to-device copy of seq_pos (it travels as a kernel argument);
// sample_gpu does not overwrite the logits and draws from its own
// counter-based generator, not cuRAND's stream.
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace blackwell {
namespace kernels {

// kernels.h:1290
cudaError_t gemv_int4_batched(float* y_out, const uint8_t* x_packed, const float* x_scale, const uint8_t* W_packed,
                              const float* W_scale, int K, int N, int M, cudaStream_t stream = 0);
// kernels.h:755
cudaError_t gemv_int4_warp(float* y_out, const void* x_packed, const float* x_scale, const void* W_packed,
                           const float* W_scale, int K, int N, cudaStream_t stream = 0);
// kernels.h:800, :810, :526
cudaError_t quantize_int4(void* x_out_packed, float* x_out_sc, const float* in_fp32, int K, cudaStream_t stream = 0);
cudaError_t quantize_int4_batched(void* x_out_packed, float* x_out_sc, const float* in_fp32, int K, int M,
                                  cudaStream_t stream = 0);
cudaError_t quantize_int8(void* out_int8, float* out_scale, const float* in_fp32, int num_elements,
                          cudaStream_t stream = 0);
// kernels.h:417, :819
cudaError_t fused_rmsnorm_quant_int4(uint8_t* x_out_packed, float* x_out_scale, const float* proj,
                                     const float* weight, int N, float eps, cudaStream_t stream = 0);
cudaError_t fused_swiglu_quant_int4(uint8_t* out_packed, float* out_scale, const float* gate, const float* up, int N,
                                    cudaStream_t stream = 0);
// kernels.h:117, :127, :145, :155, :164
cudaError_t fused_rmsnorm_batched(float* out, const float* inp, const float* weight, int H, float eps, int M,
                                  cudaStream_t stream = 0);
cudaError_t fused_rmsnorm(float* out, const float* inp, const float* weight, int num_elements, float eps,
                          cudaStream_t stream = 0);
cudaError_t fused_rope_decode(float* out_inplace, const float* cos_cache, const float* sin_cache,
                              const int* seq_pos_ptr, int heads, int head_dim, int max_seq_len,
                              cudaStream_t stream = 0);
cudaError_t apply_swiglu(float* out, const float* gate, const float* up, int num_elements, cudaStream_t stream = 0);
cudaError_t vector_add_fp32(float* out, const float* a, const float* b, int num_elements, cudaStream_t stream = 0);
// kernels.h:202, :218, :309, :322
cudaError_t attention_decode_batched_gqa(float* output, const float* Q, const float* K_cache, const float* V_cache,
                                         int seq_pos, int num_q_heads, int num_kv_heads, int head_dim,
                                         int max_seq_len, int M, size_t kv_batch_elems, size_t kv_layer_elems,
                                         cudaStream_t stream = 0);
cudaError_t attention_decode_batched_gqa_device(float* output, const float* Q, const float* K_cache,
                                                const float* V_cache, const int* d_seq_pos, int num_q_heads,
                                                int num_kv_heads, int head_dim, int max_seq_len, int M,
                                                size_t kv_batch_elems, size_t kv_layer_elems,
                                                cudaStream_t stream = 0);
cudaError_t update_kv_cache(float* k_cache, float* v_cache, const float* k_new, const float* v_new, int batch_idx,
                            int seq_pos, int num_heads, int head_dim, int max_seq_len, cudaStream_t stream = 0);
cudaError_t update_kv_cache_device(float* k_cache, float* v_cache, const float* k_new, const float* v_new,
                                   int batch_idx, const int* d_seq_pos, int num_heads, int head_dim, int max_seq_len,
                                   cudaStream_t stream = 0);
// kernels.h:1095, :1103, :1117
cudaError_t sample_argmax_gpu(const float* logits, int vocab, int* out_id, cudaStream_t stream = 0);
cudaError_t sample_gpu(const float* logits, int vocab, float temperature, int top_k, int* out_id,
                       unsigned long long rng_seed, int step, cudaStream_t stream = 0);
cudaError_t apply_repetition_penalty(float* logits, const int* recent, int num_recent, float penalty, int vocab,
                                     cudaStream_t stream = 0);

}  // namespace kernels
}  // namespace blackwell
