// Definitions of the reference's C++ entry points (namespace blackwell::kernels)
// for the decode path.  Each forwards to the C function of the same name.
#include "../../include/blackwell_b200_dropin.hpp"

#include "../../include/blackwell_b200.h"

namespace blackwell {
namespace kernels {

#define BW_ERR(expr) static_cast<cudaError_t>(expr)

cudaError_t gemv_int4_batched(float* y_out, const uint8_t* x_packed, const float* x_scale, const uint8_t* W_packed,
                              const float* W_scale, int K, int N, int M, cudaStream_t stream) {
    return BW_ERR(bw_gemv_int4_batched(y_out, x_packed, x_scale, W_packed, W_scale, K, N, M, stream));
}
cudaError_t gemv_int4_warp(float* y_out, const void* x_packed, const float* x_scale, const void* W_packed,
                           const float* W_scale, int K, int N, cudaStream_t stream) {
    return BW_ERR(bw_gemv_int4_warp(y_out, x_packed, x_scale, W_packed, W_scale, K, N, stream));
}
cudaError_t quantize_int4(void* x_out_packed, float* x_out_sc, const float* in_fp32, int K, cudaStream_t stream) {
    return BW_ERR(bw_quantize_int4(x_out_packed, x_out_sc, in_fp32, K, stream));
}
cudaError_t quantize_int4_batched(void* x_out_packed, float* x_out_sc, const float* in_fp32, int K, int M,
                                  cudaStream_t stream) {
    return BW_ERR(bw_quantize_int4_batched(x_out_packed, x_out_sc, in_fp32, K, M, stream));
}
cudaError_t quantize_int8(void* out_int8, float* out_scale, const float* in_fp32, int num_elements,
                          cudaStream_t stream) {
    return BW_ERR(bw_quantize_int8(out_int8, out_scale, in_fp32, num_elements, stream));
}
cudaError_t fused_rmsnorm_quant_int4(uint8_t* x_out_packed, float* x_out_scale, const float* proj,
                                     const float* weight, int N, float eps, cudaStream_t stream) {
    return BW_ERR(bw_fused_rmsnorm_quant_int4(x_out_packed, x_out_scale, proj, weight, N, eps, stream));
}
cudaError_t fused_swiglu_quant_int4(uint8_t* out_packed, float* out_scale, const float* gate, const float* up, int N,
                                    cudaStream_t stream) {
    return BW_ERR(bw_fused_swiglu_quant_int4(out_packed, out_scale, gate, up, N, stream));
}
cudaError_t fused_rmsnorm_batched(float* out, const float* inp, const float* weight, int H, float eps, int M,
                                  cudaStream_t stream) {
    return BW_ERR(bw_fused_rmsnorm_batched(out, inp, weight, H, eps, M, stream));
}
cudaError_t fused_rmsnorm(float* out, const float* inp, const float* weight, int num_elements, float eps,
                          cudaStream_t stream) {
    return BW_ERR(bw_fused_rmsnorm(out, inp, weight, num_elements, eps, stream));
}
cudaError_t fused_rope_decode(float* out_inplace, const float* cos_cache, const float* sin_cache,
                              const int* seq_pos_ptr, int heads, int head_dim, int max_seq_len, cudaStream_t stream) {
    return BW_ERR(bw_fused_rope_decode(out_inplace, cos_cache, sin_cache, seq_pos_ptr, heads, head_dim, max_seq_len,
                                       stream));
}
cudaError_t apply_swiglu(float* out, const float* gate, const float* up, int num_elements, cudaStream_t stream) {
    return BW_ERR(bw_apply_swiglu(out, gate, up, num_elements, stream));
}
cudaError_t vector_add_fp32(float* out, const float* a, const float* b, int num_elements, cudaStream_t stream) {
    return BW_ERR(bw_vector_add_fp32(out, a, b, num_elements, stream));
}
cudaError_t attention_decode_batched_gqa(float* output, const float* Q, const float* K_cache, const float* V_cache,
                                         int seq_pos, int num_q_heads, int num_kv_heads, int head_dim,
                                         int max_seq_len, int M, size_t kv_batch_elems, size_t kv_layer_elems,
                                         cudaStream_t stream) {
    return BW_ERR(bw_attention_decode_batched_gqa(output, Q, K_cache, V_cache, seq_pos, num_q_heads, num_kv_heads,
                                                  head_dim, max_seq_len, M, kv_batch_elems, kv_layer_elems, stream));
}
cudaError_t attention_decode_batched_gqa_device(float* output, const float* Q, const float* K_cache,
                                                const float* V_cache, const int* d_seq_pos, int num_q_heads,
                                                int num_kv_heads, int head_dim, int max_seq_len, int M,
                                                size_t kv_batch_elems, size_t kv_layer_elems, cudaStream_t stream) {
    return BW_ERR(bw_attention_decode_batched_gqa_device(output, Q, K_cache, V_cache, d_seq_pos, num_q_heads,
                                                         num_kv_heads, head_dim, max_seq_len, M, kv_batch_elems,
                                                         kv_layer_elems, stream));
}
cudaError_t update_kv_cache(float* k_cache, float* v_cache, const float* k_new, const float* v_new, int batch_idx,
                            int seq_pos, int num_heads, int head_dim, int max_seq_len, cudaStream_t stream) {
    return BW_ERR(bw_update_kv_cache(k_cache, v_cache, k_new, v_new, batch_idx, seq_pos, num_heads, head_dim,
                                     max_seq_len, stream));
}
cudaError_t update_kv_cache_device(float* k_cache, float* v_cache, const float* k_new, const float* v_new,
                                   int batch_idx, const int* d_seq_pos, int num_heads, int head_dim, int max_seq_len,
                                   cudaStream_t stream) {
    return BW_ERR(bw_update_kv_cache_device(k_cache, v_cache, k_new, v_new, batch_idx, d_seq_pos, num_heads,
                                            head_dim, max_seq_len, stream));
}
cudaError_t sample_argmax_gpu(const float* logits, int vocab, int* out_id, cudaStream_t stream) {
    return BW_ERR(bw_sample_argmax_gpu(logits, vocab, out_id, stream));
}
cudaError_t sample_gpu(const float* logits, int vocab, float temperature, int top_k, int* out_id,
                       unsigned long long rng_seed, int step, cudaStream_t stream) {
    return BW_ERR(bw_sample_gpu(logits, vocab, temperature, top_k, out_id, rng_seed, step, stream));
}
cudaError_t apply_repetition_penalty(float* logits, const int* recent, int num_recent, float penalty, int vocab,
                                     cudaStream_t stream) {
    return BW_ERR(bw_apply_repetition_penalty(logits, recent, num_recent, penalty, vocab, stream));
}

}  // namespace kernels
}  // namespace blackwell
