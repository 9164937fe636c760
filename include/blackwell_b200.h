/*
 * blackwell_b200.h -- C ABI of libblackwell_kernels (sm_100a only).
 *
 * The decode hot path of the reference engine -- the INT4 block-16 GEMV, its
 * activation quantizers, the RMSNorm / SwiGLU / residual glue, GQA decode
 * attention, KV-cache update and greedy sampling -- as hand-written CUDA for
 * B200.  Every entry point takes plain device pointers and sizes, enqueues its
 * work on the caller's stream (a cudaStream_t passed as void*; NULL = default
 * stream), never synchronises, and returns a cudaError_t value as int
 * (0 = cudaSuccess, 1 = cudaErrorInvalidValue for rejected arguments).
 *
 * "replaces" comments give the declaration in the reference's
 * include/blackwell/kernels.h (C++ `blackwell::kernels::<name>`) and the
 * definition in its src/kernels tree.  The C++ symbols of that header are also
 * exported by the library (see blackwell_b200_dropin.hpp), each forwarding to
 * the function of the same name here.
 *
 * Formats.  Weights: u8 [N][K/2], two offset-binary nibbles per byte (value =
 * nibble - 8, even k in the low nibble), one scale per 16 consecutive k.
 * INT4 activations use the same nibble format; INT8 activations are i8 [M][K].
 * Activation scales are f32 [M][K/16].  Outputs are f32 [M][N].
 */
#ifndef BLACKWELL_B200_H_
#define BLACKWELL_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ GEMV -- */

/* W4A4 GEMV, fp32 scales.  K % 16 == 0, M >= 1 (any M; the reference stops at 16
 * and also rejects N % 16 != 0 -- both are accepted here).
 * replaces gemv_int4_batched: kernels.h:1290-1299, src/kernels/gemv_int8.cu:913-1024 */
int bw_gemv_int4_batched(float* y_out, const uint8_t* x_packed, const float* x_scale, const uint8_t* W_packed,
                         const float* W_scale, int K, int N, int M, void* stream);

/* Same arithmetic, one sequence.
 * replaces gemv_int4_warp: kernels.h:755-763, src/kernels/gemv_int8.cu:481-535,881-900 */
int bw_gemv_int4_warp(float* y_out, const void* x_packed, const float* x_scale, const void* W_packed,
                      const float* W_scale, int K, int N, void* stream);

/* W4A8 GEMV: int8 activations (from bw_quantize_int8*), binary16 weight scales
 * (passed as uint16_t bit patterns).  Extension; arithmetic follows
 * src/kernels/gemv_int8.cu:937-965 with the int8 operand of :718-748.
 * Any M >= 1.  Batch routing of all bw_gemv_w4a8* entry points (by measurement; bw_set_tuning keys 5, 13, 14 move
 * the borders): up to 4 sequences run in the streaming dp4a kernel, 5 to 16 in the streaming mma.sync kernel, more
 * than 16 (K % 32 == 0, 16-byte aligned W and x) in the tcgen05 kernel, 64 sequences per launch; operands the
 * tensor-core kernel cannot take fall back to passes of 16 through the mma.sync kernel (or 8 through dp4a). */
int bw_gemv_w4a8(float* y_out, const int8_t* x_q, const float* x_scale, const uint8_t* W_packed,
                 const uint16_t* W_scale_f16, int K, int N, int M, void* stream);

/* W4A8 GEMV with the activation quantizer fused into the prologue: x is
 * binary16 [M][K].  K % 32 == 0, 16-byte aligned pointers; any M >= 1 (see the routing note above). */
int bw_gemv_w4a8_f16in(float* y_out, const uint16_t* x_f16, const uint8_t* W_packed, const uint16_t* W_scale_f16,
                       int K, int N, int M, void* stream);

/* Same with f32 activations and an optional RMSNorm (norm_weight != NULL):
 * y = W . q8(rmsnorm(x) ) -- fuses fused_rmsnorm (kernels.h:117-133) +
 * quantize_int8 (kernels.h:526-531) + the GEMV.  Same M rule as bw_gemv_w4a8_f16in. */
int bw_gemv_w4a8_f32in(float* y_out, const float* x_f32, const float* norm_weight, float eps,
                       const uint8_t* W_packed, const uint16_t* W_scale_f16, int K, int N, int M, void* stream);

/* y = W . q8(silu(gate) * up): fuses apply_swiglu (kernels.h:155-160) +
 * quantize_int8 + the GEMV (the down projection).  Same M rule as bw_gemv_w4a8_f16in. */
int bw_gemv_w4a8_swiglu(float* y_out, const float* gate, const float* up, const uint8_t* W_packed,
                        const uint16_t* W_scale_f16, int K, int N, int M, void* stream);

/* The W4A8 GEMV as the decode step uses it: f32 activations with a row stride (x_stride elements between
 * sequences; 0 = K), one of three fused prologues -- plain quantize, RMSNorm + quantize (norm_weight != NULL),
 * or SwiGLU + quantize (up != NULL, same stride as x) -- and an optional residual added to the result
 * (residual may alias y_out; both use y_stride, 0 = N).  It replaces, in one launch, the reference's
 * fused_rmsnorm / apply_swiglu + quantize + gemv + vector_add_fp32 sequences
 * (server/inference_server_int4_batched.cu:256-279).  Same M rule as bw_gemv_w4a8_f16in. */
int bw_gemv_w4a8_decode(float* y_out, long y_stride, const float* residual_or_null, const float* x_f32,
                        const float* up_or_null, long x_stride, const float* norm_weight_or_null, float eps,
                        const uint8_t* W_packed, const uint16_t* W_scale_f16, int K, int N, int M, void* stream);

/* bw_gemv_w4a8 with the output stride and residual epilogue of bw_gemv_w4a8_decode: pre-quantized int8 activations
 * [M][K] and scales [M][K/16] (from bw_quantize_int8*, or from bw_attention_decode_f16kv_fused_q8). */
int bw_gemv_w4a8_q8_decode(float* y_out, long y_stride, const float* residual_or_null, const int8_t* x_q,
                           const float* x_scale, const uint8_t* W_packed, const uint16_t* W_scale_f16, int K, int N,
                           int M, void* stream);

/* "Norm-pending" hand-over between two GEMVs of a decode step, at one sequence or 5..16 (no counterpart in the
 * reference).  The fused RMSNorm + quantize prologue makes every CTA of a GEMV quantize all M x K activations.  Here the
 * GEMV that PRODUCES those activations (O projection, down projection: y = residual + W x) also writes, from the 16
 * consecutive outputs a tile's epilogue holds, what the consumer's prologue would compute -- except the norm's scalar:
 *   next_q     i8  [N]     q8(y * next_norm_w), each 16-block with its own scale,
 *   next_scale f32 [N/16]  those scales (without the norm's 1/rms),
 *   next_block_sumsq f32 [N/16]  sum of y^2 per block,
 * and the CONSUMER (x_q = next_q, x_scale = next_scale, x_block_sumsq = next_block_sumsq, eps) sums the block sums in
 * fixed order, forms 1/rms and multiplies it into the scales: the integers of q8(y w / rms) do not depend on rms.  The
 * result differs from the fused prologue's only where a product lands on a rounding tie (one more float rounding).
 * A call is a producer (next_norm_w != NULL), a consumer (x_block_sumsq != NULL) or both.  Input: pre-quantized int8
 * (x_q, x_scale) or the SwiGLU pair (gate, up f32 [K], x_q == NULL; quantized once by a small kernel first).
 * Requirements (else cudaErrorInvalidValue): K % 32 == 0, N % 16 == 0 for a producer, 16-byte aligned operands, a shape
 * the dp4a streaming kernel takes whole. */
typedef struct {
    float* y;                       /* [N] */
    const float* residual;          /* [N] or NULL; may alias y */
    const int8_t* x_q;              /* [K] or NULL */
    const float* x_scale;           /* [K/16] */
    const float* x_block_sumsq;     /* [K/16] or NULL: norm pending on the input */
    float eps;
    const float* gate;              /* [K], with x_q == NULL */
    const float* up;                /* [K] */
    const uint8_t* W_packed;
    const uint16_t* W_scale_f16;
    int K, N;
    const float* next_norm_w;       /* [N] or NULL */
    int8_t* next_q;                 /* [N] */
    float* next_scale;              /* [N/16] */
    float* next_block_sumsq;        /* [N/16] */
    int M;                          /* sequences: 0 or 1 (dp4a kernel), or 5..16 (mma.sync kernel; every array above then
                                       has a leading dimension of M, y and residual [M][N], and a producer needs a K that
                                       the kernel prepares in one window: up to ~12,000 at 8 sequences) */
    long x_stride;                  /* elements between sequences of gate / up (0 = K) */
} bw_gemv_pending_args;
int bw_gemv_w4a8_pending(const bw_gemv_pending_args* args, void* stream);

/* Reference-format (W4A4, fp32 scales) GEMV with fused prologues: the int4
 * quantize rule of quantize_int4 (kernels.h:800-816) applied to x, to
 * rmsnorm(x) (norm_weight != NULL) or to silu(gate)*up (up != NULL).  M <= 8 (fp32 scales stay on the dp4a
 * kernel). */
int bw_gemv_int4_fused(float* y_out, const float* x_f32, const float* up_or_null, const float* norm_weight_or_null,
                       float eps, const uint8_t* W_packed, const float* W_scale, int K, int N, int M, void* stream);

/* The same reference-format GEMV as the decode step uses it: row strides and an optional residual, as
 * bw_gemv_w4a8_decode.  Any M. */
int bw_gemv_int4_decode(float* y_out, long y_stride, const float* residual_or_null, const float* x_f32,
                        const float* up_or_null, long x_stride, const float* norm_weight_or_null, float eps,
                        const uint8_t* W_packed, const float* W_scale, int K, int N, int M, void* stream);

/* Debug/inspection: per-block integer dot products of one sequence,
 * dots i32 [N][K/16], produced by the same unpack + dp4a code as the GEMVs.
 * x is INT4-packed (a8 == 0) or int8 (a8 != 0). */
int bw_gemv_block_dots(int32_t* dots, const void* x, int a8, const uint8_t* W_packed, int K, int N, void* stream);

/* ------------------------------------------------------------- quantizers -- */

/* replaces quantize_int4: kernels.h:800-805, src/kernels/gemv_int8.cu:1628-1683 */
int bw_quantize_int4(void* x_out_packed, float* x_out_sc, const float* in_fp32, int K, void* stream);
/* replaces quantize_int4_batched: kernels.h:810-816, src/kernels/gemv_int8.cu:1685-1704 */
int bw_quantize_int4_batched(void* x_out_packed, float* x_out_sc, const float* in_fp32, int K, int M, void* stream);
/* replaces quantize_int8: kernels.h:526-531, src/kernels/gemv_int8.cu:718-764 */
int bw_quantize_int8(void* out_int8, float* out_scale, const float* in_fp32, int num_elements, void* stream);
/* Extension: the same int8 rule on binary16 input. */
int bw_quantize_int8_f16(void* out_int8, float* out_scale, const uint16_t* in_f16, int num_elements, void* stream);
/* replaces fused_rmsnorm_quant_int4: kernels.h:417-424, src/kernels/fused_int4_ops.cu:155-242,335-358
 * (scale rule fmaxf(absmax/7, 1e-9), clamp +-7).  Correct for any N % 32 == 0. */
int bw_fused_rmsnorm_quant_int4(uint8_t* x_out_packed, float* x_out_scale, const float* proj, const float* weight,
                                int N, float eps, void* stream);
/* replaces fused_swiglu_quant_int4: kernels.h:819-825, src/kernels/fused_int4_ops.cu:254-389 */
int bw_fused_swiglu_quant_int4(uint8_t* out_packed, float* out_scale, const float* gate, const float* up, int N,
                               void* stream);

/* -------------------------------------------------- norm and elementwise -- */

/* replaces fused_rmsnorm: kernels.h:127-133, src/kernels/norm.cu:44-89,157-165.
 * All num_elements take part (the reference drops elements >= 4096). */
int bw_fused_rmsnorm(float* out, const float* inp, const float* weight, int num_elements, float eps, void* stream);
/* replaces fused_rmsnorm_batched: kernels.h:117-125, src/kernels/norm.cu:114-177 */
int bw_fused_rmsnorm_batched(float* out, const float* inp, const float* weight, int H, float eps, int M,
                             void* stream);
/* replaces apply_swiglu: kernels.h:155-160, src/kernels/norm.cu:94-106,179-189 */
int bw_apply_swiglu(float* out, const float* gate, const float* up, int num_elements, void* stream);
/* replaces vector_add_fp32: kernels.h:164-169, src/kernels/norm.cu:191-216 */
int bw_vector_add_fp32(float* out, const float* a, const float* b, int num_elements, void* stream);
/* replaces fused_rope_decode: kernels.h:145-153, src/kernels/rope.cu:160-239 */
int bw_fused_rope_decode(float* out_inplace, const float* cos_cache, const float* sin_cache, const int* seq_pos_ptr,
                         int heads, int head_dim, int max_seq_len, void* stream);

/* ---------------------------------------------------- KV cache, attention -- */

/* replaces update_kv_cache: kernels.h:309-319, src/kernels/decode.cu:27-46,590-618.
 * seq_pos is passed by value (no host-to-device copy is enqueued). */
int bw_update_kv_cache(float* k_cache, float* v_cache, const float* k_new, const float* v_new, int batch_idx,
                       int seq_pos, int num_heads, int head_dim, int max_seq_len, void* stream);
/* replaces update_kv_cache_device: kernels.h:322-332, src/kernels/decode.cu:620-639 */
int bw_update_kv_cache_device(float* k_cache, float* v_cache, const float* k_new, const float* v_new, int batch_idx,
                              const int* d_seq_pos, int num_heads, int head_dim, int max_seq_len, void* stream);
/* replaces attention_decode_batched_gqa: kernels.h:202-215, src/kernels/decode.cu:375-512.
 * head_dim must be 128.  Any seq_pos < max_seq_len (the reference caps the context at 3968). */
int bw_attention_decode_batched_gqa(float* output, const float* Q, const float* K_cache, const float* V_cache,
                                    int seq_pos, int num_q_heads, int num_kv_heads, int head_dim, int max_seq_len,
                                    int M, size_t kv_batch_elems, size_t kv_layer_elems, void* stream);
/* replaces attention_decode_batched_gqa_device: kernels.h:218-231, src/kernels/decode.cu:514-549 */
int bw_attention_decode_batched_gqa_device(float* output, const float* Q, const float* K_cache, const float* V_cache,
                                           const int* d_seq_pos, int num_q_heads, int num_kv_heads, int head_dim,
                                           int max_seq_len, int M, size_t kv_batch_elems, size_t kv_layer_elems,
                                           void* stream);

/* Extension: the same attention over a binary16 cache with one position per
 * sequence (d_seq_pos[M], device memory).  ctx_hint is an upper bound on
 * seq_pos + 1 used to size the context splits (0 = max_seq_len).  Arithmetic
 * follows src/kernels/decode.cu:431-465; strides are in cache elements. */
int bw_attention_decode_f16kv(float* output, const float* Q, const uint16_t* K_cache, const uint16_t* V_cache,
                              const int* d_seq_pos, int ctx_hint, int num_q_heads, int num_kv_heads, int head_dim,
                              int max_seq_len, int M, size_t kv_batch_elems, size_t kv_layer_elems, void* stream);

/* Batched decode glue, one launch for all M sequences with per-sequence positions in device memory.
 * Input: the fused QKV projection output qkv f32 [M][(nq + 2 nkv) * 128].  Query and key heads get the per-head
 * RMSNorm and the interleaved-pair RoPE (theta = pos * rope_base^(-2i/128)) of the reference's caller-side
 * kernels (server/inference_server_int4_batched.cu:49-70); queries go to q_out f32 [M][nq * 128]; keys and
 * values are written as binary16 into the cache rows at each sequence's position (the scatter of
 * update_kv_cache, src/kernels/decode.cu:27-46), cache addressed as in bw_attention_decode_f16kv. */
int bw_qk_norm_rope_kv_f16(float* q_out, uint16_t* k_cache, uint16_t* v_cache, const float* qkv,
                           const float* q_norm_w, const float* k_norm_w, const int* d_seq_pos, int num_q_heads,
                           int num_kv_heads, int head_dim, int max_seq_len, int M, size_t kv_batch_elems,
                           size_t kv_layer_elems, float eps, float rope_base, void* stream);
/* x_out f32 [M][H] = table_f16[d_tokens[m]][:] -- the embedding lookup the reference does with a host-side
 * copy (server/inference_server_int4_batched.cu:251), token ids read from device memory.  H % 8 == 0. */
int bw_embed_gather_f16(float* x_out, const uint16_t* table_f16, const int* d_tokens, int H, int vocab, int M,
                        void* stream);
/* The same lookup from an fp32 table (the form the reference keeps its dequantized embedding in,
 * server/inference_server_int4_batched.cu:196-217).  H % 4 == 0. */
int bw_embed_gather_f32(float* x_out, const float* table_f32, const int* d_tokens, int H, int vocab, int M,
                        void* stream);
/* Token bookkeeping of a batched generation that stays on the GPU (the reference decides on the host, one sequence at
 * a time: server/inference_server_int4_batched.cu:248-250, 295-299).  Sequence m consumes, at position
 * d_seq_pos[m], the id prompt[m][pos] while pos < prompt_len[m] and the previously sampled id afterwards
 * (bw_select_input_tokens); after sampling has advanced the position to p, a token beyond the prompt is stored as
 * generated token p - prompt_len[m] of gen i32 [M][max_new] (bw_record_generated). */
int bw_select_input_tokens(int* tokens_in, const int* sampled, const int* prompt, const int* prompt_len,
                           const int* d_seq_pos, int M, int max_prompt, void* stream);
int bw_record_generated(int* gen, const int* sampled, const int* prompt_len, const int* d_seq_pos, int M, int max_new,
                        void* stream);
/* Greedy argmax of each row of logits f32 [M][row_stride] (rule of sample_argmax_gpu,
 * src/kernels/sample_gpu.cu:30-60) into out_ids[M]; when seq_pos_to_advance is not NULL each of its M entries
 * is incremented, which closes a decode step inside a CUDA graph -- but never beyond pos_limit (pass
 * max_seq_len - 1; <= 0 means no limit), so that a replayed graph cannot push a position past the end of the
 * KV cache.  M <= 256. */
int bw_sample_argmax_batched(const float* logits, long row_stride, int vocab, int M, int* out_ids,
                             int* seq_pos_to_advance_or_null, int pos_limit, void* stream);
/* Tensor-parallel form of the greedy argmax (the reference is single-GPU: no counterpart): every rank reduces its
 * own vocabulary slice to one candidate per sequence, cand_out_pairs int32 [M][2] = {bits of the best value,
 * index + index_offset}; the ranks exchange these 8-byte pairs (an all-gather into [world][M][2]) instead of the
 * logits, and bw_sample_argmax_merge picks the winner per sequence -- largest value, lowest index on ties, the
 * single-GPU rule -- into out_ids and advances the positions like bw_sample_argmax_batched. */
int bw_sample_argmax_candidates(const float* logits, long row_stride, int vocab, int M, int index_offset,
                                int* cand_out_pairs, void* stream);
int bw_sample_argmax_merge(const int* cand_all_pairs, int world, int M, int* out_ids,
                           int* seq_pos_to_advance_or_null, int pos_limit, void* stream);

/* bw_qk_norm_rope_kv_f16 + bw_attention_decode_f16kv in ONE launch: qkv f32 [M][(nqh + 2 nkv) * 128] is the output
 * of the fused QKV projection; every CTA norms and rotates its own query heads, and the CTA whose context split
 * holds the sequence's position norms, rotates and stores that position's K row and stores its V row before
 * streaming the cache (a position outside the cache is not written).  Only for the shapes the tensor-core kernel
 * takes -- binary16 cache, 4 or 8 query heads per kv head -- otherwise cudaErrorInvalidValue.  Replaces, with the
 * attention call, head_norm_kernel / apply_rope_kernel / update_kv_cache of
 * server/inference_server_int4_batched.cu:49-70,262-266. */
int bw_attention_decode_f16kv_fused(float* output, const float* qkv, const float* q_norm_w, const float* k_norm_w,
                                    uint16_t* K_cache, uint16_t* V_cache, const int* d_seq_pos, int ctx_hint,
                                    int num_q_heads, int num_kv_heads, int head_dim, int max_seq_len, int M,
                                    size_t kv_batch_elems, size_t kv_layer_elems, float eps, float rope_base,
                                    void* stream);

/* The same launch with the result also (or only: output_or_null == NULL) block-16 quantized to int8 by the rule of
 * bw_quantize_int8 -- out_q8 i8 [M][num_q_heads][128], out_scale f32 [M][num_q_heads][8] -- which is what the O
 * projection takes as pre-quantized activations (bw_gemv_w4a8_q8_decode), so that no CTA of that GEMV has to
 * quantize them.  Same bits as quantizing the float result.  No counterpart in the reference. */
int bw_attention_decode_f16kv_fused_q8(float* output_or_null, int8_t* out_q8, float* out_scale, const float* qkv,
                                       const float* q_norm_w, const float* k_norm_w, uint16_t* K_cache,
                                       uint16_t* V_cache, const int* d_seq_pos, int ctx_hint, int num_q_heads,
                                       int num_kv_heads, int head_dim, int max_seq_len, int M, size_t kv_batch_elems,
                                       size_t kv_layer_elems, float eps, float rope_base, void* stream);

/* Attention for callers that must not allocate.  No counterpart in the reference: it exists for hosts
 * that cannot reach the CUDA allocator once they are serving -- a process that has given all device memory
 * to its own pool, or one that runs with allocation switched off or audited after start-up.  Arguments,
 * arithmetic and results are those of bw_attention_decode_batched_gqa_device; the per-split partial results
 * live in a fixed 2 MiB array inside the library image (every GPU that loads the library carries it until
 * exit) instead of a buffer obtained from cudaMalloc, and the call makes no cudaMalloc, cudaFree or other
 * allocating call.
 *   Limit: M * num_q_heads * splits * 130 floats must fit in 524,288 floats, where splits =
 *   min(64, ceil(max_seq_len / 64), ceil(2 * SMs / (M * num_kv_heads))) re-derived after rounding the split
 *   length up to a multiple of 4; larger problems are rejected with cudaErrorInvalidValue and a message on
 *   stderr.  On a 148-SM B200 every 32-query-head / 8-kv-head shape fits; with 64 query heads over
 *   8 kv heads, batches of 32 to 36 sequences at long context do not.
 *   The first call on each device looks up the device address of the array (cudaGetSymbolAddress, with that
 *   device current); make that first call outside any stream capture.
 *   All calls share the array and it keeps the previous call's contents (none of it needs clearing: every
 *   record read is written earlier in the same call).  Two calls whose kernels overlap on one GPU -- different
 *   streams -- race on it; keep them on one stream or order them. */
int bw_attention_decode_batched_gqa_noalloc(float* output, const float* Q, const float* K_cache,
                                            const float* V_cache, const int* d_seq_pos, int num_q_heads,
                                            int num_kv_heads, int head_dim, int max_seq_len, int M,
                                            size_t kv_batch_elems, size_t kv_layer_elems, void* stream);

/* ----------------------------------------------------------------- sampling -- */

/* replaces sample_argmax_gpu: kernels.h:1095-1099, src/kernels/sample_gpu.cu:30-60,250-254 */
int bw_sample_argmax_gpu(const float* logits, int vocab, int* out_id, void* stream);
/* replaces sample_gpu: kernels.h:1103-1111, src/kernels/sample_gpu.cu:256-330.
 * temperature < 0.01 = greedy argmax; otherwise temperature/top-k sampling. */
int bw_sample_gpu(const float* logits, int vocab, float temperature, int top_k, int* out_id,
                  unsigned long long rng_seed, int step, void* stream);
/* replaces apply_repetition_penalty: kernels.h:1117-1123, src/kernels/decode.cu:694-731 */
int bw_apply_repetition_penalty(float* logits, const int* recent, int num_recent, float penalty, int vocab,
                                void* stream);

/* ------------------------------------------------------------------ service -- */

/* Reads (and clears) the device status word: 0 = ok, 1 = a kernel gave up on a
 * bounded wait for a bulk copy.  Synchronises the device. */
int bw_device_status(int* status_out);
/* ---- Weight container of the INT4 servers ----
 * <prefix>.int4_t = int32 header [K, N, 16, K/16, 1] + N*K/2 bytes of nibbles; <prefix>.scale_t = int32 header
 * [0, 0, 0, K/16, N] + N*(K/16) float32; <name>.f32 = raw float32.  Writer in the reference:
 * better-inference/gguf_convert.cpp:62-88; reader: upload_w4, server/inference_server_int4_batched.cu:32-45.
 * Return 0 on success; -1 cannot open, -2 file shorter/longer than its header says, -3 inconsistent header,
 * -4 bad argument, -5 write failed; the upload may also return a (positive) cudaError_t. */
int bw_w4_file_write(const char* prefix, const uint8_t* packed, const float* scales, int K, int N);
int bw_w4_file_dims(const char* prefix, int* K_out, int* N_out);
int bw_w4_file_read(const char* prefix, uint8_t* packed_out, float* scales_out, int K, int N);
/* One projection in device memory: the reference's DevW4 {K, N, d, sc} (server/inference_server_int4_batched.cu:31)
 * plus the binary16 copy of the scales that the bw_gemv_w4a8* entry points take.  bw_w4_file_upload reads the two
 * files, allocates with cudaMalloc and copies (a load-time call: it synchronises); bw_w4_free releases. */
typedef struct bw_dev_w4 {
    int K, N;
    uint8_t* packed;      /* [N][K/2] */
    float* scale_f32;     /* [N][K/16] or NULL */
    uint16_t* scale_f16;  /* [N][K/16] binary16 bit patterns, or NULL */
} bw_dev_w4;
int bw_w4_file_upload(const char* prefix, int want_f32_scales, int want_f16_scales, bw_dev_w4* out);
int bw_w4_free(bw_dev_w4* w);
int bw_f32_file_write(const char* path, const float* data, size_t n);
int bw_f32_file_read(const char* path, float* data_out, size_t n);

/* ---- Batched decode-step driver ----
 * The host side of the INT4 servers' token loop above the kernel entry points: it mirrors the per-layer sequence of
 * server/inference_server_int4_batched.cu:253-298 and the captured-graph form of
 * bench/decode_int4_cgraph_8b.cu:249-399 (capture :268, instantiate :332, launch :347) for a whole batch with
 * per-sequence positions.  bw_decode_create loads a weight directory in the reference's container format (the file
 * names of load_model, server/inference_server_int4_batched.cu:150-184), allocates a binary16 KV cache of
 * batch x max_seq positions, runs one step eagerly (which sizes the library's scratch memory) and captures the step
 * in a CUDA graph (use_graph != 0); it synchronises and allocates, the calls after it do neither except where
 * stated.  act_bits 8: int8 activations, binary16 weight scales (the fast path); act_bits 4: the reference's own
 * arithmetic (quantize_int4 rule, fp32 weight scales).
 * A generation: bw_decode_begin uploads prompt_ids i32 [batch][max_prompt] and prompt_len[batch] (host memory;
 * 1 <= len <= max_prompt <= cfg.max_prompt), resets the positions to 0 and synchronises the stream; every
 * bw_decode_step then advances all sequences by one token (it feeds the prompt while it lasts, then the sampled
 * ids, greedy) with no host decision -- max(prompt_len) + max_new - 1 steps complete the longest sequence;
 * bw_decode_result copies gen i32 [batch][cfg.max_new] to the host (-1 = not generated) and synchronises.
 * bw_decode_buffers exposes the device buffers (logits f32 [batch][vocab], hidden state, positions, sampled ids,
 * caches [batch][layers][kv_heads][max_seq][128]) for inspection.  One stream at a time per engine. */
typedef struct bw_decode bw_decode;
typedef struct bw_decode_config {
    int layers, hidden, inter, n_q_heads, n_kv_heads, head_dim, vocab;
    float eps, rope_base;
    int batch, max_seq;       /* sequences per step; cache positions per sequence */
    int max_prompt, max_new;  /* capacity of the device-side prompt and result tables */
    int act_bits;             /* 8 or 4 */
    int use_graph;            /* capture the step once and replay it */
    const char* weights_dir;  /* read during bw_decode_create only */
} bw_decode_config;
int bw_decode_create(const bw_decode_config* cfg, bw_decode** out);
int bw_decode_begin(bw_decode* d, const int* prompt_ids, const int* prompt_len, int max_prompt, void* stream);
int bw_decode_step(bw_decode* d, void* stream);
int bw_decode_result(bw_decode* d, int* gen_out, void* stream);
int bw_decode_buffers(bw_decode* d, float** logits, float** hidden, int** positions, int** sampled,
                      uint16_t** k_cache, uint16_t** v_cache);
int bw_decode_destroy(bw_decode* d);

/* ---- Tensor-parallel exchange over peer memory (no counterpart in the reference, which is single-GPU) ----
 * All-reduce of the K-split projections' partial sums across the GPUs of one box through NVLink peer loads.
 * bw_peer_comm_create allocates this rank's region on the current device (two slots of slot_bytes; the GEMV writes
 * its partial sums into bw_peer_comm_slot(comm, slot) directly).  Between processes the 64-byte handle from
 * bw_peer_comm_handle is passed to every peer's bw_peer_comm_open; inside one process bw_peer_comm_attach links two
 * communicators instead (on two devices with peer access, or on one and the same device).  bw_peer_allreduce_f32 (n % 4 == 0, n * 4 <= slot_bytes, 16-byte aligned out/residual)
 * enqueues one kernel: signal, bounded wait (~2 s, then status 3 from bw_peer_comm_status and no result), sum of
 * every rank's slot in rank order (+ residual) into out.  Every rank must issue the same sequence of calls with
 * alternating slot (0, 1, 0, ...); creation and teardown synchronise the device, the all-reduce itself allocates
 * nothing and may be captured in a CUDA graph. */
int bw_peer_comm_create(int world, int rank, size_t slot_bytes, void** comm_out);
int bw_peer_comm_handle(void* comm, void* handle_out_64);
int bw_peer_comm_open(void* comm, int peer_rank, const void* handle_64);
int bw_peer_comm_attach(void* comm, int peer_rank, void* peer_comm_same_process);
float* bw_peer_comm_slot(void* comm, int slot);
int bw_peer_allreduce_f32(void* comm, int slot, float* out, const float* residual_or_null, size_t n, void* stream);
int bw_peer_comm_status(void* comm, int* status_out);
int bw_peer_comm_destroy(void* comm);

/* Library-owned scratch memory.  Two kernel families keep a per-device, grow-only scratch block: the tensor-core
 * GEMV (float-input calls from 2 sequences on: activations quantized once; more than 16 sequences: prepared activations, K-split partial sums, arrival
 * counters) and the allocating attention entry points (split partials, arrival counters).  A block is shared by all
 * streams of the device -- two calls of the same family must not overlap on one GPU -- and grows (cudaMalloc +
 * cudaMemset, synchronising) when a larger problem arrives; an outgrown block stays allocated until the library is
 * unloaded, because launches already enqueued or captured in a CUDA graph still point at it.  A call that would
 * have to grow while its stream is being captured fails with cudaErrorStreamCaptureUnsupported.  To keep the
 * serving path free of allocations, reserve the largest sizes once at start-up: bw_gemv_scratch_bytes /
 * bw_attention_scratch_bytes give upper bounds for a shape (take the maximum over the shapes in use).  No
 * counterpart in the reference, whose kernels need no scratch. */
size_t bw_gemv_scratch_bytes(int M, int N, int K);
size_t bw_attention_scratch_bytes(int M, int num_q_heads, int num_kv_heads, int max_context);
int bw_reserve_scratch(size_t gemv_bytes, size_t attention_bytes);

/* Tuning knobs for experiments: key 0 = ring stages (0 = automatic),
 * key 1 = CTAs per SM cap (0 = automatic), key 2 = force the plain-load kernel,
 * key 3 = rows per thread group and tile cap, key 4 = threads per CTA target,
 * key 5 = smallest batch sent to the tensor-core kernel (0 = default 8), key 6 = its K-split (0 = automatic),
 * key 8 = programmatic dependent launch on (1, default) / off (0), key 9 = tensor-core attention kernel
 * for the binary16 cache on (1, default) / off (0: scalar kernel, for comparison runs), key 10 = smallest vector in
 * KiB that the peer all-reduce sums in two steps on four or more ranks (0 = default 4096), key 11 = longest wait of
 * the peer all-reduce for another rank in milliseconds (0 = default, about 2000), key 12 = 32-k columns per slab of
 * the mma.sync streaming kernel (0 = default 64), keys 13 / 14 = smallest / largest batch it takes (0 = defaults 3 and
 * 16; a smallest batch above 16 switches it off), key 15 = its ring stages (0 = automatic), key 16 = shrink the
 * small-batch kernel's ring to the tiles a CTA has (1, default) or not (0), key 17 = timing experiments on the
 * mma.sync kernel (0 = off; 1 = skip its arithmetic, 2 = skip its copies: results are then meaningless), key 18 =
 * its packed form for up to 4 sequences on (1, default) / off (0), key 19 = timing experiments on the tcgen05
 * kernel (0 = off; bits: 1 no epilogue arithmetic, 2 no unpack, 4 no weight loads, 8 no MMAs, 16 / 32 no activation /
 * activation-scale copies, 64 no weight-scale loads: results are then meaningless), key 20 = smallest batch whose
 * float activations are quantized once by a separate kernel before a streaming GEMV (0 = default 2), key 21 = the
 * same for the SwiGLU prologue (0 = default 1), key 22 = decode attention: the earlier split rule with pct % of the SMs
 * as CTA slots (0 = default rule: one wave of two CTAs per SM, at least 224 positions per split). */
int bw_set_tuning(int key, int value);
/* Number of kernels launched by this library since the last call with reset != 0. */
long long bw_launch_count(int reset);
/* Library version, for load checks. */
int bw_version(void);

#ifdef __cplusplus
}
#endif
#endif /* BLACKWELL_B200_H_ */
