// Batched decode-step driver: the host side of the INT4 servers' token loop above the kernel entry points.
//
// It mirrors the reference's per-layer sequence (server/inference_server_int4_batched.cu:253-298: rmsnorm ->
// quantize -> q/k/v GEMV -> head norm, RoPE -> KV update -> attention -> quantize -> o GEMV -> residual -> rmsnorm ->
// quantize -> gate/up GEMV -> SwiGLU -> quantize -> down GEMV -> residual; then final norm, LM head, sampling) and the
// graph form of bench/decode_int4_cgraph_8b.cu:249-399 (stream capture, instantiate, launch per step), with the
// fusions of this library: 6 or 7 launches per layer for the whole batch, per-sequence positions and token bookkeeping in
// device memory, and ONE CUDA graph per step that is captured at creation and only replayed afterwards -- no
// allocation, no host-device synchronisation and no host decision inside a generation.
//
// Weights: a directory in the reference's container format (<l>_self_attn.q_proj.int4_t / .scale_t ..., see
// weight_files.cu) -- q, k, v are concatenated by rows into one matrix, gate and up likewise; the INT4 embedding is
// dequantized to fp32 once, as the reference does (:196-217).  Activation format: 8 = int8 activations with binary16
// weight scales (the fast path), 4 = the reference's own arithmetic (INT4 activations by the quantize_int4 rule, fp32
// weight scales).  The KV cache is binary16.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <new>
#include <string>
#include <vector>

#include "../../include/blackwell_b200.h"

namespace {

struct Mat {          // one (possibly concatenated) projection on the device
    int K = 0, N = 0;
    uint8_t* packed = nullptr;
    float* sc32 = nullptr;
    uint16_t* sc16 = nullptr;
};

struct Layer {
    Mat qkv, o, gu, down;
    float *rn_in = nullptr, *rn_post = nullptr, *qn = nullptr, *kn = nullptr;
};

}  // namespace

struct bw_decode {
    bw_decode_config cfg;
    std::vector<Layer> layers;
    Mat lm;
    float* rn_final = nullptr;
    float* embed = nullptr;  // fp32 [vocab][H]
    // state
    uint16_t *kc = nullptr, *vc = nullptr;
    float *x = nullptr, *qkv = nullptr, *q = nullptr, *attn = nullptr, *gu = nullptr, *logits = nullptr;
    int8_t* attn_q = nullptr;   // attention result block-16 quantized by the attention kernel (int8 mode, fused form)
    float* attn_qs = nullptr;
    // norm-pending hand-over (one sequence, int8 mode): the hidden state after O (a) and after down (b), quantized
    int8_t *pa_q = nullptr, *pb_q = nullptr;
    float *pa_s = nullptr, *pa_ss = nullptr, *pb_s = nullptr, *pb_ss = nullptr;
    int *tokens_in = nullptr, *sampled = nullptr, *pos = nullptr;
    int *prompt = nullptr, *prompt_len = nullptr, *gen = nullptr;
    int max_prompt = 0, max_new = 0;
    size_t kv_layer = 0, kv_batch = 0;
    cudaStream_t cap_stream = nullptr;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    std::vector<void*> owned;  // every device allocation, for teardown
    std::string error;
};

namespace {

#define BW_TRY(expr)                       \
    do {                                   \
        const int e_ = (int)(expr);        \
        if (e_ != 0) return e_;            \
    } while (0)

template <typename T>
int dev_alloc(bw_decode* d, T** p, size_t count) {
    void* v = nullptr;
    cudaError_t e = cudaMalloc(&v, count * sizeof(T) ? count * sizeof(T) : 1);
    if (e != cudaSuccess) return (int)e;
    d->owned.push_back(v);
    *p = static_cast<T*>(v);
    return 0;
}

template <typename T>
int upload(bw_decode* d, T** p, const std::vector<T>& h) {
    BW_TRY(dev_alloc(d, p, h.size()));
    return (int)cudaMemcpy(*p, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice);
}

uint16_t f32_to_f16_bits(float f) {
    const __half h = __float2half_rn(f);
    uint16_t b;
    memcpy(&b, &h, 2);
    return b;
}

// Reads the listed projections of one layer and uploads them stacked by rows.
int load_stacked(bw_decode* d, const std::string& dir, const std::vector<std::string>& names, int K_expect, Mat* out) {
    std::vector<uint8_t> packed;
    std::vector<float> scales;
    int N = 0;
    for (const std::string& nm : names) {
        const std::string prefix = dir + "/" + nm;
        int k = 0, n = 0;
        int e = bw_w4_file_dims(prefix.c_str(), &k, &n);
        if (e != 0) { d->error = "cannot read " + prefix + ".int4_t/.scale_t"; return e; }
        if (k != K_expect) { d->error = prefix + ": K does not match the model shape"; return -3; }
        const size_t pb = packed.size(), sb = scales.size();
        packed.resize(pb + (size_t)n * k / 2);
        scales.resize(sb + (size_t)n * (k / 16));
        e = bw_w4_file_read(prefix.c_str(), packed.data() + pb, scales.data() + sb, k, n);
        if (e != 0) { d->error = "cannot read " + prefix; return e; }
        N += n;
    }
    out->K = K_expect;
    out->N = N;
    BW_TRY(upload(d, &out->packed, packed));
    if (d->cfg.act_bits == 4) {
        BW_TRY(upload(d, &out->sc32, scales));
    } else {
        std::vector<uint16_t> h16(scales.size());
        for (size_t i = 0; i < scales.size(); ++i) h16[i] = f32_to_f16_bits(scales[i]);
        BW_TRY(upload(d, &out->sc16, h16));
    }
    return 0;
}

int load_f32(bw_decode* d, const std::string& path, size_t n, size_t offset, size_t total, float** out) {
    std::vector<float> h(total);
    const int e = bw_f32_file_read(path.c_str(), h.data(), total);
    if (e != 0) { d->error = "cannot read " + path; return e; }
    std::vector<float> part(h.begin() + offset, h.begin() + offset + n);
    return upload(d, out, part);
}

int load_model(bw_decode* d, const std::string& dir) {
    const bw_decode_config& c = d->cfg;
    const int H = c.hidden, Q = c.n_q_heads * 128, KV = c.n_kv_heads * 128, I = c.inter;
    d->layers.resize(c.layers);
    for (int l = 0; l < c.layers; ++l) {
        const std::string p = std::to_string(l) + "_";
        Layer& L = d->layers[l];
        BW_TRY(load_stacked(d, dir, {p + "self_attn.q_proj", p + "self_attn.k_proj", p + "self_attn.v_proj"}, H, &L.qkv));
        BW_TRY(load_stacked(d, dir, {p + "self_attn.o_proj"}, Q, &L.o));
        BW_TRY(load_stacked(d, dir, {p + "mlp.gate_proj", p + "mlp.up_proj"}, H, &L.gu));
        BW_TRY(load_stacked(d, dir, {p + "mlp.down_proj"}, I, &L.down));
        if (L.qkv.N != Q + 2 * KV || L.o.N != H || L.gu.N != 2 * I || L.down.N != H) {
            d->error = "layer " + std::to_string(l) + ": projection sizes do not match the model shape";
            return -3;
        }
        BW_TRY(load_f32(d, dir + "/" + p + "input_layernorm.f32", H, 0, H, &L.rn_in));
        BW_TRY(load_f32(d, dir + "/" + p + "post_attention_layernorm.f32", H, 0, H, &L.rn_post));
        // qk_norms.f32 holds, per layer, the q-head norm then the k-head norm (128 floats each)
        BW_TRY(load_f32(d, dir + "/qk_norms.f32", 128, (size_t)l * 256, (size_t)c.layers * 256, &L.qn));
        BW_TRY(load_f32(d, dir + "/qk_norms.f32", 128, (size_t)l * 256 + 128, (size_t)c.layers * 256, &L.kn));
    }
    BW_TRY(load_f32(d, dir + "/final_norm.f32", H, 0, H, &d->rn_final));
    BW_TRY(load_stacked(d, dir, {"lm_head"}, H, &d->lm));
    if (d->lm.N < c.vocab) { d->error = "lm_head has fewer rows than the vocabulary"; return -3; }
    // embedding: INT4 -> fp32 once, (nibble - 8) * scale
    {
        const std::string prefix = dir + "/embed_tokens";
        int k = 0, n = 0;
        int e = bw_w4_file_dims(prefix.c_str(), &k, &n);
        if (e != 0 || k != H || n < c.vocab) { d->error = "cannot use " + prefix; return e ? e : -3; }
        std::vector<uint8_t> packed((size_t)n * k / 2);
        std::vector<float> sc((size_t)n * (k / 16));
        e = bw_w4_file_read(prefix.c_str(), packed.data(), sc.data(), k, n);
        if (e != 0) { d->error = "cannot read " + prefix; return e; }
        std::vector<float> table((size_t)c.vocab * H);
        for (int r = 0; r < c.vocab; ++r)
            for (int kb = 0; kb < H / 16; ++kb) {
                const float s = sc[(size_t)r * (H / 16) + kb];
                for (int i = 0; i < 16; ++i) {
                    const uint8_t byte = packed[(size_t)r * H / 2 + (size_t)kb * 8 + i / 2];
                    const int nib = (i & 1) ? (byte >> 4) : (byte & 0x0F);
                    table[(size_t)r * H + kb * 16 + i] = (float)(nib - 8) * s;
                }
            }
        BW_TRY(upload(d, &d->embed, table));
    }
    return 0;
}

// y = W . quantize(prologue(x)) (+ residual) in the engine's activation format.
int gemv(const bw_decode* d, const Mat& W, float* y, const float* residual, const float* x, const float* up, long x_stride,
         const float* norm_w, int N_rows, cudaStream_t st) {
    const bw_decode_config& c = d->cfg;
    if (c.act_bits == 4)
        return bw_gemv_int4_decode(y, 0, residual, x, up, x_stride, norm_w, c.eps, W.packed, W.sc32, W.K, N_rows, c.batch, st);
    return bw_gemv_w4a8_decode(y, 0, residual, x, up, x_stride, norm_w, c.eps, W.packed, W.sc16, W.K, N_rows, c.batch, st);
}

// Enqueues one decode step for the whole batch.
int enqueue_step(bw_decode* d, cudaStream_t st) {
    const bw_decode_config& c = d->cfg;
    const int M = c.batch, H = c.hidden, nq = c.n_q_heads, nkv = c.n_kv_heads, I = c.inter;
    BW_TRY(bw_select_input_tokens(d->tokens_in, d->sampled, d->prompt, d->prompt_len, d->pos, M, d->max_prompt, st));
    BW_TRY(bw_embed_gather_f32(d->x, d->embed, d->tokens_in, H, c.vocab, M, st));
    // One sequence in int8 mode (at 5..16 the same hand-over measured no faster than the prep launches): the O and down projections hand their result to the next GEMV already quantized, so
    // that no CTA of the QKV / gate+up / LM-head GEMVs has to quantize the hidden state (bw_gemv_w4a8_pending).
    const bool pending = M == 1 && c.act_bits == 8 && (nq / nkv == 4 || nq / nkv == 8) && H % 16 == 0;
    auto pend = [&](float* y, const float* res, const Mat& W, int N, const int8_t* xq, const float* xs, const float* xss,
                    const float* gate, const float* up, const float* next_w, int8_t* nq_, float* ns, float* nss) {
        bw_gemv_pending_args g{};
        g.y = y; g.residual = res; g.x_q = xq; g.x_scale = xs; g.x_block_sumsq = xss; g.eps = c.eps;
        g.gate = gate; g.up = up; g.W_packed = W.packed; g.W_scale_f16 = W.sc16; g.K = W.K; g.N = N;
        g.next_norm_w = next_w; g.next_q = nq_; g.next_scale = ns; g.next_block_sumsq = nss;
        g.M = M; g.x_stride = gate ? 2 * (long)I : 0;
        return bw_gemv_w4a8_pending(&g, st);
    };
    for (int l = 0; l < c.layers; ++l) {
        const Layer& L = d->layers[l];
        const size_t off = (size_t)l * d->kv_layer;
        if (pending && l > 0)
            BW_TRY(pend(d->qkv, nullptr, L.qkv, L.qkv.N, d->pb_q, d->pb_s, d->pb_ss, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr));
        else
            BW_TRY(gemv(d, L.qkv, d->qkv, nullptr, d->x, nullptr, 0, L.rn_in, L.qkv.N, st));
        const bool fused = nq / nkv == 4 || nq / nkv == 8;
        const bool q8 = fused && c.act_bits == 8;   // the attention kernel quantizes its result for the O projection
        if (q8) {
            BW_TRY(bw_attention_decode_f16kv_fused_q8(nullptr, d->attn_q, d->attn_qs, d->qkv, L.qn, L.kn, d->kc, d->vc,
                                                      d->pos, c.max_seq, nq, nkv, 128, c.max_seq, M, d->kv_batch, off,
                                                      c.eps, c.rope_base, st));
        } else if (fused) {  // head norm + RoPE + KV write inside the tensor-core attention kernel
            BW_TRY(bw_attention_decode_f16kv_fused(d->attn, d->qkv, L.qn, L.kn, d->kc, d->vc, d->pos, c.max_seq, nq, nkv, 128,
                                                   c.max_seq, M, d->kv_batch, off, c.eps, c.rope_base, st));
        } else {
            BW_TRY(bw_qk_norm_rope_kv_f16(d->q, d->kc, d->vc, d->qkv, L.qn, L.kn, d->pos, nq, nkv, 128, c.max_seq, M,
                                          d->kv_batch, off, c.eps, c.rope_base, st));
            BW_TRY(bw_attention_decode_f16kv(d->attn, d->q, d->kc, d->vc, d->pos, c.max_seq, nq, nkv, 128, c.max_seq, M,
                                             d->kv_batch, off, st));
        }
        if (pending) {
            const float* next_w = l + 1 < c.layers ? d->layers[l + 1].rn_in : d->rn_final;
            BW_TRY(pend(d->x, d->x, L.o, H, d->attn_q, d->attn_qs, nullptr, nullptr, nullptr, L.rn_post, d->pa_q, d->pa_s, d->pa_ss));
            BW_TRY(pend(d->gu, nullptr, L.gu, 2 * I, d->pa_q, d->pa_s, d->pa_ss, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr));
            BW_TRY(pend(d->x, d->x, L.down, H, nullptr, nullptr, nullptr, d->gu, d->gu + I, next_w, d->pb_q, d->pb_s, d->pb_ss));
            continue;
        }
        if (q8)
            BW_TRY(bw_gemv_w4a8_q8_decode(d->x, 0, d->x, d->attn_q, d->attn_qs, L.o.packed, L.o.sc16, L.o.K, H, M, st));
        else
            BW_TRY(gemv(d, L.o, d->x, d->x, d->attn, nullptr, 0, nullptr, H, st));
        BW_TRY(gemv(d, L.gu, d->gu, nullptr, d->x, nullptr, 0, L.rn_post, 2 * I, st));
        BW_TRY(gemv(d, L.down, d->x, d->x, d->gu, d->gu + I, 2 * (long)I, nullptr, H, st));
    }
    if (pending)
        BW_TRY(pend(d->logits, nullptr, d->lm, c.vocab, d->pb_q, d->pb_s, d->pb_ss, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr));
    else
        BW_TRY(gemv(d, d->lm, d->logits, nullptr, d->x, nullptr, 0, d->rn_final, c.vocab, st));
    BW_TRY(bw_sample_argmax_batched(d->logits, c.vocab, c.vocab, M, d->sampled, d->pos, c.max_seq - 1, st));
    BW_TRY(bw_record_generated(d->gen, d->sampled, d->prompt_len, d->pos, M, d->max_new, st));
    return 0;
}

int alloc_state(bw_decode* d) {
    const bw_decode_config& c = d->cfg;
    const size_t M = c.batch, H = c.hidden;
    d->kv_layer = (size_t)c.n_kv_heads * c.max_seq * 128;
    d->kv_batch = (size_t)c.layers * d->kv_layer;
    BW_TRY(dev_alloc(d, &d->kc, M * d->kv_batch));
    BW_TRY(dev_alloc(d, &d->vc, M * d->kv_batch));
    BW_TRY(dev_alloc(d, &d->x, M * H));
    BW_TRY(dev_alloc(d, &d->qkv, M * (size_t)(c.n_q_heads + 2 * c.n_kv_heads) * 128));
    BW_TRY(dev_alloc(d, &d->q, M * (size_t)c.n_q_heads * 128));
    BW_TRY(dev_alloc(d, &d->attn, M * (size_t)c.n_q_heads * 128));
    BW_TRY(dev_alloc(d, &d->attn_q, M * (size_t)c.n_q_heads * 128));
    BW_TRY(dev_alloc(d, &d->attn_qs, M * (size_t)c.n_q_heads * 8));
    BW_TRY(dev_alloc(d, &d->pa_q, M * H));  BW_TRY(dev_alloc(d, &d->pb_q, M * H));
    BW_TRY(dev_alloc(d, &d->pa_s, M * (H / 16 + 1)));  BW_TRY(dev_alloc(d, &d->pa_ss, M * (H / 16 + 1)));
    BW_TRY(dev_alloc(d, &d->pb_s, M * (H / 16 + 1)));  BW_TRY(dev_alloc(d, &d->pb_ss, M * (H / 16 + 1)));
    BW_TRY(dev_alloc(d, &d->gu, M * 2 * (size_t)c.inter));
    BW_TRY(dev_alloc(d, &d->logits, M * (size_t)c.vocab));
    BW_TRY(dev_alloc(d, &d->tokens_in, M));
    BW_TRY(dev_alloc(d, &d->sampled, M));
    BW_TRY(dev_alloc(d, &d->pos, M));
    BW_TRY(dev_alloc(d, &d->prompt_len, M));
    d->max_prompt = c.max_prompt > 0 ? c.max_prompt : 1;
    d->max_new = c.max_new > 0 ? c.max_new : 1;
    BW_TRY(dev_alloc(d, &d->prompt, M * (size_t)d->max_prompt));
    BW_TRY(dev_alloc(d, &d->gen, M * (size_t)d->max_new));
    BW_TRY(cudaMemset(d->kc, 0, M * d->kv_batch * 2));
    BW_TRY(cudaMemset(d->vc, 0, M * d->kv_batch * 2));
    BW_TRY(cudaMemset(d->sampled, 0, M * 4));
    BW_TRY(cudaMemset(d->pos, 0, M * 4));
    BW_TRY(cudaMemset(d->prompt, 0, M * (size_t)d->max_prompt * 4));
    BW_TRY(cudaMemset(d->prompt_len, 0, M * 4));
    BW_TRY(cudaMemset(d->gen, 0, M * (size_t)d->max_new * 4));
    return 0;
}

}  // namespace

extern "C" int bw_decode_create(const bw_decode_config* cfg, bw_decode** out) {
    if (!cfg || !out) return cudaErrorInvalidValue;
    *out = nullptr;
    if (cfg->layers < 1 || cfg->hidden < 32 || cfg->hidden % 32 != 0 || cfg->inter < 32 || cfg->inter % 32 != 0 ||
        cfg->n_q_heads < 1 || cfg->n_kv_heads < 1 || cfg->n_q_heads % cfg->n_kv_heads != 0 || cfg->head_dim != 128 ||
        cfg->vocab < 1 || cfg->batch < 1 || cfg->batch > 256 || cfg->max_seq < 1 || !cfg->weights_dir ||
        (cfg->act_bits != 4 && cfg->act_bits != 8))
        return cudaErrorInvalidValue;
    bw_decode* d = new (std::nothrow) bw_decode();
    if (!d) return cudaErrorMemoryAllocation;
    d->cfg = *cfg;
    d->cfg.weights_dir = nullptr;  // not kept beyond this call
    int e = load_model(d, cfg->weights_dir);
    if (e == 0) e = alloc_state(d);
    // One eager step sizes the library's scratch memory (the capture below must not allocate), then the step is
    // captured once; afterwards bw_decode_step only replays the graph.
    if (e == 0) e = (int)cudaStreamCreateWithFlags(&d->cap_stream, cudaStreamNonBlocking);
    if (e == 0) e = enqueue_step(d, d->cap_stream);
    if (e == 0) e = (int)cudaStreamSynchronize(d->cap_stream);
    if (e == 0 && cfg->use_graph) {
        e = (int)cudaStreamBeginCapture(d->cap_stream, cudaStreamCaptureModeThreadLocal);
        if (e == 0) {
            const int se = enqueue_step(d, d->cap_stream);
            const int ee = (int)cudaStreamEndCapture(d->cap_stream, &d->graph);
            e = se ? se : ee;
        }
        if (e == 0) e = (int)cudaGraphInstantiate(&d->exec, d->graph, 0);
    }
    if (e == 0) e = (int)cudaMemset(d->pos, 0, (size_t)cfg->batch * 4);
    if (e == 0) e = (int)cudaDeviceSynchronize();
    if (e != 0) {
        if (!d->error.empty()) fprintf(stderr, "bw_decode_create: %s\n", d->error.c_str());
        bw_decode_destroy(d);
        return e;
    }
    *out = d;
    return 0;
}

extern "C" int bw_decode_begin(bw_decode* d, const int* prompt_ids, const int* prompt_len, int max_prompt, void* stream) {
    if (!d || !prompt_ids || !prompt_len || max_prompt < 1 || max_prompt > d->max_prompt) return cudaErrorInvalidValue;
    const int M = d->cfg.batch;
    for (int m = 0; m < M; ++m)
        if (prompt_len[m] < 1 || prompt_len[m] > max_prompt) return cudaErrorInvalidValue;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // the device-side table has rows of d->max_prompt ids
    std::vector<int> table((size_t)M * d->max_prompt, 0);
    for (int m = 0; m < M; ++m) memcpy(&table[(size_t)m * d->max_prompt], prompt_ids + (size_t)m * max_prompt, (size_t)max_prompt * 4);
    BW_TRY(cudaMemcpyAsync(d->prompt, table.data(), table.size() * 4, cudaMemcpyHostToDevice, st));
    BW_TRY(cudaMemcpyAsync(d->prompt_len, prompt_len, (size_t)M * 4, cudaMemcpyHostToDevice, st));
    BW_TRY(cudaMemsetAsync(d->pos, 0, (size_t)M * 4, st));
    BW_TRY(cudaMemsetAsync(d->gen, 0xFF, (size_t)M * d->max_new * 4, st));  // -1 = not generated
    return (int)cudaStreamSynchronize(st);  // the pageable host buffers above must outlive the copies
}

extern "C" int bw_decode_step(bw_decode* d, void* stream) {
    if (!d) return cudaErrorInvalidValue;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (d->exec) return (int)cudaGraphLaunch(d->exec, st);
    return enqueue_step(d, st);
}

extern "C" int bw_decode_result(bw_decode* d, int* gen_out, void* stream) {
    if (!d || !gen_out) return cudaErrorInvalidValue;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    BW_TRY(cudaMemcpyAsync(gen_out, d->gen, (size_t)d->cfg.batch * d->max_new * 4, cudaMemcpyDeviceToHost, st));
    return (int)cudaStreamSynchronize(st);
}

extern "C" int bw_decode_buffers(bw_decode* d, float** logits, float** hidden, int** positions, int** sampled,
                                 uint16_t** k_cache, uint16_t** v_cache) {
    if (!d) return cudaErrorInvalidValue;
    if (logits) *logits = d->logits;
    if (hidden) *hidden = d->x;
    if (positions) *positions = d->pos;
    if (sampled) *sampled = d->sampled;
    if (k_cache) *k_cache = d->kc;
    if (v_cache) *v_cache = d->vc;
    return 0;
}

extern "C" int bw_decode_destroy(bw_decode* d) {
    if (!d) return cudaErrorInvalidValue;
    cudaDeviceSynchronize();
    if (d->exec) cudaGraphExecDestroy(d->exec);
    if (d->graph) cudaGraphDestroy(d->graph);
    if (d->cap_stream) cudaStreamDestroy(d->cap_stream);
    for (void* p : d->owned) cudaFree(p);
    delete d;
    return 0;
}
