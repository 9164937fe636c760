// GQA decode attention (one new token per sequence) and KV-cache update.
//
// Cache layout (caller's): element type f32 (reference format) or binary16
// (extension), addressed as
//   base + m * kv_batch_elems + kv_layer_elems + kv_head * max_seq * 128 + t * 128.
//
// Flash-decoding structure: the context of every (sequence, kv head) is cut
// into splits so that the grid fills the GPU at small batch; a CTA streams its
// K and V rows once and serves all the query heads that share the kv head
// (GQA), keeping an online-softmax state per head; per-split partial results
// go to a scratch buffer and a second small kernel merges them.  head_dim is
// 128 (32 lanes x 4 elements).
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdio.h>

#include <mutex>

#include "../../include/blackwell_b200.h"
#include "attention_mma.cuh"
#include "common.cuh"
#include "host_util.h"
#include "quant_rules.cuh"
#include "rope_norm.cuh"

namespace bw {

constexpr int kHd = 128;
constexpr int kAttnWarps = 4;
constexpr int kPosPerStep = 4;  // positions handled together by one warp

__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __half* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
    return make_float4(a.x, a.y, b.x, b.y);
}

struct AttnArgs {
    float* out;            // [M][nqh][128]
    const float* Q;        // [M][nqh][128]
    const void* K;
    const void* V;
    const int* d_seq_pos;  // device positions (shared or per sequence) or nullptr
    int seq_pos;           // host value when d_seq_pos == nullptr
    int per_seq;           // d_seq_pos has M entries
    int nqh, nkv, max_seq, M;
    size_t kv_batch_elems, kv_layer_elems;
    int nsplit, split_len;
    float scale;
    float* part;           // [M][nqh][nsplit][130] when nsplit > 1
    unsigned int* tickets; // [M][nkv] arrival counters (zero between calls): the last split CTA merges; or nullptr
    // fused form (tensor-core kernel only): Q, and the K / V rows of the new position, come straight from the QKV
    // projection output [M][(nqh + 2 nkv) * 128]; qkv == nullptr selects the plain form
    const float* qkv;
    const float* q_norm_w;
    const float* k_norm_w;
    float eps, rope_base;
    // optional second output (tensor-core kernel): the result block-16 quantized to int8 with the reference's rule,
    // i8 [M][nqh][128] + f32 scales [M][nqh][8] -- what the O projection's GEMV takes as pre-quantized activations
    int8_t* out_q;
    float* out_qs;
};

// Final outputs of one head, four consecutive dimensions per lane (whole warp): float and / or quantized.
__device__ __forceinline__ void emit_head4(const AttnArgs& a, size_t head, int lane, float4 v) {
    if (a.out) *reinterpret_cast<float4*>(a.out + head * 128 + 4 * lane) = v;
    if (a.out_q) {
        float am = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
        am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 1));
        am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 2));
        const float sc = quant_scale_i8(am);
        const uint32_t q = (uint32_t)(quant_i8(v.x, sc) & 255) | ((uint32_t)(quant_i8(v.y, sc) & 255) << 8) |
                           ((uint32_t)(quant_i8(v.z, sc) & 255) << 16) | ((uint32_t)(quant_i8(v.w, sc) & 255) << 24);
        *reinterpret_cast<uint32_t*>(a.out_q + head * 128 + 4 * lane) = q;
        if ((lane & 3) == 0) a.out_qs[head * 8 + (lane >> 2)] = sc;
    }
}
// The same for one dimension per thread (16 consecutive lanes hold one block).
__device__ __forceinline__ void emit_head1(const AttnArgs& a, size_t head, int d, float v) {
    if (a.out) a.out[head * 128 + d] = v;
    if (a.out_q) {
        float am = fabsf(v);
#pragma unroll
        for (int o = 1; o < 16; o <<= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
        const float sc = quant_scale_i8(am);
        a.out_q[head * 128 + d] = (int8_t)quant_i8(v, sc);
        if ((d & 15) == 0) a.out_qs[head * 8 + (d >> 4)] = sc;
    }
}

// Partial record of one (sequence, head, split): 128 un-normalised outputs, then max and sum.
constexpr int kPartStride = kHd + 2;

// With arrival counters the CTA that finishes a (sequence, kv head) last merges all its splits itself; no second
// launch.  One warp per head: lanes first run over the splits (maxima, weights, sum), then over the 128 outputs,
// four each, with the split weights broadcast by shuffle; every record load is independent.  Called by all
// threads of the CTA after its own partial records are written.
template <int GQ>
__device__ __forceinline__ void last_arriver_merge(const AttnArgs& a, int m, int kvh, int h0, int* s_last) {
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    __threadfence();
    __syncthreads();
    if (t == 0) *s_last = (atomicAdd(&a.tickets[m * a.nkv + kvh], 1u) == (unsigned)a.nsplit - 1) ? 1 : 0;
    __syncthreads();
    if (!*s_last) return;
    __threadfence();
    for (int h = warp; h < GQ; h += kAttnWarps) {
        const size_t head = (size_t)m * a.nqh + h0 + h;
        const float* base = a.part + head * a.nsplit * kPartStride;
        // Every load is an L2 round trip, so all of them are requested up front: the (max, sum) pairs of up to 64 splits
        // (two per lane) and the first sixteen records; with four records at a time and the pairs read twice, the merge
        // of ~32 splits took longer than streaming the cache.  Records of empty splits hold zeros and get weight 0.
        float ms[2], ls[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int sp = min(lane + 32 * r, a.nsplit - 1);
            ms[r] = __ldcg(base + (size_t)sp * kPartStride + kHd);
            ls[r] = lane + 32 * r < a.nsplit ? __ldcg(base + (size_t)sp * kPartStride + kHd + 1) : 0.f;
        }
        float2 r0[16], r1[16];
        auto load_batch = [&](int j0) {
#pragma unroll
            for (int jj = 0; jj < 16; ++jj) {
                const float* rec = base + (size_t)min(j0 + jj, a.nsplit - 1) * kPartStride + 4 * lane;  // clamped: weight 0
                r0[jj] = __ldcg(reinterpret_cast<const float2*>(rec));
                r1[jj] = __ldcg(reinterpret_cast<const float2*>(rec + 2));
            }
        };
        load_batch(0);
        float mloc = -FLT_MAX;
#pragma unroll
        for (int r = 0; r < 2; ++r)
            if (ls[r] > 0.f) mloc = fmaxf(mloc, ms[r]);
        const float mall = warp_max(mloc);
        float c[2], lsum = 0.f;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            c[r] = ls[r] > 0.f ? __expf(ms[r] - mall) : 0.f;
            lsum = fmaf(ls[r], c[r], lsum);
        }
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j0 = 0; j0 < a.nsplit; j0 += 16) {
            if (j0 > 0) load_batch(j0);
#pragma unroll
            for (int jj = 0; jj < 16; ++jj) {
                const int j = j0 + jj;   // warp-uniform
                const float cj = j < a.nsplit ? __shfl_sync(0xffffffffu, j < 32 ? c[0] : c[1], j & 31) : 0.f;
                acc.x = fmaf(cj, r0[jj].x, acc.x); acc.y = fmaf(cj, r0[jj].y, acc.y);
                acc.z = fmaf(cj, r1[jj].x, acc.z); acc.w = fmaf(cj, r1[jj].y, acc.w);
            }
        }
        lsum = warp_sum(lsum);
        const float inv = 1.0f / (lsum + 1e-9f);
        emit_head4(a, head, lane, make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv));
    }
    if (t == 0) a.tickets[m * a.nkv + kvh] = 0;
}

template <typename KVT, int GQ>
__global__ void __launch_bounds__(kAttnWarps * 32) attn_decode_split_kernel(const AttnArgs a) {
    const int split = blockIdx.x, kvh = blockIdx.y, m = blockIdx.z;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    pdl_trigger();
    pdl_wait();  // Q, the cache rows of this step and the positions come from the kernels before
    const int seq_pos = a.d_seq_pos ? a.d_seq_pos[a.per_seq ? m : 0] : a.seq_pos;
    const int npos = min(seq_pos + 1, a.max_seq);
    const int p0 = split * a.split_len;
    // The last split runs to the sequence's own end: the split length is sized from a hint of the context, and a
    // sequence that has grown past the hint must still see all its positions.
    const int p1 = split == a.nsplit - 1 ? npos : min(npos, p0 + a.split_len);

    const KVT* Kb = static_cast<const KVT*>(a.K) + (size_t)m * a.kv_batch_elems + a.kv_layer_elems +
                    (size_t)kvh * a.max_seq * kHd;
    const KVT* Vb = static_cast<const KVT*>(a.V) + (size_t)m * a.kv_batch_elems + a.kv_layer_elems +
                    (size_t)kvh * a.max_seq * kHd;
    const int h0 = kvh * GQ;  // first query head of the group (head * nkv / nqh == kvh)

    __shared__ float s_scores[kAttnWarps][kPosPerStep * GQ];
    __shared__ float s_m[kAttnWarps][GQ], s_l[kAttnWarps][GQ];
    __shared__ float s_o[kAttnWarps][GQ][kHd];

    float4 q[GQ];
#pragma unroll
    for (int h = 0; h < GQ; ++h) {
        q[h] = load4(a.Q + ((size_t)m * a.nqh + h0 + h) * kHd + 4 * lane);
        q[h].x *= a.scale; q[h].y *= a.scale; q[h].z *= a.scale; q[h].w *= a.scale;
    }
    float mx[GQ], l[GQ];
    float4 o[GQ];
#pragma unroll
    for (int h = 0; h < GQ; ++h) {
        mx[h] = -FLT_MAX; l[h] = 0.f; o[h] = make_float4(0.f, 0.f, 0.f, 0.f);
    }

    for (int tb = p0 + warp * kPosPerStep; tb < p1; tb += kAttnWarps * kPosPerStep) {
        float4 kr[kPosPerStep], vr[kPosPerStep];
#pragma unroll
        for (int j = 0; j < kPosPerStep; ++j) {
            const int tt = min(tb + j, p1 - 1);  // clamped rows are masked below
            kr[j] = load4(Kb + (size_t)tt * kHd + 4 * lane);
            vr[j] = load4(Vb + (size_t)tt * kHd + 4 * lane);
        }
        float partial[kPosPerStep * GQ];
#pragma unroll
        for (int j = 0; j < kPosPerStep; ++j)
#pragma unroll
            for (int h = 0; h < GQ; ++h)
                partial[j * GQ + h] = q[h].x * kr[j].x + q[h].y * kr[j].y + q[h].z * kr[j].z + q[h].w * kr[j].w;
        const float tot = warp_sum_many<kPosPerStep * GQ>(partial, lane);
        constexpr int V = kPosPerStep * GQ;  // 4, 8, 16 or 32: already a power of two
        if ((lane & (32 / V - 1)) == 0) s_scores[warp][warp_sum_many_index<V>(lane)] = tot;
        __syncwarp();
#pragma unroll
        for (int h = 0; h < GQ; ++h) {
            float s[kPosPerStep];
            float mnew = mx[h];
#pragma unroll
            for (int j = 0; j < kPosPerStep; ++j) {
                s[j] = (tb + j < p1) ? s_scores[warp][j * GQ + h] : -FLT_MAX;
                mnew = fmaxf(mnew, s[j]);
            }
            const float corr = __expf(mx[h] - mnew);
            float psum = 0.f;
            float4 acc = make_float4(o[h].x * corr, o[h].y * corr, o[h].z * corr, o[h].w * corr);
#pragma unroll
            for (int j = 0; j < kPosPerStep; ++j) {
                const float p = (tb + j < p1) ? __expf(s[j] - mnew) : 0.f;
                psum += p;
                acc.x = fmaf(p, vr[j].x, acc.x); acc.y = fmaf(p, vr[j].y, acc.y);
                acc.z = fmaf(p, vr[j].z, acc.z); acc.w = fmaf(p, vr[j].w, acc.w);
            }
            o[h] = acc;
            l[h] = l[h] * corr + psum;
            mx[h] = mnew;
        }
        __syncwarp();
    }

    __shared__ int s_last;
    // Combines the four warps' online-softmax states; writes the final output or this split's partial record.
    auto merge_warps_and_emit = [&](bool final_out) {
#pragma unroll
        for (int h = 0; h < GQ; ++h) {
            if (lane == 0) { s_m[warp][h] = mx[h]; s_l[warp][h] = l[h]; }
            *reinterpret_cast<float4*>(&s_o[warp][h][4 * lane]) = o[h];
        }
        __syncthreads();
        for (int idx = t; idx < GQ * kHd; idx += blockDim.x) {
            const int h = idx / kHd, d = idx - h * kHd;
            float mm = -FLT_MAX;
#pragma unroll
            for (int w = 0; w < kAttnWarps; ++w) mm = fmaxf(mm, s_m[w][h]);
            float ls = 0.f, os = 0.f;
#pragma unroll
            for (int w = 0; w < kAttnWarps; ++w) {
                const float c = __expf(s_m[w][h] - mm);
                ls = fmaf(s_l[w][h], c, ls);
                os = fmaf(s_o[w][h][d], c, os);
            }
            const size_t head = (size_t)m * a.nqh + h0 + h;
            if (final_out) {
                a.out[head * kHd + d] = os * (1.0f / (ls + 1e-9f));
            } else {
                float* rec = a.part + (head * a.nsplit + split) * kPartStride;
                rec[d] = os;
                if (d == 0) { rec[kHd] = mm; rec[kHd + 1] = ls; }
            }
        }
    };
    merge_warps_and_emit(a.nsplit == 1);

    if (a.nsplit > 1 && a.tickets) last_arriver_merge<GQ>(a, m, kvh, h0, &s_last);
}

// Tensor-core variant for the binary16 cache (see attention_mma.cuh): same grid, same splits, same partial records
// and arrival counters as the scalar kernel above.
template <int GQ>
__global__ void __launch_bounds__(kAttnWarps * 32) attn_decode_mma_kernel(const AttnArgs a) {
    const int split = blockIdx.x, kvh = blockIdx.y, m = blockIdx.z;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    extern __shared__ __align__(128) unsigned char attn_dsm[];   // 4 warps x (K, V) x 2 buffers x 4 KB
    const int p0 = split * a.split_len;
    const __half* Kb = static_cast<const __half*>(a.K) + (size_t)m * a.kv_batch_elems + a.kv_layer_elems +
                       (size_t)kvh * a.max_seq * kHd;
    const __half* Vb = static_cast<const __half*>(a.V) + (size_t)m * a.kv_batch_elems + a.kv_layer_elems +
                       (size_t)kvh * a.max_seq * kHd;
    pdl_trigger();
    // Fused form: the cache rows below this step's position were written by earlier steps, so every warp requests its
    // first tile before waiting for the kernel before (whose QKV output and position this kernel needs): the tile's
    // DRAM latency then overlaps that wait and the query prologue.  Which rows are usable is decided after the wait.
    const bool early = a.qkv != nullptr && warp * amma::kTile < a.split_len && p0 + warp * amma::kTile < a.max_seq;
    if (early)
        amma::issue_tile(Kb, Vb, smem_u32(attn_dsm + warp * amma::kWarpSmem), 0, p0 + warp * amma::kTile, a.max_seq - 1);
    pdl_wait();
    const int seq_pos = a.d_seq_pos ? a.d_seq_pos[a.per_seq ? m : 0] : a.seq_pos;
    const int npos = min(seq_pos + 1, a.max_seq);
    // The last split runs to the sequence's own end: the split length is sized from a hint of the context, and a
    // sequence that has grown past the hint must still see all its positions.
    const int p1 = split == a.nsplit - 1 ? npos : min(npos, p0 + a.split_len);
    const int h0 = kvh * GQ;

    __shared__ __align__(16) float s_q[GQ][kHd];
    __shared__ float s_m[kAttnWarps][GQ], s_l[kAttnWarps][GQ];
    __shared__ int s_last;
    // The per-warp results reuse the warp's own K/V staging area once its stream has drained.
    auto s_o = [&](int w, int h) { return reinterpret_cast<float*>(attn_dsm + w * amma::kWarpSmem) + h * kHd; };
    if (a.qkv == nullptr) {
        for (int i = t; i < GQ * kHd; i += blockDim.x) s_q[i / kHd][i % kHd] = a.Q[((size_t)m * a.nqh + h0) * kHd + i];
    } else {
        // Fused head norm + RoPE + cache write (what bw_qk_norm_rope_kv_f16 does in a launch of its own): every CTA
        // norms and rotates its own query heads; the CTA whose split holds the new position also norms and rotates that
        // position's K row, converts its V row, stores both in the cache and then streams them like any other row.
        const int heads = a.nqh + 2 * a.nkv;
        const float* row = a.qkv + (size_t)m * heads * kHd;
        for (int h = warp; h < GQ; h += kAttnWarps) {
            float4 v = *reinterpret_cast<const float4*>(row + (size_t)(h0 + h) * kHd + 4 * lane);
            v = head_norm_rope(v, a.q_norm_w, a.eps, seq_pos, a.rope_base, lane);
            *reinterpret_cast<float4*>(&s_q[h][4 * lane]) = v;
        }
        if (seq_pos >= p0 && seq_pos < p1 && seq_pos < a.max_seq && warp < 2) {
            __half* Kw = const_cast<__half*>(Kb) + (size_t)seq_pos * kHd + 4 * lane;
            __half* Vw = const_cast<__half*>(Vb) + (size_t)seq_pos * kHd + 4 * lane;
            if (warp == 0) {
                float4 v = *reinterpret_cast<const float4*>(row + (size_t)(a.nqh + kvh) * kHd + 4 * lane);
                store_half4(Kw, head_norm_rope(v, a.k_norm_w, a.eps, seq_pos, a.rope_base, lane));
            } else {
                store_half4(Vw, *reinterpret_cast<const float4*>(row + (size_t)(a.nqh + a.nkv + kvh) * kHd + 4 * lane));
            }
            __threadfence();  // the rows are read back through cp.async (L2) by all four warps
        }
    }
    __syncthreads();

    float m_run, l_run, o[32];
    // rows that were final when the early tile was requested: all below this step's position (and inside the split)
    amma::warp_stream<GQ>(Kb, Vb, &s_q[0][0], a.scale, p0, p1, warp, kAttnWarps, attn_dsm + warp * amma::kWarpSmem,
                          m_run, l_run, o, early, min(p1, seq_pos));
    {
        const int g = lane >> 2, tq = lane & 3;
        if (g < GQ) {
            if (tq == 0) { s_m[warp][g] = m_run; s_l[warp][g] = l_run; }
#pragma unroll
            for (int jn = 0; jn < 16; ++jn)
                *reinterpret_cast<float2*>(s_o(warp, g) + 8 * jn + 2 * tq) = make_float2(o[2 * jn], o[2 * jn + 1]);
        }
    }
    __syncthreads();
    for (int idx = t; idx < GQ * kHd; idx += blockDim.x) {
        const int h = idx / kHd, d = idx - h * kHd;
        float mm = -FLT_MAX;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) mm = fmaxf(mm, s_m[w][h]);
        float ls = 0.f, os = 0.f;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) {
            const float c = __expf(s_m[w][h] - mm);
            ls = fmaf(s_l[w][h], c, ls);
            os = fmaf(s_o(w, h)[d], c, os);
        }
        const size_t head = (size_t)m * a.nqh + h0 + h;
        if (a.nsplit == 1) {
            emit_head1(a, head, d, os * (1.0f / (ls + 1e-9f)));
        } else {
            float* rec = a.part + (head * a.nsplit + split) * kPartStride;
            rec[d] = os;
            if (d == 0) { rec[kHd] = mm; rec[kHd + 1] = ls; }
        }
    }
    if (a.nsplit > 1 && a.tickets) last_arriver_merge<GQ>(a, m, kvh, h0, &s_last);
}

// Merges the per-split partial records of one (sequence, head).
__global__ void __launch_bounds__(kHd) attn_merge_kernel(float* out, const float* part, int nsplit) {
    const size_t head = blockIdx.x;
    const int d = threadIdx.x;
    const float* rec = part + head * nsplit * kPartStride;
    float mm = -FLT_MAX;
    for (int s = 0; s < nsplit; ++s) mm = fmaxf(mm, rec[s * kPartStride + kHd]);
    float ls = 0.f, os = 0.f;
    for (int s = 0; s < nsplit; ++s) {
        const float lsp = rec[s * kPartStride + kHd + 1];
        if (lsp > 0.f) {
            const float c = __expf(rec[s * kPartStride + kHd] - mm);
            ls = fmaf(lsp, c, ls);
            os = fmaf(rec[s * kPartStride + d], c, os);
        }
    }
    out[head * kHd + d] = os * (1.0f / (ls + 1e-9f));
}

// Scatter of the new K and V rows into the cache [head][max_seq][head_dim] at
// the position given by value or read from device memory.
template <typename KVT>
__global__ void __launch_bounds__(256) update_kv_kernel_b200(KVT* kc, KVT* vc, const float* k_new,
                                                             const float* v_new, const int* d_pos, int pos_value,
                                                             int nh, int hd, int max_seq) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= nh * hd) return;
    const int pos = d_pos ? *d_pos : pos_value;
    if ((unsigned)pos >= (unsigned)max_seq) return;  // a position outside the cache is never written
    const int h = idx / hd, d = idx - h * hd;
    const size_t off = (size_t)h * max_seq * hd + (size_t)pos * hd + d;
    kc[off] = (KVT)k_new[idx];
    vc[off] = (KVT)v_new[idx];
}

// ------------------------------------------------------------------ host side
static int g_attn_mma = 1;  // 0: keep the scalar kernel for the binary16 cache too (comparison runs)
void set_attn_mma(int v) { g_attn_mma = v; }
// Per-device scratch for the split partials and arrival counters.
static GrowScratch g_attn_scratch;
cudaError_t attn_reserve_scratch(size_t bytes) {
    unsigned char* p = nullptr;
    return bytes ? g_attn_scratch.get(bytes, (size_t)4 << 20, nullptr, &p) : cudaSuccess;
}

// Number of context splits; the grid is (sequence, kv head) pairs x splits.  Measured on a B200 (32 / 8 heads, binary16
// cache; a launch in a chain of its own kind and inside the 8B-shape decode step): the fastest grid is ONE wave of about
// two CTAs per SM -- an SM streams ~50 GB/s, so fewer CTAs cannot pull the bandwidth (8 sequences x 8 kv heads at 2048
// positions: unsplit 40.6 us, 4 splits 20.3 us), while a second wave or splits shorter than ~224 positions cost more in
// partial records, arrival counters and merges than they gain (the same case with 9 splits: 28.4 us; batch 1 at ctx
// 2048 inside the decode step: 1.90 ms per step with 33 splits of 62 positions, 1.84 ms with 9 of 228).  So: the largest
// split count whose grid still fits one wave, at least 224 positions per split, at most 64 splits.
// `bw_set_tuning(22, pct)` selects the earlier rule instead (smallest count whose last wave of pct % x SMs slots is 90 %
// full, 64 positions per split at least).
static int g_attn_slots_pct = 0;
void set_attn_slots_pct(int v) { g_attn_slots_pct = v > 0 ? v : 0; }
static int choose_splits(int pairs, int ctx, int sms) {
    if (g_attn_slots_pct > 0) {
        const int slots = g_attn_slots_pct * sms / 100 > 0 ? g_attn_slots_pct * sms / 100 : 1;
        int max_split = (ctx + 63) / 64;
        if (max_split > 64) max_split = 64;
        int lo = (slots + pairs - 1) / pairs;
        if (lo > max_split) lo = max_split;
        if (lo < 1) lo = 1;
        int best = lo;
        double best_eff = 0.0;
        for (int n = lo; n <= max_split && n <= lo + 16; ++n) {
            const long ctas = (long)pairs * n;
            const long waves = (ctas + slots - 1) / slots;
            const double eff = (double)ctas / (double)(waves * slots);
            if (eff >= 0.9) return n;
            if (eff > best_eff) { best_eff = eff; best = n; }
        }
        return best;
    }
    int n = 2 * sms / pairs;                        // one wave of two CTAs per SM
    const int by_len = ctx / 224;                   // at least 224 positions per split
    if (n > by_len) n = by_len;
    if (n > 64) n = 64;
    return n < 1 ? 1 : n;
}

// The arrival counters live in a region of fixed size at the front of the scratch block that nothing else ever
// uses: they must read zero at the start of every call (the last arriver leaves them so), and a region whose size
// followed the problem would let one call's partial records lie where a later, larger call expects its counters.
constexpr size_t kTicketBytes = 65536;   // 16,384 (sequence, kv head) pairs; beyond that the context is not split

// Upper bound of the scratch a call with up to M sequences and a context hint up to ctx can need.
size_t attn_scratch_bytes(int M, int nqh, int nkv, int ctx) {
    if (M < 1 || nqh < 1 || nkv < 1 || ctx < 1) return 0;
    return kTicketBytes + (size_t)M * nqh * 64 * kPartStride * sizeof(float);  // at most 64 splits
}

template <typename KVT>
static cudaError_t attn_launch(AttnArgs a, int ctx_hint, cudaStream_t st) {
    if ((!a.out && !a.out_q) || (!a.Q && !a.qkv) || !a.K || !a.V || a.nqh < 1 || a.nkv < 1 || a.nqh % a.nkv != 0 || a.M < 1 || a.max_seq < 1)
        return cudaErrorInvalidValue;
    const int gq = a.nqh / a.nkv;
    if (gq != 1 && gq != 2 && gq != 4 && gq != 8) return cudaErrorInvalidValue;
    if (ctx_hint < 1) ctx_hint = 1;
    if (ctx_hint > a.max_seq) ctx_hint = a.max_seq;
    const bool use_mma = sizeof(KVT) == 2 && (gq == 4 || gq == 8) && (g_attn_mma || a.qkv);  // binary16 cache with grouped heads
    if ((a.qkv || a.out_q) && !use_mma) return cudaErrorInvalidValue;  // these forms exist in the tensor-core kernel only
    int nsplit = choose_splits(a.M * a.nkv, ctx_hint, sm_count(current_device()));
    if ((size_t)a.M * a.nkv * sizeof(unsigned int) > kTicketBytes) nsplit = 1;  // thousands of pairs fill the GPU unsplit
    a.split_len = (ctx_hint + nsplit - 1) / nsplit;
    a.split_len = (a.split_len + kPosPerStep - 1) / kPosPerStep * kPosPerStep;
    nsplit = (ctx_hint + a.split_len - 1) / a.split_len;
    a.nsplit = nsplit;
    a.scale = 1.0f / sqrtf((float)kHd);
    a.part = nullptr;
    a.tickets = nullptr;
    if (nsplit > 1) {
        // scratch = [arrival counters, one per (sequence, kv head)] [partial records]
        const size_t tick_bytes = kTicketBytes;
        unsigned char* base = nullptr;
        cudaError_t e = g_attn_scratch.get(tick_bytes + (size_t)a.M * a.nqh * nsplit * kPartStride * sizeof(float),
                                           (size_t)4 << 20, st, &base);
        if (e != cudaSuccess) return e;
        a.tickets = reinterpret_cast<unsigned int*>(base);
        a.part = reinterpret_cast<float*>(base + tick_bytes);
    }
    const dim3 grid(nsplit, a.nkv, a.M);
    cudaError_t le;
    if (use_mma) {  // the tensor-core kernel
        const size_t dsm = (size_t)kAttnWarps * amma::kWarpSmem;
        static std::once_flag once[kMaxDevices];
        std::call_once(once[current_device()], [&] {
            cudaFuncSetAttribute(attn_decode_mma_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dsm);
            cudaFuncSetAttribute(attn_decode_mma_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dsm);
        });
        le = gq == 4 ? launch_pdl(attn_decode_mma_kernel<4>, grid, dim3(kAttnWarps * 32), dsm, st, a)
                     : launch_pdl(attn_decode_mma_kernel<8>, grid, dim3(kAttnWarps * 32), dsm, st, a);
        count_launch(1);
        return le != cudaSuccess ? le : cudaPeekAtLastError();
    }
    switch (gq) {
        case 1: le = launch_pdl(attn_decode_split_kernel<KVT, 1>, grid, dim3(kAttnWarps * 32), 0, st, a); break;
        case 2: le = launch_pdl(attn_decode_split_kernel<KVT, 2>, grid, dim3(kAttnWarps * 32), 0, st, a); break;
        case 4: le = launch_pdl(attn_decode_split_kernel<KVT, 4>, grid, dim3(kAttnWarps * 32), 0, st, a); break;
        default: le = launch_pdl(attn_decode_split_kernel<KVT, 8>, grid, dim3(kAttnWarps * 32), 0, st, a); break;
    }
    count_launch(1);
    return le != cudaSuccess ? le : cudaPeekAtLastError();
}

}  // namespace bw

using namespace bw;

extern "C" int bw_attention_decode_batched_gqa(float* output, const float* Q, const float* K_cache,
                                               const float* V_cache, int seq_pos, int num_q_heads, int num_kv_heads,
                                               int head_dim, int max_seq_len, int M, size_t kv_batch_elems,
                                               size_t kv_layer_elems, void* stream) {
    if (head_dim != kHd || seq_pos < 0 || seq_pos >= max_seq_len) return cudaErrorInvalidValue;
    AttnArgs a{};
    a.out = output; a.Q = Q; a.K = K_cache; a.V = V_cache; a.d_seq_pos = nullptr; a.seq_pos = seq_pos; a.per_seq = 0;
    a.nqh = num_q_heads; a.nkv = num_kv_heads; a.max_seq = max_seq_len; a.M = M;
    a.kv_batch_elems = kv_batch_elems; a.kv_layer_elems = kv_layer_elems;
    return attn_launch<float>(a, seq_pos + 1, static_cast<cudaStream_t>(stream));
}

extern "C" int bw_attention_decode_batched_gqa_device(float* output, const float* Q, const float* K_cache,
                                                      const float* V_cache, const int* d_seq_pos, int num_q_heads,
                                                      int num_kv_heads, int head_dim, int max_seq_len, int M,
                                                      size_t kv_batch_elems, size_t kv_layer_elems, void* stream) {
    if (head_dim != kHd || !d_seq_pos) return cudaErrorInvalidValue;
    AttnArgs a{};
    a.out = output; a.Q = Q; a.K = K_cache; a.V = V_cache; a.d_seq_pos = d_seq_pos; a.per_seq = 0;
    a.nqh = num_q_heads; a.nkv = num_kv_heads; a.max_seq = max_seq_len; a.M = M;
    a.kv_batch_elems = kv_batch_elems; a.kv_layer_elems = kv_layer_elems;
    return attn_launch<float>(a, max_seq_len, static_cast<cudaStream_t>(stream));
}

extern "C" int bw_attention_decode_f16kv(float* output, const float* Q, const uint16_t* K_cache,
                                         const uint16_t* V_cache, const int* d_seq_pos, int ctx_hint, int num_q_heads,
                                         int num_kv_heads, int head_dim, int max_seq_len, int M,
                                         size_t kv_batch_elems, size_t kv_layer_elems, void* stream) {
    if (head_dim != kHd || !d_seq_pos) return cudaErrorInvalidValue;
    AttnArgs a{};
    a.out = output; a.Q = Q; a.K = K_cache; a.V = V_cache; a.d_seq_pos = d_seq_pos; a.per_seq = 1;
    a.nqh = num_q_heads; a.nkv = num_kv_heads; a.max_seq = max_seq_len; a.M = M;
    a.kv_batch_elems = kv_batch_elems; a.kv_layer_elems = kv_layer_elems;
    return attn_launch<__half>(a, ctx_hint > 0 ? ctx_hint : max_seq_len, static_cast<cudaStream_t>(stream));
}

extern "C" int bw_attention_decode_f16kv_fused(float* output, const float* qkv, const float* q_norm_w,
                                               const float* k_norm_w, uint16_t* K_cache, uint16_t* V_cache,
                                               const int* d_seq_pos, int ctx_hint, int num_q_heads, int num_kv_heads,
                                               int head_dim, int max_seq_len, int M, size_t kv_batch_elems,
                                               size_t kv_layer_elems, float eps, float rope_base, void* stream) {
    if (head_dim != kHd || !d_seq_pos || !qkv || !q_norm_w || !k_norm_w) return cudaErrorInvalidValue;
    AttnArgs a{};
    a.out = output; a.Q = nullptr; a.K = K_cache; a.V = V_cache; a.d_seq_pos = d_seq_pos; a.per_seq = 1;
    a.nqh = num_q_heads; a.nkv = num_kv_heads; a.max_seq = max_seq_len; a.M = M;
    a.kv_batch_elems = kv_batch_elems; a.kv_layer_elems = kv_layer_elems;
    a.qkv = qkv; a.q_norm_w = q_norm_w; a.k_norm_w = k_norm_w; a.eps = eps; a.rope_base = rope_base;
    return attn_launch<__half>(a, ctx_hint > 0 ? ctx_hint : max_seq_len, static_cast<cudaStream_t>(stream));
}

extern "C" int bw_attention_decode_f16kv_fused_q8(float* output_or_null, int8_t* out_q8, float* out_scale,
                                                  const float* qkv, const float* q_norm_w, const float* k_norm_w,
                                                  uint16_t* K_cache, uint16_t* V_cache, const int* d_seq_pos,
                                                  int ctx_hint, int num_q_heads, int num_kv_heads, int head_dim,
                                                  int max_seq_len, int M, size_t kv_batch_elems, size_t kv_layer_elems,
                                                  float eps, float rope_base, void* stream) {
    if (head_dim != kHd || !d_seq_pos || !qkv || !q_norm_w || !k_norm_w || !out_q8 || !out_scale)
        return cudaErrorInvalidValue;
    if (num_kv_heads < 1 || (num_q_heads != 4 * num_kv_heads && num_q_heads != 8 * num_kv_heads))
        return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(out_q8) & 3) != 0) return cudaErrorInvalidValue;
    AttnArgs a{};
    a.out = output_or_null; a.out_q = out_q8; a.out_qs = out_scale;
    a.Q = nullptr; a.K = K_cache; a.V = V_cache; a.d_seq_pos = d_seq_pos; a.per_seq = 1;
    a.nqh = num_q_heads; a.nkv = num_kv_heads; a.max_seq = max_seq_len; a.M = M;
    a.kv_batch_elems = kv_batch_elems; a.kv_layer_elems = kv_layer_elems;
    a.qkv = qkv; a.q_norm_w = q_norm_w; a.k_norm_w = k_norm_w; a.eps = eps; a.rope_base = rope_base;
    return attn_launch<__half>(a, ctx_hint > 0 ? ctx_hint : max_seq_len, static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------------------
// Attention without any allocation.
//
// Some hosts of this library must never reach the CUDA allocator once they are
// running: a server that has handed the whole GPU to its own pool, a process
// that runs with allocation disabled after start-up, a caller whose memory
// budget is audited to the byte.  For them the split partials live in a
// fixed array that is part of the library image instead of a cudaMalloc'd
// buffer.  Every GPU that loads the library carries these 2 MiB until exit.
// ---------------------------------------------------------------------------
constexpr size_t kNoAllocScratchFloats = (size_t)1 << 19;  // 2 MiB of split partials at most
static __device__ __align__(256) float g_attn_noalloc_scratch[kNoAllocScratchFloats];
// Device address of the array, per device.  In host code the array's name stands for a host-side shadow of the
// symbol, not for device memory, so the address a kernel can use has to be asked for with the device current.
static float* g_attn_noalloc_ptr[kMaxDevices] = {nullptr};
static std::mutex g_attn_noalloc_mu;

static cudaError_t attn_noalloc_scratch(float** out) {
    std::lock_guard<std::mutex> lk(g_attn_noalloc_mu);
    const int dev = current_device();
    if (!g_attn_noalloc_ptr[dev]) {
        float* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_attn_noalloc_scratch);
        if (e != cudaSuccess) return e;
        g_attn_noalloc_ptr[dev] = p;
    }
    *out = g_attn_noalloc_ptr[dev];
    return cudaSuccess;
}

// Same arithmetic and the same split kernel as bw_attention_decode_batched_gqa_device, with the partial records in
// the fixed array and a separate merge launch.  No partial has to start from zero: every (head, split) record that the
// merge kernel reads is written in full by the split kernel of the same call, empty splits included.
extern "C" int bw_attention_decode_batched_gqa_noalloc(float* output, const float* Q, const float* K_cache,
                                                       const float* V_cache, const int* d_seq_pos, int num_q_heads,
                                                       int num_kv_heads, int head_dim, int max_seq_len, int M,
                                                       size_t kv_batch_elems, size_t kv_layer_elems, void* stream) {
    if (head_dim != kHd || !d_seq_pos) return cudaErrorInvalidValue;
    if (!output || !Q || !K_cache || !V_cache || num_q_heads < 1 || num_kv_heads < 1 ||
        num_q_heads % num_kv_heads != 0 || M < 1 || max_seq_len < 1)
        return cudaErrorInvalidValue;
    const int gq = num_q_heads / num_kv_heads;
    if (gq != 1 && gq != 2 && gq != 4 && gq != 8) return cudaErrorInvalidValue;
    AttnArgs a{};
    a.out = output; a.Q = Q; a.K = K_cache; a.V = V_cache; a.d_seq_pos = d_seq_pos; a.per_seq = 0;
    a.nqh = num_q_heads; a.nkv = num_kv_heads; a.max_seq = max_seq_len; a.M = M;
    a.kv_batch_elems = kv_batch_elems; a.kv_layer_elems = kv_layer_elems;
    // Its own fixed split rule (the allocating entry points size their splits by waves; the merge accepts any
    // split count): about two CTAs per SM, at least 64 positions per split, at most 64 splits, over the whole cache.
    const int ctx = max_seq_len;
    const int sms = sm_count(current_device());
    int nsplit = (2 * sms + M * a.nkv - 1) / (M * a.nkv);
    const int max_split = (ctx + 63) / 64;
    if (nsplit > max_split) nsplit = max_split;
    if (nsplit > 64) nsplit = 64;
    if (nsplit < 1) nsplit = 1;
    a.split_len = (ctx + nsplit - 1) / nsplit;
    a.split_len = (a.split_len + kPosPerStep - 1) / kPosPerStep * kPosPerStep;
    nsplit = (ctx + a.split_len - 1) / a.split_len;
    a.nsplit = nsplit;
    a.scale = 1.0f / sqrtf((float)kHd);
    a.part = nullptr;
    const size_t need = (size_t)M * a.nqh * nsplit * kPartStride;
    if (nsplit > 1) {
        if (need > kNoAllocScratchFloats) {
            fprintf(stderr,
                    "bw_attention_decode_batched_gqa_noalloc: M * num_q_heads * splits * %d = %zu floats of split "
                    "partials exceed the fixed scratch of %zu floats; use the allocating entry point or a smaller "
                    "batch\n", kPartStride, need, kNoAllocScratchFloats);
            return cudaErrorInvalidValue;
        }
        cudaError_t e = attn_noalloc_scratch(&a.part);
        if (e != cudaSuccess) return e;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const dim3 grid(nsplit, a.nkv, a.M);
    switch (gq) {
        case 1: attn_decode_split_kernel<float, 1><<<grid, kAttnWarps * 32, 0, st>>>(a); break;
        case 2: attn_decode_split_kernel<float, 2><<<grid, kAttnWarps * 32, 0, st>>>(a); break;
        case 4: attn_decode_split_kernel<float, 4><<<grid, kAttnWarps * 32, 0, st>>>(a); break;
        default: attn_decode_split_kernel<float, 8><<<grid, kAttnWarps * 32, 0, st>>>(a); break;
    }
    count_launch(1);
    cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) return e;
    if (nsplit > 1) {
        attn_merge_kernel<<<a.M * a.nqh, kHd, 0, st>>>(a.out, a.part, nsplit);
        count_launch(1);
        e = cudaPeekAtLastError();
    }
    return e;
}

static int update_kv_impl(float* k_cache, float* v_cache, const float* k_new, const float* v_new, int batch_idx,
                          const int* d_pos, int pos, int num_heads, int head_dim, int max_seq_len, void* stream) {
    if (!k_cache || !v_cache || !k_new || !v_new || num_heads < 1 || head_dim < 1 || max_seq_len < 1)
        return cudaErrorInvalidValue;
    if (batch_idx != 0) return cudaErrorInvalidValue;  // same contract as the reference
    if (!d_pos && (pos < 0 || pos >= max_seq_len)) return cudaErrorInvalidValue;
    const int total = num_heads * head_dim;
    update_kv_kernel_b200<float><<<(total + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        k_cache, v_cache, k_new, v_new, d_pos, pos, num_heads, head_dim, max_seq_len);
    count_launch(1);
    return cudaPeekAtLastError();
}

extern "C" int bw_update_kv_cache(float* k_cache, float* v_cache, const float* k_new, const float* v_new,
                                  int batch_idx, int seq_pos, int num_heads, int head_dim, int max_seq_len,
                                  void* stream) {
    return update_kv_impl(k_cache, v_cache, k_new, v_new, batch_idx, nullptr, seq_pos, num_heads, head_dim,
                          max_seq_len, stream);
}

extern "C" int bw_update_kv_cache_device(float* k_cache, float* v_cache, const float* k_new, const float* v_new,
                                         int batch_idx, const int* d_seq_pos, int num_heads, int head_dim,
                                         int max_seq_len, void* stream) {
    if (!d_seq_pos) return cudaErrorInvalidValue;
    return update_kv_impl(k_cache, v_cache, k_new, v_new, batch_idx, d_seq_pos, 0, num_heads, head_dim, max_seq_len,
                          stream);
}
