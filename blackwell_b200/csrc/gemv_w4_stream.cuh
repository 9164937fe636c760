// Streaming INT4 block-16 GEMV for small batch (M <= 8 per launch) on sm_100a.
//
//   y[m][n] = sum_kb dot16(W[n,kb], x[m,kb]) * w_sc[n,kb] * x_sc[m,kb]
//
// Data layout in HBM (caller's, unchanged): W u8 [N][K/2] (two offset-binary
// nibbles per byte, even k in the low nibble), weight scales [N][K/16] as
// binary16 or fp32, y f32 [M][N].
//
// Structure.  A persistent CTA owns a contiguous range of output rows and walks
// it in tiles of R rows.  One elected thread streams each tile (R*K/2 bytes of
// nibbles and the R*K/16 scales, both contiguous in HBM) into a ring of shared
// memory stages with cp.async.bulk, completion counted on one mbarrier per
// stage.  The activations are turned once per CTA into signed bytes laid out to
// match the nibble order (even-k bytes and odd-k bytes in separate words) and
// held in registers (or in shared memory when K needs several passes).  Every
// thread owns 16-byte weight chunks (32 nibbles = two k-blocks): LOP3 moves the
// nibbles to 16*q signed bytes, four dp4a per k-block accumulate an exact
// int32 dot product on top of a float bit pattern, one FADD turns it into a
// float and one FMA applies the scale product.  Row sums are finished with a
// transposing warp-shuffle reduction and a small cross-warp add.
#pragma once
#include "common.cuh"
#include "quant_rules.cuh"

namespace bw {

// How the activations arrive.
enum XKind : int {
    kXInt8 = 0,      // i8 [M][K] + f32 scales [M][K/16]      (already quantized)
    kXInt4 = 1,      // u8 [M][K/2] nibbles + f32 scales        (already quantized)
    kXHalf = 2,      // f16 [M][K]   -> int8 block-16 quantize in the prologue
    kXFloat = 3,     // f32 [M][K]   -> int8 block-16 quantize in the prologue
    kXFloatNorm = 4, // f32 [M][K], RMSNorm(weight, eps) -> quantize in the prologue
    kXSwiglu = 5,    // f32 gate [M][K], f32 up [M][K]: silu(g)*u -> quantize
    kXFloatI4 = 6,     // f32 [M][K] -> int4 block-16 quantize (reference rule) in the prologue
    kXFloatNormI4 = 7, // RMSNorm then int4 quantize
    kXSwigluI4 = 8,    // SwiGLU then int4 quantize
};

struct XChunk {      // one 32-element activation chunk of one sequence
    uint32_t e[4];   // even-k bytes of weight word i
    uint32_t o[4];   // odd-k bytes of weight word i
    float s[2];      // block scales, pre-divided by 16
};

struct GemvArgs {
    float* y;               // [M][N]
    const uint8_t* W;       // [N][K/2]
    const void* Wsc;        // [N][K/16] half or float
    const void* x;          // see XKind
    const void* x2;         // up-projection for kXSwiglu
    const float* xsc;       // [M][K/16] for the pre-quantized kinds
    const float* norm_w;    // [K] for kXFloatNorm
    const float* residual;  // optional [M][y_stride]: added to the result (may alias y)
    int* status;            // device status word (bw_device_status)
    // "Norm-pending" hand-over between two GEMVs of a decode step (dp4a streaming kernel at one sequence, mma.sync
    // streaming kernel at 5..16; the arrays below then have a leading dimension of M sequences).  The
    // producer's epilogue, which holds 16 consecutive outputs in 16 lanes, also writes what the consumer's fused
    // RMSNorm + quantize prologue would compute from them, except the norm's scalar: q = q8(y * next_norm_w) with the
    // block's own scale, and the block's sum of y^2.  The consumer (xkind kXInt8 with x_sumsq set) sums the per-block
    // sums in fixed order, forms rstd and multiplies it into the block scales: the integers of q8(y * w * rstd) do
    // not depend on rstd.  Saves every consumer CTA the quantization of all K activations.
    const float* x_sumsq;       // consumer: [K/16] per-block sums of squares of the un-normed activations, or nullptr
    const float* next_norm_w;   // producer: [N] norm weights of the consumer, or nullptr
    int8_t* next_q;             // producer: [N]
    float* next_sc;             // producer: [N/16] block scales without rstd
    float* next_sumsq;          // producer: [N/16]
#ifdef BW_GEMV_TIMELINE
    unsigned long long* timeline;  // experiment builds only: per-phase %globaltimer stamps of a few CTAs
#endif
    long x_stride;          // elements between sequences of x / x2 (f16 and f32 kinds)
    long y_stride;          // elements between sequences of y and residual
    float eps;
    int xkind;
    int K, N;               // N = row count of y; rows >= n_rows are not touched
    int n_rows;             // rows handled by this launch (multiple of row_unit)
    int row_unit;           // row ranges start at multiples of this
    int nch;                // K / 32
    int Tg, G, J;           // threads covering K, groups, passes over K
    int S;                  // ring stages
    int rg;                 // rows per group in one tile (<= RowsPerGroup<M>)
};

// 16 floats (one k-block) -> signed bytes in nibble order + scale/16, with the reference's bits (q = roundf(v / sc),
// IEEE division, ties away from zero).  The common path avoids the sixteen divisions and roundf sequences: with
// rcp = 1 / sc, v * rcp lies within 1.6e-5 of the true quotient (|v / sc| <= 127), so rint(v * rcp) is the reference's
// integer unless that product sits within 3e-5 of a half; a block with such an element (about one in a thousand), or
// with a non-finite value, is redone with the reference's own formula.  No clamp is needed on the common path: sc is
// absmax / 127 (or / 7), which bounds |v * rcp| by 127.0001 (7.000001).
template <bool kInt4Rule>
__device__ __forceinline__ void quantize_block(const float (&v)[16], uint32_t (&e)[2], uint32_t (&o)[2], float& s) {
    float am = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) am = fmaxf(am, fabsf(v[i]));
    const float sc = kInt4Rule ? quant_scale_i4(am) : quant_scale_i8(am);
    const float rcp = 1.0f / sc;
    s = sc * 0.0625f;
    // Rounding without the conversion unit (FRND / F2I issue at a fraction of the FP32 rate, and sixteen of each per
    // thread were most of this prologue's time): r + 1.5 * 2^23 rounds r to the nearest integer (ties to even) in the
    // low mantissa bits, whose low byte is the two's complement result.
    uint32_t qb[16];
    bool exact_needed = !(am < 3.0e38f);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const float r = v[i] * rcp;
        const float mg = r + kMagicFloat;
        const float ri = mg - kMagicFloat;
        exact_needed |= !(fabsf(fabsf(r - ri) - 0.5f) > 3e-5f);  // also true for a NaN
        qb[i] = __float_as_uint(mg);
    }
    if (exact_needed) {
#pragma unroll
        for (int i = 0; i < 16; ++i) qb[i] = (uint32_t)(kInt4Rule ? quant_i4(v[i], sc) : quant_i8(v[i], sc));
    }
    // low bytes of four registers -> one word, even-k and odd-k elements apart
#pragma unroll
    for (int wd = 0; wd < 2; ++wd) {
        const uint32_t* q = qb + 8 * wd;
        e[wd] = prmt(prmt(q[0], q[2], 0x0040), prmt(q[4], q[6], 0x0040), 0x5410);
        o[wd] = prmt(prmt(q[1], q[3], 0x0040), prmt(q[5], q[7], 0x0040), 0x5410);
    }
}

// Builds the register form of k-block kb (16 elements) of sequence m: the even-k
// and odd-k signed bytes of its two weight words and the block scale / 16.
__device__ __forceinline__ void make_xblock(const GemvArgs& a, int m, int kb, float rstd, uint32_t (&e)[2],
                                            uint32_t (&o)[2], float& s) {
    const int K = a.K;
    const size_t nkb = (size_t)(K / 16);
    if (a.xkind == kXInt8) {
        const uint2* p = reinterpret_cast<const uint2*>(static_cast<const int8_t*>(a.x) + (size_t)m * K + 16 * (size_t)kb);
        const uint2 q0 = __ldg(p), q1 = __ldg(p + 1);
        e[0] = prmt(q0.x, q0.y, 0x6420); o[0] = prmt(q0.x, q0.y, 0x7531);
        e[1] = prmt(q1.x, q1.y, 0x6420); o[1] = prmt(q1.x, q1.y, 0x7531);
        s = __ldg(a.xsc + (size_t)m * nkb + kb) * 0.0625f * rstd;   // rstd is 1 unless the norm is pending
    } else if (a.xkind == kXInt4) {
        const uint2 q = __ldg(reinterpret_cast<const uint2*>(static_cast<const uint8_t*>(a.x) + (size_t)m * (K / 2) + 8 * (size_t)kb));
        e[0] = bytes_minus8(q.x & 0x0F0F0F0Fu); o[0] = bytes_minus8((q.x >> 4) & 0x0F0F0F0Fu);
        e[1] = bytes_minus8(q.y & 0x0F0F0F0Fu); o[1] = bytes_minus8((q.y >> 4) & 0x0F0F0F0Fu);
        s = __ldg(a.xsc + (size_t)m * nkb + kb) * 0.0625f;
    } else {
        float v[16];
        if (a.xkind == kXHalf) {
            const uint4* p = reinterpret_cast<const uint4*>(static_cast<const __half*>(a.x) + (size_t)m * a.x_stride + 16 * (size_t)kb);
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const uint4 q = __ldg(p + i);
                const __half2* h = reinterpret_cast<const __half2*>(&q);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __half22float2(h[j]);
                    v[8 * i + 2 * j] = f.x;
                    v[8 * i + 2 * j + 1] = f.y;
                }
            }
        } else {
            const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(a.x) + (size_t)m * a.x_stride + 16 * (size_t)kb);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float4 f = __ldg(p + i);
                v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
            }
            if (a.xkind == kXFloatNorm || a.xkind == kXFloatNormI4) {
                const float4* wp = reinterpret_cast<const float4*>(a.norm_w + 16 * (size_t)kb);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float4 gw = __ldg(wp + i);
                    v[4 * i] = v[4 * i] * gw.x * rstd;
                    v[4 * i + 1] = v[4 * i + 1] * gw.y * rstd;
                    v[4 * i + 2] = v[4 * i + 2] * gw.z * rstd;
                    v[4 * i + 3] = v[4 * i + 3] * gw.w * rstd;
                }
            } else if (a.xkind == kXSwiglu || a.xkind == kXSwigluI4) {
                const float4* up = reinterpret_cast<const float4*>(static_cast<const float*>(a.x2) + (size_t)m * a.x_stride + 16 * (size_t)kb);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float4 u = __ldg(up + i);
                    v[4 * i] = silu_mul(v[4 * i], u.x);
                    v[4 * i + 1] = silu_mul(v[4 * i + 1], u.y);
                    v[4 * i + 2] = silu_mul(v[4 * i + 2], u.z);
                    v[4 * i + 3] = silu_mul(v[4 * i + 3], u.w);
                }
            }
        }
        if (a.xkind >= kXFloatI4) quantize_block<true>(v, e, o, s);
        else quantize_block<false>(v, e, o, s);
    }
}

// Chunk c = k-blocks 2c and 2c+1.
__device__ __forceinline__ void make_xchunk(const GemvArgs& a, int m, int c, float rstd, XChunk& xc) {
    uint32_t e[2], o[2];
    float s;
    make_xblock(a, m, 2 * c, rstd, e, o, s);
    xc.e[0] = e[0]; xc.e[1] = e[1]; xc.o[0] = o[0]; xc.o[1] = o[1]; xc.s[0] = s;
    make_xblock(a, m, 2 * c + 1, rstd, e, o, s);
    xc.e[2] = e[0]; xc.e[3] = e[1]; xc.o[2] = o[0]; xc.o[3] = o[1]; xc.s[1] = s;
}

// One 16-byte weight chunk against M activation chunks.
template <int M>
__device__ __forceinline__ void chunk_fma(const uint4 w, const float ws0, const float ws1, const XChunk (&x)[M],
                                          float* acc /* [M] */) {
    uint32_t lo[4], hi[4];
    nibbles_to_s8x16(w.x, lo[0], hi[0]);
    nibbles_to_s8x16(w.y, lo[1], hi[1]);
    nibbles_to_s8x16(w.z, lo[2], hi[2]);
    nibbles_to_s8x16(w.w, lo[3], hi[3]);
#pragma unroll
    for (int m = 0; m < M; ++m) {
        int d0 = kMagicInt, d1 = kMagicInt;
        d0 = dp4a_ss(lo[0], x[m].e[0], d0);
        d1 = dp4a_ss(lo[2], x[m].e[2], d1);
        d0 = dp4a_ss(hi[0], x[m].o[0], d0);
        d1 = dp4a_ss(hi[2], x[m].o[2], d1);
        d0 = dp4a_ss(lo[1], x[m].e[1], d0);
        d1 = dp4a_ss(lo[3], x[m].e[3], d1);
        d0 = dp4a_ss(hi[1], x[m].o[1], d0);
        d1 = dp4a_ss(hi[3], x[m].o[3], d1);
        const float f0 = __int_as_float(d0) - kMagicFloat;
        const float f1 = __int_as_float(d1) - kMagicFloat;
        acc[m] = fmaf(f0, ws0 * x[m].s[0], acc[m]);
        acc[m] = fmaf(f1, ws1 * x[m].s[1], acc[m]);
    }
}

template <typename WS> struct ScalePair;
template <> struct ScalePair<__half> {
    static __device__ __forceinline__ void load(const void* base, size_t pair_index, float& s0, float& s1) {
        const __half2 h = *(reinterpret_cast<const __half2*>(base) + pair_index);
        const float2 f = __half22float2(h);
        s0 = f.x; s1 = f.y;
    }
};
template <> struct ScalePair<float> {
    static __device__ __forceinline__ void load(const void* base, size_t pair_index, float& s0, float& s1) {
        const float2 f = *(reinterpret_cast<const float2*>(base) + pair_index);
        s0 = f.x; s1 = f.y;
    }
};

// NR rows of one chunk column, all valid: every weight and scale load is issued
// before the arithmetic so that the rows overlap in the pipelines.
template <int M, typename WS, int NR>
__device__ __forceinline__ void rows_full(const unsigned char* st, size_t stage_nib, uint32_t row_nib,
                                          uint32_t row_sc, int g, int G, int c, const XChunk (&xr)[M],
                                          float* acc) {
    uint4 w[NR];
    float ws0[NR], ws1[NR];
#pragma unroll
    for (int rr = 0; rr < NR; ++rr) {
        const int r = g + G * rr;
        w[rr] = *reinterpret_cast<const uint4*>(st + (size_t)r * row_nib + 16 * (size_t)c);
        ScalePair<WS>::load(st + stage_nib + (size_t)r * row_sc, (size_t)c, ws0[rr], ws1[rr]);
    }
#pragma unroll
    for (int rr = 0; rr < NR; ++rr) chunk_fma<M>(w[rr], ws0[rr], ws1[rr], xr, acc + rr * M);
}

// One chunk column of a tile for this thread's group: `rg` rows when the tile is
// full, a predicated walk over the valid rows of a ragged last tile otherwise.
template <int M, typename WS, int RG>
__device__ __forceinline__ void tile_column(const unsigned char* st, size_t stage_nib, uint32_t row_nib,
                                            uint32_t row_sc, int g, int G, int c, int rows, int rg,
                                            const XChunk (&xr)[M], float* acc) {
    const bool full = g + G * (rg - 1) < rows;
    if (full && rg == RG) {
        rows_full<M, WS, RG>(st, stage_nib, row_nib, row_sc, g, G, c, xr, acc);
    } else if (full && RG >= 4 && rg == RG / 2) {
        rows_full<M, WS, (RG >= 2 ? RG / 2 : 1)>(st, stage_nib, row_nib, row_sc, g, G, c, xr, acc);
    } else {
#pragma unroll
        for (int rr = 0; rr < RG; ++rr) {
            const int r = g + G * rr;
            if (r < rows) {
                const uint4 w = *reinterpret_cast<const uint4*>(st + (size_t)r * row_nib + 16 * (size_t)c);
                float ws0, ws1;
                ScalePair<WS>::load(st + stage_nib + (size_t)r * row_sc, (size_t)c, ws0, ws1);
                chunk_fma<M>(w, ws0, ws1, xr, acc + rr * M);
            }
        }
    }
}

template <int M> struct RowsPerGroup { static constexpr int value = M <= 2 ? 8 : (M <= 4 ? 4 : 2); };

// Shared memory carve-up (byte offsets from the 128-aligned dynamic base).
struct GemvSmem {
    static constexpr int kBarOff = 0;        // 8 mbarriers
    static constexpr int kFlagOff = 64;      // abort flag
    static constexpr int kRstdOff = 96;      // rstd per sequence (8 floats)
    static constexpr int kWarpScratchOff = 128;  // 16 floats per sequence for block reductions
    static constexpr int kRedOff = 1024;     // 2 x 16 warps x 32 floats
    static constexpr int kXOff = 1024 + 2 * 16 * 32 * 4;  // activations (J > 1 only), then the stages
};

__host__ __device__ inline size_t gemv_x_smem_bytes(int M, int nch, int J) {
    (void)J;
    return (size_t)M * nch * 40;
}
__host__ __device__ inline size_t align128(size_t v) { return (v + 127) & ~(size_t)127; }

// kPending: the instantiation that serves the norm-pending hand-over (one sequence); the ordinary one carries none of
// its code (the hand-over's extra registers cost the M = 1 kernel 3 % on the small matrices).
template <int M, typename WS, bool kMultiPass, bool kPending = false>
__global__ void __launch_bounds__(M <= 2 ? 512 : 256, 1)
gemv_w4_stream_kernel(const GemvArgs a) {
    constexpr int RG = RowsPerGroup<M>::value;
    constexpr int V = RG * M;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    unsigned char* smem = smem_raw;

    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int T = blockDim.x;
    const int K = a.K, nch = a.nch, Tg = a.Tg, G = a.G, S = a.S;
#ifdef BW_GEMV_TIMELINE
    unsigned long long*& tl_base = *reinterpret_cast<unsigned long long**>(smem + 80);
    if (t == 0) {
        tl_base = nullptr;
        const int sel = blockIdx.x == 0 ? 0 : (blockIdx.x == gridDim.x / 2 ? 1 : (blockIdx.x == gridDim.x - 1 ? 2 : -1));
        if (a.timeline && sel >= 0) {
            unsigned long long li = sel == 0 ? atomicAdd(a.timeline, 1ull) : a.timeline[0];
            tl_base = a.timeline + 16 + (li % 32) * 48 + sel * 16;
            tl_base[0] = global_ns();
        }
    }
#define BW_TL(i) do { if (t == 0 && tl_base) tl_base[i] = global_ns(); } while (0)
#else
#define BW_TL(i) do { } while (0)
#endif
    const int R = a.rg * G;  // rows per tile; a.rg <= RG
    const int g = t / Tg, tg = t - g * Tg;
    const int warps_per_group = Tg >> 5;
    const uint32_t row_nib = (uint32_t)(K / 2);
    const uint32_t row_sc = (uint32_t)((K / 16) * (int)sizeof(WS));
    const size_t stage_nib = align128((size_t)R * row_nib);
    const size_t stage_bytes = stage_nib + align128((size_t)R * row_sc);

    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + GemvSmem::kBarOff);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + GemvSmem::kFlagOff);
    float* rstd_s = reinterpret_cast<float*>(smem + GemvSmem::kRstdOff);
    float* wscratch = reinterpret_cast<float*>(smem + GemvSmem::kWarpScratchOff);
    float* red = reinterpret_cast<float*>(smem + GemvSmem::kRedOff);
    unsigned char* xs_base = smem + GemvSmem::kXOff;
    unsigned char* stages = xs_base + align128(gemv_x_smem_bytes(M, nch, a.J));

    // Row range of this CTA, in units of row_unit rows.
    const int units = a.n_rows / a.row_unit;
    const int u0 = (int)(((long long)units * blockIdx.x) / gridDim.x);
    const int u1 = (int)(((long long)units * (blockIdx.x + 1)) / gridDim.x);
    const int row_begin = u0 * a.row_unit, row_end = u1 * a.row_unit;
    const int ntiles = (row_end - row_begin + R - 1) / R;

    if (t == 0) {
        for (int s = 0; s < S; ++s) mbar_init(smem_u32(&bars[s]), 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();

    const uint64_t policy = l2_policy_evict_first();
    auto issue_tile = [&](int tile) {
        const int s = tile % S;
        const int r0 = row_begin + tile * R;
        const int rows = min(R, row_end - r0);
        const uint32_t nb = (uint32_t)rows * row_nib, sb = (uint32_t)rows * row_sc;
        const uint32_t bar = smem_u32(&bars[s]);
        unsigned char* st = stages + (size_t)s * stage_bytes;
        mbar_expect_tx(bar, nb + sb);
        bulk_g2s(smem_u32(st), a.W + (size_t)r0 * row_nib, nb, bar, policy);
        bulk_g2s(smem_u32(st + stage_nib), static_cast<const unsigned char*>(a.Wsc) + (size_t)r0 * row_sc, sb, bar,
                 policy);
    };
    if (t == 0) {
        const int pre = min(S, ntiles);
        for (int i = 0; i < pre; ++i) issue_tile(i);
    }
    // The weights never depend on the previous kernel, the activations and y do: only now wait for it.
    BW_TL(1);
    pdl_trigger();
    pdl_wait();
    BW_TL(2);

    // ---- activation prologue (overlaps the first weight tiles in flight) ----
    const bool pending_norm = kPending && a.x_sumsq != nullptr;   // one sequence: per-block sums of squares from the producer
    const bool needs_norm = (a.xkind == kXFloatNorm || a.xkind == kXFloatNormI4) || pending_norm;
    if (needs_norm) {
        // sum of squares of every sequence, all threads cooperating
        for (int m = 0; m < M; ++m) {
            float ss = 0.f;
            if (pending_norm) {
                for (int i = t; i < K / 16; i += T) ss += __ldcg(a.x_sumsq + i);
            } else {
                const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(a.x) + (size_t)m * a.x_stride);
                for (int i = t; i < K / 4; i += T) {
                    const float4 f = __ldg(p + i);
                    ss = fmaf(f.x, f.x, ss); ss = fmaf(f.y, f.y, ss); ss = fmaf(f.z, f.z, ss); ss = fmaf(f.w, f.w, ss);
                }
            }
            ss = warp_sum(ss);
            if (lane == 0) wscratch[m * 16 + warp] = ss;
        }
        __syncthreads();
        if (t < M) {
            float tot = 0.f;
            for (int w = 0; w < (T >> 5); ++w) tot += wscratch[t * 16 + w];
            rstd_s[t] = rsqrtf(tot / (float)K + a.eps);
        }
        __syncthreads();
    }

    // Every k-block of every sequence is produced exactly once per CTA and staged in shared memory in
    // chunk order: [m][c] x {uint4 even-k words, uint4 odd-k words, float2 scales}.
    {
        uint2* xe2 = reinterpret_cast<uint2*>(xs_base);
        uint2* xo2 = xe2 + (size_t)M * nch * 2;
        float* xs1 = reinterpret_cast<float*>(xo2 + (size_t)M * nch * 2);
        const int nkb = 2 * nch;
        for (int idx = t; idx < M * nkb; idx += T) {
            const int m = idx / nkb, kb = idx - m * nkb;
            uint32_t e[2], o[2];
            float sc;
            make_xblock(a, m, kb, needs_norm ? rstd_s[m] : 1.f, e, o, sc);
            xe2[idx] = make_uint2(e[0], e[1]);
            xo2[idx] = make_uint2(o[0], o[1]);
            xs1[idx] = sc;
        }
        __syncthreads();
    }
    const uint4* xe = reinterpret_cast<const uint4*>(xs_base);
    const uint4* xo = xe + (size_t)M * nch;
    const float2* xsv = reinterpret_cast<const float2*>(xo + (size_t)M * nch);
    XChunk xr[M];
    auto load_x = [&](int c) {
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const uint4 e = xe[m * nch + c], o = xo[m * nch + c];
            const float2 sv = xsv[m * nch + c];
            xr[m].e[0] = e.x; xr[m].e[1] = e.y; xr[m].e[2] = e.z; xr[m].e[3] = e.w;
            xr[m].o[0] = o.x; xr[m].o[1] = o.y; xr[m].o[2] = o.z; xr[m].o[3] = o.w;
            xr[m].s[0] = sv.x; xr[m].s[1] = sv.y;
        }
    };
    if (!kMultiPass && tg < nch) load_x(tg);
    BW_TL(3);

    // ------------------------------------------------------------- main loop
    bool aborted = false;
    float held = 0.f;   // norm-pending hand-over with tiles of 8 rows: the even tile's value of this lane
    for (int tile = 0; tile < ntiles; ++tile) {
        const int s = tile % S;
        const uint32_t parity = (uint32_t)(tile / S) & 1u;
        if (!mbar_wait(smem_u32(&bars[s]), parity)) *abort_flag = 1;
        if (tile == 0) BW_TL(4);

        const unsigned char* st = stages + (size_t)s * stage_bytes;
        const int r0 = row_begin + tile * R;
        const int rows = min(R, row_end - r0);

        float acc[V];
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] = 0.f;

        if (!kMultiPass) {
            if (tg < nch) tile_column<M, WS, RG>(st, stage_nib, row_nib, row_sc, g, G, tg, rows, a.rg, xr, acc);
        } else {
            for (int j = 0; j < a.J; ++j) {
                const int c = tg + Tg * j;
                if (c < nch) {
                    load_x(c);
                    tile_column<M, WS, RG>(st, stage_nib, row_nib, row_sc, g, G, c, rows, a.rg, xr, acc);
                }
            }
        }

        if (tile == 0) BW_TL(5);
        // warp totals of the V = RG*M partial sums, one value index per lane group
        const float tot = warp_sum_many<V>(acc, lane);
        constexpr int P = V <= 1 ? 1 : V <= 2 ? 2 : V <= 4 ? 4 : V <= 8 ? 8 : V <= 16 ? 16 : 32;
        float* redb = red + (size_t)(tile & 1) * 16 * 32;
        if ((lane & (32 / P - 1)) == 0) {
            const int idx = warp_sum_many_index<V>(lane);
            if (idx < V) redb[warp * 32 + idx] = tot;
        }
        __syncthreads();  // partial sums visible; stage s fully consumed

        if (*abort_flag) { aborted = true; break; }
        if (t == 0 && tile + S < ntiles) issue_tile(tile + S);

        if (t < R * M) {
            const int r = t / M, m = t - r * M;
            float val = 0.f;
            if (r < rows) {
                const int gg = r % G, rr = r / G;
                float sum = 0.f;
                for (int w = 0; w < warps_per_group; ++w) sum += redb[(gg * warps_per_group + w) * 32 + rr * M + m];
                const size_t yi = (size_t)m * a.y_stride + r0 + r;
                val = a.residual ? sum + a.residual[yi] : sum;
                a.y[yi] = val;
            }
            if (kPending && M == 1 && a.next_q) {
                // Norm-pending hand-over.  The host guarantees row ranges that start at multiples of 16 and hold a
                // multiple of 16 rows, and tiles of 8, 16 or a multiple of 32 rows: lanes 16 j .. 16 j + 15 hold one
                // k-block of the consumer, or (tiles of 8, long K) lanes 0..7 hold half of one and keep the even tile's
                // half until the odd tile arrives.
                if (R == 8) {
                    if ((tile & 1) == 0) {
                        held = val;
                    } else {
                        const int col = r0 - 8 + r;          // the first half's row; the second is col + 8
                        const float v0 = held * __ldg(a.next_norm_w + col), v1 = val * __ldg(a.next_norm_w + col + 8);
                        float am = fmaxf(fabsf(v0), fabsf(v1)), ss = fmaf(held, held, val * val);
#pragma unroll
                        for (int o = 1; o < 8; o <<= 1) {
                            am = fmaxf(am, __shfl_xor_sync(0xFFu, am, o));
                            ss += __shfl_xor_sync(0xFFu, ss, o);
                        }
                        const float sc = quant_scale_i8(am);
                        a.next_q[col] = (int8_t)quant_i8(v0, sc);
                        a.next_q[col + 8] = (int8_t)quant_i8(v1, sc);
                        if (r == 0) { a.next_sc[col >> 4] = sc; a.next_sumsq[col >> 4] = ss; }
                    }
                } else {
                    const unsigned mask = R == 16 ? 0xFFFFu : 0xFFFFFFFFu;
                    const int col = r0 + r;
                    const float v = r < rows ? val * __ldg(a.next_norm_w + col) : 0.f;
                    float am = fabsf(v), ss = val * val;
#pragma unroll
                    for (int o = 1; o < 16; o <<= 1) {
                        am = fmaxf(am, __shfl_xor_sync(mask, am, o));
                        ss += __shfl_xor_sync(mask, ss, o);
                    }
                    const float sc = quant_scale_i8(am);
                    if (r < rows) {
                        a.next_q[col] = (int8_t)quant_i8(v, sc);
                        if ((r & 15) == 0) { a.next_sc[col >> 4] = sc; a.next_sumsq[col >> 4] = ss; }
                    }
                }
            }
        }
    }

    BW_TL(6);
    if (aborted && t == 0) {
        // Give copies still in flight a bounded chance to land before the CTA's
        // shared memory is released, then report.
        for (int s = 0; s < S; ++s) {
            (void)mbar_wait(smem_u32(&bars[s]), 0);
        }
        atomicExch(a.status, kStatusMbarTimeout);
    }
}

}  // namespace bw
