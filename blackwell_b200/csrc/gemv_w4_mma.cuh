// Streaming INT4 block-16 GEMV for 3..16 sequences per launch on sm_100a: the weight stream of the small-batch
// kernel (bulk copies into a shared-memory ring) with the integer dot products on the warp-level tensor-core
// instruction mma.sync.m16n8k32.s8 instead of dp4a, so that the instruction count per weight byte no longer
// grows with the number of sequences.
//
//   y[m][n] = sum_kb dot16(W[n,kb], xq[m,kb]) * w_sc[n,kb] * x_sc[m,kb]
//
// Work decomposition.  A persistent CTA owns a contiguous range of output rows and walks it in tiles of 32 rows;
// a tile is streamed in slabs of 32-k columns (1 KB of nibbles per row by default).  Two producer warps fill a ring
// stage per slab: the nibbles by one bulk copy per row, the scales by cp.async (lanes along a row), both into rows
// whose pitch is 16 mod 128 bytes, so that the eight rows an ldmatrix or a scale load touches fall into eight
// different bank groups.
// Sixteen consumer warps split the columns of a slab.  For one column (32 k = two k-blocks) of the 32
// rows a warp
//   * reads the packed nibbles with one ldmatrix.x4: thread (g, t) of the warp gets word t of rows g, g+8, g+16, g+24,
//   * turns each word into 16*q signed bytes of its even-k and odd-k nibbles (LOP3): exactly the A fragment
//     {a0, a1, a2, a3} of an m16n8k32 MMA whose k slots are (t, even) and (t, odd),
//   * multiplies with the B fragment of eight sequences, prepared once per CTA in the same k-slot order.  A k-block
//     is 16 k but the instruction sums 32: it is issued twice, once with the second block's B lanes zeroed and once
//     with the first's, so each accumulator tile is the exact int32 dot of ONE block.  Accumulators start from the
//     bit pattern of 1.5 * 2^23, so the result read as a float is 12582912 + 16 * dot exactly,
//   * applies the scales with packed fp32 FMAs: t = fma(F, w, -12582912 w) (exact for binary16 w; for fp32 scales
//     F - 12582912 first), acc = fma(t, x_sc / 16, acc).
// Each (row, sequence) accumulator lives in exactly one thread of the warp; after the last slab of a tile the
// consumer warps' partial sums are added through shared memory in fixed order (deterministic) and stored.
//
// When the prepared activations of all K do not fit beside the ring, K is processed in windows: the CTA prepares a
// window, runs all its row tiles over the window's slabs and accumulates into y (its rows are its own).
// Every wait is bounded (common.cuh); a wait that gives up raises the CTA's abort flag and the status word.
#pragma once
#include "gemv_w4_stream.cuh"

namespace bw {
namespace mma {

constexpr int kRows = 32;          // rows per tile
// Consumer warps per CTA (one more warp produces).  Sixteen: a warp's chain ldmatrix -> unpack -> MMA -> scale FMAs
// has little instruction-level parallelism, and at HBM speed a 32-row column step may take an SM only ~28 cycles, so
// the latency has to be covered by many warps.
constexpr int kConsumerWarps = 16;
constexpr int kThreads = (kConsumerWarps + 2) * 32;  // + one warp that copies the nibbles, one that copies the scales
constexpr int kXColBytes = 320;    // prepared activations of one (column, group of 8 sequences): B fragments + scales
__host__ __device__ constexpr int red_stride(int MG) { return 8 * MG + 1; }  // floats per row of a warp's partial sums (odd: no bank conflicts)

struct MmaPlan {
    int slab_cols;      // 32-k columns per slab
    int win_cols;       // columns per activation window (multiple of slab_cols, or all)
    int S;              // ring stages
    int pitch_n;        // bytes between the nibble rows of a stage
    int ablate;         // timing experiments: 1 = consumers skip the arithmetic, 2 = the producer copies nothing
    int pitch_s;        // bytes between the scale rows of a stage
    int scale_gran;     // size of one cp.async of scales: 16, 8 or 4 bytes (what the rows' alignment in HBM allows)
    int lanes_per_row;  // producer lanes that share one scale row of a slab (power of two, at most 32)
    size_t x_off, stage_off, red_off, smem;
};

struct Smem {
    static constexpr int kFull = 0;        // S mbarriers
    static constexpr int kEmpty = 64;      // S mbarriers
    static constexpr int kAbort = 128;
    static constexpr int kRstd = 192;      // 16 floats
    static constexpr int kScratch = 256;   // 16 sequences x 16 warps floats for the norm's block reduction
    static constexpr int kX = 2048;
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
// D = A (16 x 32, s8) * B (32 x 8, s8) + C, int32.
__device__ __forceinline__ void mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1, int c) {
    // not volatile: a pure function of its register operands, free to be scheduled around the loads of the next column
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c));
}
__device__ __forceinline__ void ffma2(float& d0, float& d1, float a0, float a1, float b0, float b1, float c0, float c1) {
    unsigned long long A, B, C, D;
    asm("mov.b64 %0, {%1, %2};" : "=l"(A) : "f"(a0), "f"(a1));
    asm("mov.b64 %0, {%1, %2};" : "=l"(B) : "f"(b0), "f"(b1));
    asm("mov.b64 %0, {%1, %2};" : "=l"(C) : "f"(c0), "f"(c1));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(D) : "l"(A), "l"(B), "l"(C));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d0), "=f"(d1) : "l"(D));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async8(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32) : "memory"); }

template <typename WS> struct ScalePairF;
template <> struct ScalePairF<__half> {
    static __device__ __forceinline__ float2 load(const unsigned char* p) {
        return __half22float2(*reinterpret_cast<const __half2*>(p));
    }
};
template <> struct ScalePairF<float> {
    static __device__ __forceinline__ float2 load(const unsigned char* p) { return *reinterpret_cast<const float2*>(p); }
};

// MG groups of 8 sequences (M <= 8 MG); WS = weight scale type.  kPack (MG = 1, M <= 4): the eight B columns of one MMA
// are the four sequences against the first k-block (other half of K zero) and the same four against the second, so
// ONE instruction per 16 rows yields both blocks' dots; the accumulators of the two blocks of a (row, sequence) then
// sit in two threads and meet in the cross-warp sum.
// kPending: the instantiation that serves the norm-pending hand-over (see GemvArgs), here for 5..16 sequences: the
// tile's 32 rows of one sequence sit in the 32 lanes of a warp when y is written, so a half warp holds one k-block of the
// consumer.  Row ranges then start at multiples of 16 and K must fit one window.
template <int MG, typename WS, bool kPack, bool kPending = false>
__global__ void __launch_bounds__(kThreads, 1) gemv_w4_mma_kernel(const GemvArgs a, const MmaPlan p, int M) {
    static_assert(!kPack || MG == 1, "packing is for one group of sequences");
    extern __shared__ __align__(128) unsigned char smem[];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int K = a.K, nch = a.nch, S = p.S;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + Smem::kFull);
    uint64_t* empty = reinterpret_cast<uint64_t*>(smem + Smem::kEmpty);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + Smem::kAbort);
    float* rstd_s = reinterpret_cast<float*>(smem + Smem::kRstd);
    float* nscratch = reinterpret_cast<float*>(smem + Smem::kScratch);
    unsigned char* xbase = smem + p.x_off;
    unsigned char* stages = smem + p.stage_off;
    float* red = reinterpret_cast<float*>(smem + p.red_off);
    const size_t stage_sc = (size_t)kRows * p.pitch_n;  // scales follow the nibbles inside a stage
    const size_t stage_bytes = stage_sc + (size_t)kRows * p.pitch_s;

    // this CTA's rows
    const int row_unit = (kPending && a.next_q) ? 16 : 1;   // a producer's row ranges are whole k-blocks of its consumer
    const int row_begin = row_unit * (int)(((long long)(a.N / row_unit) * blockIdx.x) / gridDim.x);
    const int row_end = row_unit * (int)(((long long)(a.N / row_unit) * (blockIdx.x + 1)) / gridDim.x);
    const int ntiles = (row_end - row_begin + kRows - 1) / kRows;
    const int nwin = (nch + p.win_cols - 1) / p.win_cols;

    if (t == 0) {
        // full: the arrive.expect_tx of the producer's lane 0 (nibbles) and one arrival per producer lane, made by the
        // hardware when the lane's cp.async copies (scales) have landed
        for (int s = 0; s < S; ++s) {
            mbar_init(smem_u32(&full[s]), 33);
            mbar_init(smem_u32(&empty[s]), kConsumerWarps);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();
    pdl_trigger();

    if (warp >= kConsumerWarps) {
        // ------------------------------------------------------------------ producers
        // Warp 16 copies the nibbles (one bulk copy per row, lane = row), warp 17 the scales (cp.async, lanes along a
        // row): two warps because each works through its copies one instruction after the other, and together they
        // would take longer than a slab lasts at HBM speed.
        const bool nib_warp = warp == kConsumerWarps;
        const int ws = (int)sizeof(WS);
        const uint64_t policy = l2_policy_evict_first();
        int item = 0;
        bool ok = true;
        for (int w = 0; w < nwin && ok; ++w) {
            const int wc0 = w * p.win_cols, wc1 = min(nch, wc0 + p.win_cols);
            for (int tile = 0; tile < ntiles && ok; ++tile) {
                const int r0 = row_begin + tile * kRows;
                const int rows = min(kRows, row_end - r0);
                for (int c0 = wc0; c0 < wc1; c0 += p.slab_cols, ++item) {
                    const int cols = min(p.slab_cols, wc1 - c0);
                    const int s = item % S;
                    if (item >= S) {
                        if (!mbar_wait(smem_u32(&empty[s]), ((item / S) & 1) ^ 1)) { *abort_flag = 1; ok = false; break; }
                    }
                    if (*abort_flag) { ok = false; break; }
                    const uint32_t fb = smem_u32(&full[s]);
                    unsigned char* st = stages + (size_t)s * stage_bytes;
                    if (nib_warp) {
                        const uint32_t nb = (p.ablate & 2) ? 0u : (uint32_t)cols * 16u;
                        if (lane == 0) mbar_expect_tx(fb, (uint32_t)rows * nb);
                        __syncwarp();
                        if (lane < rows && nb)
                            bulk_g2s(smem_u32(st + (size_t)lane * p.pitch_n),
                                     a.W + (size_t)(r0 + lane) * (size_t)(K / 2) + (size_t)c0 * 16, nb, fb, policy);
                        continue;
                    }
                    // scales: `lpr` lanes run along a row (coalesced), `gran` bytes per copy, 32 / lpr rows per pass
                    const uint32_t sb = (uint32_t)cols * 2u * ws;      // bytes per row in this slab
                    const uint32_t per_row = (p.ablate & 2) ? 0u : sb / (uint32_t)p.scale_gran;
                    const unsigned char* sbase = static_cast<const unsigned char*>(a.Wsc) +
                                                 ((size_t)r0 * (size_t)(K / 16) + (size_t)c0 * 2) * ws;
                    const size_t srow = (size_t)(K / 16) * ws;
                    const uint32_t lpr = (uint32_t)p.lanes_per_row, rstep = 32u / lpr;
                    const uint32_t dbase = smem_u32(st + stage_sc);
                    for (uint32_t oi = lane & (lpr - 1u); oi < per_row; oi += lpr) {
                        const uint32_t o = oi * (uint32_t)p.scale_gran;
                        uint32_t rr = lane / lpr;  // lpr is a power of two
                        uint32_t dst = dbase + rr * (uint32_t)p.pitch_s + o;
                        const unsigned char* src = sbase + (size_t)rr * srow + o;
                        for (; rr < (uint32_t)rows; rr += rstep, dst += rstep * (uint32_t)p.pitch_s, src += rstep * srow) {
                            if (p.scale_gran == 16) cp_async16(dst, src);
                            else if (p.scale_gran == 8) cp_async8(dst, src);
                            else cp_async4(dst, src);
                        }
                    }
                    cp_async_arrive_noinc(fb);
                }
            }
        }
        if (!nib_warp) asm volatile("cp.async.wait_all;" ::: "memory");
        return;
    }

    // ---------------------------------------------------------------------- consumers
    const int g = lane >> 2, tq = lane & 3;
    const int ct = t;  // consumer thread index 0..255
    pdl_wait();        // the activations (and y, the residual) come from the kernels before

    float acc[2][2][MG][2];  // [row group][row g / g+8][sequence group][sequence 2t / 2t+1]
    int item = 0;
    bool ok = true;

    for (int w = 0; w < nwin; ++w) {
        const int wc0 = w * p.win_cols, wc1 = min(nch, wc0 + p.win_cols);
        // ---- prepare the window's activations: B fragments in k-slot order and block scales / 16
        if (w > 0) consumer_sync();  // every warp is done with the previous window's fragments
        const bool pending_in = kPending && a.x_sumsq != nullptr;   // per-block sums of squares from the producer
        const bool needs_norm = (a.xkind == kXFloatNorm || a.xkind == kXFloatNormI4) || pending_in;
        if (pending_in && w == 0) {
            // one warp per sequence, all loads of a lane independent: a loop over the sequences would pay an L2 round
            // trip each (measured: 3 us at 8 sequences)
            if (warp < M) {
                float ss = 0.f;
                for (int i = lane; i < K / 16; i += 32) ss += __ldcg(a.x_sumsq + (size_t)warp * (K / 16) + i);
                ss = warp_sum(ss);   // fixed order: deterministic
                if (lane == 0) rstd_s[warp] = rsqrtf(ss / (float)K + a.eps);
            }
            consumer_sync();
        } else if (needs_norm && w == 0) {
            for (int m = 0; m < M; ++m) {
                float ss = 0.f;
                const float4* px = reinterpret_cast<const float4*>(static_cast<const float*>(a.x) + (size_t)m * a.x_stride);
                for (int i = ct; i < K / 4; i += kConsumerWarps * 32) {
                    const float4 f = __ldg(px + i);
                    ss = fmaf(f.x, f.x, ss); ss = fmaf(f.y, f.y, ss); ss = fmaf(f.z, f.z, ss); ss = fmaf(f.w, f.w, ss);
                }
                ss = warp_sum(ss);
                if (lane == 0) nscratch[m * kConsumerWarps + warp] = ss;
            }
            consumer_sync();
            if (ct < M) {
                float tot = 0.f;
                for (int i = 0; i < kConsumerWarps; ++i) tot += nscratch[ct * kConsumerWarps + i];
                rstd_s[ct] = rsqrtf(tot / (float)K + a.eps);
            }
            consumer_sync();
        }
        {
            const int wcols = wc1 - wc0;
            constexpr int SEQ = kPack ? 4 : 8 * MG;  // sequence slots per column
            const int nblk = 2 * wcols * SEQ;        // (column, block of the column, sequence)
            for (int idx = ct; idx < nblk; idx += kConsumerWarps * 32) {
                const int m = idx % SEQ;
                const int cb = idx / SEQ;
                const int cl = cb >> 1, blk = cb & 1;
                uint32_t e[2] = {0u, 0u}, o[2] = {0u, 0u};
                float sc = 0.f;
                if (m < M) make_xblock(a, m, 2 * (wc0 + cl) + blk, needs_norm ? rstd_s[m] : 1.f, e, o, sc);
                if (kPack) {
                    // B column g = m + 4 blk: the block's two words in the k slots of lanes t = 2 blk, 2 blk + 1, zeros in
                    // the other two; scales: thread t reads {sequence 2 (t & 1), 2 (t & 1) + 1} of block t >> 1
                    unsigned char* xc = xbase + (size_t)cl * kXColBytes;
                    uint2* bf = reinterpret_cast<uint2*>(xc) + (m + 4 * blk) * 4;
                    bf[2 * blk] = make_uint2(e[0], o[0]);
                    bf[2 * blk + 1] = make_uint2(e[1], o[1]);
                    bf[2 * (1 - blk)] = make_uint2(0u, 0u);
                    bf[2 * (1 - blk) + 1] = make_uint2(0u, 0u);
                    reinterpret_cast<float*>(xc + 256)[(2 * blk + (m >> 1)) * 2 + (m & 1)] = sc;
                } else {
                    unsigned char* xc = xbase + ((size_t)cl * MG + (m >> 3)) * kXColBytes;
                    // lanes (g = m % 8, t = 2 blk) and (g, 2 blk + 1): {even-k bytes, odd-k bytes} of the block's two words
                    uint2* bf = reinterpret_cast<uint2*>(xc) + (m & 7) * 4 + 2 * blk;
                    bf[0] = make_uint2(e[0], o[0]);
                    bf[1] = make_uint2(e[1], o[1]);
                    // scales: per pair of sequences (2t, 2t+1): {A 2t, A 2t+1, B 2t, B 2t+1}
                    float* sf = reinterpret_cast<float*>(xc + 256) + ((m & 7) >> 1) * 4 + 2 * blk + (m & 1);
                    *sf = sc;
                }
            }
            consumer_sync();
        }

        for (int tile = 0; tile < ntiles; ++tile) {
            const int r0 = row_begin + tile * kRows;
            const int rows = min(kRows, row_end - r0);
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int c = 0; c < MG; ++c) { acc[i][h][c][0] = 0.f; acc[i][h][c][1] = 0.f; }

            for (int c0 = wc0; c0 < wc1; c0 += p.slab_cols, ++item) {
                const int cols = min(p.slab_cols, wc1 - c0);
                const int s = item % S;
                if (ok && !mbar_wait(smem_u32(&full[s]), (item / S) & 1)) { *abort_flag = 1; ok = false; }
                if (ok && !(p.ablate & 1)) {
                    const unsigned char* st = stages + (size_t)s * stage_bytes;
                    const uint32_t st_n = smem_u32(st) + (uint32_t)lane * (uint32_t)p.pitch_n;
                    const unsigned char* st_s = st + stage_sc + (size_t)g * p.pitch_s;
#pragma unroll 4
                    for (int cl = warp; cl < cols; cl += kConsumerWarps) {
                        uint32_t r[4];
                        ldmatrix_x4(st_n + 16u * (uint32_t)cl, r);
                        uint32_t lo[4], hi[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) nibbles_to_s8x16(r[j], lo[j], hi[j]);
                        float2 wsc[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            wsc[j] = ScalePairF<WS>::load(st_s + (size_t)(8 * j) * p.pitch_s + (size_t)cl * (2 * sizeof(WS)));
                        const unsigned char* xc = xbase + (size_t)(c0 - wc0 + cl) * MG * kXColBytes;
                        if constexpr (kPack) {
                            const uint2 bf = *reinterpret_cast<const uint2*>(xc + lane * 8);
                            const float2 xs = *reinterpret_cast<const float2*>(xc + 256 + tq * 8);
#pragma unroll
                            for (int i = 0; i < 2; ++i) {
                                int d[4];
                                mma_s8(d, lo[2 * i], lo[2 * i + 1], hi[2 * i], hi[2 * i + 1], bf.x, bf.y, kMagicInt);
#pragma unroll
                                for (int h = 0; h < 2; ++h) {
                                    const float2 w2 = wsc[2 * i + h];
                                    const float w = tq < 2 ? w2.x : w2.y;  // this thread's columns belong to one block
                                    float t0, t1;
                                    if (sizeof(WS) == 2) {
                                        const float cw = -kMagicFloat * w;  // exact
                                        t0 = fmaf(__int_as_float(d[2 * h]), w, cw);
                                        t1 = fmaf(__int_as_float(d[2 * h + 1]), w, cw);
                                    } else {
                                        t0 = (__int_as_float(d[2 * h]) - kMagicFloat) * w;
                                        t1 = (__int_as_float(d[2 * h + 1]) - kMagicFloat) * w;
                                    }
                                    ffma2(acc[i][h][0][0], acc[i][h][0][1], t0, t1, xs.x, xs.y, acc[i][h][0][0], acc[i][h][0][1]);
                                }
                            }
                        } else {
#pragma unroll
                        for (int c = 0; c < MG; ++c) {
                            const uint2 bf = *reinterpret_cast<const uint2*>(xc + c * kXColBytes + lane * 8);
                            const float4 xs = *reinterpret_cast<const float4*>(xc + c * kXColBytes + 256 + tq * 16);
                            // block A lives in the k slots of lanes t = 0, 1, block B in those of t = 2, 3
                            const uint32_t bA0 = tq < 2 ? bf.x : 0u, bA1 = tq < 2 ? bf.y : 0u;
                            const uint32_t bB0 = tq < 2 ? 0u : bf.x, bB1 = tq < 2 ? 0u : bf.y;
#pragma unroll
                            for (int i = 0; i < 2; ++i) {
                                int dA[4], dB[4];
                                mma_s8(dA, lo[2 * i], lo[2 * i + 1], hi[2 * i], hi[2 * i + 1], bA0, bA1, kMagicInt);
                                mma_s8(dB, lo[2 * i], lo[2 * i + 1], hi[2 * i], hi[2 * i + 1], bB0, bB1, kMagicInt);
#pragma unroll
                                for (int h = 0; h < 2; ++h) {
                                    const float2 w2 = wsc[2 * i + h];
                                    float tA0, tA1, tB0, tB1;
                                    if (sizeof(WS) == 2) {
                                        // scalar here (a packed FMA would need w and c duplicated into register pairs),
                                        // packed below where all three operands already sit in pairs
                                        const float cA = -kMagicFloat * w2.x, cB = -kMagicFloat * w2.y;  // exact
                                        tA0 = fmaf(__int_as_float(dA[2 * h]), w2.x, cA);
                                        tA1 = fmaf(__int_as_float(dA[2 * h + 1]), w2.x, cA);
                                        tB0 = fmaf(__int_as_float(dB[2 * h]), w2.y, cB);
                                        tB1 = fmaf(__int_as_float(dB[2 * h + 1]), w2.y, cB);
                                    } else {
                                        tA0 = (__int_as_float(dA[2 * h]) - kMagicFloat) * w2.x;
                                        tA1 = (__int_as_float(dA[2 * h + 1]) - kMagicFloat) * w2.x;
                                        tB0 = (__int_as_float(dB[2 * h]) - kMagicFloat) * w2.y;
                                        tB1 = (__int_as_float(dB[2 * h + 1]) - kMagicFloat) * w2.y;
                                    }
                                    ffma2(acc[i][h][c][0], acc[i][h][c][1], tA0, tA1, xs.x, xs.y, acc[i][h][c][0], acc[i][h][c][1]);
                                    ffma2(acc[i][h][c][0], acc[i][h][c][1], tB0, tB1, xs.z, xs.w, acc[i][h][c][0], acc[i][h][c][1]);
                                }
                            }
                        }
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&empty[s]));  // this warp is done with the stage
            }

            // ---- the consumer warps' partial sums of the tile -> y (fixed order: deterministic)
            constexpr int RS = red_stride(MG);
            float* mine = red + (size_t)warp * (kRows * RS);
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int c = 0; c < MG; ++c) {
                        float* dst = mine + (16 * i + 8 * h + g) * RS + 8 * c + 2 * tq;
                        dst[0] = acc[i][h][c][0];
                        dst[1] = acc[i][h][c][1];
                    }
            consumer_sync();
            if (*abort_flag) ok = false;
            if (ok) {
                for (int o = ct; o < kRows * (kPack ? 4 : 8 * MG); o += kConsumerWarps * 32) {
                    const int row = o & (kRows - 1), m = o >> 5;   // a warp: the 32 rows of one sequence
                    const bool valid = row < rows && m < M;
                    float val = 0.f;
                    if (valid) {
                        float sum = 0.f;
#pragma unroll
                        for (int wv = 0; wv < kConsumerWarps; ++wv) {
                            const float* rp = red + (size_t)wv * (kRows * RS) + row * RS + m;
                            sum += kPack ? rp[0] + rp[4] : rp[0];  // packed: first block's column + second block's
                        }
                        const size_t yi = (size_t)m * a.y_stride + r0 + row;
                        if (w == 0) { val = a.residual ? sum + a.residual[yi] : sum; a.y[yi] = val; }
                        else a.y[yi] += sum;
                    }
                    if (kPending && a.next_q && m < M) {   // one window of K (the host's rule): val is final
                        const int col = r0 + row;
                        const float v = valid ? val * __ldg(a.next_norm_w + col) : 0.f;
                        float am = fabsf(v), ss = val * val;
#pragma unroll
                        for (int sh = 1; sh < 16; sh <<= 1) {
                            am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, sh));
                            ss += __shfl_xor_sync(0xffffffffu, ss, sh);
                        }
                        const float sc = quant_scale_i8(am);
                        if (valid) {
                            a.next_q[(size_t)m * a.N + col] = (int8_t)quant_i8(v, sc);
                            if ((row & 15) == 0) {
                                a.next_sc[(size_t)m * (a.N / 16) + (col >> 4)] = sc;
                                a.next_sumsq[(size_t)m * (a.N / 16) + (col >> 4)] = ss;
                            }
                        }
                    }
                }
            }
            consumer_sync();  // the buffer is free for the next tile's partial sums
        }
    }
    if (!ok && ct == 0) {
        // give copies still in flight a bounded chance to land before the CTA's shared memory is released
        for (int s = 0; s < S; ++s) (void)mbar_wait(smem_u32(&full[s]), 0);
        atomicExch(a.status, kStatusMbarTimeout);
    }
}

}  // namespace mma
}  // namespace bw
