// tcgen05 path of the INT4 block-16 GEMV family for 9..64 sequences per launch: activation prep kernel, the
// warp-specialised MMA kernel and the host launcher.  See gemm_w4a8_tc.cuh for the arithmetic.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <mutex>

#include "../../include/blackwell_b200.h"
#include "gemm_w4a8_tc.cuh"
#include "gemv_w4_stream.cuh"
#include "host_util.h"

namespace bw {
#ifdef BW_GEMV_TIMELINE
void* debug_timeline_ptr();
#define TC_TL(slot, idx) do { if (blockIdx.x == 0 && a.timeline && (idx) < 256) a.timeline[(slot) * 256 + (idx)] = clock64(); } while (0)
#else
#define TC_TL(slot, idx) do { } while (0)
#endif
namespace tc {

// ----------------------------------------------------------------------------------------------------------
// Activation prep: quantizes every 16-element k-block of every sequence once (the same make_xblock code as the
// streaming kernel's prologue: plain / RMSNorm / SwiGLU, int8 rule) and stores it in the layout the MMA's B
// operand wants, chunk by chunk:
//   chunk c: [block 0..15][Mpad rows x 16 B]   then   [block 0..15][Mpad] float scales / 16 * 2^39
// Rows >= M and k-blocks >= K/16 are zero with scale 0.  Grid (ceil(nkb_pad / 256), Mpad), 256 threads.
// ----------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) prep_x_kernel(unsigned char* xb, const GemvArgs a, int M, int Mpad,
                                                     int nchunks) {
    __shared__ float part[8];
    __shared__ float rstd_s;
    const int m = blockIdx.y, t = threadIdx.x;
    const int nkb = a.K / 16;
    float rstd = 1.f;
    const bool needs_norm = (a.xkind == kXFloatNorm);
    if (needs_norm && m < M) {
        float ss = 0.f;
        const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(a.x) + (size_t)m * a.x_stride);
        for (int i = t; i < a.K / 4; i += 256) {
            const float4 f = __ldg(p + i);
            ss = fmaf(f.x, f.x, ss); ss = fmaf(f.y, f.y, ss); ss = fmaf(f.z, f.z, ss); ss = fmaf(f.w, f.w, ss);
        }
        ss = warp_sum(ss);
        if ((t & 31) == 0) part[t >> 5] = ss;
        __syncthreads();
        if (t == 0) {
            float tot = 0.f;
            for (int w = 0; w < 8; ++w) tot += part[w];
            rstd_s = rsqrtf(tot / (float)a.K + a.eps);
        }
        __syncthreads();
        rstd = rstd_s;
    }
    const int kb = blockIdx.x * 256 + t;
    if (kb >= nchunks * kBlocksPerChunk) return;
    uint32_t e[2] = {0, 0}, o[2] = {0, 0};
    float s = 0.f;
    if (m < M && kb < nkb) make_xblock(a, m, kb, rstd, e, o, s);
    const int c = kb / kBlocksPerChunk, b = kb % kBlocksPerChunk;
    unsigned char* chunk = xb + (size_t)c * xb_chunk_bytes(Mpad);
    *reinterpret_cast<uint4*>(chunk + ((size_t)b * Mpad + m) * 16) = make_uint4(e[0], o[0], e[1], o[1]);
    reinterpret_cast<float*>(chunk + (size_t)b_chunk_bytes(Mpad))[b * Mpad + m] = s * kXScaleUp;
}

// The same quantize for the streaming kernels (2 to 16 sequences): plain int8 [M][K] and fp32 scales [M][K/16], the
// layout of pre-quantized activations.  Without it every CTA of the GEMV quantizes all M x K activations itself
// (RMSNorm or SwiGLU included), which at 8 sequences costs more than the weight stream of the per-layer matrices
// (measured, 8B shape, 8 sequences: QKV 18.6 -> 10.0 us, gate+up 31.1 -> 22.6, down with SwiGLU 45.5 -> 18.4 without the
// prologue).  Grid (ceil(K / 1024), M), 256 threads; starts early under programmatic dependent launch.
__global__ void __launch_bounds__(256) prep_plain_kernel(int8_t* xq, float* xs, const GemvArgs a, int M) {
    __shared__ float part[8];
    __shared__ float rstd_s;
    pdl_trigger();
    pdl_wait();   // the activations come from the kernel before
    const int m = blockIdx.y, t = threadIdx.x;
    float rstd = 1.f;
    if (a.xkind == kXFloatNorm) {
        float ss = 0.f;
        const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(a.x) + (size_t)m * a.x_stride);
        for (int i = t; i < a.K / 4; i += 256) {
            const float4 f = __ldg(p + i);
            ss = fmaf(f.x, f.x, ss); ss = fmaf(f.y, f.y, ss); ss = fmaf(f.z, f.z, ss); ss = fmaf(f.w, f.w, ss);
        }
        ss = warp_sum(ss);
        if ((t & 31) == 0) part[t >> 5] = ss;
        __syncthreads();
        if (t == 0) {
            float tot = 0.f;
            for (int w = 0; w < 8; ++w) tot += part[w];
            rstd_s = rsqrtf(tot / (float)a.K + a.eps);
        }
        __syncthreads();
        rstd = rstd_s;
    }
    // Four consecutive elements per thread, four threads per k-block (K % 32 == 0, so a block's threads are valid or
    // not together); the element arithmetic is that of make_xblock, the rounding that of quantize_block.
    const int e0 = (blockIdx.x * 256 + t) * 4;
    const bool valid = e0 < a.K;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (valid) {
        if (a.xkind == kXHalf) {
            const uint2 u = __ldg(reinterpret_cast<const uint2*>(static_cast<const __half*>(a.x) + (size_t)m * a.x_stride + e0));
            const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
            const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
            v[0] = f0.x; v[1] = f0.y; v[2] = f1.x; v[3] = f1.y;
        } else {
            const float4 f = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(a.x) + (size_t)m * a.x_stride + e0));
            v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
            if (a.xkind == kXFloatNorm) {
                const float4 gw = __ldg(reinterpret_cast<const float4*>(a.norm_w + e0));
                v[0] = v[0] * gw.x * rstd; v[1] = v[1] * gw.y * rstd; v[2] = v[2] * gw.z * rstd; v[3] = v[3] * gw.w * rstd;
            } else if (a.xkind == kXSwiglu) {
                const float4 u = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(a.x2) + (size_t)m * a.x_stride + e0));
                v[0] = silu_mul(v[0], u.x); v[1] = silu_mul(v[1], u.y); v[2] = silu_mul(v[2], u.z); v[3] = silu_mul(v[3], u.w);
            }
        }
    }
    float am = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
    am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 1));
    am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 2));
    if (!valid) return;
    const float sc = quant_scale_i8(am);
    const float rcp = 1.0f / sc;
    uint32_t qb[4];
    bool exact_needed = !(am < 3.0e38f);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float r = v[i] * rcp;
        const float mg = r + kMagicFloat;
        const float ri = mg - kMagicFloat;
        exact_needed |= !(fabsf(fabsf(r - ri) - 0.5f) > 3e-5f);
        qb[i] = __float_as_uint(mg);
    }
    if (exact_needed) {
#pragma unroll
        for (int i = 0; i < 4; ++i) qb[i] = (uint32_t)quant_i8(v[i], sc);
    }
    *reinterpret_cast<uint32_t*>(xq + (size_t)m * a.K + e0) = prmt(prmt(qb[0], qb[1], 0x0040), prmt(qb[2], qb[3], 0x0040), 0x5410);
    if ((t & 3) == 0) xs[(size_t)m * (a.K / 16) + (e0 >> 4)] = sc;
}

// ----------------------------------------------------------------------------------------------------------
// Shared memory map of the MMA kernel (offsets from the 1024-aligned base).
// ----------------------------------------------------------------------------------------------------------
// A TMA box brings 128 rows x (128 * SUB) bytes: SUB consecutive 256-k chunks of every row in one request, so
// that DRAM sees 256- or 512-byte runs per row instead of 128-byte ones (which measured at a fifth of the
// bandwidth).  Unpack, MMA and epilogue still work chunk by chunk.
__host__ __device__ constexpr int sub_chunks(int Mpad) { return Mpad > 0 ? 2 : 2; }
__host__ __device__ constexpr int packed_slots(int Mpad) { return Mpad <= 16 ? 3 : 2; }
// The activation ring runs deeper than the operand ring: its slots are refilled from L2 only after the MMAs that
// read them retire, and with two slots that latency was the period of the whole pipeline.
__host__ __device__ constexpr int b_slots(int Mpad) { return Mpad <= 32 ? 4 : 3; }
__host__ __device__ constexpr int s_slots(int Mpad) { return Mpad <= 32 ? 4 : 3; }
__host__ __device__ constexpr int packed_slot_bytes(int Mpad) { return kRows * 128 * sub_chunks(Mpad); }

struct Smem {
    static constexpr int kBars = 0;                                      // mbarriers, 8 B each
    static constexpr int kTmemPtr = 512;                                 // TMEM base address from tcgen05.alloc
    static constexpr int kAbort = 516;
    static constexpr int kLast = 520;
    static constexpr int kPacked = 1024;                                 // packed_slots x packed_slot_bytes
    __host__ __device__ static constexpr int a_off(int Mpad) { return kPacked + packed_slots(Mpad) * packed_slot_bytes(Mpad); }
    __host__ __device__ static constexpr int b_off(int Mpad) { return a_off(Mpad) + kSA * kAStageBytes; }
    __host__ __device__ static constexpr int scales(int Mpad) { return b_off(Mpad) + b_slots(Mpad) * b_chunk_bytes(Mpad); }
    __host__ __device__ static constexpr int scale_slot_bytes(int Mpad) { return kBlocksPerChunk * Mpad * 4; }  // x_sc / 16
    __host__ __device__ static constexpr int wscales(int Mpad) { return scales(Mpad) + s_slots(Mpad) * scale_slot_bytes(Mpad); }
    __host__ __device__ static constexpr int const_a(int Mpad) { return wscales(Mpad) + kSW * kWScaleBytes; }  // 128 rows x 16 B of -128
    __host__ __device__ static constexpr int const_b(int Mpad) { return const_a(Mpad) + kRows * 16; }           // Mpad rows x 16 B of -127
    __host__ __device__ static constexpr int total(int Mpad) { return const_b(Mpad) + Mpad * 16; }
};
// The 512 accumulator columns form a ring of four groups: the MMAs of a group are issued as soon as every epilogue
// warp has read the group four back, so a slow warp delays the tensor core only after three groups of slack (with
// two groups the epilogue waited about 400 cycles for the next group's MMAs at every group boundary).
constexpr int kGroups = 2, kGroupCols = 512 / kGroups;
// barrier indices
enum : int {
    kFullP = 0,                 // + slot (up to 4): packed nibbles landed
    kEmptyP = kFullP + 4,       // packed slot unpacked
    kReadyA = kEmptyP + 4,      // + slot (kSA): int8 operand written
    kFreeAB = kReadyA + kSA,    // MMAs that read the operand slot have completed
    kFullB = kFreeAB + kSA,     // + slot (up to 4): activations landed
    kFreeB = kFullB + 4,        // MMAs that read the activation slot have completed
    kFullS = kFreeB + 4,        // + slot (up to 4): scales landed
    kEmptyS = kFullS + 4,       // scales consumed by the epilogue
    kDFull = kEmptyS + 4,       // + group (kGroups): accumulator group complete
    kDEmpty = kDFull + kGroups, // accumulator group read out
    kFullW = kDEmpty + kGroups,       // + slot (kSW): weight scales of a chunk landed
    kEmptyW = kFullW + kSW,     // weight scales consumed
    kNumBars = kEmptyW + kSW,
};

template <int NMMA>
__global__ void __launch_bounds__(kThreads, 1)
gemm_w4a8_tc_kernel(const __grid_constant__ CUtensorMap map_w, const TcArgs a) {
    constexpr int GB = kGroupCols / NMMA;               // k-blocks per accumulator group
    constexpr int GPC = kBlocksPerChunk / GB;           // groups per chunk
    constexpr int SUB = sub_chunks(NMMA), SPS = packed_slots(NMMA), PSLOT = packed_slot_bytes(NMMA);
    constexpr int SB = b_slots(NMMA), SS = s_slots(NMMA);
    extern __shared__ __align__(1024) unsigned char smem[];
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int units = ((a.N + kRows - 1) / kRows) * a.ksplit;   // (row tile, K part) pairs, walked round-robin
    auto unit_range = [&](int u, int& tile, int& kpart, int& c0, int& nloc) {
        tile = u / a.ksplit;
        kpart = u - tile * a.ksplit;
        const int nsuper = (a.nchunks + SUB - 1) / SUB;  // K parts begin on box boundaries
        c0 = SUB * (int)(((long long)nsuper * kpart) / a.ksplit);
        const int c1 = min(a.nchunks, SUB * (int)(((long long)nsuper * (kpart + 1)) / a.ksplit));
        nloc = c1 - c0;
    };

    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Smem::kBars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + Smem::kAbort);
    volatile uint32_t* tmem_ptr = reinterpret_cast<volatile uint32_t*>(smem + Smem::kTmemPtr);
    auto bar = [&](int i) { return smem_u32(&bars[i]); };
    auto wait = [&](int i, uint32_t parity) {
        if (mbar_try_wait(bar(i), parity)) return true;   // the common case costs one probe
        if (*abort_flag) return false;
        if (!mbar_wait(bar(i), parity)) { *abort_flag = 1; return false; }
        return true;
    };
    const int s_off = Smem::scales(NMMA);
    const int s_slot = Smem::scale_slot_bytes(NMMA);
    const int b_slot = b_chunk_bytes(NMMA);

    if (t == 0) {
        for (int i = 0; i < 4; ++i) { mbar_init(bar(kFullP + i), 1); mbar_init(bar(kEmptyP + i), 4); }
        for (int i = 0; i < kSA; ++i) { mbar_init(bar(kReadyA + i), 4); mbar_init(bar(kFreeAB + i), 1); }
        for (int i = 0; i < 4; ++i) { mbar_init(bar(kFullB + i), 1); mbar_init(bar(kFreeB + i), 1); }
        for (int i = 0; i < 4; ++i) { mbar_init(bar(kFullS + i), 1); mbar_init(bar(kEmptyS + i), kEpiWarps); }
        for (int i = 0; i < kSW; ++i) { mbar_init(bar(kFullW + i), 64); mbar_init(bar(kEmptyW + i), kEpiWarps); }
        for (int i = 0; i < kGroups; ++i) { mbar_init(bar(kDFull + i), 1); mbar_init(bar(kDEmpty + i), kEpiWarps); }
        *abort_flag = 0;
        mbar_fence_init();
    }
    // the constant second K step of both operands (the MMA reads them through the async proxy)
    for (int i = t; i < kRows * 4; i += kThreads) reinterpret_cast<uint32_t*>(smem + Smem::const_a(NMMA))[i] = 0x80808080u;
    for (int i = t; i < NMMA * 4; i += kThreads) reinterpret_cast<uint32_t*>(smem + Smem::const_b(NMMA))[i] = 0x81818181u;
    fence_proxy_async();
    if (warp == 0) {
        tmem_alloc(smem_u32(smem + Smem::kTmemPtr), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_ptr;

    if (warp == 0) {
        // ------------------------------------------------------------------------------------ producer
        if (lane == 0) {
            int n = 0, np = 0;  // chunks / boxes issued so far by this CTA: ring slots and phases follow them
            bool ok = true;
            for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
                int tile, kpart, c0, nloc;
                unit_range(u, tile, kpart, c0, nloc);
                const int row0 = tile * kRows;
                for (int i = 0; i < nloc; ++i, ++n) {
                    const int c = c0 + i;
                    const int sb = n % SB, ss = n % SS;
                    if (!wait(kEmptyS + ss, ((n / SS) & 1) ^ 1)) { ok = false; break; }
                    unsigned char* sslot = smem + s_off + ss * s_slot;
                    const unsigned char* xchunk = a.xb + (size_t)c * xb_chunk_bytes(NMMA);
                    if (a.ablate & 32) {
                        mbar_arrive(bar(kFullS + ss));
                    } else {
                        mbar_expect_tx(bar(kFullS + ss), s_slot);
                        bulk_g2s_plain(smem_u32(sslot), xchunk + b_slot, s_slot, bar(kFullS + ss));
                    }
                    if (i % SUB == 0) {  // a new box: SUB chunks of packed nibbles at once
                        const int sp = np % SPS;
                        if (!wait(kEmptyP + sp, ((np / SPS) & 1) ^ 1)) { ok = false; break; }
                        if (a.ablate & 4) {
                            mbar_arrive(bar(kFullP + sp));
                        } else {
                            mbar_expect_tx(bar(kFullP + sp), PSLOT);
                            tma_load_2d(smem_u32(smem + Smem::kPacked + sp * PSLOT), &map_w,
                                        c * (kKc / 2) / a.map_elem, row0, bar(kFullP + sp));
                        }
                        TC_TL(0, np);
                        ++np;
                    }
                    if (!wait(kFreeB + sb, ((n / SB) & 1) ^ 1)) { ok = false; break; }
                    TC_TL(1, n);
                    if (a.ablate & 16) {
                        mbar_arrive(bar(kFullB + sb));
                    } else {
                        mbar_expect_tx(bar(kFullB + sb), b_slot);
                        bulk_g2s_plain(smem_u32(smem + Smem::b_off(NMMA) + sb * b_slot), xchunk, b_slot, bar(kFullB + sb));
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = idesc_i8(NMMA);
            const uint32_t const_a = smem_u32(smem + Smem::const_a(NMMA)), const_b = smem_u32(smem + Smem::const_b(NMMA));
            int gcount = 0, n = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
                int tile, kpart, c0, nloc;
                unit_range(u, tile, kpart, c0, nloc);
                for (int i = 0; i < nloc && ok; ++i, ++n) {
                    const int sa = n % kSA, sb = n % SB;
                    if (!wait(kReadyA + sa, (n / kSA) & 1)) { ok = false; break; }
                    if (!wait(kFullB + sb, (n / SB) & 1)) { ok = false; break; }
                    tc_fence_after();
                    TC_TL(4, n);
                    const uint32_t a_base = smem_u32(smem + Smem::a_off(NMMA) + sa * kAStageBytes);
                    const uint32_t b_base = smem_u32(smem + Smem::b_off(NMMA) + sb * b_slot);
                    for (int g = 0; g < GPC && ok; ++g, ++gcount) {
                        const int dg = gcount % kGroups;
                        if (!wait(kDEmpty + dg, ((gcount / kGroups) & 1) ^ 1)) { ok = false; break; }
                        tc_fence_after();
                        TC_TL(5, gcount);
                        // one MMA per k-block: K step 1 = the block, K step 2 = the constants
#pragma unroll
                        for (int bi = 0; bi < GB; ++bi) {
                            const int b = g * GB + bi;
                            const uint32_t a_addr = a_base + b * kABlockStride;
                            const uint64_t da = smem_desc(a_addr, const_a - a_addr, 128);
                            const uint32_t b_addr = b_base + b * NMMA * 16;
                            const uint64_t db = smem_desc(b_addr, const_b - b_addr, 128);
                            if (!(a.ablate & 8)) tc_mma_i8(tmem + dg * kGroupCols + bi * NMMA, da, db, idesc, 0u);
                        }
                        tc_commit(bar(kDFull + dg));
                    }
                    if (ok) {
                        tc_commit(bar(kFreeAB + sa));
                        tc_commit(bar(kFreeB + sb));
                    }
                }
            }
        }
    } else if (warp == 2 || warp == 3) {
        // ------------------------------------------------------------------------------------ weight-scale loader
        // The 16 scales of a row for one chunk are 32 bytes at a row pitch that is only 4-byte aligned in general, so
        // they come through 4-byte cp.async copies (zero-filled past the end of K), two rows per thread, eight
        // chunks ahead of the epilogue; completion is signalled on the slot's mbarrier by the copies themselves.
        const int lt = t - 64;  // 0..63
        int n = 0;
        bool ok = true;
        for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
            int tile, kpart, c0, nloc;
            unit_range(u, tile, kpart, c0, nloc);
            for (int i = 0; i < nloc; ++i, ++n) {
                const int sw = n % kSW;
                if (!wait(kEmptyW + sw, ((n / kSW) & 1) ^ 1)) { ok = false; break; }
                if (lt == 0) TC_TL(10, n);
                unsigned char* slot = smem + Smem::wscales(NMMA) + sw * kWScaleBytes;
#pragma unroll
                for (int rr = 0; rr < ((a.ablate & 64) ? 0 : 2); ++rr) {
                    const int r = lt * 2 + rr;
                    const int grow = min(tile * kRows + r, a.N - 1);
                    const uint32_t* src = reinterpret_cast<const uint32_t*>(a.Wsc + (size_t)grow * a.nkb) + (c0 + i) * 8;
                    const uint32_t dst = smem_u32(slot + r * 32);
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        const bool in = 2 * ((c0 + i) * 8 + q) < a.nkb;
                        cp_async4(dst + 4 * q, in ? src + q : src, in ? 4u : 0u);
                    }
                }
                cp_async_arrive(bar(kFullW + sw));
            }
        }
    } else if (warp >= 4 + kEpiWarps) {
        // ------------------------------------------------------------------------------------ unpack
        const int ut = t - (4 + kEpiWarps) * 32;  // 0..127
        int n = 0, np = 0;
        bool ok = true;
        for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
          int tile, kpart, c0, nloc;
          unit_range(u, tile, kpart, c0, nloc);
          for (int i = 0; i < nloc; ++i, ++n) {
            const int sub = i % SUB, sa = n % kSA;
            if (sub == 0) ++np;
            const int sp = (np - 1) % SPS;
            if (sub == 0 && !wait(kFullP + sp, ((np - 1) / SPS) & 1)) { ok = false; break; }
            if (!wait(kFreeAB + sa, ((n / kSA) & 1) ^ 1)) { ok = false; break; }
            if (ut == 0) TC_TL(2, n);
            const unsigned char* src = smem + Smem::kPacked + sp * PSLOT + sub * 128;
            unsigned char* dst = smem + Smem::a_off(NMMA) + sa * kAStageBytes;
            // All eight loads are issued before the first store: source and destination are both shared memory, so the
            // compiler would otherwise keep every load behind the previous iteration's stores and the loop would run
            // at one shared-memory round trip per iteration.
            // A quarter warp (one shared-memory phase of a 16-byte access) takes eight rows on a diagonal of 16-byte
            // columns: its reads fall in eight different bank groups (the column) and so do its writes (the row within
            // its group of eight).  With rows-then-columns order the stores hit every bank group four times.
            const int j = ut & 7, dg8 = (ut >> 3) & 7, rhi = ut >> 6;
            const int cc = (j + dg8) & 7;
            uint4 wv[8];
            if (!(a.ablate & 2)) {
#pragma unroll
            for (int it = 0; it < 8; ++it) {
                const int row = (rhi + 2 * it) * 8 + j;
                wv[it] = *reinterpret_cast<const uint4*>(src + row * (128 * SUB) + cc * 16);
            }
#pragma unroll
            for (int it = 0; it < 8; ++it) {
                const uint4 w = wv[it];
                uint4 o0, o1;
                nibbles_to_s8x16(w.x, o0.x, o0.y);
                nibbles_to_s8x16(w.y, o0.z, o0.w);
                nibbles_to_s8x16(w.z, o1.x, o1.y);
                nibbles_to_s8x16(w.w, o1.z, o1.w);
                unsigned char* d0 = dst + (2 * cc) * kABlockStride + (rhi + 2 * it) * 128 + j * 16;
                *reinterpret_cast<uint4*>(d0) = o0;
                *reinterpret_cast<uint4*>(d0 + kABlockStride) = o1;
            }
            }
            // one arrival per warp: hundreds of per-thread arrivals on one barrier serialise in shared memory
            fence_proxy_async();
            __syncwarp();
            if (ut == 0) TC_TL(3, n);
            if (lane == 0) {
                mbar_arrive(bar(kReadyA + sa));
                if (sub == SUB - 1 || i == nloc - 1) mbar_arrive(bar(kEmptyP + sp));  // the box is used up
            }
          }
        }
    } else if (warp >= 4) {
        // ------------------------------------------------------------------------------------ epilogue
        constexpr int CW = NMMA / 2;                            // sequences (columns of a block) per thread
        constexpr int PW = CW < 16 ? CW : 16;                   // ... read and scaled in pieces of PW columns of
        constexpr int PB = 32 / CW < 1 ? 1 : 32 / CW;           // PB consecutive k-blocks (32 values unless CW is 32)
        constexpr int PP = CW / PW;                             // column pieces per k-block (2 for 64 sequences)
        constexpr int NP = kBlocksPerChunk * PP / PB;           // pieces per chunk
        static_assert(GB % PB == 0 && NP % 2 == 0 && (PP == 1 || PB == 1), "piece shape");
        const int part = (warp - 4) >> 2;                       // sequences [part * CW, part * CW + CW)
        const int row = (warp & 3) * 32 + lane;                 // weight row of the tile = TMEM lane
        const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16) + part * CW;
        int gcount = 0, n = 0;                                  // accumulator groups / chunks consumed so far
        bool ok = true;
        uint32_t v0[PB * PW], v1[PB * PW];                      // the piece being scaled and the one being read
        for (int u = blockIdx.x; u < units; u += gridDim.x) {
            int tile, kpart, c0, nloc;
            unit_range(u, tile, kpart, c0, nloc);
            const int row0 = tile * kRows;
            unsigned long long acc2[CW / 2];                    // packed pairs of fp32 accumulators
#pragma unroll
            for (int j = 0; j < CW / 2; ++j) acc2[j] = 0ull;
            for (int i = 0; i < nloc && ok; ++i, ++n, gcount += GPC) {
                const int ss = n % SS;
                const int sw = n % kSW;
                ok = ok && wait(kFullW + sw, (n / kSW) & 1);
                uint32_t wcur[8];                               // this row's 16 weight scales of the chunk
                {
                    const uint4* wp = reinterpret_cast<const uint4*>(smem + Smem::wscales(NMMA) + sw * kWScaleBytes + row * 32);
                    const uint4 w0 = wp[0], w1 = wp[1];
                    wcur[0] = w0.x; wcur[1] = w0.y; wcur[2] = w0.z; wcur[3] = w0.w;
                    wcur[4] = w1.x; wcur[5] = w1.y; wcur[6] = w1.z; wcur[7] = w1.w;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(kEmptyW + sw));
                ok = ok && wait(kFullS + ss, (n / SS) & 1);
                if (t == 128) TC_TL(6, n);
                const float* sx = reinterpret_cast<const float*>(smem + s_off + ss * s_slot) + part * CW;
                // Piece p of this chunk: k-blocks [b0, b0 + PB) with b0 = (p / PP) * PB, columns (p % PP) * PW.  Block b
                // lives in accumulator group gcount + b / GB at columns (b % GB) * NMMA.
                auto group_ready = [&](int b) {   // before the first read of a group: its MMAs have completed
                    const int G = gcount + b / GB;
                    ok = ok && wait(kDFull + G % kGroups, (G / kGroups) & 1);
                    tc_fence_after();
                    if (t == 128) TC_TL(7, G);
                };
                auto read_piece = [&](int p, uint32_t (&dst)[PB * PW]) {
                    const int b0 = (p / PP) * PB;
                    if (b0 % GB == 0 && p % PP == 0) group_ready(b0);
#pragma unroll
                    for (int j = 0; j < PB; ++j) {
                        const int b = b0 + j;
                        tmem_ld_cols<PW>(lane_addr + ((gcount + b / GB) % kGroups) * kGroupCols + (b % GB) * NMMA + (p % PP) * PW,
                                         *reinterpret_cast<uint32_t(*)[PW]>(&dst[j * PW]));
                    }
                };
                // One piece: its values are in `cur` (read issued earlier).  Hand the accumulator group back after its
                // last piece (before the next read is issued: the fence waits for reads in flight), start the read of the
                // next piece into `nxt`, then scale and accumulate `cur`.
                auto step = [&](int p, uint32_t (&cur)[PB * PW], uint32_t (&nxt)[PB * PW]) {
                    const int b0 = (p / PP) * PB, h = p % PP;
                    tmem_wait_ld();
                    if (h == PP - 1 && (b0 + PB) % GB == 0) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar(kDEmpty + (gcount + b0 / GB) % kGroups));
                        if (t == 128) TC_TL(8, gcount + b0 / GB);
                    }
                    if (p + 1 < NP || i + 1 < nloc) read_piece(p + 1, nxt);   // p + 1 == NP: the unit's next chunk
                    if (a.ablate & 1) { acc2[0] += cur[0]; return; }
#pragma unroll
                    for (int j = 0; j < PB; ++j) {
                        const int b = b0 + j;
                        const float2 wf = __half22float2(*reinterpret_cast<const __half2*>(&wcur[b >> 1]));
                        const float w = (b & 1) ? wf.y : wf.x;
                        const unsigned long long W2 = pack2(w * kWScaleUp), CN2 = pack2(w * kOffsetTerm);   // both exact
#pragma unroll
                        for (int q = 0; q < PW / 4; ++q) {
                            const ulonglong2 s4 = *reinterpret_cast<const ulonglong2*>(sx + b * NMMA + h * PW + 4 * q);
                            scale_acc2(acc2[h * (PW / 2) + 2 * q], cur[j * PW + 4 * q], cur[j * PW + 4 * q + 1], W2, CN2, s4.x);
                            scale_acc2(acc2[h * (PW / 2) + 2 * q + 1], cur[j * PW + 4 * q + 2], cur[j * PW + 4 * q + 3], W2, CN2, s4.y);
                        }
                    }
                };
                if (i == 0) read_piece(0, v0);   // nothing was read ahead across the unit boundary
#pragma unroll
                for (int p = 0; p < NP; p += 2) {
                    step(p, v0, v1);
                    step(p + 1, v1, v0);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(kEmptyS + ss));
                if (t == 128) TC_TL(9, n);
            }
            float acc[CW];
#pragma unroll
            for (int j = 0; j < CW / 2; ++j) {
                acc[2 * j] = __uint_as_float((uint32_t)acc2[j]);
                acc[2 * j + 1] = __uint_as_float((uint32_t)(acc2[j] >> 32));
            }

            // ---- results: straight to y, or through the K-split partial buffer with a last-arriver sum
            const int grow = row0 + row;
            const int mbase = part * CW;
            if (a.ksplit == 1) {
                if (grow < a.N && ok && !*abort_flag) {
#pragma unroll
                    for (int j = 0; j < CW; ++j)
                        if (mbase + j < a.M) {
                            const size_t yi = (size_t)(mbase + j) * a.y_stride + grow;
                            a.y[yi] = a.residual ? acc[j] + a.residual[yi] : acc[j];
                        }
                }
            } else {
                float* mine = a.partial + ((size_t)(tile * a.ksplit + kpart) * NMMA) * kRows;
#pragma unroll
                for (int j = 0; j < CW; ++j) mine[(mbase + j) * kRows + row] = acc[j];
                __threadfence();
                asm volatile("bar.sync 1, %0;" ::"n"(kEpiWarps * 32) : "memory");
                volatile int* last = reinterpret_cast<volatile int*>(smem + Smem::kLast);
                if (t == 128) *last = (atomicAdd(&a.tickets[tile], 1u) == (unsigned)a.ksplit - 1) ? 1 : 0;
                asm volatile("bar.sync 1, %0;" ::"n"(kEpiWarps * 32) : "memory");
                if (*last) {
                    __threadfence();
                    if (grow < a.N && !*abort_flag) {
                        for (int j = 0; j < CW && mbase + j < a.M; ++j) {
                            float sum = 0.f;
                            for (int p = 0; p < a.ksplit; ++p)
                                sum += __ldcg(a.partial + ((size_t)(tile * a.ksplit + p) * NMMA + mbase + j) * kRows + row);
                            const size_t yi = (size_t)(mbase + j) * a.y_stride + grow;
                            a.y[yi] = a.residual ? sum + a.residual[yi] : sum;
                        }
                    }
                    asm volatile("bar.sync 1, %0;" ::"n"(kEpiWarps * 32) : "memory");
                    if (t == 128) a.tickets[tile] = 0;
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
    if (t == 0 && *abort_flag) atomicExch(a.status, kStatusMbarTimeout);
}

// ----------------------------------------------------------------------------------------------------------
// Host side
// ----------------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's tensor-map encoder, looked up through the runtime so that the library carries no link-time
// dependency on libcuda (it must load on machines without a driver).
static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// Per-device scratch: activation chunks, K-split partials, tickets (kept zero between calls).
static GrowScratch g_tc_scratch;
cudaError_t reserve_scratch(size_t bytes) {
    unsigned char* p = nullptr;
    return bytes ? g_tc_scratch.get(bytes, (size_t)16 << 20, nullptr, &p) : cudaSuccess;
}

constexpr size_t kTicketBytes = 65536;  // arrival counters: 16,384 row tiles; larger matrices are not K-split

// Quantizes the activations of a streaming-kernel call once (see prep_plain_kernel) into the scratch block and returns
// the pre-quantized operand.  Calls that go on to the tensor-core kernel do not use this (its own prep writes the same
// region).
cudaError_t prepare_plain(const GemvArgs& a, int M, cudaStream_t st, const int8_t** xq_out, const float** xs_out) {
    const size_t q_bytes = ((size_t)M * a.K + 255) & ~(size_t)255;
    const size_t s_bytes = (size_t)M * (a.K / 16) * sizeof(float);
    unsigned char* scratch = nullptr;
    cudaError_t e = g_tc_scratch.get(kTicketBytes + q_bytes + s_bytes, (size_t)16 << 20, st, &scratch);
    if (e != cudaSuccess) return e;
    int8_t* xq = reinterpret_cast<int8_t*>(scratch + kTicketBytes);
    float* xs = reinterpret_cast<float*>(scratch + kTicketBytes + q_bytes);
    const dim3 grid((a.K + 1023) / 1024, M);
    e = launch_pdl(prep_plain_kernel, grid, dim3(256), 0, st, xq, xs, a, M);
    count_launch(1);
    if (e != cudaSuccess) return e;
    *xq_out = xq;
    *xs_out = xs;
    return cudaPeekAtLastError();
}

static int g_tc_ksplit_override = 0;
void set_ksplit_override(int v) { g_tc_ksplit_override = v; }
static int g_tc_ablate = 0;
void set_ablate(int v) { g_tc_ablate = v; }

bool eligible(const GemvArgs& a, int M) {
    if (M < 1 || M > 64 || a.K % 32 != 0 || a.K < 32) return false;
    if ((reinterpret_cast<uintptr_t>(a.W) & 15) || (reinterpret_cast<uintptr_t>(a.Wsc) & 3)) return false;
    if (reinterpret_cast<uintptr_t>(a.x) & 15) return false;
    if (a.xkind != kXInt8 && a.xkind != kXHalf && a.xkind != kXFloat && a.xkind != kXFloatNorm && a.xkind != kXSwiglu)
        return false;
    return encode_fn() != nullptr;
}

template <int NMMA>
static cudaError_t launch_n(const CUtensorMap& map_w, const TcArgs& t, int grid, cudaStream_t st) {
    auto kern = gemm_w4a8_tc_kernel<NMMA>;
    static std::once_flag once[kMaxDevices];
    cudaError_t attr = cudaSuccess;
    std::call_once(once[current_device()], [&] {
        attr = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynSmem);
    });
    if (attr != cudaSuccess) return attr;
    kern<<<grid, kThreads, Smem::total(NMMA) + 1024, st>>>(map_w, t);
    count_launch(1);
    return cudaPeekAtLastError();
}

// Launch geometry and scratch layout of one call: [tickets][activation chunks][K-split partials].

struct TcLayout {
    int Mpad, nchunks, tiles, ksplit;
    size_t xb_off, part_off, part_bytes;
};
static TcLayout tc_layout(int M, int N, int K) {
    TcLayout l;
    l.Mpad = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    l.nchunks = (K + kKc - 1) / kKc;
    l.tiles = (N + kRows - 1) / kRows;
    const int sms = sm_count(current_device());
    int ksplit = g_tc_ksplit_override > 0 ? g_tc_ksplit_override : sms / l.tiles;  // whole waves of one CTA per SM
    if (ksplit > l.nchunks) ksplit = l.nchunks;
    if (ksplit < 1) ksplit = 1;
    l.ksplit = ksplit;
    const size_t xb_bytes = (size_t)l.nchunks * xb_chunk_bytes(l.Mpad);
    l.part_bytes = ksplit > 1 ? (size_t)l.tiles * ksplit * l.Mpad * kRows * sizeof(float) : 0;
    // The arrival counters own a region of fixed size at the front of the block: they must read zero at the start of
    // every call, and a region sized by the problem would let one call's activations lie where a later, larger call
    // expects its counters.
    if ((size_t)l.tiles * sizeof(unsigned int) > kTicketBytes) { l.ksplit = 1; l.part_bytes = 0; }
    l.xb_off = kTicketBytes;
    l.part_off = (l.xb_off + xb_bytes + 255) & ~(size_t)255;
    return l;
}
size_t scratch_bytes(int M, int N, int K) {
    if (M < 1 || N < 1 || K < 32) return 0;
    const TcLayout l = tc_layout(M < 64 ? M : 64, N, K);
    const size_t plain = kTicketBytes + (((size_t)M * K + 255) & ~(size_t)255) + (size_t)M * (K / 16) * sizeof(float);
    return l.part_off + l.part_bytes > plain ? l.part_off + l.part_bytes : plain;
}

// y = W . q8(prologue(x)) for 1..64 sequences on the tensor cores.  `a` carries the operands as for the streaming
// kernel (x kinds int8 / f16 / f32 / f32+norm / swiglu; binary16 weight scales).
cudaError_t launch(const GemvArgs& a, int M, cudaStream_t st) {
    const TcLayout lay = tc_layout(M, a.N, a.K);
    const int Mpad = lay.Mpad, nchunks = lay.nchunks, tiles = lay.tiles, ksplit = lay.ksplit;
    const int sms = sm_count(current_device());
    const size_t xb_off = lay.xb_off, part_off = lay.part_off, part_bytes = lay.part_bytes;
    unsigned char* scratch = nullptr;
    cudaError_t e = g_tc_scratch.get(part_off + part_bytes, (size_t)16 << 20, st, &scratch);
    if (e != cudaSuccess) return e;

    CUtensorMap map_w;
    // 4-byte elements: a box row is 128 * SUB bytes, beyond the 256-element limit of a byte-typed map
    const int box_bytes = 128 * sub_chunks(Mpad);
    const cuuint64_t dims[2] = {(cuuint64_t)(a.K / 8), (cuuint64_t)a.N};
    const cuuint64_t strides[1] = {(cuuint64_t)(a.K / 2)};
    const cuuint32_t box[2] = {(cuuint32_t)(box_bytes / 4), (cuuint32_t)kRows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = encode_fn()(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint8_t*>(a.W), dims, strides,
                                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;

    const dim3 pgrid((nchunks * kBlocksPerChunk + 255) / 256, Mpad);
    prep_x_kernel<<<pgrid, 256, 0, st>>>(scratch + xb_off, a, M, Mpad, nchunks);
    count_launch(1);
    e = cudaPeekAtLastError();
    if (e != cudaSuccess) return e;

    TcArgs t{};
    t.y = a.y; t.residual = a.residual; t.y_stride = a.y_stride;
    t.xb = scratch + xb_off;
    t.Wsc = static_cast<const __half*>(a.Wsc);
    t.nkb = a.K / 16;
    t.partial = reinterpret_cast<float*>(scratch + part_off);
    t.tickets = reinterpret_cast<unsigned int*>(scratch);
    t.status = a.status;
    t.N = a.N; t.M = M; t.Mpad = Mpad; t.nchunks = nchunks; t.ksplit = ksplit; t.map_elem = 4; t.ablate = g_tc_ablate;
#ifdef BW_GEMV_TIMELINE
    t.timeline = static_cast<long long*>(debug_timeline_ptr());
#endif
    const int grid = tiles * ksplit < sms ? tiles * ksplit : sms;  // persistent: one CTA per SM at most
    if (Mpad == 16) return launch_n<16>(map_w, t, grid, st);
    if (Mpad == 32) return launch_n<32>(map_w, t, grid, st);
    return launch_n<64>(map_w, t, grid, st);
}

}  // namespace tc
}  // namespace bw
