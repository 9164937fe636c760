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
namespace tc {

// ----------------------------------------------------------------------------------------------------------
// Activation prep: quantizes every 16-element k-block of every sequence once (the same make_xblock code as the
// streaming kernel's prologue: plain / RMSNorm / SwiGLU, int8 rule) and stores it in the layout the MMA's B
// operand wants, chunk by chunk:
//   chunk c: [block 0..15][row group 0..Mpad/8-1][8 rows][16 B]   then   [block 0..15][Mpad] float scales / 16
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
    reinterpret_cast<float*>(chunk + (size_t)kBlocksPerChunk * Mpad * 16)[b * Mpad + m] = s;
}

// ----------------------------------------------------------------------------------------------------------
// Shared memory map of the MMA kernel (offsets from the 1024-aligned base).
// ----------------------------------------------------------------------------------------------------------
struct Smem {
    static constexpr int kBars = 0;                                      // mbarriers, 8 B each
    static constexpr int kTmemPtr = 512;                                 // TMEM base address from tcgen05.alloc
    static constexpr int kAbort = 516;
    static constexpr int kLast = 520;
    static constexpr int kPacked = 1024;                                 // kSP x 16 KB
    static constexpr int kA = kPacked + kSP * kPackedBytes;              // kSA x 33,024 B
    static constexpr int kZero = kA + kSA * kAStageBytes;                // 2 KB of zeros (after every A tile)
    static constexpr int kB = kZero + kZeroBytes;                        // kSA x (16 blocks x Mpad x 16 B)
    __host__ __device__ static int scales(int Mpad) { return kB + kSA * kBlocksPerChunk * Mpad * 16; }
    __host__ __device__ static int scale_slot_bytes(int Mpad) { return kBlocksPerChunk * Mpad * 4; }  // x_sc / 16
    __host__ __device__ static int total(int Mpad) { return scales(Mpad) + kSS * scale_slot_bytes(Mpad); }
};
// barrier indices
enum : int {
    kFullP = 0,                 // + slot (kSP): packed nibbles landed
    kEmptyP = kFullP + kSP,     // packed slot unpacked
    kReadyA = kEmptyP + kSP,    // + slot (kSA): int8 operand written
    kFullB = kReadyA + kSA,     // activations landed
    kFreeAB = kFullB + kSA,     // MMAs that read the slot have completed
    kFullS = kFreeAB + kSA,     // + slot (kSS): scales landed
    kEmptyS = kFullS + kSS,     // scales consumed by the epilogue
    kDFull = kEmptyS + kSS,     // + group (2): accumulator group complete
    kDEmpty = kDFull + 2,       // accumulator group drained and refilled
    kNumBars = kDEmpty + 2,
};

template <int NMMA>
__global__ void __launch_bounds__(kThreads, 1)
gemm_w4a8_tc_kernel(const __grid_constant__ CUtensorMap map_w, const TcArgs a) {
    constexpr int GB = 256 / NMMA;                      // k-blocks per accumulator group (256 TMEM columns)
    constexpr int GPC = kBlocksPerChunk / GB;           // groups per chunk
    extern __shared__ __align__(1024) unsigned char smem[];
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int tile = blockIdx.x / a.ksplit, kpart = blockIdx.x % a.ksplit;
    const int c0 = (int)(((long long)a.nchunks * kpart) / a.ksplit);
    const int c1 = (int)(((long long)a.nchunks * (kpart + 1)) / a.ksplit);
    const int nloc = c1 - c0;
    const int row0 = tile * kRows;

    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Smem::kBars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + Smem::kAbort);
    volatile uint32_t* tmem_ptr = reinterpret_cast<volatile uint32_t*>(smem + Smem::kTmemPtr);
    auto bar = [&](int i) { return smem_u32(&bars[i]); };
    auto wait = [&](int i, uint32_t parity) {
        if (*abort_flag) return false;
        if (!mbar_wait(bar(i), parity)) { *abort_flag = 1; return false; }
        return true;
    };
    const int s_off = Smem::scales(NMMA);
    const int s_slot = Smem::scale_slot_bytes(NMMA);
    const int b_slot = kBlocksPerChunk * NMMA * 16;

    if (t == 0) {
        for (int i = 0; i < kSP; ++i) { mbar_init(bar(kFullP + i), 1); mbar_init(bar(kEmptyP + i), 128); }
        for (int i = 0; i < kSA; ++i) { mbar_init(bar(kReadyA + i), 128); mbar_init(bar(kFullB + i), 1); mbar_init(bar(kFreeAB + i), 1); }
        for (int i = 0; i < kSS; ++i) { mbar_init(bar(kFullS + i), 1); mbar_init(bar(kEmptyS + i), 128); }
        for (int i = 0; i < 2; ++i) { mbar_init(bar(kDFull + i), 1); mbar_init(bar(kDEmpty + i), 128); }
        *abort_flag = 0;
        mbar_fence_init();
    }
    for (int i = t; i < kZeroBytes / 4; i += kThreads) reinterpret_cast<uint32_t*>(smem + Smem::kZero)[i] = 0u;
    if (warp == 0) {
        tmem_alloc(smem_u32(smem + Smem::kTmemPtr), 512);
        tmem_relinquish();
    }
    fence_proxy_async();  // the zero region is read by the tensor core's shared-memory path
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_ptr;

    if (warp >= 4 && warp < 8) {
        // every accumulator column of this thread's lane starts at the magic pattern
        const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        for (int c = 0; c < 512; c += 16) tmem_st16_const(lane_addr + c, (uint32_t)kMagicInt);
        tmem_wait_st();
        tc_fence_before();
    }
    __syncthreads();
    tc_fence_after();

    if (warp == 0) {
        // ------------------------------------------------------------------------------------ producer
        if (lane == 0) {
            for (int i = 0; i < nloc; ++i) {
                const int c = c0 + i;
                const int sp = i % kSP, sa = i % kSA, ss = i % kSS;
                if (!wait(kEmptyS + ss, ((i / kSS) & 1) ^ 1)) break;
                unsigned char* sslot = smem + s_off + ss * s_slot;
                mbar_expect_tx(bar(kFullS + ss), s_slot);
                const unsigned char* xchunk = a.xb + (size_t)c * xb_chunk_bytes(NMMA);
                bulk_g2s_plain(smem_u32(sslot), xchunk + b_slot, s_slot, bar(kFullS + ss));
                if (!wait(kEmptyP + sp, ((i / kSP) & 1) ^ 1)) break;
                mbar_expect_tx(bar(kFullP + sp), kPackedBytes);
                tma_load_2d(smem_u32(smem + Smem::kPacked + sp * kPackedBytes), &map_w, c * (kKc / 2), row0, bar(kFullP + sp));
                if (!wait(kFreeAB + sa, ((i / kSA) & 1) ^ 1)) break;
                mbar_expect_tx(bar(kFullB + sa), b_slot);
                bulk_g2s_plain(smem_u32(smem + Smem::kB + sa * b_slot), xchunk, b_slot, bar(kFullB + sa));
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = idesc_i8(NMMA);
            const uint32_t zero_addr = smem_u32(smem + Smem::kZero);
            int gcount = 0;
            for (int i = 0; i < nloc; ++i) {
                const int sa = i % kSA;
                const uint32_t par = (i / kSA) & 1;
                if (!wait(kReadyA + sa, par)) break;
                if (!wait(kFullB + sa, par)) break;
                tc_fence_after();
                const uint32_t a_base = smem_u32(smem + Smem::kA + sa * kAStageBytes);
                const uint32_t b_base = smem_u32(smem + Smem::kB + sa * b_slot);
                bool ok = true;
                for (int g = 0; g < GPC && ok; ++g, ++gcount) {
                    const int dg = gcount & 1;
                    if (!wait(kDEmpty + dg, ((gcount >> 1) & 1) ^ 1)) { ok = false; break; }
                    tc_fence_after();
                    for (int bi = 0; bi < GB; ++bi) {
                        const int b = g * GB + bi;
                        const uint32_t a_addr = a_base + b * kABlockStride;
                        // A: first K step = the block, second K step = the zero region
                        const uint64_t da = smem_desc(a_addr, zero_addr - a_addr, 128);
                        // B: first K step = the block; the second multiplies zeros, any valid rows will do
                        const uint32_t b_addr = b_base + b * NMMA * 16;
                        const uint64_t db = smem_desc(b_addr, b == kBlocksPerChunk - 1 ? 0 : NMMA * 16, 128);
                        tc_mma_i8(tmem + dg * 256 + bi * NMMA, da, db, idesc);
                    }
                    tc_commit(bar(kDFull + dg));
                }
                if (!ok) break;
                tc_commit(bar(kFreeAB + sa));
            }
        }
    } else if (warp >= 8) {
        // ------------------------------------------------------------------------------------ unpack
        const int ut = t - 256;  // 0..127
        for (int i = 0; i < nloc; ++i) {
            const int sp = i % kSP, sa = i % kSA;
            if (!wait(kFullP + sp, (i / kSP) & 1)) break;
            if (!wait(kFreeAB + sa, ((i / kSA) & 1) ^ 1)) break;
            const unsigned char* src = smem + Smem::kPacked + sp * kPackedBytes;
            unsigned char* dst = smem + Smem::kA + sa * kAStageBytes;
#pragma unroll
            for (int it = 0; it < 8; ++it) {
                const int gidx = it * 128 + ut;       // 16-byte chunk of the packed tile
                const int row = gidx >> 3, cc = gidx & 7;
                const uint4 w = *reinterpret_cast<const uint4*>(src + gidx * 16);
                uint4 o0, o1;
                nibbles_to_s8x16(w.x, o0.x, o0.y);
                nibbles_to_s8x16(w.y, o0.z, o0.w);
                nibbles_to_s8x16(w.z, o1.x, o1.y);
                nibbles_to_s8x16(w.w, o1.z, o1.w);
                unsigned char* d0 = dst + (2 * cc) * kABlockStride + (row >> 3) * 128 + (row & 7) * 16;
                *reinterpret_cast<uint4*>(d0) = o0;
                *reinterpret_cast<uint4*>(d0 + kABlockStride) = o1;
            }
            fence_proxy_async();
            mbar_arrive(bar(kReadyA + sa));
            mbar_arrive(bar(kEmptyP + sp));
        }
    } else if (warp >= 4) {
        // ------------------------------------------------------------------------------------ epilogue
        const int row = (warp & 3) * 32 + lane;                 // weight row of the tile = TMEM lane
        const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        float acc[NMMA];
#pragma unroll
        for (int j = 0; j < NMMA; ++j) acc[j] = 0.f;
        int gcount = 0;
        bool ok = true;
        // Weight scales of this thread's row come straight from global memory (a row's scales are only 4-byte
        // aligned in general, which rules out bulk copies); the next chunk's 16 are fetched while the current
        // chunk is scaled.  Blocks past the end of K read as scale 0.
        const int grow_s = min(row0 + row, a.N - 1);
        const uint32_t* wrow = reinterpret_cast<const uint32_t*>(a.Wsc + (size_t)grow_s * a.nkb);
        uint32_t wnext[8];
        auto fetch_scales = [&](int c) {
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const int b2 = c * 8 + q;  // pair index
                wnext[q] = (2 * b2 < a.nkb) ? __ldg(wrow + b2) : 0u;
            }
        };
        if (nloc > 0) fetch_scales(c0);
        for (int i = 0; i < nloc && ok; ++i) {
            const int ss = i % kSS;
            float wsc[kBlocksPerChunk];
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&wnext[q]));
                wsc[2 * q] = f.x; wsc[2 * q + 1] = f.y;
            }
            if (i + 1 < nloc) fetch_scales(c0 + i + 1);
            if (!wait(kFullS + ss, (i / kSS) & 1)) break;
            const float* sx = reinterpret_cast<const float*>(smem + s_off + ss * s_slot);
#pragma unroll
            for (int g = 0; g < GPC; ++g, ++gcount) {
                const int dg = gcount & 1;
                if (!wait(kDFull + dg, (gcount >> 1) & 1)) { ok = false; break; }
                tc_fence_after();
#pragma unroll
                for (int bi = 0; bi < GB; ++bi) {
                    const int b = g * GB + bi;
                    const float w = wsc[b];
                    const float cneg = -kMagicFloat * w;       // exact: a binary16 scale times 1.5 * 2^23
#pragma unroll
                    for (int cb = 0; cb < NMMA; cb += 16) {
                        uint32_t v[16];
                        tmem_ld16(lane_addr + dg * 256 + bi * NMMA + cb, v);
                        tmem_wait_ld();
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const float4 s4 = *reinterpret_cast<const float4*>(sx + b * NMMA + cb + 4 * q);
                            acc[cb + 4 * q + 0] = fmaf(fmaf(__uint_as_float(v[4 * q + 0]), w, cneg), s4.x, acc[cb + 4 * q + 0]);
                            acc[cb + 4 * q + 1] = fmaf(fmaf(__uint_as_float(v[4 * q + 1]), w, cneg), s4.y, acc[cb + 4 * q + 1]);
                            acc[cb + 4 * q + 2] = fmaf(fmaf(__uint_as_float(v[4 * q + 2]), w, cneg), s4.z, acc[cb + 4 * q + 2]);
                            acc[cb + 4 * q + 3] = fmaf(fmaf(__uint_as_float(v[4 * q + 3]), w, cneg), s4.w, acc[cb + 4 * q + 3]);
                        }
                    }
                }
                // hand the group back holding the magic pattern again
#pragma unroll
                for (int c = 0; c < 256; c += 16) tmem_st16_const(lane_addr + dg * 256 + c, (uint32_t)kMagicInt);
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive(bar(kDEmpty + dg));
            }
            if (ok) mbar_arrive(bar(kEmptyS + ss));
        }

        // ---- results: straight to y, or through the K-split partial buffer with a last-arriver sum
        const int grow = row0 + row;
        if (a.ksplit == 1) {
            if (grow < a.N && !*abort_flag) {
#pragma unroll
                for (int m = 0; m < NMMA; ++m)
                    if (m < a.M) {
                        const size_t yi = (size_t)m * a.y_stride + grow;
                        a.y[yi] = a.residual ? acc[m] + a.residual[yi] : acc[m];
                    }
            }
        } else {
            float* mine = a.partial + ((size_t)(tile * a.ksplit + kpart) * NMMA) * kRows;
#pragma unroll
            for (int m = 0; m < NMMA; ++m) mine[m * kRows + row] = acc[m];
            __threadfence();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            volatile int* last = reinterpret_cast<volatile int*>(smem + Smem::kLast);
            if (t == 128) *last = (atomicAdd(&a.tickets[tile], 1u) == (unsigned)a.ksplit - 1) ? 1 : 0;
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (*last) {
                __threadfence();
                if (grow < a.N && !*abort_flag) {
                    for (int m = 0; m < a.M; ++m) {
                        float sum = 0.f;
                        for (int p = 0; p < a.ksplit; ++p)
                            sum += __ldcg(a.partial + ((size_t)(tile * a.ksplit + p) * NMMA + m) * kRows + row);
                        const size_t yi = (size_t)m * a.y_stride + grow;
                        a.y[yi] = a.residual ? sum + a.residual[yi] : sum;
                    }
                }
                if (t == 128) a.tickets[tile] = 0;
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
    if (t == 0 && *abort_flag) atomicExch(&g_status, kStatusMbarTimeout);
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

struct TcScratch {
    unsigned char* ptr = nullptr;
    size_t bytes = 0;
};
static TcScratch g_tc_scratch[kMaxDevices];
static std::mutex g_tc_mu;

// Grow-only per-device scratch: activation chunks, K-split partials, tickets (kept zero between calls).
static cudaError_t tc_scratch(size_t bytes, unsigned char** out) {
    std::lock_guard<std::mutex> lk(g_tc_mu);
    TcScratch& s = g_tc_scratch[current_device()];
    if (s.bytes < bytes) {
        if (s.ptr) cudaFree(s.ptr);
        s.ptr = nullptr; s.bytes = 0;
        const size_t want = bytes < ((size_t)16 << 20) ? ((size_t)16 << 20) : bytes;
        cudaError_t e = cudaMalloc(&s.ptr, want);
        if (e != cudaSuccess) return e;
        e = cudaMemset(s.ptr, 0, want);
        if (e != cudaSuccess) return e;
        s.bytes = want;
    }
    *out = s.ptr;
    return cudaSuccess;
}

static int g_tc_ksplit_override = 0;
void set_ksplit_override(int v) { g_tc_ksplit_override = v; }

int read_clear_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_status, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_status, &zero, sizeof(int));
    }
    return v;
}

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

// y = W . q8(prologue(x)) for 1..64 sequences on the tensor cores.  `a` carries the operands as for the streaming
// kernel (x kinds int8 / f16 / f32 / f32+norm / swiglu; binary16 weight scales).
cudaError_t launch(const GemvArgs& a, int M, cudaStream_t st) {
    const int Mpad = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    const int nchunks = (a.K + kKc - 1) / kKc;
    const int tiles = (a.N + kRows - 1) / kRows;
    const int sms = sm_count(current_device());
    int ksplit = g_tc_ksplit_override > 0 ? g_tc_ksplit_override : sms / tiles;  // whole waves of one CTA per SM
    if (ksplit > nchunks) ksplit = nchunks;
    if (ksplit < 1) ksplit = 1;
    const size_t xb_bytes = (size_t)nchunks * xb_chunk_bytes(Mpad);
    const size_t part_bytes = ksplit > 1 ? (size_t)tiles * ksplit * Mpad * kRows * sizeof(float) : 0;
    const size_t ticket_bytes = (size_t)tiles * sizeof(unsigned int);
    const size_t xb_off = (ticket_bytes + 255) & ~(size_t)255;
    const size_t part_off = (xb_off + xb_bytes + 255) & ~(size_t)255;
    unsigned char* scratch = nullptr;
    cudaError_t e = tc_scratch(part_off + part_bytes, &scratch);
    if (e != cudaSuccess) return e;

    CUtensorMap map_w;
    const cuuint64_t dims[2] = {(cuuint64_t)(a.K / 2), (cuuint64_t)a.N};
    const cuuint64_t strides[1] = {(cuuint64_t)(a.K / 2)};
    const cuuint32_t box[2] = {(cuuint32_t)(kKc / 2), (cuuint32_t)kRows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = encode_fn()(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(a.W), dims, strides,
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
    t.N = a.N; t.M = M; t.Mpad = Mpad; t.nchunks = nchunks; t.ksplit = ksplit;
    const int grid = tiles * ksplit;
    if (Mpad == 16) return launch_n<16>(map_w, t, grid, st);
    if (Mpad == 32) return launch_n<32>(map_w, t, grid, st);
    return launch_n<64>(map_w, t, grid, st);
}

}  // namespace tc
}  // namespace bw
