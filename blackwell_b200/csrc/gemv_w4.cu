// Host dispatch and C entry points of the INT4 block-16 GEMV family, plus the
// plain-load kernel used for ragged tails / unaligned operands / M > 8 and the
// per-block integer dot product inspection kernel.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <string.h>

#include <atomic>
#include <mutex>

#include "../../include/blackwell_b200.h"
#include "gemv_w4_mma.cuh"
#include "gemv_w4_stream.cuh"
#include "host_util.h"

namespace bw {

void set_attn_slots_pct(int v);
void set_attn_mma(int v);  // attention_decode.cu
cudaError_t attn_reserve_scratch(size_t bytes);
size_t attn_scratch_bytes(int M, int nqh, int nkv, int ctx);
namespace peer { void set_two_step_min_kb(int kb); void set_wait_limit_ms(int ms); }  // peer_allreduce.cu

namespace tc {  // tensor-core path, gemm_w4a8_tc.cu
bool eligible(const GemvArgs& a, int M);
cudaError_t launch(const GemvArgs& a, int M, cudaStream_t st);
cudaError_t reserve_scratch(size_t bytes);
size_t scratch_bytes(int M, int N, int K);
void set_ksplit_override(int v);
void set_ablate(int v);
cudaError_t prepare_plain(const GemvArgs& a, int M, cudaStream_t st, const int8_t** xq_out, const float** xs_out);
}  // namespace tc

// --------------------------------------------------------------------------
// Plain-load kernel: one warp per output row, lanes stride over k-blocks, up to
// 8 sequences per pass.  Any K % 16 == 0, any N, 8-byte aligned weights.  Same
// integer arithmetic as the streaming kernel (same helpers).
// --------------------------------------------------------------------------
template <int M, typename WS>
__global__ void __launch_bounds__(128) gemv_w4_rows_kernel(const GemvArgs a, int row0, int row_count) {
    const int lane = threadIdx.x & 31;
    const int row = row0 + blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= row0 + row_count) return;
    const int K = a.K, nkb = K / 16;

    float rstd[M];
#pragma unroll
    for (int m = 0; m < M; ++m) rstd[m] = 1.f;
    if (a.xkind == kXFloatNorm || a.xkind == kXFloatNormI4) {
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const float* xr = static_cast<const float*>(a.x) + (size_t)m * a.x_stride;
            float ss = 0.f;
            for (int i = lane; i < K; i += 32) ss = fmaf(xr[i], xr[i], ss);
            ss = warp_sum(ss);
            rstd[m] = rsqrtf(ss / (float)K + a.eps);
        }
    }

    float acc[M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = 0.f;
    const uint2* wrow = reinterpret_cast<const uint2*>(a.W + (size_t)row * (K / 2));
    const WS* srow = static_cast<const WS*>(a.Wsc) + (size_t)row * nkb;
    for (int kb = lane; kb < nkb; kb += 32) {
        const uint2 w = __ldg(wrow + kb);
        const float ws = (float)srow[kb];
        uint32_t lo0, hi0, lo1, hi1;
        nibbles_to_s8x16(w.x, lo0, hi0);
        nibbles_to_s8x16(w.y, lo1, hi1);
#pragma unroll
        for (int m = 0; m < M; ++m) {
            uint32_t e[2], o[2];
            float s;
            make_xblock(a, m, kb, rstd[m], e, o, s);
            int d = kMagicInt;
            d = dp4a_ss(lo0, e[0], d);
            d = dp4a_ss(hi0, o[0], d);
            d = dp4a_ss(lo1, e[1], d);
            d = dp4a_ss(hi1, o[1], d);
            acc[m] = fmaf(__int_as_float(d) - kMagicFloat, ws * s, acc[m]);
        }
    }
#pragma unroll
    for (int m = 0; m < M; ++m) {
        const float tot = warp_sum(acc[m]);
        if (lane == 0) {
            const size_t yi = (size_t)m * a.y_stride + row;
            a.y[yi] = a.residual ? tot + a.residual[yi] : tot;
        }
    }
}

// Per-block integer dots of one sequence: dots[n][kb].  x is int8 [K] or
// INT4-packed [K/2]; scales play no part.
__global__ void __launch_bounds__(128) block_dots_kernel(int32_t* dots, const uint8_t* W, const void* x, int a8,
                                                         int K, int N) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= N) return;
    const int nkb = K / 16;
    const uint2* wrow = reinterpret_cast<const uint2*>(W + (size_t)row * (K / 2));
    for (int kb = lane; kb < nkb; kb += 32) {
        const uint2 w = __ldg(wrow + kb);
        uint32_t lo0, hi0, lo1, hi1, e0, o0, e1, o1;
        nibbles_to_s8x16(w.x, lo0, hi0);
        nibbles_to_s8x16(w.y, lo1, hi1);
        if (a8) {
            const uint2* p = reinterpret_cast<const uint2*>(static_cast<const int8_t*>(x) + 16 * (size_t)kb);
            const uint2 q0 = __ldg(p), q1 = __ldg(p + 1);
            e0 = prmt(q0.x, q0.y, 0x6420); o0 = prmt(q0.x, q0.y, 0x7531);
            e1 = prmt(q1.x, q1.y, 0x6420); o1 = prmt(q1.x, q1.y, 0x7531);
        } else {
            const uint2 q = __ldg(reinterpret_cast<const uint2*>(static_cast<const uint8_t*>(x) + 8 * (size_t)kb));
            e0 = bytes_minus8(q.x & 0x0F0F0F0Fu); o0 = bytes_minus8((q.x >> 4) & 0x0F0F0F0Fu);
            e1 = bytes_minus8(q.y & 0x0F0F0F0Fu); o1 = bytes_minus8((q.y >> 4) & 0x0F0F0F0Fu);
        }
        int d = kMagicInt;
        d = dp4a_ss(lo0, e0, d);
        d = dp4a_ss(hi0, o0, d);
        d = dp4a_ss(lo1, e1, d);
        d = dp4a_ss(hi1, o1, d);
        // the accumulated value is 16 * dot on top of the float bit pattern
        dots[(size_t)row * nkb + kb] = (int)(__int_as_float(d) - kMagicFloat) / 16;
    }
}

// --------------------------------------------------------------------------
// Host side
// --------------------------------------------------------------------------
static std::atomic<int> g_tune_stages{0}, g_tune_ctas{0}, g_tune_force_plain{0}, g_tune_rg{0}, g_tune_threads{0}, g_tune_tc_min{0};
static std::atomic<int> g_tune_shrink_ring{1};
static std::atomic<int> g_tune_mma_mode{0};
static std::atomic<int> g_tune_mma_pack{1};
static std::atomic<int> g_tune_prep_min{0}, g_tune_prep_min_swiglu{0};
#ifdef BW_GEMV_TIMELINE
static unsigned long long* g_timeline_ptr = nullptr;
extern "C" void bw_debug_set_timeline(void* dev_ptr) { g_timeline_ptr = static_cast<unsigned long long*>(dev_ptr); }
void* debug_timeline_ptr() { return g_timeline_ptr; }
#endif
static std::atomic<int> g_tune_mma_slab{0}, g_tune_mma_min{0}, g_tune_mma_max{0}, g_tune_mma_stages{0};
static std::atomic<long long> g_launches{0};

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
static std::atomic<int> g_pdl{1};
bool pdl_enabled() { return g_pdl.load() != 0; }

// One status word per device for the whole library: kernels that give up on a bounded wait store a code here.
static __device__ int g_status_word = 0;
int* status_word_ptr() {
    static int* ptr[kMaxDevices] = {nullptr};
    static std::mutex mu;
    std::lock_guard<std::mutex> lk(mu);
    const int dev = current_device();
    if (!ptr[dev]) {
        int* p = nullptr;
        if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_status_word) != cudaSuccess) return nullptr;
        ptr[dev] = p;
    }
    return ptr[dev];
}

struct StreamPlan {
    bool ok = false;
    int Tg = 0, G = 0, J = 0, S = 0, T = 0, rg = 0, row_unit = 1, n_rows = 0, grid = 0, ctas_per_sm = 2;
    size_t smem = 0;
};

template <int M, typename WS, bool kMulti, bool kPending = false>
static cudaError_t launch_stream_inst(const GemvArgs& a, const StreamPlan& p, cudaStream_t st) {
    auto kern = gemv_w4_stream_kernel<M, WS, kMulti, kPending>;
    static std::once_flag once[kMaxDevices];
    const int dev = current_device();
    cudaError_t attr_err = cudaSuccess;
    std::call_once(once[dev], [&] {
        attr_err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynSmem);
    });
    if (attr_err != cudaSuccess) return attr_err;
    // resident CTAs per SM for this launch shape, remembered per device (a handful of shapes recur)
    struct OccEntry { int T; size_t smem; int occ; };
    static OccEntry cache[kMaxDevices][8];
    static int cache_n[kMaxDevices] = {0};
    static std::mutex cache_mu;
    int occ = 0;
    {
        std::lock_guard<std::mutex> lk(cache_mu);
        for (int i = 0; i < cache_n[dev]; ++i)
            if (cache[dev][i].T == p.T && cache[dev][i].smem == p.smem) occ = cache[dev][i].occ;
        if (occ == 0) {
            cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, p.T, p.smem);
            if (e != cudaSuccess) return e;
            if (occ < 1) return cudaErrorInvalidConfiguration;
            cache[dev][cache_n[dev] % 8] = OccEntry{p.T, p.smem, occ};
            if (cache_n[dev] < 8) ++cache_n[dev];
        }
    }
    // two resident CTAs per SM measured best (they hide each other's barrier and reduction phases); a smaller
    // footprint leaves the rest of the SM to the next kernel's early CTAs
    const int cap = p.ctas_per_sm;
    if (occ > cap) occ = cap;
    const int units = p.n_rows / p.row_unit;
    int grid = sm_count(dev) * occ;
    if (grid > units) grid = units;
    cudaError_t le = launch_pdl(kern, dim3(grid), dim3(p.T), p.smem, st, a);
    count_launch(1);
    return le != cudaSuccess ? le : cudaPeekAtLastError();
}

template <int M, typename WS>
static cudaError_t launch_stream_m(const GemvArgs& a, const StreamPlan& p, cudaStream_t st) {
    return p.J > 1 ? launch_stream_inst<M, WS, true>(a, p, st) : launch_stream_inst<M, WS, false>(a, p, st);
}

template <typename WS>
static cudaError_t launch_stream(const GemvArgs& a, const StreamPlan& p, int M, cudaStream_t st) {
    switch (M) {
        case 1: return launch_stream_m<1, WS>(a, p, st);
        case 2: return launch_stream_m<2, WS>(a, p, st);
        case 3: return launch_stream_m<3, WS>(a, p, st);
        case 4: return launch_stream_m<4, WS>(a, p, st);
        case 5: return launch_stream_m<5, WS>(a, p, st);
        case 6: return launch_stream_m<6, WS>(a, p, st);
        case 7: return launch_stream_m<7, WS>(a, p, st);
        case 8: return launch_stream_m<8, WS>(a, p, st);
        default: return cudaErrorInvalidValue;
    }
}

template <typename WS>
static cudaError_t launch_rows(const GemvArgs& a, int M, int row0, int row_count, cudaStream_t st) {
    if (row_count <= 0) return cudaSuccess;
    const int wpb = 4;
    const int grid = (row_count + wpb - 1) / wpb;
    switch (M) {
        case 1: gemv_w4_rows_kernel<1, WS><<<grid, 32 * wpb, 0, st>>>(a, row0, row_count); break;
        case 2: gemv_w4_rows_kernel<2, WS><<<grid, 32 * wpb, 0, st>>>(a, row0, row_count); break;
        case 3: gemv_w4_rows_kernel<3, WS><<<grid, 32 * wpb, 0, st>>>(a, row0, row_count); break;
        case 4: gemv_w4_rows_kernel<4, WS><<<grid, 32 * wpb, 0, st>>>(a, row0, row_count); break;
        case 5: gemv_w4_rows_kernel<5, WS><<<grid, 32 * wpb, 0, st>>>(a, row0, row_count); break;
        case 6: gemv_w4_rows_kernel<6, WS><<<grid, 32 * wpb, 0, st>>>(a, row0, row_count); break;
        case 7: gemv_w4_rows_kernel<7, WS><<<grid, 32 * wpb, 0, st>>>(a, row0, row_count); break;
        case 8: gemv_w4_rows_kernel<8, WS><<<grid, 32 * wpb, 0, st>>>(a, row0, row_count); break;
        default: return cudaErrorInvalidValue;
    }
    count_launch(1);
    return cudaPeekAtLastError();
}

static inline bool aligned(const void* p, size_t n) { return (reinterpret_cast<uintptr_t>(p) & (n - 1)) == 0; }

// Decides whether the streaming kernel can take the launch and with what shape.
static StreamPlan plan_stream(const GemvArgs& a, int M, int ws_bytes, int min_row_unit = 1) {
    StreamPlan p;
    const int K = a.K, N = a.N;
    if (g_tune_force_plain.load() || M < 1 || M > 8 || K % 32 != 0 || N < 1) return p;
    if (!aligned(a.W, 16) || !aligned(a.Wsc, 16) || !aligned(a.x, 16)) return p;
    if (a.xsc && !aligned(a.xsc, 8)) return p;
    if (a.x2 && !aligned(a.x2, 16)) return p;
    if (a.norm_w && !aligned(a.norm_w, 16)) return p;
    const int nch = K / 32;
    const int tmax = M <= 2 ? 512 : 256;
    p.J = (nch + tmax - 1) / tmax;
    p.Tg = (((nch + p.J - 1) / p.J) + 31) / 32 * 32;
    const int tt = g_tune_threads.load() > 0 ? g_tune_threads.load() : 256;
    int rg = M <= 2 ? 8 : (M <= 4 ? 4 : 2);
    p.G = tt / p.Tg;
    if (p.G < 1) p.G = 1;
    p.T = p.Tg * p.G;
    if (g_tune_rg.load() > 0 && g_tune_rg.load() < rg) rg = g_tune_rg.load();
    const size_t row_nib = (size_t)K / 2, row_sc = (size_t)(K / 16) * ws_bytes;
    const size_t fixed = GemvSmem::kXOff + align128(gemv_x_smem_bytes(M, nch, p.J));
    if (fixed >= (size_t)kMaxDynSmem) return p;
    auto stage_of = [&](int rows_per_group) {
        const size_t R = (size_t)rows_per_group * p.G;
        return align128(R * row_nib) + align128(R * row_sc);
    };
    // fewer rows per tile when three stages of the full tile do not fit
    while (rg > 1 && fixed + 3 * stage_of(rg) > (size_t)kMaxDynSmem) rg /= 2;
    const size_t stage = stage_of(rg);
    p.rg = rg;
    if (fixed + 2 * stage > (size_t)kMaxDynSmem) return p;
    int S = (int)(((size_t)kMaxDynSmem - fixed) / stage);
    int want = g_tune_stages.load();
    if (want <= 0) {
        // Two resident CTAs per SM hide each other's barrier and reduction phases, which measured faster
        // than one CTA with a deeper ring: take as many stages (up to 4) as half an SM's shared memory holds.
        const size_t half_sm = (size_t)(228 * 1024 / 2 - 1024 - 512);
        want = fixed + 2 * stage <= half_sm ? (int)((half_sm - fixed) / stage) : 4;
        if (want > 4) want = 4;
    }
    if (S > want) S = want;
    if (S > 8) S = 8;
    if (S < 2) return p;
    // A CTA never needs more stages than it has tiles: on the small per-layer matrices (a tile or two per CTA) the
    // spare stages would only keep the next kernel's CTAs from becoming resident early, and with them the weight
    // prefetch they do ahead of their grid-dependency wait.
    // Matrices with between two and three row tiles per SM (the 6144-row QKV projection: 384 tiles of 16 rows on 148
    // SMs) run one tile per CTA on three CTAs per SM instead of one or two tiles on two (measured 5.2 against 5.7 us);
    // everywhere else two CTAs per SM measured best.
    p.ctas_per_sm = 2;
    {
        const long long sms = sm_count(current_device());
        const long long all_tiles = ((long long)N + (long long)rg * p.G - 1) / ((long long)rg * p.G);
        if (M == 1 && all_tiles > 2 * sms && all_tiles <= 3 * sms) p.ctas_per_sm = 3;
    }
    if (g_tune_ctas.load() > 0) p.ctas_per_sm = g_tune_ctas.load();
    if (g_tune_shrink_ring.load() != 0) {
        const int ctas_per_sm = p.ctas_per_sm;
        const long long grid = (long long)sm_count(current_device()) * ctas_per_sm;
        const long long rows_per_cta = ((long long)N + grid - 1) / grid;
        const int tiles = (int)((rows_per_cta + (long long)rg * p.G - 1) / ((long long)rg * p.G));
        if (S > tiles) S = tiles < 1 ? 1 : tiles;
    }
    p.S = S;
    p.smem = fixed + (size_t)S * stage;
    int tile_unit = 1;
    while ((tile_unit * row_sc) % 16 != 0) tile_unit *= 2;
    // Every tile must start on a row whose scale bytes are 16-byte aligned in global memory (the bulk copy's rule):
    // with one row per tile and a scale row of 8 mod 16 bytes, odd tiles would not.  Such shapes take the plain kernel.
    if ((rg * p.G) % tile_unit != 0) return p;
    p.row_unit = tile_unit > min_row_unit ? tile_unit : min_row_unit;   // powers of two: the larger is the common multiple
    p.n_rows = N - N % p.row_unit;
    p.ok = p.n_rows > 0;
    return p;
}

// ---- tensor-core streaming kernel (mma.sync), 3..16 sequences per launch ----
// Decides whether it can take the launch and lays out its shared memory: [barriers, flags | prepared activations
// (a window of K) | ring of S stages | two reduction buffers].
static bool plan_mma_slab(const GemvArgs& a, int M, int ws_bytes, int slab, mma::MmaPlan& p, bool* whole_k) {
    const int K = a.K;
    const int MG = M <= 8 ? 1 : 2;
    const int nch = K / 32;
    if (slab > nch) slab = nch;
    p.slab_cols = slab;
    p.pitch_n = (slab * 16 + 127) / 128 * 128 + 16;
    p.ablate = g_tune_mma_mode.load();
    p.pitch_s = (slab * 2 * ws_bytes + 127) / 128 * 128 + 16;
    // Scales travel as cp.async of the largest size the rows' alignment in HBM allows (K % 32 == 0 makes a binary16
    // scale row a multiple of 4 bytes and an fp32 one a multiple of 8).
    const size_t scale_row = (size_t)(K / 16) * ws_bytes;
    p.scale_gran = 4;
    for (int gran = 16; gran >= 4; gran /= 2)
        if (scale_row % gran == 0 && ((size_t)slab * 2 * ws_bytes) % gran == 0 && aligned(a.Wsc, gran)) { p.scale_gran = gran; break; }
    if (scale_row % 4 != 0 || !aligned(a.Wsc, 4)) return false;
    {
        const int per_row = slab * 2 * ws_bytes / p.scale_gran;
        int lpr = 1;
        while (lpr < per_row && lpr < 32) lpr *= 2;
        p.lanes_per_row = lpr;
    }
    const size_t stage = (size_t)mma::kRows * (p.pitch_n + p.pitch_s);
    const size_t red = (size_t)mma::kConsumerWarps * mma::kRows * mma::red_stride(MG) * sizeof(float);
    const size_t fixed = mma::Smem::kX;
    const size_t xcol = (size_t)MG * mma::kXColBytes;
    const size_t total = (size_t)kMaxDynSmem;
    const int nslab = (nch + slab - 1) / slab;
    // Prefer the whole K prepared at once with the deepest ring that fits (at most 4 stages); otherwise two stages
    // and as wide a window as fits.
    int S = g_tune_mma_stages.load() > 0 ? g_tune_mma_stages.load() : 4;
    if (S > 8) S = 8;
    for (; S >= 2; --S)
        if (fixed + align128(xcol * nch) + S * stage + red <= total) break;
    *whole_k = S >= 2;
    if (S >= 2) {
        p.win_cols = nch;
    } else {
        S = 2;
        if (fixed + S * stage + red + align128(xcol * slab) > total) return false;
        const size_t avail = total - fixed - S * stage - red - 128;
        int wc = (int)(avail / xcol) / slab * slab;
        if (wc < slab) return false;
        // equal windows rather than a full one and a sliver
        const int nwin = (nslab * slab + wc - 1) / wc;
        wc = ((nslab + nwin - 1) / nwin) * slab;
        p.win_cols = wc;
    }
    p.S = S;
    p.x_off = fixed;
    p.stage_off = fixed + align128(xcol * (size_t)(p.win_cols < nch ? p.win_cols : nch));
    p.red_off = p.stage_off + (size_t)S * stage;
    p.smem = p.red_off + red;
    return p.smem <= total;
}

// Decides whether the kernel can take the launch and lays out its shared memory: [barriers, flags | prepared
// activations (all of K, or a window) | ring of S stages | reduction buffer].  Slabs of 128 columns (2 KB of nibbles
// per row and copy: the copy engine's request rate favours large copies) where two stages of them fit beside the
// activations of the whole K, else slabs of 64.
static bool plan_mma(const GemvArgs& a, int M, int ws_bytes, mma::MmaPlan& p) {
    const int K = a.K;
    if (g_tune_force_plain.load() || M < 1 || M > 16 || K % 32 != 0 || a.N < 1) return false;
    if (!aligned(a.W, 16) || !aligned(a.Wsc, 4) || !aligned(a.x, 16)) return false;
    if (a.xsc && !aligned(a.xsc, 8)) return false;
    if (a.x2 && !aligned(a.x2, 16)) return false;
    if (a.norm_w && !aligned(a.norm_w, 16)) return false;
    if ((a.xkind == kXHalf) && a.x_stride % 8 != 0) return false;
    bool whole = false;
    if (g_tune_mma_slab.load() > 0) return plan_mma_slab(a, M, ws_bytes, g_tune_mma_slab.load(), p, &whole);
    if (plan_mma_slab(a, M, ws_bytes, 128, p, &whole) && whole) return true;
    return plan_mma_slab(a, M, ws_bytes, 64, p, &whole);
}

template <int MG, typename WS, bool kPack, bool kPending = false>
static cudaError_t launch_mma_inst(const GemvArgs& a, const mma::MmaPlan& p, int M, cudaStream_t st) {
    auto kern = mma::gemv_w4_mma_kernel<MG, WS, kPack, kPending>;
    static std::once_flag once[kMaxDevices];
    const int dev = current_device();
    cudaError_t attr_err = cudaSuccess;
    std::call_once(once[dev], [&] {
        attr_err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynSmem);
    });
    if (attr_err != cudaSuccess) return attr_err;
    int grid = sm_count(dev);  // one persistent CTA per SM; at least 8 rows each
    const int by_rows = (a.N + 7) / 8;
    if (grid > by_rows) grid = by_rows;
    cudaError_t le = launch_pdl(kern, dim3(grid), dim3(mma::kThreads), p.smem, st, a, p, M);
    count_launch(1);
    return le != cudaSuccess ? le : cudaPeekAtLastError();
}

template <typename WS>
static cudaError_t launch_mma(const GemvArgs& a, const mma::MmaPlan& p, int M, cudaStream_t st) {
    if (M <= 4 && g_tune_mma_pack.load() != 0) return launch_mma_inst<1, WS, true>(a, p, M, st);
    return M <= 8 ? launch_mma_inst<1, WS, false>(a, p, M, st) : launch_mma_inst<2, WS, false>(a, p, M, st);
}

template <typename WS>
static cudaError_t gemv_dispatch(GemvArgs a, int M, cudaStream_t st) {
    if (a.K <= 0 || a.K % 16 != 0 || a.N < 1 || M < 1) return cudaErrorInvalidValue;
    if (!a.y || !a.W || !a.Wsc || !a.x) return cudaErrorInvalidValue;
    if (!aligned(a.W, 8) || !aligned(a.x, 8)) return cudaErrorInvalidValue;
    a.status = status_word_ptr();
    if (!a.status) return cudaErrorInitializationError;
#ifdef BW_GEMV_TIMELINE
    a.timeline = g_timeline_ptr;
#endif
    const bool prequant = (a.xkind == kXInt8 || a.xkind == kXInt4);
    a.nch = a.K / 32;
    if (a.x_stride <= 0) a.x_stride = a.K;
    if (a.y_stride <= 0) a.y_stride = a.N;
    if (a.x_stride % 4 != 0 || a.y_stride < a.N) return cudaErrorInvalidValue;
    if (!prequant && !aligned(a.x, 16)) return cudaErrorInvalidValue;
    // 5..16 sequences: the streaming kernel with warp-level tensor-core dots, either scale type (routing by
    // measurement: up to 4 sequences the dp4a kernel is as fast or faster; from 9 sequences on, shapes whose prepared
    // activations need several windows of K are faster on the tcgen05 kernel).
    const int mma_min = g_tune_mma_min.load() > 0 ? g_tune_mma_min.load() : 5;
    const int mma_max = g_tune_mma_max.load() > 0 ? g_tune_mma_max.load() : 16;
    const int tc_min = g_tune_tc_min.load() > 0 ? g_tune_tc_min.load() : 8;
    mma::MmaPlan mp;
    bool use_mma = false;
    if (M >= mma_min && M <= mma_max && M <= 16 && plan_mma(a, M, (int)sizeof(WS), mp)) {
        const bool windows = mp.win_cols < a.K / 32;
        const bool tc_can = sizeof(WS) == 2 && M > 8 && tc::eligible(a, M);
        const bool forced = g_tune_mma_min.load() > 0;  // an explicit range (tests, experiments) takes the kernel as it is
        use_mma = forced || !(windows && tc_can);
    }
    const bool use_tc = !use_mma && sizeof(WS) == 2 && M >= tc_min && tc::eligible(a, M < 64 ? M : 64);
    // From 2 sequences on, a call of a streaming kernel with an int8 prologue (f16 / f32 / RMSNorm / SwiGLU input) has
    // its activations quantized once by a small kernel instead of once per CTA; the GEMV then runs on the result as on
    // any pre-quantized operand (same quantize code, same bits).
    const int prep_min = g_tune_prep_min.load() > 0 ? g_tune_prep_min.load() : 2;   // measured: a loss at 1
    const int prep_min_sw = g_tune_prep_min_swiglu.load() > 0 ? g_tune_prep_min_swiglu.load() : 1;   // SwiGLU: a gain at 1 too
    if (!use_tc && M >= (a.xkind == kXSwiglu ? prep_min_sw : prep_min) && a.K % 32 == 0 &&
        (a.xkind == kXHalf || a.xkind == kXFloat || a.xkind == kXFloatNorm || a.xkind == kXSwiglu)) {
        const int8_t* xq = nullptr;
        const float* xs = nullptr;
        cudaError_t e = tc::prepare_plain(a, M, st, &xq, &xs);
        if (e != cudaSuccess) return e;
        a.x = xq; a.xsc = xs; a.x2 = nullptr; a.norm_w = nullptr; a.xkind = kXInt8; a.x_stride = a.K;
        if (use_mma && !plan_mma(a, M, (int)sizeof(WS), mp)) use_mma = false;   // the plan depends on the operand kind
    }
    // Norm-pending hand-over (see GemvArgs): one sequence on the dp4a streaming kernel (every row streamed, tiles that
    // are whole or half k-blocks of the consumer), 5..16 sequences on the mma.sync kernel (a producer needs all of K in
    // one window).  Anything else is refused: the caller chose this form for a shape it knows.
    if (a.next_q || a.x_sumsq) {
        if (sizeof(WS) != 2 || a.xkind != kXInt8 || a.K % 32 != 0) return cudaErrorInvalidValue;   // (a SwiGLU input
        // has been quantized by the prep kernel above)
        if (a.next_q && (!a.next_sc || !a.next_sumsq || !a.next_norm_w || a.N % 16 != 0)) return cudaErrorInvalidValue;
        if (M == 1) {
            const StreamPlan p = plan_stream(a, 1, (int)sizeof(WS), a.next_q ? 16 : 1);
            const int R = p.rg * p.G;
            if (!p.ok || p.n_rows != a.N || (a.next_q && !(R == 8 || R == 16 || R % 32 == 0))) return cudaErrorInvalidValue;
            a.Tg = p.Tg; a.G = p.G; a.J = p.J; a.S = p.S; a.rg = p.rg;
            a.row_unit = p.row_unit; a.n_rows = p.n_rows;
            return p.J > 1 ? launch_stream_inst<1, WS, true, true>(a, p, st) : launch_stream_inst<1, WS, false, true>(a, p, st);
        }
        if (M < 5 || M > 16) return cudaErrorInvalidValue;
        mma::MmaPlan pp;
        if (!plan_mma(a, M, (int)sizeof(WS), pp)) return cudaErrorInvalidValue;
        if (a.next_q && pp.win_cols < a.K / 32) return cudaErrorInvalidValue;
        return M <= 8 ? launch_mma_inst<1, WS, false, true>(a, pp, M, st) : launch_mma_inst<2, WS, false, true>(a, pp, M, st);
    }
    if (use_mma) return launch_mma<WS>(a, mp, M, st);
    // Larger batches go to the tcgen05 kernel, up to 64 sequences per launch.
    if (use_tc) {
        for (int m0 = 0; m0 < M; m0 += 64) {
            const int mc = (M - m0) < 64 ? (M - m0) : 64;
            GemvArgs b = a;
            b.y = a.y + (size_t)m0 * a.y_stride;
            if (a.residual) b.residual = a.residual + (size_t)m0 * a.y_stride;
            if (a.xkind == kXInt8) {
                b.x = static_cast<const int8_t*>(a.x) + (size_t)m0 * a.K;
                b.xsc = a.xsc + (size_t)m0 * (a.K / 16);
            } else if (a.xkind == kXHalf) {
                b.x = static_cast<const __half*>(a.x) + (size_t)m0 * a.x_stride;
            } else {
                b.x = static_cast<const float*>(a.x) + (size_t)m0 * a.x_stride;
                if (a.x2) b.x2 = static_cast<const float*>(a.x2) + (size_t)m0 * a.x_stride;
            }
            cudaError_t e = tc::launch(b, mc, st);
            if (e != cudaSuccess) return e;
        }
        return cudaSuccess;
    }
    // M > 8: passes of up to 16 (tensor-core streaming kernel) or 8 sequences.
    int pass = 8;
    if (M > 8 && mma_max >= 16) {
        mma::MmaPlan mp;
        if (plan_mma(a, 16, (int)sizeof(WS), mp)) pass = 16;
    }
    for (int m0 = 0; m0 < M; m0 += pass) {
        const int mc = (M - m0) < pass ? (M - m0) : pass;
        GemvArgs b = a;
        b.y = a.y + (size_t)m0 * a.y_stride;
        if (a.residual) b.residual = a.residual + (size_t)m0 * a.y_stride;
        if (a.xkind == kXInt8) b.x = static_cast<const int8_t*>(a.x) + (size_t)m0 * a.K;
        else if (a.xkind == kXInt4) b.x = static_cast<const uint8_t*>(a.x) + (size_t)m0 * (a.K / 2);
        else if (a.xkind == kXHalf) b.x = static_cast<const __half*>(a.x) + (size_t)m0 * a.x_stride;
        else {
            b.x = static_cast<const float*>(a.x) + (size_t)m0 * a.x_stride;
            if (a.x2) b.x2 = static_cast<const float*>(a.x2) + (size_t)m0 * a.x_stride;
        }
        if (a.xsc) b.xsc = a.xsc + (size_t)m0 * (a.K / 16);
        if (mc >= mma_min && mc <= mma_max) {
            mma::MmaPlan mp;
            if (plan_mma(b, mc, (int)sizeof(WS), mp)) {
                cudaError_t e = launch_mma<WS>(b, mp, mc, st);
                if (e != cudaSuccess) return e;
                continue;
            }
        }
        const StreamPlan p = plan_stream(b, mc, (int)sizeof(WS));
        int done = 0;
        if (p.ok) {
            b.Tg = p.Tg; b.G = p.G; b.J = p.J; b.S = p.S; b.rg = p.rg;
            b.row_unit = p.row_unit; b.n_rows = p.n_rows;
            cudaError_t e = launch_stream<WS>(b, p, mc, st);
            if (e != cudaSuccess) return e;
            done = p.n_rows;
        }
        cudaError_t e = launch_rows<WS>(b, mc, done, a.N - done, st);
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

}  // namespace bw

// ----------------------------------------------------------------------------
// C entry points
// ----------------------------------------------------------------------------
using namespace bw;

extern "C" int bw_gemv_int4_batched(float* y_out, const uint8_t* x_packed, const float* x_scale,
                                    const uint8_t* W_packed, const float* W_scale, int K, int N, int M,
                                    void* stream) {
    GemvArgs a{};
    a.y = y_out; a.W = W_packed; a.Wsc = W_scale; a.x = x_packed; a.xsc = x_scale;
    a.xkind = kXInt4; a.K = K; a.N = N;
    if (!x_scale) return cudaErrorInvalidValue;
    return gemv_dispatch<float>(a, M, static_cast<cudaStream_t>(stream));
}

extern "C" int bw_gemv_int4_warp(float* y_out, const void* x_packed, const float* x_scale, const void* W_packed,
                                 const float* W_scale, int K, int N, void* stream) {
    return bw_gemv_int4_batched(y_out, static_cast<const uint8_t*>(x_packed), x_scale,
                                static_cast<const uint8_t*>(W_packed), W_scale, K, N, 1, stream);
}

extern "C" int bw_gemv_w4a8(float* y_out, const int8_t* x_q, const float* x_scale, const uint8_t* W_packed,
                            const uint16_t* W_scale_f16, int K, int N, int M, void* stream) {
    GemvArgs a{};
    a.y = y_out; a.W = W_packed; a.Wsc = W_scale_f16; a.x = x_q; a.xsc = x_scale;
    a.xkind = kXInt8; a.K = K; a.N = N;
    if (!x_scale) return cudaErrorInvalidValue;
    return gemv_dispatch<__half>(a, M, static_cast<cudaStream_t>(stream));
}

extern "C" int bw_gemv_w4a8_f16in(float* y_out, const uint16_t* x_f16, const uint8_t* W_packed,
                                  const uint16_t* W_scale_f16, int K, int N, int M, void* stream) {
    GemvArgs a{};
    a.y = y_out; a.W = W_packed; a.Wsc = W_scale_f16; a.x = x_f16;
    a.xkind = kXHalf; a.K = K; a.N = N;
    return gemv_dispatch<__half>(a, M, static_cast<cudaStream_t>(stream));
}

extern "C" int bw_gemv_w4a8_f32in(float* y_out, const float* x_f32, const float* norm_weight, float eps,
                                  const uint8_t* W_packed, const uint16_t* W_scale_f16, int K, int N, int M,
                                  void* stream) {
    GemvArgs a{};
    a.y = y_out; a.W = W_packed; a.Wsc = W_scale_f16; a.x = x_f32; a.norm_w = norm_weight; a.eps = eps;
    a.xkind = norm_weight ? kXFloatNorm : kXFloat; a.K = K; a.N = N;
    return gemv_dispatch<__half>(a, M, static_cast<cudaStream_t>(stream));
}

extern "C" int bw_gemv_w4a8_swiglu(float* y_out, const float* gate, const float* up, const uint8_t* W_packed,
                                   const uint16_t* W_scale_f16, int K, int N, int M, void* stream) {
    if (!up) return cudaErrorInvalidValue;
    GemvArgs a{};
    a.y = y_out; a.W = W_packed; a.Wsc = W_scale_f16; a.x = gate; a.x2 = up;
    a.xkind = kXSwiglu; a.K = K; a.N = N;
    return gemv_dispatch<__half>(a, M, static_cast<cudaStream_t>(stream));
}

extern "C" int bw_gemv_w4a8_decode(float* y_out, long y_stride, const float* residual_or_null, const float* x_f32,
                                   const float* up_or_null, long x_stride, const float* norm_weight_or_null,
                                   float eps, const uint8_t* W_packed, const uint16_t* W_scale_f16, int K, int N,
                                   int M, void* stream) {
    if (up_or_null && norm_weight_or_null) return cudaErrorInvalidValue;
    GemvArgs a{};
    a.y = y_out; a.y_stride = y_stride; a.residual = residual_or_null;
    a.W = W_packed; a.Wsc = W_scale_f16; a.x = x_f32; a.x2 = up_or_null; a.x_stride = x_stride;
    a.norm_w = norm_weight_or_null; a.eps = eps;
    a.xkind = up_or_null ? kXSwiglu : (norm_weight_or_null ? kXFloatNorm : kXFloat);
    a.K = K; a.N = N;
    return gemv_dispatch<__half>(a, M, static_cast<cudaStream_t>(stream));
}

extern "C" int bw_gemv_w4a8_q8_decode(float* y_out, long y_stride, const float* residual_or_null, const int8_t* x_q,
                                      const float* x_scale, const uint8_t* W_packed, const uint16_t* W_scale_f16, int K,
                                      int N, int M, void* stream) {
    if (!x_scale) return cudaErrorInvalidValue;
    GemvArgs a{};
    a.y = y_out; a.y_stride = y_stride; a.residual = residual_or_null;
    a.W = W_packed; a.Wsc = W_scale_f16; a.x = x_q; a.xsc = x_scale;
    a.xkind = kXInt8; a.K = K; a.N = N;
    return gemv_dispatch<__half>(a, M, static_cast<cudaStream_t>(stream));
}

extern "C" int bw_gemv_w4a8_pending(const bw_gemv_pending_args* g, void* stream) {
    if (!g || (!g->x_q && !g->gate)) return cudaErrorInvalidValue;
    if (g->x_q && (!g->x_scale || g->gate || g->up)) return cudaErrorInvalidValue;
    if (g->gate && (!g->up || g->x_block_sumsq)) return cudaErrorInvalidValue;
    if (!g->next_norm_w && !g->x_block_sumsq) return cudaErrorInvalidValue;   // nothing pending: use the plain entries
    const int M = g->M > 0 ? g->M : 1;
    GemvArgs a{};
    a.y = g->y; a.residual = g->residual;
    a.W = g->W_packed; a.Wsc = g->W_scale_f16; a.K = g->K; a.N = g->N; a.eps = g->eps;
    if (g->x_q) {
        a.x = g->x_q; a.xsc = g->x_scale; a.x_sumsq = g->x_block_sumsq; a.xkind = kXInt8;
    } else {
        a.x = g->gate; a.x2 = g->up; a.x_stride = g->x_stride > 0 ? g->x_stride : g->K; a.xkind = kXSwiglu;
    }
    if (g->next_norm_w) {
        a.next_norm_w = g->next_norm_w; a.next_q = g->next_q; a.next_sc = g->next_scale; a.next_sumsq = g->next_block_sumsq;
        if (!a.next_q || !a.next_sc || !a.next_sumsq) return cudaErrorInvalidValue;
    }
    return gemv_dispatch<__half>(a, M, static_cast<cudaStream_t>(stream));
}

extern "C" int bw_gemv_int4_fused(float* y_out, const float* x_f32, const float* up_or_null,
                                  const float* norm_weight_or_null, float eps, const uint8_t* W_packed,
                                  const float* W_scale, int K, int N, int M, void* stream) {
    if (up_or_null && norm_weight_or_null) return cudaErrorInvalidValue;
    GemvArgs a{};
    a.y = y_out; a.W = W_packed; a.Wsc = W_scale; a.x = x_f32; a.x2 = up_or_null; a.norm_w = norm_weight_or_null;
    a.eps = eps;
    a.xkind = up_or_null ? kXSwigluI4 : (norm_weight_or_null ? kXFloatNormI4 : kXFloatI4);
    a.K = K; a.N = N;
    return gemv_dispatch<float>(a, M, static_cast<cudaStream_t>(stream));
}

extern "C" int bw_gemv_int4_decode(float* y_out, long y_stride, const float* residual_or_null, const float* x_f32,
                                   const float* up_or_null, long x_stride, const float* norm_weight_or_null,
                                   float eps, const uint8_t* W_packed, const float* W_scale, int K, int N, int M,
                                   void* stream) {
    if (up_or_null && norm_weight_or_null) return cudaErrorInvalidValue;
    GemvArgs a{};
    a.y = y_out; a.y_stride = y_stride; a.residual = residual_or_null;
    a.W = W_packed; a.Wsc = W_scale; a.x = x_f32; a.x2 = up_or_null; a.x_stride = x_stride;
    a.norm_w = norm_weight_or_null; a.eps = eps;
    a.xkind = up_or_null ? kXSwigluI4 : (norm_weight_or_null ? kXFloatNormI4 : kXFloatI4);
    a.K = K; a.N = N;
    return gemv_dispatch<float>(a, M, static_cast<cudaStream_t>(stream));
}

extern "C" int bw_gemv_block_dots(int32_t* dots, const void* x, int a8, const uint8_t* W_packed, int K, int N,
                                  void* stream) {
    if (!dots || !x || !W_packed || K <= 0 || K % 16 != 0 || N < 1) return cudaErrorInvalidValue;
    if (!aligned(W_packed, 8) || !aligned(x, 8)) return cudaErrorInvalidValue;
    block_dots_kernel<<<(N + 3) / 4, 128, 0, static_cast<cudaStream_t>(stream)>>>(dots, W_packed, x, a8, K, N);
    count_launch(1);
    return cudaPeekAtLastError();
}

extern "C" int bw_device_status(int* status_out) {
    int* p = status_word_ptr();
    if (!p) return cudaErrorInitializationError;
    int v = 0;
    cudaError_t e = cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return e;
    if (v != 0) {
        const int zero = 0;
        e = cudaMemcpy(p, &zero, sizeof(int), cudaMemcpyHostToDevice);
    }
    if (status_out) *status_out = v;
    return e;
}

extern "C" size_t bw_gemv_scratch_bytes(int M, int N, int K) { return tc::scratch_bytes(M, N, K); }
extern "C" size_t bw_attention_scratch_bytes(int M, int num_q_heads, int num_kv_heads, int max_context) {
    return attn_scratch_bytes(M, num_q_heads, num_kv_heads, max_context);
}

extern "C" int bw_reserve_scratch(size_t gemv_bytes, size_t attention_bytes) {
    cudaError_t e = tc::reserve_scratch(gemv_bytes);
    if (e != cudaSuccess) return e;
    return attn_reserve_scratch(attention_bytes);
}

extern "C" int bw_set_tuning(int key, int value) {
    switch (key) {
        case 0: g_tune_stages = value; return 0;
        case 1: g_tune_ctas = value; return 0;
        case 2: g_tune_force_plain = value; return 0;
        case 3: g_tune_rg = value; return 0;
        case 4: g_tune_threads = value; return 0;
        case 5: g_tune_tc_min = value; return 0;
        case 6: tc::set_ksplit_override(value); return 0;
        case 8: g_pdl = value; return 0;
        case 9: set_attn_mma(value); return 0;
        case 10: peer::set_two_step_min_kb(value); return 0;
        case 11: peer::set_wait_limit_ms(value); return 0;
        case 12: g_tune_mma_slab = value; return 0;
        case 13: g_tune_mma_min = value; return 0;
        case 14: g_tune_mma_max = value; return 0;
        case 15: g_tune_mma_stages = value; return 0;
        case 16: g_tune_shrink_ring = value; return 0;
        case 17: g_tune_mma_mode = value; return 0;
        case 18: g_tune_mma_pack = value; return 0;
        case 19: tc::set_ablate(value); return 0;
        case 20: g_tune_prep_min = value; return 0;
        case 21: g_tune_prep_min_swiglu = value; return 0;
        case 22: set_attn_slots_pct(value); return 0;
        default: return cudaErrorInvalidValue;
    }
}

extern "C" long long bw_launch_count(int reset) {
    return reset ? g_launches.exchange(0) : g_launches.load();
}

extern "C" int bw_version(void) { return 100; }
