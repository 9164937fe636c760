// Shared device helpers for the sm_100a decode-path kernels: PTX wrappers for
// mbarrier / bulk-async copies, byte-wise integer tricks, warp reductions, and
// the device status word that bounded waits report through.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace bw {

// ---------------------------------------------------------------- status word
// Non-zero after a kernel gave up on a bounded wait.  Read back through
// bw_device_status().
enum : int { kStatusOk = 0, kStatusMbarTimeout = 1, kStatusTmemAlloc = 2 };

// ------------------------------------------------------------------ mbarrier
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// The same probe with a suspend-time hint: the hardware may keep the thread parked for up to `ns` nanoseconds while the
// phase is incomplete (it wakes when the phase completes), so a waiting warp issues few instructions.
__device__ __forceinline__ bool mbar_try_wait_parked(uint32_t bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(ns)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Waits for the phase with the given parity.  Bounded: gives up after about one
// second of wall time and returns false; the caller then flags the status word
// and leaves the kernel in an orderly way.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    // The limit is counted on the SM's own cycle counter (cheap to read); the global nanosecond timer costs
    // on the order of a microsecond per read, which would quantise every wake-up.
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
#pragma unroll 1
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 32; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (clock64() - t0 > 2500000000ll) return false;  // more than a second at any SM clock
    }
}

// The same bounded wait for roles that wait long and share their scheduler with working warps: parked probes.
__device__ __forceinline__ bool mbar_wait_parked(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
#pragma unroll 1
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 32; ++i)
            if (mbar_try_wait_parked(bar, parity, 4000u)) return true;
        if (clock64() - t0 > 2500000000ll) return false;
    }
}

// ------------------------------------------- programmatic dependent launch
// A kernel launched with the programmatic-serialization attribute may start while its predecessor in the stream
// is still running.  pdl_wait() blocks until the predecessor has completed and its writes are visible: everything
// that reads the predecessor's output, or writes what it may still read, comes after it.  pdl_trigger() lets the
// successor begin its own preamble.  Both are no-ops for a kernel launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// -------------------------------------------------------- bulk async copies
// 1-D bulk copy global -> shared of this CTA, completion counted in bytes on an
// mbarrier.  Both addresses 16-byte aligned, size a multiple of 16.  No cluster
// multicast is used anywhere in this library.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar,
                                         uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy)
        : "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ----------------------------------------------------------- integer helpers
// Signed 8-bit x 8-bit 4-way dot product with 32-bit accumulate.
__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
// (a & b) ^ c in one LOP3.
__device__ __forceinline__ uint32_t and_xor(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0x6a;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// A 32-bit word holds 8 offset-binary nibbles n_j = q_j + 8 (k order: low
// nibble of byte 0 first).  Returns, as signed bytes, 16*q for the four even-k
// nibbles (lo16) and for the four odd-k nibbles (hi16): moving a nibble to the
// top of its byte and flipping the sign bit turns offset binary into two's
// complement scaled by 16.
__device__ __forceinline__ void nibbles_to_s8x16(uint32_t w, uint32_t& lo16, uint32_t& hi16) {
    hi16 = and_xor(w, 0xF0F0F0F0u, 0x80808080u);
    lo16 = and_xor(w << 4, 0xF0F0F0F0u, 0x80808080u);
}
// Per-byte (v - 8) for bytes v in [0, 15], no borrow between bytes.
__device__ __forceinline__ uint32_t bytes_minus8(uint32_t v) {
    return ((v | 0x80808080u) - 0x08080808u) ^ 0x80808080u;
}

// dp4a accumulators start from the bit pattern of 1.5 * 2^23; after integer
// additions of magnitude < 2^22 the pattern read as a float is 12582912 + sum
// exactly, so one FADD replaces an int->float conversion.
constexpr int kMagicInt = 0x4B400000;
constexpr float kMagicFloat = 12582912.0f;

// ------------------------------------------------------------ warp reductions
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sums V per-lane values across the 32 lanes of a warp.  On return lane l holds
// the total of value number (l % V') in `out`, V' = V rounded up to a power of
// two (at most 32).  Uses V'-1 + (5 - log2 V') shuffles instead of 5*V.
template <int V>
__device__ __forceinline__ float warp_sum_many(const float (&v)[V], int lane) {
    constexpr int P = V <= 1 ? 1 : V <= 2 ? 2 : V <= 4 ? 4 : V <= 8 ? 8 : V <= 16 ? 16 : 32;
    static_assert(V <= 32, "at most 32 values");
    float a[P];
#pragma unroll
    for (int i = 0; i < P; ++i) a[i] = i < V ? v[i] : 0.f;
    // Halving steps: at width w, the lane keeps the half of the live values
    // selected by one bit of its lane id and hands the other half to its partner.
    int off = 16;
#pragma unroll
    for (int w = P; w > 1; w >>= 1) {
        const bool upper = (lane & off) != 0;
#pragma unroll
        for (int i = 0; i < w / 2; ++i) {
            const float keep = upper ? a[i + w / 2] : a[i];
            const float send = upper ? a[i] : a[i + w / 2];
            a[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
        }
        off >>= 1;
    }
#pragma unroll
    for (; off > 0; off >>= 1) a[0] += __shfl_xor_sync(0xffffffffu, a[0], off);
    return a[0];
}
// Which value index lane `lane` holds after warp_sum_many<V>.
template <int V>
__device__ __forceinline__ int warp_sum_many_index(int lane) {
    constexpr int P = V <= 1 ? 1 : V <= 2 ? 2 : V <= 4 ? 4 : V <= 8 ? 8 : V <= 16 ? 16 : 32;
    int idx = 0, off = 16;
#pragma unroll
    for (int w = P; w > 1; w >>= 1) {
        if (lane & off) idx += w / 2;
        off >>= 1;
    }
    return idx;
}

}  // namespace bw
