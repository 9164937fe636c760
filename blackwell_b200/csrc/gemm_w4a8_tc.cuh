// INT4-weight x INT8-activation block-16 GEMM for batches of 9..64 sequences on the 5th-generation tensor cores
// (tcgen05.mma kind::i8, accumulators in tensor memory).  Device side.
//
//   y[m][n] = sum_kb dot16(W[n,kb], xq[m,kb]) * w_sc[n,kb] * x_sc[m,kb]
//
// The scale changes every 16 k, the MMA consumes 32 k: each k-block gets its own MMA (fresh accumulator, no
// accumulation) whose first 16-byte K core matrix is the block and whose second is a constant shared by all blocks
// (the descriptor's leading-dimension offset points there): -128 in every weight row, -127 in every sequence.  The
// accumulator is then the int32  260096 + 16 * dot  -- never negative, because |16 * dot| <= 16 * 16 * 8 * 127 =
// 260096 -- and below 2^23, so its bit pattern read as a float is the denormal (260096 + 16 * dot) * 2^-149 exactly:
// no int-to-float conversion, no accumulator to re-arm.  The per-block scaling is two FMAs per (row, sequence, block):
//   t = fma(F, w_sc * 2^110, -260096 * 2^-39 * w_sc)  =  16 * dot * w_sc * 2^-39
//   acc = fma(t, x_sc / 16 * 2^39, acc)
// (the powers of two keep every intermediate normal; the prep kernel stores x_sc / 16 * 2^39), both issued as packed
// fp32x2 instructions, two sequences at a time.  The packed instruction issues to half of the FMA pipe only; a scalar
// first stage (which can use the other half) and an all-scalar epilogue both measured slower (498 and 547 us against
// 482 us at 64 sequences): the epilogue is short of issue slots and latency hiding, not of FMA throughput.
//
// Roles inside a persistent CTA of 16 warps (a work unit is 128 weight rows x a range of 256-k chunks):
//   warp 0      producer: TMA 2-D loads of packed nibbles and weight scales, bulk copies of the activations
//   warp 1      MMA issuer (one elected lane)
//   warps 2-3   weight-scale loader: cp.async of each row's 16 scales per chunk into a ring, eight chunks ahead
//   warps 4-11  epilogue: tcgen05.ld, scaling, fp32 accumulation in registers, final store (thread = weight row
//               = TMEM lane; warps 4-7 take the first half of the sequences, warps 8-11 the second).  Accumulators are
//               read in pieces of 32 values (16 for 64 sequences) and the read of the next piece is issued before the
//               arithmetic of the current one: a tensor-memory read takes 100-150 cycles to return and only one batch
//               of reads can be in flight per warp (tcgen05.wait::ld has no count).
//   warps 12-15 unpack: nibbles -> signed bytes 16*q in the K-major core-matrix layout the MMA reads
// Measured on the 151,643 x 4096 matrix (tuning key 19 switches parts off): 16 / 32 / 64 sequences take 227 / 331 /
// 482 us; without the scaling arithmetic 182 / 219 / 347; with nothing but the barrier traffic and the accumulator
// reads 90 / 134 / 327.  The kernel is bound by the latency chain of the epilogue warps (issue slots 50 % busy, no
// pipe above 70 %), not by HBM (weights alone would take 58 us) or the tensor pipe (6 % busy).  Tried and measured
// slower: 16 epilogue warps with a quarter of the sequences each (545 us at 64 sequences: 80 registers, spills), a
// ring of four accumulator groups (616), 32-column reads at 64 sequences (534).
// All waits are bounded; a wait that gives up raises an abort flag that every role polls.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace bw {
namespace tc {

constexpr int kKc = 256;          // k per chunk = 16 k-blocks
constexpr int kBlocksPerChunk = 16;
constexpr int kRows = 128;        // weight rows per CTA tile = MMA M
constexpr int kSP = 4;            // packed-nibble ring slots
constexpr int kSA = 2;            // operand (A int8 + B) ring slots
constexpr int kSS = 4;            // scale ring slots
constexpr int kSW = 8;            // weight-scale ring slots (one chunk of one tile each)
constexpr int kABlockStride = 2048 + 16;  // bytes between the int8 tiles of consecutive k-blocks (odd 16-byte count
                                          // spreads the unpack stores over the shared-memory banks)
constexpr int kPackedBytes = kRows * (kKc / 2);                  // 16384
constexpr int kWScaleBytes = kRows * kBlocksPerChunk * 2;        // 4096
constexpr int kAStageBytes = kBlocksPerChunk * kABlockStride;    // 33024
constexpr int kEpiWarps = 8;     // epilogue warps: two per TMEM lane quarter, each half of the sequences
constexpr int kThreads = (4 + kEpiWarps + 4) * 32;   // + producer, MMA issuer, two scale-loader and four unpack warps

struct TcArgs {
    float* y;                 // [M][y_stride]
    const float* residual;    // optional, same layout as y
    long y_stride;
    const unsigned char* xb;  // activations in chunk layout (see prep kernel)
    const __half* Wsc;        // [N][nkb] weight scales
    int nkb;                  // K / 16
    float* partial;           // [tiles][ksplit][Mpad][128] when ksplit > 1
    unsigned int* tickets;    // [tiles], zero before and after the call
    int* status;              // device status word
    int N, M, Mpad;           // Mpad = MMA N in {16, 32, 64}
    int nchunks;              // ceil(K / 256)
    int ksplit;               // CTAs sharing one row tile
    int map_elem;             // bytes per element of the weight tensor map (its x coordinate is in elements)
#ifdef BW_GEMV_TIMELINE
    long long* timeline;      // experiment builds only: SM-clock stamps of CTA 0's roles, [slot][256]
#endif
    int ablate;               // measurement only (tuning key 19): 1 no epilogue math, 2 no unpack, 4 no weight loads, 8 no MMAs
};

// B operand of one chunk: 16 blocks of [Mpad sequences x 16 B]; the MMA's second K step reads the shared constant.
constexpr int kOffsetInt = 260096;                 // 16 (k) x (-128) x (-127): what the constant K step adds
constexpr float kWScaleUp = 0x1p110f;              // first-stage factor:  w_sc * 2^110 (binary16 scales stay finite)
constexpr float kXScaleUp = 0x1p39f;               // second-stage factor: x_sc / 16 * 2^39
constexpr float kOffsetTerm = -260096.0f * 0x1p-39f;  // times w_sc: cancels the constant K step
__host__ __device__ constexpr int b_chunk_bytes(int Mpad) { return kBlocksPerChunk * Mpad * 16; }
// bytes of one activation chunk in global memory: the B operand, then 16 x Mpad block scales
__host__ __device__ inline size_t xb_chunk_bytes(int Mpad) { return (size_t)b_chunk_bytes(Mpad) + (size_t)kBlocksPerChunk * Mpad * 4; }

// ------------------------------------------------------------------ tcgen05 wrappers
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D = A * B (accumulate == 0) or D += A * B.
__device__ __forceinline__ void tc_mma_i8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t addr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(addr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t addr, uint32_t (&v)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(addr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld4(uint32_t addr, uint32_t (&v)[4]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3])
                 : "r"(addr)
                 : "memory");
}
template <int CW>
__device__ __forceinline__ void tmem_ld_cols(uint32_t addr, uint32_t (&v)[CW]) {
    static_assert(CW == 4 || CW == 8 || CW == 16, "columns per read");
    if constexpr (CW == 4) tmem_ld4(addr, v);
    else if constexpr (CW == 8) tmem_ld8(addr, v);
    else tmem_ld16(addr, v);
}
// acc (two packed fp32) += ({f0, f1} * W2 + CN2) * xs2: the two scaling stages of one k-block for two sequences, both
// as packed fp32 instructions.  f0 / f1 are accumulator words read as (denormal) floats; W2 = {W, W}, CN2 = {CN, CN}.
__device__ __forceinline__ void scale_acc2(unsigned long long& acc, uint32_t f0, uint32_t f1, unsigned long long W2,
                                                  unsigned long long CN2, unsigned long long xs2) {
    asm("{\n\t.reg .b64 ff, tt;\n\t"
        "mov.b64 ff, {%1, %2};\n\t"
        "fma.rn.f32x2 tt, ff, %3, %4;\n\t"
        "fma.rn.f32x2 %0, tt, %5, %0;\n\t}"
        : "+l"(acc)
        : "r"(f0), "r"(f1), "l"(W2), "l"(CN2), "l"(xs2));
}
__device__ __forceinline__ unsigned long long pack2(float a) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %1};" : "=l"(r) : "f"(a));
    return r;
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// 2-D tiled TMA load (no multicast): box -> shared memory of this CTA, bytes counted on an mbarrier.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
// 4-byte asynchronous copy global -> shared; src_bytes 0 writes zeros.
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.ca.shared.global.L2::256B [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
// Makes the mbarrier receive one (pre-counted) arrival when all earlier cp.async of this thread have landed.
__device__ __forceinline__ void cp_async_arrive(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void bulk_g2s_plain(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

// Shared-memory matrix descriptor, K-major, no swizzle: rows of a core matrix 16 B apart, 8-row groups `sbo`
// bytes apart, the two 16-byte K steps of one MMA `lbo` bytes apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;  // descriptor version of this architecture
    return d;
}
// Instruction descriptor: D = s32, A = B = signed 8-bit, both K-major, M = 128, N = n.
__host__ __device__ inline uint32_t idesc_i8(int n) {
    return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kRows >> 4) << 24);
}

}  // namespace tc
}  // namespace bw
