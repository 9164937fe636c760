// INT4-weight x INT8-activation block-16 GEMM for batches of 9..64 sequences on the 5th-generation tensor cores
// (tcgen05.mma kind::i8, accumulators in tensor memory).  Device side.
//
//   y[m][n] = sum_kb dot16(W[n,kb], xq[m,kb]) * w_sc[n,kb] * x_sc[m,kb]
//
// The scale changes every 16 k, the MMA consumes 32 k: each k-block gets its own MMA whose A operand holds the
// block in its first 16-byte K core matrix and a shared all-zero core matrix in the second (the descriptor's
// leading-dimension offset points the second K step at the zero region), so every accumulator tile is the exact
// int32 dot product of ONE k-block.  Accumulator tiles start from the bit pattern of 1.5 * 2^23 (the epilogue stores
// it back after every read), so the value read is a float holding 12582912 + 16 * dot exactly and the per-block
// scaling is two FMAs per (row, sequence, block): t = fma(F, w_sc, -12582912 * w_sc) (exact for binary16
// scales), acc = fma(t, x_sc/16, acc) -- issued as packed fp32x2 instructions, two sequences at a time.
//
// Roles inside a persistent CTA of 12 warps (a work unit is 128 weight rows x a range of 256-k chunks):
//   warp 0      producer: TMA 2-D loads of packed nibbles and weight scales, bulk copies of the activations
//   warp 1      MMA issuer (one elected lane)
//   warps 2-3   weight-scale loader: cp.async of each row's 16 scales per chunk into a ring, eight chunks ahead
//   warps 4-11  epilogue: tcgen05.ld, scaling, fp32 accumulation in registers, final store (thread = weight row
//               = TMEM lane; warps 4-7 take the first half of the sequences, warps 8-11 the second, so that
//               every scheduler has two epilogue warps to overlap and each thread keeps half the accumulators)
//   warps 12-15 unpack: nibbles -> signed bytes 16*q in the K-major core-matrix layout the MMA reads
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
constexpr int kThreads = 512;

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
};

// B operand of one chunk: 8 block pairs, each [block 2p: Mpad rows x 16 B][Mpad rows of zeros][block 2p + 1].
// One MMA (K = 32) takes a pair: its first K step reads rows [0, 2 Mpad) from the start of the pair (block 2p, then
// the zeros), its second K step the same number of rows starting at the zeros (zeros, then block 2p + 1), so the
// accumulator columns [0, Mpad) hold the dots of block 2p and [Mpad, 2 Mpad) those of block 2p + 1.
__host__ __device__ constexpr int b_chunk_bytes(int Mpad) { return (kBlocksPerChunk / 2) * 3 * Mpad * 16; }
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
__device__ __forceinline__ void tmem_st8_const(uint32_t addr, uint32_t c) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %1, %1, %1, %1, %1, %1, %1};" ::"r"(addr), "r"(c) : "memory");
}
__device__ __forceinline__ void tmem_st16_const(uint32_t addr, uint32_t c) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1};"
        ::"r"(addr), "r"(c)
        : "memory");
}
// Two fp32 FMAs in one instruction (sm_100 packed single precision): d = a * b + c lane-wise on register pairs.
__device__ __forceinline__ void ffma2(float& d0, float& d1, float a0, float a1, float b0, float b1, float c0, float c1) {
    unsigned long long A, B, C, D;
    asm("mov.b64 %0, {%1, %2};" : "=l"(A) : "f"(a0), "f"(a1));
    asm("mov.b64 %0, {%1, %2};" : "=l"(B) : "f"(b0), "f"(b1));
    asm("mov.b64 %0, {%1, %2};" : "=l"(C) : "f"(c0), "f"(c1));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(D) : "l"(A), "l"(B), "l"(C));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d0), "=f"(d1) : "l"(D));
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

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
