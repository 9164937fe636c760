// GQA decode attention over a binary16 cache on the tensor cores (warp-level mma.sync m16n8k16, f16 x f16 -> f32).
//
// With eight (or four) query heads per KV head the scalar kernel spends more instructions per cache byte than an SM
// can issue at HBM speed; here the heads of one KV head form the 16 rows of an MMA tile (rows >= the group size are
// zero), K and V rows stream through shared memory (cp.async, double-buffered per warp, XOR-swizzled 16-byte chunks,
// read back with ldmatrix), and a warp handles 16 positions per step:
//     S = Q K^T   : 8 k-steps x 2 position tiles                 (Q fragments live in registers)
//     online softmax on the accumulator fragment (row = head: quad shuffles)
//     O += P V    : 16 dimension tiles, P taken straight from the S fragment
// Q and P are split into a binary16 high part and a binary16 remainder and multiplied twice, so the products carry
// ~22 significant bits although the operands of one MMA are binary16; K and V are binary16 in the cache already.
// Splits, per-warp merge and the last-arriver split merge are those of the scalar kernel.
#pragma once
#include <cuda_fp16.h>

#include "common.cuh"

namespace bw {
namespace amma {

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
// D(16x8) += A(16x16) B(16x8); rows 8..15 of A are zero here (a1 = a3 = 0), so c2/c3 stay zero.
__device__ __forceinline__ void mma_16816(float& c0, float& c1, float& c2, float& c3, uint32_t a0, uint32_t a2,
                                          uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c0), "+f"(c1), "+f"(c2), "+f"(c3)
        : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}
// (x, y) -> packed binary16 high parts and packed binary16 remainders.
__device__ __forceinline__ void split_hi_lo(float x, float y, uint32_t& hi, uint32_t& lo) {
    const __half2 h = __floats2half2_rn(x, y);
    const float2 hf = __half22float2(h);
    const __half2 l = __floats2half2_rn(x - hf.x, y - hf.y);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = *reinterpret_cast<const uint32_t*>(&l);
}

constexpr int kTile = 16;                   // positions per warp step
constexpr int kTileBytes = kTile * 256;     // one K or V tile: 16 rows x 128 halves
constexpr int kWarpSmem = 4 * kTileBytes;   // K and V, two buffers each
// byte offset of 16-byte chunk c of row r inside a tile (chunks XOR-swizzled by the row)
__device__ __forceinline__ uint32_t tile_off(int r, int c) { return (uint32_t)(r * 256 + ((c ^ (r & 7)) << 4)); }

// One 16-position K/V tile of a warp into buffer `buf` of its staging area: rows past `last_row` are clamped to it
// (the caller masks them, and a clamped row is real data where memory past the sequence's end may hold anything).
__device__ __forceinline__ void issue_tile(const __half* Kb, const __half* Vb, uint32_t sbase, int buf, int tpos,
                                           int last_row) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int idx = i * 32 + lane;          // 256 chunks per tile
        const int r = idx >> 4, c = idx & 15;
        const int pos = min(tpos + r, last_row);
        cp_async16(sbase + buf * 2 * kTileBytes + tile_off(r, c), Kb + (size_t)pos * 128 + c * 8);
        cp_async16(sbase + buf * 2 * kTileBytes + kTileBytes + tile_off(r, c), Vb + (size_t)pos * 128 + c * 8);
    }
    cp_async_commit();
}

// Streams the positions [p0, p1) of one (sequence, kv head) through one warp: returns, for head g = lane / 4, the
// running maximum, this thread's share of the softmax sum and the un-normalised outputs of dimensions
// 8 * j + 2 * (lane % 4) + {0, 1}, j = 0..15, in o[2 * j + {0, 1}].
template <int GQ>
__device__ __forceinline__ void warp_stream(const __half* Kb, const __half* Vb, const float* q_heads /* [GQ][128] */,
                                            float scale, int p0, int p1, int warp, int nwarps, unsigned char* wsmem,
                                            float& m_run, float& l_run, float (&o)[32], bool first_issued = false,
                                            int fresh_end = 0) {
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    // Q fragments for the 8 k-steps: a0 = Q[g][16 ks + 2t, +1], a2 = Q[g][16 ks + 8 + 2t, +1]
    uint32_t qh0[8], qh2[8], ql0[8], ql2[8];
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
        float2 v0 = make_float2(0.f, 0.f), v2 = make_float2(0.f, 0.f);
        if (g < GQ) {
            v0 = *reinterpret_cast<const float2*>(q_heads + g * 128 + 16 * ks + 2 * t);
            v2 = *reinterpret_cast<const float2*>(q_heads + g * 128 + 16 * ks + 8 + 2 * t);
        }
        split_hi_lo(v0.x * scale, v0.y * scale, qh0[ks], ql0[ks]);
        split_hi_lo(v2.x * scale, v2.y * scale, qh2[ks], ql2[ks]);
    }
    m_run = -FLT_MAX;
    l_run = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) o[i] = 0.f;

    const uint32_t sbase = smem_u32(wsmem);
    const int ntile = (p1 - p0 + kTile - 1) / kTile;
    // tiles of this warp: warp, warp + nwarps, ...
    auto issue = [&](int tile_idx, int buf) { issue_tile(Kb, Vb, sbase, buf, p0 + tile_idx * kTile, p1 - 1); };
    int it = 0;
    // `first_issued`: the caller requested this warp's first tile (rows p0 + 16 warp ...) before it knew the sequence's
    // position.  The copy is good if all its rows lie below `fresh_end` (the end of the rows that were final then);
    // otherwise it is requested again (after the first has landed: both write the same buffer).
    if (first_issued && p0 + (warp + 1) * kTile > fresh_end) {
        cp_async_wait<0>();
        __syncwarp();
        first_issued = false;
    }
    if (warp < ntile && !first_issued) issue(warp, 0);
    for (int ti = warp; ti < ntile; ti += nwarps, ++it) {
        const int buf = it & 1;
        if (ti + nwarps < ntile) {
            issue(ti + nwarps, buf ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncwarp();
        const uint32_t kt = sbase + buf * 2 * kTileBytes, vt = kt + kTileBytes;
        const int tpos = p0 + ti * kTile;

        // ---- S = Q K^T for 16 positions: s0/s1 = positions 2t, 2t+1 ; s4/s5 = positions 8 + 2t, 8 + 2t + 1
        // four independent accumulator chains (high and low part of Q, two position tiles): a chain of dependent
        // MMAs runs at one MMA per MMA latency, so the shorter the chains the better the tensor pipe is fed
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f, s4 = 0.f, s5 = 0.f, s6 = 0.f, s7 = 0.f;
        float r0 = 0.f, r1 = 0.f, r2 = 0.f, r3 = 0.f, r4 = 0.f, r5 = 0.f, r6 = 0.f, r7 = 0.f;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            uint32_t b0, b1, b2, b3;
            const int mi = lane >> 3, rr = lane & 7;
            ldmatrix_x4(kt + tile_off((mi >> 1) * 8 + rr, 2 * ks + (mi & 1)), b0, b1, b2, b3);
            mma_16816(s0, s1, s2, s3, qh0[ks], qh2[ks], b0, b1);
            mma_16816(r0, r1, r2, r3, ql0[ks], ql2[ks], b0, b1);
            mma_16816(s4, s5, s6, s7, qh0[ks], qh2[ks], b2, b3);
            mma_16816(r4, r5, r6, r7, ql0[ks], ql2[ks], b2, b3);
        }
        s0 += r0; s1 += r1; s4 += r4; s5 += r5;
        // ---- online softmax for head g over the 16 positions (4 per thread, 4 threads per head)
        const int pa = tpos + 2 * t, pb = tpos + 8 + 2 * t;
        s0 = pa < p1 ? s0 : -FLT_MAX;
        s1 = pa + 1 < p1 ? s1 : -FLT_MAX;
        s4 = pb < p1 ? s4 : -FLT_MAX;
        s5 = pb + 1 < p1 ? s5 : -FLT_MAX;
        float mx = fmaxf(fmaxf(s0, s1), fmaxf(s4, s5));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float mnew = fmaxf(m_run, mx);
        const float corr = __expf(m_run - mnew);
        const float e0 = pa < p1 ? __expf(s0 - mnew) : 0.f;
        const float e1 = pa + 1 < p1 ? __expf(s1 - mnew) : 0.f;
        const float e4 = pb < p1 ? __expf(s4 - mnew) : 0.f;
        const float e5 = pb + 1 < p1 ? __expf(s5 - mnew) : 0.f;
        l_run = l_run * corr + (e0 + e1 + e4 + e5);
        m_run = mnew;
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] *= corr;
        uint32_t ph0, pl0, ph2, pl2;   // A fragment of P: a0 = positions 2t, 2t+1 ; a2 = positions 8 + 2t, +1
        split_hi_lo(e0, e1, ph0, pl0);
        split_hi_lo(e4, e5, ph2, pl2);
        // ---- O += P V : 16 dimension tiles of 8, two per ldmatrix
        float z0 = 0.f, z1 = 0.f;
#pragma unroll
        for (int jn = 0; jn < 16; jn += 2) {
            uint32_t b0, b1, b2, b3;
            const int mi = lane >> 3, rr = lane & 7;
            ldmatrix_x4_trans(vt + tile_off((mi & 1) * 8 + rr, jn + (mi >> 1)), b0, b1, b2, b3);
            mma_16816(o[2 * jn], o[2 * jn + 1], z0, z1, ph0, ph2, b0, b1);
            mma_16816(o[2 * jn], o[2 * jn + 1], z0, z1, pl0, pl2, b0, b1);
            mma_16816(o[2 * jn + 2], o[2 * jn + 3], z0, z1, ph0, ph2, b2, b3);
            mma_16816(o[2 * jn + 2], o[2 * jn + 3], z0, z1, pl0, pl2, b2, b3);
        }
        __syncwarp();  // the buffer is refilled two iterations later by this same warp
    }
    cp_async_wait<0>();   // an early first tile this warp turned out not to need
    // the four threads of a head each hold a quarter of the sum
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
}

}  // namespace amma
}  // namespace bw
