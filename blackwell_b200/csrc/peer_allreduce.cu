// All-reduce of the K-split GEMV partial sums over peer memory (NVLink), for tensor-parallel decode on the GPUs of
// one box.  The reference is single-GPU (server/inference_server_int4_batched.cu holds one device's weights), so
// nothing here replaces a reference function; it is the exchange the O and down projections need once their K
// dimension is split across ranks.
//
// Every rank owns one region (cudaMalloc): [flags][flags 2][epochs][status][slot 0][slot 1][result].  Peers map it (CUDA IPC between
// processes, or direct peer access inside one process).  The GEMV writes its partial sums straight into the local
// slot; one kernel then
//   1. tells every peer "my slot is complete" (a release store of the call's epoch into the peer's flag array),
//   2. waits for the same word from every peer (acquire loads, bounded: gives up after ~2 s -- or the limit set
//      through bw_set_tuning key 11 -- sets the status word to 3, leaves the output untouched and returns),
//   3. sums the slot of every rank, in rank order, with plain 16-byte peer loads, adds an optional residual, and
//      writes the result to local memory.  All ranks add in the same order, so they hold bit-identical results.
// Slots alternate between consecutive exchanges: a rank overwrites a slot only after it finished the following
// exchange, whose step 2 proves that every peer had finished reading it.  Flags and epochs are per CTA index, so CTAs
// never wait for one another on the same GPU; the grid is capped at the SM count (all CTAs resident).
// Large vectors (4 MiB and up by default) on four or more ranks take the two-step form: after the same barrier a rank sums only its own
// 1/world slice, stores the sums into every rank's result area (plain peer stores), and a second barrier tells when
// all slices have landed; that moves 2 (world-1)/world of the vector per GPU instead of (world-1) vectors.  The
// result area needs no double buffering: a peer stores into it only after this rank signalled the call's first
// barrier, i.e. after every earlier reader of the area on this rank has completed.
// Loads and stores are plain peer accesses: no multimem, no TMA, no cluster multicast.
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <new>

#include "../../include/blackwell_b200.h"
#include "common.cuh"
#include "host_util.h"

namespace bw {
namespace peer {

constexpr int kMaxWorld = 8;
constexpr int kMaxCtas = 160;
constexpr int kThreads = 256;
constexpr size_t kFlagBytes = (size_t)kMaxCtas * kMaxWorld * sizeof(uint32_t);   // flags[cta][source rank]
constexpr size_t kFlag2Off = kFlagBytes;                                          // second barrier of the two-step form
constexpr size_t kEpochOff = 2 * kFlagBytes;                                      // epochs[cta]
constexpr size_t kStatusOff = kEpochOff + (size_t)kMaxCtas * sizeof(uint32_t);
constexpr size_t kHeaderBytes = 16384;                                            // slots start here; then the result area
static_assert(kStatusOff + sizeof(int) <= kHeaderBytes, "header too small");

// Smallest vector (KiB) that takes the two-step form on four or more ranks; 0 = the default.
static int g_two_step_min_kb = 0;
void set_two_step_min_kb(int kb) { g_two_step_min_kb = kb; }
// Longest time a CTA waits for a peer's flag, in milliseconds; 0 = the default of about two seconds.
static int g_wait_limit_ms = 0;
void set_wait_limit_ms(int ms) { g_wait_limit_ms = ms; }

struct Comm {
    int world, rank, device;
    size_t slot_bytes;
    unsigned char* base[kMaxWorld];   // base[rank] = local region, others peer-mapped
    bool ipc_mapped[kMaxWorld];
};

struct Args {
    float* out;
    const float* residual;
    const float* slot[kMaxWorld];
    float* result[kMaxWorld];         // two-step form: every rank's result area
    uint32_t* flags[kMaxWorld];
    uint32_t* epochs;
    int* status;
    int world, rank;
    unsigned long long n4;            // number of float4
    long long wait_cycles;            // a wait for a peer gives up after this many SM clock cycles
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// Peer data changes between calls: bypass the L1 (which does not snoop the peer) with a volatile 16-byte load.
__device__ __forceinline__ float4 ld_peer_f4(const float* p) {
    float4 v;
    asm volatile("ld.volatile.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}

// residual + slot[0] + slot[1] + ... for one float4, in rank order.  The loads of all ranks are issued before the
// first add: a peer load takes a couple of microseconds, and one after the other they would add up.
__device__ __forceinline__ float4 sum_ranks(const Args& a, unsigned long long i) {
    float4 v[kMaxWorld];
#pragma unroll
    for (int r = 0; r < kMaxWorld; ++r)
        if (r < a.world) v[r] = ld_peer_f4(a.slot[r] + 4 * i);
    float4 s = a.residual ? *reinterpret_cast<const float4*>(a.residual + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int r = 0; r < kMaxWorld; ++r)
        if (r < a.world) { s.x += v[r].x; s.y += v[r].y; s.z += v[r].z; s.w += v[r].w; }
    return s;
}

// Bounded wait of thread t < world for peer t's word in this rank's flag array; false when it gave up.
__device__ __forceinline__ bool wait_peer_flag(const uint32_t* mine, uint32_t e, long long limit) {
    const long long t0 = clock64();
#pragma unroll 1
    while (true) {
        if ((int)(ld_acquire_sys(mine) - e) >= 0) return true;
        if (clock64() - t0 > limit) return false;
        __nanosleep(20);
    }
}

__global__ void __launch_bounds__(kThreads) peer_allreduce_kernel(const Args a) {
    __shared__ uint32_t s_epoch;
    __shared__ int s_fail;
    const int t = threadIdx.x, c = blockIdx.x;
    // Programmatic dependent launch on both sides: this kernel may become resident while the GEMV that fills the
    // slot is still running (it waits here for it), and the kernel after it may start its own weight prefetch while
    // this one waits for the peers (that kernel's own wait covers this kernel's completion).
    pdl_trigger();
    pdl_wait();
    if (t == 0) {
        s_epoch = a.epochs[c] + 1u;
        s_fail = 0;
    }
    __syncthreads();
    const uint32_t e = s_epoch;
    if (t < a.world) {
        st_release_sys(a.flags[t] + c * kMaxWorld + a.rank, e);            // to peer t: rank's slot is complete
        if (!wait_peer_flag(a.flags[a.rank] + c * kMaxWorld + t, e, a.wait_cycles)) s_fail = 1;   // from peer t
    }
    __syncthreads();
    if (s_fail) {
        if (t == 0) {
            atomicExch(a.status, 3);
            a.epochs[c] = e;
        }
        return;
    }
    for (unsigned long long i = (unsigned long long)c * kThreads + t; i < a.n4; i += (unsigned long long)gridDim.x * kThreads) {
        *reinterpret_cast<float4*>(a.out + 4 * i) = sum_ranks(a, i);
    }
    if (t == 0) a.epochs[c] = e;
}


// Two-step form.  The vector is cut into world slices of slice4 float4 (the last may be short); CTA c of rank r sums
// the float4 [c * per_cta, (c + 1) * per_cta) of slice r and stores them to every rank; after the second barrier CTA c
// copies that range of every slice from the local result area to out.
__global__ void __launch_bounds__(kThreads) peer_allreduce2_kernel(const Args a, unsigned long long slice4,
                                                                   unsigned long long per_cta) {
    __shared__ uint32_t s_epoch;
    __shared__ int s_fail;
    const int t = threadIdx.x, c = blockIdx.x;
    pdl_trigger();
    pdl_wait();
    if (t == 0) {
        s_epoch = a.epochs[c] + 1u;
        s_fail = 0;
    }
    __syncthreads();
    const uint32_t e = s_epoch;
    if (t < a.world) {
        st_release_sys(a.flags[t] + c * kMaxWorld + a.rank, e);
        if (!wait_peer_flag(a.flags[a.rank] + c * kMaxWorld + t, e, a.wait_cycles)) s_fail = 1;
    }
    __syncthreads();
    const bool fail1 = s_fail != 0;
    if (!fail1) {
        const unsigned long long lo = (unsigned long long)a.rank * slice4 + (unsigned long long)c * per_cta;
        unsigned long long hi = lo + per_cta;
        const unsigned long long slice_end = min((unsigned long long)(a.rank + 1) * slice4, a.n4);
        if (hi > slice_end) hi = slice_end;
        for (unsigned long long i = lo + t; i < hi; i += kThreads) {
            const float4 s = sum_ranks(a, i);
#pragma unroll
            for (int r = 0; r < kMaxWorld; ++r)
                if (r < a.world) *reinterpret_cast<float4*>(a.result[r] + 4 * i) = s;
        }
        __threadfence_system();   // this thread's peer stores are visible before the CTA signals
    }
    __syncthreads();
    // second barrier: always signalled, so that a peer never waits for a rank that merely failed the first one
    uint32_t* f2 = nullptr;
    if (t < a.world) {
        f2 = reinterpret_cast<uint32_t*>(reinterpret_cast<unsigned char*>(a.flags[t]) + kFlag2Off);
        st_release_sys(f2 + c * kMaxWorld + a.rank, e);
        const uint32_t* mine2 = reinterpret_cast<const uint32_t*>(reinterpret_cast<const unsigned char*>(a.flags[a.rank]) + kFlag2Off);
        if (!wait_peer_flag(mine2 + c * kMaxWorld + t, e, a.wait_cycles)) s_fail = 1;
    }
    __syncthreads();
    if (s_fail) {
        if (t == 0) {
            atomicExch(a.status, 3);
            a.epochs[c] = e;
        }
        return;
    }
    for (int r = 0; r < a.world; ++r) {
        const unsigned long long lo = (unsigned long long)r * slice4 + (unsigned long long)c * per_cta;
        unsigned long long hi = lo + per_cta;
        const unsigned long long slice_end = min((unsigned long long)(r + 1) * slice4, a.n4);
        if (hi > slice_end) hi = slice_end;
        for (unsigned long long i = lo + t; i < hi; i += kThreads)
            *reinterpret_cast<float4*>(a.out + 4 * i) = ld_peer_f4(a.result[a.rank] + 4 * i);
    }
    if (t == 0) a.epochs[c] = e;
}

}  // namespace peer
}  // namespace bw

using namespace bw;
using namespace bw::peer;

extern "C" int bw_peer_comm_create(int world, int rank, size_t slot_bytes, void** comm_out) {
    if (!comm_out || world < 2 || world > kMaxWorld || rank < 0 || rank >= world || slot_bytes == 0) return cudaErrorInvalidValue;
    slot_bytes = (slot_bytes + 255) & ~(size_t)255;
    Comm* cm = new (std::nothrow) Comm();
    if (!cm) return cudaErrorMemoryAllocation;
    cm->world = world; cm->rank = rank; cm->device = current_device(); cm->slot_bytes = slot_bytes;
    for (int i = 0; i < kMaxWorld; ++i) { cm->base[i] = nullptr; cm->ipc_mapped[i] = false; }
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, kHeaderBytes + 3 * slot_bytes);
    if (e == cudaSuccess) e = cudaMemset(p, 0, kHeaderBytes + 3 * slot_bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        if (p) cudaFree(p);
        delete cm;
        return e;
    }
    cm->base[rank] = static_cast<unsigned char*>(p);
    *comm_out = cm;
    return cudaSuccess;
}

extern "C" int bw_peer_comm_handle(void* comm, void* handle_out_64) {
    Comm* cm = static_cast<Comm*>(comm);
    if (!cm || !handle_out_64) return cudaErrorInvalidValue;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    return cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle_out_64), cm->base[cm->rank]);
}

extern "C" int bw_peer_comm_open(void* comm, int peer_rank, const void* handle_64) {
    Comm* cm = static_cast<Comm*>(comm);
    if (!cm || !handle_64 || peer_rank < 0 || peer_rank >= cm->world || peer_rank == cm->rank || cm->base[peer_rank])
        return cudaErrorInvalidValue;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle_64, sizeof(h));
    void* p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return e;
    cm->base[peer_rank] = static_cast<unsigned char*>(p);
    cm->ipc_mapped[peer_rank] = true;
    return cudaSuccess;
}

extern "C" int bw_peer_comm_attach(void* comm, int peer_rank, void* peer_comm_same_process) {
    Comm* cm = static_cast<Comm*>(comm);
    Comm* pc = static_cast<Comm*>(peer_comm_same_process);
    if (!cm || !pc || peer_rank < 0 || peer_rank >= cm->world || peer_rank == cm->rank || pc->rank != peer_rank ||
        pc->slot_bytes != cm->slot_bytes || cm->base[peer_rank])
        return cudaErrorInvalidValue;
    if (cm->device != pc->device) {  // two communicators on one device see each other's memory as it is
        int can = 0;
        cudaError_t e = cudaDeviceCanAccessPeer(&can, cm->device, pc->device);
        if (e != cudaSuccess) return e;
        if (!can) return cudaErrorPeerAccessUnsupported;
        int prev = 0;
        cudaGetDevice(&prev);
        cudaSetDevice(cm->device);
        e = cudaDeviceEnablePeerAccess(pc->device, 0);
        if (e == cudaErrorPeerAccessAlreadyEnabled) { e = cudaSuccess; cudaGetLastError(); }
        cudaSetDevice(prev);
        if (e != cudaSuccess) return e;
    }
    cm->base[peer_rank] = pc->base[pc->rank];
    return cudaSuccess;
}

extern "C" float* bw_peer_comm_slot(void* comm, int slot) {
    Comm* cm = static_cast<Comm*>(comm);
    if (!cm || slot < 0 || slot > 1) return nullptr;
    return reinterpret_cast<float*>(cm->base[cm->rank] + kHeaderBytes + (size_t)slot * cm->slot_bytes);
}

extern "C" int bw_peer_allreduce_f32(void* comm, int slot, float* out, const float* residual_or_null, size_t n,
                                     void* stream) {
    Comm* cm = static_cast<Comm*>(comm);
    if (!cm || slot < 0 || slot > 1 || !out || n == 0 || n % 4 != 0 || n * sizeof(float) > cm->slot_bytes)
        return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(out) & 15) || (reinterpret_cast<uintptr_t>(residual_or_null) & 15)) return cudaErrorInvalidValue;
    Args a;
    for (int r = 0; r < kMaxWorld; ++r) { a.slot[r] = nullptr; a.flags[r] = nullptr; }
    for (int r = 0; r < cm->world; ++r) {
        if (!cm->base[r]) return cudaErrorInvalidValue;  // a peer was never opened
        a.slot[r] = reinterpret_cast<const float*>(cm->base[r] + kHeaderBytes + (size_t)slot * cm->slot_bytes);
        a.flags[r] = reinterpret_cast<uint32_t*>(cm->base[r]);
    }
    unsigned char* mine = cm->base[cm->rank];
    a.epochs = reinterpret_cast<uint32_t*>(mine + kEpochOff);
    a.status = reinterpret_cast<int*>(mine + kStatusOff);
    a.out = out; a.residual = residual_or_null; a.world = cm->world; a.rank = cm->rank; a.n4 = n / 4;
    // counted on the SM clock (at most ~2.1 GHz): the default is about two seconds at any clock
    a.wait_cycles = g_wait_limit_ms > 0 ? (long long)g_wait_limit_ms * 2100000ll : 4000000000ll;
    for (int r = 0; r < cm->world; ++r)
        a.result[r] = reinterpret_cast<float*>(cm->base[r] + kHeaderBytes + 2 * cm->slot_bytes);
    const int cap = sm_count(cm->device) < kMaxCtas ? sm_count(cm->device) : kMaxCtas;
    cudaError_t le;
    // measured on 4 and 8 GPUs: at 1.3 MB the one-step form is still the faster one (22.1 vs 22.7 ms per 32B-shape step)
    const size_t two_step_min = (size_t)(g_two_step_min_kb > 0 ? g_two_step_min_kb : 4096) << 10;
    if (cm->world >= 4 && n * sizeof(float) >= two_step_min) {
        // two-step form: CTAs split one slice; every CTA must be resident (it waits for peers), hence at most one per SM
        const unsigned long long slice4 = (a.n4 + cm->world - 1) / cm->world;
        int grid = (int)((slice4 + (size_t)kThreads - 1) / (size_t)kThreads);
        if (grid > cap) grid = cap;
        if (grid < 1) grid = 1;
        const unsigned long long per_cta = (slice4 + grid - 1) / grid;
        le = launch_pdl(peer_allreduce2_kernel, dim3(grid), dim3(kThreads), 0, static_cast<cudaStream_t>(stream), a, slice4,
                        per_cta);
    } else {
        // one float4 per thread where the SM count allows (every CTA must be resident: it waits for a peer)
        int grid = (int)((a.n4 + (size_t)kThreads - 1) / (size_t)kThreads);
        if (grid > cap) grid = cap;
        if (grid < 1) grid = 1;
        le = launch_pdl(peer_allreduce_kernel, dim3(grid), dim3(kThreads), 0, static_cast<cudaStream_t>(stream), a);
    }
    count_launch(1);
    return le != cudaSuccess ? le : cudaPeekAtLastError();
}

extern "C" int bw_peer_comm_status(void* comm, int* status_out) {
    Comm* cm = static_cast<Comm*>(comm);
    if (!cm || !status_out) return cudaErrorInvalidValue;
    int v = 0;
    cudaError_t e = cudaMemcpy(&v, cm->base[cm->rank] + kStatusOff, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return e;
    if (v != 0) {
        const int zero = 0;
        e = cudaMemcpy(cm->base[cm->rank] + kStatusOff, &zero, sizeof(int), cudaMemcpyHostToDevice);
    }
    *status_out = v;
    return e;
}

extern "C" int bw_peer_comm_destroy(void* comm) {
    Comm* cm = static_cast<Comm*>(comm);
    if (!cm) return cudaErrorInvalidValue;
    cudaError_t first = cudaSuccess;
    for (int r = 0; r < cm->world; ++r) {
        if (r != cm->rank && cm->base[r] && cm->ipc_mapped[r]) {
            cudaError_t e = cudaIpcCloseMemHandle(cm->base[r]);
            if (first == cudaSuccess) first = e;
        }
    }
    if (cm->base[cm->rank]) {
        cudaError_t e = cudaFree(cm->base[cm->rank]);
        if (first == cudaSuccess) first = e;
    }
    delete cm;
    return first;
}
