// Small host-side helpers shared by the launch wrappers.
#pragma once
#include <cuda_runtime.h>

#include <mutex>
#include <vector>

namespace bw {

constexpr int kMaxDevices = 16;
constexpr int kMaxDynSmem = 232448;  // 227 KB of dynamic shared memory per CTA on sm_100

inline int current_device() {
    int d = 0;
    cudaGetDevice(&d);
    return (d >= 0 && d < kMaxDevices) ? d : 0;
}

// SM count of a device, queried once.
inline int sm_count(int dev) {
    static int cached[kMaxDevices] = {0};
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

// Launch with programmatic stream serialization: the kernel may begin before its predecessor in the stream has
// finished and must call pdl_wait() before touching anything the predecessor produces or still reads.
bool pdl_enabled();
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Launch accounting (bw_launch_count).
void count_launch(int n);

// Device address of the library's status word on the current device (see bw_device_status); nullptr on failure.
int* status_word_ptr();

// Grow-only per-device scratch memory of one kernel family, zero-filled when allocated.  A block that has been
// handed out is never freed while the library is loaded: kernel launches already enqueued -- or captured in a CUDA
// graph -- keep pointing at it, so growth parks the old block instead of freeing it.  Growth allocates (and
// synchronises), so it cannot happen while the calling stream is being captured: such a call fails with
// cudaErrorStreamCaptureUnsupported and the caller must size the scratch beforehand (bw_reserve_scratch, or one
// eager call of the same shape).  All streams of a device share the block: two calls that use it must not overlap.
class GrowScratch {
public:
    cudaError_t get(size_t bytes, size_t floor_bytes, cudaStream_t st, unsigned char** out) {
        std::lock_guard<std::mutex> lk(mu_);
        Block& b = cur_[current_device()];
        if (b.bytes < bytes) {
            cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
            if (cudaStreamIsCapturing(st, &cs) == cudaSuccess && cs != cudaStreamCaptureStatusNone)
                return cudaErrorStreamCaptureUnsupported;
            size_t want = bytes < floor_bytes ? floor_bytes : bytes;
            if (want < 2 * b.bytes) want = 2 * b.bytes;  // geometric growth bounds what the parked blocks hold
            unsigned char* p = nullptr;
            cudaError_t e = cudaMalloc(&p, want);
            if (e != cudaSuccess) return e;
            e = cudaMemset(p, 0, want);  // arrival counters inside must start at zero
            if (e != cudaSuccess) { cudaFree(p); return e; }
            if (b.ptr) retired_.push_back(b.ptr);
            b.ptr = p;
            b.bytes = want;
        }
        *out = b.ptr;
        return cudaSuccess;
    }

private:
    struct Block { unsigned char* ptr = nullptr; size_t bytes = 0; };
    Block cur_[kMaxDevices];
    std::vector<unsigned char*> retired_;
    std::mutex mu_;
};

}  // namespace bw
