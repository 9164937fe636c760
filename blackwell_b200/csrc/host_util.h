// Small host-side helpers shared by the launch wrappers.
#pragma once
#include <cuda_runtime.h>

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

}  // namespace bw
