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

// Launch accounting (bw_launch_count).
void count_launch(int n);

}  // namespace bw
