// Host-side helpers shared by the kernel launchers.
#pragma once
#include <cuda_runtime.h>

#include <atomic>

namespace b200 {

// launches issued by this library since load (reported by b200_launch_count)
extern std::atomic<unsigned long long> g_launches;

// call right after a <<<>>> launch: counts it and returns 0 or the cudaError_t
inline int after_launch() {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}

} // namespace b200
