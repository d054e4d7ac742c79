// Host-side helpers shared by the launchers: per-device one-time set-up that is safe when several host
// threads make their first call on a device at the same moment, the cached SM count, and the
// benchmark-only tuning overrides (compiled out of the shipped library).
#pragma once

#include <cuda_runtime.h>

#include <atomic>
#include <cstdlib>
#include <mutex>

namespace pg {

constexpr int kMaxDevices = 64;

// Runs `f` once per device ordinal.  The ready flag is published (release) only after `f` has filled
// whatever tables it owns, so a thread that sees it set (acquire) also sees the tables.  A failing
// `f` leaves the flag clear: the next call tries again.
class DeviceOnce {
public:
    template <class F>
    cudaError_t run(int dev, F &&f) {
        if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
        if (ready_[dev].load(std::memory_order_acquire)) return cudaSuccess;
        std::lock_guard<std::mutex> lock(mu_);
        if (ready_[dev].load(std::memory_order_relaxed)) return cudaSuccess;
        const cudaError_t e = f();
        if (e == cudaSuccess) ready_[dev].store(true, std::memory_order_release);
        return e;
    }

private:
    std::mutex mu_;
    std::atomic<bool> ready_[kMaxDevices] = {};
};

// Ordinal of the current device, checked against the tables' size.
inline cudaError_t current_device(int *dev) {
    const cudaError_t e = cudaGetDevice(dev);
    if (e != cudaSuccess) return e;
    return (*dev < 0 || *dev >= kMaxDevices) ? cudaErrorInvalidDevice : cudaSuccess;
}

// SM count of the current device, queried once per device.
inline cudaError_t current_device_sm_count(int *out) {
    static DeviceOnce once;
    static int table[kMaxDevices] = {};
    int dev = 0;
    cudaError_t e = current_device(&dev);
    if (e != cudaSuccess) return e;
    e = once.run(dev, [&]() { return cudaDeviceGetAttribute(&table[dev], cudaDevAttrMultiProcessorCount, dev); });
    if (e != cudaSuccess) return e;
    *out = table[dev];
    return cudaSuccess;
}

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per device for one kernel instantiation: every
// launcher template holds its own DeviceOnce.
template <class Kernel>
cudaError_t allow_dynamic_smem(DeviceOnce &once, Kernel kernel, int bytes) {
    int dev = 0;
    const cudaError_t e = current_device(&dev);
    if (e != cudaSuccess) return e;
    return once.run(dev, [&]() { return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes); });
}

// Records a failed CUDA call for pg_last_cuda_error() of the calling thread, clears the runtime's error state
// and returns PG_ERR_CUDA (api.cu).
int record_cuda_failure(cudaError_t e);

// Benchmark-only override from the environment (PEAKGEMM_TUNE_*).  The shipped library is built without
// PG_ENABLE_TUNING and never reads the environment: the function then returns `fallback`.
inline int tune_env_int(const char *name, int fallback) {
#ifdef PG_ENABLE_TUNING
    const char *v = std::getenv(name);
    return v ? std::atoi(v) : fallback;
#else
    (void)name;
    return fallback;
#endif
}

}  // namespace pg
