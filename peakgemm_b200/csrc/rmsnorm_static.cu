// pg_rmsnorm_bwd_static: RMSNorm backward for callers that must not allocate.
//
// Who this is for: code that runs where device allocation is off the table — a
// plugin called from inside someone else's stream-ordered region, a real-time
// loop that may not take the allocator's locks, a host that hands this library
// raw pointers and owns no allocator of its own (a plain C or Fortran caller,
// for instance).  pg_rmsnorm_bwd wants such a caller to bring a workspace; this
// entry point brings its own instead: a fixed array that lives in the library
// image on every GPU that loads it.
//
// The backward kernel's only scratch is the table of fp32 dgamma partial rows
// (one row of h floats per CTA).  Here that table is the file-scope array below.
// In host code the array's NAME is just a host-side handle, not something a
// kernel can dereference, so the device address is looked up once per device
// with cudaGetSymbolAddress (while that device is current) and that pointer is
// what the kernels receive.
#include <cuda_runtime.h>
#include <mutex>
#include <stdint.h>

#include "../../include/peakgemm.h"
#include "host_util.h"
#include "rmsnorm.h"

namespace {

// 160 partial rows x 8192 floats = 5 MiB per GPU, held from library load to exit.
constexpr size_t kStaticScratchFloats = static_cast<size_t>(PG_STATIC_SCRATCH_BYTES) / sizeof(float);

static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];

std::mutex g_setup_mutex;
float *g_scratch_ptr[64] = {};

// Device address of g_static_scratch on the current device; looked up on first use.
cudaError_t scratch_address(float **out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_ptr[dev] == nullptr) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return e;
        g_scratch_ptr[dev] = static_cast<float *>(p);
    }
    *out = g_scratch_ptr[dev];
    return cudaSuccess;
}

}  // namespace

extern "C" int pg_rmsnorm_bwd_static(void *dx, float *dgamma, const void *dy, const void *x, const float *gamma,
                                     int64_t rows, int64_t h, float eps, int dtype, void *stream) {
    if (rows < 0 || h <= 0) return PG_ERR_BAD_ARG;
    if (dtype != PG_F16 && dtype != PG_BF16) return PG_ERR_BAD_ARG;
    if (h % 8 != 0) return PG_ERR_UNSUPPORTED;
    // how many partial rows would this shape need on this device?
    size_t need_bytes = 0;
    if (rows > 0) {
        need_bytes = pg_rmsnorm_bwd_workspace_bytes(rows, h);
        if (need_bytes == 0) return PG_ERR_UNSUPPORTED;            // h beyond what the kernels support
        if (need_bytes > PG_STATIC_SCRATCH_BYTES) return PG_ERR_STATIC_SCRATCH;
    }
    float *scratch = nullptr;
    const cudaError_t e = scratch_address(&scratch);
    if (e != cudaSuccess) return pg::record_cuda_failure(e);      // pg_last_cuda_error() then names the failed call
    // Same kernels, same order of operations as pg_rmsnorm_bwd: the results are bit-identical.
    return pg_rmsnorm_bwd(dx, dgamma, dy, x, gamma, rows, h, eps, dtype, scratch, PG_STATIC_SCRATCH_BYTES, stream);
}
