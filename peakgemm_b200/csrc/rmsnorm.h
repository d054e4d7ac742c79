// Internal interface between the C ABI (api.cu) and the RMSNorm kernels (rmsnorm.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace pg {

struct RmsFwdArgs {
    void *y;
    const void *x;
    const float *gamma;
    int64_t rows, h;
    float eps;
    bool bf16;
};

struct RmsBwdArgs {
    void *dx;
    float *dgamma;
    const void *dy;
    const void *x;
    const float *gamma;
    int64_t rows, h;
    float eps;
    bool bf16;
    void *workspace;   // [ctas, h] fp32
};

// Largest h the backward kernel supports.
int64_t rmsnorm_max_h();

// fp32 partial rows of dgamma the backward kernel writes for this shape on the current device.
cudaError_t rmsnorm_bwd_ctas(int64_t rows, int64_t h, bool bf16, int *ctas);

cudaError_t rmsnorm_fwd_launch(const RmsFwdArgs &a, cudaStream_t stream);
cudaError_t rmsnorm_bwd_launch(const RmsBwdArgs &a, int ctas, cudaStream_t stream);

// rstd[r] = rsqrt(mean(x[r,:]^2) + eps), fp32 (rmsnorm_rstd.cu).
cudaError_t rmsnorm_rstd_launch(float *rstd, const void *x, int64_t rows, int64_t h, float eps, bool bf16,
                                cudaStream_t stream);

// Bulk-copy staged variants (rmsnorm_staged.cu), used for 2048 <= h <= 16384.
bool rmsnorm_staged_supported(int64_t h, bool bwd);
cudaError_t rmsnorm_staged_ctas(int64_t rows, int64_t h, bool bwd, int *ctas, int *partial_rows);
cudaError_t rmsnorm_staged_fwd(const RmsFwdArgs &a, cudaStream_t stream);
cudaError_t rmsnorm_staged_bwd(const RmsBwdArgs &a, cudaStream_t stream);   // writes the partial rows only
// Synchronises the stream, returns and clears the staged kernels' device status word.
cudaError_t rmsnorm_device_status(int *out, cudaStream_t stream);

}  // namespace pg
