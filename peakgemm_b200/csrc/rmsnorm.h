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

// CTAs (= fp32 partial rows of dgamma) the backward kernel uses for this shape on the current device.
cudaError_t rmsnorm_bwd_ctas(int64_t rows, int64_t h, bool bf16, int *ctas);

cudaError_t rmsnorm_fwd_launch(const RmsFwdArgs &a, cudaStream_t stream);
cudaError_t rmsnorm_bwd_launch(const RmsBwdArgs &a, int ctas, cudaStream_t stream);

}  // namespace pg
