// Internal interface between the C ABI (api.cu) and the GEMM kernels (gemm_sm100.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace pg {

struct GemmArgs {
    void *c;
    const void *a;
    const void *b;
    int64_t m, n, k;
    int64_t lda, ldb, ldc;   // row pitches in elements
    bool bf16;               // false: fp16
    int n_extra_dst = 0;     // further destinations of C (same extents and pitch as c), at most 7
    void *extra_dst[7] = {};
    // Fused epilogue, every term optional (null = absent):
    //   C[i,j] = round(row_scale[i] * sum_k A[i,k] B[j,k] + bias[j] + residual[i,j])
    const float *row_scale = nullptr;   // [m] fp32
    const void *bias = nullptr;         // [n], the matrices' element type
    const void *residual = nullptr;     // [m, n] with row pitch ldr, the matrices' element type; may be c itself
    int64_t ldr = 0;
    bool pdl_wait = false;              // the epilogue waits for the preceding kernel of the stream before it reads
                                        // row_scale (programmatic dependent launch); the main loop does not wait
    void *mc_dst = nullptr;             // non-null: C is written through this multicast address (row pitch ldc) with
                                        // multimem.st instead of TMA stores to c; c must still be a local address
    void *workspace = nullptr;          // optional scratch for the tail split of the 256-wide CTA-pair kernel
    size_t workspace_bytes = 0;
};

enum LaunchResult { kLaunchOk = 0, kLaunchCuda = 1, kLaunchNotSm100 = 2, kLaunchBadConfig = 3 };

// variant: 0 auto, 1 = one CTA per tile, 2 = CTA pair per tile, 3 = cluster split-K, 4 = skinny,
// 5 = CTA pair with two row blocks per CTA (512 x 256 tiles); block_n: 0 auto, 64, 128, 256.
// max_sms: 0 = all SMs, else an upper bound on the SMs the persistent grid occupies.
int hgemm_launch(const GemmArgs &g, int variant, int block_n, int max_sms, cudaStream_t stream,
                 cudaError_t *cuda_err);

// Resolves variant/block_n == 0 to concrete values for a device with sm_count SMs.
void choose_config(const GemmArgs &g, int sm_count, int *variant, int *block_n);

// Workspace (bytes) that lets hgemm_launch split the last, partial wave of this shape over idle SM pairs; 0 if none.
size_t hgemm_workspace_bytes(int64_t m, int64_t n, int64_t k, int sm_count);

// Synchronises the stream, returns and clears the kernels' device status word.
int gemm_device_status(int *out, cudaStream_t stream, cudaError_t *cuda_err);

}  // namespace pg
