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
};

enum LaunchResult { kLaunchOk = 0, kLaunchCuda = 1, kLaunchNotSm100 = 2, kLaunchBadConfig = 3 };

// variant: 0 auto, 1 = one CTA per tile, 2 = CTA pair per tile; block_n: 0 auto, 64, 128, 256.
// max_sms: 0 = all SMs, else an upper bound on the SMs the persistent grid occupies.
int hgemm_launch(const GemmArgs &g, int variant, int block_n, int max_sms, cudaStream_t stream,
                 cudaError_t *cuda_err);

// Resolves variant/block_n == 0 to concrete values for a device with sm_count SMs.
void choose_config(const GemmArgs &g, int sm_count, int *variant, int *block_n);

// Synchronises the stream, returns and clears the kernels' device status word.
int gemm_device_status(int *out, cudaStream_t stream, cudaError_t *cuda_err);

}  // namespace pg
