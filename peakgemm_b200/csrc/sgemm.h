// Internal interface between the C ABI (api.cu) and the fp32 GEMM kernel (sgemm.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace pg {
cudaError_t sgemm_launch(float *c, const float *a, const float *b, int64_t m, int64_t n, int64_t k, int64_t lda,
                         int64_t ldb, int64_t ldc, cudaStream_t stream);
}
