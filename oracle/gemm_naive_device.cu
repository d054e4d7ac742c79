// TEST INFRASTRUCTURE — not part of the product.  Only tests/ may build, load or
// call this file.
//
// Device restatement of the reference's oracle kernel sgemm::sgemm_naive_kernel<T>
// (src/impl/sgemm_impl.h:9-40): one thread per output, fp32 accumulation over k in
// increasing order, result cast to T.  Used where the CPU oracle would take too
// long (full-size shapes).  64-bit indexing, and a row pitch for C so a
// column-block of a wider matrix can be checked in place.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

template <typename T>
__global__ void naive_kernel(T *c, const T *a, const T *b, int64_t m, int64_t n, int64_t k, int64_t ldc) {
    const int64_t mi = blockIdx.y * 16 + threadIdx.y;
    const int64_t ni = blockIdx.x * 16 + threadIdx.x;
    if (mi < m && ni < n) {
        float acc = 0.f;
        const T *ar = a + mi * k;
        const T *br = b + ni * k;
        for (int64_t ki = 0; ki < k; ++ki) acc += static_cast<float>(ar[ki]) * static_cast<float>(br[ki]);
        c[mi * ldc + ni] = static_cast<T>(acc);
    }
}

extern "C" int oracle_gemm_naive_device(void *c, const void *a, const void *b, int64_t m, int64_t n, int64_t k,
                                        int64_t ldc, int is_bf16, void *stream) {
    if (m <= 0 || n <= 0) return 0;
    dim3 block(16, 16);
    dim3 grid(static_cast<unsigned>((n + 15) / 16), static_cast<unsigned>((m + 15) / 16));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (is_bf16)
        naive_kernel<__nv_bfloat16><<<grid, block, 0, s>>>(static_cast<__nv_bfloat16 *>(c),
                                                            static_cast<const __nv_bfloat16 *>(a),
                                                            static_cast<const __nv_bfloat16 *>(b), m, n, k, ldc);
    else
        naive_kernel<__half><<<grid, block, 0, s>>>(static_cast<__half *>(c), static_cast<const __half *>(a),
                                                    static_cast<const __half *>(b), m, n, k, ldc);
    return static_cast<int>(cudaGetLastError());
}
