// fp32 GEMM  C[m,n] = A[m,k] * B[n,k]^T  for the float branch of the gemm_peak operator.
//
// The reference routes float tensors to sgemm::sgemm_peak (src/ops/gemm.cpp:34-43,
// src/impl/sgemm_impl.h:56-320), a CUDA-core FFMA kernel its README calls an unoptimised
// reference path (README.md:46-47).  This is the same class of kernel, written for this
// library: 128 x 128 x 16 tiles, 256 threads, 8 x 8 outputs per thread as four 4 x 4 blocks,
// operands transposed into shared memory so the inner loop reads float4, register prefetch
// of the next k-block.  True fp32 FMA accumulation (no TF32), so it meets the reference
// test's absolute bound of 1e-4 (test/cpp/test_gemm_float.cpp:151).  It exists to keep the
// operator surface complete; the half-precision kernels are the hot path.
#include <cuda_runtime.h>
#include <stdint.h>

#include "sgemm.h"

namespace pg {
namespace {

constexpr int kBM = 128, kBN = 128, kBK = 16, kPad = 4;

__global__ void __launch_bounds__(256)
sgemm_kernel(float *__restrict__ c, const float *__restrict__ a, const float *__restrict__ b, int m, int n, int k,
             int64_t lda, int64_t ldb, int64_t ldc) {
    __shared__ float As[kBK][kBM + kPad];
    __shared__ float Bs[kBK][kBN + kPad];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;          // 16 x 16 threads
    const int m0 = blockIdx.y * kBM, n0 = blockIdx.x * kBN;

    // global -> register staging: each thread carries two float4 of A and two of B per k-block
    float4 ra[2], rb[2];
    auto load_tiles = [&](int k0) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int idx = tid + 256 * i;
            const int row = idx >> 2, kc = (idx & 3) * 4;
            const bool kin = k0 + kc < k;
            ra[i] = (kin && m0 + row < m) ? *reinterpret_cast<const float4 *>(a + (int64_t)(m0 + row) * lda + k0 + kc)
                                          : make_float4(0.f, 0.f, 0.f, 0.f);
            rb[i] = (kin && n0 + row < n) ? *reinterpret_cast<const float4 *>(b + (int64_t)(n0 + row) * ldb + k0 + kc)
                                          : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    auto store_tiles = [&]() {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int idx = tid + 256 * i;
            const int row = idx >> 2, kc = (idx & 3) * 4;
            As[kc + 0][row] = ra[i].x; As[kc + 1][row] = ra[i].y; As[kc + 2][row] = ra[i].z; As[kc + 3][row] = ra[i].w;
            Bs[kc + 0][row] = rb[i].x; Bs[kc + 1][row] = rb[i].y; Bs[kc + 2][row] = rb[i].z; Bs[kc + 3][row] = rb[i].w;
        }
    };

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

    load_tiles(0);
    store_tiles();
    __syncthreads();
    for (int k0 = 0; k0 < k; k0 += kBK) {
        if (k0 + kBK < k) load_tiles(k0 + kBK);
#pragma unroll
        for (int kk = 0; kk < kBK; ++kk) {
            // rows ty*4 .. +3 and 64 + ty*4 .. +3; columns tx*4 .. +3 and 64 + tx*4 .. +3 (conflict-free float4 reads)
            const float4 a0 = *reinterpret_cast<const float4 *>(&As[kk][ty * 4]);
            const float4 a1 = *reinterpret_cast<const float4 *>(&As[kk][64 + ty * 4]);
            const float4 b0 = *reinterpret_cast<const float4 *>(&Bs[kk][tx * 4]);
            const float4 b1 = *reinterpret_cast<const float4 *>(&Bs[kk][64 + tx * 4]);
            const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
        if (k0 + kBK < k) {
            store_tiles();
            __syncthreads();
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int row = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + i - 4);
        if (row >= m) continue;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int col = n0 + (h == 0 ? tx * 4 : 64 + tx * 4);
            if (col + 3 < n) {
                *reinterpret_cast<float4 *>(c + (int64_t)row * ldc + col) =
                    make_float4(acc[i][4 * h], acc[i][4 * h + 1], acc[i][4 * h + 2], acc[i][4 * h + 3]);
            } else {
                for (int j = 0; j < 4; ++j)
                    if (col + j < n) c[(int64_t)row * ldc + col + j] = acc[i][4 * h + j];
            }
        }
    }
}

__global__ void zero_fill_f32_kernel(float *c, int64_t m, int64_t n, int64_t ldc) {
    const int64_t total = m * n;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x)
        c[(i / n) * ldc + (i % n)] = 0.f;
}

}  // namespace

cudaError_t sgemm_launch(float *c, const float *a, const float *b, int64_t m, int64_t n, int64_t k, int64_t lda,
                         int64_t ldb, int64_t ldc, cudaStream_t stream) {
    if (k == 0) {
        zero_fill_f32_kernel<<<592, 256, 0, stream>>>(c, m, n, ldc);
        return cudaGetLastError();
    }
    dim3 grid(static_cast<unsigned>((n + kBN - 1) / kBN), static_cast<unsigned>((m + kBM - 1) / kBM));
    sgemm_kernel<<<grid, 256, 0, stream>>>(c, a, b, static_cast<int>(m), static_cast<int>(n), static_cast<int>(k),
                                           lda, ldb, ldc);
    return cudaGetLastError();
}

}  // namespace pg
