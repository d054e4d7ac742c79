// rstd[r] = rsqrt(mean_j(x[r,j]^2) + eps) for every row of a 16-bit matrix: the only part of RMSNorm
// that a following GEMM cannot absorb.  With gamma folded into the weights once
// (W'[n,k] = W[n,k] * gamma[k]), RMSNorm followed by a projection is
//     out[i,n] = rstd[i] * sum_k x[i,k] W'[n,k]
// so the GEMM reads x itself and applies rstd as a per-row scale in its epilogue; the normalised
// activations are never written or re-read.  No counterpart in the reference project (no RMSNorm).
//
// One warp per row, 16-byte loads, fp32 sum of squares, same rstd formula as the forward kernel
// (rsqrtf(fmaf(sum, 1/h, eps))).  HBM-bound: reads rows * h * 2 bytes, writes rows * 4.
// The kernel releases its dependents at once (griddepcontrol.launch_dependents), so a GEMM launched
// behind it with programmatic stream serialisation runs its main loop concurrently and only its
// epilogue waits for these results.

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"
#include "host_util.h"
#include "rmsnorm.h"

namespace pg {

namespace {

constexpr int kWarpsPerCta = 8;

template <bool BF16>
__device__ __forceinline__ float sumsq8(const uint4 &w) {
    float a, b, s = 0.f;
    ptx::unpack2<BF16>(w.x, a, b); s = fmaf(a, a, s); s = fmaf(b, b, s);
    ptx::unpack2<BF16>(w.y, a, b); s = fmaf(a, a, s); s = fmaf(b, b, s);
    ptx::unpack2<BF16>(w.z, a, b); s = fmaf(a, a, s); s = fmaf(b, b, s);
    ptx::unpack2<BF16>(w.w, a, b); s = fmaf(a, a, s); s = fmaf(b, b, s);
    return s;
}

template <bool BF16>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
rmsnorm_rstd_kernel(float *__restrict__ rstd, const uint4 *__restrict__ x, int64_t rows, uint32_t vecs_per_row,
                    float inv_h, float eps) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint32_t lane = threadIdx.x & 31u;
    const int64_t warp0 = static_cast<int64_t>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kWarpsPerCta;
    for (int64_t r = warp0; r < rows; r += stride) {
        const uint4 *row = x + r * vecs_per_row;
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
        uint32_t i = lane;
        for (; i + 96u < vecs_per_row; i += 128u) {       // four independent 16-byte loads in flight per lane
            const uint4 w0 = __ldcs(row + i), w1 = __ldcs(row + i + 32u), w2 = __ldcs(row + i + 64u),
                        w3 = __ldcs(row + i + 96u);
            s0 += sumsq8<BF16>(w0);
            s1 += sumsq8<BF16>(w1);
            s2 += sumsq8<BF16>(w2);
            s3 += sumsq8<BF16>(w3);
        }
        for (; i < vecs_per_row; i += 32u) s0 += sumsq8<BF16>(__ldcs(row + i));
        float s = (s0 + s1) + (s2 + s3);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) rstd[r] = rsqrtf(fmaf(s, inv_h, eps));
    }
}

}  // namespace

cudaError_t rmsnorm_rstd_launch(float *rstd, const void *x, int64_t rows, int64_t h, float eps, bool bf16,
                                cudaStream_t stream) {
    int sms = 0;
    const cudaError_t e = current_device_sm_count(&sms);
    if (e != cudaSuccess) return e;
    const int64_t want = (rows + kWarpsPerCta - 1) / kWarpsPerCta;
    const int64_t cap = static_cast<int64_t>(sms) * 8;      // 64 warps per SM
    const unsigned grid = static_cast<unsigned>(want < cap ? want : cap);
    const uint32_t vecs = static_cast<uint32_t>(h / 8);
    const float inv_h = 1.0f / static_cast<float>(h);
    if (bf16)
        rmsnorm_rstd_kernel<true><<<grid, kWarpsPerCta * 32, 0, stream>>>(rstd, static_cast<const uint4 *>(x), rows,
                                                                         vecs, inv_h, eps);
    else
        rmsnorm_rstd_kernel<false><<<grid, kWarpsPerCta * 32, 0, stream>>>(rstd, static_cast<const uint4 *>(x), rows,
                                                                          vecs, inv_h, eps);
    return cudaGetLastError();
}

}  // namespace pg
