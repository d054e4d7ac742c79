// RMSNorm forward / backward for B200: memory-bound row kernels.
//
// The reference project has no RMSNorm; its only related material is the unused
// warp_reduce / block_reduce / vec_t helpers in src/common/kernel_utils.h:28-98.
// These kernels are new and follow the conventions of the GEMM entry point
// (outputs first, caller-allocated, asynchronous on the caller's stream).
//
// Data layout: x, y, dy, dx are dense row-major [rows, h] 16-bit (bf16 or fp16),
// gamma and dgamma are [h] fp32.  Every global access to the 16-bit tensors is a
// 128-bit vector of 8 elements, consecutive threads touch consecutive vectors.
//
// Forward: one warp per row.  The row is held in registers between the
// sum-of-squares pass and the scaling pass, so x is read from HBM exactly once.
// Algorithmic traffic: 4*rows*h + 4*h bytes.
//
// Backward: one CTA per batch of kRB rows; each thread owns kVPT column vectors
// for the CTA's whole lifetime, so its share of dgamma stays in registers while
// the CTA walks its rows.  Both row reductions (sum x^2 and sum dy*gamma*x) are
// done in one pass over registers.  Each CTA finally writes one fp32 partial row;
// a second kernel sums the partial rows in a fixed order (deterministic).
// Algorithmic traffic: 6*rows*h + 8*h bytes; the partials add 8*h*n_cta bytes.

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "host_util.h"
#include "rmsnorm.h"

namespace pg {
namespace {

template <bool BF16>
__device__ __forceinline__ void unpack8(const uint4 &v, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if constexpr (BF16) {
            // bf16 -> fp32 is a 16-bit shift
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        } else {
            const __half2 h = *reinterpret_cast<const __half2 *>(&w[i]);
            const float2 t = __half22float2(h);
            f[2 * i] = t.x;
            f[2 * i + 1] = t.y;
        }
    }
}

template <bool BF16>
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if constexpr (BF16) {
            const __nv_bfloat162 t = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t *>(&t);
        } else {
            const __half2 t = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t *>(&t);
        }
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ void load_gamma8(const float *gamma, int vec_idx, float (&g)[8]) {
    const float4 a = __ldg(reinterpret_cast<const float4 *>(gamma) + 2 * vec_idx);
    const float4 b = __ldg(reinterpret_cast<const float4 *>(gamma) + 2 * vec_idx + 1);
    g[0] = a.x; g[1] = a.y; g[2] = a.z; g[3] = a.w;
    g[4] = b.x; g[5] = b.y; g[6] = b.z; g[7] = b.w;
}

// ---------------------------------------------------------------- forward ----

constexpr int kFwdWarps = 8;

// One warp per row; lane l holds vectors l, l+32, ... (NVEC of them).
template <int NVEC, bool BF16>
__global__ void __launch_bounds__(kFwdWarps * 32)
rmsnorm_fwd_warp_kernel(uint4 *__restrict__ y, const uint4 *__restrict__ x,
                        const float *__restrict__ gamma, int64_t rows, int h8, float h_f, float eps) {
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = static_cast<int64_t>(blockIdx.x) * kFwdWarps + (threadIdx.x >> 5);
    const int64_t nwarps = static_cast<int64_t>(gridDim.x) * kFwdWarps;
    for (int64_t row = warp0; row < rows; row += nwarps) {
        const uint4 *xr = x + row * h8;
        uint4 v[NVEC];
#pragma unroll
        for (int i = 0; i < NVEC; ++i) {
            const int idx = lane + 32 * i;
            v[i] = (idx < h8) ? __ldcs(xr + idx) : make_uint4(0, 0, 0, 0);
        }
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < NVEC; ++i) {
            float f[8];
            unpack8<BF16>(v[i], f);
#pragma unroll
            for (int e = 0; e < 8; ++e) ss = fmaf(f[e], f[e], ss);
        }
        ss = warp_sum(ss);
        const float rstd = 1.0f / sqrtf(ss / h_f + eps);
        uint4 *yr = y + row * h8;
#pragma unroll
        for (int i = 0; i < NVEC; ++i) {
            const int idx = lane + 32 * i;
            if (idx < h8) {
                float f[8], g[8];
                unpack8<BF16>(v[i], f);
                load_gamma8(gamma, idx, g);
#pragma unroll
                for (int e = 0; e < 8; ++e) f[e] = (f[e] * rstd) * g[e];
                __stcs(yr + idx, pack8<BF16>(f));
            }
        }
    }
}

// Any h (multiple of 8): one CTA per row, x is read twice (the second read hits L2).
template <bool BF16>
__global__ void __launch_bounds__(256)
rmsnorm_fwd_generic_kernel(uint4 *__restrict__ y, const uint4 *__restrict__ x,
                           const float *__restrict__ gamma, int64_t rows, int h8, float h_f, float eps) {
    __shared__ float red[8];
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const uint4 *xr = x + row * h8;
        float ss = 0.f;
        for (int idx = threadIdx.x; idx < h8; idx += 256) {
            float f[8];
            unpack8<BF16>(__ldg(xr + idx), f);
#pragma unroll
            for (int e = 0; e < 8; ++e) ss = fmaf(f[e], f[e], ss);
        }
        ss = warp_sum(ss);
        __syncthreads();   // red[] of the previous row has been consumed
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) tot += red[w];
        const float rstd = 1.0f / sqrtf(tot / h_f + eps);
        uint4 *yr = y + row * h8;
        for (int idx = threadIdx.x; idx < h8; idx += 256) {
            float f[8], g[8];
            unpack8<BF16>(__ldg(xr + idx), f);
            load_gamma8(gamma, idx, g);
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = (f[e] * rstd) * g[e];
            __stcs(yr + idx, pack8<BF16>(f));
        }
    }
}

// --------------------------------------------------------------- backward ----

// THREADS threads own THREADS*VPT column vectors (>= h8); RB rows per batch.
template <int THREADS, int VPT, int RB, bool BF16>
__global__ void __launch_bounds__(THREADS, (THREADS >= 512 ? 1 : 512 / THREADS))
rmsnorm_bwd_kernel(uint4 *__restrict__ dx, float *__restrict__ partial, const uint4 *__restrict__ dy,
                   const uint4 *__restrict__ x, const float *__restrict__ gamma, int64_t rows, int h8,
                   float h_f, float eps) {
    constexpr int kWarps = THREADS / 32;
    __shared__ float red[2][kWarps][2 * RB];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    float gam[VPT][8], acc[VPT][8];
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int idx = threadIdx.x + THREADS * j;
        if (idx < h8) load_gamma8(gamma, idx, gam[j]);
        else {
#pragma unroll
            for (int e = 0; e < 8; ++e) gam[j][e] = 0.f;
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[j][e] = 0.f;
    }

    int it = 0;
    for (int64_t row0 = static_cast<int64_t>(blockIdx.x) * RB; row0 < rows;
         row0 += static_cast<int64_t>(gridDim.x) * RB, it ^= 1) {
        uint4 xv[RB][VPT], dv[RB][VPT];
#pragma unroll
        for (int r = 0; r < RB; ++r) {
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                const int idx = threadIdx.x + THREADS * j;
                const bool in = (row0 + r < rows) && (idx < h8);
                xv[r][j] = in ? __ldcs(x + (row0 + r) * h8 + idx) : make_uint4(0, 0, 0, 0);
                dv[r][j] = in ? __ldcs(dy + (row0 + r) * h8 + idx) : make_uint4(0, 0, 0, 0);
            }
        }
        float s[2 * RB];
#pragma unroll
        for (int r = 0; r < RB; ++r) {
            float s1 = 0.f, s2 = 0.f;
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                float xf[8], df[8];
                unpack8<BF16>(xv[r][j], xf);
                unpack8<BF16>(dv[r][j], df);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    s1 = fmaf(xf[e], xf[e], s1);
                    s2 = fmaf(df[e] * gam[j][e], xf[e], s2);
                }
            }
            s[2 * r] = warp_sum(s1);
            s[2 * r + 1] = warp_sum(s2);
        }
        if (lane == 0) {
#pragma unroll
            for (int i = 0; i < 2 * RB; ++i) red[it][warp][i] = s[i];
        }
        // One barrier per batch: red[] is double-buffered, and a thread can only
        // overwrite buffer `it` two batches later, after every thread has passed
        // the barrier of the batch in between.
        __syncthreads();
#pragma unroll
        for (int r = 0; r < RB; ++r) {
            float S1 = 0.f, S2 = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                S1 += red[it][w][2 * r];
                S2 += red[it][w][2 * r + 1];
            }
            const float rstd = 1.0f / sqrtf(S1 / h_f + eps);
            const float cm = (S2 * rstd) / h_f;          // mean_j(g * xhat)
            if (row0 + r < rows) {
#pragma unroll
                for (int j = 0; j < VPT; ++j) {
                    const int idx = threadIdx.x + THREADS * j;
                    if (idx < h8) {
                        float xf[8], df[8], o[8];
                        unpack8<BF16>(xv[r][j], xf);
                        unpack8<BF16>(dv[r][j], df);
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const float xhat = xf[e] * rstd;
                            o[e] = rstd * (df[e] * gam[j][e] - xhat * cm);
                            acc[j][e] = fmaf(df[e], xhat, acc[j][e]);
                        }
                        __stcs(dx + (row0 + r) * h8 + idx, pack8<BF16>(o));
                    }
                }
            }
        }
    }
    float *prow = partial + static_cast<int64_t>(blockIdx.x) * h8 * 8;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int idx = threadIdx.x + THREADS * j;
        if (idx < h8) {
            float4 *p = reinterpret_cast<float4 *>(prow) + 2 * idx;
            p[0] = make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
            p[1] = make_float4(acc[j][4], acc[j][5], acc[j][6], acc[j][7]);
        }
    }
}

// dgamma[c] = sum_p partial[p][c], p in a fixed order.  Block = 32 float4 columns
// x 32 slices of the partial rows; slices are combined by a shared-memory tree.
__global__ void __launch_bounds__(1024)
rmsnorm_dgamma_reduce_kernel(float *__restrict__ dgamma, const float *partial, int nparts, int h4) {
    __shared__ float4 red[32][33];
    // Launched with programmatic stream serialization: this grid may be scheduled while the backward kernel
    // is still draining; nothing of its output is touched before the dependency has fully completed; and it lets
    // its own successor in the stream be launched at once (that kernel orders itself the same way).  `partial`
    // is written by that kernel AFTER this grid may have started, so it is not read-only for this grid's
    // lifetime: plain L2 loads (ld.global.cg), never the read-only path.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int cx = threadIdx.x & 31, sl = threadIdx.x >> 5;
    const int col = blockIdx.x * 32 + cx;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    if (col < h4) {
        for (int p = sl; p < nparts; p += 32) {
            const float4 v = __ldcg(reinterpret_cast<const float4 *>(partial) + static_cast<int64_t>(p) * h4 + col);
            a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
        }
    }
    red[sl][cx] = a;
    __syncthreads();
    for (int s = 16; s > 0; s >>= 1) {
        if (sl < s) {
            const float4 o = red[sl + s][cx];
            float4 m = red[sl][cx];
            m.x += o.x; m.y += o.y; m.z += o.z; m.w += o.w;
            red[sl][cx] = m;
        }
        __syncthreads();
    }
    if (sl == 0 && col < h4) reinterpret_cast<float4 *>(dgamma)[col] = red[0][cx];
}

struct BwdPlan {
    int threads;   // 0: unsupported
    int vpt;
    int rb;
};

BwdPlan bwd_plan(int64_t h) {
    const int64_t h8 = h / 8;
    if (h8 <= 64 * 2) return {64, 2, 2};
    if (h8 <= 128 * 2) return {128, 2, 2};
    if (h8 <= 256 * 2) return {256, 2, 2};
    if (h8 <= 512 * 2) return {512, 2, 2};
    if (h8 <= 1024 * 2) return {1024, 2, 1};
    if (h8 <= 1024 * 8) return {1024, 8, 1};
    return {0, 0, 0};
}

template <int THREADS, int VPT, int RB>
cudaError_t bwd_grid(bool bf16, int sm_count, int *ctas_per_sm) {
    int n = 0;
    cudaError_t e = bf16 ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(
                               &n, rmsnorm_bwd_kernel<THREADS, VPT, RB, true>, THREADS, 0)
                         : cudaOccupancyMaxActiveBlocksPerMultiprocessor(
                               &n, rmsnorm_bwd_kernel<THREADS, VPT, RB, false>, THREADS, 0);
    (void)sm_count;
    *ctas_per_sm = n < 1 ? 1 : n;
    return e;
}

template <int THREADS, int VPT, int RB>
cudaError_t bwd_launch(const RmsBwdArgs &a, int grid, cudaStream_t stream) {
    const int h8 = static_cast<int>(a.h / 8);
    if (a.bf16)
        rmsnorm_bwd_kernel<THREADS, VPT, RB, true><<<grid, THREADS, 0, stream>>>(
            static_cast<uint4 *>(a.dx), static_cast<float *>(a.workspace), static_cast<const uint4 *>(a.dy),
            static_cast<const uint4 *>(a.x), a.gamma, a.rows, h8, static_cast<float>(a.h), a.eps);
    else
        rmsnorm_bwd_kernel<THREADS, VPT, RB, false><<<grid, THREADS, 0, stream>>>(
            static_cast<uint4 *>(a.dx), static_cast<float *>(a.workspace), static_cast<const uint4 *>(a.dy),
            static_cast<const uint4 *>(a.x), a.gamma, a.rows, h8, static_cast<float>(a.h), a.eps);
    return cudaGetLastError();
}

#define PG_BWD_DISPATCH(plan, FN, ...)                                              \
    ((plan).threads == 64     ? FN<64, 2, 2>(__VA_ARGS__)                           \
     : (plan).threads == 128  ? FN<128, 2, 2>(__VA_ARGS__)                          \
     : (plan).threads == 256  ? FN<256, 2, 2>(__VA_ARGS__)                          \
     : (plan).threads == 512  ? FN<512, 2, 2>(__VA_ARGS__)                          \
     : (plan).vpt == 2        ? FN<1024, 2, 1>(__VA_ARGS__)                         \
                              : FN<1024, 8, 1>(__VA_ARGS__))

cudaError_t sm_count(int *out) { return current_device_sm_count(out); }

}  // namespace

int64_t rmsnorm_max_h() { return 1024 * 8 * 8; }

// Number of CTAs (= partial rows) the backward kernel uses for this shape.
cudaError_t rmsnorm_bwd_ctas(int64_t rows, int64_t h, bool bf16, int *ctas) {
    if (rmsnorm_staged_supported(h, true)) {
        int grid = 0;
        return rmsnorm_staged_ctas(rows, h, true, &grid, ctas);
    }
    const BwdPlan p = bwd_plan(h);
    if (p.threads == 0) { *ctas = 0; return cudaSuccess; }
    int sms = 0;
    cudaError_t e = sm_count(&sms);
    if (e != cudaSuccess) return e;
    int per_sm = 1;
    e = PG_BWD_DISPATCH(p, bwd_grid, bf16, sms, &per_sm);
    if (e != cudaSuccess) return e;
    int64_t g = static_cast<int64_t>(sms) * per_sm;
    const int64_t batches = (rows + p.rb - 1) / p.rb;
    if (g > batches) g = batches;
    if (g < 1) g = 1;
    *ctas = static_cast<int>(g);
    return cudaSuccess;
}

cudaError_t rmsnorm_fwd_launch(const RmsFwdArgs &a, cudaStream_t stream) {
    if (rmsnorm_staged_supported(a.h, false)) return rmsnorm_staged_fwd(a, stream);
    const int h8 = static_cast<int>(a.h / 8);
    const float h_f = static_cast<float>(a.h);
    int sms = 0;
    cudaError_t e = sm_count(&sms);
    if (e != cudaSuccess) return e;
    uint4 *y = static_cast<uint4 *>(a.y);
    const uint4 *x = static_cast<const uint4 *>(a.x);
    if (h8 <= 32 * 32) {
        int64_t grid = (a.rows + kFwdWarps - 1) / kFwdWarps;
        const int64_t cap = static_cast<int64_t>(sms) * 64;
        if (grid > cap) grid = cap;
        const int nvec = (h8 + 31) / 32;
#define PG_FWD(NV)                                                                                     \
    do {                                                                                               \
        if (a.bf16)                                                                                    \
            rmsnorm_fwd_warp_kernel<NV, true><<<static_cast<unsigned>(grid), kFwdWarps * 32, 0, stream>>>( \
                y, x, a.gamma, a.rows, h8, h_f, a.eps);                                                \
        else                                                                                           \
            rmsnorm_fwd_warp_kernel<NV, false><<<static_cast<unsigned>(grid), kFwdWarps * 32, 0, stream>>>( \
                y, x, a.gamma, a.rows, h8, h_f, a.eps);                                                \
    } while (0)
        if (nvec <= 1) PG_FWD(1);
        else if (nvec <= 2) PG_FWD(2);
        else if (nvec <= 4) PG_FWD(4);
        else if (nvec <= 8) PG_FWD(8);
        else if (nvec <= 16) PG_FWD(16);
        else PG_FWD(32);
#undef PG_FWD
    } else {
        int64_t grid = a.rows;
        const int64_t cap = static_cast<int64_t>(sms) * 8;
        if (grid > cap) grid = cap;
        if (a.bf16)
            rmsnorm_fwd_generic_kernel<true><<<static_cast<unsigned>(grid), 256, 0, stream>>>(
                y, x, a.gamma, a.rows, h8, h_f, a.eps);
        else
            rmsnorm_fwd_generic_kernel<false><<<static_cast<unsigned>(grid), 256, 0, stream>>>(
                y, x, a.gamma, a.rows, h8, h_f, a.eps);
    }
    return cudaGetLastError();
}

cudaError_t rmsnorm_bwd_launch(const RmsBwdArgs &a, int ctas, cudaStream_t stream) {
    cudaError_t e;
    if (rmsnorm_staged_supported(a.h, true)) {
        if (ctas < 1) return cudaErrorInvalidValue;
        e = rmsnorm_staged_bwd(a, stream);
    } else {
        const BwdPlan p = bwd_plan(a.h);
        if (p.threads == 0 || ctas < 1) return cudaErrorInvalidValue;
        e = PG_BWD_DISPATCH(p, bwd_launch, a, ctas, stream);
    }
    if (e != cudaSuccess) return e;
    const int h4 = static_cast<int>(a.h / 4);
    // Programmatic dependent launch: the reduction's launch latency (~3 us of a ~140 us step) overlaps the
    // tail of the backward kernel; griddepcontrol.wait inside it orders the data.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>((h4 + 31) / 32), 1, 1);
    cfg.blockDim = dim3(1024, 1, 1);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, rmsnorm_dgamma_reduce_kernel, a.dgamma,
                              static_cast<const float *>(a.workspace), ctas, h4);
}

}  // namespace pg
