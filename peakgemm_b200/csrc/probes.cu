// Roofline probes: what the machine can do with nothing in the way.
//
// Counterparts of the reference's stand-alone probes
//   test/cpp/test_wmma_compute.cpp:142-173   MMA issue-rate loop (the README's "PEAK" column, README.md:8-11)
//   test/cpp/test_memory_bandwidth.cpp:95-114 vectorised copy GB/s
// for sm_100a: a CTA pair issues tcgen05.mma.cta_group::2 (256 x 256 x 16, the headline kernel's
// instruction) back to back on operand tiles that already sit in shared memory, with no loads in the
// loop; and a 128-bit streaming copy.  The tensor probe shows what the power cap and the MMA pipe allow
// when TMA, barriers and the epilogue cost nothing; the GEMM kernel is judged against it.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/peakgemm.h"
#include "ptx.cuh"

namespace {

using namespace pg::ptx;

constexpr uint32_t kTileBytes = 128 * 64 * 2;   // one 128-row x 64-k operand tile, 128-byte rows

// grid = SM count (even), cluster of 2, 128 threads.  Each pair: `iters` rounds of 4 MMAs (k = 64).
template <bool BF16>
__global__ void __launch_bounds__(128, 1)
probe_mma_kernel(uint32_t iters, uint32_t seed, int *status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar = smem_base + 2 * kTileBytes;
    const uint32_t slot = bar + 8;
    volatile uint32_t *slot_gen = reinterpret_cast<volatile uint32_t *>(smem_gen + 2 * kTileBytes + 8);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const bool leader = cluster_ctarank() == 0;

    // operand tiles with pseudo-random 16-bit patterns of moderate magnitude (random data toggles the
    // datapath as real inputs do; zeros would flatter the power-limited clock)
    uint32_t x = seed * 2654435761u + blockIdx.x * 97u + threadIdx.x;
    for (uint32_t i = threadIdx.x; i < 2 * kTileBytes / 4; i += blockDim.x) {
        x = x * 1664525u + 1013904223u;
        const uint32_t lo = BF16 ? (0x3f00u | ((x >> 8) & 0xffu) | ((x >> 3) & 0x8000u))
                                 : (0x3800u | ((x >> 8) & 0x3ffu) | ((x >> 3) & 0x8000u));
        const uint32_t hi = BF16 ? (0x3f00u | ((x >> 20) & 0xffu) | ((x >> 1) & 0x8000u))
                                 : (0x3800u | ((x >> 18) & 0x3ffu) | ((x >> 1) & 0x8000u));
        reinterpret_cast<uint32_t *>(smem_gen)[i] = lo | (hi << 16);
    }
    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        fence_mbar_init();
    }
    fence_proxy_async_smem();
    if (warp == 0) {
        tmem_alloc<2>(slot, 256);
        tmem_relinquish<2>();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_arrive();
    cluster_wait();
    tc_fence_after_sync();
    const uint32_t tmem = *slot_gen;

    if (warp == 0 && lane == 0 && leader) {
        const uint32_t idesc = instr_desc_f16(BF16, 256, 256);
        const uint64_t da = smem_desc_k_sw128(smem_base);
        const uint64_t db = smem_desc_k_sw128(smem_base + kTileBytes);
        for (uint32_t it = 0; it < iters; ++it) {
#pragma unroll
            for (uint32_t k = 0; k < 4; ++k) umma_f16<2>(tmem, da + 2 * k, db + 2 * k, idesc, (it | k) ? 1u : 0u);
        }
        umma_commit<2>(bar);
        // bounded wait for the whole chain (iters * 4 * 128 cycles)
        uint64_t t0 = globaltimer_ns();
        uint32_t spins = 0;
        while (!mbar_try_wait(bar, 0)) {
            if ((++spins & 1023u) == 0 && globaltimer_ns() - t0 > 4000000000ull) {
                atomicCAS(status, 0, 21);
                break;
            }
        }
    }
    __syncwarp();
    tc_fence_before_sync();
    __syncthreads();
    cluster_arrive();
    cluster_wait();
    if (warp == 0) {
        tc_fence_after_sync();
        tmem_dealloc<2>(tmem, 256);
    }
}

// One CTA per 16 KiB chunk: thread t moves the 16-byte vectors t, t + 256, t + 512, t + 768 of its chunk.
__global__ void __launch_bounds__(256)
probe_copy_kernel(uint4 *__restrict__ dst, const uint4 *__restrict__ src, int64_t n16) {
    const int64_t base = static_cast<int64_t>(blockIdx.x) * 1024 + threadIdx.x;
    uint4 v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
        if (base + 256 * j < n16) v[j] = __ldcs(src + base + 256 * j);
#pragma unroll
    for (int j = 0; j < 4; ++j)
        if (base + 256 * j < n16) __stcs(dst + base + 256 * j, v[j]);
}

__device__ int g_probe_status;

}  // namespace

extern "C" {

// Tensor-core probe: runs `iters` k = 64 rounds of 256 x 256 pair MMAs on every SM pair and writes the
// TFLOP/s reached (2 * 256 * 256 * 64 flop per round and pair).  Synchronises; allocates nothing.
int pg_probe_tensor_peak(int dtype, int iters, float *tflops_out, float *ms_out) {
    // The kernel's one wait (for its whole MMA chain) is bounded at 4 s; 2^20 rounds take about 0.4 s, so a run
    // within the cap can never outlast the wait and tear down tensor memory under MMAs still in flight.
    if ((dtype != PG_F16 && dtype != PG_BF16) || iters < 1 || iters > PG_PROBE_MAX_ITERS || !tflops_out)
        return PG_ERR_BAD_ARG;
    int dev = 0, sms = 0, cc = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return PG_ERR_CUDA;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&cc, cudaDevAttrComputeCapabilityMajor, dev);
    if (cc != 10) return PG_ERR_NOT_SM100;
    void *status = nullptr;
    if (cudaGetSymbolAddress(&status, g_probe_status) != cudaSuccess) return PG_ERR_CUDA;
    cudaMemset(status, 0, sizeof(int));
    const int grid = sms / 2 * 2;
    const size_t smem = 2 * kTileBytes + 64 + 1024;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(128, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    auto launch = [&](uint32_t n) {
        return dtype == PG_BF16 ? cudaLaunchKernelEx(&cfg, probe_mma_kernel<true>, n, 7u, static_cast<int *>(status))
                                : cudaLaunchKernelEx(&cfg, probe_mma_kernel<false>, n, 7u, static_cast<int *>(status));
    };
    cudaError_t e = launch(64);   // warm-up
    if (e == cudaSuccess) {
        cudaEventRecord(e0);
        e = launch(static_cast<uint32_t>(iters));
        cudaEventRecord(e1);
    }
    if (e == cudaSuccess) e = cudaEventSynchronize(e1);
    float ms = 0.f;
    if (e == cudaSuccess) cudaEventElapsedTime(&ms, e0, e1);
    int st = 0;
    cudaMemcpy(&st, status, sizeof(int), cudaMemcpyDeviceToHost);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return PG_ERR_CUDA;
    }
    if (st != 0) return PG_ERR_DEVICE_TIMEOUT;
    const double flop = 2.0 * 256 * 256 * 64 * static_cast<double>(iters) * (grid / 2);
    *tflops_out = static_cast<float>(flop / (ms * 1e-3) / 1e12);
    if (ms_out) *ms_out = ms;
    return PG_OK;
}

// Streaming copy of `bytes` (a multiple of 16) from src to dst on `stream`; asynchronous.
int pg_probe_copy(void *dst, const void *src, size_t bytes, void *stream) {
    if (!dst || !src || bytes % 16 != 0) return PG_ERR_BAD_ARG;
    if (bytes == 0) return PG_OK;
    const int64_t n16 = static_cast<int64_t>(bytes / 16);
    const int64_t ctas = (n16 + 1023) / 1024;
    if (ctas > 0x7fffffff) return PG_ERR_UNSUPPORTED;
    probe_copy_kernel<<<static_cast<unsigned>(ctas), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<uint4 *>(dst), static_cast<const uint4 *>(src), n16);
    return cudaGetLastError() == cudaSuccess ? PG_OK : PG_ERR_CUDA;
}

}  // extern "C"
