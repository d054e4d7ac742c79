// RMSNorm forward / backward, bulk-copy staged variant for 256 <= h <= 16384.
//
// HBM-bound work: what matters is that every SM keeps enough bytes in flight all
// the time and that no latency chain on the compute side is exposed.
//   * One producer thread per CTA streams rows of x (and of dy for the backward
//     pass) into a ring of shared-memory slots with cp.async.bulk (16-byte aligned,
//     completion counted on an mbarrier), up to 16 rows ahead: bytes in flight do
//     not depend on registers or occupancy.
//   * The consumer warps are split into kG independent groups of T threads.  Group
//     g takes every kG-th row of the CTA; a row's chain (shared -> registers,
//     warp-shuffle + cross-warp reduction through ONE named barrier of the group,
//     scaling, 128-bit streaming stores) overlaps with the other groups' chains.
//   * Each thread owns VPT column vectors (8 elements each) for the whole kernel:
//     gamma is read from a shared-memory copy and, in the backward pass, the
//     thread's share of dgamma accumulates in registers.  A slot is released as soon
//     as it has been copied into registers.
// Backward: at the end the groups fold their dgamma shares, in a fixed order, into
// one fp32 partial row per CTA; the fixed-order column reduction kernel in
// rmsnorm.cu sums the CTAs' rows (deterministic).
//
// Every mbarrier wait is bounded (same scheme as the GEMM kernel).

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include "host_util.h"
#include "ptx.cuh"
#include "rmsnorm.h"

namespace pg {

using namespace ptx;

namespace {

// Consumer threads per CTA (G groups x T threads); the producer warp comes on top.  Forward: up to 960 (more rows
// in flight per SM: its per-row chain is latency-bound and needs few registers) — 768 when a thread owns 4 or more
// column vectors, which is all that shape uses (3 groups of 256) and leaves 80 registers per thread, enough to keep
// its gamma values in registers; backward: 512 (its dgamma shares and both operands need ~96 registers per thread).
template <bool BWD, int VPT>
struct Threads {
    // Backward with 8 vectors per thread (h > 8192): 64 dgamma sums, both operands and the output of a row need about
    // 160 registers; at 544 threads the compiler has 96 and spills (3.3-3.6 TB/s).  One group of 256 instead.
    static constexpr int kConsumers = BWD ? (VPT == 8 ? 256 : 512) : (VPT >= 4 ? 768 : 960);   // + 32 <= 1024 threads per CTA
    static constexpr int kTotal = kConsumers + 32;
};
template <bool BWD> struct RowIndex { using type = int64_t; };
template <> struct RowIndex<true> { using type = int; };
constexpr int kMaxStages = 16;
constexpr int kGammaRegsMaxVpt = 4;     // forward: gamma in registers up to this many vectors per thread
#ifdef PG_TEST_SHORT_WAIT
// Test build (libPeakGemm_device_waittest.so, never shipped as the product): waits give up after 2 ms, and a
// switch in device memory makes the first CTA's producer leave out its LAST row (no copy, no arrival), so that the
// consumer group waiting for that row exercises the give-up path with no copy in flight.
constexpr uint64_t kWaitTimeoutNs = 2000000ull;
__device__ int g_test_withhold_last_row;
#else
constexpr uint64_t kWaitTimeoutNs = 2000000000ull;
#endif
constexpr uint32_t kSmemBudget = 200 * 1024;      // bytes of dynamic shared memory we ask for at most

enum : int { kStRmsProducer = 11, kStRmsConsumer = 12 };

__device__ int g_rms_status_word;

struct WaitCtx {
    volatile uint32_t *abort_flag;
    int *status;
};

__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, const WaitCtx &ctx, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    uint64_t t0 = 0;
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 1023u) == 0) {
            if (*ctx.abort_flag) return false;
            const uint64_t now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > kWaitTimeoutNs) {
                *ctx.abort_flag = 1;
                if (ctx.status) atomicCAS(ctx.status, 0, code);
                return false;
            }
        }
    }
}

// 1-D bulk copy global -> shared; both addresses 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void *src, uint32_t bytes, uint32_t bar,
                                          uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
                 "[%0], [%1], %2, [%3], %4;"
                 ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar), "l"(policy)
                 : "memory");
}

// Named barrier `id` over `nthreads` consumer threads that also ORs a predicate across
// them, so that "somebody abandoned a wait" is decided identically by the whole group.
__device__ __forceinline__ bool group_barrier_or(uint32_t id, uint32_t nthreads, bool pred) {
    uint32_t r;
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        "setp.ne.u32 q, %1, 0;\n\t"
        "bar.red.or.pred p, %2, %3, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(r)
        : "r"(static_cast<uint32_t>(pred)), "r"(id), "r"(nthreads)
        : "memory");
    return r != 0;
}

template <bool BF16>
__device__ __forceinline__ void unpack8(const uint4 &v, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if constexpr (BF16) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        } else {
            const float2 t = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
            f[2 * i] = t.x;
            f[2 * i + 1] = t.y;
        }
    }
}

template <bool BF16>
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    return make_uint4(pack2<BF16>(f[0], f[1]), pack2<BF16>(f[2], f[3]), pack2<BF16>(f[4], f[5]),
                      pack2<BF16>(f[6], f[7]));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Shared memory: [gamma: h fp32][slots x (x row [+ dy row])][red][barriers][abort flag]
struct Layout {
    uint32_t off_slot, slot_bytes, row_bytes, off_red, off_bar, total;
};

__host__ __device__ inline Layout make_layout(int h, bool bwd, int stages) {
    Layout l;
    l.off_slot = static_cast<uint32_t>(h) * 4;                       // gamma; a multiple of 32 bytes
    l.row_bytes = static_cast<uint32_t>(h) * 2;
    l.slot_bytes = l.row_bytes * (bwd ? 2 : 1);
    l.off_red = l.off_slot + stages * l.slot_bytes;
    l.off_bar = l.off_red + 2 * 32 * 2 * static_cast<uint32_t>(sizeof(float));   // [2 buffers][32 warps][2]
    l.total = l.off_bar + 2 * stages * 8 + 16;
    return l;
}

// T threads per group (a multiple of 32), G groups, VPT * T >= h / 8.
// INCR: the consumers keep slot / phase / output-row pointer incrementally instead of deriving them from the row
// index with two runtime divisions.  Same results; which form is faster depends on the shape (measured on
// [32768, h] bf16: backward h = 8192 269 -> 250 us with INCR, but forward h = 4096 91 -> 98 us and backward
// h = 4096 136 -> 139 us), so the host picks per shape.
template <bool BWD, int VPT, bool BF16, bool INCR>
__global__ void __launch_bounds__(Threads<BWD, VPT>::kTotal, 1)
rms_staged_kernel(uint4 *__restrict__ out, float *__restrict__ partial, const uint4 *__restrict__ x,
                  const uint4 *__restrict__ dy, const float *__restrict__ gamma, int64_t rows, int h8,
                  float h_f, float eps, int stages, int T, int G, int *status) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int kMaxConsumers = Threads<BWD, VPT>::kConsumers;
    constexpr int kThreads = Threads<BWD, VPT>::kTotal;
    const int h = h8 * 8;
    const Layout L = make_layout(h, BWD, stages);
    const uint32_t sbase = smem_u32(smem);
    const float *s_gamma = reinterpret_cast<const float *>(smem);
    float(*s_red)[32][2] = reinterpret_cast<float(*)[32][2]>(smem + L.off_red);
    const uint32_t bar_full = sbase + L.off_bar;
    const uint32_t bar_empty = bar_full + stages * 8;
    volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(smem + L.off_bar + 2 * stages * 8);
    const WaitCtx ctx{abort_flag, status};

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Launched under programmatic stream serialisation: the next kernel of the stream (the dgamma reduction after a
    // backward pass, or the next call of this library) may be launched at once; it orders itself with
    // griddepcontrol.wait, as this kernel does below before its first access to global memory.  What overlaps is the
    // launch latency and the barrier set-up, about 3 us of an 88-250 us kernel in a back-to-back sequence.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int consumers = T * G;
    const int group_warps = T >> 5;
    // rows of this CTA: blockIdx.x, blockIdx.x + gridDim.x, ...; its i-th row goes to slot i % stages, group i % G
    const int64_t my_rows = rows > blockIdx.x ? (rows - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(bar_full + s * 8, 1);                 // producer's arrive.expect_tx (+ copied bytes)
            mbar_init(bar_empty + s * 8, group_warps);      // one arrive per warp of the consuming group
        }
        *abort_flag = 0;
        fence_mbar_init();
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");      // the preceding kernel has completed (a no-op without one)
    for (int i = threadIdx.x; i < h / 4; i += kThreads)
        reinterpret_cast<float4 *>(smem)[i] = __ldg(reinterpret_cast<const float4 *>(gamma) + i);
    __syncthreads();

    const bool is_consumer = threadIdx.x < consumers;
    const int g = is_consumer ? threadIdx.x / T : 0;   // group (warps of a group are contiguous)
    const int t = threadIdx.x - g * T;                 // thread within the group
    float acc[VPT][8];
#pragma unroll
    for (int j = 0; j < VPT; ++j)
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[j][e] = 0.f;

    if (threadIdx.x >= kMaxConsumers) {
        // ===== producer =====
        if (lane == 0) {
            int slot = 0;
            uint32_t phase = 0;
            const uint64_t pol = l2_policy_evict_first();     // every row is read exactly once
            for (int64_t i = 0; i < my_rows; ++i) {
#ifdef PG_TEST_SHORT_WAIT
                if (blockIdx.x == 0 && i == my_rows - 1 &&
                    *reinterpret_cast<volatile int *>(&g_test_withhold_last_row) != 0)
                    break;
#endif
                if (!wait_bar(bar_empty + slot * 8, phase ^ 1u, ctx, kStRmsProducer)) break;
                const int64_t row = blockIdx.x + i * gridDim.x;
                mbar_arrive_expect_tx(bar_full + slot * 8, L.slot_bytes);
                const uint32_t dst = sbase + L.off_slot + slot * L.slot_bytes;
                bulk_load(dst, x + row * h8, L.row_bytes, bar_full + slot * 8, pol);
                if constexpr (BWD) bulk_load(dst + L.row_bytes, dy + row * h8, L.row_bytes, bar_full + slot * 8, pol);
                if (++slot == stages) { slot = 0; phase ^= 1u; }
            }
        }
        __syncwarp();
    } else if (is_consumer) {
        // ===== consumers =====
        const int gw = t >> 5;                   // warp within the group
        int it = 0;
        // the group's rows are i = g, g + G, ...; slot = i % stages and phase = (i / stages) & 1 are kept
        // incrementally (stages is a multiple of G), as is the output row pointer
        int slot = g;
        uint32_t phase = 0;
        uint4 *orow = out + (static_cast<int64_t>(blockIdx.x) + static_cast<int64_t>(g) * gridDim.x) * h8;
        const int64_t orow_step = static_cast<int64_t>(G) * gridDim.x * h8;
        // Forward: a thread scales the same columns in every row, so its gamma values stay in registers
        // (the backward pass has its dgamma shares there instead and reads gamma from shared memory).
        constexpr bool kGammaRegs = !BWD && VPT <= kGammaRegsMaxVpt;
        float gm_reg[kGammaRegs ? VPT : 1][8];
        if constexpr (kGammaRegs) {
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                const int idx = min(t + T * j, h8 - 1);
                const float4 g0 = reinterpret_cast<const float4 *>(s_gamma)[2 * idx];
                const float4 g1 = reinterpret_cast<const float4 *>(s_gamma)[2 * idx + 1];
                gm_reg[j][0] = g0.x; gm_reg[j][1] = g0.y; gm_reg[j][2] = g0.z; gm_reg[j][3] = g0.w;
                gm_reg[j][4] = g1.x; gm_reg[j][5] = g1.y; gm_reg[j][6] = g1.z; gm_reg[j][7] = g1.w;
            }
        }
        // Row counter: 32-bit in the backward kernel (rows per CTA are far below 2^31; the 64-bit i % stages and
        // i / stages cost ~100 instructions per row and thread: backward h = 4096 132 -> 128 us), 64-bit in the
        // forward kernel, which measured SLOWER with the cheaper form (89 -> 93 us at h = 4096, as it did with the
        // incremental form above): its consumers then return to polling the next slot's barrier sooner.
        using RowIdx = typename RowIndex<BWD>::type;
        const RowIdx my_rows_i = static_cast<RowIdx>(my_rows);
        for (RowIdx i = g; i < my_rows_i; i += G, it ^= 1) {
            if constexpr (INCR) {
                if (i != g) {
                    slot += G;
                    if (slot >= stages) { slot -= stages; phase ^= 1u; }
                    orow += orow_step;
                }
            } else {
                slot = static_cast<int>(i % stages);
                phase = static_cast<uint32_t>(i / stages) & 1u;
                orow = out + (static_cast<int64_t>(blockIdx.x) + static_cast<int64_t>(i) * gridDim.x) * h8;
            }
            bool ok = wait_bar(bar_full + slot * 8, phase, ctx, kStRmsConsumer);
            ok = __all_sync(0xffffffffu, ok);
            // A warp that gave up still walks to the barrier below (on zeros), where the whole group
            // learns of it together; leaving here would strand the others at that barrier.
            const uint8_t *sx = smem + L.off_slot + slot * L.slot_bytes;
            uint4 xv[VPT], dv[VPT];
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                const int idx = t + T * j;
                const bool in = ok && (idx < h8);
                xv[j] = in ? reinterpret_cast<const uint4 *>(sx)[idx] : make_uint4(0, 0, 0, 0);
                if constexpr (BWD)
                    dv[j] = in ? reinterpret_cast<const uint4 *>(sx + L.row_bytes)[idx] : make_uint4(0, 0, 0, 0);
            }
            // the row lives in registers now: hand the slot back to the producer
            __syncwarp();
            if (lane == 0 && ok) mbar_arrive(bar_empty + slot * 8);

            float s1 = 0.f, s2 = 0.f;
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                const int idx = t + T * j;
                float xf[8];
                unpack8<BF16>(xv[j], xf);
                if constexpr (BWD) {
                    float df[8];
                    unpack8<BF16>(dv[j], df);
                    if (idx < h8) {
                        const float4 g0 = reinterpret_cast<const float4 *>(s_gamma)[2 * idx];
                        const float4 g1 = reinterpret_cast<const float4 *>(s_gamma)[2 * idx + 1];
                        const float gm[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            s1 = fmaf(xf[e], xf[e], s1);
                            s2 = fmaf(df[e] * gm[e], xf[e], s2);
                        }
                    }
                } else {
#pragma unroll
                    for (int e = 0; e < 8; ++e) s1 = fmaf(xf[e], xf[e], s1);
                }
            }
            s1 = warp_sum(s1);
            if constexpr (BWD) s2 = warp_sum(s2);
            if (lane == 0) {
                s_red[it][warp][0] = s1;
                s_red[it][warp][1] = s2;
            }
            // One barrier per row: s_red is double-buffered, and buffer `it` is only rewritten two
            // rows later, after every thread of the group has passed the barrier in between.
            if (group_barrier_or(1 + g, T, !ok || *abort_flag != 0)) break;
            float S1 = 0.f, S2 = 0.f;
            for (int w = 0; w < group_warps; ++w) {
                S1 += s_red[it][warp - gw + w][0];
                if constexpr (BWD) S2 += s_red[it][warp - gw + w][1];
            }
            // rsqrt.approx (2 ulp of fp32) and a multiply by 1/h instead of sqrt + two IEEE divisions: ~45 fewer
            // instructions per thread and row; the result is rounded to a 16-bit type anyway
            const float inv_h = 1.0f / h_f;
            const float rstd = rsqrtf(fmaf(S1, inv_h, eps));
            const float cm = (S2 * rstd) * inv_h;   // backward: mean_j(g * xhat)
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                const int idx = t + T * j;
                if (idx < h8) {
                    float gm[8];
                    if constexpr (kGammaRegs) {
#pragma unroll
                        for (int e = 0; e < 8; ++e) gm[e] = gm_reg[j][e];
                    } else {
                        const float4 g0 = reinterpret_cast<const float4 *>(s_gamma)[2 * idx];
                        const float4 g1 = reinterpret_cast<const float4 *>(s_gamma)[2 * idx + 1];
                        gm[0] = g0.x; gm[1] = g0.y; gm[2] = g0.z; gm[3] = g0.w;
                        gm[4] = g1.x; gm[5] = g1.y; gm[6] = g1.z; gm[7] = g1.w;
                    }
                    float xf[8], o[8];
                    unpack8<BF16>(xv[j], xf);
                    if constexpr (BWD) {
                        float df[8];
                        unpack8<BF16>(dv[j], df);
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const float xhat = xf[e] * rstd;
                            o[e] = rstd * (df[e] * gm[e] - xhat * cm);
                            acc[j][e] = fmaf(df[e], xhat, acc[j][e]);
                        }
                    } else {
#pragma unroll
                        for (int e = 0; e < 8; ++e) o[e] = (xf[e] * rstd) * gm[e];
                    }
                    __stcs(orow + idx, pack8<BF16>(o));
                }
            }
        }
    }
    __syncthreads();
    if constexpr (BWD) {
        // The ring is idle now: fold the groups' dgamma shares into one fp32 row in shared memory,
        // group after group (a fixed order), and write ONE partial row per CTA.  Done even after an
        // abandoned wait, so the reduction kernel never reads uninitialised scratch.
        float *s_acc = reinterpret_cast<float *>(smem + L.off_slot);
        for (int gg = 0; gg < G; ++gg) {
            if (is_consumer && g == gg) {
#pragma unroll
                for (int j = 0; j < VPT; ++j) {
                    const int idx = t + T * j;
                    if (idx < h8) {
                        float4 *p = reinterpret_cast<float4 *>(s_acc) + 2 * idx;
                        float4 a0 = make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
                        float4 a1 = make_float4(acc[j][4], acc[j][5], acc[j][6], acc[j][7]);
                        if (gg > 0) {
                            const float4 o0 = p[0], o1 = p[1];
                            a0.x += o0.x; a0.y += o0.y; a0.z += o0.z; a0.w += o0.w;
                            a1.x += o1.x; a1.y += o1.y; a1.z += o1.z; a1.w += o1.w;
                        }
                        p[0] = a0;
                        p[1] = a1;
                    }
                }
            }
            __syncthreads();
        }
        float4 *prow = reinterpret_cast<float4 *>(partial + static_cast<int64_t>(blockIdx.x) * h);
        for (int i = threadIdx.x; i < h / 4; i += kThreads) prow[i] = reinterpret_cast<const float4 *>(s_acc)[i];
    }
    if (*abort_flag) __nanosleep(50000);   // let bulk copies still in flight land before shared memory goes away
}

struct Plan {
    bool ok;
    int vpt, T, G, stages;
    uint32_t smem;
};

Plan make_plan(int64_t h, bool bwd) {
    Plan p{false, 0, 0, 0, 0, 0};
    const int64_t h8 = h / 8;
    if (h8 < 32 || h8 > 2048) return p;
    // groups of 32..256 threads; aim at 4 vectors per thread in the backward pass and 2 in the forward pass
    // (measured at h = 4096 with up to 960 consumer threads: forward 91.0 us with T = 256 / 3 groups against
    // 100.0 us with T = 128 / 7 groups; backward 136 us with T = 128 against 158 us with T = 256)
    const int per_thread = bwd ? 4 : 2;
    int T = static_cast<int>((h8 / per_thread + 31) / 32 * 32);
    if (T < 32) T = 32;
    if (T > 256) T = 256;
    // Forward, 4096 < h < 8192: groups of 256 would own 3-4 vectors per thread with up to a quarter of the slots
    // empty and leave 3 rows in flight per CTA; groups of 128 (5-7 vectors, 6 groups) measured 6072 against 4749 GB/s
    // at h = 5120, 5997 against 5460 at 6144, 5751 against 5373 at 7168 ([32768, h] bf16).  At h = 4096 and 8192 the
    // groups of 256 are faster (6298 against 5869, 5927 against 5724).
    if (!bwd && h8 > 512 && h8 < 1024) T = 128;
    // Benchmark override (builds with PG_ENABLE_TUNING only), read once: PEAKGEMM_TUNE_RMS_T = threads per
    // consumer group (32..256).
    static const int env_t = tune_env_int("PEAKGEMM_TUNE_RMS_T", 0);
    if (env_t >= 32 && env_t <= 256 && env_t % 32 == 0 && (h8 + env_t - 1) / env_t <= 8) T = env_t;
    const int need = static_cast<int>((h8 + T - 1) / T);
    p.vpt = need <= 1 ? 1 : need <= 2 ? 2 : need <= 4 ? 4 : 8;
    p.T = T;
    p.G = (bwd ? (p.vpt == 8 ? Threads<true, 8>::kConsumers : Threads<true, 1>::kConsumers) : p.vpt >= 4 ? Threads<false, 4>::kConsumers : Threads<false, 1>::kConsumers) / T;
    if (p.G > 8) p.G = 8;
    // Ring depth.  More rows in flight are not always better in the forward pass: with groups of 256 threads (three
    // groups) about 64 KiB of rows in flight per SM measured best on [32768, h] bf16 — h = 4096: 9 slots 6500 GB/s
    // against 6324 with 15; h = 8192: 3 slots (one per group, refilled as soon as the group has the row in registers)
    // 6144 against 6009 with 12; h = 12288: 3 slots 6107 against 5965 with 6.  The backward pass and the narrower
    // groups keep the deepest ring that fits (h = 8192 backward: 6604 with 6 slots, 6361 with 3).
    // PEAKGEMM_TUNE_RMS_STAGES (builds with PG_ENABLE_TUNING only) caps the depth instead.
    int max_stages = kMaxStages;
    if (!bwd && T == 256) {
        const int64_t per_round = 3 * h * 2;                      // one row of 16-bit elements per group
        int rounds = static_cast<int>((65536 + per_round / 2) / per_round);
        if (rounds < 1) rounds = 1;
        max_stages = 3 * rounds < kMaxStages ? 3 * rounds : kMaxStages;
    }
    static const int env_stages = tune_env_int("PEAKGEMM_TUNE_RMS_STAGES", 0);
    if (env_stages >= 2 && env_stages <= kMaxStages) max_stages = env_stages;
    for (int s = max_stages; s >= 2; --s) {
        const Layout l = make_layout(static_cast<int>(h), bwd, s);
        if (l.total > kSmemBudget) continue;
        // The ring depth must be a multiple of the number of groups, so that a slot is always consumed by the SAME
        // group.  A consumer waits on full[slot] by phase parity only, which is sound as long as it can be at most
        // one phase early: true for a group that consumed the slot's previous round itself.  With a rotating
        // assignment a group that runs ahead can poll a slot two phases early, see the parity of the phase before
        // last as "complete", read a slot that is still being filled and arrive on empty[slot] out of turn; the
        // surplus arrival breaks the barrier (seen as "unspecified launch failure" once the ring wrapped, i.e. only
        // with hundreds of rows per CTA).
        if (p.G > s) p.G = s;
        const int depth = s / p.G * p.G;
        const Layout ld = make_layout(static_cast<int>(h), bwd, depth);
        p.stages = depth;
        p.smem = ld.total;
        p.ok = true;
        return p;
    }
    return p;
}

int g_sms[kMaxDevices] = {};
int *g_status_ptr[kMaxDevices] = {};
DeviceOnce g_setup_once;

// SM count and the address of the status word, looked up on the first call on a device.  Both tables are
// filled under g_setup_once before its ready flag is published, so no thread can see the SM count without
// the status pointer.
cudaError_t device_setup(int *sms, int **status) {
    int dev = 0;
    cudaError_t e = current_device(&dev);
    if (e != cudaSuccess) return e;
    e = g_setup_once.run(dev, [dev]() {
        int n = 0;
        void *p = nullptr;
        cudaError_t e2;
        if ((e2 = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e2;
        if ((e2 = cudaGetSymbolAddress(&p, g_rms_status_word)) != cudaSuccess) return e2;
        g_status_ptr[dev] = static_cast<int *>(p);
        g_sms[dev] = n;
        return cudaSuccess;
    });
    if (e != cudaSuccess) return e;
    *sms = g_sms[dev];
    *status = g_status_ptr[dev];
    return cudaSuccess;
}

template <bool BWD, int VPT, bool BF16, bool INCR>
cudaError_t launch_one(void *out, float *partial, const void *x, const void *dy, const float *gamma,
                       int64_t rows, int64_t h, float eps, const Plan &p, int grid, int *status,
                       cudaStream_t stream) {
    auto kernel = rms_staged_kernel<BWD, VPT, BF16, INCR>;
    static DeviceOnce smem_once;
    {
        const cudaError_t e = allow_dynamic_smem(smem_once, kernel, static_cast<int>(kSmemBudget));
        if (e != cudaSuccess) return e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
    cfg.blockDim = dim3(Threads<BWD, VPT>::kTotal, 1, 1);
    cfg.dynamicSmemBytes = p.smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<uint4 *>(out), partial, static_cast<const uint4 *>(x),
                              static_cast<const uint4 *>(dy), gamma, rows, static_cast<int>(h / 8),
                              static_cast<float>(h), eps, p.stages, p.T, p.G, status);
}

template <bool BWD>
cudaError_t launch_any(void *out, float *partial, const void *x, const void *dy, const float *gamma, int64_t rows,
                       int64_t h, float eps, bool bf16, const Plan &p, int grid, int *status, cudaStream_t stream) {
    const bool incr = BWD && h > 4096;
#define PG_RMS_CASE(V)                                                                                             \
    if (p.vpt == V) {                                                                                              \
        if (incr)                                                                                                  \
            return bf16 ? launch_one<BWD, V, true, true>(out, partial, x, dy, gamma, rows, h, eps, p, grid, status, stream)   \
                        : launch_one<BWD, V, false, true>(out, partial, x, dy, gamma, rows, h, eps, p, grid, status, stream); \
        return bf16 ? launch_one<BWD, V, true, false>(out, partial, x, dy, gamma, rows, h, eps, p, grid, status, stream)      \
                    : launch_one<BWD, V, false, false>(out, partial, x, dy, gamma, rows, h, eps, p, grid, status, stream);    \
    }
    PG_RMS_CASE(1)
    PG_RMS_CASE(2)
    PG_RMS_CASE(4)
    PG_RMS_CASE(8)
#undef PG_RMS_CASE
    return cudaErrorInvalidValue;
}

}  // namespace

bool rmsnorm_staged_supported(int64_t h, bool bwd) {
    // Benchmark override (builds with PG_ENABLE_TUNING only), read once: PEAKGEMM_TUNE_RMS_STAGED=0 falls back to
    // the register-resident kernels.
    static const bool disabled = tune_env_int("PEAKGEMM_TUNE_RMS_STAGED", 1) == 0;
    if (disabled) return false;
    return make_plan(h, bwd).ok;
}

// CTAs the staged kernels launch for this shape, and (backward) the number of dgamma partial rows
// they write: one per CTA.
cudaError_t rmsnorm_staged_ctas(int64_t rows, int64_t h, bool bwd, int *ctas, int *partial_rows) {
    const Plan p = make_plan(h, bwd);
    if (!p.ok) return cudaErrorInvalidValue;
    int sms = 0, *status = nullptr;
    cudaError_t e = device_setup(&sms, &status);
    if (e != cudaSuccess) return e;
    *ctas = static_cast<int>(rows < sms ? rows : sms);
    *partial_rows = *ctas;
    return cudaSuccess;
}

cudaError_t rmsnorm_staged_fwd(const RmsFwdArgs &a, cudaStream_t stream) {
    const Plan p = make_plan(a.h, false);
    int sms = 0, *status = nullptr, grid = 0, nparts = 0;
    cudaError_t e = device_setup(&sms, &status);
    if (e != cudaSuccess) return e;
    if ((e = rmsnorm_staged_ctas(a.rows, a.h, false, &grid, &nparts)) != cudaSuccess) return e;
    return launch_any<false>(a.y, nullptr, a.x, nullptr, a.gamma, a.rows, a.h, a.eps, a.bf16, p, grid, status, stream);
}

cudaError_t rmsnorm_staged_bwd(const RmsBwdArgs &a, cudaStream_t stream) {
    const Plan p = make_plan(a.h, true);
    int sms = 0, *status = nullptr, ctas = 0, nparts = 0;
    cudaError_t e = device_setup(&sms, &status);
    if (e != cudaSuccess) return e;
    if ((e = rmsnorm_staged_ctas(a.rows, a.h, true, &ctas, &nparts)) != cudaSuccess) return e;
    return launch_any<true>(a.dx, static_cast<float *>(a.workspace), a.x, a.dy, a.gamma, a.rows, a.h, a.eps, a.bf16,
                            p, ctas, status, stream);
}

cudaError_t rmsnorm_device_status(int *out, cudaStream_t stream) {
    int sms = 0, *status = nullptr;
    cudaError_t e = device_setup(&sms, &status);
    if (e != cudaSuccess) return e;
    int host = 0;
    if ((e = cudaMemcpyAsync(&host, status, sizeof(int), cudaMemcpyDeviceToHost, stream)) != cudaSuccess) return e;
    if ((e = cudaStreamSynchronize(stream)) != cudaSuccess) return e;
    if (host != 0 && (e = cudaMemsetAsync(status, 0, sizeof(int), stream)) != cudaSuccess) return e;
    *out = host;
    return cudaSuccess;
}

}  // namespace pg

#ifdef PG_TEST_SHORT_WAIT
// Test build only: 1 = the first CTA's producer leaves out its last row.
extern "C" int pg_test_withhold_rmsnorm_row(int on) {
    return static_cast<int>(cudaMemcpyToSymbol(pg::g_test_withhold_last_row, &on, sizeof(int)));
}
#endif
