// Half-precision GEMM for B200 (sm_100a):  C[m,n] = A[m,k] * B[n,k]^T, fp32
// accumulation, 16-bit output.  Takes the place of the reference project's
// mma.sync kernel and launcher (src/impl/hgemm_wmma_impl.h:288-423).
//
// One persistent, warp-specialised kernel, templated on
//   CTA_GROUP  1: one CTA owns a 128 x BN tile            (tcgen05 cta_group::1)
//              2: a CTA pair owns a 256 x BN tile; each CTA loads its own 128
//                 rows of A and its own BN/2 rows of B, the leader CTA issues one
//                 256 x BN x 16 MMA that reads both CTAs' shared memory and writes
//                 both CTAs' tensor memory                 (tcgen05 cta_group::2)
//   BN         tile width (64, 128, 256)
//   STAGES     depth of the TMA -> MMA shared-memory ring (>= 4)
//
// Warp roles (192 threads):
//   warp 0    producer: one thread issues the TMA loads of A and B k-blocks
//             (128-byte swizzled, 64 elements of k per block) and arms full[s]
//   warp 1    allocates tensor memory; one thread issues tcgen05.mma for each
//             k-block, frees the stage through tcgen05.commit -> empty[s], and
//             hands the finished accumulator to the epilogue through acc_full[a]
//   warps 2-5 epilogue: tensor memory -> registers (tcgen05.ld) -> round to
//             bf16/fp16 -> swizzled shared memory -> TMA store; each warp owns the
//             32 accumulator lanes its warp id allows it to read and stores its
//             own 32-row slab, so the epilogue warps never synchronise with one
//             another.  Two accumulators (2 x BN tensor-memory columns) let the
//             epilogue of tile i overlap the main loop of tile i+1.
//
// Tiles are walked in a grouped raster (bands of kGroupM tile rows) so that the
// tiles in flight at any time share A and B panels in L2; the reference's CUDA
// path uses the identity map (hgemm_wmma_impl.h:245-249).
//
// Row, column and k tails need no special code: TMA zero-fills loads outside the
// tensor and clips stores, which also removes the reference kernel's
// out-of-bounds reads for m or n not a multiple of 128 (hgemm_wmma_impl.h:61-84).
//
// In the pair kernel, signals that must cross to the other CTA use plain remote
// mbarrier arrives relayed by a thread that has already observed the event
// (no multicast anywhere):
//   * stage s free in the peer: the leader's producer, once it has seen its own
//     empty[s] complete, arrives on the peer's empty[s];
//   * accumulator a ready in the peer: the leader's first epilogue warp, once it
//     has seen acc_full[a], arrives on the peer's acc_full[a];
//   * accumulator a drained: the peer's epilogue warps arrive on the leader's
//     acc_empty[a] (count 8 = 4 local + 4 remote warps).
//
// Every wait is bounded: a role that waits longer than kWaitTimeoutNs records a
// code in a device status word, raises a CTA-wide abort flag and all roles fall
// through to the common teardown (tensor memory is freed, the kernel returns).

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include "gemm_sm100.h"
#include "ptx.cuh"

namespace pg {

using namespace ptx;

namespace {

constexpr uint32_t kBM = 128;           // rows of A per CTA
constexpr uint32_t kBK = 64;            // k elements per stage = one 128-byte swizzle row
constexpr uint32_t kUmmaK = 16;         // k elements per tcgen05.mma (16-bit inputs)
constexpr uint32_t kThreads = 192;
constexpr uint32_t kEpiWarps = 4;
constexpr uint32_t kStoreCols = 64;     // columns per TMA store box (128 bytes)
constexpr uint32_t kStoreRows = 32;     // rows per TMA store box (one warp's lanes)
constexpr uint32_t kStageBufBytes = kStoreRows * kStoreCols * 2;  // 4096
constexpr uint64_t kWaitTimeoutNs = 2000000000ull;                // 2 s
constexpr uint32_t kDefaultFlags = 0;

// Tuning switches (kernel argument `flags`).
enum : uint32_t {
    kFlagEpiLanePoll = 1u,       // epilogue: one lane polls acc_full with a back-off
    kFlagStoreEvictFirst = 2u,   // C stores carry an L2 evict-first hint
    kFlagLoadEvictLast = 4u,     // A/B loads carry an L2 evict-last hint
};

// Codes written to the device status word (role that gave up).
enum : int {
    kStProducerEmpty = 1,
    kStMmaFull = 2,
    kStMmaAccEmpty = 3,
    kStEpiAccFull = 4,
};

template <int CTA_GROUP, int BN, int STAGES>
struct Cfg {
    static constexpr uint32_t kBRows = BN / CTA_GROUP;          // rows of B this CTA loads
    static constexpr uint32_t kABytes = kBM * kBK * 2;          // 16 KiB
    static constexpr uint32_t kBBytes = kBRows * kBK * 2;
    static constexpr uint32_t kStageBytes = kABytes + kBBytes;
    static constexpr uint32_t kTmemCols = 2 * BN;               // two accumulators
    static constexpr uint32_t kOffA = 0;
    static constexpr uint32_t kOffB = kOffA + STAGES * kABytes;
    static constexpr uint32_t kOffC = kOffB + STAGES * kBBytes;
    static constexpr uint32_t kOffBar = kOffC + kEpiWarps * 2 * kStageBufBytes;
    // full[STAGES], empty[STAGES], acc_full[2], acc_empty[2], then tmem slot + abort flag
    static constexpr uint32_t kNumBars = 2 * STAGES + 4;
    static constexpr uint32_t kOffMisc = kOffBar + kNumBars * 8;
    static constexpr uint32_t kSmemBytes = kOffMisc + 16 + 1024;  // + slack to align the base to 1024
    static_assert(kTmemCols == 128 || kTmemCols == 256 || kTmemCols == 512, "tmem columns: power of 2");
    static_assert(kSmemBytes <= 232448, "exceeds 227 KiB of shared memory");
    static_assert(BN % kStoreCols == 0, "BN must be a multiple of the store box");
    static_assert((BN / CTA_GROUP) % 8 == 0 && BN % 16 == 0 && BN <= 256, "invalid MMA N");
};

struct WaitCtx {
    volatile uint32_t *abort_flag;  // shared memory
    int *status;                    // global memory
};

// Bounded mbarrier wait.  Returns false if the wait was abandoned.  The clock is
// only consulted every 1024 failed probes (each probe already suspends the thread
// for a hardware-defined interval), so the common short wait costs nothing extra.
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
                atomicCAS(ctx.status, 0, code);
                return false;
            }
        }
    }
}

// Like wait_bar, for waits that normally last a whole tile: sleeps between probes.
__device__ __forceinline__ bool wait_bar_backoff(uint32_t bar, uint32_t parity, const WaitCtx &ctx, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    uint64_t t0 = 0;
    uint32_t spins = 0;
    while (true) {
        __nanosleep(200);
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 1023u) == 0) {
            if (*ctx.abort_flag) return false;
            const uint64_t now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > kWaitTimeoutNs) {
                *ctx.abort_flag = 1;
                atomicCAS(ctx.status, 0, code);
                return false;
            }
        }
    }
}

// Grouped raster: tile t -> (mi, ni).  Tiles are numbered down the rows of a band
// of kGroupM tile rows first, then across the columns, band after band.
__device__ __forceinline__ void tile_coords(uint32_t kGroupM, uint32_t t, uint32_t m_tiles, uint32_t n_tiles,
                                            uint32_t &mi, uint32_t &ni) {
    const uint32_t per_band = kGroupM * n_tiles;
    const uint32_t band = t / per_band;
    const uint32_t first_m = band * kGroupM;
    const uint32_t band_rows = min(kGroupM, m_tiles - first_m);
    const uint32_t r = t - band * per_band;
    mi = first_m + r % band_rows;
    ni = r / band_rows;
}

template <int CTA_GROUP, int BN, int STAGES, bool BF16>
__global__ void __launch_bounds__(kThreads, 1)
hgemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_a,
                     const __grid_constant__ CUtensorMap tm_b,
                     const __grid_constant__ CUtensorMap tm_c,
                     uint32_t M, uint32_t N, uint32_t K, uint32_t group_m, uint32_t flags, int *status) {
    using C = Cfg<CTA_GROUP, BN, STAGES>;
    constexpr uint32_t kTileM = kBM * CTA_GROUP;

    extern __shared__ uint8_t smem_raw[];
    // Swizzled TMA tiles and UMMA descriptors want 1024-byte aligned bases.
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

    const uint32_t warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t rank = (CTA_GROUP == 2) ? cluster_ctarank() : 0u;
    const bool leader = (rank == 0);

    const uint32_t bar_full = smem_base + C::kOffBar;
    const uint32_t bar_empty = bar_full + STAGES * 8;
    const uint32_t bar_acc_full = bar_empty + STAGES * 8;
    const uint32_t bar_acc_empty = bar_acc_full + 2 * 8;
    const uint32_t tmem_slot = smem_base + C::kOffMisc;
    volatile uint32_t *tmem_slot_gen = reinterpret_cast<volatile uint32_t *>(smem_gen + C::kOffMisc);
    volatile uint32_t *abort_flag = tmem_slot_gen + 1;
    const WaitCtx ctx{abort_flag, status};

    const uint32_t m_tiles = (M + kTileM - 1) / kTileM;
    const uint32_t n_tiles = (N + BN - 1) / BN;
    const uint32_t k_blocks = (K + kBK - 1) / kBK;
    const uint32_t total_tiles = m_tiles * n_tiles;
    const uint32_t worker = blockIdx.x / CTA_GROUP;       // cluster index (CTA index when CTA_GROUP == 1)
    const uint32_t workers = gridDim.x / CTA_GROUP;

    // ------------------------------------------------------------- set-up ----
    if (warp == 0 && lane == 0) {
        for (uint32_t s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + s * 8, 1);    // producer's arrive.expect_tx (+ TMA bytes)
            mbar_init(bar_empty + s * 8, 1);   // tcgen05.commit, or the leader's relay in the peer CTA
        }
        for (uint32_t a = 0; a < 2; ++a) {
            mbar_init(bar_acc_full + a * 8, 1);                          // tcgen05.commit / relay
            mbar_init(bar_acc_empty + a * 8, kEpiWarps * CTA_GROUP);     // one arrive per epilogue warp
        }
        *abort_flag = 0;
        fence_mbar_init();
        prefetch_tensormap(&tm_a);
        prefetch_tensormap(&tm_b);
        prefetch_tensormap(&tm_c);
    }
    if (warp == 1) {
        tmem_alloc<CTA_GROUP>(tmem_slot, C::kTmemCols);
        tmem_relinquish<CTA_GROUP>();
    }
    tc_fence_before_sync();
    __syncthreads();
    if constexpr (CTA_GROUP == 2) {  // the peer's barriers must exist before anything signals them
        cluster_arrive();
        cluster_wait();
    }
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot_gen;

    // -------------------------------------------------------------- roles ----
    if (warp == 0) {
        if (lane == 0) {
            // ===== producer =====
            // In a pair, both CTAs' loads complete on the LEADER's full[s].
            const uint32_t full0 = (CTA_GROUP == 2) ? mapa(bar_full, 0) : bar_full;
            const uint32_t peer_empty0 = (CTA_GROUP == 2) ? mapa(bar_empty, 1) : 0u;
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            const uint64_t pol_load = l2_policy_evict_last();
            for (uint32_t t = worker; ok && t < total_tiles; t += workers) {
                uint32_t mi, ni;
                tile_coords(group_m, t, m_tiles, n_tiles, mi, ni);
                const int32_t row_a = static_cast<int32_t>(mi * kTileM + rank * kBM);
                const int32_t row_b = static_cast<int32_t>(ni * BN + rank * C::kBRows);
                for (uint32_t kb = 0; kb < k_blocks; ++kb) {
                    if (leader) {
                        // wait until the MMAs that read this stage have completed
                        ok = wait_bar(bar_empty + stage * 8, phase ^ 1u, ctx, kStProducerEmpty);
                        if (!ok) break;
                        if constexpr (CTA_GROUP == 2) {
                            mbar_arrive_cluster(peer_empty0 + stage * 8);   // relay to the peer
                            mbar_arrive_expect_tx(bar_full + stage * 8, 2 * C::kStageBytes);
                        } else {
                            mbar_arrive_expect_tx(bar_full + stage * 8, C::kStageBytes);
                        }
                    } else {
                        ok = wait_bar(bar_empty + stage * 8, phase, ctx, kStProducerEmpty);
                        if (!ok) break;
                    }
                    const uint32_t dst_a = smem_base + C::kOffA + stage * C::kABytes;
                    const uint32_t dst_b = smem_base + C::kOffB + stage * C::kBBytes;
                    const int32_t kx = static_cast<int32_t>(kb * kBK);
                    if (flags & kFlagLoadEvictLast) {
                        if constexpr (CTA_GROUP == 2) {
                            tma_load_2d_pair_hint(dst_a, &tm_a, full0 + stage * 8, kx, row_a, pol_load);
                            tma_load_2d_pair_hint(dst_b, &tm_b, full0 + stage * 8, kx, row_b, pol_load);
                        } else {
                            tma_load_2d_hint(dst_a, &tm_a, bar_full + stage * 8, kx, row_a, pol_load);
                            tma_load_2d_hint(dst_b, &tm_b, bar_full + stage * 8, kx, row_b, pol_load);
                        }
                    } else if constexpr (CTA_GROUP == 2) {
                        tma_load_2d_pair(dst_a, &tm_a, full0 + stage * 8, kx, row_a);
                        tma_load_2d_pair(dst_b, &tm_b, full0 + stage * 8, kx, row_b);
                    } else {
                        tma_load_2d(dst_a, &tm_a, bar_full + stage * 8, kx, row_a);
                        tma_load_2d(dst_b, &tm_b, bar_full + stage * 8, kx, row_b);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            // ===== MMA issuer =====
            constexpr uint32_t idesc = instr_desc_f16(BF16, kBM * CTA_GROUP, BN);
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            for (uint32_t t = worker; ok && t < total_tiles; t += workers) {
                // the epilogue must have drained this accumulator (passes at once the first two times)
                ok = wait_bar(bar_acc_empty + acc * 8, acc_phase ^ 1u, ctx, kStMmaAccEmpty);
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t tmem_d = tmem_base + acc * BN;
                for (uint32_t kb = 0; kb < k_blocks; ++kb) {
                    ok = wait_bar(bar_full + stage * 8, phase, ctx, kStMmaFull);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint64_t da = smem_desc_k_sw128(smem_base + C::kOffA + stage * C::kABytes);
                    const uint64_t db = smem_desc_k_sw128(smem_base + C::kOffB + stage * C::kBBytes);
#pragma unroll
                    for (uint32_t k = 0; k < kBK / kUmmaK; ++k) {
                        // 16 elements of k = 32 bytes inside the 128-byte swizzle row = +2 in the >>4 address field
                        umma_f16<CTA_GROUP>(tmem_d, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0u ? 1u : 0u);
                    }
                    umma_commit<CTA_GROUP>(bar_empty + stage * 8);   // stage free once these MMAs are done
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                umma_commit<CTA_GROUP>(bar_acc_full + acc * 8);      // accumulator complete
                if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
            }
        }
        __syncwarp();
    } else {
        // ===== epilogue =====
        const uint32_t q = warp & 3u;                 // lane quarter this warp may read
        const uint32_t e = warp - 2u;                 // 0..3: staging buffers
        const uint32_t buf0 = smem_base + C::kOffC + e * 2 * kStageBufBytes;
        uint8_t *buf0_gen = smem_gen + C::kOffC + e * 2 * kStageBufBytes;
        const uint32_t acc_empty_leader = (CTA_GROUP == 2) ? mapa(bar_acc_empty, 0) : bar_acc_empty;
        const uint32_t peer_acc_full = (CTA_GROUP == 2) ? mapa(bar_acc_full, 1) : 0u;
        uint32_t acc = 0, acc_phase = 0, nbuf = 0;
        bool ok = true;
        const uint64_t pol_store = l2_policy_evict_first();
        for (uint32_t t = worker; ok && t < total_tiles; t += workers) {
            uint32_t mi, ni;
            tile_coords(group_m, t, m_tiles, n_tiles, mi, ni);
            if (flags & kFlagEpiLanePoll) {
                // one lane polls, with a back-off: the other 31 (x4 warps) sleep at the warp barrier
                if (lane == 0) ok = wait_bar_backoff(bar_acc_full + acc * 8, acc_phase, ctx, kStEpiAccFull);
                ok = __shfl_sync(0xffffffffu, ok, 0);
            } else {
                ok = wait_bar(bar_acc_full + acc * 8, acc_phase, ctx, kStEpiAccFull);
                ok = __all_sync(0xffffffffu, ok);
            }
            if (!ok) break;
            if constexpr (CTA_GROUP == 2) {
                if (leader && e == 0 && lane == 0) mbar_arrive_cluster(peer_acc_full + acc * 8);  // relay
            }
            tc_fence_after_sync();
            const uint32_t row0 = mi * kTileM + rank * kBM + q * 32u;   // first row of this warp's slab
            const uint32_t taddr = tmem_base + acc * BN + ((q * 32u) << 16);
#pragma unroll 1
            for (uint32_t ch = 0; ch < BN / kStoreCols; ++ch) {
                uint32_t v[2][32];
                tmem_ld_32x32b_x32(taddr + ch * kStoreCols, v[0]);
                tmem_ld_32x32b_x32(taddr + ch * kStoreCols + 32u, v[1]);
                tmem_ld_wait();
                if (ch == BN / kStoreCols - 1) {
                    // every tcgen05.ld of this accumulator has completed: give it back to the MMA warp
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) {
                        if constexpr (CTA_GROUP == 2) mbar_arrive_cluster(acc_empty_leader + acc * 8);
                        else mbar_arrive(bar_acc_empty + acc * 8);
                    }
                }
                // the store issued two chunks ago from this buffer must have finished reading it
                if (lane == 0) bulk_wait_group_read<1>();
                __syncwarp();
                const uint32_t sbuf = buf0 + nbuf * kStageBufBytes;
                uint8_t *sbuf_gen = buf0_gen + nbuf * kStageBufBytes;
                // row `lane`, 8 chunks of 16 bytes, chunk c stored at position c ^ (row % 8)  (128-byte swizzle)
#pragma unroll
                for (uint32_t c = 0; c < 8; ++c) {
                    const uint32_t *src = &v[c >> 2][(c & 3u) * 8u];
                    uint4 o;
                    o.x = pack2<BF16>(__uint_as_float(src[0]), __uint_as_float(src[1]));
                    o.y = pack2<BF16>(__uint_as_float(src[2]), __uint_as_float(src[3]));
                    o.z = pack2<BF16>(__uint_as_float(src[4]), __uint_as_float(src[5]));
                    o.w = pack2<BF16>(__uint_as_float(src[6]), __uint_as_float(src[7]));
                    *reinterpret_cast<uint4 *>(sbuf_gen + lane * 128u + ((c ^ (lane & 7u)) << 4)) = o;
                }
                fence_proxy_async_smem();
                __syncwarp();
                const uint32_t col0 = ni * BN + ch * kStoreCols;
                if (lane == 0) {
                    if (row0 < M && col0 < N) {
                        if (flags & kFlagStoreEvictFirst)
                            tma_store_2d_hint(&tm_c, sbuf, static_cast<int32_t>(col0), static_cast<int32_t>(row0),
                                              pol_store);
                        else
                            tma_store_2d(&tm_c, sbuf, static_cast<int32_t>(col0), static_cast<int32_t>(row0));
                    }
                    bulk_commit_group();
                }
                nbuf ^= 1u;
            }
            if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
        if (lane == 0) bulk_wait_group<0>();   // shared memory must outlive the stores that read it
        __syncwarp();
    }

    // ----------------------------------------------------------- teardown ----
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) __nanosleep(50000);   // let copies still in flight land before shared memory goes away
    if constexpr (CTA_GROUP == 2) {        // neither CTA may exit while its peer can still touch it
        cluster_arrive();
        cluster_wait();
    }
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc<CTA_GROUP>(tmem_base, C::kTmemCols);
    }
}

// Zero-fills C when k == 0 (an empty sum).
__global__ void zero_fill_kernel(uint16_t *c, int64_t m, int64_t n, int64_t ldc) {
    const int64_t total = m * n;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        c[(i / n) * ldc + (i % n)] = 0;
    }
}

// ------------------------------------------------------------------- host ----

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// Row-major [rows, cols] 16-bit matrix with row pitch ld (elements); box = box_rows x 64 columns.
bool make_tmap(CUtensorMap *tm, const void *base, int64_t rows, int64_t cols, int64_t ld,
               uint32_t box_rows, bool bf16, bool is_output) {
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return false;
    cuuint64_t gdim[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    cuuint64_t gstride[1] = {static_cast<cuuint64_t>(ld) * 2};
    cuuint32_t box[2] = {kBK, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(tm, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                     const_cast<void *>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B,
                     is_output ? CU_TENSOR_MAP_L2_PROMOTION_NONE : CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

struct DeviceInfo {
    bool ready = false;
    int sm_count = 0;
    int cc_major = 0;
    int *status_word = nullptr;
};

__device__ int g_gemm_status_word;

DeviceInfo g_dev[64];

cudaError_t device_info(DeviceInfo **out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    DeviceInfo &d = g_dev[dev];
    if (!d.ready) {
        if ((e = cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
        if ((e = cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev)) != cudaSuccess) return e;
        if (d.cc_major == 10) {
            void *p = nullptr;
            if ((e = cudaGetSymbolAddress(&p, g_gemm_status_word)) != cudaSuccess) return e;
            d.status_word = static_cast<int *>(p);
        }
        d.ready = true;
    }
    *out = &d;
    return cudaSuccess;
}

template <int CTA_GROUP, int BN, int STAGES, bool BF16>
cudaError_t launch(const GemmArgs &g, const DeviceInfo &d, int sms, cudaStream_t stream) {
    using C = Cfg<CTA_GROUP, BN, STAGES>;
    auto kernel = hgemm_tcgen05_kernel<CTA_GROUP, BN, STAGES, BF16>;
    static bool attr_done[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
        if (e != cudaSuccess) return e;
        attr_done[dev] = true;
    }
    CUtensorMap tm_a, tm_b, tm_c;
    if (!make_tmap(&tm_a, g.a, g.m, g.k, g.lda, kBM, BF16, false) ||
        !make_tmap(&tm_b, g.b, g.n, g.k, g.ldb, C::kBRows, BF16, false) ||
        !make_tmap(&tm_c, g.c, g.m, g.n, g.ldc, kStoreRows, BF16, true))
        return cudaErrorInvalidValue;

    const uint32_t tile_m = kBM * CTA_GROUP;
    const uint64_t m_tiles = (g.m + tile_m - 1) / tile_m;
    const uint64_t n_tiles = (g.n + BN - 1) / BN;
    const uint64_t tiles = m_tiles * n_tiles;
    uint64_t workers = static_cast<uint64_t>(sms / CTA_GROUP);
    if (tiles < workers) workers = tiles;

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(workers * CTA_GROUP), 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = C::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CTA_GROUP;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    uint32_t group_m = 16 / CTA_GROUP, flags = kDefaultFlags;
    if (const char *e = getenv("PEAKGEMM_TUNE_GROUP_M")) group_m = static_cast<uint32_t>(atoi(e));
    if (const char *e = getenv("PEAKGEMM_TUNE_FLAGS")) flags = static_cast<uint32_t>(atoi(e));
    if (group_m < 1) group_m = 1;
    return cudaLaunchKernelEx(&cfg, kernel, tm_a, tm_b, tm_c, static_cast<uint32_t>(g.m),
                              static_cast<uint32_t>(g.n), static_cast<uint32_t>(g.k), group_m, flags,
                              d.status_word);
}

template <int CTA_GROUP, int BN, int STAGES>
cudaError_t launch_dt(const GemmArgs &g, const DeviceInfo &d, int sms, cudaStream_t stream) {
    return g.bf16 ? launch<CTA_GROUP, BN, STAGES, true>(g, d, sms, stream)
                  : launch<CTA_GROUP, BN, STAGES, false>(g, d, sms, stream);
}

}  // namespace

// Picks the kernel variant and tile width when the caller leaves them open, by a
// small cost model: waves of tiles over the SMs (or SM pairs) times the tile
// width, divided by how efficient that configuration is per tile.  (The reference
// has one fixed configuration: hgemm_wmma_impl.h:410.)
void choose_config(const GemmArgs &g, int sm_count, int *variant, int *block_n) {
    const int v_lo = (*variant == 0) ? 1 : *variant, v_hi = (*variant == 0) ? 2 : *variant;
    double best = 1e300;
    int best_v = v_lo, best_bn = (*block_n == 0) ? 256 : *block_n;
    for (int v = v_hi; v >= v_lo; --v) {
        if (*variant == 0 && v == 2 && g.m <= 128) continue;   // a pair needs two 128-row halves
        for (int bn = 256; bn >= 64; bn /= 2) {
            if (*block_n != 0 && bn != *block_n) continue;
            const int64_t tile_m = 128 * v;
            const int64_t tiles = ((g.m + tile_m - 1) / tile_m) * ((g.n + bn - 1) / bn);
            const int64_t workers = sm_count / v;
            const int64_t waves = (tiles + workers - 1) / workers;
            // measured at 8192^3: block_n 128 runs at ~0.72 of block_n 256 per flop (operand traffic per flop doubles)
            const double eff = (bn == 256 ? 1.0 : bn == 128 ? 0.72 : 0.45) * (v == 2 ? 1.06 : 1.0);
            const double cost = static_cast<double>(waves) * bn / eff;
            if (cost < best) { best = cost; best_v = v; best_bn = bn; }
        }
    }
    *variant = best_v;
    *block_n = best_bn;
}

int hgemm_launch(const GemmArgs &g, int variant, int block_n, int max_sms, cudaStream_t stream,
                 cudaError_t *cuda_err) {
    DeviceInfo *d = nullptr;
    cudaError_t e = device_info(&d);
    if (e != cudaSuccess) { *cuda_err = e; return kLaunchCuda; }
    if (d->cc_major != 10) return kLaunchNotSm100;

    if (g.k == 0) {
        zero_fill_kernel<<<d->sm_count * 4, 256, 0, stream>>>(static_cast<uint16_t *>(g.c), g.m, g.n, g.ldc);
        e = cudaGetLastError();
        if (e != cudaSuccess) { *cuda_err = e; return kLaunchCuda; }
        return kLaunchOk;
    }
    int sms = d->sm_count;
    if (max_sms > 0 && max_sms < sms) sms = max_sms < 2 ? 2 : max_sms;
    choose_config(g, sms, &variant, &block_n);

    if (variant == 1) {
        if (block_n == 256) e = launch_dt<1, 256, 4>(g, *d, sms, stream);
        else if (block_n == 128) e = launch_dt<1, 128, 6>(g, *d, sms, stream);
        else if (block_n == 64) e = launch_dt<1, 64, 8>(g, *d, sms, stream);
        else return kLaunchBadConfig;
    } else if (variant == 2) {
        if (block_n == 256) e = launch_dt<2, 256, 6>(g, *d, sms, stream);
        else if (block_n == 128) e = launch_dt<2, 128, 8>(g, *d, sms, stream);
        else if (block_n == 64) e = launch_dt<2, 64, 8>(g, *d, sms, stream);
        else return kLaunchBadConfig;
    } else {
        return kLaunchBadConfig;
    }
    if (e != cudaSuccess) { *cuda_err = e; return kLaunchCuda; }
    return kLaunchOk;
}

int gemm_device_status(int *out, cudaStream_t stream, cudaError_t *cuda_err) {
    DeviceInfo *d = nullptr;
    cudaError_t e = device_info(&d);
    if (e != cudaSuccess) { *cuda_err = e; return kLaunchCuda; }
    if (d->cc_major != 10) return kLaunchNotSm100;
    int host = 0;
    if ((e = cudaMemcpyAsync(&host, d->status_word, sizeof(int), cudaMemcpyDeviceToHost, stream)) != cudaSuccess ||
        (e = cudaStreamSynchronize(stream)) != cudaSuccess ||
        (host != 0 && (e = cudaMemsetAsync(d->status_word, 0, sizeof(int), stream)) != cudaSuccess)) {
        *cuda_err = e;
        return kLaunchCuda;
    }
    *out = host;
    return kLaunchOk;
}

}  // namespace pg
