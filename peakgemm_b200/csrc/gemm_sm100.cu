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
//   MT         row blocks per CTA.  1: the tile is 128*CTA_GROUP rows.  2 (CTA pair, BN = 256): the pair owns a
//              512 x 256 tile as two 256-row blocks that share every k-block of B; their two accumulators fill
//              tensor memory.  Per flop this moves 25 % fewer operand bytes from L2 into shared memory than the
//              256 x 256 tile ((512 + 256) against 2 * (256 + 256) rows per two 256 x 256 x 64 blocks of work),
//              which on a power-capped part is clock: the price is that the epilogue of a tile no longer overlaps
//              the next tile's first MMAs (the second block's accumulator drains while the first block's restart).
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
//
// Optional extras of the same kernel, all off (null pointers) in a plain GEMM:
//   * fused epilogue terms  out = row_scale[row] * acc + bias[col] + residual[row, col]  (EpiArgs);
//   * several destinations for the output tile (DstMaps): the column-sharded caller's gather over NVLink;
//   * tail split (TailArgs): the last partial wave of tiles cut into k-slices over the idle workers, partial
//     sums through a caller workspace, launched cooperatively;
//   * producer synchronisation (TailArgs::wave_sync, large problems): the producers of all workers meet at the first
//     and every 8th k-block of a tile through one global counter, so that workers sharing an A or B panel fetch the
//     same k-block at nearly the same time (L2 hits and merged requests instead of repeated DRAM reads).  A wait
//     there has a short patience and no consequence for the result, so it needs no cooperative launch.
// The file also holds the two kernels for few output tiles (cluster split-K, swapped-operand skinny), which
// share the fused epilogue terms, and the host side: tensor-map cache, configuration choice, launches.

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <math.h>
#include <stdlib.h>

#include "gemm_sm100.h"
#include "host_util.h"
#include "ptx.cuh"

namespace pg {

using namespace ptx;

namespace {

constexpr uint32_t kBM = 128;           // rows of A per CTA
constexpr uint32_t kBK = 64;            // k elements per stage = one 128-byte swizzle row
constexpr uint32_t kUmmaK = 16;         // k elements per tcgen05.mma (16-bit inputs)
constexpr uint32_t kThreads = 192;
constexpr uint32_t kEpiWarps = 4;
// The two-row-block kernel (MT == 2) runs 8 epilogue warps: two per tensor-memory lane quarter, each holding
// 128 columns of one accumulator in registers, so that an accumulator is handed back after ONE round of loads.
constexpr uint32_t kEpiWarpsWide = 8;
constexpr uint32_t kThreadsWide = 64 + 32 * kEpiWarpsWide;
constexpr uint32_t kStoreCols = 64;     // columns per TMA store box (128 bytes)
constexpr uint32_t kStoreRows = 32;     // rows per TMA store box (one warp's lanes)
constexpr uint32_t kStageBufBytes = kStoreRows * kStoreCols * 2;  // 4096
#ifdef PG_TEST_SHORT_WAIT
// Test build (libPeakGemm_device_waittest.so, never shipped as the product): waits give up after 2 ms, and a
// switch in device memory makes ONE signal go missing, so that the give-up path itself can be exercised: the
// waiting role records its code, the CTA drains, the kernel returns and the context stays usable.  The missing
// signal is chosen so that nothing is in flight when the roles drain: the MMAs have completed, only the
// "accumulator ready" commit is withheld, so the epilogue warps are the ones that give up.
constexpr uint64_t kWaitTimeoutNs = 2000000ull;
__device__ int g_test_withhold_acc_commit;
#else
constexpr uint64_t kWaitTimeoutNs = 2000000000ull;                // 2 s
#endif
// Default switches.  ncu sweep at 8192^3 (pair kernel, band height 8): serpentine + A evict-last reads 943 MB
// from DRAM against 1051 MB with no hints; an evict-first hint on B costs +60 %.
constexpr uint32_t kDefaultFlags = 4u | 32u;

// Tuning switches (kernel argument `flags`).
enum : uint32_t {
    kFlagStoreEvictFirst = 2u,   // C stores carry an L2 evict-first hint
    kFlagAEvictLast = 4u,        // A loads carry an L2 evict-last hint (keep the band's A panel resident)
    kFlagBEvictFirst = 8u,       // B loads carry an L2 evict-first hint (B streams through once per band)
    kFlagBEvictLast = 16u,       // B loads carry an L2 evict-last hint
    kFlagSerpentine = 32u,       // odd bands walk their columns right to left
    kFlagRasterAlongN = 64u,     // bands of group_m tile COLUMNS walked row by row: consecutive workers share an A panel
    // Launched under programmatic stream serialisation: the grid lets its successor in the stream start at once
    // (griddepcontrol.launch_dependents) and itself touches no global memory before its predecessor has completed
    // (griddepcontrol.wait at the start of every role that loads or stores).  Back-to-back GEMMs then overlap the
    // launch latency and the set-up of one kernel (barriers, tensor-memory allocation, descriptor prefetch) with the
    // last tiles of the one before.  Behind any other kernel the wait returns when that kernel has completed: the
    // ordinary stream order.
    kFlagPdl = 128u,
};

// Codes written to the device status word (role that gave up).
enum : int {
    kStProducerEmpty = 1,
    kStMmaFull = 2,
    kStMmaAccEmpty = 3,
    kStEpiAccFull = 4,
    kStEpiTailFlag = 5,
};

template <int CTA_GROUP, int BN, int STAGES, int MT = 1>
struct Cfg {
    static constexpr uint32_t kBRows = BN / CTA_GROUP;          // rows of B this CTA loads
    static constexpr uint32_t kABox = kBM * kBK * 2;            // one 128-row box of A: 16 KiB
    static constexpr uint32_t kABytes = MT * kABox;             // MT row blocks of A per stage
    static constexpr uint32_t kBBytes = kBRows * kBK * 2;
    static constexpr uint32_t kStageBytes = kABytes + kBBytes;
    // MT == 1: two accumulators, tile i's epilogue overlaps tile i+1's main loop.
    // MT == 2: the two row blocks' accumulators fill tensor memory; both belong to the tile in flight.
    static constexpr uint32_t kTmemCols = 2 * BN;
    // Columns of one TMA store box.  MT == 2: 8 epilogue warps share the staging area, 4 KiB each; two 32 x 32
    // boxes (64-byte swizzle) per warp let the conversion of one box overlap the store of the other.
    static constexpr uint32_t kStoreBoxCols = (MT == 2) ? 32 : kStoreCols;
    static_assert(MT == 1 || (MT == 2 && CTA_GROUP == 2 && BN == 256), "two row blocks: CTA pair, 256 columns");
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

// Destinations of the output tile: the epilogue stores every 32 x 64 box to each of them from the
// same staging buffer.  One entry for a plain GEMM; one per GPU when a column-sharded caller wants C
// replicated (the other entries then describe the same column block inside the PEERS' C buffers,
// reached by TMA stores over NVLink — stores only: nothing is ever loaded from a peer).
constexpr int kMaxDst = 8;
struct DstMaps {
    CUtensorMap m[kMaxDst];
};

// Fused epilogue terms (all optional): out = row_scale[row] * acc + bias[col] + residual[row, col], one
// rounding at the end.  The reference's epilogue is a plain cast (wmma_utils.h:101-112).
struct EpiArgs {
    const float *row_scale;     // [M] fp32 or null
    const uint16_t *bias;       // [N] 16-bit or null
    const uint16_t *residual;   // [M, ldr] 16-bit or null (may be the output itself: each element is read by the
                                // thread that produces it, before that thread hands it to the store)
    uint32_t ldr;
    uint32_t pdl_wait;          // non-zero: griddepcontrol.wait before the first read of row_scale
    uint32_t pdl_all;           // non-zero (split-K and skinny kernels; the persistent kernel has kFlagPdl): launched
                                // under programmatic stream serialisation: let the successor start after set-up, touch
                                // no global memory before the predecessor has completed
    // Non-null: the output goes out through this address instead of the TMA stores.  It is a MULTICAST address
    // (one mapping bound to a buffer on every GPU of the group): each 16-byte multimem.st is replicated by the
    // NVLink switch into every GPU's copy, the issuing GPU's own included, so a column-sharded caller's block
    // leaves the GPU once, not once per peer.  Row pitch ld_mc elements.
    uint16_t *mc_dst;
    uint32_t ld_mc;
    __device__ __forceinline__ bool any() const { return row_scale || bias || residual; }
};

// One staged output box (ROWS x 64 or 32 columns, written with the swizzle of the matching TMA store box) goes to
// the multicast address: the warp reads it back so that 8 (or 4) lanes cover one row's contiguous bytes and
// consecutive lane groups consecutive rows, 16 bytes per lane and instruction.
template <uint32_t BOX_COLS>
__device__ __forceinline__ void mc_store_box(const uint8_t *box_gen, uint16_t *mc, uint32_t ld, uint32_t row0,
                                             uint32_t col0, uint32_t M, uint32_t N, uint32_t lane) {
    constexpr uint32_t kChunks = BOX_COLS / 8;             // 16-byte chunks per row: 8 or 4
    constexpr uint32_t kRowsPerIt = 32 / kChunks;          // rows one instruction covers: 4 or 8
    const uint32_t ch = lane % kChunks, r_in = lane / kChunks;
#pragma unroll
    for (uint32_t it = 0; it < kStoreRows / kRowsPerIt; ++it) {
        const uint32_t r = it * kRowsPerIt + r_in;
        const uint32_t sw = (BOX_COLS == 64) ? (ch ^ (r & 7u)) : (ch ^ ((r >> 1) & 3u));
        const uint4 v = *reinterpret_cast<const uint4 *>(box_gen + r * (BOX_COLS * 2u) + (sw << 4));
        if (row0 + r < M && col0 + ch * 8u < N) {
            uint16_t *dst = mc + static_cast<size_t>(row0 + r) * ld + col0 + ch * 8u;
            asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};"
                         ::"l"(dst), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
        }
    }
}

// Eight consecutive columns starting at `col` of row `row`: f[i] = f[i] * rs + bias + residual.
template <bool BF16>
__device__ __forceinline__ void epi_apply8(float (&f)[8], float rs, const EpiArgs &epi, bool row_ok, size_t row,
                                           uint32_t col) {
    float add[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) add[i] = 0.f;
    if (epi.bias) {
        const uint4 w = __ldg(reinterpret_cast<const uint4 *>(epi.bias + col));
        float lo, hi;
        unpack2<BF16>(w.x, lo, hi); add[0] = lo; add[1] = hi;
        unpack2<BF16>(w.y, lo, hi); add[2] = lo; add[3] = hi;
        unpack2<BF16>(w.z, lo, hi); add[4] = lo; add[5] = hi;
        unpack2<BF16>(w.w, lo, hi); add[6] = lo; add[7] = hi;
    }
    if (epi.residual && row_ok) {
        // plain load (not the read-only path): the residual may be the output buffer of this same kernel
        const uint4 w = *reinterpret_cast<const uint4 *>(epi.residual + row * epi.ldr + col);
        float lo, hi;
        unpack2<BF16>(w.x, lo, hi); add[0] += lo; add[1] += hi;
        unpack2<BF16>(w.y, lo, hi); add[2] += lo; add[3] += hi;
        unpack2<BF16>(w.z, lo, hi); add[4] += lo; add[5] += hi;
        unpack2<BF16>(w.w, lo, hi); add[6] += lo; add[7] += hi;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = fmaf(f[i], rs, add[i]);
}

__device__ __forceinline__ float epi_row_scale(const EpiArgs &epi, bool row_ok, size_t row) {
    if (!epi.row_scale) return 1.f;
    if (epi.pdl_wait) asm volatile("griddepcontrol.wait;" ::: "memory");
    return row_ok ? *(epi.row_scale + row) : 1.f;
}

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
                if (ctx.status) atomicCAS(ctx.status, 0, code);
                return false;
            }
        }
    }
}

// Grouped raster: tile t -> (mi, ni).  Tiles are numbered down the rows of a band
// of kGroupM tile rows first, then across the columns, band after band.
__device__ __forceinline__ void tile_coords(uint32_t kGroupM, uint32_t t, uint32_t m_tiles, uint32_t n_tiles,
                                            uint32_t &mi, uint32_t &ni, bool serpentine = false) {
    if (kGroupM & 0x10000u) {        // kFlagRasterAlongN folded into the argument: the same walk with m and n swapped
        const uint32_t g = kGroupM & 0xffffu;
        const uint32_t per_band = g * m_tiles;
        const uint32_t band = t / per_band;
        const uint32_t first_n = band * g;
        const uint32_t band_cols = min(g, n_tiles - first_n);
        const uint32_t r = t - band * per_band;
        ni = first_n + r % band_cols;
        mi = r / band_cols;
        if (serpentine && (band & 1u)) mi = m_tiles - 1 - mi;
        return;
    }
    const uint32_t per_band = kGroupM * n_tiles;
    const uint32_t band = t / per_band;
    const uint32_t first_m = band * kGroupM;
    const uint32_t band_rows = min(kGroupM, m_tiles - first_m);
    const uint32_t r = t - band * per_band;
    mi = first_m + r % band_rows;
    ni = r / band_rows;
    if (serpentine && (band & 1u)) ni = n_tiles - 1 - ni;
}

// Tail split.  With T tiles on W workers the last, partial wave keeps only T mod W workers busy for a whole
// tile time.  When that remainder is at most W/2, the remainder tiles are cut into `split` k-slices and handed to
// `split` workers each: slice 0 (the owner) keeps the tile, slices 1.. (helpers) write their fp32 partial
// accumulators to a caller-provided workspace and raise a flag; the owner's epilogue adds the partials in slice
// order (deterministic) before it rounds.  Helpers never wait for anybody and every worker runs its whole tiles
// first, so an owner only ever waits for work that is already running; its wait is bounded like every other.
//   full_tiles  tiles [0, full_tiles) are walked whole, worker-strided; a multiple of the worker count when
//               split >= 2, the tile count otherwise
//   split       0: no split; >= 2: k-slices per remainder tile (remainder * split <= workers)
//   ws          [remainder][split-1][CTA of the pair][BN/4][128 rows][4] fp32
//   flags       [remainder][split-1][CTA of the pair][epilogue warp], zero at launch
struct TailArgs {
    uint32_t full_tiles;
    uint32_t split;
    float *ws;
    uint32_t *flags;
    uint32_t *wave_sync;    // null, or a zeroed pair {arrivals, workers checked out}: the producers keep in step
    uint32_t sync_kb;       // k-blocks between two synchronisation points inside a tile (0: only at the tile's start)
    uint32_t sync_lag;      // the wait for a point comes this many k-blocks after the arrival at it
};

struct Unit {
    uint32_t tile, kb0, kb1, slice, tail_idx;
    bool valid, is_tail;
};

// The i-th piece of work of `worker`: its whole tiles first, then at most one k-slice of a remainder tile.
__device__ __forceinline__ Unit unit_at(uint32_t i, uint32_t worker, uint32_t workers, uint32_t total_tiles,
                                        uint32_t k_blocks, const TailArgs &tail) {
    Unit u;
    u.kb0 = 0;
    u.kb1 = k_blocks;
    u.slice = 0;
    u.tail_idx = 0;
    u.is_tail = false;
    u.tile = worker + i * workers;
    u.valid = u.tile < tail.full_tiles;
    if (!u.valid && tail.split >= 2 && i == tail.full_tiles / workers) {
        const uint32_t rem = total_tiles - tail.full_tiles;
        if (worker < rem * tail.split) {
            u.tail_idx = worker / tail.split;
            u.slice = worker - u.tail_idx * tail.split;
            u.tile = tail.full_tiles + u.tail_idx;
            const uint32_t per = (k_blocks + tail.split - 1) / tail.split;
            u.kb0 = min(k_blocks, u.slice * per);
            u.kb1 = min(k_blocks, u.kb0 + per);
            u.valid = true;
            u.is_tail = true;
        }
    }
    return u;
}

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// Counter of a pure timing barrier: no data is published through it, so neither side needs a fence.
__device__ __forceinline__ void red_relaxed_gpu_add(uint32_t *p, uint32_t v) {
    asm volatile("red.relaxed.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_relaxed_gpu(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_gpu(uint32_t *p, uint32_t v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Bounded wait for a helper's flag.  Returns false if the wait was abandoned.
__device__ __forceinline__ bool wait_flag(const uint32_t *flag, const WaitCtx &ctx) {
    uint64_t t0 = 0;
    uint32_t spins = 0;
    while (ld_acquire_gpu(flag) == 0u) {
        if ((++spins & 255u) == 0) {
            if (*ctx.abort_flag) return false;
            const uint64_t now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > kWaitTimeoutNs) {
                *ctx.abort_flag = 1;
                if (ctx.status) atomicCAS(ctx.status, 0, static_cast<int>(kStEpiTailFlag));
                return false;
            }
        }
    }
    return true;
}

// Waits until the counter has reached `target` (wrap-safe), for at most kSyncPatienceNs.  The counter only keeps
// workers in step, nothing is published through it, so running out of patience is not an error: the caller stops
// waiting at further points (it keeps announcing its own arrivals) and the kernel's results are the same.  This is
// also what makes the scheme safe without a cooperative launch: if part of the grid is not resident yet (another
// kernel holds some SMs), the resident workers lose one patience interval and then run unsynchronised.
constexpr uint64_t kSyncPatienceNs = 50000ull;
__device__ __forceinline__ bool wait_count_patiently(const uint32_t *counter, uint32_t target) {
    uint64_t t0 = 0;
    uint32_t spins = 0;
    while (static_cast<int32_t>(ld_relaxed_gpu(counter) - target) < 0) {
        if ((++spins & 15u) == 0) {
            const uint64_t now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > kSyncPatienceNs) return false;
        }
    }
    return true;
}

template <int CTA_GROUP, int BN, int STAGES, int MT, bool BF16>
__global__ void __launch_bounds__(MT == 2 ? kThreadsWide : kThreads, 1)
hgemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_a,
                     const __grid_constant__ CUtensorMap tm_b,
                     const __grid_constant__ DstMaps tm_c, uint32_t n_dst,
                     uint32_t M, uint32_t N, uint32_t K, uint32_t group_m, uint32_t flags, const EpiArgs epi,
                     const TailArgs tail, int *status) {
    using C = Cfg<CTA_GROUP, BN, STAGES, MT>;
    constexpr uint32_t kBlockM = kBM * CTA_GROUP;         // rows one MMA covers
    constexpr uint32_t kTileM = kBlockM * MT;

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
    if (flags & kFlagRasterAlongN) group_m |= 0x10000u;   // tile_coords reads the raster direction from here
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
            mbar_init(bar_acc_empty + a * 8, (MT == 2 ? kEpiWarpsWide : kEpiWarps) * CTA_GROUP);   // one arrive per epilogue warp
        }
        *abort_flag = 0;
        fence_mbar_init();
        prefetch_tensormap(&tm_a);
        prefetch_tensormap(&tm_b);
        for (uint32_t d = 0; d < n_dst; ++d) prefetch_tensormap(&tm_c.m[d]);
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
    const bool pdl = (flags & kFlagPdl) != 0;
    if (pdl) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // -------------------------------------------------------------- roles ----
    if (warp == 0) {
        if (lane == 0) {
            // ===== producer =====
            if (pdl) asm volatile("griddepcontrol.wait;" ::: "memory");
            // In a pair, both CTAs' loads complete on the LEADER's full[s].
            const uint32_t full0 = (CTA_GROUP == 2) ? mapa(bar_full, 0) : bar_full;
            const uint32_t peer_empty0 = (CTA_GROUP == 2) ? mapa(bar_empty, 1) : 0u;
            uint32_t stage = 0, phase = 0, sync_target = 0, sync_wait_at = 0xffffffffu;
            bool ok = true, sync_waits = true;
            const bool hint_a = (flags & kFlagAEvictLast) != 0;
            const bool hint_b = (flags & (kFlagBEvictFirst | kFlagBEvictLast)) != 0;
            const uint64_t pol_a = l2_policy_evict_last();
            const uint64_t pol_b = (flags & kFlagBEvictFirst) ? l2_policy_evict_first() : l2_policy_evict_last();
            for (uint32_t it = 0; ok; ++it) {
                const Unit u = unit_at(it, worker, workers, total_tiles, k_blocks, tail);
                if (!u.valid) break;
                uint32_t mi, ni;
                tile_coords(group_m, u.tile, m_tiles, n_tiles, mi, ni, (flags & kFlagSerpentine) != 0);
                const int32_t row_a = static_cast<int32_t>(mi * kTileM + rank * kBM);    // + mt * kBlockM
                const int32_t row_b = static_cast<int32_t>(ni * BN + rank * C::kBRows);
                for (uint32_t kb = u.kb0; kb < u.kb1; ++kb) {
                    if (tail.wave_sync != nullptr && leader) {
                        // Synchronisation points of the producers (the first k-block of every tile and every
                        // sync_kb-th after it): a worker announces that it has reached the point, and sync_lag
                        // k-blocks later waits until every worker of this wave of tiles has.  Workers that share an
                        // A or a B panel therefore ask for the same k-block within a few k-block times of each
                        // other: one's fetch from DRAM is the others' L2 hit, or is merged with theirs on the way to
                        // L2.  The lag hides the counter's round trip behind loads that are already allowed.  (The
                        // peer CTA's producer is paced by the relayed empty[s].)
                        const uint32_t rel = kb - u.kb0;
                        if (rel == 0 || (tail.sync_kb != 0 && rel % tail.sync_kb == 0)) {
                            red_relaxed_gpu_add(tail.wave_sync, 1u);
                            sync_target += min(workers, total_tiles - it * workers);
                            sync_wait_at = kb + tail.sync_lag;
                        }
                        // (letting a wait end when all but 4-37 workers had arrived was measured: no gain)
                        if (kb == sync_wait_at && sync_waits) sync_waits = wait_count_patiently(tail.wave_sync, sync_target);
                    }
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
                    const uint32_t fb = (CTA_GROUP == 2) ? full0 + stage * 8 : bar_full + stage * 8;
#pragma unroll
                    for (uint32_t mt = 0; mt < MT; ++mt) {
                        const uint32_t da = dst_a + mt * C::kABox;
                        const int32_t ra = row_a + static_cast<int32_t>(mt * kBlockM);
                        if (hint_a) {
                            if constexpr (CTA_GROUP == 2) tma_load_2d_pair_hint(da, &tm_a, fb, kx, ra, pol_a);
                            else tma_load_2d_hint(da, &tm_a, fb, kx, ra, pol_a);
                        } else {
                            if constexpr (CTA_GROUP == 2) tma_load_2d_pair(da, &tm_a, fb, kx, ra);
                            else tma_load_2d(da, &tm_a, fb, kx, ra);
                        }
                    }
                    if (hint_b) {
                        if constexpr (CTA_GROUP == 2) tma_load_2d_pair_hint(dst_b, &tm_b, fb, kx, row_b, pol_b);
                        else tma_load_2d_hint(dst_b, &tm_b, fb, kx, row_b, pol_b);
                    } else {
                        if constexpr (CTA_GROUP == 2) tma_load_2d_pair(dst_b, &tm_b, fb, kx, row_b);
                        else tma_load_2d(dst_b, &tm_b, fb, kx, row_b);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            // ===== MMA issuer =====
            constexpr uint32_t idesc = instr_desc_f16(BF16, kBlockM, BN);
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            for (uint32_t it = 0; ok; ++it) {
                const Unit u = unit_at(it, worker, workers, total_tiles, k_blocks, tail);
                if (!u.valid) break;
                if constexpr (MT == 1) {
                    // the epilogue must have drained this accumulator (passes at once the first two times)
                    ok = wait_bar(bar_acc_empty + acc * 8, acc_phase ^ 1u, ctx, kStMmaAccEmpty);
                    if (!ok) break;
                    tc_fence_after_sync();
                }
                for (uint32_t kb = u.kb0; kb < u.kb1; ++kb) {
                    ok = wait_bar(bar_full + stage * 8, phase, ctx, kStMmaFull);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint64_t db = smem_desc_k_sw128(smem_base + C::kOffB + stage * C::kBBytes);
#pragma unroll
                    for (uint32_t mt = 0; mt < MT; ++mt) {
                        if constexpr (MT == 2) {
                            // Row block mt accumulates into accumulator mt.  The previous tile's epilogue drains
                            // accumulator 0 first: block 0 of this tile restarts while accumulator 1 still drains.
                            if (kb == u.kb0) {
                                ok = wait_bar(bar_acc_empty + mt * 8, acc_phase ^ 1u, ctx, kStMmaAccEmpty);
                                if (!ok) break;
                                tc_fence_after_sync();
                            }
                        }
                        const uint32_t tmem_d = tmem_base + (MT == 2 ? mt : acc) * BN;
                        const uint64_t da = smem_desc_k_sw128(smem_base + C::kOffA + stage * C::kABytes + mt * C::kABox);
#pragma unroll
                        for (uint32_t k = 0; k < kBK / kUmmaK; ++k) {
                            // 16 elements of k = 32 bytes inside the 128-byte swizzle row = +2 in the >>4 address field
                            umma_f16<CTA_GROUP>(tmem_d, da + 2 * k, db + 2 * k, idesc,
                                                (kb != u.kb0 || k != 0u) ? 1u : 0u);
                        }
                    }
                    if (!ok) break;
                    umma_commit<CTA_GROUP>(bar_empty + stage * 8);   // stage free once these MMAs are done
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
#ifdef PG_TEST_SHORT_WAIT
                const bool withhold = worker == 0 && it == 0 &&
                                      *reinterpret_cast<volatile int *>(&g_test_withhold_acc_commit) != 0;
#else
                constexpr bool withhold = false;
#endif
                if constexpr (MT == 2) {
                    if (!withhold) umma_commit<CTA_GROUP>(bar_acc_full);            // both accumulators complete
                    acc_phase ^= 1u;
                } else {
                    if (!withhold) umma_commit<CTA_GROUP>(bar_acc_full + acc * 8);  // accumulator complete
                    if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
                }
            }
        }
        __syncwarp();
    } else {
        if (pdl) asm volatile("griddepcontrol.wait;" ::: "memory");
        if constexpr (MT == 2) {
            // ===== epilogue, two row blocks per CTA: 8 warps =====
            // Warp w reads lane quarter w % 4 (the hardware rule) and column half (w - 2) / 4 of each accumulator:
            // 32 rows x 128 columns = 128 registers per thread.  One round of loads empties an accumulator; it goes
            // back to the MMA warp before anything is converted or stored, accumulator 0 first, so the next tile's
            // first row block restarts while accumulator 1 is still being read.
            const uint32_t q = warp & 3u;
            const uint32_t e = warp - 2u;                 // 0..7: 4 KiB of staging each = two 32 x 32 boxes
            const uint32_t half = e >> 2;                 // columns [128 * half, 128 * half + 128)
            const uint32_t sbuf = smem_base + C::kOffC + e * kStageBufBytes;
            uint8_t *sbuf_gen = smem_gen + C::kOffC + e * kStageBufBytes;
            const uint32_t acc_empty_leader = mapa(bar_acc_empty, 0);
            const uint32_t peer_acc_full = mapa(bar_acc_full, 1);
            uint32_t acc_phase = 0, nbuf = 0;
            bool ok = true;
            const uint64_t pol_store = l2_policy_evict_first();
            const bool fused = epi.any();
            const bool wide_boxes = n_dst > 1 || epi.mc_dst != nullptr;      // the launcher encodes 64-column boxes then
            for (uint32_t it = 0; ok; ++it) {
                const Unit u = unit_at(it, worker, workers, total_tiles, k_blocks, tail);
                if (!u.valid) break;
                uint32_t mi, ni;
                tile_coords(group_m, u.tile, m_tiles, n_tiles, mi, ni, (flags & kFlagSerpentine) != 0);
                ok = wait_bar(bar_acc_full, acc_phase, ctx, kStEpiAccFull);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                if (leader && e == 0 && lane == 0) mbar_arrive_cluster(peer_acc_full);   // relay to the peer CTA
                tc_fence_after_sync();
    #pragma unroll 1
                for (uint32_t mt = 0; mt < 2; ++mt) {
                    const uint32_t row0 = mi * kTileM + mt * kBlockM + rank * kBM + q * 32u;
                    const uint32_t taddr = tmem_base + mt * BN + half * 128u + ((q * 32u) << 16);
                    uint32_t v[4][32];
                    tmem_ld_32x32b_x32(taddr, v[0]);
                    tmem_ld_32x32b_x32(taddr + 32u, v[1]);
                    tmem_ld_32x32b_x32(taddr + 64u, v[2]);
                    tmem_ld_32x32b_x32(taddr + 96u, v[3]);
                    tmem_ld_wait();
                    // this warp's part of accumulator mt is in registers: hand it back
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(acc_empty_leader + mt * 8);
                    const bool row_ok = row0 + lane < M;
                    const float rs = fused ? epi_row_scale(epi, row_ok, row0 + lane) : 1.f;
                    if (wide_boxes) {
                        // Stores that cross NVLink (peer destinations, or a multicast one): two 32 x 64 boxes with
                        // 128-byte rows over the warp's whole staging area, one at a time.  Half as many, twice as
                        // long writes arrive at every peer as with the 64-byte rows of the 32 x 32 boxes.
#pragma unroll
                        for (uint32_t cp = 0; cp < 2; ++cp) {
                            const uint32_t col0 = ni * BN + half * 128u + cp * 64u;
                            uint4 o[8];
#pragma unroll
                            for (uint32_t c = 0; c < 8; ++c) {
                                const uint32_t *src = &v[2u * cp + (c >> 2)][(c & 3u) * 8u];
                                o[c].x = pack2<BF16>(__uint_as_float(src[0]), __uint_as_float(src[1]));
                                o[c].y = pack2<BF16>(__uint_as_float(src[2]), __uint_as_float(src[3]));
                                o[c].z = pack2<BF16>(__uint_as_float(src[4]), __uint_as_float(src[5]));
                                o[c].w = pack2<BF16>(__uint_as_float(src[6]), __uint_as_float(src[7]));
                            }
                            // the previous store from this area must have finished reading it
                            if (lane == 0) bulk_wait_group_read<0>();
                            __syncwarp();
                            // row `lane` = 128 bytes, chunk c at position c ^ (row % 8)  (128-byte swizzle)
#pragma unroll
                            for (uint32_t c = 0; c < 8; ++c)
                                *reinterpret_cast<uint4 *>(sbuf_gen + lane * 128u + ((c ^ (lane & 7u)) << 4)) = o[c];
                            fence_proxy_async_smem();
                            __syncwarp();
                            if (epi.mc_dst != nullptr) {
                                mc_store_box<64>(sbuf_gen, epi.mc_dst, epi.ld_mc, row0, col0, M, N, lane);
                            } else if (lane == 0) {
                                if (row0 < M && col0 < N) {
                                    for (uint32_t d = 0; d < n_dst; ++d)
                                        tma_store_2d(&tm_c.m[d], sbuf, static_cast<int32_t>(col0),
                                                     static_cast<int32_t>(row0));
                                }
                                bulk_commit_group();
                            }
                        }
                        continue;
                    }
#pragma unroll
                    for (uint32_t cb = 0; cb < 4; ++cb) {       // four 32 x 32 boxes, two staging buffers in turn
                        const uint32_t col0 = ni * BN + half * 128u + cb * 32u;
                        if (fused) {
#pragma unroll
                            for (uint32_t c = 0; c < 4; ++c) {
                                if (col0 + c * 8u < N) {      // n is a multiple of 8: a group of 8 columns is in or out
                                    float f[8];
#pragma unroll
                                    for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(v[cb][c * 8u + i]);
                                    epi_apply8<BF16>(f, rs, epi, row_ok, row0 + lane, col0 + c * 8u);
#pragma unroll
                                    for (int i = 0; i < 8; ++i) v[cb][c * 8u + i] = __float_as_uint(f[i]);
                                }
                            }
                        }
                        uint4 o[4];
#pragma unroll
                        for (uint32_t c = 0; c < 4; ++c) {
                            const uint32_t *src = &v[cb][c * 8u];
                            o[c].x = pack2<BF16>(__uint_as_float(src[0]), __uint_as_float(src[1]));
                            o[c].y = pack2<BF16>(__uint_as_float(src[2]), __uint_as_float(src[3]));
                            o[c].z = pack2<BF16>(__uint_as_float(src[4]), __uint_as_float(src[5]));
                            o[c].w = pack2<BF16>(__uint_as_float(src[6]), __uint_as_float(src[7]));
                        }
                        // the store issued two boxes ago from this buffer must have finished reading it
                        if (lane == 0) bulk_wait_group_read<1>();
                        __syncwarp();
                        const uint32_t box = sbuf + nbuf * (kStageBufBytes / 2);
                        uint8_t *box_gen = sbuf_gen + nbuf * (kStageBufBytes / 2);
                        // row `lane` = 64 bytes, 4 chunks of 16 bytes, chunk c stored at position c ^ ((row / 2) % 4)
                        // (the 64-byte swizzle: address bits 4-5 xor bits 7-8)
#pragma unroll
                        for (uint32_t c = 0; c < 4; ++c)
                            *reinterpret_cast<uint4 *>(box_gen + lane * 64u + ((c ^ ((lane >> 1) & 3u)) << 4)) = o[c];
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (epi.mc_dst != nullptr) {
                            mc_store_box<32>(box_gen, epi.mc_dst, epi.ld_mc, row0, col0, M, N, lane);
                        } else if (lane == 0) {
                            if (row0 < M && col0 < N) {
                                for (uint32_t d = 0; d < n_dst; ++d) {
                                    if (flags & kFlagStoreEvictFirst)
                                        tma_store_2d_hint(&tm_c.m[d], box, static_cast<int32_t>(col0),
                                                          static_cast<int32_t>(row0), pol_store);
                                    else
                                        tma_store_2d(&tm_c.m[d], box, static_cast<int32_t>(col0),
                                                     static_cast<int32_t>(row0));
                                }
                            }
                            bulk_commit_group();
                        }
                        nbuf ^= 1u;
                    }
                }
                acc_phase ^= 1u;
            }
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
            for (uint32_t it = 0; ok; ++it) {
                const Unit u = unit_at(it, worker, workers, total_tiles, k_blocks, tail);
                if (!u.valid) break;
                uint32_t mi, ni;
                tile_coords(group_m, u.tile, m_tiles, n_tiles, mi, ni, (flags & kFlagSerpentine) != 0);
                // All 32 lanes probe: a failed try_wait parks the warp in hardware, so this costs nothing (a
                // one-lane poll with __nanosleep back-off executed 40 % MORE instructions and ran 0.7 % slower).
                ok = wait_bar(bar_acc_full + acc * 8, acc_phase, ctx, kStEpiAccFull);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                if constexpr (CTA_GROUP == 2) {
                    if (leader && e == 0 && lane == 0) mbar_arrive_cluster(peer_acc_full + acc * 8);  // relay
                }
                tc_fence_after_sync();
                const uint32_t row0 = mi * kTileM + rank * kBM + q * 32u;   // first row of this warp's slab
                const uint32_t taddr = tmem_base + acc * BN + ((q * 32u) << 16);
                const bool fused = epi.any();
                const bool row_ok = row0 + lane < M;
                const float rs = fused ? epi_row_scale(epi, row_ok, row0 + lane) : 1.f;
                // k-slices of a remainder tile: where this warp's rows of slice j live in the workspace, and its flag
                constexpr uint32_t kPartFloats = kBM * BN;                  // one CTA's partial tile
                const uint32_t n_parts = (u.is_tail && u.slice == 0) ? tail.split - 1u : 0u;
                const uint32_t part0 = u.is_tail ? (u.tail_idx * (tail.split - 1u)) * CTA_GROUP + rank : 0u;   // slice 1 of this tile
                if (u.is_tail && u.slice > 0) {
                    // ===== helper: fp32 partial sums to the workspace, then the flag =====
                    const uint32_t part = part0 + (u.slice - 1u) * CTA_GROUP;
                    float4 *dst = reinterpret_cast<float4 *>(tail.ws + static_cast<size_t>(part) * kPartFloats) +
                                  (q * 32u + lane);
    #pragma unroll 1
                    for (uint32_t ch = 0; ch < BN / kStoreCols; ++ch) {
                        uint32_t v[2][32];
                        tmem_ld_32x32b_x32(taddr + ch * kStoreCols, v[0]);
                        tmem_ld_32x32b_x32(taddr + ch * kStoreCols + 32u, v[1]);
                        tmem_ld_wait();
    #pragma unroll
                        for (uint32_t c4 = 0; c4 < 16; ++c4) {      // column group c4 of this chunk: [group][row][4]
                            const uint32_t *src = &v[c4 >> 3][(c4 & 7u) * 4u];
                            dst[(ch * 16u + c4) * kBM] = make_float4(__uint_as_float(src[0]), __uint_as_float(src[1]),
                                                                     __uint_as_float(src[2]), __uint_as_float(src[3]));
                        }
                    }
                    tc_fence_before_sync();
                    __threadfence();
                    __syncwarp();
                    if (lane == 0) {
                        if constexpr (CTA_GROUP == 2) mbar_arrive_cluster(acc_empty_leader + acc * 8);
                        else mbar_arrive(bar_acc_empty + acc * 8);
                        st_release_gpu(tail.flags + part * kEpiWarps + e, 1u);
                    }
                    if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
                    continue;
                }
                if (n_parts) {
                    // ===== owner: the helpers' partial sums must have landed =====
                    for (uint32_t j = 0; ok && j < n_parts; ++j)
                        ok = wait_flag(tail.flags + (part0 + j * CTA_GROUP) * kEpiWarps + e, ctx);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                }
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
                    for (uint32_t j = 0; j < n_parts; ++j) {      // slice order: deterministic
                        const float4 *src = reinterpret_cast<const float4 *>(
                                                tail.ws + static_cast<size_t>(part0 + j * CTA_GROUP) * kPartFloats) +
                                            (q * 32u + lane);
    #pragma unroll
                        for (uint32_t c4 = 0; c4 < 16; ++c4) {
                            const float4 p = __ldcg(src + (ch * 16u + c4) * kBM);
                            uint32_t *d = &v[c4 >> 3][(c4 & 7u) * 4u];
                            d[0] = __float_as_uint(__uint_as_float(d[0]) + p.x);
                            d[1] = __float_as_uint(__uint_as_float(d[1]) + p.y);
                            d[2] = __float_as_uint(__uint_as_float(d[2]) + p.z);
                            d[3] = __float_as_uint(__uint_as_float(d[3]) + p.w);
                        }
                    }
                    // the store issued two chunks ago from this buffer must have finished reading it
                    if (lane == 0) bulk_wait_group_read<1>();
                    __syncwarp();
                    const uint32_t sbuf = buf0 + nbuf * kStageBufBytes;
                    uint8_t *sbuf_gen = buf0_gen + nbuf * kStageBufBytes;
                    const uint32_t col0 = ni * BN + ch * kStoreCols;
                    if (fused) {
    #pragma unroll
                        for (uint32_t c = 0; c < 8; ++c) {
                            if (col0 + c * 8u < N) {      // n is a multiple of 8: a group of 8 columns is in or out
                                float f[8];
    #pragma unroll
                                for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(v[c >> 2][(c & 3u) * 8u + i]);
                                epi_apply8<BF16>(f, rs, epi, row_ok, row0 + lane, col0 + c * 8u);
    #pragma unroll
                                for (int i = 0; i < 8; ++i) v[c >> 2][(c & 3u) * 8u + i] = __float_as_uint(f[i]);
                            }
                        }
                    }
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
                    if (epi.mc_dst != nullptr) {
                        mc_store_box<64>(sbuf_gen, epi.mc_dst, epi.ld_mc, row0, col0, M, N, lane);
                    } else if (lane == 0) {
                        if (row0 < M && col0 < N) {
                            for (uint32_t d = 0; d < n_dst; ++d) {
                                if (flags & kFlagStoreEvictFirst)
                                    tma_store_2d_hint(&tm_c.m[d], sbuf, static_cast<int32_t>(col0),
                                                      static_cast<int32_t>(row0), pol_store);
                                else
                                    tma_store_2d(&tm_c.m[d], sbuf, static_cast<int32_t>(col0),
                                                 static_cast<int32_t>(row0));
                            }
                        }
                        bulk_commit_group();
                    }
                    nbuf ^= 1u;
                }
                if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
            }
        }
        // Shared memory must outlive the stores that read it; their global writes are complete when the grid is.
        // With peer destinations the thread waits for the writes themselves, to stay on the safe side of NVLink.
        if (lane == 0) {
            if (n_dst == 1) bulk_wait_group_read<0>();
            else bulk_wait_group<0>();
        }
        if (epi.mc_dst != nullptr) __threadfence_system();     // the multicast stores are performed before the grid ends
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
    // Producer synchronisation: the counter pair is handed back zeroed.  Every worker's producer has left its loop
    // before its CTA gets here, so when the last worker checks out nobody reads the counter any more.
    if (tail.wave_sync != nullptr && leader && threadIdx.x == 0) {
        if (atomicAdd(tail.wave_sync + 1, 1u) == workers - 1u) {
            tail.wave_sync[0] = 0u;
            tail.wave_sync[1] = 0u;
            __threadfence();
        }
    }
}

// ---------------------------------------------------------------- split-K ----
//
// Shapes with few output tiles (small m, moderate n) cannot fill 148 SMs with one CTA per tile, and
// their k loop is long.  Here a thread-block CLUSTER of S CTAs shares one 128 x BN tile: CTA r
// accumulates k-blocks [r*per, (r+1)*per) in its own tensor memory, then the partial accumulators
// are combined without any global scratch, reduce-scatter style through distributed shared memory:
//   send    CTA r reads its accumulator and writes, for every peer p, the columns p owns
//           (BN/S of them) into slot r of p's receive buffer (st.shared::cluster);
//   barrier one cluster barrier (release/acquire) makes all slots visible;
//   reduce  CTA r adds its own slice (read again from tensor memory) and the S-1 received slices
//           in rank order (deterministic), rounds, and stores its BN/S columns with 16-byte stores.
// Not persistent: one cluster per tile, S in {2, 4, 8}.
template <int BN, int STAGES>
struct SkCfg {
    static constexpr uint32_t kABytes = kBM * kBK * 2;
    static constexpr uint32_t kBBytes = BN * kBK * 2;
    static constexpr uint32_t kStageBytes = kABytes + kBBytes;
    static constexpr uint32_t kTmemCols = BN;
    static constexpr uint32_t kOffA = 0;
    static constexpr uint32_t kOffB = kOffA + STAGES * kABytes;
    static constexpr uint32_t kOffRecv = kOffB + STAGES * kBBytes;     // [S slots][BN/S/4][128 rows][4] fp32: a warp's 32
                                                                       // rows are 32 consecutive 16-byte words
    static constexpr uint32_t kOffBar = kOffRecv + kBM * BN * 4;       // full[STAGES], empty[STAGES], acc_full
    static constexpr uint32_t kNumBars = 2 * STAGES + 1;
    static constexpr uint32_t kOffMisc = kOffBar + kNumBars * 8;
    static constexpr uint32_t kSmemBytes = kOffMisc + 16 + 1024;
    static_assert(kTmemCols == 32 || kTmemCols == 64 || kTmemCols == 128 || kTmemCols == 256, "tmem columns");
    static_assert(kSmemBytes <= 232448, "exceeds 227 KiB of shared memory");
};

template <int BN, int STAGES, bool BF16>
__global__ void __launch_bounds__(kThreads, 1)
hgemm_splitk_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                    uint16_t *c, uint32_t ldc, uint32_t M, uint32_t N, uint32_t K, const EpiArgs epi, int *status) {
    using C = SkCfg<BN, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

    const uint32_t warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t S = cluster_nctarank();
    const uint32_t rank = cluster_ctarank();
    const uint32_t W = BN / S;                       // columns each CTA finally owns (>= 8)

    const uint32_t bar_full = smem_base + C::kOffBar;
    const uint32_t bar_empty = bar_full + STAGES * 8;
    const uint32_t bar_acc_full = bar_empty + STAGES * 8;
    const uint32_t tmem_slot = smem_base + C::kOffMisc;
    volatile uint32_t *tmem_slot_gen = reinterpret_cast<volatile uint32_t *>(smem_gen + C::kOffMisc);
    volatile uint32_t *abort_flag = tmem_slot_gen + 1;
    const WaitCtx ctx{abort_flag, status};

    const uint32_t m_tiles = (M + kBM - 1) / kBM;
    const uint32_t tile = blockIdx.x / S;
    const uint32_t mi = tile % m_tiles, ni = tile / m_tiles;
    const uint32_t k_blocks = (K + kBK - 1) / kBK;
    const uint32_t per = (k_blocks + S - 1) / S;
    const uint32_t kb0 = min(k_blocks, rank * per), kb1 = min(k_blocks, kb0 + per);
    const bool has_k = kb1 > kb0;                    // an empty slice contributes zeros

    if (warp == 0 && lane == 0) {
        for (uint32_t s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + s * 8, 1);
            mbar_init(bar_empty + s * 8, 1);
        }
        mbar_init(bar_acc_full, 1);
        *abort_flag = 0;
        fence_mbar_init();
        prefetch_tensormap(&tm_a);
        prefetch_tensormap(&tm_b);
    }
    if (warp == 1) {
        tmem_alloc<1>(tmem_slot, C::kTmemCols);
        tmem_relinquish<1>();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_arrive();       // every CTA of the cluster is running before anyone writes into its shared memory
    cluster_wait();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot_gen;
    if (epi.pdl_all) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0) {
        if (lane == 0) {
            if (epi.pdl_all) asm volatile("griddepcontrol.wait;" ::: "memory");
            uint32_t stage = 0, phase = 0;
            // the weights pass through once (evict first); the activations are what every CTA re-reads (evict last)
            const uint64_t pol_stream = l2_policy_evict_first(), pol_keep = l2_policy_evict_last();
            for (uint32_t kb = kb0; kb < kb1; ++kb) {
                if (!wait_bar(bar_empty + stage * 8, phase ^ 1u, ctx, kStProducerEmpty)) break;
                mbar_arrive_expect_tx(bar_full + stage * 8, C::kStageBytes);
                const int32_t kx = static_cast<int32_t>(kb * kBK);
                tma_load_2d_hint(smem_base + C::kOffA + stage * C::kABytes, &tm_a, bar_full + stage * 8, kx,
                                 static_cast<int32_t>(mi * kBM), pol_keep);
                tma_load_2d_hint(smem_base + C::kOffB + stage * C::kBBytes, &tm_b, bar_full + stage * 8, kx,
                                 static_cast<int32_t>(ni * BN), pol_stream);
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0 && has_k) {
            constexpr uint32_t idesc = instr_desc_f16(BF16, kBM, BN);
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (uint32_t kb = kb0; kb < kb1; ++kb) {
                ok = wait_bar(bar_full + stage * 8, phase, ctx, kStMmaFull);
                if (!ok) break;
                tc_fence_after_sync();
                const uint64_t da = smem_desc_k_sw128(smem_base + C::kOffA + stage * C::kABytes);
                const uint64_t db = smem_desc_k_sw128(smem_base + C::kOffB + stage * C::kBBytes);
#pragma unroll
                for (uint32_t k = 0; k < kBK / kUmmaK; ++k)
                    umma_f16<1>(tmem_base, da + 2 * k, db + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                umma_commit<1>(bar_empty + stage * 8);
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
            if (ok) umma_commit<1>(bar_acc_full);
        }
        __syncwarp();
    } else {
        // ===== send: my partial sums of the columns each peer owns go to that peer =====
        const uint32_t q = warp & 3u;
        const uint32_t row = q * 32u + lane;                       // accumulator lane = tile row
        bool ok = true;
        if (has_k) {
            ok = wait_bar(bar_acc_full, 0, ctx, kStEpiAccFull);
            ok = __all_sync(0xffffffffu, ok);
            tc_fence_after_sync();
        }
        const uint32_t taddr = tmem_base + ((q * 32u) << 16);
        const uint32_t recv_local = smem_base + C::kOffRecv;
#pragma unroll 1
        for (uint32_t ch = 0; ch < BN / 32; ++ch) {
            uint32_t v[32];
            if (has_k && ok) {
                tmem_ld_32x32b_x32(taddr + ch * 32u, v);
                tmem_ld_wait();
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = 0u;
            }
#pragma unroll
            for (uint32_t j = 0; j < 8; ++j) {
                const uint32_t col = ch * 32u + 4u * j;
                const uint32_t p = col / W;
                if (p != rank) {
                    const uint32_t dst = recv_local + ((rank * (W / 4) + ((col - p * W) >> 2)) * kBM + row) * 16u;
                    st_cluster_v4(mapa(dst, p), __uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                  __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
                }
            }
        }
        tc_fence_before_sync();
    }

    // all partial slices delivered (every thread of every CTA of the cluster takes part)
    __syncwarp();
    cluster_arrive();
    cluster_wait();

    if (warp >= 2) {
        // ===== reduce my W columns and store them =====
        if (epi.pdl_all) asm volatile("griddepcontrol.wait;" ::: "memory");
        const uint32_t q = warp & 3u;
        const uint32_t row = q * 32u + lane;
        const uint32_t grow = mi * kBM + row;
        const uint32_t taddr = tmem_base + ((q * 32u) << 16) + rank * W;
        const float *recv = reinterpret_cast<const float *>(smem_gen + C::kOffRecv);
        tc_fence_after_sync();
        const bool acc_ok = has_k && (*abort_flag == 0);
        const bool fused = epi.any();
        const float rs = fused ? epi_row_scale(epi, grow < M, grow) : 1.f;
#pragma unroll 1
        for (uint32_t g0 = 0; g0 < W / 8; g0 += 4) {           // up to 32 columns per round of tensor-memory loads
            const uint32_t ng = min(4u, W / 8 - g0);
            uint32_t o[32];
            if (acc_ok) {
                if (ng == 4) {
                    tmem_ld_32x32b_x32(taddr + 8u * g0, o);
                } else {
                    for (uint32_t gg = 0; gg < ng; ++gg)
                        tmem_ld_32x32b_x8(taddr + 8u * (g0 + gg), *reinterpret_cast<uint32_t(*)[8]>(&o[8 * gg]));
                }
                tmem_ld_wait();
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) o[i] = 0u;
            }
#pragma unroll
            for (uint32_t gg = 0; gg < 4; ++gg) {
                if (gg < ng) {
                    const uint32_t g = g0 + gg;
                    float f[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(o[8 * gg + i]);
                    for (uint32_t r2 = 0; r2 < S; ++r2) {
                        if (r2 == rank) continue;
                        const float4 *src = reinterpret_cast<const float4 *>(recv) + (r2 * (W / 4) + 2u * g) * kBM + row;
                        const float4 a = src[0], b = src[kBM];
                        f[0] += a.x; f[1] += a.y; f[2] += a.z; f[3] += a.w;
                        f[4] += b.x; f[5] += b.y; f[6] += b.z; f[7] += b.w;
                    }
                    const uint32_t gcol = ni * BN + rank * W + 8u * g;
                    if (grow < M && gcol < N) {
                        if (fused) epi_apply8<BF16>(f, rs, epi, true, grow, gcol);
                        uint4 out;
                        out.x = pack2<BF16>(f[0], f[1]);
                        out.y = pack2<BF16>(f[2], f[3]);
                        out.z = pack2<BF16>(f[4], f[5]);
                        out.w = pack2<BF16>(f[6], f[7]);
                        *reinterpret_cast<uint4 *>(c + static_cast<size_t>(grow) * ldc + gcol) = out;
                    }
                }
            }
        }
        tc_fence_before_sync();
    }
    __syncthreads();
    if (*abort_flag) __nanosleep(50000);
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc<1>(tmem_base, C::kTmemCols);
    }
}

// ------------------------------------------------------- pair split-K ----
//
// One tile row (64 < m <= 128) against a weight matrix: pure weight streaming, and with one CTA per
// 128 x BN tile two thirds of what an SM pulls from L2 is the SHARED A panel (every tile re-reads all of
// it).  Here a CTA PAIR owns the 128 x BN tile (tcgen05 cta_group::2 at M = 128): each CTA loads only
// its own 64 rows of A and BN/2 rows of B, so the A panel crosses from L2 half as often — without any
// multicast.  A cluster holds S pairs (S = 1 or 2; cluster of 2S CTAs): pair p accumulates k-blocks
// [p*per, (p+1)*per), and the partial sums are combined through distributed shared memory as in the
// cluster split-K kernel above, between the two CTAs that hold the same rows.
//
// Tensor-memory layout of this MMA shape (read out with a one-hot probe): CTA h of the pair holds rows
// 64h..64h+63 of the tile; lanes 0-63 carry those rows for columns [0, BN/2), lanes 64-127 the same rows
// for columns [BN/2, BN), both at tensor-memory columns 0..BN/2-1.  So an accumulator takes BN/2 columns,
// and epilogue warp q (lane quarter q) reads rows 32*(q&1)..+31, column half q>>1.
//
// ROWS = rows of A per CTA.  64: the shape above (one tile row, 64 < m <= 128).  128: the ordinary M = 256 pair MMA
// (lane = row, BN tensor-memory columns), for problems of a few 256 x BN tiles (128 < m <= 512 or so) that would
// leave most SM pairs idle: two pairs per cluster share a tile's k range, with the operand traffic per flop of the
// 256 x 256 pair tile.  At most two pairs per cluster: a CTA receives from one other pair only, so the receive buffer
// is half a tile.
template <int ROWS, int BN, int STAGES>
struct PsCfg {
    static constexpr uint32_t kARows = ROWS;
    static constexpr uint32_t kABytes = kARows * kBK * 2;          // 8 or 16 KiB
    static constexpr uint32_t kBRows = BN / 2;
    static constexpr uint32_t kBBytes = kBRows * kBK * 2;
    static constexpr uint32_t kStageBytes = kABytes + kBBytes;
    static constexpr uint32_t kHalfCols = (ROWS == 64) ? BN / 2 : BN;  // columns one epilogue warp reads = tmem columns
    static constexpr uint32_t kTmemCols = kHalfCols;
    static constexpr uint32_t kOffA = 0;
    static constexpr uint32_t kOffB = kOffA + STAGES * kABytes;
    static constexpr uint32_t kOffRecv = kOffB + STAGES * kBBytes;     // [BN/2/4][ROWS][4] fp32 from the other pair (S = 2)
    static constexpr uint32_t kOffBar = kOffRecv + kARows * (BN / 2) * 4;   // full[STAGES], empty[STAGES], acc_full
    static constexpr uint32_t kNumBars = 2 * STAGES + 1;
    static constexpr uint32_t kOffMisc = kOffBar + kNumBars * 8;
    static constexpr uint32_t kSmemBytes = kOffMisc + 16 + 1024;
    static_assert(kTmemCols == 64 || kTmemCols == 128 || kTmemCols == 256, "tmem columns");
    static_assert(ROWS == 64 || ROWS == 128, "rows of A per CTA");
    static_assert(kSmemBytes <= 232448, "exceeds 227 KiB of shared memory");
};

template <int ROWS, int BN, int STAGES, bool BF16>
__global__ void __launch_bounds__(kThreads, 1)
hgemm_pair_splitk_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                         uint16_t *c, uint32_t ldc, uint32_t M, uint32_t N, uint32_t K, const EpiArgs epi,
                         int *status) {
    using C = PsCfg<ROWS, BN, STAGES>;
    constexpr uint32_t HW = C::kHalfCols;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

    const uint32_t warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t rank = cluster_ctarank();
    const uint32_t S = cluster_nctarank() / 2;       // pairs per cluster = k-slices (1 or 2)
    const uint32_t pair = rank >> 1;                 // k-slice of this CTA's pair
    const uint32_t half = rank & 1u;                 // which 64 rows of A / which BN/2 rows of B this CTA loads
    const bool leader = half == 0;
    const uint32_t W = BN / S;                       // columns each pair finally owns (>= 64)

    const uint32_t bar_full = smem_base + C::kOffBar;
    const uint32_t bar_empty = bar_full + STAGES * 8;
    const uint32_t bar_acc_full = bar_empty + STAGES * 8;
    const uint32_t tmem_slot = smem_base + C::kOffMisc;
    volatile uint32_t *tmem_slot_gen = reinterpret_cast<volatile uint32_t *>(smem_gen + C::kOffMisc);
    volatile uint32_t *abort_flag = tmem_slot_gen + 1;
    const WaitCtx ctx{abort_flag, status};

    const uint32_t m_tiles = (M + 2 * ROWS - 1) / (2 * ROWS);
    const uint32_t tile = blockIdx.x / (2 * S);
    const uint32_t mi = tile % m_tiles, ni = tile / m_tiles;
    const uint32_t k_blocks = (K + kBK - 1) / kBK;
    const uint32_t per = (k_blocks + S - 1) / S;
    const uint32_t kb0 = min(k_blocks, pair * per), kb1 = min(k_blocks, kb0 + per);
    const bool has_k = kb1 > kb0;                    // an empty slice contributes zeros

    if (warp == 0 && lane == 0) {
        for (uint32_t s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + s * 8, 1);          // the leader's: its expect_tx covers both CTAs' loads
            mbar_init(bar_empty + s * 8, 1);         // tcgen05.commit, or the leader's relay in the peer CTA
        }
        mbar_init(bar_acc_full, 1);
        *abort_flag = 0;
        fence_mbar_init();
        prefetch_tensormap(&tm_a);
        prefetch_tensormap(&tm_b);
    }
    if (warp == 1) {
        tmem_alloc<2>(tmem_slot, C::kTmemCols);
        tmem_relinquish<2>();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_arrive();       // every CTA of the cluster is running before anyone signals or writes into it
    cluster_wait();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot_gen;
    if (epi.pdl_all) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0) {
        if (lane == 0) {
            // ===== producer: both CTAs' loads complete on the LEADER's full[s] =====
            if (epi.pdl_all) asm volatile("griddepcontrol.wait;" ::: "memory");
            const uint32_t full_leader = mapa(bar_full, rank & ~1u);
            const uint32_t peer_empty = mapa(bar_empty, rank | 1u);
            uint32_t stage = 0, phase = 0;
            // the weights pass through once (evict first); the activations are what every tile re-reads (evict last)
            const uint64_t pol_stream = l2_policy_evict_first(), pol_keep = l2_policy_evict_last();
            const int32_t row_a = static_cast<int32_t>(mi * 2 * ROWS + half * C::kARows);
            const int32_t row_b = static_cast<int32_t>(ni * BN + half * C::kBRows);
            for (uint32_t kb = kb0; kb < kb1; ++kb) {
                if (leader) {
                    if (!wait_bar(bar_empty + stage * 8, phase ^ 1u, ctx, kStProducerEmpty)) break;
                    mbar_arrive_cluster(peer_empty + stage * 8);          // relay "stage free" to the peer
                    mbar_arrive_expect_tx(bar_full + stage * 8, 2 * C::kStageBytes);
                } else {
                    if (!wait_bar(bar_empty + stage * 8, phase, ctx, kStProducerEmpty)) break;
                }
                const int32_t kx = static_cast<int32_t>(kb * kBK);
                tma_load_2d_pair_hint(smem_base + C::kOffA + stage * C::kABytes, &tm_a, full_leader + stage * 8, kx,
                                      row_a, pol_keep);
                tma_load_2d_pair_hint(smem_base + C::kOffB + stage * C::kBBytes, &tm_b, full_leader + stage * 8, kx,
                                      row_b, pol_stream);
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0 && leader && has_k) {
            // ===== MMA issuer (leader CTA of the pair): (2 * ROWS) x BN x 16 per instruction =====
            constexpr uint32_t idesc = instr_desc_f16(BF16, 2 * ROWS, BN);
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (uint32_t kb = kb0; kb < kb1; ++kb) {
                ok = wait_bar(bar_full + stage * 8, phase, ctx, kStMmaFull);
                if (!ok) break;
                tc_fence_after_sync();
                const uint64_t da = smem_desc_k_sw128(smem_base + C::kOffA + stage * C::kABytes);
                const uint64_t db = smem_desc_k_sw128(smem_base + C::kOffB + stage * C::kBBytes);
#pragma unroll
                for (uint32_t k = 0; k < kBK / kUmmaK; ++k)
                    umma_f16<2>(tmem_base, da + 2 * k, db + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                umma_commit<2>(bar_empty + stage * 8);
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
            if (ok) umma_commit<2>(bar_acc_full);
        }
        __syncwarp();
    } else {
        // ===== send: my partial sums of the columns another pair owns go to that pair's CTA with my rows =====
        const uint32_t q = warp & 3u;
        const uint32_t row = (ROWS == 64 ? (q & 1u) : q) * 32u + lane;   // row within this CTA's ROWS
        const uint32_t col_half = (ROWS == 64) ? q >> 1 : 0u;            // columns [col_half * HW, +HW)
        bool ok = true;
        if (has_k) {
            ok = wait_bar(bar_acc_full, 0, ctx, kStEpiAccFull);
            ok = __all_sync(0xffffffffu, ok);
            if (ok && leader && warp == 2 && lane == 0) mbar_arrive_cluster(mapa(bar_acc_full, rank | 1u));   // relay
            tc_fence_after_sync();
        }
        const uint32_t taddr = tmem_base + ((q * 32u) << 16);
        const uint32_t recv_local = smem_base + C::kOffRecv;
        if (S > 1) {
#pragma unroll 1
            for (uint32_t ch = 0; ch < HW / 32; ++ch) {
                if ((col_half * HW + ch * 32u) / W == pair) continue;      // my pair keeps these columns
                uint32_t v[32];
                if (has_k && ok) {
                    tmem_ld_32x32b_x32(taddr + ch * 32u, v);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = 0u;
                }
#pragma unroll
                for (uint32_t j = 0; j < 8; ++j) {
                    const uint32_t col = col_half * HW + ch * 32u + 4u * j;
                    const uint32_t p = col / W;
                    if (p != pair) {
                        const uint32_t dst = recv_local + ((((col - p * W) >> 2)) * C::kARows + row) * 16u;
                        st_cluster_v4(mapa(dst, 2u * p + half), __uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                      __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
                    }
                }
            }
        }
        tc_fence_before_sync();
    }

    // all partial slices delivered (every thread of every CTA of the cluster takes part)
    __syncwarp();
    cluster_arrive();
    cluster_wait();

    if (warp >= 2) {
        // ===== reduce the columns my pair owns (those of them that lie in this warp's column half) and store =====
        if (epi.pdl_all) asm volatile("griddepcontrol.wait;" ::: "memory");
        const uint32_t q = warp & 3u;
        const uint32_t row = (ROWS == 64 ? (q & 1u) : q) * 32u + lane;
        const uint32_t col_half = (ROWS == 64) ? q >> 1 : 0u;
        const uint32_t grow = mi * 2 * ROWS + half * C::kARows + row;
        const uint32_t own_lo = pair * W, own_hi = own_lo + W;
        const uint32_t half_lo = col_half * HW, half_hi = half_lo + HW;
        const uint32_t lo = max(own_lo, half_lo), hi = min(own_hi, half_hi);
        const float *recv = reinterpret_cast<const float *>(smem_gen + C::kOffRecv);
        tc_fence_after_sync();
        const bool acc_ok = has_k && (*abort_flag == 0);
        const bool fused = epi.any();
        const float rs = fused ? epi_row_scale(epi, grow < M, grow) : 1.f;
#pragma unroll 1
        for (uint32_t col = lo; col < hi; col += 32) {        // 32 columns per round of tensor-memory loads
            uint32_t o[32];
            if (acc_ok) {
                tmem_ld_32x32b_x32(tmem_base + ((q * 32u) << 16) + (col - half_lo), o);
                tmem_ld_wait();
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) o[i] = 0u;
            }
#pragma unroll
            for (uint32_t g8 = 0; g8 < 4; ++g8) {
                float f[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(o[8 * g8 + i]);
                if (S > 1) {                                       // the other pair's partial sums of my columns
                    const float4 *src =
                        reinterpret_cast<const float4 *>(recv) + ((col + 8 * g8 - own_lo) >> 2) * C::kARows + row;
                    const float4 a = src[0], b = src[C::kARows];
                    // k order: the pair with the lower k-slice first, whichever side of the sum it is on
                    if (pair == 0) {
                        f[0] += a.x; f[1] += a.y; f[2] += a.z; f[3] += a.w;
                        f[4] += b.x; f[5] += b.y; f[6] += b.z; f[7] += b.w;
                    } else {
                        f[0] = a.x + f[0]; f[1] = a.y + f[1]; f[2] = a.z + f[2]; f[3] = a.w + f[3];
                        f[4] = b.x + f[4]; f[5] = b.y + f[5]; f[6] = b.z + f[6]; f[7] = b.w + f[7];
                    }
                }
                const uint32_t gcol = ni * BN + col + 8 * g8;
                if (grow < M && gcol < N) {
                    if (fused) epi_apply8<BF16>(f, rs, epi, true, grow, gcol);
                    uint4 out;
                    out.x = pack2<BF16>(f[0], f[1]);
                    out.y = pack2<BF16>(f[2], f[3]);
                    out.z = pack2<BF16>(f[4], f[5]);
                    out.w = pack2<BF16>(f[6], f[7]);
                    *reinterpret_cast<uint4 *>(c + static_cast<size_t>(grow) * ldc + gcol) = out;
                }
            }
        }
        tc_fence_before_sync();
    }
    __syncthreads();
    if (*abort_flag) __nanosleep(50000);
    // neither CTA of a pair may free tensor memory or exit while its peer can still signal it
    cluster_arrive();
    cluster_wait();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc<2>(tmem_base, C::kTmemCols);
    }
}

// ----------------------------------------------------------------- skinny ----
//
// m <= 64 (a handful of tokens against a weight matrix): pure weight streaming, HBM-bound.  The roles
// of the operands are swapped so that no shared memory or bandwidth is spent on padding rows: the
// WEIGHTS B[n,k] feed the 128-row side of the MMA, the tokens A[m,k] its narrow side (N = TOK = 16, 32
// or 64 >= m), and tensor memory holds the TRANSPOSED tile D[n_local, m].  A stage is 16 KiB of
// weights + TOK*128 bytes of tokens, so 8-12 stages (up to 200 KiB) of weights are in flight per SM.
// One CTA per 128 weight rows (not persistent); with a cluster of S CTAs each takes a slice of k and
// the partial tiles are combined through distributed shared memory: CTA r owns 128/S of the tile's
// rows, every other CTA writes its partial values for those rows into r's receive buffer, one cluster
// barrier, then r sums in rank order (deterministic) and stores.  S == 1: no exchange, and the launch
// leaves the receive buffer out of its shared memory.
// The configurations with few stages (at most 113 KiB per CTA) put TWO CTAs on an SM: one CTA's set-up,
// first-load latency and epilogue overlap the other's streaming, a launch of more CTAs than SMs loses
// less to the last wave, and a dependent launch can become resident while its predecessor drains.
template <int TOK, int STAGES>
struct SnCfg {
    static constexpr uint32_t kWBytes = kBM * kBK * 2;              // weights tile, 16 KiB
    static constexpr uint32_t kTBytes = TOK * kBK * 2;              // token tile
    static constexpr uint32_t kStageBytes = kWBytes + kTBytes;
    static constexpr uint32_t kTmemCols = TOK < 32 ? 32 : TOK;
    static constexpr uint32_t kOffW = 0;
    static constexpr uint32_t kOffT = kOffW + STAGES * kWBytes;
    static constexpr uint32_t kOffBar = kOffT + STAGES * kTBytes;
    static constexpr uint32_t kNumBars = 2 * STAGES + 1;
    static constexpr uint32_t kOffMisc = kOffBar + kNumBars * 8;
    static constexpr uint32_t kOffRecv = (kOffMisc + 16 + 15) & ~15u;   // [TOK/4][S slots x 128/S rows][4] fp32, S > 1 only
    static constexpr uint32_t kRecvBytes = kBM * TOK * 4;
    static constexpr uint32_t kSmemNoRecv = kOffRecv + 1024;
    static constexpr uint32_t kSmemBytes = kSmemNoRecv + kRecvBytes;
    static constexpr uint32_t kTwoPerSm = 115712;                   // (228 KiB - 2 x 1 KiB reserved) / 2
    static_assert(kSmemBytes <= 232448, "exceeds 227 KiB of shared memory");
    static_assert(TOK == 16 || TOK == 32 || TOK == 64, "token tile");
};

template <int TOK, int STAGES, bool BF16>
__global__ void __launch_bounds__(kThreads, 1)
hgemm_skinny_kernel(const __grid_constant__ CUtensorMap tm_tok, const __grid_constant__ CUtensorMap tm_w,
                    uint16_t *c, uint32_t ldc, uint32_t M, uint32_t N, uint32_t K, const EpiArgs epi, int *status) {
    using C = SnCfg<TOK, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

    const uint32_t warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t S = cluster_nctarank();
    const uint32_t rank = cluster_ctarank();
    const uint32_t rows_per = kBM / S;                 // tile rows (weight rows) each CTA finally owns: 128 .. 16

    const uint32_t bar_full = smem_base + C::kOffBar;
    const uint32_t bar_empty = bar_full + STAGES * 8;
    const uint32_t bar_acc_full = bar_empty + STAGES * 8;
    const uint32_t tmem_slot = smem_base + C::kOffMisc;
    volatile uint32_t *tmem_slot_gen = reinterpret_cast<volatile uint32_t *>(smem_gen + C::kOffMisc);
    volatile uint32_t *abort_flag = tmem_slot_gen + 1;
    const WaitCtx ctx{abort_flag, status};

    const uint32_t ni = blockIdx.x / S;               // which 128 weight rows
    const uint32_t k_blocks = (K + kBK - 1) / kBK;
    const uint32_t per = (k_blocks + S - 1) / S;
    const uint32_t kb0 = min(k_blocks, rank * per), kb1 = min(k_blocks, kb0 + per);
    const bool has_k = kb1 > kb0;

    if (warp == 0 && lane == 0) {
        for (uint32_t s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + s * 8, 1);
            mbar_init(bar_empty + s * 8, 1);
        }
        mbar_init(bar_acc_full, 1);
        *abort_flag = 0;
        fence_mbar_init();
        prefetch_tensormap(&tm_tok);
        prefetch_tensormap(&tm_w);
    }
    if (warp == 1) {
        tmem_alloc<1>(tmem_slot, C::kTmemCols);
        tmem_relinquish<1>();
    }
    tc_fence_before_sync();
    __syncthreads();
    if (S > 1) {           // every CTA of the cluster is running before anyone writes into its shared memory
        cluster_arrive();
        cluster_wait();
    }
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot_gen;
    if (epi.pdl_all) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0) {
        if (lane == 0) {
            if (epi.pdl_all) asm volatile("griddepcontrol.wait;" ::: "memory");
            uint32_t stage = 0, phase = 0;
            // the weights pass through once (evict first); the activations are what every CTA re-reads (evict last)
            const uint64_t pol_stream = l2_policy_evict_first(), pol_keep = l2_policy_evict_last();
            for (uint32_t kb = kb0; kb < kb1; ++kb) {
                if (!wait_bar(bar_empty + stage * 8, phase ^ 1u, ctx, kStProducerEmpty)) break;
                mbar_arrive_expect_tx(bar_full + stage * 8, C::kStageBytes);
                const int32_t kx = static_cast<int32_t>(kb * kBK);
                tma_load_2d_hint(smem_base + C::kOffW + stage * C::kWBytes, &tm_w, bar_full + stage * 8, kx,
                                 static_cast<int32_t>(ni * kBM), pol_stream);
                tma_load_2d_hint(smem_base + C::kOffT + stage * C::kTBytes, &tm_tok, bar_full + stage * 8, kx, 0,
                                 pol_keep);
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0 && has_k) {
            constexpr uint32_t idesc = instr_desc_f16(BF16, kBM, TOK);
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (uint32_t kb = kb0; kb < kb1; ++kb) {
                ok = wait_bar(bar_full + stage * 8, phase, ctx, kStMmaFull);
                if (!ok) break;
                tc_fence_after_sync();
                const uint64_t dw = smem_desc_k_sw128(smem_base + C::kOffW + stage * C::kWBytes);
                const uint64_t dt = smem_desc_k_sw128(smem_base + C::kOffT + stage * C::kTBytes);
#pragma unroll
                for (uint32_t k = 0; k < kBK / kUmmaK; ++k)
                    umma_f16<1>(tmem_base, dw + 2 * k, dt + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                umma_commit<1>(bar_empty + stage * 8);
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
            if (ok) umma_commit<1>(bar_acc_full);
        }
        __syncwarp();
    } else {
        // ===== epilogue warps: thread = one weight row (n) of the tile, TOK partial sums (one per token) =====
        const uint32_t q = warp & 3u;
        const uint32_t row = q * 32u + lane;
        bool ok = true;
        if (has_k) {
            ok = wait_bar(bar_acc_full, 0, ctx, kStEpiAccFull);
            ok = __all_sync(0xffffffffu, ok);
            tc_fence_after_sync();
        }
        float f[TOK];
        if (has_k && ok) {
#pragma unroll
            for (uint32_t g8 = 0; g8 < TOK / 8; ++g8) {
                uint32_t o[8];
                tmem_ld_32x32b_x8(tmem_base + ((q * 32u) << 16) + 8u * g8, o);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 8; ++i) f[8 * g8 + i] = __uint_as_float(o[i]);
            }
        } else {
#pragma unroll
            for (int i = 0; i < TOK; ++i) f[i] = 0.f;
        }
        tc_fence_before_sync();
        const uint32_t owner = row / rows_per;
        const uint32_t recv_local = smem_base + C::kOffRecv;
        if (S > 1 && owner != rank) {
            // my partial sums for a row another CTA owns: slot `rank` of the owner's receive buffer
            // layout [TOK/4][S slots x rows][4]: the 32 rows of a warp are 32 consecutive 16-byte words (no bank conflicts)
            const uint32_t dst = mapa(recv_local + (rank * rows_per + (row - owner * rows_per)) * 16u, owner);
#pragma unroll
            for (uint32_t j = 0; j < TOK / 4; ++j)
                st_cluster_v4(dst + j * (kBM * 16u), f[4 * j], f[4 * j + 1], f[4 * j + 2], f[4 * j + 3]);
        }
        if (S > 1) {
            __syncwarp();
            cluster_arrive();
            cluster_wait();
        }
        if (owner == rank) {
            if (epi.pdl_all) asm volatile("griddepcontrol.wait;" ::: "memory");
            const float *recv = reinterpret_cast<const float *>(smem_gen + C::kOffRecv);
            for (uint32_t r2 = 0; r2 < S; ++r2) {
                if (r2 == rank) continue;
                const float4 *src = reinterpret_cast<const float4 *>(recv) + (r2 * rows_per + (row - rank * rows_per));
#pragma unroll
                for (uint32_t j = 0; j < TOK / 4; ++j) {
                    const float4 v = src[j * kBM];
                    f[4 * j] += v.x; f[4 * j + 1] += v.y; f[4 * j + 2] += v.z; f[4 * j + 3] += v.w;
                }
            }
            // C[mi, n] = D[n, mi]: for each token the 32 lanes of a warp write 32 consecutive columns of C
            const uint32_t n_glob = ni * kBM + row;
            if (n_glob < N) {
                if (epi.any()) {
                    // thread = one column of C: its bias once, then per token the row scale (one address for the
                    // whole warp) and the residual element (32 consecutive columns per warp)
                    float bias = 0.f, unused;
                    if (epi.bias) unpack2<BF16>(static_cast<uint32_t>(epi.bias[n_glob]), bias, unused);
                    if (epi.row_scale && epi.pdl_wait) asm volatile("griddepcontrol.wait;" ::: "memory");
#pragma unroll
                    for (uint32_t mi = 0; mi < TOK; ++mi) {
                        if (mi < M) {
                            float add = bias, r = 0.f;
                            if (epi.residual)
                                unpack2<BF16>(static_cast<uint32_t>(epi.residual[static_cast<size_t>(mi) * epi.ldr + n_glob]),
                                              r, unused);
                            add += r;
                            const float rs = epi.row_scale ? epi.row_scale[mi] : 1.f;
                            f[mi] = fmaf(f[mi], rs, add);
                        }
                    }
                }
#pragma unroll
                for (uint32_t mi = 0; mi < TOK; ++mi) {
                    if (mi < M) {
                        const uint32_t w = pack2<BF16>(f[mi], 0.f);
                        c[static_cast<size_t>(mi) * ldc + n_glob] = static_cast<uint16_t>(w & 0xffffu);
                    }
                }
            }
        }
    }
    if (S > 1 && warp < 2) {      // the cluster barrier counts every thread of every CTA
        __syncwarp();
        cluster_arrive();
        cluster_wait();
    }
    __syncthreads();
    if (*abort_flag) __nanosleep(50000);
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc<1>(tmem_base, C::kTmemCols);
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
bool encode_tmap(CUtensorMap *tm, const void *base, int64_t rows, int64_t cols, int64_t ld,
                 uint32_t box_rows, bool bf16, bool is_output, uint32_t box_cols) {
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return false;
    cuuint64_t gdim[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    cuuint64_t gstride[1] = {static_cast<cuuint64_t>(ld) * 2};
    cuuint32_t box[2] = {box_cols, box_rows};     // 64 columns: 128-byte swizzle; 32 columns: 64-byte swizzle
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(tm, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                     const_cast<void *>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     box_cols == 32 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                     is_output ? CU_TENSOR_MAP_L2_PROMOTION_NONE : CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// A tensor map depends only on (address, extents, pitch, box, type), not on the memory's contents, so
// repeated calls on the same buffers (the common case: weights, a reused activation buffer) reuse the
// encoded 128-byte descriptor instead of paying the driver call (~1 us each, three per GEMM).
// Small per-thread direct-mapped cache; no locking, no allocation.
struct TmapKey {
    const void *base;
    int64_t rows, cols, ld;
    uint32_t box_rows;
    uint32_t kind;   // bit 0: bf16, bit 1: output, bit 2: 32-column box
    bool operator==(const TmapKey &o) const {
        return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows &&
               kind == o.kind;
    }
};
struct TmapSlot {
    TmapKey key;
    bool valid;
    alignas(64) CUtensorMap map;
};
constexpr int kTmapSlots = 32;

bool make_tmap(CUtensorMap *tm, const void *base, int64_t rows, int64_t cols, int64_t ld,
               uint32_t box_rows, bool bf16, bool is_output, uint32_t box_cols = kBK) {
    thread_local TmapSlot cache[kTmapSlots] = {};
    const TmapKey key{base, rows, cols, ld, box_rows,
                      (bf16 ? 1u : 0u) | (is_output ? 2u : 0u) | (box_cols == 32 ? 4u : 0u)};
    uint64_t h = reinterpret_cast<uint64_t>(base) >> 8;
    h ^= static_cast<uint64_t>(rows) * 0x9E3779B97F4A7C15ull + static_cast<uint64_t>(cols) * 31 + box_rows + key.kind;
    TmapSlot &slot = cache[(h ^ (h >> 17)) % kTmapSlots];
    if (!(slot.valid && slot.key == key)) {
        if (!encode_tmap(&slot.map, base, rows, cols, ld, box_rows, bf16, is_output, box_cols)) {
            slot.valid = false;
            return false;
        }
        slot.key = key;
        slot.valid = true;
    }
    *tm = slot.map;
    return true;
}

struct DeviceInfo {
    int sm_count = 0;
    int cc_major = 0;
    int *status_word = nullptr;
    uint32_t *wave_sync = nullptr;
};

__device__ int g_gemm_status_word;
// Counters of the producers' synchronisation, one per launch in flight: a launch takes the next slot (zeroed on its
// stream just before the kernel), so launches that overlap on different streams do not share one.
constexpr unsigned kWaveSyncSlots = 32;
__device__ uint32_t g_wave_sync[2 * kWaveSyncSlots];      // zero at load; every kernel leaves its pair zeroed

DeviceInfo g_dev[kMaxDevices];
DeviceOnce g_dev_once;

// Filled on the first call on a device, under g_dev_once: a second host thread either waits for the table or
// finds it complete.
cudaError_t device_info(DeviceInfo **out) {
    int dev = 0;
    cudaError_t e = current_device(&dev);
    if (e != cudaSuccess) return e;
    e = g_dev_once.run(dev, [dev]() {
        DeviceInfo d;
        cudaError_t e2;
        if ((e2 = cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e2;
        if ((e2 = cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev)) != cudaSuccess) return e2;
        if (d.cc_major == 10) {
            void *p = nullptr;
            if ((e2 = cudaGetSymbolAddress(&p, g_gemm_status_word)) != cudaSuccess) return e2;
            d.status_word = static_cast<int *>(p);
            if ((e2 = cudaGetSymbolAddress(&p, g_wave_sync)) != cudaSuccess) return e2;
            d.wave_sync = static_cast<uint32_t *>(p);
        }
        g_dev[dev] = d;
        return cudaSuccess;
    });
    if (e != cudaSuccess) return e;
    *out = &g_dev[dev];
    return cudaSuccess;
}

// Ordinary launches go out under programmatic stream serialisation (PEAKGEMM_TUNE_PDL=0 in a tuning build: off).
bool pdl_enabled() {
    static const int env_pdl = tune_env_int("PEAKGEMM_TUNE_PDL", 1);
    return env_pdl != 0;
}

EpiArgs make_epi(const GemmArgs &g) {
    EpiArgs e;
    e.row_scale = g.row_scale;
    e.bias = static_cast<const uint16_t *>(g.bias);
    e.residual = static_cast<const uint16_t *>(g.residual);
    e.ldr = static_cast<uint32_t>(g.ldr);
    e.pdl_wait = (g.pdl_wait && g.row_scale) ? 1u : 0u;
    e.pdl_all = (!e.pdl_wait && pdl_enabled()) ? 1u : 0u;
    e.mc_dst = static_cast<uint16_t *>(g.mc_dst);
    e.ld_mc = static_cast<uint32_t>(g.ldc);
    return e;
}

// Launch attributes common to the three kernels: the cluster shape, and for a caller that chained this
// GEMM behind the kernel producing row_scale, programmatic stream serialisation (the grid may start
// while that kernel drains; only the epilogue's griddepcontrol.wait orders the read of row_scale).
int fill_attrs(cudaLaunchAttribute *attr, unsigned cluster_x, const GemmArgs &g) {
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster_x;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    if (!(g.pdl_wait && g.row_scale) && !pdl_enabled()) return 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    return 2;
}

}  // namespace

// Tail split plan for the 256-wide CTA-pair kernel on `workers` SM pairs: k-slices per remainder tile (0 = none)
// and the workspace it needs.  The remainder must be at most half a wave, and the split must pay: the owner of a
// tile reads its helpers' partial sums one after the other (about 3 us each, L2 latency bound), and a remainder
// wave on a mostly idle, un-throttled GPU runs at about 0.75 of a tile time anyway.  Measured on B200
// (1024 x 14336 x k): k = 4096 no gain with any slice count, k = 16384 455 -> 365 us with 8 slices.  So the slice
// count minimises  tile/s + 3.2 (s - 1) + 4 us  (tile = 0.38 us per k-block) and the split is used only when that
// is under 0.6 of a tile time.
void plan_tail(int64_t m, int64_t n, int64_t k, int workers, uint32_t *full_tiles, uint32_t *split, size_t *bytes,
               double *tail_frac = nullptr) {
    const int64_t tiles = ((m + 255) / 256) * ((n + 255) / 256);
    const int64_t k_blocks = (k + 63) / 64;
    *full_tiles = static_cast<uint32_t>(tiles);
    *split = 0;
    *bytes = 0;
    if (workers < 2) return;
    // A problem of at most half a wave is all remainder: every tile is split (mid-size m with a long k, where 32
    // tiles would leave 42 SM pairs idle for the whole run; 512 x 4096 x 14336: 67 -> 54 us, 512 x 4096 x 8192:
    // 42 -> 37, but 512 x 4096 x 4096: 25.6 -> 27.5).  Nothing runs un-throttled beside it then, so the bar is 0.7
    // of a tile time instead of 0.6.
    const bool all_remainder = tiles * 2 <= workers;
    if (!all_remainder && tiles <= workers) return;
    const int64_t rem = all_remainder ? tiles : tiles % workers;
    if (rem == 0 || rem * 2 > workers) return;
    int64_t s_max = workers / rem;
    if (s_max > 8) s_max = 8;
    if (s_max > k_blocks / 8) s_max = k_blocks / 8;
    const double tile_us = 0.38 * static_cast<double>(k_blocks);
    double best = (all_remainder ? 0.7 : 0.6) * tile_us;
    int64_t s = 0;
    for (int64_t c = 2; c <= s_max; ++c) {
        const double cost = tile_us / c + 3.2 * (c - 1) + 4.0;
        if (cost < best) { best = cost; s = c; }
    }
    if (s < 2) return;
    if (tail_frac) *tail_frac = best / tile_us;        // the split remainder wave, in tile times
    *full_tiles = static_cast<uint32_t>(tiles - rem);
    *split = static_cast<uint32_t>(s);
    const size_t parts = static_cast<size_t>(rem) * (s - 1) * 2;
    const size_t flag_bytes = (parts * kEpiWarps * sizeof(uint32_t) + 255) / 256 * 256;
    *bytes = flag_bytes + parts * kBM * 256 * sizeof(float);
}

namespace {

template <int CTA_GROUP, int BN, int STAGES, int MT, bool BF16>
cudaError_t launch(const GemmArgs &g, const DeviceInfo &d, int sms, cudaStream_t stream) {
    using C = Cfg<CTA_GROUP, BN, STAGES, MT>;
    auto kernel = hgemm_tcgen05_kernel<CTA_GROUP, BN, STAGES, MT, BF16>;
    static DeviceOnce smem_once;
    {
        const cudaError_t e = allow_dynamic_smem(smem_once, kernel, C::kSmemBytes);
        if (e != cudaSuccess) return e;
    }
    CUtensorMap tm_a, tm_b;
    DstMaps tm_c = {};
    // several destinations (or a multicast one): every store box is 64 columns wide, 128-byte rows (see the kernel)
    const uint32_t store_box_cols = (g.n_extra_dst > 0 || g.mc_dst) ? kStoreCols : C::kStoreBoxCols;
    if (!make_tmap(&tm_a, g.a, g.m, g.k, g.lda, kBM, BF16, false) ||
        !make_tmap(&tm_b, g.b, g.n, g.k, g.ldb, C::kBRows, BF16, false) ||
        !make_tmap(&tm_c.m[0], g.c, g.m, g.n, g.ldc, kStoreRows, BF16, true, store_box_cols))
        return cudaErrorInvalidValue;
    for (int i = 0; i < g.n_extra_dst; ++i)
        if (!make_tmap(&tm_c.m[1 + i], g.extra_dst[i], g.m, g.n, g.ldc, kStoreRows, BF16, true, store_box_cols))
            return cudaErrorInvalidValue;
    const uint32_t n_dst = 1u + static_cast<uint32_t>(g.n_extra_dst);

    const uint32_t tile_m = kBM * CTA_GROUP * MT;
    const uint64_t m_tiles = (g.m + tile_m - 1) / tile_m;
    const uint64_t n_tiles = (g.n + BN - 1) / BN;
    const uint64_t tiles = m_tiles * n_tiles;
    uint64_t workers = static_cast<uint64_t>(sms / CTA_GROUP);

    TailArgs tail = {static_cast<uint32_t>(tiles), 0u, nullptr, nullptr, nullptr, 0u, 0u};
    if (CTA_GROUP == 2 && BN == 256 && MT == 1 && g.workspace && g.n_extra_dst == 0 && !g.mc_dst) {
        uint32_t full = 0, split = 0;
        size_t need = 0;
        plan_tail(g.m, g.n, g.k, static_cast<int>(workers), &full, &split, &need);
        if (split >= 2 && need <= g.workspace_bytes) {
            if (full == 0) workers = tiles * split;     // all remainder: one worker per k-slice
            const size_t parts = static_cast<size_t>(tiles - full) * (split - 1) * 2;
            const size_t flag_bytes = (parts * kEpiWarps * sizeof(uint32_t) + 255) / 256 * 256;
            cudaError_t e = cudaMemsetAsync(g.workspace, 0, flag_bytes, stream);
            if (e != cudaSuccess) return e;
            tail.full_tiles = full;
            tail.split = split;
            tail.flags = static_cast<uint32_t *>(g.workspace);
            tail.ws = reinterpret_cast<float *>(static_cast<uint8_t *>(g.workspace) + flag_bytes);
        }
    }
    if (tail.split < 2 && tiles < workers) workers = tiles;

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(workers * CTA_GROUP), 1, 1);
    cfg.blockDim = dim3(MT == 2 ? kThreadsWide : kThreads, 1, 1);
    cfg.dynamicSmemBytes = C::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[3];
    cfg.attrs = attr;
    cfg.numAttrs = fill_attrs(attr, CTA_GROUP, g);
    // Benchmark overrides (builds with PG_ENABLE_TUNING only), read once: PEAKGEMM_TUNE_GROUP_M (raster band
    // height in tiles), PEAKGEMM_TUNE_FLAGS (the kFlag* switches).
    static const int env_group_m = tune_env_int("PEAKGEMM_TUNE_GROUP_M", 0);
    static const int env_flags = tune_env_int("PEAKGEMM_TUNE_FLAGS", -1);
    const uint32_t group_m = env_group_m > 0 ? static_cast<uint32_t>(env_group_m) : 16 / (CTA_GROUP * MT);
    // one tile row (m <= 128): every weight byte is read exactly once, so B streams through L2 (evict first)
    const uint32_t shape_flags = (CTA_GROUP == 1 && g.m <= 128) ? kFlagBEvictFirst : 0u;
    const uint32_t flags = env_flags >= 0 ? static_cast<uint32_t>(env_flags) : (kDefaultFlags | shape_flags);
    // Producer synchronisation (see the producer role): for problems of at least two waves of tiles and about 0.2
    // TFLOP.  Measured on B200
    // against the same kernel without it: 8192^3 +1 %, 8192 x 32768 x 16384 +2-4 %, 32768 x 32768 x 16384 +9 % (DRAM
    // reads of the second shape 8.9-12.4 -> 6.4 GB, requests merged on the way to L2 x 3-5).
    // PEAKGEMM_TUNE_WAVESYNC (builds with PG_ENABLE_TUNING only): 0 off, 1 on, -1 automatic.
    static const int env_wave = tune_env_int("PEAKGEMM_TUNE_WAVESYNC", -1);
    // Only with two row blocks per CTA (k-blocks of 1024 tensor-pipe cycles, 4 stages): the 256 x 256 pair kernel lost
    // with the same scheme (4096 x 14336 x 4096: 314 -> 362 us).
    const bool wave_auto = MT == 2 && tiles >= 2 * workers && g.k >= 2048 &&
                           static_cast<double>(g.m) * static_cast<double>(g.n) * static_cast<double>(g.k) >= 1.0e11;
    if ((env_wave > 0 || (env_wave < 0 && wave_auto)) && tail.split < 2 && tiles > workers && d.wave_sync) {
        static std::atomic<unsigned> slot_counter{0};
        tail.wave_sync = d.wave_sync + 2 * (slot_counter.fetch_add(1) % kWaveSyncSlots);
        static const int env_sync_kb = tune_env_int("PEAKGEMM_TUNE_SYNC_KB", 8);
        tail.sync_kb = static_cast<uint32_t>(env_sync_kb);
        static const int env_sync_lag = tune_env_int("PEAKGEMM_TUNE_SYNC_LAG", 1);
        tail.sync_lag = static_cast<uint32_t>(env_sync_lag);
    }
    if (tail.split >= 2) {
        // Owners wait for helper CTAs of the same grid: ask for a cooperative launch, which starts the grid only
        // when all of it can be resident at once.  If the device refuses, run without the split.
        // (without the programmatic-serialisation attribute: this launch neither triggers nor waits)
        if (!(g.pdl_wait && g.row_scale)) cfg.numAttrs = 1;
        attr[cfg.numAttrs].id = cudaLaunchAttributeCooperative;
        attr[cfg.numAttrs].val.cooperative = 1;
        ++cfg.numAttrs;
        const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, tm_a, tm_b, tm_c, n_dst, static_cast<uint32_t>(g.m),
                                                 static_cast<uint32_t>(g.n), static_cast<uint32_t>(g.k), group_m,
                                                 flags, make_epi(g), tail, d.status_word);
        if (e == cudaSuccess) return e;
        cudaGetLastError();
        cfg.numAttrs = fill_attrs(attr, CTA_GROUP, g);
        tail = TailArgs{static_cast<uint32_t>(tiles), 0u, nullptr, nullptr, nullptr, 0u, 0u};
    }
    // An ordinary (not cooperative) launch goes out under programmatic stream serialisation, see kFlagPdl.  Not
    // when the caller chained this GEMM behind the kernel that produces row_scale: that mode has its own, later wait.
    uint32_t launch_flags = flags;
    if (pdl_enabled() && !(g.pdl_wait && g.row_scale)) launch_flags |= kFlagPdl;    // fill_attrs set the attribute
    return cudaLaunchKernelEx(&cfg, kernel, tm_a, tm_b, tm_c, n_dst, static_cast<uint32_t>(g.m),
                              static_cast<uint32_t>(g.n), static_cast<uint32_t>(g.k), group_m, launch_flags,
                              make_epi(g), tail, d.status_word);
}

template <int BN, int STAGES, bool BF16>
cudaError_t launch_splitk(const GemmArgs &g, const DeviceInfo &d, int split, cudaStream_t stream) {
    using C = SkCfg<BN, STAGES>;
    auto kernel = hgemm_splitk_kernel<BN, STAGES, BF16>;
    static DeviceOnce smem_once;
    {
        const cudaError_t e = allow_dynamic_smem(smem_once, kernel, C::kSmemBytes);
        if (e != cudaSuccess) return e;
    }
    CUtensorMap tm_a, tm_b;
    if (!make_tmap(&tm_a, g.a, g.m, g.k, g.lda, kBM, BF16, false) ||
        !make_tmap(&tm_b, g.b, g.n, g.k, g.ldb, BN, BF16, false))
        return cudaErrorInvalidValue;
    const uint64_t tiles = ((g.m + kBM - 1) / kBM) * ((g.n + BN - 1) / BN);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(tiles * split), 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = C::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    cfg.attrs = attr;
    cfg.numAttrs = fill_attrs(attr, static_cast<unsigned>(split), g);
    (void)d;
    return cudaLaunchKernelEx(&cfg, kernel, tm_a, tm_b, static_cast<uint16_t *>(g.c), static_cast<uint32_t>(g.ldc),
                              static_cast<uint32_t>(g.m), static_cast<uint32_t>(g.n), static_cast<uint32_t>(g.k),
                              make_epi(g), d.status_word);
}

template <int ROWS, int BN, int STAGES, bool BF16>
cudaError_t launch_pair_splitk(const GemmArgs &g, const DeviceInfo &d, int pairs, cudaStream_t stream) {
    using C = PsCfg<ROWS, BN, STAGES>;
    auto kernel = hgemm_pair_splitk_kernel<ROWS, BN, STAGES, BF16>;
    static DeviceOnce smem_once;
    {
        const cudaError_t e = allow_dynamic_smem(smem_once, kernel, C::kSmemBytes);
        if (e != cudaSuccess) return e;
    }
    CUtensorMap tm_a, tm_b;
    if (!make_tmap(&tm_a, g.a, g.m, g.k, g.lda, C::kARows, BF16, false) ||
        !make_tmap(&tm_b, g.b, g.n, g.k, g.ldb, C::kBRows, BF16, false))
        return cudaErrorInvalidValue;
    const uint64_t tiles = ((g.m + 2 * ROWS - 1) / (2 * ROWS)) * ((g.n + BN - 1) / BN);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(tiles * 2 * pairs), 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = C::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    cfg.attrs = attr;
    cfg.numAttrs = fill_attrs(attr, static_cast<unsigned>(2 * pairs), g);
    return cudaLaunchKernelEx(&cfg, kernel, tm_a, tm_b, static_cast<uint16_t *>(g.c), static_cast<uint32_t>(g.ldc),
                              static_cast<uint32_t>(g.m), static_cast<uint32_t>(g.n), static_cast<uint32_t>(g.k),
                              make_epi(g), d.status_word);
}

// Tile width (256 or 128) and pairs per cluster (1 or 2) for the pair split-K kernel (tiles of 128 rows for m <= 128,
// of 256 rows above): the combination with the most CTAs that stays within ~1.1 waves of the SMs, the wider tile on
// a tie (less operand traffic per flop); every k-slice keeps at least four k-blocks.  pairs = 0: even 256-wide
// tiles with one pair exceed that (the persistent kernels take such shapes).  Clusters of 8 CTAs (4 pairs) are left
// out: 16 of them do not fit the GPU at once (128 x 4096 x 4096 with 4 pairs per cluster: 30 us against 16 us for
// the same work in clusters of 4).
void choose_pair_split(const GemmArgs &g, int sm_count, int block_n, int *bn_out, int *pairs_out) {
    const int64_t k_blocks = (g.k + 63) / 64;
    const int64_t m_tiles = g.m <= 128 ? 1 : (g.m + 255) / 256;
    int64_t best_ctas = 0;
    *bn_out = 256;
    *pairs_out = 0;
    for (int bn = 256; bn >= 128; bn /= 2) {
        if (block_n != 0 && block_n != bn) continue;
        const int64_t tiles = m_tiles * ((g.n + bn - 1) / bn);
        for (int s = 1; s <= 2; ++s) {
            if (s > 1 && k_blocks < 4 * s) continue;
            const int64_t ctas = tiles * 2 * s;
            if (ctas * 10 > static_cast<int64_t>(sm_count) * 11) continue;
            if (ctas > best_ctas) { best_ctas = ctas; *bn_out = bn; *pairs_out = s; }
        }
    }
}

// Whether the automatic choice takes the pair split-K kernel with 256 x 256 tiles and two pairs per tile (asked after
// the one-CTA cluster split-K kernel, which keeps m <= 256 wherever it has a plan).
bool pair_split_pays(int64_t m, int64_t n, int64_t k, int sm_count) {
    if (m <= 128 || k < 4096) return false;
    const int64_t tiles = ((m + 255) / 256) * ((n + 255) / 256);
    return tiles * 4 * 10 <= static_cast<int64_t>(sm_count) * 11;
}

template <int ROWS>
cudaError_t launch_pair_splitk_any(const GemmArgs &g, const DeviceInfo &d, int bn, int pairs, cudaStream_t stream) {
    constexpr int kStages256 = ROWS == 64 ? 6 : 5, kStages128 = 8;
    if (bn == 256)
        return g.bf16 ? launch_pair_splitk<ROWS, 256, kStages256, true>(g, d, pairs, stream)
                      : launch_pair_splitk<ROWS, 256, kStages256, false>(g, d, pairs, stream);
    return g.bf16 ? launch_pair_splitk<ROWS, 128, kStages128, true>(g, d, pairs, stream)
                  : launch_pair_splitk<ROWS, 128, kStages128, false>(g, d, pairs, stream);
}

template <int TOK, int STAGES, bool BF16>
cudaError_t launch_skinny(const GemmArgs &g, const DeviceInfo &d, int split, cudaStream_t stream) {
    using C = SnCfg<TOK, STAGES>;
    auto kernel = hgemm_skinny_kernel<TOK, STAGES, BF16>;
    static DeviceOnce smem_once;
    {
        const cudaError_t e = allow_dynamic_smem(smem_once, kernel, C::kSmemBytes);
        if (e != cudaSuccess) return e;
    }
    CUtensorMap tm_tok, tm_w;
    if (!make_tmap(&tm_tok, g.a, g.m, g.k, g.lda, TOK, BF16, false) ||
        !make_tmap(&tm_w, g.b, g.n, g.k, g.ldb, kBM, BF16, false))
        return cudaErrorInvalidValue;
    const uint64_t tiles = (g.n + kBM - 1) / kBM;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(tiles * split), 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = split == 1 ? C::kSmemNoRecv : C::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    cfg.attrs = attr;
    cfg.numAttrs = fill_attrs(attr, static_cast<unsigned>(split), g);
    return cudaLaunchKernelEx(&cfg, kernel, tm_tok, tm_w, static_cast<uint16_t *>(g.c), static_cast<uint32_t>(g.ldc),
                              static_cast<uint32_t>(g.m), static_cast<uint32_t>(g.n), static_cast<uint32_t>(g.k),
                              make_epi(g), d.status_word);
}

// Cluster size for the skinny kernel: the largest S in {1,2,4,8} that keeps tiles * S within ~1.1 waves
// of the CTA slots (SMs, or twice that for the configurations of which two fit on an SM) and leaves every
// k-slice at least four k-blocks.
int choose_skinny_split(const GemmArgs &g, int slots) {
    const int64_t tiles = (g.n + 127) / 128, k_blocks = (g.k + 63) / 64;
    int best = 1;
    for (int s = 2; s <= 8; s *= 2)
        if (tiles * s * 10 <= static_cast<int64_t>(slots) * 11 && k_blocks >= 4 * s) best = s;
    return best;
}

// Skinny kernel: which instantiation.  Up to 16 tokens: always two CTAs per SM (5 stages of 18 KiB with the
// receive buffer, 6 without).  17-32 tokens: two per SM (5 x 20 KiB, no receive buffer) once there are more
// tiles than SMs, where one CTA per SM would run in waves; the deep single-CTA pipelines (10 x 20 KiB,
// 8 x 24 KiB) otherwise and for 33-64 tokens.  Measured, us (one per SM -> two per SM; cuBLAS): 16 x 4096 x
// 4096 12.7 -> 11.1 (15.2), 16 x 14336 x 4096 24.0 -> 22.2 (23.8), 16 x 128256 x 4096 171.6 -> 158.3 (158.2),
// 8 x 8192 x 8192 27.0 -> 23.8 (25.7), 32 x 128256 x 4096 177.1 -> 161.9 (164.7).  Not taken: 32 x 4096 x 4096
// with two per SM and a cluster of 8 (12.0 -> 13.0), 64 x 128256 x 4096 with two per SM and 4 stages of
// 24 KiB (184.2 -> 198.4).  17-32 tokens with one wave of tiles that one CTA per SM leaves unsplit (82-162 tiles):
// two per SM with 4 x 20 KiB and k split in two, 32 x 14336 x 4096 24.0 -> 22.9 (23.4), 32 x 11008 x 4096
// 22.1 -> 19.5 (20.5), 32 x 14336 x 8192 40.6 -> 41.3 (39.4).
template <bool BF16>
cudaError_t launch_skinny_any(const GemmArgs &g, const DeviceInfo &d, int sms, int forced_split, cudaStream_t stream) {
    const int64_t tiles = (g.n + 127) / 128;
    const bool two = g.m <= 16 || (g.m <= 32 && tiles > sms);
    int sp = choose_skinny_split(g, two ? 2 * sms : sms);
    if (forced_split > 0) sp = forced_split;
    // 17-32 tokens, one wave of tiles that one CTA per SM cannot split over k (more than 0.55 x SMs tiles): two CTAs
    // per SM, each half of k
    static const bool env_two32 = tune_env_int("PEAKGEMM_TUNE_SKINNY_TWO32", 1) != 0;
    if (env_two32 && forced_split <= 0 && !two && g.m > 16 && g.m <= 32 && sp == 1 && tiles * 20 <= sms * 22 &&
        (g.k + 63) / 64 >= 8)
        return launch_skinny<32, 4, BF16>(g, d, 2, stream);
    if (g.m <= 16) return sp == 1 ? launch_skinny<16, 6, BF16>(g, d, sp, stream) : launch_skinny<16, 5, BF16>(g, d, sp, stream);
    if (g.m <= 32) return two && sp == 1 ? launch_skinny<32, 5, BF16>(g, d, sp, stream)
                                         : launch_skinny<32, 10, BF16>(g, d, sp, stream);
    return launch_skinny<64, 8, BF16>(g, d, sp, stream);
}

template <int CTA_GROUP, int BN, int STAGES, int MT = 1>
cudaError_t launch_dt(const GemmArgs &g, const DeviceInfo &d, int sms, cudaStream_t stream) {
    return g.bf16 ? launch<CTA_GROUP, BN, STAGES, MT, true>(g, d, sms, stream)
                  : launch<CTA_GROUP, BN, STAGES, MT, false>(g, d, sms, stream);
}

}  // namespace

// Picks the kernel variant and tile width when the caller leaves them open, by a
// small cost model: waves of tiles over the SMs (or SM pairs) times the tile
// width, divided by how efficient that configuration is per tile.  (The reference
// has one fixed configuration: hgemm_wmma_impl.h:410.)
void choose_config(const GemmArgs &g, int sm_count, int *variant, int *block_n) {
    if (*variant == 5) {          // two row blocks per CTA exist at one tile width only
        if (*block_n == 0) *block_n = 256;
        return;
    }
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
            double waves = static_cast<double>((tiles + workers - 1) / workers);
            if (v == 2 && bn == 256 && g.workspace && g.n_extra_dst == 0) {
                // with a workspace the last partial wave of this configuration is cut into k-slices
                uint32_t full = 0, split = 0;
                size_t need = 0;
                double frac = 1.0;
                plan_tail(g.m, g.n, g.k, static_cast<int>(workers), &full, &split, &need, &frac);
                if (split >= 2 && need <= g.workspace_bytes) waves = static_cast<double>(full / workers) + frac;
            }
            // measured at 8192^3: block_n 128 runs at ~0.72 of block_n 256 per flop (operand traffic per flop doubles)
            const double eff = (bn == 256 ? 1.0 : bn == 128 ? 0.72 : 0.45) * (v == 2 ? 1.06 : 1.0);
            const double cost = waves * bn / eff;
            if (cost < best) { best = cost; best_v = v; best_bn = bn; }
        }
    }
    // Two row blocks per CTA pair (512 x 256 tiles): a quarter less operand traffic per flop, measured 1.04-1.06 of
    // the 256 x 256 pair tile per flop when the waves are full (8192^3, 16384^3, 32768 x 4096 x 16384), but tiles
    // twice as large quantise worse (4096 x 14336 x 4096: 7 waves of 448 tiles against 13 of 896: 0.87).
    if (*variant == 0 && (*block_n == 0 || *block_n == 256) && g.m > 256) {
        const int64_t tiles = ((g.m + 511) / 512) * ((g.n + 255) / 256);
        const int64_t workers = sm_count / 2;
        const int64_t waves = (tiles + workers - 1) / workers;
        // the 5 % only show over several waves; one or two waves of large tiles run no faster per flop than the
        // 256 x 256 tile, which then wins the tie (512 x 14336 x 4096: 48.8 against 51.3 us, 2048 x 4096 x 4096: 48.2
        // against 50.3)
        const double cost = static_cast<double>(waves) * 512.0 / (1.06 * (waves >= 3 ? 1.05 : 1.0));
        if (cost < best) { best = cost; best_v = 5; best_bn = 256; }
    }
    *variant = best_v;
    *block_n = best_bn;
}

// Cluster split-K plan: tile width and cluster size S (0 = do not split).  Used when one CTA per
// tile would leave most SMs idle: picks the (block_n, S) whose tiles * S comes closest to the SM
// count without exceeding ~1.1 waves; every k-slice keeps at least two k-blocks and every CTA ends
// up owning at least 8 columns.  block_n == 0: free choice between 128 and 64.
void choose_splitk(const GemmArgs &g, int sm_count, int block_n, int *bn_out, int *split_out) {
    *bn_out = 0;
    *split_out = 0;
    const int64_t k_blocks = (g.k + 63) / 64;
    int64_t best_ctas = 0;
    for (int bn = 128; bn >= 64; bn /= 2) {
        if (block_n != 0 && block_n != bn) continue;
        const int64_t tiles = ((g.m + 127) / 128) * ((g.n + bn - 1) / bn);
        for (int s = 8; s >= 2; s /= 2) {
            if (k_blocks < 2 * s || bn / s < 8) continue;
            const int64_t ctas = tiles * s;
            if (ctas * 10 > static_cast<int64_t>(sm_count) * 11) continue;
            // on a tie a short k prefers the narrower tile with the smaller cluster (less to exchange; measured
            // 16.5 vs 18.6 us at 128 x 4096 x 4096), a long k the deeper split (32.5 vs 37.1 us at k = 14336)
            const bool tie_wins = ctas == best_ctas && k_blocks < 128 && s < *split_out;
            if (ctas > best_ctas || tie_wins) { best_ctas = ctas; *bn_out = bn; *split_out = s; }
        }
    }
}

// One tile row (64 < m <= 128): which of the one-CTA persistent kernel (block_n 64/128/256) and the cluster split-K
// kernel (block_n 64/128, S = 2/4/8) streams the weights fastest.  Model fitted to B200 measurements (us):
//   t = max(weight bytes / 6.0 TB/s, bytes one CTA pulls / 100 GB/s) + exchange + 6
// where a CTA pulls (128 + block_n) * 128 bytes per k-block (the A panel comes from L2 but costs SM ingest all the
// same) and the split-K exchange costs 1.5 + KiB sent / 10.7.  E.g. 128 x 8192 x 8192: one CTA per 64-wide tile
// 37 (measured 39), split-K 128 x 2: 31 (32); 128 x 4096 x 14336: split-K 64 x 2: 36 (37), 128 x 4: 32 (31).
// Returns split = 0 for the persistent kernel (block_n then its tile width).
void plan_one_tile_row(const GemmArgs &g, int sms, int *block_n, int *split) {
    const double k_blocks = static_cast<double>((g.k + 63) / 64);
    const double t_dram = static_cast<double>(g.n) * g.k * 2.0 / 6.0e6;
    double best = 1e300;
    *block_n = 128;
    *split = 0;
    for (int bn = 256; bn >= 64; bn /= 2) {
        const int64_t tiles = (g.n + bn - 1) / bn;
        const double waves = static_cast<double>((tiles + sms - 1) / sms);
        const double t = fmax(t_dram, waves * k_blocks * (128 + bn) * 128.0 / 1.0e5) + 6.0;
        if (t < best) { best = t; *block_n = bn; *split = 0; }
    }
    for (int bn = 128; bn >= 64; bn /= 2) {
        const int64_t tiles = (g.n + bn - 1) / bn;
        for (int sp = 2; sp <= 8; sp *= 2) {
            if (k_blocks < 2 * sp || bn / sp < 8 || tiles * sp * 10 > static_cast<int64_t>(sms) * 11) continue;
            const double per = ceil(k_blocks / sp);
            const double exch = 1.5 + (sp - 1.0) / sp * bn * 128 * 4 / 1024.0 / 10.7;
            const double t = fmax(t_dram, per * (128 + bn) * 128.0 / 1.0e5) + exch + 6.0;
            if (t < best) { best = t; *block_n = bn; *split = sp; }
        }
    }
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
    // variant 3 = cluster split-K; chosen automatically when one CTA per tile would leave more than
    // 40 % of the SMs without a tile and k is long enough to split
    const bool staged_store = g.n_extra_dst > 0 || g.mc_dst != nullptr;    // several destinations or a multicast one:
    if (staged_store && variant == 0)                                       // the persistent kernels only
        choose_config(g, sms, &variant, &block_n);
    if (staged_store && (variant == 3 || variant == 4)) return kLaunchBadConfig;
    if (staged_store && (g.row_scale || g.bias || g.residual)) return kLaunchBadConfig;
    if (g.n_extra_dst > 0 && g.mc_dst != nullptr) return kLaunchBadConfig;
    static const int env_split = tune_env_int("PEAKGEMM_TUNE_SPLITK", -1);
    // variant 4 = skinny kernel (m <= 64, operands swapped); the automatic choice for such m
    static const bool env_no_skinny = tune_env_int("PEAKGEMM_TUNE_SKINNY", 1) == 0;
    if (variant == 4 || (variant == 0 && g.m <= 64 && !env_no_skinny)) {
        if (g.m > 64) return kLaunchBadConfig;
        int forced = 0;
        if (variant == 4 && env_split >= 1 && env_split <= 8 && (env_split & (env_split - 1)) == 0) forced = env_split;
        e = g.bf16 ? launch_skinny_any<true>(g, *d, sms, forced, stream) : launch_skinny_any<false>(g, *d, sms, forced, stream);
        if (e != cudaSuccess) { *cuda_err = e; return kLaunchCuda; }
        return kLaunchOk;
    }
    // variant 6 = pair split-K: a CTA pair per 128 x block_n (m <= 128) or 256 x block_n tile, 1 or 2 pairs over k per
    // cluster; for problems of few tiles
    if (variant == 6) {
        if (staged_store || (block_n != 0 && block_n != 128 && block_n != 256)) return kLaunchBadConfig;
        int ps_bn = 0, sp = 0;
        choose_pair_split(g, sms, block_n, &ps_bn, &sp);
        if (sp == 0) return kLaunchBadConfig;
        if (env_split == 1 || (env_split == 2 && (g.k + 63) / 64 >= 8)) sp = env_split;
        e = g.m <= 128 ? launch_pair_splitk_any<64>(g, *d, ps_bn, sp, stream)
                       : launch_pair_splitk_any<128>(g, *d, ps_bn, sp, stream);
        if (e != cudaSuccess) { *cuda_err = e; return kLaunchCuda; }
        return kLaunchOk;
    }
    if (variant == 0 || variant == 3) {
        int sk_bn = 0, sk_s = 0;
        choose_splitk(g, sms, block_n == 256 ? 0 : block_n, &sk_bn, &sk_s);
        bool use = sk_s >= 2;
        if (variant == 0 && g.m <= 128 && block_n == 0 && env_split != 0) {
            int bn = 0, sp = 0;
            plan_one_tile_row(g, sms, &bn, &sp);
            use = sp >= 2;
            if (use) { sk_bn = bn; sk_s = sp; }
            else { variant = 1; block_n = bn; }
        } else if (use && variant == 0) {
            // Two tile rows (128 < m <= 256): a cluster over k wherever a plan exists and k is long enough to
            // share out (256 x 4096 x 4096: 17.9 us against 21.5-22.4 for the best one-CTA and CTA-pair
            // configurations, cuBLAS 16.4).
            use = env_split != 0 && g.m <= 256 && g.k >= 2048;
        }
        if (variant == 3 && !use) return kLaunchBadConfig;
        if (use) {
            if (env_split >= 2 && variant == 3) sk_s = env_split;
            if (sk_bn == 128) e = g.bf16 ? launch_splitk<128, 5, true>(g, *d, sk_s, stream)
                                         : launch_splitk<128, 5, false>(g, *d, sk_s, stream);
            else e = g.bf16 ? launch_splitk<64, 8, true>(g, *d, sk_s, stream)
                            : launch_splitk<64, 8, false>(g, *d, sk_s, stream);
            if (e != cudaSuccess) { *cuda_err = e; return kLaunchCuda; }
            return kLaunchOk;
        }
    }
    // Few 256 x 256 tiles and a long k (at most 40 tiles, so that two pairs per tile fit the SMs at once): two CTA
    // pairs per cluster share each tile's k range and combine through distributed shared memory.  Measured against
    // the best of the other kernels (us): 512 x 2048 x 8192 25.3 / 31.6, 512 x 4096 x 8192 30.2 / 38.9, 256 x 8192 x
    // 8192 33.9 / 41.9, 384 x 4096 x 14336 47.0 / 53.2, 512 x 4096 x 4096 19.6 / 23.5.
    if (variant == 0 && block_n == 0 && !staged_store && pair_split_pays(g.m, g.n, g.k, sms)) {
        int ps_bn = 0, sp = 0;
        choose_pair_split(g, sms, 0, &ps_bn, &sp);       // 128-wide tiles where 256-wide ones leave SMs idle
        if (sp == 2) {
            e = launch_pair_splitk_any<128>(g, *d, ps_bn, sp, stream);
            if (e != cudaSuccess) { *cuda_err = e; return kLaunchCuda; }
            return kLaunchOk;
        }
    }
    if (variant == 0 && block_n == 0 && g.workspace && g.m > 256 && g.n_extra_dst == 0) {
        uint32_t full = 0, split = 0;
        size_t need = 0;
        plan_tail(g.m, g.n, g.k, sms / 2, &full, &split, &need);
        if (split >= 2 && full == 0 && need <= g.workspace_bytes) { variant = 2; block_n = 256; }
    }
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
    } else if (variant == 5) {
        if (block_n != 256 && block_n != 0) return kLaunchBadConfig;
        e = launch_dt<2, 256, 4, 2>(g, *d, sms, stream);
    } else {
        return kLaunchBadConfig;
    }
    if (e != cudaSuccess) { *cuda_err = e; return kLaunchCuda; }
    return kLaunchOk;
}

// Bytes of workspace with which hgemm_launch (automatic configuration, all SMs) would split the last wave of this
// shape; 0 when it would not.
size_t hgemm_workspace_bytes(int64_t m, int64_t n, int64_t k, int sm_count) {
    if (m <= 256 || k <= 0 || n <= 0) return 0;      // small m: skinny / split-K / one-CTA kernels
    if (pair_split_pays(m, n, k, sm_count)) return 0;   // two pairs per tile through shared memory: no scratch
    uint32_t full = 0, split = 0;
    size_t bytes = 0;
    plan_tail(m, n, k, sm_count / 2, &full, &split, &bytes);
    if (split < 2) return 0;
    if (full == 0) return bytes;                      // all remainder: the launch takes the 256-wide pair kernel for it
    GemmArgs g{nullptr, nullptr, nullptr, m, n, k, k, k, n, true};
    g.workspace = &g;                                 // "a workspace of that size is available": the choice counts on it
    g.workspace_bytes = bytes;
    int variant = 0, block_n = 0;
    choose_config(g, sm_count, &variant, &block_n);
    return (variant == 2 && block_n == 256) ? bytes : 0;
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

#ifdef PG_TEST_SHORT_WAIT
// Test build only: 1 = the first worker's MMA issuer withholds the "accumulator ready" signal of its first tile.
extern "C" int pg_test_withhold_gemm_signal(int on) {
    return static_cast<int>(cudaMemcpyToSymbol(pg::g_test_withhold_acc_commit, &on, sizeof(int)));
}
#endif
