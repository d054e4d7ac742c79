/*
 * peakgemm.h — C ABI of libPeakGemm_device.so (B200 / sm_100a only).
 *
 * Torch-free.  Every pointer is a DEVICE pointer on the device that is current
 * when the call is made; every call is asynchronous on `stream` (a cudaStream_t
 * passed as void*; NULL = the legacy default stream) and returns a pg_status.
 * No call synchronises the device, and none allocates device memory except
 * where a comment says so.
 *
 * The interface it replaces in the reference project (xytpai/PeakGemm) is the
 * header-only launcher
 *     hgemm::hgemm_peak(short* c, const short* a, const short* b,
 *                       uint32 m, uint32 n, uint32 k, bool is_bf16, stream)
 *         src/impl/hgemm_wmma_impl.h:412-423
 * that src/ops/gemm.cpp:14-33 calls from the `gemm_peak` torch operator
 * (src/register.cpp:4-7).
 */
#ifndef PEAKGEMM_H_
#define PEAKGEMM_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Element types of A, B, C (GEMM) and x, y, dy, dx (RMSNorm). */
enum pg_dtype { PG_F16 = 0, PG_BF16 = 1 };

enum pg_status {
    PG_OK = 0,
    PG_ERR_BAD_ARG = 1,        /* null pointer, negative size, unknown dtype           */
    PG_ERR_MISALIGNED = 2,     /* a base pointer is not 16-byte aligned                */
    PG_ERR_UNSUPPORTED = 3,    /* n%8, k%8, ld%8 or H%8 violated, or size over a limit */
    PG_ERR_WORKSPACE = 4,      /* caller's workspace is too small                      */
    PG_ERR_CUDA = 5,           /* a CUDA runtime/driver call failed (see pg_last_cuda_error) */
    PG_ERR_DEVICE_TIMEOUT = 6, /* a kernel gave up on a bounded wait (see pg_device_status)  */
    PG_ERR_NOT_SM100 = 7,      /* the current device is not compute capability 10.x    */
    PG_ERR_STATIC_SCRATCH = 8  /* shape needs more than PG_STATIC_SCRATCH_BYTES of built-in scratch */
};

/* Human-readable name of a pg_status value; never NULL. */
const char *pg_status_string(int status);

/* cudaError_t (as int) of the last failing CUDA call made by this library on the
 * calling thread, 0 if none. */
int pg_last_cuda_error(void);

/* Library version, "major.minor". */
const char *pg_version(void);

/*
 * C[m,n] = A[m,k] * B[n,k]^T  (the reference's "TN" problem: A row-major,
 * B stored [n,k] i.e. column-major [k,n]); products of the 16-bit inputs are
 * accumulated in fp32 and rounded to nearest-even into C's 16-bit type; C is
 * overwritten (no alpha/beta).
 *
 * Replaces hgemm::hgemm_peak (src/impl/hgemm_wmma_impl.h:412-423), with three
 * additions: explicit row pitches lda/ldb/ldc in ELEMENTS (pass k, k, n for the
 * reference's dense layout; ldc > n lets a column-sharded caller write its block
 * straight into a full-width C), 64-bit sizes, and a status code in place of the
 * reference's host assert (hgemm_wmma_impl.h:389-390).
 *
 * Preconditions (same as the reference's): n % 8 == 0, k % 8 == 0; additionally
 * lda, ldb, ldc % 8 == 0 and 16-byte aligned base pointers.  m, n, k may be any
 * size otherwise (row/column/k tails are handled; the reference reads out of
 * bounds for m or n not a multiple of 128).  m == 0 or n == 0 is a no-op; k == 0
 * zero-fills C.
 *
 * The kernel is a persistent, warp-specialised TMA + tcgen05 kernel with fp32
 * accumulators in tensor memory.  It uses no scratch memory.
 */
int pg_hgemm(void *c, const void *a, const void *b,
             int64_t m, int64_t n, int64_t k,
             int64_t lda, int64_t ldb, int64_t ldc,
             int dtype, void *stream);

/*
 * Same contract as pg_hgemm, with the kernel variant chosen by the caller:
 *   variant 0 = automatic (what pg_hgemm uses)
 *   variant 1 = one CTA per 128 x block_n tile   (tcgen05 cta_group::1)
 *   variant 2 = CTA pair per 256 x block_n tile  (tcgen05 cta_group::2)
 *   variant 3 = cluster split-K: a cluster of 2, 4 or 8 CTAs shares one 128 x block_n
 *               tile (block_n 64 or 128), each CTA a slice of k; the partial sums are
 *               combined through distributed shared memory, no global scratch.
 *               PG_ERR_BAD_ARG if the shape admits no split (k < 256, or too many tiles)
 *   variant 4 = skinny kernel for m <= 64 (weight streaming): the weights take the
 *               128-row side of the MMA, the tokens its 16/32/64-wide side, 8-10 TMA
 *               stages deep (or two resident CTAs per SM of 5-6 stages each: up to 16 tokens,
 *               and 17-32 tokens with more tiles than SMs), optional cluster split-K as in
 *               variant 3; block_n ignored.
 *               PG_ERR_BAD_ARG if m > 64
 *   variant 5 = CTA pair per 512 x 256 tile: two 256-row blocks share every k-block of B
 *               and their two accumulators fill tensor memory (25 % fewer operand bytes
 *               per flop from L2 than variant 2 at block_n 256); block_n 0 or 256
 *   variant 6 = pair split-K for problems of few tiles: a CTA pair per 256 x block_n tile (m <= 128:
 *               per 128 x block_n tile, a 2-CTA MMA at M = 128 in which each CTA loads 64 rows of
 *               A), 1 or 2 pairs over k per cluster, partial sums through distributed shared
 *               memory; block_n 0, 128 or 256.  The automatic choice for 128 < m, at most 40
 *               tiles of 256 x 256 and k >= 4096 (for m <= 128 it measured slower than variants
 *               1 and 3 and is never chosen); PG_ERR_BAD_ARG if the tiles exceed one wave of CTAs
 *   block_n   = 0 (automatic), 64, 128 or 256
 *   max_sms   = 0 (all SMs), or the number of SMs the persistent grid may occupy;
 *               a caller that overlaps a collective with the GEMM leaves a few
 *               SMs free for the collective's kernels this way
 * Meant for benchmarks, tests and the sharded caller; the reference fixes one
 * configuration at compile time (REGISTER_HGEMM_WMMA_M16N8K16_IMPL,
 * hgemm_wmma_impl.h:410) and launches one CTA per tile (get_grid, :373-378).
 */
int pg_hgemm_ex(void *c, const void *a, const void *b,
                int64_t m, int64_t n, int64_t k,
                int64_t lda, int64_t ldb, int64_t ldc,
                int dtype, int variant, int block_n, int max_sms, void *stream);

/*
 * pg_hgemm with an optional scratch buffer that lets the kernel split the LAST, partial wave of output
 * tiles: when the tiles do not fill a whole number of waves of the persistent grid and the remainder
 * occupies at most half of the SM pairs and k is long enough for the exchange to pay (about k >= 8192), each
 * remainder tile is cut into 2-8 slices of k that run on the otherwise idle SM pairs (a problem of at most half
 * a wave is all remainder: every tile is split); the slices' fp32 partial sums pass through `workspace` and are added in slice
 * order (deterministic) before the one rounding.  Results differ from pg_hgemm only by the fp32 summation
 * order of those tiles.  pg_hgemm_workspace_bytes(m, n, k) gives the size that enables the split on the
 * current device (0: this shape would not be split; then workspace may be NULL).  A smaller or NULL
 * workspace simply disables the split.  workspace: 256-byte aligned device memory, private to this call until
 * the kernel has finished (two calls that overlap on the GPU need two buffers); it needs no
 * initialisation (the call clears the flag words it uses with one cudaMemsetAsync on `stream`).  A split
 * launch is a cooperative launch (the tile owners wait, bounded, for helper CTAs of the same grid); where
 * the device refuses that, the call runs unsplit.
 * The reference has no counterpart: it launches one CTA per tile (get_grid, hgemm_wmma_impl.h:373-378).
 */
size_t pg_hgemm_workspace_bytes(int64_t m, int64_t n, int64_t k);
int pg_hgemm_ws(void *c, const void *a, const void *b,
                int64_t m, int64_t n, int64_t k,
                int64_t lda, int64_t ldb, int64_t ldc,
                int dtype, void *workspace, size_t workspace_bytes, void *stream);

/*
 * pg_hgemm with a fused epilogue, every term optional (null pointer = absent):
 *     d[i,j] = round_to_dtype(row_scale[i] * sum_k a[i,k] b[j,k] + bias[j] + residual[i,j])
 * evaluated in fp32 from the fp32 accumulator with ONE rounding at the end (the
 * unfused sequence rounds after the GEMM and again after each addition).
 *   row_scale  [m] fp32.  With row_scale = the rstd of RMSNorm (pg_rmsnorm_rstd) and
 *              gamma folded into the weights once (b[j,k] = w[j,k] * gamma[k]) this is
 *              RMSNorm followed by the projection, without the normalised
 *              activations ever being written or re-read
 *   bias       [n] of `dtype`
 *   residual   [m, n] of `dtype`, row pitch ldr (elements, % 8 == 0, >= n); may be d
 *              itself with ldr == ldd (d += ...): every element is read by the thread
 *              that produces it before it is stored.  Any other overlap of d with an
 *              input is undefined
 *   flags      PG_FUSED_PDL: launch with programmatic stream serialisation.  The
 *              grid may start while the PREVIOUS kernel on `stream` is still
 *              draining, and only the epilogue waits for it (griddepcontrol.wait)
 *              before reading row_scale.  Set it only when that previous kernel is
 *              the pg_rmsnorm_rstd call producing row_scale and a, b, bias,
 *              residual were complete before that call was issued; ignored when
 *              row_scale is null
 * Same preconditions and kernels as pg_hgemm (the automatic choice between the
 * persistent, split-K and skinny kernels; all three carry the epilogue).  k == 0
 * is not accepted here (PG_ERR_UNSUPPORTED).  The reference's epilogue is a plain
 * cast (src/impl/wmma_utils.h:101-112); it has no fused variant.
 */
#define PG_FUSED_PDL 1
int pg_hgemm_fused(void *d, const void *a, const void *b,
                   int64_t m, int64_t n, int64_t k,
                   int64_t lda, int64_t ldb, int64_t ldd,
                   const float *row_scale, const void *bias,
                   const void *residual, int64_t ldr,
                   int dtype, int flags, void *stream);

/*
 * fp32 C[m,n] = A[m,k] * B[n,k]^T with true fp32 FMA accumulation (CUDA cores, no
 * TF32): the float branch of the gemm_peak operator, where the reference calls
 * sgemm::sgemm_peak (src/ops/gemm.cpp:34-43, src/impl/sgemm_impl.h:310-320) — by its
 * README an unoptimised reference path (README.md:46-47), and not the hot path here
 * either.  Pitches in elements; k, lda, ldb, ldc multiples of 4; 16-byte aligned
 * pointers; any m, n.
 */
int pg_sgemm(float *c, const float *a, const float *b, int64_t m, int64_t n, int64_t k,
             int64_t lda, int64_t ldb, int64_t ldc, void *stream);

/*
 * pg_hgemm with n_dst (1..8) destinations: the same C block is stored to every
 * buffer in c_list (all with row pitch ldc), each 32 x 64 output box going out by
 * one TMA store per destination straight from the epilogue's staging buffer.
 *
 * This is the fused "GEMM + all-gather" of the column-sharded layout: c_list[0] is
 * the rank's own column block inside its full-width C, the other entries are the
 * same block inside the PEER GPUs' C buffers (peer-mapped device pointers, e.g.
 * from CUDA IPC), so the gather crosses NVLink tile by tile while the GEMM runs and
 * no collective library call is needed.  Only stores ever touch peer memory.
 * The writes are complete when the kernel has finished; ranks still need their own
 * barrier before reading what the others wrote.  Uses the persistent kernels
 * (variants 1 and 2).  The reference project has no multi-GPU code.
 */
int pg_hgemm_multi(void *const *c_list, int n_dst, const void *a, const void *b,
                   int64_t m, int64_t n, int64_t k,
                   int64_t lda, int64_t ldb, int64_t ldc,
                   int dtype, int max_sms, void *stream);

/*
 * pg_hgemm with the output written through a MULTICAST address: c_multicast is one
 * virtual address bound to a buffer on every GPU of a group (an NVLink-switch
 * multicast mapping, e.g. torch symmetric memory's multicast_ptr or
 * cuMulticastBindMem), offset to this caller's column block; ldc is the row pitch of
 * the full matrix.  Every 16-byte store (multimem.st) is replicated by the switch
 * into every GPU's copy, the caller's own included: a column-sharded caller's block
 * leaves its GPU once instead of once per peer, and after the callers' barrier every
 * GPU holds the whole row-major C.  Nothing is loaded through the address.
 * c_local is the same element in the caller's OWN copy (a plain device address); the
 * kernel does not write through it.  The persistent kernels only; no fused epilogue
 * terms.  The memory must stay bound until every rank's kernel has completed.
 * The reference project has no multi-GPU code.
 */
int pg_hgemm_mcast(void *c_local, void *c_multicast, const void *a, const void *b,
                   int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldb, int64_t ldc,
                   int dtype, int max_sms, void *stream);

/*
 * Buffers that GPUs of other processes can store into (for pg_hgemm_multi), one
 * node.  pg_peer_alloc: cudaMalloc + CUDA IPC export (handle_out receives
 * PG_PEER_HANDLE_BYTES bytes to send to the peers).  pg_peer_open: maps a peer's
 * buffer into the calling process FOR THE DEVICE THAT IS CURRENT at the call (peer
 * access is enabled lazily); the returned pointer is valid in kernels of that
 * device.  pg_peer_close / pg_peer_free undo them.  These four calls allocate or map
 * memory and synchronise; they belong to set-up, not to the hot path.
 * No counterpart in the reference project (it has no multi-GPU code).
 */
#define PG_PEER_HANDLE_BYTES 64
int pg_peer_alloc(size_t bytes, void **ptr, void *handle_out);
int pg_peer_open(const void *handle, void **ptr);
int pg_peer_close(void *ptr);
int pg_peer_free(void *ptr);
int pg_peer_last_cuda_error(void);

/*
 * The configuration pg_hgemm would choose for this shape on a device with
 * sm_count SMs: writes variant (1, 2 or 5) and block_n (64, 128, 256).  Pure host
 * arithmetic, needs no GPU.  (The reference's counterpart is the fixed
 * instantiation at hgemm_wmma_impl.h:410,421.)
 */
int pg_hgemm_config(int64_t m, int64_t n, int64_t k, int sm_count, int *variant, int *block_n);

/*
 * Device-side status word of the kernels on the current device: 0 if no kernel
 * has given up on a bounded wait since the last call, otherwise a code that names
 * the waiting role (1-5: GEMM producer / MMA / epilogue; 11-12: RMSNorm).
 * Synchronises `stream`, reads the word, clears it and writes it to
 * *device_status.  Returns PG_OK when the word was 0, PG_ERR_DEVICE_TIMEOUT when a
 * kernel had given up (the output of that launch is then incomplete; the context
 * stays usable and later launches are unaffected), or another error status.
 * The word belongs to the DEVICE, not to a stream: kernels of every stream report
 * into it and a read clears it, so poll from ONE place per device, after the
 * streams of interest have been synchronised; two pollers would take each
 * other's codes.
 */
int pg_device_status(int *device_status, void *stream);

/*
 * RMSNorm forward over `rows` rows of length h:
 *     rstd_r = rsqrt(mean_j(x[r,j]^2) + eps)
 *     y[r,j] = round_to_dtype((x[r,j] * rstd_r) * gamma[j])
 * x, y: [rows, h] of `dtype`, dense row-major; gamma: [h] fp32.  All arithmetic
 * in fp32.  Requires h % 8 == 0.  Uses no scratch memory.
 *
 * The reference project has no RMSNorm operator; this entry point follows the
 * conventions of its GEMM launcher (outputs first, caller-allocated buffers,
 * asynchronous on the given stream).
 */
int pg_rmsnorm_fwd(void *y, const void *x, const float *gamma,
                   int64_t rows, int64_t h, float eps, int dtype, void *stream);

/*
 * rstd[r] = rsqrt(mean_j(x[r,j]^2) + eps), fp32, for the rows of x ([rows, h] of
 * `dtype`, dense): the per-row scale pg_hgemm_fused applies (see there).  Reads x
 * once; h % 8 == 0.  The kernel releases its stream dependents as soon as it
 * starts, which only matters to a following launch that asks for programmatic
 * serialisation (PG_FUSED_PDL).  No counterpart in the reference project.
 */
int pg_rmsnorm_rstd(float *rstd, const void *x, int64_t rows, int64_t h, float eps,
                    int dtype, void *stream);

/* Bytes of scratch pg_rmsnorm_bwd needs for this shape on the current device. */
size_t pg_rmsnorm_bwd_workspace_bytes(int64_t rows, int64_t h);

/*
 * RMSNorm backward.  With xhat = x * rstd and g = dy * gamma (fp32):
 *     dx[r,j]   = round_to_dtype(rstd_r * (g[r,j] - xhat[r,j] * mean_j(g[r,:] * xhat[r,:])))
 *     dgamma[j] = sum_r dy[r,j] * xhat[r,j]                       (fp32, overwritten)
 * rstd is recomputed from x, so no saved state crosses the interface.
 * dy, x, dx: [rows, h] of `dtype`; gamma, dgamma: [h] fp32.  Requires h % 8 == 0.
 *
 * dgamma is reduced in two passes and is deterministic: every CTA writes one
 * fp32 partial row into `workspace` ([n_cta, h] fp32, at least
 * pg_rmsnorm_bwd_workspace_bytes bytes, 16-byte aligned), then a second kernel
 * sums the partial rows in a fixed order.  The workspace needs no initialisation.
 */
int pg_rmsnorm_bwd(void *dx, float *dgamma, const void *dy, const void *x,
                   const float *gamma, int64_t rows, int64_t h, float eps,
                   int dtype, void *workspace, size_t workspace_bytes, void *stream);

/*
 * RMSNorm backward without any allocation — no counterpart in the reference
 * project (which has neither RMSNorm nor a scratch-using kernel).
 *
 * Same arithmetic, same kernels and bit-identical results as pg_rmsnorm_bwd, but
 * the caller passes no workspace: the table of fp32 dgamma partial rows lives in
 * a fixed array inside the library (PG_STATIC_SCRATCH_BYTES per GPU, resident
 * from the moment the library is loaded on that GPU until the process exits).
 * Meant for hosts that cannot call cudaMalloc or any allocator where this runs:
 * plugins invoked inside another framework's stream-ordered region, latency-
 * critical loops that must not take allocator locks, plain C/Fortran hosts that
 * only hold raw device pointers.  The call itself makes no cudaMalloc, cudaFree
 * or other allocating call.
 *
 * Limits and rules:
 *  - the shape must fit: pg_rmsnorm_bwd_workspace_bytes(rows, h) <=
 *    PG_STATIC_SCRATCH_BYTES (e.g. h <= 8192 on a 148-SM B200); otherwise the
 *    call does nothing and returns PG_ERR_STATIC_SCRATCH;
 *  - the first call on each device looks up the array's device address (the
 *    device must be current); make that first call before starting any stream
 *    capture;
 *  - every call on a device shares the one array.  Nothing in it has to start at
 *    zero (each partial row is fully written before it is read), but two calls
 *    whose kernels overlap on the GPU — different streams, no ordering between
 *    them — race on it and corrupt each other's dgamma.  Serialise them, or use
 *    pg_rmsnorm_bwd with separate workspaces.
 *  - The looked-up device address is cached per device ordinal for the life of
 *    the process; it assumes the device's primary context is not reset
 *    (cudaDeviceReset) between calls.
 */
#define PG_STATIC_SCRATCH_BYTES (160u * 8192u * 4u)
int pg_rmsnorm_bwd_static(void *dx, float *dgamma, const void *dy, const void *x,
                          const float *gamma, int64_t rows, int64_t h, float eps,
                          int dtype, void *stream);

/*
 * Roofline probes, the sm_100a counterparts of the reference's stand-alone probes
 * (test/cpp/test_wmma_compute.cpp:142-173, the README's "PEAK" column; and
 * test/cpp/test_memory_bandwidth.cpp:95-114).
 * pg_probe_tensor_peak: every SM pair issues tcgen05.mma.cta_group::2 256x256x16
 * back to back on pseudo-random operand tiles resident in shared memory, `iters`
 * rounds of k = 64, no loads in the loop; writes the TFLOP/s reached (and the
 * milliseconds).  Synchronises the device's default stream; allocates nothing.
 * 1 <= iters <= PG_PROBE_MAX_ITERS (about 0.4 s of MMAs; PG_ERR_BAD_ARG beyond).
 * pg_probe_copy: 128-bit streaming copy, asynchronous on `stream`.
 */
#define PG_PROBE_MAX_ITERS (1 << 20)
int pg_probe_tensor_peak(int dtype, int iters, float *tflops_out, float *ms_out);
int pg_probe_copy(void *dst, const void *src, size_t bytes, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* PEAKGEMM_H_ */
