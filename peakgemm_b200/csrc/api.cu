// The C ABI of libPeakGemm_device.so: argument checks, status codes, dispatch.
// Declarations and contracts: include/peakgemm.h.

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/peakgemm.h"
#include "gemm_sm100.h"
#include "host_util.h"
#include "rmsnorm.h"
#include "sgemm.h"

namespace {

thread_local int t_last_cuda_error = 0;

int cuda_fail(cudaError_t e) {
    t_last_cuda_error = static_cast<int>(e);
    cudaGetLastError();   // clear the sticky-free error state of this thread
    return PG_ERR_CUDA;
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int from_launch(int r, cudaError_t e) {
    switch (r) {
        case pg::kLaunchOk: return PG_OK;
        case pg::kLaunchCuda: return cuda_fail(e);
        case pg::kLaunchNotSm100: return PG_ERR_NOT_SM100;
        default: return PG_ERR_BAD_ARG;
    }
}

constexpr int64_t kMaxDim = (int64_t(1) << 31) - 1;

}  // namespace

namespace pg {
int record_cuda_failure(cudaError_t e) { return cuda_fail(e); }
}  // namespace pg

extern "C" {

const char *pg_status_string(int status) {
    switch (status) {
        case PG_OK: return "PG_OK";
        case PG_ERR_BAD_ARG: return "PG_ERR_BAD_ARG: null pointer, negative size or unknown dtype/variant";
        case PG_ERR_MISALIGNED: return "PG_ERR_MISALIGNED: base pointers must be 16-byte aligned";
        case PG_ERR_UNSUPPORTED: return "PG_ERR_UNSUPPORTED: n, k, lda, ldb, ldc and h must be multiples of 8 and within limits";
        case PG_ERR_WORKSPACE: return "PG_ERR_WORKSPACE: workspace too small";
        case PG_ERR_CUDA: return "PG_ERR_CUDA: a CUDA call failed (pg_last_cuda_error)";
        case PG_ERR_DEVICE_TIMEOUT: return "PG_ERR_DEVICE_TIMEOUT: a kernel abandoned a bounded wait";
        case PG_ERR_NOT_SM100: return "PG_ERR_NOT_SM100: the current device is not compute capability 10.x";
        case PG_ERR_STATIC_SCRATCH:
            return "PG_ERR_STATIC_SCRATCH: this shape needs more scratch than the library's built-in "
                   "PG_STATIC_SCRATCH_BYTES; use pg_rmsnorm_bwd with a caller workspace";
        default: return "unknown pg_status";
    }
}

int pg_last_cuda_error(void) { return t_last_cuda_error; }

const char *pg_version(void) { return "0.1"; }

int pg_hgemm_ex(void *c, const void *a, const void *b, int64_t m, int64_t n, int64_t k, int64_t lda,
                int64_t ldb, int64_t ldc, int dtype, int variant, int block_n, int max_sms, void *stream) {
    if (m < 0 || n < 0 || k < 0 || max_sms < 0) return PG_ERR_BAD_ARG;
    if (dtype != PG_F16 && dtype != PG_BF16) return PG_ERR_BAD_ARG;
    if (variant < 0 || variant > 6) return PG_ERR_BAD_ARG;
    if (block_n != 0 && block_n != 64 && block_n != 128 && block_n != 256) return PG_ERR_BAD_ARG;
    if (m == 0 || n == 0) return PG_OK;
    if (!c || (k > 0 && (!a || !b))) return PG_ERR_BAD_ARG;
    if (lda < k || ldb < k || ldc < n) return PG_ERR_BAD_ARG;
    if (n % 8 != 0 || k % 8 != 0 || lda % 8 != 0 || ldb % 8 != 0 || ldc % 8 != 0) return PG_ERR_UNSUPPORTED;
    if (m > kMaxDim || n > kMaxDim || k > kMaxDim) return PG_ERR_UNSUPPORTED;
    if (!aligned16(c) || (k > 0 && (!aligned16(a) || !aligned16(b)))) return PG_ERR_MISALIGNED;
    pg::GemmArgs g{c, a, b, m, n, k, lda, ldb, ldc, dtype == PG_BF16};
    cudaError_t e = cudaSuccess;
    const int r = pg::hgemm_launch(g, variant, block_n, max_sms, static_cast<cudaStream_t>(stream), &e);
    return from_launch(r, e);
}

size_t pg_hgemm_workspace_bytes(int64_t m, int64_t n, int64_t k) {
    if (m <= 0 || n <= 0 || k <= 0) return 0;
    int sms = 0;
    if (pg::current_device_sm_count(&sms) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return pg::hgemm_workspace_bytes(m, n, k, sms);
}

int pg_hgemm_ws(void *c, const void *a, const void *b, int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldb,
                int64_t ldc, int dtype, void *workspace, size_t workspace_bytes, void *stream) {
    if (m < 0 || n < 0 || k < 0) return PG_ERR_BAD_ARG;
    if (dtype != PG_F16 && dtype != PG_BF16) return PG_ERR_BAD_ARG;
    if (m == 0 || n == 0) return PG_OK;
    if (!c || (k > 0 && (!a || !b))) return PG_ERR_BAD_ARG;
    if (lda < k || ldb < k || ldc < n) return PG_ERR_BAD_ARG;
    if (n % 8 != 0 || k % 8 != 0 || lda % 8 != 0 || ldb % 8 != 0 || ldc % 8 != 0) return PG_ERR_UNSUPPORTED;
    if (m > kMaxDim || n > kMaxDim || k > kMaxDim) return PG_ERR_UNSUPPORTED;
    if (!aligned16(c) || (k > 0 && (!aligned16(a) || !aligned16(b)))) return PG_ERR_MISALIGNED;
    if (workspace && (reinterpret_cast<uintptr_t>(workspace) & 255u)) return PG_ERR_MISALIGNED;
    pg::GemmArgs g{c, a, b, m, n, k, lda, ldb, ldc, dtype == PG_BF16};
    g.workspace = workspace_bytes ? workspace : nullptr;
    g.workspace_bytes = workspace ? workspace_bytes : 0;
    cudaError_t e = cudaSuccess;
    const int r = pg::hgemm_launch(g, 0, 0, 0, static_cast<cudaStream_t>(stream), &e);
    return from_launch(r, e);
}

int pg_hgemm_multi(void *const *c_list, int n_dst, const void *a, const void *b, int64_t m, int64_t n, int64_t k,
                   int64_t lda, int64_t ldb, int64_t ldc, int dtype, int max_sms, void *stream) {
    if (!c_list || n_dst < 1 || n_dst > 8) return PG_ERR_BAD_ARG;
    if (m < 0 || n < 0 || k < 0 || max_sms < 0) return PG_ERR_BAD_ARG;
    if (dtype != PG_F16 && dtype != PG_BF16) return PG_ERR_BAD_ARG;
    if (m == 0 || n == 0) return PG_OK;
    if (k == 0) return PG_ERR_UNSUPPORTED;                 // zero-fill of several buffers: use pg_hgemm per buffer
    if (!a || !b) return PG_ERR_BAD_ARG;
    if (lda < k || ldb < k || ldc < n) return PG_ERR_BAD_ARG;
    if (n % 8 != 0 || k % 8 != 0 || lda % 8 != 0 || ldb % 8 != 0 || ldc % 8 != 0) return PG_ERR_UNSUPPORTED;
    if (m > kMaxDim || n > kMaxDim || k > kMaxDim) return PG_ERR_UNSUPPORTED;
    if (!aligned16(a) || !aligned16(b)) return PG_ERR_MISALIGNED;
    for (int i = 0; i < n_dst; ++i) {
        if (!c_list[i]) return PG_ERR_BAD_ARG;
        if (!aligned16(c_list[i])) return PG_ERR_MISALIGNED;
    }
    pg::GemmArgs g{c_list[0], a, b, m, n, k, lda, ldb, ldc, dtype == PG_BF16};
    g.n_extra_dst = n_dst - 1;
    for (int i = 1; i < n_dst; ++i) g.extra_dst[i - 1] = c_list[i];
    cudaError_t e = cudaSuccess;
    const int r = pg::hgemm_launch(g, 0, 0, max_sms, static_cast<cudaStream_t>(stream), &e);
    return from_launch(r, e);
}

int pg_hgemm_mcast(void *c_local, void *c_multicast, const void *a, const void *b, int64_t m, int64_t n, int64_t k,
                   int64_t lda, int64_t ldb, int64_t ldc, int dtype, int max_sms, void *stream) {
    if (m < 0 || n < 0 || k < 0 || max_sms < 0) return PG_ERR_BAD_ARG;
    if (dtype != PG_F16 && dtype != PG_BF16) return PG_ERR_BAD_ARG;
    if (m == 0 || n == 0) return PG_OK;
    if (k == 0) return PG_ERR_UNSUPPORTED;
    if (!a || !b || !c_local || !c_multicast) return PG_ERR_BAD_ARG;
    if (lda < k || ldb < k || ldc < n) return PG_ERR_BAD_ARG;
    if (n % 8 != 0 || k % 8 != 0 || lda % 8 != 0 || ldb % 8 != 0 || ldc % 8 != 0) return PG_ERR_UNSUPPORTED;
    if (m > kMaxDim || n > kMaxDim || k > kMaxDim) return PG_ERR_UNSUPPORTED;
    if (!aligned16(a) || !aligned16(b) || !aligned16(c_local) || !aligned16(c_multicast)) return PG_ERR_MISALIGNED;
    pg::GemmArgs g{c_local, a, b, m, n, k, lda, ldb, ldc, dtype == PG_BF16};
    g.mc_dst = c_multicast;
    cudaError_t e = cudaSuccess;
    const int r = pg::hgemm_launch(g, 0, 0, max_sms, static_cast<cudaStream_t>(stream), &e);
    return from_launch(r, e);
}

int pg_hgemm_fused(void *d, const void *a, const void *b, int64_t m, int64_t n, int64_t k, int64_t lda,
                   int64_t ldb, int64_t ldd, const float *row_scale, const void *bias, const void *residual,
                   int64_t ldr, int dtype, int flags, void *stream) {
    if (m < 0 || n < 0 || k < 0) return PG_ERR_BAD_ARG;
    if (dtype != PG_F16 && dtype != PG_BF16) return PG_ERR_BAD_ARG;
    if (flags & ~PG_FUSED_PDL) return PG_ERR_BAD_ARG;
    if (m == 0 || n == 0) return PG_OK;
    if (k == 0) return PG_ERR_UNSUPPORTED;
    if (!d || !a || !b) return PG_ERR_BAD_ARG;
    if (lda < k || ldb < k || ldd < n) return PG_ERR_BAD_ARG;
    if (residual && ldr < n) return PG_ERR_BAD_ARG;
    if (n % 8 != 0 || k % 8 != 0 || lda % 8 != 0 || ldb % 8 != 0 || ldd % 8 != 0) return PG_ERR_UNSUPPORTED;
    if (residual && ldr % 8 != 0) return PG_ERR_UNSUPPORTED;
    if (m > kMaxDim || n > kMaxDim || k > kMaxDim || (residual && ldr > kMaxDim)) return PG_ERR_UNSUPPORTED;
    if (!aligned16(d) || !aligned16(a) || !aligned16(b)) return PG_ERR_MISALIGNED;
    if ((bias && !aligned16(bias)) || (residual && !aligned16(residual)) ||
        (row_scale && (reinterpret_cast<uintptr_t>(row_scale) & 3u)))
        return PG_ERR_MISALIGNED;
    pg::GemmArgs g{d, a, b, m, n, k, lda, ldb, ldd, dtype == PG_BF16};
    g.row_scale = row_scale;
    g.bias = bias;
    g.residual = residual;
    g.ldr = residual ? ldr : 0;
    g.pdl_wait = (flags & PG_FUSED_PDL) != 0;
    cudaError_t e = cudaSuccess;
    const int r = pg::hgemm_launch(g, 0, 0, 0, static_cast<cudaStream_t>(stream), &e);
    return from_launch(r, e);
}

int pg_rmsnorm_rstd(float *rstd, const void *x, int64_t rows, int64_t h, float eps, int dtype, void *stream) {
    if (rows < 0 || h <= 0) return PG_ERR_BAD_ARG;
    if (dtype != PG_F16 && dtype != PG_BF16) return PG_ERR_BAD_ARG;
    if (rows == 0) return PG_OK;
    if (!rstd || !x) return PG_ERR_BAD_ARG;
    if (h % 8 != 0 || h > kMaxDim) return PG_ERR_UNSUPPORTED;
    if (!aligned16(x) || (reinterpret_cast<uintptr_t>(rstd) & 3u)) return PG_ERR_MISALIGNED;
    const cudaError_t e = pg::rmsnorm_rstd_launch(rstd, x, rows, h, eps, dtype == PG_BF16,
                                                  static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? PG_OK : cuda_fail(e);
}

int pg_hgemm(void *c, const void *a, const void *b, int64_t m, int64_t n, int64_t k, int64_t lda,
             int64_t ldb, int64_t ldc, int dtype, void *stream) {
    return pg_hgemm_ex(c, a, b, m, n, k, lda, ldb, ldc, dtype, 0, 0, 0, stream);
}

int pg_sgemm(float *c, const float *a, const float *b, int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldb,
             int64_t ldc, void *stream) {
    if (m < 0 || n < 0 || k < 0) return PG_ERR_BAD_ARG;
    if (m == 0 || n == 0) return PG_OK;
    if (!c || (k > 0 && (!a || !b))) return PG_ERR_BAD_ARG;
    if (lda < k || ldb < k || ldc < n) return PG_ERR_BAD_ARG;
    if (k % 4 != 0 || lda % 4 != 0 || ldb % 4 != 0 || ldc % 4 != 0) return PG_ERR_UNSUPPORTED;
    if (m > kMaxDim || n > kMaxDim || k > kMaxDim) return PG_ERR_UNSUPPORTED;
    if (!aligned16(c) || (k > 0 && (!aligned16(a) || !aligned16(b)))) return PG_ERR_MISALIGNED;
    const cudaError_t e = pg::sgemm_launch(c, a, b, m, n, k, lda, ldb, ldc, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? PG_OK : cuda_fail(e);
}

int pg_hgemm_config(int64_t m, int64_t n, int64_t k, int sm_count, int *variant, int *block_n) {
    if (m <= 0 || n <= 0 || k < 0 || sm_count < 2 || !variant || !block_n) return PG_ERR_BAD_ARG;
    pg::GemmArgs g{nullptr, nullptr, nullptr, m, n, k, k, k, n, true};
    *variant = 0;
    *block_n = 0;
    pg::choose_config(g, sm_count, variant, block_n);
    return PG_OK;
}

int pg_device_status(int *device_status, void *stream) {
    if (!device_status) return PG_ERR_BAD_ARG;
    cudaError_t e = cudaSuccess;
    int gemm = 0, rms = 0;
    const int r = pg::gemm_device_status(&gemm, static_cast<cudaStream_t>(stream), &e);
    if (r != pg::kLaunchOk) return from_launch(r, e);
    e = pg::rmsnorm_device_status(&rms, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(e);
    *device_status = gemm != 0 ? gemm : rms;
    return *device_status != 0 ? PG_ERR_DEVICE_TIMEOUT : PG_OK;
}

int pg_rmsnorm_fwd(void *y, const void *x, const float *gamma, int64_t rows, int64_t h, float eps,
                   int dtype, void *stream) {
    if (rows < 0 || h <= 0) return PG_ERR_BAD_ARG;
    if (dtype != PG_F16 && dtype != PG_BF16) return PG_ERR_BAD_ARG;
    if (rows == 0) return PG_OK;
    if (!y || !x || !gamma) return PG_ERR_BAD_ARG;
    if (h % 8 != 0 || h > kMaxDim) return PG_ERR_UNSUPPORTED;
    if (!aligned16(y) || !aligned16(x) || !aligned16(gamma)) return PG_ERR_MISALIGNED;
    pg::RmsFwdArgs a{y, x, gamma, rows, h, eps, dtype == PG_BF16};
    const cudaError_t e = pg::rmsnorm_fwd_launch(a, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? PG_OK : cuda_fail(e);
}

size_t pg_rmsnorm_bwd_workspace_bytes(int64_t rows, int64_t h) {
    if (rows <= 0 || h <= 0 || h % 8 != 0 || h > pg::rmsnorm_max_h()) return 0;
    int ctas = 0;
    // the CTA count does not depend on the element type; bf16 and fp16 kernels have the same footprint
    if (pg::rmsnorm_bwd_ctas(rows, h, true, &ctas) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    int ctas16 = 0;
    if (pg::rmsnorm_bwd_ctas(rows, h, false, &ctas16) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    if (ctas16 > ctas) ctas = ctas16;
    return static_cast<size_t>(ctas) * static_cast<size_t>(h) * sizeof(float);
}

int pg_rmsnorm_bwd(void *dx, float *dgamma, const void *dy, const void *x, const float *gamma,
                   int64_t rows, int64_t h, float eps, int dtype, void *workspace,
                   size_t workspace_bytes, void *stream) {
    if (rows < 0 || h <= 0) return PG_ERR_BAD_ARG;
    if (dtype != PG_F16 && dtype != PG_BF16) return PG_ERR_BAD_ARG;
    if (!dgamma) return PG_ERR_BAD_ARG;
    if (h % 8 != 0 || h > pg::rmsnorm_max_h()) return PG_ERR_UNSUPPORTED;
    if (!aligned16(dgamma)) return PG_ERR_MISALIGNED;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (rows == 0) {   // an empty sum
        const cudaError_t e = cudaMemsetAsync(dgamma, 0, static_cast<size_t>(h) * sizeof(float), s);
        return e == cudaSuccess ? PG_OK : cuda_fail(e);
    }
    if (!dx || !dy || !x || !gamma || !workspace) return PG_ERR_BAD_ARG;
    if (!aligned16(dx) || !aligned16(dy) || !aligned16(x) || !aligned16(gamma) || !aligned16(workspace))
        return PG_ERR_MISALIGNED;
    int ctas = 0;
    cudaError_t e = pg::rmsnorm_bwd_ctas(rows, h, dtype == PG_BF16, &ctas);
    if (e != cudaSuccess) return cuda_fail(e);
    if (workspace_bytes < static_cast<size_t>(ctas) * static_cast<size_t>(h) * sizeof(float))
        return PG_ERR_WORKSPACE;
    pg::RmsBwdArgs a{dx, dgamma, dy, x, gamma, rows, h, eps, dtype == PG_BF16, workspace};
    e = pg::rmsnorm_bwd_launch(a, ctas, s);
    return e == cudaSuccess ? PG_OK : cuda_fail(e);
}

}  // extern "C"
