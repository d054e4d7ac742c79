// libPeakGemm.so: the PyTorch operator surface over the C ABI (include/peakgemm.h).
// Plain C++ (no CUDA code in this file), so it never needs nvcc.
//
// Mirrors the reference project's registration and host code:
//   TORCH_LIBRARY(PeakGemm, m) with the schema string of src/register.cpp:4-7,
//   gemm_peak(Tensor& c, Tensor& a, Tensor& b, int64 m, n, k) of src/ops/gemm.cpp:5-45:
//   contiguity check, device guard on `a`, the current CUDA stream, dispatch on a's dtype,
//   asynchronous launch, nothing returned, `c` written in place.
// Differences, all on the error side: arguments the reference leaves unchecked
// (device, dtype equality, shapes against m/n/k) raise c10::Error here instead of
// reading out of bounds, and fp64 inputs are refused with a message (in the reference
// they fall into the float branch and throw inside data_ptr<float>, gemm.cpp:34-37).
// float32 goes to pg_sgemm, as the reference sends it to sgemm_peak.
//
// rms_norm_fwd / rms_norm_bwd have no counterpart in the reference; they follow
// the same conventions: outputs first, caller-allocated, in place, return ().
//
// The reference's schema does not say that `c` is written (no `Tensor(a!)`), so a tracing
// compiler sees an operator without outputs or side effects and may drop it.  The schema string
// is kept verbatim for compatibility; next to it every operator has a twin `<name>_out` whose schema
// marks the written tensors, registered for the CUDA key only (so fake/meta tracing never reaches the
// kernels; the fake implementations live in the Python package).  gemm_peak_fused and rms_norm_rstd
// (fused epilogue, RMSNorm folded into the projection) exist only in the annotated form.

#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/core/DeviceGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include "../../include/peakgemm.h"

namespace {

using at::Tensor;

int dtype_code(const Tensor &t, const char *op) {
    if (t.scalar_type() == at::kHalf) return PG_F16;
    if (t.scalar_type() == at::kBFloat16) return PG_BF16;
    TORCH_CHECK(false, op, ": only float16 and bfloat16 are built for sm_100a, got ", t.scalar_type());
    return -1;
}

void check_status(int st, const char *op) {
    TORCH_CHECK(st == PG_OK, op, ": ", pg_status_string(st),
                st == PG_ERR_CUDA ? " cudaError=" : "", st == PG_ERR_CUDA ? std::to_string(pg_last_cuda_error()) : "");
}

void gemm_peak(Tensor &c, Tensor &a, Tensor &b, int64_t m, int64_t n, int64_t k) {
    TORCH_CHECK(c.is_contiguous() && a.is_contiguous() && b.is_contiguous());
    TORCH_CHECK(a.is_cuda() && b.is_cuda() && c.is_cuda(), "gemm_peak: tensors must be on a CUDA device");
    TORCH_CHECK(a.device() == b.device() && a.device() == c.device(), "gemm_peak: tensors on different devices");
    TORCH_CHECK(a.scalar_type() == b.scalar_type() && a.scalar_type() == c.scalar_type(),
                "gemm_peak: a, b, c must have one dtype");
    TORCH_CHECK(m >= 0 && n >= 0 && k >= 0 && a.numel() == m * k && b.numel() == n * k && c.numel() == m * n,
                "gemm_peak: tensor sizes do not match m, n, k");
    c10::DeviceGuard device_guard(a.device());
    auto stream = at::cuda::getCurrentCUDAStream();
    if (a.scalar_type() == at::kFloat) {      // the reference's sgemm_peak branch (src/ops/gemm.cpp:34-43)
        check_status(pg_sgemm(c.data_ptr<float>(), a.data_ptr<float>(), b.data_ptr<float>(), m, n, k, k, k, n,
                              stream.stream()),
                     "gemm_peak");
        return;
    }
    const int dt = dtype_code(a, "gemm_peak");
    // Shapes whose last wave of tiles is mostly empty run that wave split over k; the scratch for the partial
    // sums comes from torch's caching allocator (stream-ordered, no cudaMalloc in steady state, capturable).
    const size_t ws_bytes = pg_hgemm_workspace_bytes(m, n, k);
    if (ws_bytes > 0) {
        Tensor ws = at::empty({static_cast<int64_t>(ws_bytes)}, a.options().dtype(at::kByte));
        check_status(pg_hgemm_ws(c.data_ptr(), a.data_ptr(), b.data_ptr(), m, n, k, k, k, n, dt, ws.data_ptr(),
                                 ws_bytes, stream.stream()),
                     "gemm_peak");
        return;
    }
    check_status(pg_hgemm(c.data_ptr(), a.data_ptr(), b.data_ptr(), m, n, k, k, k, n, dt, stream.stream()),
                 "gemm_peak");
}

void rms_norm_fwd(Tensor &y, Tensor &x, Tensor &gamma, double eps) {
    TORCH_CHECK(y.is_contiguous() && x.is_contiguous() && gamma.is_contiguous());
    TORCH_CHECK(x.is_cuda() && y.is_cuda() && gamma.is_cuda(), "rms_norm_fwd: tensors must be on a CUDA device");
    TORCH_CHECK(x.device() == y.device() && x.device() == gamma.device(), "rms_norm_fwd: tensors on different devices");
    TORCH_CHECK(x.dim() >= 1 && x.sizes() == y.sizes() && x.scalar_type() == y.scalar_type(),
                "rms_norm_fwd: y must have x's shape and dtype");
    const int64_t h = x.size(-1);
    TORCH_CHECK(gamma.scalar_type() == at::kFloat && gamma.numel() == h, "rms_norm_fwd: gamma must be float32 [h]");
    const int64_t rows = h > 0 ? x.numel() / h : 0;
    const int dt = dtype_code(x, "rms_norm_fwd");
    c10::DeviceGuard device_guard(x.device());
    auto stream = at::cuda::getCurrentCUDAStream();
    check_status(pg_rmsnorm_fwd(y.data_ptr(), x.data_ptr(), gamma.data_ptr<float>(), rows, h,
                                static_cast<float>(eps), dt, stream.stream()),
                 "rms_norm_fwd");
}

void rms_norm_bwd(Tensor &dx, Tensor &dgamma, Tensor &dy, Tensor &x, Tensor &gamma, double eps) {
    TORCH_CHECK(dx.is_contiguous() && dgamma.is_contiguous() && dy.is_contiguous() && x.is_contiguous() &&
                gamma.is_contiguous());
    TORCH_CHECK(x.is_cuda() && dx.is_cuda() && dy.is_cuda() && gamma.is_cuda() && dgamma.is_cuda(),
                "rms_norm_bwd: tensors must be on a CUDA device");
    TORCH_CHECK(x.device() == dx.device() && x.device() == dy.device() && x.device() == gamma.device() &&
                    x.device() == dgamma.device(),
                "rms_norm_bwd: tensors on different devices");
    TORCH_CHECK(x.dim() >= 1 && x.sizes() == dx.sizes() && x.sizes() == dy.sizes() &&
                    x.scalar_type() == dx.scalar_type() && x.scalar_type() == dy.scalar_type(),
                "rms_norm_bwd: dx and dy must have x's shape and dtype");
    const int64_t h = x.size(-1);
    TORCH_CHECK(gamma.scalar_type() == at::kFloat && gamma.numel() == h && dgamma.scalar_type() == at::kFloat &&
                    dgamma.numel() == h,
                "rms_norm_bwd: gamma and dgamma must be float32 [h]");
    const int64_t rows = h > 0 ? x.numel() / h : 0;
    const int dt = dtype_code(x, "rms_norm_bwd");
    c10::DeviceGuard device_guard(x.device());
    auto stream = at::cuda::getCurrentCUDAStream();
    // Scratch for the per-CTA dgamma partial rows comes from torch's caching
    // allocator: stream-ordered, no cudaMalloc in steady state.
    const size_t ws_bytes = pg_rmsnorm_bwd_workspace_bytes(rows, h);
    Tensor ws = at::empty({static_cast<int64_t>(ws_bytes > 0 ? ws_bytes : 16)}, x.options().dtype(at::kByte));
    check_status(pg_rmsnorm_bwd(dx.data_ptr(), dgamma.data_ptr<float>(), dy.data_ptr(), x.data_ptr(),
                                gamma.data_ptr<float>(), rows, h, static_cast<float>(eps), dt, ws.data_ptr(),
                                ws_bytes, stream.stream()),
                 "rms_norm_bwd");
}

void gemm_peak_out(Tensor &c, const Tensor &a, const Tensor &b) {
    TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && c.dim() == 2, "gemm_peak_out: a [m,k], b [n,k], c [m,n]");
    Tensor a2 = a, b2 = b;
    gemm_peak(c, a2, b2, a.size(0), b.size(0), a.size(1));
}

void rms_norm_fwd_out(Tensor &y, const Tensor &x, const Tensor &gamma, double eps) {
    Tensor x2 = x, g2 = gamma;
    rms_norm_fwd(y, x2, g2, eps);
}

void rms_norm_bwd_out(Tensor &dx, Tensor &dgamma, const Tensor &dy, const Tensor &x, const Tensor &gamma,
                      double eps) {
    Tensor dy2 = dy, x2 = x, g2 = gamma;
    rms_norm_bwd(dx, dgamma, dy2, x2, g2, eps);
}

void rms_norm_rstd(Tensor &rstd, const Tensor &x, double eps) {
    TORCH_CHECK(x.is_cuda() && rstd.is_cuda() && x.device() == rstd.device(), "rms_norm_rstd: CUDA tensors on one device");
    TORCH_CHECK(x.is_contiguous() && rstd.is_contiguous() && x.dim() >= 1);
    const int64_t h = x.size(-1);
    const int64_t rows = h > 0 ? x.numel() / h : 0;
    TORCH_CHECK(rstd.scalar_type() == at::kFloat && rstd.numel() == rows, "rms_norm_rstd: rstd must be float32 [rows]");
    const int dt = dtype_code(x, "rms_norm_rstd");
    c10::DeviceGuard device_guard(x.device());
    auto stream = at::cuda::getCurrentCUDAStream();
    check_status(pg_rmsnorm_rstd(rstd.data_ptr<float>(), x.data_ptr(), rows, h, static_cast<float>(eps), dt,
                                 stream.stream()),
                 "rms_norm_rstd");
}

// d[m,n] = row_scale[:,None] * (a[m,k] @ b[n,k]^T) + bias[None,:] + residual, each term optional.
void gemm_peak_fused(Tensor &d, const Tensor &a, const Tensor &b, const std::optional<Tensor> &row_scale,
                     const std::optional<Tensor> &bias, const std::optional<Tensor> &residual, bool pdl) {
    TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && d.dim() == 2, "gemm_peak_fused: a [m,k], b [n,k], d [m,n]");
    TORCH_CHECK(d.is_contiguous() && a.is_contiguous() && b.is_contiguous());
    TORCH_CHECK(a.is_cuda() && b.is_cuda() && d.is_cuda() && a.device() == b.device() && a.device() == d.device(),
                "gemm_peak_fused: tensors must be on one CUDA device");
    TORCH_CHECK(a.scalar_type() == b.scalar_type() && a.scalar_type() == d.scalar_type(),
                "gemm_peak_fused: a, b, d must have one dtype");
    const int64_t m = a.size(0), k = a.size(1), n = b.size(0);
    TORCH_CHECK(b.size(1) == k && d.size(0) == m && d.size(1) == n, "gemm_peak_fused: shapes do not match");
    const float *rs = nullptr;
    const void *bias_p = nullptr, *res_p = nullptr;
    if (row_scale) {
        TORCH_CHECK(row_scale->is_cuda() && row_scale->device() == a.device() && row_scale->is_contiguous() &&
                        row_scale->scalar_type() == at::kFloat && row_scale->numel() == m,
                    "gemm_peak_fused: row_scale must be float32 [m] on a's device");
        rs = row_scale->data_ptr<float>();
    }
    if (bias) {
        TORCH_CHECK(bias->is_cuda() && bias->device() == a.device() && bias->is_contiguous() &&
                        bias->scalar_type() == a.scalar_type() && bias->numel() == n,
                    "gemm_peak_fused: bias must be [n] of a's dtype on a's device");
        bias_p = bias->data_ptr();
    }
    if (residual) {
        TORCH_CHECK(residual->is_cuda() && residual->device() == a.device() && residual->is_contiguous() &&
                        residual->scalar_type() == a.scalar_type() && residual->dim() == 2 &&
                        residual->size(0) == m && residual->size(1) == n,
                    "gemm_peak_fused: residual must be [m,n] of a's dtype on a's device");
        res_p = residual->data_ptr();
    }
    const int dt = dtype_code(a, "gemm_peak_fused");
    c10::DeviceGuard device_guard(a.device());
    auto stream = at::cuda::getCurrentCUDAStream();
    check_status(pg_hgemm_fused(d.data_ptr(), a.data_ptr(), b.data_ptr(), m, n, k, k, k, n, rs, bias_p, res_p, n, dt,
                                pdl ? PG_FUSED_PDL : 0, stream.stream()),
                 "gemm_peak_fused");
}

}  // namespace

TORCH_LIBRARY(PeakGemm, m) {
    m.def("gemm_peak(Tensor c, Tensor a, Tensor b, SymInt m, SymInt n, SymInt k) -> ()");
    m.impl("gemm_peak", &gemm_peak);
    m.def("rms_norm_fwd(Tensor y, Tensor x, Tensor gamma, float eps) -> ()");
    m.impl("rms_norm_fwd", &rms_norm_fwd);
    m.def("rms_norm_bwd(Tensor dx, Tensor dgamma, Tensor dy, Tensor x, Tensor gamma, float eps) -> ()");
    m.impl("rms_norm_bwd", &rms_norm_bwd);
    // annotated forms (see the note at the top of this file)
    m.def("gemm_peak_out(Tensor(a!) c, Tensor a, Tensor b) -> ()");
    m.def("rms_norm_fwd_out(Tensor(a!) y, Tensor x, Tensor gamma, float eps) -> ()");
    m.def("rms_norm_bwd_out(Tensor(a!) dx, Tensor(b!) dgamma, Tensor dy, Tensor x, Tensor gamma, float eps) -> ()");
    m.def("rms_norm_rstd(Tensor(a!) rstd, Tensor x, float eps) -> ()");
    m.def("gemm_peak_fused(Tensor(a!) d, Tensor a, Tensor b, Tensor? row_scale, Tensor? bias, Tensor? residual, "
          "bool pdl=False) -> ()");
}

TORCH_LIBRARY_IMPL(PeakGemm, CUDA, m) {
    m.impl("gemm_peak_out", &gemm_peak_out);
    m.impl("rms_norm_fwd_out", &rms_norm_fwd_out);
    m.impl("rms_norm_bwd_out", &rms_norm_bwd_out);
    m.impl("rms_norm_rstd", &rms_norm_rstd);
    m.impl("gemm_peak_fused", &gemm_peak_fused);
}
