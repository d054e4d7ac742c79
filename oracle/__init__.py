"""TEST INFRASTRUCTURE — the correctness oracle.  Not part of the product.

Only tests/, __graft_entry__.smoke() and the CPU-baseline legs of bench.py may
import this package; nothing under peakgemm_b200/ does.

GEMM oracle: the reference project checks its half-precision kernel against
``sgemm::sgemm_naive_kernel`` (src/impl/sgemm_impl.h:9-26; used by
test/cpp/test_gemm_half.cpp:62-63): ``acc_fp32 += float(a[mi*k+ki]) * float(b[ni*k+ki])``
over increasing ki, then a cast to the 16-bit type.  ``gemm_exact`` is that loop
in C (oracle/gemm_oracle.c, bit-identical to the reference kernel because the
products are exact in fp32); ``gemm_fp32`` is the same contraction through
torch's CPU fp32 matmul (summation order differs; what test/test_gemm.py:37-38
does with F.linear) and is the fast form used for large shapes and as the timed
CPU baseline.

PARITY PINNING.  The reference ships no golden vectors for this path (its tests
use unseeded random inputs and print, test/cpp/test_gemm_half.cpp:37-46,
test/test_gemm.py:55-60).  The GEMM oracle is pinned against outputs of the
reference's own kernels run on a B200 (tests/golden/, made by
tests/golden/make_golden.py from oracle/_ref/libref_peakgemm.so).

RMSNorm oracle: PARITY UNPINNED — the reference has no RMSNorm operator, kernel or
test.  The oracle is the textbook definition in fp32 (what
torch.nn.functional.rms_norm computes) with the closed-form gradients.
"""
from __future__ import annotations

import ctypes
import importlib.util
import math
import os

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))


def _builder():
    spec = importlib.util.spec_from_file_location("_oracle_build", os.path.join(_HERE, "build_oracle.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


_cpu_lib = None


def cpu_lib() -> ctypes.CDLL:
    global _cpu_lib
    if _cpu_lib is None:
        path = _builder().build_cpu()
        lib = ctypes.CDLL(path)
        i64, p = ctypes.c_int64, ctypes.c_void_p
        for name in ("oracle_gemm", "oracle_gemm_acc"):
            fn = getattr(lib, name)
            fn.restype = ctypes.c_int
            fn.argtypes = [p, p, p, i64, i64, i64, ctypes.c_int]
        _cpu_lib = lib
    return _cpu_lib


def _bits(t: torch.Tensor) -> np.ndarray:
    assert t.dtype in (torch.bfloat16, torch.float16) and t.device.type == "cpu"
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def gemm_exact(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """C = A @ B^T exactly as sgemm_naive_kernel computes it (k-ordered fp32 sum, cast to a.dtype)."""
    m, k = a.shape
    n = b.shape[0]
    assert b.shape[1] == k and a.dtype == b.dtype
    ab, bb = _bits(a), _bits(b)
    c = np.empty((m, n), dtype=np.uint16)
    r = cpu_lib().oracle_gemm(c.ctypes.data, ab.ctypes.data, bb.ctypes.data, m, n, k, int(a.dtype == torch.bfloat16))
    assert r == 0
    return torch.from_numpy(c.view(np.int16)).view(a.dtype)


def gemm_exact_acc(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """The unrounded fp32 accumulators of gemm_exact."""
    m, k = a.shape
    n = b.shape[0]
    ab, bb = _bits(a), _bits(b)
    acc = np.empty((m, n), dtype=np.float32)
    r = cpu_lib().oracle_gemm_acc(acc.ctypes.data, ab.ctypes.data, bb.ctypes.data, m, n, k,
                                  int(a.dtype == torch.bfloat16))
    assert r == 0
    return torch.from_numpy(acc)


def gemm_fp32(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """fp32 C = A.float() @ B.float()^T on the CPU (torch); unrounded."""
    return torch.nn.functional.linear(a.float(), b.float())


def gemm_tolerance(k: int, c_ref: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16) -> float:
    """Acceptance bound on max|C - C_ref| for a 16-bit output.

    2e-2 * sqrt(k/4096) * max|C_ref|  (the accumulation term), plus one unit of output rounding at
    max|C_ref|: 2^-8 relative for bf16, 2^-11 for fp16.  Without the second term the bound drops
    below the rounding of the output type itself for k < ~160 (bf16), which no kernel could meet.
    """
    cmax = float(c_ref.abs().max())
    eps_out = 2.0 ** -8 if out_dtype == torch.bfloat16 else 2.0 ** -11
    return 2e-2 * math.sqrt(max(k, 1) / 4096.0) * cmax + eps_out * cmax


def reference_abs_tolerance(k: int) -> float:
    """The reference test's own bound: |out - ref| <= 0.5 * k / 4096 (test_gemm_half.cpp:158,167)."""
    return 0.5 * k / 4096.0


# ------------------------------------------------------------------ RMSNorm ----

def rmsnorm_fwd(x: torch.Tensor, gamma: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """fp32 y (unrounded) = x * rsqrt(mean(x^2) + eps) * gamma over the last dimension."""
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    return (xf * rstd) * gamma.float()


def rmsnorm_bwd(dy: torch.Tensor, x: torch.Tensor, gamma: torch.Tensor, eps: float = 1e-6):
    """fp32 (dx, dgamma), closed form:  dx = rstd * (g - xhat * mean(g * xhat)),  dgamma = sum_rows dy * xhat."""
    xf, dyf, g32 = x.float(), dy.float(), gamma.float()
    rstd = torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    xhat = xf * rstd
    g = dyf * g32
    dx = rstd * (g - xhat * (g * xhat).mean(dim=-1, keepdim=True))
    dgamma = (dyf * xhat).reshape(-1, x.shape[-1]).double().sum(dim=0).float()
    return dx, dgamma


def rmsnorm_bwd_dx_slack(dy: torch.Tensor, x: torch.Tensor, gamma: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """Per-element absolute slack for dx on top of one 16-bit ulp: the fp32 error of the formula itself.

    dx = rstd * (g - xhat * c), c = mean_j(g * xhat), subtracts two fp32 numbers that can nearly cancel,
    and c is itself a sum of h terms of mixed sign.  Two correct fp32 evaluations that differ only in the
    order of the row reductions can therefore differ by about
        2^-24 * rstd * ( 8 |g| + 8 |xhat c| + |xhat| * sqrt(h) * mean_j |g xhat| )
    (a few roundings on each operand, plus the summation error of c, ~ sqrt(h) * 2^-24 * mean|terms|),
    which exceeds one 16-bit ulp only where dx cancelled to almost nothing.  This returns that bound.
    """
    xf, dyf, g32 = x.float(), dy.float(), gamma.float()
    h = x.shape[-1]
    rstd = torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    xhat = xf * rstd
    g = dyf * g32
    gx = g * xhat
    c = gx.mean(dim=-1, keepdim=True)
    c_err = math.sqrt(h) * gx.abs().mean(dim=-1, keepdim=True)
    return 2.0 ** -24 * rstd * (8.0 * g.abs() + 8.0 * (xhat * c).abs() + xhat.abs() * c_err)


def within_ulp_or_slack(out: torch.Tensor, ref_fp32: torch.Tensor, slack: torch.Tensor | None = None,
                        ulps: int = 1) -> torch.Tensor:
    """Elementwise: out within `ulps` 16-bit ulps of round(ref), or |out - ref| <= slack."""
    ok = ulp_distance_16(out, ref_fp32) <= ulps
    if slack is not None:
        ok |= (out.float() - ref_fp32).abs() <= slack + (ref_fp32.to(out.dtype).float() - ref_fp32).abs()
    return ok


def ulp_distance_16(out: torch.Tensor, ref_fp32: torch.Tensor) -> torch.Tensor:
    """|out - round(ref)| in units of out's 16-bit ulp at round(ref), elementwise (int64).

    Both are mapped to a monotone integer line (sign-magnitude -> two's complement),
    so the difference counts representable values between them."""
    ref = ref_fp32.to(out.dtype)

    def line(t):
        i = t.contiguous().view(torch.int16).to(torch.int64)
        return torch.where(i < 0, -(i & 0x7FFF), i)

    return (line(out) - line(ref)).abs()


# ---------------------------------------------------- fused epilogue / chains ----
# PARITY UNPINNED: the reference has no fused epilogue and no RMSNorm; these restate the definitions.

def rmsnorm_rstd(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """rstd[r] = rsqrt(mean(x[r,:]^2) + eps), evaluated in float64, returned as float64."""
    xd = x.double()
    return torch.rsqrt(xd.pow(2).mean(dim=-1) + eps)


def gemm_fused(a: torch.Tensor, b: torch.Tensor, row_scale=None, bias=None, residual=None) -> torch.Tensor:
    """Unrounded fp32 row_scale[:,None] * (A @ B^T) + bias[None,:] + residual (absent terms skipped)."""
    out = gemm_fp32(a, b).double()
    if row_scale is not None:
        out = out * row_scale.double()[:, None]
    if bias is not None:
        out = out + bias.double()[None, :]
    if residual is not None:
        out = out + residual.double()
    return out.float()


def gemm_fused_slack(a: torch.Tensor, b: torch.Tensor, row_scale=None) -> torch.Tensor:
    """Per-element slack for a fp32 accumulation in another order: 2^-17 * |row_scale| * (|A| @ |B|^T).

    The forward error of a length-k fp32 dot product is bounded by k * 2^-24 * sum|a_i b_i| and is
    typically sqrt(k) * 2^-24 of it; 2^-17 covers k up to 16384 at the typical rate."""
    s = torch.nn.functional.linear(a.float().abs(), b.float().abs()) * 2.0 ** -17
    if row_scale is not None:
        s = s * row_scale.float().abs()[:, None]
    return s


def rmsnorm_linear(x: torch.Tensor, gamma: torch.Tensor, w: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """Unrounded fp32 rms_norm(x; gamma) @ w^T by the definition (no folding, no intermediate rounding)."""
    y = x.double() * rmsnorm_rstd(x, eps)[:, None] * gamma.double()[None, :]
    return (y @ w.double().t()).float()


# ------------------------------------------------------------ input generators ----
# Seeded on the CPU so the oracle and the GPU see identical bits.

def gemm_inputs_uniform(m: int, n: int, k: int, dtype: torch.dtype, seed: int):
    """A[m,k], B[n,k] ~ U[-1,1] (the distribution of test/test_gemm.py:24-29), drawn A then B."""
    g = torch.Generator().manual_seed(seed)
    a = (torch.rand(m, k, generator=g) * 2 - 1).to(dtype)
    b = (torch.rand(n, k, generator=g) * 2 - 1).to(dtype)
    return a, b


def gemm_inputs_llm(m: int, n: int, k: int, dtype: torch.dtype, seed: int):
    """Activations A ~ N(0,1), weights B ~ N(0, 0.02)."""
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(m, k, generator=g).to(dtype)
    b = (0.02 * torch.randn(n, k, generator=g)).to(dtype)
    return a, b


def rmsnorm_inputs(rows: int, h: int, dtype: torch.dtype, seed: int):
    """x, dy ~ N(0,1) in `dtype`; gamma ~ N(1, 0.1) fp32; drawn x, dy, gamma."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, h, generator=g).to(dtype)
    dy = torch.randn(rows, h, generator=g).to(dtype)
    gamma = 1 + 0.1 * torch.randn(h, generator=g)
    return x, dy, gamma
