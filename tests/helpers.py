"""Shared helpers of the test-suite (checker side only)."""
from __future__ import annotations

import ctypes
import os

import torch

import oracle

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(REPO, "tests", "golden")

_dev_lib = None
_ref_lib = None


def oracle_device_lib():
    """oracle/_build/liboracle_device.so: device restatement of the reference's naive oracle kernel."""
    global _dev_lib
    if _dev_lib is None:
        path = os.path.join(REPO, "oracle", "_build", "liboracle_device.so")
        if not os.path.exists(path):
            oracle._builder().build_device()
        lib = ctypes.CDLL(path)
        i64, p = ctypes.c_int64, ctypes.c_void_p
        lib.oracle_gemm_naive_device.restype = ctypes.c_int
        lib.oracle_gemm_naive_device.argtypes = [p, p, p, i64, i64, i64, i64, ctypes.c_int, p]
        _dev_lib = lib
    return _dev_lib


def gemm_naive_device(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    m, k = a.shape
    n = b.shape[0]
    c = torch.empty(m, n, dtype=a.dtype, device=a.device)
    r = oracle_device_lib().oracle_gemm_naive_device(
        c.data_ptr(), a.data_ptr(), b.data_ptr(), m, n, k, n, int(a.dtype == torch.bfloat16),
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert r == 0, f"cuda error {r}"
    return c


def reference_lib():
    """oracle/_ref/libref_peakgemm.so (the reference's own kernels), or None if it was not built."""
    global _ref_lib
    if _ref_lib is None:
        path = os.path.join(REPO, "oracle", "_ref", "libref_peakgemm.so")
        if not os.path.exists(path):
            return None
        lib = ctypes.CDLL(path)
        p, u, i = ctypes.c_void_p, ctypes.c_uint, ctypes.c_int
        lib.ref_hgemm_peak.restype = i
        lib.ref_hgemm_peak.argtypes = [p, p, p, u, u, u, i, p]
        lib.ref_sgemm_naive.restype = i
        lib.ref_sgemm_naive.argtypes = [p, p, p, i, i, i, i, p]
        _ref_lib = lib
    return _ref_lib


def garbage_like(shape, dtype, device):
    """Pre-filled output, as the reference's tests do (test/test_gemm.py:32-34): catches unwritten tiles."""
    g = torch.Generator(device="cpu").manual_seed(12345)
    return (torch.randn(shape, generator=g) * 100).to(dtype).to(device)


def spacing_16(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """Distance between neighbouring values of the 16-bit type `dtype` at magnitude |x| (fp32 tensor in, fp32 out)."""
    mant, min_exp = (7, -126) if dtype == torch.bfloat16 else (10, -14)
    _, e = torch.frexp(x.float().abs())                 # |x| = f * 2^e, f in [0.5, 1)  ->  floor(log2|x|) = e - 1
    e = torch.clamp(e - 1, min=min_exp)
    return torch.ldexp(torch.ones_like(x, dtype=torch.float32), e - mant)


def elementwise_ok(out: torch.Tensor, ref_fp32: torch.Tensor, slack: torch.Tensor) -> torch.Tensor:
    """True where `out` is the round-to-nearest 16-bit value of SOME number within `slack` of `ref_fp32`:
    |out - ref| <= slack + half the spacing of the output type there.  A truncating epilogue (error up to a whole
    spacing) or a lost product (error of a product's size) fails this; another fp32 summation order does not."""
    o = out.float()
    half = 0.5 * torch.maximum(spacing_16(ref_fp32, out.dtype), spacing_16(o, out.dtype))
    return (o - ref_fp32).abs() <= slack + half


def check_gemm(c_gpu: torch.Tensor, a_cpu: torch.Tensor, b_cpu: torch.Tensor, *, exact_rows=None):
    """Parity of a GPU result with the oracle.  Three checks, all enforced:

    1. The acceptance bound: max|C - C_ref| <= (2e-2 * sqrt(k/4096) + eps_out) * max|C_ref|, C_ref the
       fp32-accumulated product, eps_out = 2^-8 (bf16) or 2^-11 (fp16) for the rounding of the output; no NaN.
    2. Per element: C is the correctly ROUNDED value of a number within the fp32 accumulation slack
       (oracle.gemm_fused_slack: 2^-17 * |A| |B|^T) of the oracle's unrounded sum.  Against torch's fp32
       matmul twice that slack (both sides sum in an order of their own); against the exact k-ordered sum once.
    3. Where the exact k-ordered oracle is affordable: the reference test's own bound, 0.5 * k / 4096
       (test/cpp/test_gemm_half.cpp:158,167), floored at one rounding step of the output at max|C| (for k < 64 the
       reference's bound is below the output rounding itself).
    """
    k = a_cpu.shape[1]
    c = c_gpu.cpu()
    cf = c.float()
    assert not torch.isnan(cf).any(), "NaN in output"
    ref = oracle.gemm_fp32(a_cpu, b_cpu)
    tol = oracle.gemm_tolerance(k, ref, c_gpu.dtype)
    err = (cf - ref).abs().max().item()
    assert err <= tol, f"max|C-C_ref| = {err} > {tol}"
    slack = oracle.gemm_fused_slack(a_cpu, b_cpu)
    bad = ~elementwise_ok(c, ref, 2.0 * slack)
    assert not bad.any(), (f"{int(bad.sum())} elements are not the rounding of a value within the fp32 slack of the "
                           f"oracle; worst |diff| = {(cf - ref).abs()[bad].max().item()}")
    if exact_rows is None:
        exact_rows = a_cpu.shape[0] * b_cpu.shape[0] * k <= 2048 ** 3
    if exact_rows:
        acc = oracle.gemm_exact_acc(a_cpu, b_cpu)
        bad = ~elementwise_ok(c, acc, slack)
        assert not bad.any(), f"{int(bad.sum())} elements off the exact k-ordered sum by more than slack + half a step"
        ex = acc.to(c.dtype).float()
        err2 = (cf - ex).abs().max().item()
        one_step = float(spacing_16(ex.abs().max(), c.dtype))
        bound2 = max(oracle.reference_abs_tolerance(k), one_step)
        assert err2 <= bound2, f"vs k-ordered oracle: {err2} > {bound2}"
    return err, tol


def check_gemm_device(c: torch.Tensor, a: torch.Tensor, b: torch.Tensor, band: int = 2048):
    """Every element of a full-size result against the device restatement of the reference's naive kernel
    (all tensors on the GPU).  Both results are roundings of fp32 sums that differ by summation order only, so per
    element |C - C_naive| <= one step of the 16-bit type + 2 * slack, slack = 2^-17 * |a_i|_2 |b_j|_2
    (>= 2^-17 * sum|a||b| by Cauchy-Schwarz); and the reference test's bound 0.5 * k / 4096 on the maximum.
    Returns the maximum difference."""
    m, k = a.shape
    ref = gemm_naive_device(a, b)
    an = a.float().norm(dim=1)
    bn = b.float().norm(dim=1)
    worst = 0.0
    for r0 in range(0, m, band):
        r1 = min(m, r0 + band)
        cf, rf = c[r0:r1].float(), ref[r0:r1].float()
        d = (cf - rf).abs()
        assert not torch.isnan(cf).any(), "NaN in output"
        step = torch.maximum(spacing_16(rf, c.dtype), spacing_16(cf, c.dtype))
        slack = 2.0 ** -17 * an[r0:r1, None] * bn[None, :]
        bad = d > step + 2.0 * slack
        assert not bad.any(), (f"rows {r0}-{r1}: {int(bad.sum())} elements differ from the naive kernel by more than "
                               f"one step + slack; worst {d[bad].max().item()}")
        worst = max(worst, d.max().item())
    assert worst <= max(oracle.reference_abs_tolerance(k), float(spacing_16(ref.float().abs().max(), c.dtype))), worst
    return worst
