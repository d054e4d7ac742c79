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


def check_gemm(c_gpu: torch.Tensor, a_cpu: torch.Tensor, b_cpu: torch.Tensor, *, exact_rows=None):
    """Parity of a GPU result with the oracle.

    Bound (written here once): max|C - C_ref| <= (2e-2 * sqrt(k/4096) + eps_out) * max|C_ref|, C_ref the
    fp32-accumulated product, eps_out = 2^-8 (bf16) or 2^-11 (fp16) for the rounding of the output; and no NaN.  Where the exact k-ordered oracle is affordable it is compared too, with the bound
    of the reference's own test, 0.5 * k / 4096 (test/cpp/test_gemm_half.cpp:158,167).
    """
    k = a_cpu.shape[1]
    c = c_gpu.float().cpu()
    assert not torch.isnan(c).any(), "NaN in output"
    ref = oracle.gemm_fp32(a_cpu, b_cpu)
    tol = oracle.gemm_tolerance(k, ref, c_gpu.dtype)
    err = (c - ref).abs().max().item()
    assert err <= tol, f"max|C-C_ref| = {err} > {tol}"
    if exact_rows is None:
        exact_rows = a_cpu.shape[0] * b_cpu.shape[0] * k <= 2048 ** 3
    if exact_rows:
        ex = oracle.gemm_exact(a_cpu, b_cpu).float()
        err2 = (c - ex).abs().max().item()
        # the reference's bound, floored at one output rounding step for very small k
        bound2 = max(oracle.reference_abs_tolerance(k), tol)
        assert err2 <= bound2, f"vs k-ordered oracle: {err2}"
    return err, tol
