"""Pins the oracle against the reference project's own kernels, run on this GPU.

oracle/_ref/libref_peakgemm.so is the reference's src/impl headers compiled unmodified for sm_100a
(recipe: oracle/build_oracle.py).  Its naive kernel must agree bit for bit with the CPU oracle; its
mma.sync kernel and ours must both sit within the reference test's own bound of that oracle.
Shapes are multiples of 128 (m, n) and 16 (k): the reference kernel reads out of bounds otherwise.
"""
import ctypes

import pytest
import torch

import oracle
from tests import helpers

pytestmark = pytest.mark.gpu


def _ref():
    lib = helpers.reference_lib()
    assert lib is not None, "oracle/_ref/libref_peakgemm.so missing: run python oracle/build_oracle.py where the reference is mounted"
    return lib


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (256, 384, 1024), (512, 512, 2048)])
def test_cpu_oracle_equals_reference_naive_kernel(cuda, m, n, k, dtype):
    a, b = oracle.gemm_inputs_uniform(m, n, k, dtype, 31)
    c = helpers.garbage_like((m, n), dtype, "cuda")
    ad, bd = a.cuda(), b.cuda()
    r = _ref().ref_sgemm_naive(c.data_ptr(), ad.data_ptr(), bd.data_ptr(), m, n, k,
                               int(dtype == torch.bfloat16), _stream())
    assert r == 0
    torch.cuda.synchronize()
    assert torch.equal(c.cpu().view(torch.int16), oracle.gemm_exact(a, b).view(torch.int16))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (512, 384, 1024), (2048, 2048, 2048)])
def test_reference_kernel_and_ours_agree(cuda, m, n, k, dtype):
    from peakgemm_b200 import capi

    a, b = oracle.gemm_inputs_uniform(m, n, k, dtype, 32)
    ad, bd = a.cuda(), b.cuda()
    c_ref = helpers.garbage_like((m, n), dtype, "cuda")
    c_our = helpers.garbage_like((m, n), dtype, "cuda")
    r = _ref().ref_hgemm_peak(c_ref.data_ptr(), ad.data_ptr(), bd.data_ptr(), m, n, k,
                              int(dtype == torch.bfloat16), _stream())
    assert r == 0
    capi.hgemm(c_our, ad, bd)
    torch.cuda.synchronize()
    helpers.check_gemm(c_ref, a, b)      # the reference's kernel passes our parity bound ...
    helpers.check_gemm(c_our, a, b)      # ... and so does ours
    # both round an fp32 sum of the same exact products; they differ only in summation order
    assert (c_ref.float() - c_our.float()).abs().max().item() <= oracle.reference_abs_tolerance(k)
