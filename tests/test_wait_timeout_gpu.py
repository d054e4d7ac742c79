"""GPU: a bounded wait that runs out.  Every wait in the kernels has a limit; this makes one run out for real.

The test build of the device library (libPeakGemm_device_waittest.so: the same sources with -DPG_TEST_SHORT_WAIT)
waits 2 ms instead of 2 s and has a switch that makes ONE signal go missing, chosen so that nothing is in flight when
the roles drain: the MMA issuer withholds the "accumulator ready" commit of the first tile (its MMAs complete, the
epilogue warps are the ones that give up), and the RMSNorm producer leaves out its last row (no copy, no arrival).
Expected every time: the launch returns, pg_device_status returns PG_ERR_DEVICE_TIMEOUT with the code of the role
that gave up, the context stays usable, and the next ordinary call is bit-correct.  No trap, no fault, no unbounded
wait is involved.  (The reference has host asserts only: src/impl/hgemm_wmma_impl.h:389-390.)
"""
import ctypes
import os

import pytest
import torch

import oracle
from tests import helpers

pytestmark = pytest.mark.gpu
REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PG_OK, PG_ERR_DEVICE_TIMEOUT = 0, 6
EPILOGUE_GAVE_UP, RMS_CONSUMER_GAVE_UP = 4, 12


@pytest.fixture(scope="module")
def wlib():
    path = os.path.join(REPO, "peakgemm_b200", "libPeakGemm_device_waittest.so")
    assert os.path.exists(path), "build first: python __graft_entry__.py"
    lib = ctypes.CDLL(path)
    i64, p, i, f = ctypes.c_int64, ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.pg_hgemm_ex.restype = i
    lib.pg_hgemm_ex.argtypes = [p, p, p, i64, i64, i64, i64, i64, i64, i, i, i, i, p]
    lib.pg_rmsnorm_fwd.restype = i
    lib.pg_rmsnorm_fwd.argtypes = [p, p, p, i64, i64, f, i, p]
    lib.pg_device_status.restype = i
    lib.pg_device_status.argtypes = [ctypes.POINTER(i), p]
    lib.pg_test_withhold_gemm_signal.restype = i
    lib.pg_test_withhold_gemm_signal.argtypes = [i]
    lib.pg_test_withhold_rmsnorm_row.restype = i
    lib.pg_test_withhold_rmsnorm_row.argtypes = [i]
    yield lib
    lib.pg_test_withhold_gemm_signal(0)
    lib.pg_test_withhold_rmsnorm_row(0)


def _status(lib):
    code = ctypes.c_int(-1)
    st = lib.pg_device_status(ctypes.byref(code), None)
    return st, code.value


# one tile of each persistent kernel: one CTA, CTA pair, CTA pair with two row blocks
@pytest.mark.parametrize("variant,m,n", [(1, 128, 256), (2, 256, 256), (5, 512, 256)])
def test_gemm_epilogue_gives_up_and_the_next_call_is_correct(cuda, wlib, variant, m, n):
    k = 512
    a, b = oracle.gemm_inputs_uniform(m, n, k, torch.bfloat16, 40)
    ad, bd = a.cuda(), b.cuda()
    s = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def run(c):
        return wlib.pg_hgemm_ex(c.data_ptr(), ad.data_ptr(), bd.data_ptr(), m, n, k, k, k, n, 1, variant, 256, 0, s)

    good = helpers.garbage_like((m, n), torch.bfloat16, "cuda")
    assert run(good) == PG_OK
    torch.cuda.synchronize()
    assert _status(wlib) == (PG_OK, 0)
    helpers.check_gemm(good, a, b)

    assert wlib.pg_test_withhold_gemm_signal(1) == 0
    lost = helpers.garbage_like((m, n), torch.bfloat16, "cuda")
    before = lost.clone()
    assert run(lost) == PG_OK                      # the launch itself succeeds; the kernel gives up on the device
    torch.cuda.synchronize()                       # returns: the kernel has ended by itself
    assert _status(wlib) == (PG_ERR_DEVICE_TIMEOUT, EPILOGUE_GAVE_UP)
    assert torch.equal(lost, before)               # the epilogue never ran: nothing was written
    assert _status(wlib) == (PG_OK, 0)             # reading the word cleared it

    assert wlib.pg_test_withhold_gemm_signal(0) == 0
    again = helpers.garbage_like((m, n), torch.bfloat16, "cuda")
    assert run(again) == PG_OK
    torch.cuda.synchronize()
    assert _status(wlib) == (PG_OK, 0)
    assert torch.equal(again.view(torch.int16), good.view(torch.int16))


def test_rmsnorm_consumers_give_up_and_the_next_call_is_correct(cuda, wlib):
    rows, h = 300, 4096
    x, _, gamma = oracle.rmsnorm_inputs(rows, h, torch.bfloat16, 41)
    xd, gd = x.cuda(), gamma.cuda()

    def run(y):
        return wlib.pg_rmsnorm_fwd(y.data_ptr(), xd.data_ptr(), gd.data_ptr(), rows, h, 1e-6, 1, None)

    good = torch.empty_like(xd)
    assert run(good) == PG_OK
    torch.cuda.synchronize()
    assert _status(wlib) == (PG_OK, 0)
    assert oracle.ulp_distance_16(good.cpu(), oracle.rmsnorm_fwd(x, gamma)).max().item() <= 1

    assert wlib.pg_test_withhold_rmsnorm_row(1) == 0
    lost = torch.zeros_like(xd)
    assert run(lost) == PG_OK
    torch.cuda.synchronize()
    assert _status(wlib) == (PG_ERR_DEVICE_TIMEOUT, RMS_CONSUMER_GAVE_UP)
    assert wlib.pg_test_withhold_rmsnorm_row(0) == 0

    again = torch.empty_like(xd)
    assert run(again) == PG_OK
    torch.cuda.synchronize()
    assert _status(wlib) == (PG_OK, 0)
    assert torch.equal(again.view(torch.int16), good.view(torch.int16))
