"""pg_rmsnorm_bwd_static: the RMSNorm backward pass for hosts that cannot allocate device memory.

Some callers of this library hold nothing but raw device pointers, or run where an allocator call is not
allowed (inside another framework's stream-ordered region, in a loop that must not block on allocator
locks).  For them the library keeps the kernel's scratch — the fp32 dgamma partial rows — in a fixed
array of PG_STATIC_SCRATCH_BYTES inside its own image.  This test calls that entry point through the
C ABI twice in a row (the second call meets the first call's leftovers in the shared array) and
requires exactly the output of the workspace-taking entry point, which runs the same kernels.

The file name sorts last on purpose: a run that stops at the first failure has then already run every
other test.  It does not depend on them and also passes alone in a fresh process.
"""
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,h,dtype", [(4096, 4096, torch.bfloat16), (333, 8192, torch.float16),
                                          (50, 512, torch.bfloat16)])
def test_static_scratch_matches_workspace_entry_point(cuda, rows, h, dtype):
    from peakgemm_b200 import capi

    x, dy, gamma = oracle.rmsnorm_inputs(rows, h, dtype, 41)
    xd, dyd, gd = x.cuda(), dy.cuda(), gamma.cuda()
    ws = torch.empty(capi.rmsnorm_bwd_workspace_bytes(rows, h) // 4, device="cuda")
    dx_ref, dg_ref = torch.empty_like(xd), torch.empty_like(gd)
    capi.rmsnorm_bwd(dx_ref, dg_ref, dyd, xd, gd, ws)
    torch.cuda.synchronize()
    for call in range(2):                       # two calls in a row share the built-in array
        dx = torch.full_like(xd, float("nan"))
        dg = torch.full_like(gd, float("nan"))
        capi.rmsnorm_bwd_static(dx, dg, dyd, xd, gd)
        torch.cuda.synchronize()
        # same kernels, same summation order: the tolerance the other RMSNorm tests use (1 ulp / 1e-3)
        # is met with equality
        assert torch.equal(dx, dx_ref), f"dx differs on call {call}"
        assert torch.equal(dg, dg_ref), f"dgamma differs on call {call}"
    # and against the oracle, with the bounds of tests/test_rmsnorm_gpu.py
    dxo, dgo = oracle.rmsnorm_bwd(dy, x, gamma)
    assert oracle.within_ulp_or_slack(dx.cpu(), dxo, oracle.rmsnorm_bwd_dx_slack(dy, x, gamma)).all()
    assert (dg.cpu() - dgo).abs().max() <= 1e-3 * dgo.abs().max()


def test_static_scratch_rejects_oversized_shapes(cuda):
    from peakgemm_b200 import capi

    L = capi.lib()
    rows, h = 4096, 16384                       # 148 partial rows x 16384 floats > 5 MiB
    assert capi.rmsnorm_bwd_workspace_bytes(rows, h) > capi.PG_STATIC_SCRATCH_BYTES
    x = torch.zeros(rows, h, dtype=torch.bfloat16, device="cuda")
    g = torch.ones(h, device="cuda")
    dg = torch.full((h,), 7.0, device="cuda")
    dx = torch.full_like(x, 7.0)
    st = L.pg_rmsnorm_bwd_static(dx.data_ptr(), dg.data_ptr(), x.data_ptr(), x.data_ptr(), g.data_ptr(),
                                 rows, h, 1e-6, capi.PG_BF16, None)
    assert st == 8 and b"PG_STATIC_SCRATCH_BYTES" in L.pg_status_string(st)
    torch.cuda.synchronize()
    assert (dg == 7.0).all() and (dx == 7.0).all()    # nothing ran
    # rows == 0 needs no scratch at all: dgamma is an empty sum
    assert L.pg_rmsnorm_bwd_static(None, dg.data_ptr(), None, None, None, 0, h, 1e-6, capi.PG_BF16, None) == 0
    torch.cuda.synchronize()
    assert (dg == 0).all()
