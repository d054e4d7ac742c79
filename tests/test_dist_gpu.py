"""GPU (needs >= 2 devices): the column-sharded GEMM with the CUDA kernel and NCCL, against the oracle."""
import os
import socket
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, errors):
    try:
        sys.path.insert(0, REPO)
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        import torch.distributed as dist

        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        import oracle
        from peakgemm_b200 import capi
        from peakgemm_b200.dist import ShardedGemm

        m, n, k = 1536, 2048, 512
        a, b = oracle.gemm_inputs_uniform(m, n, k, torch.bfloat16, 4)
        ref = oracle.gemm_fp32(a, b)
        tol = oracle.gemm_tolerance(k, ref, torch.bfloat16)
        sg = ShardedGemm(n)
        ad, bd = a.cuda(), b[sg.start:sg.stop].contiguous().cuda()
        blk = sg.local(ad, bd)
        assert (blk.float().cpu() - ref[:, sg.start:sg.stop]).abs().max().item() <= tol
        c_full = torch.zeros(m, n, dtype=torch.bfloat16, device="cuda")
        sg.local_into_full(c_full, ad, bd)
        assert torch.equal(c_full[:, sg.start:sg.stop], blk)
        for bands, max_sms in ((1, 0), (3, 132)):
            got = sg.gathered(ad, bd, layout="row_major", bands=bands, max_sms=max_sms)
            torch.cuda.synchronize()
            assert (got.float().cpu() - ref).abs().max().item() <= tol
            assert torch.equal(got[:, sg.start:sg.stop], blk)
            sm = sg.gathered(ad, bd, layout="shard_major", bands=bands, max_sms=max_sms)
            torch.cuda.synchronize()
            for r in range(world):
                assert torch.equal(sm[r], got[:, r * sg.n_local:(r + 1) * sg.n_local])
        # the gather fused into the GEMM epilogue: peer stores over NVLink, no collective
        from peakgemm_b200.dist import PeerMatrix

        pm = PeerMatrix(m, n, torch.bfloat16)
        pm.local.fill_(float("nan"))
        dist.barrier()
        for max_sms in (0, 140):
            fused = sg.gathered_fused(pm, ad, bd, max_sms=max_sms)
            torch.cuda.synchronize()
            assert torch.equal(fused, got), "fused gather differs from the NCCL gather"
            dist.barrier()
        assert capi.device_status() == 0
        pm.close()
        dist.barrier()
        dist.destroy_process_group()
    except Exception as e:  # noqa: BLE001
        errors.put(f"rank {rank}: {e!r}")
        raise


def test_sharded_gemm_nccl(cuda):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    errors = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, errors)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    msgs = []
    while not errors.empty():
        msgs.append(errors.get())
    assert not msgs, msgs
    assert all(p.exitcode == 0 for p in procs)
