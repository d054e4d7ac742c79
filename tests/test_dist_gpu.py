"""GPU (needs >= 2 devices): the column-sharded GEMM and the row-sharded RMSNorm with the CUDA kernels and NCCL,
against the oracle."""
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


def _run_gpu_ranks(target, world, timeout=300):
    """Spawns one process per GPU; a rank that is still alive after the joins is terminated before the asserts, so a
    failed run leaves no process holding a GPU or an IPC mapping."""
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    errors = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=target, args=(r, world, port, errors)) for r in range(world)]
    try:
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout)
    finally:
        for p in procs:
            if p.is_alive():
                p.terminate()
                p.join(10)
                if p.is_alive():
                    p.kill()
    msgs = []
    while not errors.empty():
        msgs.append(errors.get())
    assert not msgs, msgs
    assert all(p.exitcode == 0 for p in procs)


def test_sharded_gemm_nccl(cuda):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    _run_gpu_ranks(_worker, world)


def _worker_benchmark_tiling(rank, world, port, errors):
    """A shape that tiles like the sharded benchmark shape (every rank's block is whole 512 x 256 tiles of the
    CTA-pair kernel, several per SM pair, ldc = n): block in place into the full-width C, NCCL gather and fused
    gather, each against the oracle on sampled rows and against each other bit for bit."""
    try:
        sys.path.insert(0, REPO)
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        import torch.distributed as dist

        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        import oracle
        from peakgemm_b200 import capi
        from peakgemm_b200.dist import PeerMatrix, ShardedGemm
        from tests import helpers

        m, k = 8192, 1024
        n = 3328 * world                  # 16 x 13 = 208 large tiles per rank: 2.8 waves on 74 SM pairs
        a, b = oracle.gemm_inputs_uniform(m, n, k, torch.bfloat16, 4)
        sg = ShardedGemm(n)
        assert capi.hgemm_config(m, sg.n_local, k) == (5, 256)
        ad, bd = a.cuda(), b[sg.start:sg.stop].contiguous().cuda()
        c_full = helpers.garbage_like((m, n), torch.bfloat16, "cuda")
        sg.local_into_full(c_full, ad, bd)
        torch.cuda.synchronize()
        rows = torch.arange(32) * (m // 32) + 3
        helpers.check_gemm(c_full[rows.cuda(), sg.start:sg.stop], a[rows], b[sg.start:sg.stop], exact_rows=False)
        got = sg.gathered(ad, bd, layout="row_major", bands=2, max_sms=140)
        torch.cuda.synchronize()
        helpers.check_gemm(got[rows.cuda()], a[rows], b, exact_rows=False)
        assert torch.equal(got[:, sg.start:sg.stop], c_full[:, sg.start:sg.stop])
        pm = PeerMatrix(m, n, torch.bfloat16)
        pm.local.fill_(float("nan"))
        dist.barrier()
        fused = sg.gathered_fused(pm, ad, bd)
        torch.cuda.synchronize()
        assert torch.equal(fused, got), "fused gather differs from the NCCL gather"
        assert capi.device_status() == 0
        dist.barrier()
        pm.close()
        dist.barrier()
        dist.destroy_process_group()
    except Exception as e:  # noqa: BLE001
        errors.put(f"rank {rank}: {e!r}")
        raise


def _worker_multicast(rank, world, port, errors):
    """The gather done by the NVLink switch: every rank's block written through the multicast address
    (pg_hgemm_mcast) must give, on every rank, the same bits as the NCCL gather; at a shape of the one-CTA / CTA-pair
    kernels and at one whose per-rank block takes the 512 x 256 kernel.  Every rank stays until the matrix is closed."""
    try:
        sys.path.insert(0, REPO)
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        import torch.distributed as dist

        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        import oracle
        from peakgemm_b200 import capi
        from peakgemm_b200.dist import MulticastMatrix, ShardedGemm
        from tests import helpers

        for (m, n_per, k) in ((1536, 1024, 512), (8192, 3328, 1024), (300, 264, 136)):
            n = n_per * world
            a, b = oracle.gemm_inputs_uniform(m, n, k, torch.bfloat16, 4)
            sg = ShardedGemm(n)
            ad, bd = a.cuda(), b[sg.start:sg.stop].contiguous().cuda()
            got = sg.gathered(ad, bd, layout="row_major")
            torch.cuda.synchronize()
            rows = torch.arange(min(m, 16)) * max(1, m // 16)
            helpers.check_gemm(got[rows.cuda()], a[rows], b, exact_rows=False)
            try:
                mm = MulticastMatrix(m, n, torch.bfloat16)
            except RuntimeError as e:          # no NVSwitch multicast on this machine: nothing to test
                if "multicast" in str(e):
                    break
                raise
            mm.local.fill_(float("nan"))
            torch.cuda.synchronize()
            dist.barrier()
            out = sg.gathered_multicast(mm, ad, bd)
            torch.cuda.synchronize()
            dist.barrier()
            assert torch.equal(out, got), "multicast gather differs from the NCCL gather"
            assert capi.device_status() == 0
            mm.close()
        dist.barrier()
        dist.destroy_process_group()
    except Exception as e:  # noqa: BLE001
        errors.put(f"rank {rank}: {e!r}")
        raise


def test_sharded_gemm_multicast_store(cuda):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    _run_gpu_ranks(_worker_multicast, world)


def test_sharded_gemm_benchmark_tiling(cuda):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    _run_gpu_ranks(_worker_benchmark_tiling, 2)


def _worker_rmsnorm(rank, world, port, errors):
    try:
        sys.path.insert(0, REPO)
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        import torch.distributed as dist

        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        import oracle
        from peakgemm_b200 import capi
        from peakgemm_b200.dist import ShardedRmsNorm

        rows, h = 4099, 4096                       # ragged: the last rank owns fewer rows
        x, dy, gamma = oracle.rmsnorm_inputs(rows, h, torch.bfloat16, 3)
        dx_ref, dg_ref = oracle.rmsnorm_bwd(dy, x, gamma)
        sn = ShardedRmsNorm(rows)
        sl = slice(sn.start, sn.stop)
        xs, dys, gd = x[sl].cuda(), dy[sl].cuda(), gamma.cuda()
        y = sn.forward(xs, gd)
        torch.cuda.synchronize()
        assert oracle.ulp_distance_16(y.cpu(), oracle.rmsnorm_fwd(x[sl], gamma)).max().item() <= 1
        bits = []
        for how in ("all_reduce", "ordered"):
            dx, dg = sn.backward(dys, xs, gd, reduce=how)
            torch.cuda.synchronize()
            assert oracle.within_ulp_or_slack(dx.cpu(), dx_ref[sl], oracle.rmsnorm_bwd_dx_slack(dy[sl], x[sl], gamma)).all()
            assert (dg.cpu() - dg_ref).abs().max().item() <= 1e-3 * dg_ref.abs().max().item()
            bits.append(dg)
        everyone = [torch.empty_like(bits[1]) for _ in range(world)]
        dist.all_gather(everyone, bits[1])
        assert all(torch.equal(everyone[0], e) for e in everyone), "rank-ordered dgamma differs between ranks"
        _, dg_local = sn.backward(dys, xs, gd, reduce="none")
        _, dg_local_ref = oracle.rmsnorm_bwd(dy[sl], x[sl], gamma)
        assert (dg_local.cpu() - dg_local_ref).abs().max().item() <= 1e-3 * dg_local_ref.abs().max().item()
        assert capi.device_status() == 0
        dist.barrier()
        dist.destroy_process_group()
    except Exception as e:  # noqa: BLE001
        errors.put(f"rank {rank}: {e!r}")
        raise


def test_sharded_rmsnorm_nccl(cuda):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    _run_gpu_ranks(_worker_rmsnorm, world)
