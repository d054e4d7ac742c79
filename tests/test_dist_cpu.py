"""CPU: the column-sharding and gather logic of peakgemm_b200.dist on two gloo ranks.

The ranks' compute step is injected (the CPU oracle stands in for the CUDA kernel, which the product
path always uses), so what is tested is the host logic: shard bounds, ldc writes into a full-width C,
the band-pipelined all-gather and both output layouts.
"""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_column_shard_properties():
    sys.path.insert(0, REPO)
    from peakgemm_b200.dist import column_shard, row_bands

    for n in (0, 8, 64, 1000, 4096, 128256, 32768):
        for world in (1, 2, 3, 4, 8):
            spans = [column_shard(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            for (s0, e0), (s1, e1) in zip(spans, spans[1:]):
                assert e0 == s1 and s0 <= e0
            assert all(s % 8 == 0 for s, _ in spans)
            sizes = [e - s for s, e in spans if e > s]
            assert not sizes or max(sizes) - min(sizes[:-1] or sizes) <= 0 or len(sizes) == 1 or sizes[-1] <= sizes[0]
    assert column_shard(32768, 8, 3) == (12288, 16384)
    with pytest.raises(ValueError):
        column_shard(64, 2, 2)
    assert row_bands(1000, 4) == [(0, 256), (256, 512), (512, 768), (768, 1000)]
    assert row_bands(100, 4) == [(0, 100)]
    assert row_bands(32768, 4) == [(0, 8192), (8192, 16384), (16384, 24576), (24576, 32768)]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_gemm(c, a, b, ldc, max_sms):
    import oracle

    c.copy_(oracle.gemm_exact(a.contiguous(), b.contiguous()))


def _worker(rank, world, port, m, n, k, bands, errors):
    try:
        sys.path.insert(0, REPO)
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        import oracle
        from peakgemm_b200.dist import ShardedGemm

        a, b = oracle.gemm_inputs_uniform(m, n, k, torch.bfloat16, 4)       # every rank draws the same A and B
        full = oracle.gemm_exact(a, b)
        sg = ShardedGemm(n, gemm=_oracle_gemm)
        b_shard = b[sg.start:sg.stop].contiguous()
        # no gather: own block only
        assert torch.equal(sg.local(a, b_shard), full[:, sg.start:sg.stop])
        # own block written in place into a full-width C
        c_full = torch.zeros(m, n, dtype=torch.bfloat16)
        sg.local_into_full(c_full, a, b_shard)
        assert torch.equal(c_full[:, sg.start:sg.stop], full[:, sg.start:sg.stop])
        assert (c_full[:, :sg.start] == 0).all() and (c_full[:, sg.stop:] == 0).all()
        # replicated C, both layouts
        got = sg.gathered(a, b_shard, layout="row_major", bands=bands)
        assert torch.equal(got, full)
        sm = sg.gathered(a, b_shard, layout="shard_major", bands=bands)
        assert sm.shape == (world, m, n // world)
        for r in range(world):
            assert torch.equal(sm[r], full[:, r * (n // world):(r + 1) * (n // world)])
        dist.barrier()
        dist.destroy_process_group()
    except Exception as e:  # noqa: BLE001
        errors.put(f"rank {rank}: {e!r}")
        raise


def _run_ranks(target, args, world=2, timeout=120):
    """Runs `target(rank, world, port, *args, errors)` on `world` spawned CPU ranks; no rank is left behind."""
    ctx = mp.get_context("spawn")
    errors = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=target, args=(r, world, port, *args, errors)) for r in range(world)]
    try:
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout)
    finally:
        for p in procs:
            if p.is_alive():
                p.terminate()
                p.join(5)
                if p.is_alive():
                    p.kill()
    msgs = []
    while not errors.empty():
        msgs.append(errors.get())
    assert not msgs, msgs
    assert all(p.exitcode == 0 for p in procs)


@pytest.mark.parametrize("m,n,k,bands", [
    (600, 256, 64, 1),
    (600, 256, 64, 3),
    (1024, 1024, 128, 2),     # tiles like the sharded benchmark shape: each rank's block is whole 512 x 256 tiles
])
def test_sharded_gemm_two_ranks(m, n, k, bands):
    _run_ranks(_worker, (m, n, k, bands))


def _oracle_rms_fwd(y, x, gamma, eps):
    import oracle

    y.copy_(oracle.rmsnorm_fwd(x, gamma, eps).to(y.dtype))


def _oracle_rms_bwd(dx, dgamma, dy, x, gamma, eps):
    import oracle

    d, g = oracle.rmsnorm_bwd(dy, x, gamma, eps)
    dx.copy_(d.to(dx.dtype))
    dgamma.copy_(g)


def _rms_worker(rank, world, port, rows, h, errors):
    try:
        sys.path.insert(0, REPO)
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        import oracle
        from peakgemm_b200.dist import ShardedRmsNorm

        x, dy, gamma = oracle.rmsnorm_inputs(rows, h, torch.bfloat16, 3)     # every rank draws the same tensors
        y_ref = oracle.rmsnorm_fwd(x, gamma).to(torch.bfloat16)
        dx_ref, dg_ref = oracle.rmsnorm_bwd(dy, x, gamma)
        sn = ShardedRmsNorm(rows, fwd=_oracle_rms_fwd, bwd=_oracle_rms_bwd)
        xs, dys = x[sn.start:sn.stop].contiguous(), dy[sn.start:sn.stop].contiguous()
        assert torch.equal(sn.forward(xs, gamma), y_ref[sn.start:sn.stop])
        dx, dg_local = sn.backward(dys, xs, gamma, reduce="none")
        assert torch.equal(dx, dx_ref[sn.start:sn.stop].to(torch.bfloat16))
        _, dg_local_ref = oracle.rmsnorm_bwd(dys, xs, gamma)
        assert torch.equal(dg_local, dg_local_ref)
        for how in ("all_reduce", "ordered"):
            _, dg = sn.backward(dys, xs, gamma, reduce=how)
            assert (dg - dg_ref).abs().max().item() <= 1e-3 * dg_ref.abs().max().item()
            everyone = [torch.empty_like(dg) for _ in range(world)]
            dist.all_gather(everyone, dg)
            if how == "ordered":           # rank-ordered sum: the same bits on every rank
                assert all(torch.equal(everyone[0], e) for e in everyone)
        with pytest.raises(ValueError):
            sn.backward(dys, xs, gamma, reduce="tree")
        dist.barrier()
        dist.destroy_process_group()
    except Exception as e:  # noqa: BLE001
        errors.put(f"rank {rank}: {e!r}")
        raise


@pytest.mark.parametrize("rows,h,world", [(64, 256, 2), (37, 128, 2), (5, 64, 3)])
def test_sharded_rmsnorm_ranks(rows, h, world):
    """Rows split over the ranks (ragged last block, and a rank with fewer rows than the others); dgamma local,
    all-reduced and rank-ordered."""
    _run_ranks(_rms_worker, (rows, h), world=world)


def test_row_shard_properties():
    sys.path.insert(0, REPO)
    from peakgemm_b200.dist import row_shard

    for rows in (0, 1, 5, 64, 1000, 32768):
        for world in (1, 2, 3, 8):
            spans = [row_shard(rows, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == rows
            for (s0, e0), (s1, e1) in zip(spans, spans[1:]):
                assert e0 == s1 and s0 <= e0
    assert row_shard(32768, 8, 7) == (28672, 32768)
    with pytest.raises(ValueError):
        row_shard(8, 2, 2)


def test_single_process_is_one_shard():
    sys.path.insert(0, REPO)
    import oracle
    from peakgemm_b200.dist import ShardedGemm

    a, b = oracle.gemm_inputs_uniform(32, 64, 64, torch.float16, 1)
    sg = ShardedGemm(64, gemm=_oracle_gemm)
    assert (sg.start, sg.stop, sg.world) == (0, 64, 1)
    assert torch.equal(sg.gathered(a, b), oracle.gemm_exact(a, b))
