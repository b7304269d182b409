"""CPU tests of the multi-GPU host logic: partitioning rules, and the sharded GEMM with its
all-gather run as two gloo ranks."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from b200k import shard


@pytest.mark.parametrize("N", [128, 4096, 11008, 12288, 100, 1000])
@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_gemm_column_slabs_cover_once(N, world):
    slabs = shard.gemm_column_slabs(N, world)
    assert len(slabs) == world
    assert slabs[0][0] == 0 and slabs[-1][1] == N
    for (s0, e0), (s1, e1) in zip(slabs, slabs[1:]):
        assert e0 == s1 and s0 <= e0
    for (s, e) in slabs:
        if e > s:  # ranks beyond the tile count own nothing
            assert s % shard.TILE_N == 0 and (e % shard.TILE_N == 0 or e == N)
    widths = [e - s for s, e in slabs]
    assert max(widths) - min(widths) <= 2 * shard.TILE_N


@pytest.mark.parametrize("B,Hq,Hkv,world", [(1, 32, 8, 8), (1, 32, 8, 4), (8, 32, 32, 8), (2, 8, 2, 3), (1, 4, 1, 2)])
def test_head_shards_cover_once(B, Hq, Hkv, world):
    shards = shard.head_shards(B, Hq, Hkv, world)
    seen = set()
    for items in shards:
        for (b, hk0, n) in items:
            for hk in range(hk0, hk0 + n):
                assert (b, hk) not in seen
                seen.add((b, hk))
    assert seen == {(b, hk) for b in range(B) for hk in range(Hkv)}
    sizes = [sum(n for _, _, n in items) for items in shards]
    assert max(sizes) - min(sizes) <= 1


def test_balance_sequences():
    from b200k import inputs
    lens = inputs.decode_lens(64).tolist()
    for world in (1, 2, 4, 8):
        parts = shard.balance_sequences(lens, world)
        assert sorted(i for p in parts for i in p) == list(range(64))
        loads = [sum(lens[i] for i in p) for p in parts]
        assert max(loads) - min(loads) <= max(lens)  # greedy bound
    assert inputs.decode_lens(64).min() >= 512 and inputs.decode_lens(64).max() <= 32768


def _worker(rank, world, port, N, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        a = torch.randn(16, 64, generator=g)
        b = torch.randn(64, N, generator=g)
        full, slabs = shard.sharded_gemm(a, b, True, torch.matmul)
        local, _ = shard.sharded_gemm(a, b, False, torch.matmul)
        s, e = slabs[rank]
        ok = torch.equal(full, a @ b) or torch.allclose(full, a @ b, atol=1e-5)
        ok = ok and torch.allclose(local, (a @ b)[:, s:e], atol=1e-5)
        # the collective's own layout: [ranks, M, widest slab], entry r = C[:, slab_r] (zero-padded)
        recv = shard.all_gather_slabs(local, slabs)
        widest = max(e1 - s1 for (s1, e1) in slabs)
        ok = ok and recv.shape == (world, 16, widest)
        for r, (s1, e1) in enumerate(slabs):
            ok = ok and torch.allclose(recv[r, :, :e1 - s1], (a @ b)[:, s1:e1], atol=1e-5)
            ok = ok and bool((recv[r, :, e1 - s1:] == 0).all())
        # reassembly into a caller's buffer (one strided copy when all slabs have one width)
        out = torch.full((16, N), float("nan"))
        got = shard.all_gather_columns(local, slabs, out=out)
        ok = ok and got is out and torch.allclose(out, a @ b, atol=1e-5)
        results[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("N", [256, 300, 1000])
def test_sharded_gemm_two_gloo_ranks(N):
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        results = mgr.dict()
        port = 29500 + (os.getpid() + N) % 2000
        procs = [ctx.Process(target=_worker, args=(r, 2, port, N, results)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0
        assert dict(results) == {0: True, 1: True}


def _preflight_worker(rank, world, port, mode, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    try:
        desc = {"ok": True, "key": ("gemm", 8192, 4096, 11008)}
        if mode == "shape_mismatch" and rank == 1:
            desc["key"] = ("gemm", 8192, 4096, 4096)
        if mode == "rank_failed" and rank == 1:
            desc = {"ok": False, "error": "allocation failed", "key": None}
        try:
            shard.preflight_agree(desc)
            results[rank] = "agreed"
        except shard.ShardMismatch as e:
            results[rank] = "mismatch"
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode,expect", [("fine", "agreed"), ("shape_mismatch", "mismatch"), ("rank_failed", "mismatch")])
def test_preflight_detects_host_injected_faults(mode, expect):
    """Failures are injected on the host (a rank with a different shape, a rank that reports an
    error) and must be detected on every rank before any launch or data-path collective."""
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        results = mgr.dict()
        port = 31500 + (os.getpid() + len(mode)) % 2000
        procs = [ctx.Process(target=_preflight_worker, args=(r, 2, port, mode, results)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0
        assert dict(results) == {0: expect, 1: expect}
