"""Two-rank NCCL run of the sharded paths (needs 2 GPUs; skipped on a single-GPU box, where
the same host logic is covered by the gloo tests in test_shard_cpu.py): column-sharded GEMM
reassembled by NCCL all-gather and by the fused epilogue (peer TMA stores) both equal the
single-GPU product bit for bit; (batch, head)-sharded attention equals the unsharded slices."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from b200k import _lib, fmha, gemm, inputs, shard
        ok = True
        M, K, N = 1024, 512, 1280
        a, w = inputs.gemm_llm(M, K, N, torch.bfloat16, device=dev, seed=5)
        shard.preflight_agree({"ok": True, "key": ("gemm", M, K, N)})
        full = gemm.gemm(a, w)
        gathered, slabs = shard.sharded_gemm(a, w, True, gemm.gemm)
        ok &= torch.equal(gathered, full)
        fused = shard.FusedAllGatherGemm(M, N, torch.bfloat16, dev)
        s, e = slabs[rank]
        # Back-to-back calls with DIFFERENT activations and no host synchronisation in between: a peer
        # that ran ahead and overwrote a result before it was read would show as a mismatch (identical
        # inputs would hide it).  Results are read on the calling stream (clone) and on a side stream
        # that is made a dependency of the calling stream before the next call, as documented.
        acts = [inputs.gemm_llm(M, K, N, torch.bfloat16, device=dev, seed=50 + i)[0] for i in range(6)]
        wants = [gemm.gemm(x, w) for x in acts]
        side = torch.cuda.Stream()
        same_stream, side_stream = [], []
        for x in acts:
            c = fused(x, w[:, s:e])
            same_stream.append(c.clone())
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                side_stream.append(c.clone())
            torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        for got1, got2, want in zip(same_stream, side_stream, wants):
            ok &= torch.equal(got1, want) and torch.equal(got2, want)
        # the NCCL path in both layouts: column slabs as delivered, and reassembled row-major
        recv = shard.all_gather_slabs(gemm.gemm(a, w[:, s:e]), slabs)
        for r, (s0, e0) in enumerate(slabs):
            ok &= torch.equal(recv[r, :, :e0 - s0], full[:, s0:e0])
        # attention sharded over (batch, kv-head group)
        q, k, v = inputs.fmha_inputs(2, 8, 2, 300, 300, 128, torch.float16, device=dev, seed=9)
        whole = fmha.fmha_fwd(q, k, v, causal=True)
        for (b, hk0, n) in shard.head_shards(2, 8, 2, world)[rank]:
            g = 4
            part = fmha.fmha_fwd(q[b:b + 1, hk0 * g:(hk0 + n) * g], k[b:b + 1, hk0:hk0 + n], v[b:b + 1, hk0:hk0 + n],
                                 causal=True)
            ok &= torch.equal(part, whole[b:b + 1, hk0 * g:(hk0 + n) * g])
        ok &= _lib.device_status() == (0, 0)
        results[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_two_ranks_nccl_and_fused_gather():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        results = mgr.dict()
        port = 30500 + os.getpid() % 2000
        procs = [ctx.Process(target=_worker, args=(r, 2, port, results)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(300)
            assert p.exitcode == 0
        assert dict(results) == {0: True, 1: True}
