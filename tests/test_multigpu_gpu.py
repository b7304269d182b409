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
        for _ in range(2):  # twice: the symmetric buffer is reused
            c = fused(a, w[:, s:e])
            torch.cuda.synchronize()
            ok &= torch.equal(c, full)
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
