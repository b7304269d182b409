"""Partitioning of the two paths over the GPUs of one node (one process per GPU).

The reference has no multi-GPU code at all (no torch.distributed / NCCL call site);
this is new work that shards only where the math is independent:
  * GEMM: the weight B[K,N] is cut into contiguous column slabs whose widths are
    multiples of the 128-column tile, rank r computes C[:, slab_r]; a collective
    (all-gather over NCCL) is needed only when the full C must be reassembled.
  * FMHA prefill: (batch, KV-head group) pairs are independent; no collective.
  * Decode: sequences are independent; they are assigned greedily, longest first,
    to the rank with the least total KV length; no collective.
All functions here are pure host logic (testable on CPU with the gloo backend).
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch
import torch.distributed as dist

TILE_N = 128


def gemm_column_slabs(N: int, world: int, tile: int = TILE_N) -> List[Tuple[int, int]]:
    """[start, end) column ranges, one per rank: whole tiles spread as evenly as possible,
    the ragged tail (N % tile) goes to the last rank that owns any tile."""
    n_tiles = (N + tile - 1) // tile
    base, extra = divmod(n_tiles, world)
    out, t0 = [], 0
    for r in range(world):
        t1 = t0 + base + (1 if r < extra else 0)
        out.append((min(t0 * tile, N), min(t1 * tile, N)))
        t0 = t1
    return out


def head_shards(B: int, Hq: int, Hkv: int, world: int) -> List[List[Tuple[int, int, int]]]:
    """Work items (batch, first kv head, number of kv heads) per rank.  KV-head groups are
    kept whole (a query head and its KV head never separate); heads are split first,
    then batches."""
    items = [(b, hk) for b in range(B) for hk in range(Hkv)]
    per, extra = divmod(len(items), world)
    shards, i = [], 0
    for r in range(world):
        n = per + (1 if r < extra else 0)
        mine = items[i:i + n]
        i += n
        merged: List[Tuple[int, int, int]] = []
        for (b, hk) in mine:
            if merged and merged[-1][0] == b and merged[-1][1] + merged[-1][2] == hk:
                merged[-1] = (b, merged[-1][1], merged[-1][2] + 1)
            else:
                merged.append((b, hk, 1))
        shards.append(merged)
    return shards


def balance_sequences(kv_lens: Sequence[int], world: int) -> List[List[int]]:
    """Greedy longest-first assignment of sequence indices to ranks by total KV length."""
    order = sorted(range(len(kv_lens)), key=lambda i: (-int(kv_lens[i]), i))
    loads = [0] * world
    out: List[List[int]] = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda j: (loads[j], j))
        out[r].append(i)
        loads[r] += int(kv_lens[i])
    for lst in out:
        lst.sort()
    return out


def all_gather_slabs(c_local: torch.Tensor, slabs: Sequence[Tuple[int, int]], group=None) -> torch.Tensor:
    """The one collective of the GEMM path: every rank's column slab of C on every rank, as the
    collective delivers it: a [world, M, widest slab] tensor whose entry r holds C[:, slab_r] in its
    first (end_r - start_r) columns (narrower slabs are zero-padded).  No reassembly copy: a consumer
    that can take C as column slabs (the next column-sharded layer, a reduction over rows) reads this
    directly."""
    world = dist.get_world_size(group)
    M = c_local.size(0)
    wmax = max(e - s for (s, e) in slabs)
    send = c_local
    if c_local.size(1) != wmax:
        send = c_local.new_zeros((M, wmax))
        send[:, :c_local.size(1)] = c_local
    send = send.contiguous()
    recv = send.new_empty((world * M, wmax))  # rank-major concatenation along dim 0
    dist.all_gather_into_tensor(recv, send, group=group)
    return recv.view(world, M, wmax)


def all_gather_columns(c_local: torch.Tensor, slabs: Sequence[Tuple[int, int]], group=None,
                       out: torch.Tensor | None = None) -> torch.Tensor:
    """Reassembles the row-major C[M,N] from per-rank column slabs: all_gather_slabs plus the copy
    into column windows (one strided copy when all slabs have one width, else one per slab)."""
    recv = all_gather_slabs(c_local, slabs, group)
    world, M, wmax = recv.shape
    N = slabs[-1][1]
    if out is None:
        out = recv.new_empty((M, N))
    if all(e - s == wmax for (s, e) in slabs):
        out.view(M, world, wmax).copy_(recv.permute(1, 0, 2))
    else:
        for r, (s, e) in enumerate(slabs):
            out[:, s:e] = recv[r, :, :e - s]
    return out


class ShardMismatch(RuntimeError):
    """Ranks disagree about the problem they are about to run."""


def preflight_agree(description, group=None, timeout_s: float = 30.0) -> None:
    """Host-side agreement step run BEFORE any data-path launch or collective: every rank
    publishes a small description of its shard (shapes, dtypes, slab bounds); all ranks
    raise ShardMismatch if any rank reported something different from what rank 0 expects
    of it, or reported a failure.  A rank that died or never arrives turns into the process
    group's timeout error here, on the host, while no kernel or NCCL collective is in flight.
    `description` is a dict with at least {"ok": bool, "key": hashable}; "key" must be equal
    on all ranks."""
    world = dist.get_world_size(group)
    gathered = [None] * world
    dist.all_gather_object(gathered, description, group=group)
    bad = [r for r, d in enumerate(gathered) if not d.get("ok", False)]
    if bad:
        raise ShardMismatch(f"ranks {bad} reported a failure before the launch: "
                            f"{[gathered[r].get('error') for r in bad]}")
    keys = {repr(d.get("key")) for d in gathered}
    if len(keys) != 1:
        raise ShardMismatch(f"ranks disagree about the problem: {sorted(keys)}")


def sharded_gemm(a: torch.Tensor, b_full: torch.Tensor, gather: bool, matmul, group=None):
    """Rank-local slab of a @ b_full (and the gathered full product when `gather`).
    With the library GEMM the gathered product equals the unsharded one bit for bit for more than 128
    rows (the tile kernels sum every output element in one order); up to 128 rows the weight-streaming
    kernel splits K according to the number of slabs, so the two agree to rounding only.
    `matmul(a, b_slab)` is the local kernel (the library GEMM on GPU; torch.matmul in
    the CPU tests of this host logic)."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    slabs = gemm_column_slabs(b_full.size(1), world)
    s, e = slabs[rank]
    c_local = matmul(a, b_full[:, s:e]) if e > s else a.new_empty((a.size(0), 0))
    if not gather:
        return c_local, slabs
    return all_gather_columns(c_local, slabs, group), slabs


class FusedAllGatherGemm:
    """C = a @ b_full reassembled on every rank by the GEMM epilogue itself: rank r computes
    its column slab and stores every finished tile into the C buffers of all ranks, which live
    in symmetric (peer-mapped) memory; a symmetric-memory barrier then orders the ranks.  No NCCL
    collective and no multicast load is involved: the data crosses NVLink as plain TMA stores
    while later tiles are still being computed.  GPU only (needs the library).

    Reuse: two symmetric C buffers alternate from call to call.  The result of call n is this rank's
    buffer n % 2; peers next write it in call n + 2, and they can only reach that call after this rank
    has passed the barrier of call n + 1, which sits behind this rank's own work on the calling stream.
    So a result may be read, ON THE CALLING STREAM, until the call after the next is issued; a
    consumer on another stream must be made a dependency of the calling stream (wait_stream / event)
    before call n + 1 is issued."""

    def __init__(self, M: int, N: int, dtype, device, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if self.world > 8:
            raise RuntimeError("at most 8 destinations (one node)")
        self.M, self.N = M, N
        self.slabs = gemm_column_slabs(N, self.world)
        self.bufs, self.handles, self.ptrs = [], [], []
        for _ in range(2):
            buf = symm_mem.empty((M, N), dtype=dtype, device=device)
            handle = symm_mem.rendezvous(buf, self.group)
            self.bufs.append(buf)
            self.handles.append(handle)
            self.ptrs.append([int(p) for p in handle.buffer_ptrs])
        self.calls = 0

    def __call__(self, a: torch.Tensor, b_slab: torch.Tensor) -> torch.Tensor:
        """a [M,K]; b_slab = this rank's columns of the weight, [K, slab width].  Returns the
        full C [M,N] (one of this rank's two symmetric buffers), valid on return in stream order."""
        import ctypes
        from . import _lib
        from .gemm import _DTYPES
        s, e = self.slabs[self.rank]
        if b_slab.size(1) != e - s or a.size(0) != self.M or a.size(1) != b_slab.size(0):
            raise RuntimeError("operand shapes do not match this rank's slab")
        which = self.calls % 2
        self.calls += 1
        if e > s:
            esz = self.bufs[which].element_size()
            # destinations start with this rank's own buffer and go round the ring, so that at any
            # moment the ranks' stores head for different GPUs (the kernel also rotates per tile)
            order = [(self.rank + i) % self.world for i in range(self.world)]
            dsts = (ctypes.c_void_p * self.world)(*[self.ptrs[which][r] + s * esz for r in order])
            code = _lib.lib().b200k_gemm_scatter(
                a.data_ptr(), b_slab.data_ptr(), dsts, self.world, self.M, e - s, a.size(1),
                a.stride(0), b_slab.stride(0), self.N, _DTYPES[a.dtype],
                _lib.raw_stream(a.device))
            _lib.check(code, "b200k_gemm_scatter")
        self.handles[which].barrier()
        return self.bufs[which]
