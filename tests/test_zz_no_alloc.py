"""The allocation-free decode entry point, b200k_fmha_decode_splitkv_static.

It exists for callers that may not allocate device memory while serving (a fixed
memory pool, a plugin that does not own the allocator, a loop that cannot afford
cudaMalloc's synchronisation): its split-KV partials live in a 16 MiB array built
into the library instead of a caller workspace.  The test drives it through the C
ABI directly (ctypes, raw device pointers) and compares with the ordinary entry
point, which takes the workspace from the caller, and with the CPU oracle, on calls
in a row with different inputs, so stale contents of the shared array from one call
would show in the next.  Around every call it also checks the property the entry
point is named for: the driver's free-memory figure and torch's allocation counter
do not move.  This file sorts last so a run that stops at the first failure
has already run every other test; it also passes when run alone."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_static(L, q, k, v, out, lens, splits):
    from b200k import _lib
    B, Hq, Sq, D = q.shape
    return L.b200k_fmha_decode_splitkv_static(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, Hq, k.size(1), Sq, k.size(2), D,
        _lib.strides3(q), _lib.strides3(k), _lib.strides3(v), _lib.strides3(out), float(D) ** -0.5,
        lens.data_ptr() if lens is not None else None, splits, _lib.F16,
        torch.cuda.current_stream().cuda_stream)


def _memory_marks():
    torch.cuda.synchronize()
    return torch.cuda.mem_get_info()[0], torch.cuda.memory_stats()["allocation.all.allocated"]


def test_static_scratch_matches_workspace_entry_point(cuda_device):
    from b200k import _lib, fmha, inputs
    from oracle import oracle
    L = _lib.lib()
    assert L.b200k_fmha_decode_static_scratch_bytes() == 16 << 20
    B, Hq, Hkv, Skv, D = 8, 32, 8, 4096, 128
    lens_a = torch.tensor([4096, 1, 777, 2048, 4095, 64, 3000, 129], dtype=torch.int32, device=cuda_device)
    lens_b = torch.tensor([5, 4096, 4096, 100, 1, 4000, 63, 2049], dtype=torch.int32, device=cuda_device)
    # the first call on a device looks the array's address up (documented); it comes before the marks
    q, k, v = inputs.fmha_inputs(B, Hq, Hkv, 1, Skv, D, torch.float16, device=cuda_device, seed=30)
    assert _call_static(L, q, k, v, torch.empty_like(q), lens_a, 4) == 0
    for seed, lens, splits in ((31, lens_a, 4), (32, lens_b, 4), (33, lens_a, 0)):
        q, k, v = inputs.fmha_inputs(B, Hq, Hkv, 1, Skv, D, torch.float16, device=cuda_device, seed=seed)
        expect = fmha.fmha_decode(q, k, v, kv_lens=lens, num_splits=splits)
        ref = oracle.fmha_ref(q, k, v, kv_lens=lens)
        got = torch.full_like(q, float("nan"))
        free0, allocs0 = _memory_marks()
        rc = _call_static(L, q, k, v, got, lens, splits)
        free1, allocs1 = _memory_marks()
        assert rc == 0, _lib.strerror(rc)
        # nothing was allocated: neither by the driver (free bytes) nor through torch's allocator
        assert free1 == free0 and allocs1 == allocs0
        assert not torch.isnan(got).any()
        assert oracle.max_abs(got, ref) <= oracle.FMHA_MAX_ABS_TOL
        # same kernels, same split count: the results are expected to agree to the bit;
        # the bound asserted is the 2e-3 max-abs tolerance the other decode tests use
        assert float((got.float() - expect.float()).abs().max()) <= 2e-3
        if splits:
            assert torch.equal(got, expect)


def test_static_scratch_rejects_what_does_not_fit(cuda_device):
    from b200k import _lib, inputs
    L = _lib.lib()
    # 64 sequences x 32 heads x 64 splits x 130 floats = 68 MB of partials: beyond 16 MiB
    q, k, v = inputs.fmha_inputs(64, 32, 8, 1, 128, 128, torch.float16, device=cuda_device, seed=1)
    out = torch.zeros_like(q)
    rc = _call_static(L, q, k, v, out, None, 64)
    assert rc == -11 and "scratch" in _lib.strerror(rc)
    assert torch.count_nonzero(out) == 0  # nothing was launched
    # the same problem with the split count left to the library fits and runs
    assert _call_static(L, q, k, v, out, None, 0) == 0
    torch.cuda.synchronize()
    from oracle import oracle
    assert oracle.max_abs(out, oracle.fmha_ref(q, k, v)) <= 2e-3
    # one split per sequence keeps no partials, so no size is too large for it: 40960 rows x 130 floats
    # would be 21 MB of partials if they existed
    q, k, v = inputs.fmha_inputs(1280, 32, 8, 1, 64, 128, torch.float16, device=cuda_device, seed=2)
    out = torch.full_like(q, float("nan"))
    assert _call_static(L, q, k, v, out, None, 1) == 0
    torch.cuda.synchronize()
    assert oracle.max_abs(out[::97], oracle.fmha_ref(q[::97], k[::97], v[::97])) <= 2e-3
    assert not torch.isnan(out).any()
