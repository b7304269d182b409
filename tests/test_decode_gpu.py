"""GPU parity of the split-KV decode path against the CPU oracle, through the C ABI
(b200k_fmha_decode_splitkv via ctypes) and the reference-facing ops.
Tolerance: max-abs <= 2e-3 against fp32 softmax(QK^T scale)V (the stated bar)."""
import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu

TOL = oracle.FMHA_MAX_ABS_TOL


def _decode(q, k, v, lens, dev, **kw):
    from b200k import fmha
    o = fmha.fmha_decode(q.to(dev), k.to(dev), v.to(dev),
                         kv_lens=None if lens is None else lens.to(dev), **kw)
    torch.cuda.synchronize()
    return o.cpu()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("Skv", [1, 15, 64, 65, 200, 1000, 4096])
def test_parity_uniform_length(cuda_device, Skv, D, dtype):
    from b200k import inputs
    q, k, v = inputs.fmha_inputs(3, 8, 2, 1, Skv, D, dtype, seed=Skv + D)
    o = _decode(q, k, v, None, cuda_device)
    ref = oracle.fmha_ref(q, k, v)
    # fp16: 2e-3 max-abs; bf16: 2e-3 + one bf16 spacing around the formula rounded to bf16, element-wise
    absref = oracle.fmha_ref(q, k, v.abs()) if dtype == torch.bfloat16 else None
    ok, err = oracle.fmha_within_tolerance(o, ref, absref=absref)
    assert ok, err


@pytest.mark.parametrize("splits", [0, 1, 2, 7, 32])
def test_parity_varlen_nan_padding(cuda_device, splits):
    """Per-sequence lengths over a padded batch; the padding holds NaN, which must never
    reach the result; every split count gives the same answer within tolerance."""
    from b200k import inputs
    B, Hq, Hkv, Skv, D = 6, 32, 8, 2048, 128
    q, k, v = inputs.fmha_inputs(B, Hq, Hkv, 1, Skv, D, torch.float16, seed=4)
    lens = torch.tensor([1, 63, 64, 700, 2047, 2048], dtype=torch.int32)
    for b in range(B):
        k[b, :, int(lens[b]):] = float("nan")
        v[b, :, int(lens[b]):] = float("nan")
    o = _decode(q, k, v, lens, cuda_device, num_splits=splits)
    assert not torch.isnan(o).any()
    err = oracle.max_abs(o, oracle.fmha_ref(q, k, v, kv_lens=lens))
    assert err <= TOL, err


@pytest.mark.parametrize("Hq,Hkv,Sq", [(8, 8, 1), (8, 1, 1), (16, 1, 1), (4, 2, 4), (8, 2, 3)])
def test_parity_row_groups(cuda_device, Hq, Hkv, Sq):
    """GQA ratios 1, 8, 16 and several query rows per sequence (all rows see every key)."""
    from b200k import inputs
    q, k, v = inputs.fmha_inputs(2, Hq, Hkv, Sq, 777, 128, torch.float16, seed=Hq * 10 + Sq)
    o = _decode(q, k, v, None, cuda_device)
    assert oracle.max_abs(o, oracle.fmha_ref(q, k, v)) <= TOL


@pytest.mark.parametrize("Hq,Hkv,Sq", [(32, 1, 1), (32, 4, 4), (24, 2, 3), (8, 1, 8)])
def test_wide_groups_through_reference_wrapper(cuda_device, Hq, Hkv, Sq):
    """MQA and wide GQA groups, where more than 16 query rows share a KV head: shapes the reference's
    op accepts must go through the drop-in wrapper too (the group is taken in slices of at most 16
    rows); uniform length through fine_fmha(is_decode=True), ragged lengths through the varlen op."""
    from b200k import inputs
    import fmha_unified
    q, k, v = inputs.fmha_inputs(3, Hq, Hkv, Sq, 1000, 128, torch.float16, seed=Hq + Hkv + Sq)
    qd, kd, vd = q.to(cuda_device), k.to(cuda_device), v.to(cuda_device)
    o = fmha_unified.ops.fine_fmha(qd, kd, vd, False, True, 4)
    assert o.shape == q.shape
    assert oracle.max_abs(o, oracle.fmha_ref(q, k, v)) <= TOL
    lens = torch.tensor([1000, 1, 513], dtype=torch.int32)
    o = fmha_unified.ops.fine_fmha_decode_varlen(qd, kd, vd, lens.to(cuda_device))
    assert oracle.max_abs(o, oracle.fmha_ref(q, k, v, kv_lens=lens)) <= TOL


def test_zero_length_sequence_gives_zeros(cuda_device):
    from b200k import inputs
    q, k, v = inputs.fmha_inputs(2, 8, 2, 1, 256, 128, torch.float16, seed=8)
    lens = torch.tensor([0, 100], dtype=torch.int32)
    o = _decode(q, k, v, lens, cuda_device)
    assert torch.count_nonzero(o[0]) == 0
    assert oracle.max_abs(o[1:], oracle.fmha_ref(q[1:], k[1:], v[1:], kv_lens=lens[1:])) <= TOL


def test_config5_shape_reduced_batch(cuda_device):
    """The decode configuration (fp16, 32 query / 8 KV heads, d=128, lengths uniform in
    [512, 32768], padded batch) with 8 of its 64 sequences checked on the CPU, through the
    reference-facing varlen op; plus determinism (bit-identical reruns)."""
    from b200k import inputs
    import fmha_unified
    B, Hq, Hkv, Skv, D = 8, 32, 8, 32768, 128
    lens = inputs.decode_lens(64)[:B].clone()
    lens[0], lens[1] = 512, 32768  # make sure both extremes are present
    q = inputs.randn16((B, Hq, 1, D), 40, dtype=torch.float16)
    k = inputs.device_randn16((B, Hkv, Skv, D), 41, dtype=torch.float16, device=cuda_device)
    v = inputs.device_randn16((B, Hkv, Skv, D), 42, dtype=torch.float16, device=cuda_device)
    dl = lens.to(cuda_device)
    o1 = fmha_unified.ops.fine_fmha_decode_varlen(q.to(cuda_device), k, v, dl)
    o2 = fmha_unified.ops.fine_fmha_decode_varlen(q.to(cuda_device), k, v, dl)
    assert torch.equal(o1, o2)
    ref = oracle.fmha_ref(q, k.cpu(), v.cpu(), kv_lens=lens)
    assert oracle.max_abs(o1, ref) <= TOL


def test_config5_all_64_sequences(cuda_device):
    """The decode configuration at its own size: fp16, B=64, s_q=1, 32 query / 8 KV heads, d=128, the
    padded [64, 8, 32768, 128] cache (4 GiB each for K and V, drawn on the device) with the 64 seeded
    lengths in [512, 32768] and NaN in every padding position.  EVERY sequence meets the CPU oracle:
    for sequence b the four query heads of KV head b mod 8 (valid keys copied back)."""
    from b200k import inputs
    import fmha_unified
    B, Hq, Hkv, Skv, D = 64, 32, 8, 32768, 128
    lens = inputs.decode_lens(B)
    q = inputs.randn16((B, Hq, 1, D), 40, dtype=torch.float16)
    k = inputs.device_randn16((B, Hkv, Skv, D), 41, dtype=torch.float16, device=cuda_device)
    v = inputs.device_randn16((B, Hkv, Skv, D), 42, dtype=torch.float16, device=cuda_device)
    for b in range(B):
        k[b, :, int(lens[b]):] = float("nan")
        v[b, :, int(lens[b]):] = float("nan")
    o = fmha_unified.ops.fine_fmha_decode_varlen(q.to(cuda_device), k, v, lens.to(cuda_device))
    torch.cuda.synchronize()
    assert not torch.isnan(o).any()
    worst = 0.0
    for b in range(B):
        n, g = int(lens[b]), b % Hkv
        ref = oracle.fmha_ref(q[b:b + 1, 4 * g:4 * g + 4], k[b:b + 1, g:g + 1, :n].cpu(), v[b:b + 1, g:g + 1, :n].cpu())
        err = oracle.max_abs(o[b:b + 1, 4 * g:4 * g + 4], ref)
        worst = max(worst, err)
        assert err <= TOL, (b, n, err)
    del k, v
    torch.cuda.empty_cache()


def test_reference_signature_decode(cuda_device):
    """fine_fmha(..., causal=False, is_decode=True, idx): the reference's decode call
    (benchmarks/flashattn-cuda/modeling_llama.py:687-688) with a single query row."""
    import fmha_unified
    from b200k import inputs
    q, k, v = inputs.fmha_inputs(2, 32, 8, 1, 900, 128, torch.float16, device=cuda_device, seed=6)
    o = fmha_unified.ops.fine_fmha(q, k, v, False, True, 5)
    assert o.shape == (2, 32, 1, 128)
    assert oracle.max_abs(o, oracle.fmha_ref(q, k, v)) <= TOL


def test_matches_prefill_kernel(cuda_device):
    """The split-KV path and the tcgen05 prefill path agree on the same decode input."""
    from b200k import fmha, inputs
    q, k, v = inputs.fmha_inputs(4, 32, 8, 1, 3000, 128, torch.float16, device=cuda_device, seed=13)
    a = fmha.fmha_decode(q, k, v)
    b = fmha.fmha_fwd(q, k, v, causal=False)
    assert float((a.float() - b.float()).abs().max()) <= TOL


def test_workspace_errors(cuda_device):
    from b200k import _lib, fmha, inputs
    q, k, v = inputs.fmha_inputs(1, 8, 2, 1, 512, 128, torch.float16, device=cuda_device, seed=2)
    small = torch.empty(16, dtype=torch.uint8, device=cuda_device)
    with pytest.raises(_lib.B200KError) as e:
        fmha.fmha_decode(q, k, v, num_splits=4, workspace=small)
    assert e.value.code == -5
    with pytest.raises(_lib.B200KError):  # 17 query rows per sequence do not fit the 16-row tile
        fmha.fmha_decode(*inputs.fmha_inputs(1, 2, 2, 17, 128, 128, torch.float16, device=cuda_device))


@pytest.mark.parametrize("page_size", [64, 128, 256])
def test_paged_cache_matches_dense(cuda_device, page_size):
    """A paged cache holding the same keys/values as a dense one (pages scattered by a random
    permutation, unused table entries pointing nowhere) gives bit-identical results."""
    from b200k import fmha, inputs
    B, Hq, Hkv, Skv, D = 5, 32, 8, 2048, 128
    q, k, v = inputs.fmha_inputs(B, Hq, Hkv, 1, Skv, D, torch.float16, device=cuda_device, seed=61)
    lens = torch.tensor([2048, 1, 700, 65, 1999], dtype=torch.int32, device=cuda_device)
    blocks = Skv // page_size
    g = torch.Generator().manual_seed(3)
    perm = torch.randperm(B * blocks + 7, generator=g)[:B * blocks].to(torch.int32)  # 7 spare pages
    table = perm.view(B, blocks).to(cuda_device)
    num_pages = B * blocks + 7
    k_pages = torch.full((num_pages, Hkv, page_size, D), float("nan"), dtype=torch.float16, device=cuda_device)
    v_pages = torch.full_like(k_pages, float("nan"))
    for b in range(B):
        for n in range(blocks):
            k_pages[table[b, n]] = k[b, :, n * page_size:(n + 1) * page_size]
            v_pages[table[b, n]] = v[b, :, n * page_size:(n + 1) * page_size]
    # blocks entirely beyond a sequence's length are never looked at: poison their table entries
    poisoned = table.clone()
    for b in range(B):
        first_unused = (int(lens[b]) + page_size - 1) // page_size
        poisoned[b, first_unused:] = -12345
    dense = fmha.fmha_decode(q, k, v, kv_lens=lens, num_splits=4)
    paged = fmha.fmha_decode_paged(q, k_pages, v_pages, poisoned, lens, num_splits=4)
    assert torch.equal(paged, dense)
    assert oracle.max_abs(paged, oracle.fmha_ref(q, k, v, kv_lens=lens)) <= TOL


@pytest.mark.parametrize("D,dtype", [(128, torch.float16), (64, torch.bfloat16)])
@pytest.mark.parametrize("Hq,Hkv,splits", [(24, 6, 1), (8, 8, 1), (32, 8, 3)])
def test_heads_grouped_per_cta_bit_identical(cuda_device, Hq, Hkv, splits, D, dtype):
    """A CTA may walk several KV heads of its sequence (B200K_OPT_DECODE_HEADS_PER_CTA forces the
    group size; the library's own work lists are covered by the single-split test below).  Every
    grouping - including one that does not divide the head count and one larger than it - gives
    the bits of one head per CTA, with ragged lengths, an empty sequence and NaN padding."""
    from b200k import inputs
    B, Skv = 5, 640
    q, k, v = inputs.fmha_inputs(B, Hq, Hkv, 1, Skv, D, dtype, seed=Hq + splits)
    lens = torch.tensor([640, 0, 1, 333, 64], dtype=torch.int32)
    for b in range(B):
        k[b, :, int(lens[b]):] = float("nan")
        v[b, :, int(lens[b]):] = float("nan")
    from b200k import _lib
    with _lib.option(_lib.OPT_DECODE_HEADS_PER_CTA, 1):
        base = _decode(q, k, v, lens, cuda_device, num_splits=splits)
    ref = oracle.fmha_ref(q, k, v, kv_lens=lens)
    absref = oracle.fmha_ref(q, k, v.abs(), kv_lens=lens) if dtype == torch.bfloat16 else None
    ok, err = oracle.fmha_within_tolerance(base, ref, absref=absref)
    assert ok, err
    assert torch.equal(base[1], torch.zeros_like(base[1]))
    for h in (2, 4, 16):
        with _lib.option(_lib.OPT_DECODE_HEADS_PER_CTA, h):
            o = _decode(q, k, v, lens, cuda_device, num_splits=splits)
        assert torch.equal(o.view(torch.int16), base.view(torch.int16)), h


def test_single_split_writes_output_directly(cuda_device):
    """With one split per sequence the split kernel normalises and writes O itself (one launch,
    no partials), and with more (sequence, head) pairs than SMs its CTAs walk strided lists of
    pairs.  The result has the bits of one CTA per pair, also through a strided, 2-byte-aligned
    output view (scalar stores), with ragged lengths and empty sequences in the lists."""
    from b200k import fmha, _lib, inputs
    dev = cuda_device
    B, Hq, Hkv, Skv, D = 41, 32, 8, 300, 128  # 328 pairs on 148 SMs: lists of 2 or 3 pairs
    q, k, v = inputs.fmha_inputs(B, Hq, Hkv, 1, Skv, D, torch.float16, seed=11)
    lens = torch.randint(0, Skv + 1, (B,), generator=torch.Generator().manual_seed(5), dtype=torch.int32)
    lens[0], lens[3], lens[B - 1], lens[7] = 0, 0, 0, Skv
    qd, kd, vd, ld = q.to(dev), k.to(dev), v.to(dev), lens.to(dev)
    n0 = _lib.launch_count()
    o1 = fmha.fmha_decode(qd, kd, vd, kv_lens=ld, num_splits=1)
    assert _lib.launch_count() - n0 == 1
    o2 = fmha.fmha_decode(qd, kd, vd, kv_lens=ld, num_splits=2)
    assert _lib.launch_count() - n0 == 3
    big = torch.full((B, Hq, 1, D + 2), 7.0, dtype=torch.float16, device=dev)
    o3 = fmha.fmha_decode(qd, kd, vd, kv_lens=ld, num_splits=1, out=big[..., 1:D + 1])
    torch.cuda.synchronize()
    ref = oracle.fmha_ref(q, k, v, kv_lens=lens)
    assert oracle.max_abs(o1.cpu(), ref) <= TOL
    assert oracle.max_abs(o2.cpu(), ref) <= TOL
    assert torch.equal(o3, o1)
    assert torch.all(big[..., 0] == 7.0) and torch.all(big[..., D + 1] == 7.0)
    with _lib.option(_lib.OPT_DECODE_HEADS_PER_CTA, 1):
        o4 = fmha.fmha_decode(qd, kd, vd, kv_lens=ld, num_splits=1)
    torch.cuda.synchronize()
    assert torch.equal(o4, o1)
    assert torch.equal(o1[0], torch.zeros_like(o1[0])) and torch.equal(o1[B - 1], torch.zeros_like(o1[0]))
