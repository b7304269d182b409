"""GPU parity of the FMHA forward path against the CPU oracle, through the C ABI
(b200k_fmha_fwd via ctypes) and the reference-facing op (fmha_unified.ops.fine_fmha).
Tolerance: max-abs <= 2e-3 against fp32 softmax(QK^T scale)V for N(0,1) inputs
(the stated bar)."""
import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu

TOL = oracle.FMHA_MAX_ABS_TOL


def _assert_close(o, ref, where=None, extra=0.0, absref=None):
    """fp16: the stated 2e-3 max-abs.  bf16 (8 significant bits in the output and in P): overall,
    average and per-element bounds that state the unavoidable rounding apart from the kernel's own
    error (oracle.fmha_within_tolerance)."""
    ok, err = oracle.fmha_within_tolerance(o, ref, extra, absref)
    assert ok, (where, err)


def _refs(q, k, v, causal, kv_lens=None):
    """(formula, formula on |V| for bf16 inputs: the per-element conditioning of the output)."""
    ref = oracle.fmha_ref(q, k, v, causal=causal, kv_lens=kv_lens)
    absref = oracle.fmha_ref(q, k, v.abs(), causal=causal, kv_lens=kv_lens) if q.dtype == torch.bfloat16 else None
    return ref, absref


def _check(q, k, v, causal, dev, kv_len=None):
    from b200k import fmha
    o = fmha.fmha_fwd(q.to(dev), k.to(dev), v.to(dev), causal=causal, kv_len=kv_len)
    torch.cuda.synchronize()
    ref, absref = _refs(q, k, v, causal, kv_len)
    _assert_close(o, ref, absref=absref)
    assert not torch.isnan(o).any()
    return o


def test_uniform_v_and_onehot(cuda_device):
    """Structured inputs that pin operand layouts exactly: with V constant along keys
    the output equals that constant row; with one very large logit per query the
    output equals the selected V row."""
    from b200k import fmha, inputs
    B, H, S, D = 1, 2, 256, 128
    q, k, v = inputs.fmha_inputs(B, H, H, S, S, D, torch.float16, seed=7)
    vconst = torch.arange(D, dtype=torch.float16).view(1, 1, 1, D).expand(B, H, S, D).contiguous() / 16
    o = fmha.fmha_fwd(q.to(cuda_device), k.to(cuda_device), vconst.to(cuda_device))
    assert torch.allclose(o.cpu().float(), vconst.float(), atol=2e-2)
    # q_i = 12 * e_{i mod D}, k_j = 12 * e_{perm[j] mod D} on the first D keys, others 0
    q = torch.zeros(B, H, S, D, dtype=torch.float16)
    k = torch.zeros(B, H, S, D, dtype=torch.float16)
    g = torch.Generator().manual_seed(3)
    perm = torch.randperm(D, generator=g)
    for i in range(S):
        q[..., i, i % D] = 12.0
    for j in range(D):
        k[..., j, perm[j]] = 12.0
    o = fmha.fmha_fwd(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), scale=1.0).cpu()
    ref = oracle.fmha_ref(q, k, v, scale=1.0)
    assert oracle.max_abs(o, ref) <= 4e-3


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("S", [128, 256, 384, 1024])
def test_parity_square(cuda_device, S, D, causal, dtype):
    from b200k import inputs
    q, k, v = inputs.fmha_inputs(2, 4, 4, S, S, D, dtype, seed=S + D)
    _check(q, k, v, causal, cuda_device)


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("S", [1, 17, 64, 65, 129, 257, 300, 513])
def test_parity_ragged(cuda_device, S, causal):
    """Sequence lengths that are not multiples of the tile (the reference pads to 64 in
    Python; here the kernel clips)."""
    from b200k import inputs
    q, k, v = inputs.fmha_inputs(1, 4, 4, S, S, 128, torch.float16, seed=S)
    _check(q, k, v, causal, cuda_device)


@pytest.mark.parametrize("group", [1, 4, 8])
def test_parity_gqa(cuda_device, group):
    from b200k import inputs
    q, k, v = inputs.fmha_inputs(2, 8, 8 // group, 384, 384, 128, torch.float16, seed=group)
    _check(q, k, v, True, cuda_device)


@pytest.mark.parametrize("causal", [False, True])
def test_parity_cross_lengths(cuda_device, causal):
    """Sq != Skv (bottom-right aligned diagonal) and a valid length below Skv with NaN
    in the padding: padded keys must never reach the result."""
    from b200k import inputs
    q, k, v = inputs.fmha_inputs(1, 4, 2, 200, 700, 128, torch.float16, seed=9)
    _check(q, k, v, causal, cuda_device)
    k[:, :, 555:] = float("nan")
    v[:, :, 555:] = float("nan")
    _check(q, k, v, causal, cuda_device, kv_len=555)
    # more queries than keys: the first rows see no key at all under the causal rule -> zeros
    q2, k2, v2 = inputs.fmha_inputs(1, 2, 2, 300, 100, 128, torch.float16, seed=10)
    _check(q2, k2, v2, causal, cuda_device)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("shape", [(257, 257, 173), (128, 258, 108), (520, 520, 25), (256, 256, 64), (200, 140, 31)])
def test_rows_without_a_visible_key_are_zero(cuda_device, shape, D, dtype):
    """Causal with fewer valid keys than queries (diagonal aligned bottom-right to kv_len): the first
    Sq - kv_len rows see no key and are zero, also when they share a 128-row tile with rows that do see
    keys - then the tile's blocks run, every score of such a row is masked, and nothing of V may leak into
    it.  (In bf16 the clamped 2^-125 of an emulated exponential survives the rounding of P; a row's
    denominator made of those once turned its output into a mean of V.)  All kernel variants."""
    from b200k import fmha, inputs
    Sq, Skv, kv_len = shape
    q, k, v = inputs.fmha_inputs(2, 4, 2, Sq, Skv, D, dtype, seed=31 + Sq)
    k[:, :, kv_len:] = float("nan")
    v[:, :, kv_len:] = float("nan")
    ref, absref = _refs(q, k, v, True, kv_len)
    dead = max(0, Sq - kv_len)
    assert dead > 0 and float(ref[:, :, :dead].abs().max()) == 0.0
    for variant in (0, 1, 2, 3, 11, 12, 13):
        o = fmha.fmha_fwd(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), causal=True, kv_len=kv_len,
                          variant=variant)
        torch.cuda.synchronize()
        assert float(o[:, :, :dead].float().abs().max()) == 0.0, variant
        _assert_close(o, ref, absref=absref)


def test_bshd_storage_is_zero_copy(cuda_device):
    """Tensors stored [B,S,H,D] and viewed [B,H,S,D] are consumed through strides."""
    from b200k import fmha, inputs
    q, k, v = inputs.fmha_inputs(2, 8, 2, 320, 320, 128, torch.float16, seed=12)
    qs, ks, vs = inputs.fmha_inputs(2, 8, 2, 320, 320, 128, torch.float16, device=cuda_device, seed=12, layout="bshd")
    assert not qs.is_contiguous()
    out = torch.empty(2, 320, 8, 128, dtype=torch.float16, device=cuda_device).transpose(1, 2)
    fmha.fmha_fwd(qs, ks, vs, causal=True, out=out)
    assert oracle.max_abs(out, oracle.fmha_ref(q, k, v, causal=True)) <= TOL


@pytest.mark.parametrize("layout", ["bhsd", "bshd"])
def test_config3_sample_heads(cuda_device, layout):
    """Causal fp16 B=1, 32/8 heads, s=4096, d=128 from seed 2, stored [B,H,S,D] and stored [B,S,H,D]
    viewed as [B,H,S,D] (no copy): CPU check of the first and last query head of two KV groups (all
    4096 rows each), through fine_fmha; both storages give the same bits."""
    from b200k import inputs
    import fmha_unified
    q, k, v = inputs.fmha_c3()
    qd, kd, vd = inputs.fmha_c3(cuda_device, layout=layout)
    assert qd.is_contiguous() == (layout == "bhsd")
    o = fmha_unified.ops.fine_fmha(qd, kd, vd, True, False, 5)
    assert o.shape == q.shape and o.dtype == q.dtype
    for h in (0, 3, 28, 31):
        ref = oracle.fmha_ref(q[:, h:h + 1], k[:, h // 4:h // 4 + 1], v[:, h // 4:h // 4 + 1], causal=True)
        err = oracle.max_abs(o[:, h:h + 1], ref)
        assert err <= TOL, (h, err)
    if layout == "bshd":
        qc, kc, vc = inputs.fmha_c3(cuda_device)
        assert torch.equal(o, fmha_unified.ops.fine_fmha(qc, kc, vc, True, False, 5))


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("S", [1024, 2048, 8192])
@pytest.mark.parametrize("D", [64, 128])
def test_config4_bf16_all_cases(cuda_device, D, S, causal):
    """All twelve bf16 MHA prefill cases at their own size (B=8, 32 heads, d in {64, 128}, s in {1024,
    2048, 8192}, full and causal).  The operands are drawn on the device; three (batch, head) pairs
    (first, last, one inside) are copied back and checked on the CPU against the fp32 formula, all
    s rows each."""
    from b200k import fmha, inputs
    shape = (8, 32, S, D)
    q = inputs.device_randn16(shape, 300 + D + S, 1.0, torch.bfloat16, cuda_device)
    k = inputs.device_randn16(shape, 301 + D + S, 1.0, torch.bfloat16, cuda_device)
    v = inputs.device_randn16(shape, 302 + D + S, 1.0, torch.bfloat16, cuda_device)
    o = fmha.fmha_fwd(q, k, v, causal=causal)
    assert not torch.isnan(o).any()
    for (b, h) in ((0, 0), (7, 31), (3, 17)):
        ref, absref = _refs(q[b:b + 1, h:h + 1].cpu(), k[b:b + 1, h:h + 1].cpu(), v[b:b + 1, h:h + 1].cpu(), causal)
        _assert_close(o[b:b + 1, h:h + 1], ref, where=(b, h), absref=absref)


def test_determinism_and_batch_independence(cuda_device):
    """Same launch three times is bit-identical; a (batch, head) shard computed alone equals
    the same slice of the full launch bit for bit (the sharding used across GPUs)."""
    from b200k import fmha, inputs
    q, k, v = inputs.fmha_inputs(4, 8, 2, 512, 512, 128, torch.float16, device=cuda_device, seed=21)
    outs = [fmha.fmha_fwd(q, k, v, causal=True) for _ in range(3)]
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    part = fmha.fmha_fwd(q[1:3, 4:8], k[1:3, 1:2], v[1:3, 1:2], causal=True)
    assert torch.equal(part, outs[0][1:3, 4:8])


def test_reference_wrapper_semantics(cuda_device):
    """fine_fmha keeps the reference's signature, shapes and error behaviour."""
    import fmha_unified
    from b200k import inputs
    q, k, v = inputs.fmha_inputs(1, 4, 1, 100, 100, 128, torch.float16, device=cuda_device, seed=4)
    for idx in range(6):
        o = fmha_unified.ops.fine_fmha(q, k, v, True, False, idx)
        assert o.shape == (1, 4, 100, 128)
    ref = oracle.fmha_ref(q, k, v, causal=True)
    assert oracle.max_abs(o, ref) <= TOL
    with pytest.raises(RuntimeError):
        fmha_unified.ops.fine_fmha(q, k, v, True, True, 0)       # causal together with decode
    with pytest.raises((RuntimeError, NotImplementedError)):
        fmha_unified.ops.fine_fmha(q, k, v, True, False, 6)      # declared, not implemented
    with pytest.raises(RuntimeError):
        fmha_unified.ops.fine_fmha(q.float(), k.float(), v.float(), True, False, 0)


@pytest.mark.parametrize("variant", [1, 2, 3, 4, 5, 11, 12, 13, 14, 15])
def test_kernel_variants_agree(cuda_device, variant):
    """One-item-per-CTA and persistent kernels, with 0 to 4 of every 8 exponentials on the FMA pipe:
    all within tolerance of the oracle, causal with ragged length and GQA."""
    from b200k import fmha, inputs
    q, k, v = inputs.fmha_inputs(2, 8, 2, 700, 700, 128, torch.float16, seed=44)
    o = fmha.fmha_fwd(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), causal=True, variant=variant)
    assert oracle.max_abs(o, oracle.fmha_ref(q, k, v, causal=True)) <= TOL
    q, k, v = inputs.fmha_inputs(3, 4, 4, 130, 5000, 64, torch.bfloat16, seed=45)
    o = fmha.fmha_fwd(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), causal=False, variant=variant)
    ref, absref = _refs(q, k, v, False)
    _assert_close(o, ref, absref=absref)


@pytest.mark.parametrize("variant", [0, 2, 12])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_d64_separate_and_shared_p_buffers(cuda_device, variant, dtype):
    """Head dimension 64 can keep P in TMEM columns of its own (B200K_OPT_FMHA_SPLIT_P = 1), so that the next
    block's QK^T is issued ahead of this block's PV product; by default P goes over its S columns.  Both orders
    of issue meet the oracle on the shapes that stress the hand-overs (many blocks per tile, tiles with
    different block counts under the causal mask, ragged ends, GQA, keys beyond 4096 for the
    one-item-per-CTA kernel) and agree with each other within the tolerance."""
    from b200k import _lib, fmha, inputs
    cases = [(2, 8, 2, 700, 700, True), (1, 4, 4, 300, 5000, False), (1, 2, 1, 1500, 1500, True),
             (3, 4, 4, 130, 130, False)]
    for (B, Hq, Hkv, Sq, Skv, causal) in cases:
        q, k, v = inputs.fmha_inputs(B, Hq, Hkv, Sq, Skv, 64, dtype, seed=Sq + Skv)
        qd, kd, vd = q.to(cuda_device), k.to(cuda_device), v.to(cuda_device)
        ref, absref = _refs(q, k, v, causal)
        outs = []
        for mode in (1, 0):
            with _lib.option(_lib.OPT_FMHA_SPLIT_P, mode):
                o = fmha.fmha_fwd(qd, kd, vd, causal=causal, variant=variant)
                o2 = fmha.fmha_fwd(qd, kd, vd, causal=causal, variant=variant)
            assert torch.equal(o, o2)
            _assert_close(o, ref, where=(Sq, Skv, causal, mode), absref=absref)
            outs.append(o)
        assert float((outs[0].float() - outs[1].float()).abs().max()) <= 2 * TOL + float(ref.abs().max()) * 2.0 ** -7


@pytest.mark.parametrize("variant", [2, 12])
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_rising_row_maximum(cuda_device, variant, D, dtype):
    """Keys whose magnitude grows along the sequence: the running row maximum climbs by far more than
    the lazy-rescale threshold (2^8), in steps small and large, so both kernels' rescale path (O and l
    scaled in place) runs many times per row.
    Non-causal and causal, the causal case with the ragged tail masked."""
    from b200k import fmha, inputs
    S = 1500
    q, k, v = inputs.fmha_inputs(1, 4, 2, S, S, D, dtype, seed=91 + D)
    ramp = torch.linspace(0.05, 6.0, S).view(1, 1, S, 1)
    ramp[:, :, 640:] *= 2.5  # one large jump in the middle of a block
    k = (k.float() * ramp).to(dtype)
    for causal in (False, True):
        o = fmha.fmha_fwd(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), causal=causal, variant=variant)
        ref, absref = _refs(q, k, v, causal)
        assert not torch.isnan(o).any()
        # the softmax is nearly one-hot here, so |o| reaches several units: allow the output's own
        # rounding (half an ulp at max|o|: 2^-11 relative in fp16) on top of the stated tolerance
        _assert_close(o, ref, where=(causal,), extra=float(ref.abs().max()) * 2.0 ** -10, absref=absref)
