"""Property tests over random shapes (hypothesis, fixed seed database off, derandomised):
every (M, N, K) with TMA-legal strides and every attention geometry the entry points accept
must match the CPU oracle within the stated tolerances, whichever kernel variant AUTO picks."""
import pytest
import torch
from hypothesis import HealthCheck, given, settings, strategies as st

from oracle import oracle

pytestmark = pytest.mark.gpu

_SETTINGS = dict(max_examples=30, deadline=None, derandomize=True, database=None,
                 suppress_health_check=[HealthCheck.function_scoped_fixture, HealthCheck.too_slow])


@settings(**_SETTINGS)
@given(m=st.integers(1, 520), n8=st.integers(1, 130), k8=st.integers(1, 130), bf16=st.booleans(),
       variant=st.sampled_from([0, 0, 1, 2, 4]))
def test_gemm_random_shapes(cuda_device, m, n8, k8, bf16, variant):
    from b200k import gemm
    N, K = n8 * 8, k8 * 8
    dtype = torch.bfloat16 if bf16 else torch.float16
    g = torch.Generator().manual_seed(m * 1000003 + N * 1009 + K)
    a = torch.randn(m, K, generator=g).to(dtype)
    b = (torch.randn(K, N, generator=g) * 0.1).to(dtype)
    c = gemm.gemm(a.to(cuda_device), b.to(cuda_device), variant=variant)
    err = oracle.rel_frobenius(c, oracle.gemm_ref(a, b))
    assert err <= oracle.GEMM_REL_FRO_TOL, (m, N, K, dtype, variant, err)


@settings(**_SETTINGS)
@given(b=st.integers(1, 2), hkv=st.integers(1, 3), group=st.sampled_from([1, 2, 4]), sq=st.integers(1, 400),
       extra=st.integers(0, 300), d=st.sampled_from([64, 128]), causal=st.booleans())
def test_fmha_random_geometry(cuda_device, b, hkv, group, sq, extra, d, causal):
    from b200k import fmha
    skv = sq + extra
    g = torch.Generator().manual_seed(b + 7 * hkv + 31 * group + 101 * sq + 1009 * extra + d)
    q = torch.randn(b, hkv * group, sq, d, generator=g).half()
    k = torch.randn(b, hkv, skv, d, generator=g).half()
    v = torch.randn(b, hkv, skv, d, generator=g).half()
    o = fmha.fmha_fwd(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), causal=causal)
    err = oracle.max_abs(o, oracle.fmha_ref(q, k, v, causal=causal))
    assert err <= oracle.FMHA_MAX_ABS_TOL, (b, hkv, group, sq, skv, d, causal, err)


@settings(**_SETTINGS)
@given(b=st.integers(1, 5), hkv=st.integers(1, 3), group=st.sampled_from([1, 4, 8]), skv=st.integers(1, 1500),
       d=st.sampled_from([64, 128]), splits=st.sampled_from([0, 1, 3, 8]), data=st.data())
def test_decode_random_lengths(cuda_device, b, hkv, group, skv, d, splits, data):
    from b200k import fmha
    lens = torch.tensor([data.draw(st.integers(0, skv)) for _ in range(b)], dtype=torch.int32)
    g = torch.Generator().manual_seed(b + 7 * hkv + 31 * group + 101 * skv + d)
    q = torch.randn(b, hkv * group, 1, d, generator=g).half()
    k = torch.randn(b, hkv, skv, d, generator=g).half()
    v = torch.randn(b, hkv, skv, d, generator=g).half()
    o = fmha.fmha_decode(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), kv_lens=lens.to(cuda_device),
                         num_splits=splits)
    ref = oracle.fmha_ref(q, k, v, kv_lens=lens)
    assert oracle.max_abs(o, ref) <= oracle.FMHA_MAX_ABS_TOL, (lens.tolist(), skv, d, splits)


@settings(**dict(_SETTINGS, max_examples=40))
@given(m=st.integers(1, 128), n16=st.sampled_from([1, 2, 5, 8, 9, 17, 40, 64, 129, 344, 600, 768]), k8=st.integers(1, 300),
       bf16=st.booleans(), epilogue=st.sampled_from(["none", "add", "swiglu"]))
def test_skinny_random_shapes_and_epilogues(cuda_device, m, n16, k8, bf16, epilogue):
    """Decode-shaped GEMMs (M <= 128) over narrow to very wide weights: every combination of slab width
    (128 / 256 columns), cluster size (1 = direct store, push and pull reductions) and epilogue that the
    heuristics can pick must match the oracle."""
    from b200k import gemm
    N, K = n16 * 16, k8 * 8
    dtype = torch.bfloat16 if bf16 else torch.float16
    g = torch.Generator().manual_seed(m * 1000003 + N * 1009 + K)
    a = torch.randn(m, K, generator=g).to(dtype)
    b = (torch.randn(K, N, generator=g) * 0.1).to(dtype)
    ref = oracle.gemm_ref(a, b)
    ad, bd = a.to(cuda_device), b.to(cuda_device)
    if epilogue == "none":
        got, want = gemm.gemm(ad, bd), ref
    elif epilogue == "add":
        r = torch.randn(m, N, generator=g).to(dtype)
        got, want = gemm.gemm_add(ad, bd, r.to(cuda_device)), ref + r.float()
    else:
        got, want = gemm.gemm_swiglu(ad, bd), torch.nn.functional.silu(ref[:, 0::2]) * ref[:, 1::2]
    err = oracle.rel_frobenius(got, want)
    assert err <= oracle.GEMM_REL_FRO_TOL, (m, N, K, dtype, epilogue, err)
