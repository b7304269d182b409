"""GPU parity of the GEMM path against the CPU oracle, through the C ABI
(b200k_gemm via ctypes) and through the reference-facing op
(gemm_unified.ops.fine_gemm).  Tolerance: relative Frobenius error <= 1e-2
against the fp32 CPU matmul (the stated bar); in practice fp32 accumulation
lands near the 16-bit output rounding (~1e-3)."""
import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu

TOL = oracle.GEMM_REL_FRO_TOL


@pytest.fixture
def skinny_splits():
    """Forces the K-split count (cluster size) of the weight-streaming GEMM for one test through the
    library's tuning override and puts the library's own choice back afterwards."""
    from b200k import _lib
    before = []

    def force(splits: int):
        before.append(_lib.lib().b200k_set_option(_lib.OPT_SKINNY_S, int(splits)))

    yield force
    if before:
        _lib.lib().b200k_set_option(_lib.OPT_SKINNY_S, before[0])


def _run(a, b, variant, dev):
    from b200k import gemm
    c = gemm.gemm(a.to(dev), b.to(dev), variant=variant)
    torch.cuda.synchronize()
    return c.cpu()


def _inputs(M, N, K, dtype, seed=0, std_b=1.0):
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(M, K, generator=g).to(dtype)
    b = (torch.randn(K, N, generator=g) * std_b).to(dtype)
    return a, b


@pytest.mark.parametrize("variant", [1, 2, 4, 6, 7])
def test_structured_identity(cuda_device, variant):
    """A = I picks rows of B; B = I picks columns of A: catches operand-layout
    (descriptor / swizzle / major-ness) mistakes exactly, with no tolerance."""
    from b200k import gemm
    n = 256
    eye = torch.eye(n, dtype=torch.float16)
    g = torch.Generator().manual_seed(5)
    x = torch.randint(-8, 9, (n, n), generator=g).to(torch.float16)
    assert torch.equal(_run(eye, x, variant, cuda_device), x)
    assert torch.equal(_run(x, eye, variant, cuda_device), x)
    # one-hot rows: C[i, :] = B[perm[i], :]
    perm = torch.randperm(n, generator=g)
    onehot = torch.zeros(n, n, dtype=torch.float16)
    onehot[torch.arange(n), perm] = 1
    assert torch.equal(_run(onehot, x, variant, cuda_device), x[perm])


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("variant", [0, 1, 2, 4, 5, 6, 7])
@pytest.mark.parametrize("shape", [(128, 256, 64), (128, 128, 128), (256, 512, 256), (1024, 1024, 1024),
                                   (384, 768, 4096)])
def test_parity_aligned(cuda_device, shape, variant, dtype):
    M, N, K = shape
    a, b = _inputs(M, N, K, dtype, seed=M + N + K)
    c = _run(a, b, variant, cuda_device)
    err = oracle.rel_frobenius(c, oracle.gemm_ref(a, b))
    assert err <= TOL, err


@pytest.mark.parametrize("variant", [0, 1, 2, 4, 6, 7])
@pytest.mark.parametrize("shape", [(1, 8, 8), (7, 72, 40), (63, 136, 72), (65, 264, 200), (129, 520, 1000),
                                   (16, 4096, 4096), (300, 11008, 136)])
def test_parity_ragged_edges(cuda_device, shape, variant):
    """Tails in every dimension (TMA zero-fill on loads, clipping on stores)."""
    M, N, K = shape
    a, b = _inputs(M, N, K, torch.float16, seed=M * 3 + N * 5 + K * 7, std_b=0.1)
    out = torch.full((M + 2, N + 8), float("nan"), dtype=torch.float16, device=cuda_device)
    from b200k import gemm
    view = out[1:M + 1, :N]  # ldc = N + 8: keeps 16-byte alignment, leaves a NaN frame
    gemm.gemm(a.to(cuda_device), b.to(cuda_device), out=view, variant=variant)
    torch.cuda.synchronize()
    host = out.cpu()
    err = oracle.rel_frobenius(host[1:M + 1, :N], oracle.gemm_ref(a, b))
    assert err <= TOL, err
    # nothing outside the [M, N] window was written
    assert torch.isnan(host[0]).all() and torch.isnan(host[M + 1]).all() and torch.isnan(host[:, N:]).all()


@pytest.mark.parametrize("shape", [(5, 7, 3), (33, 65, 129), (130, 250, 77)])
def test_generic_unaligned(cuda_device, shape):
    """Shapes that break the 16-byte rules go to the CUDA-core kernel under AUTO."""
    M, N, K = shape
    a, b = _inputs(M, N, K, torch.float16, seed=11)
    c = _run(a, b, 0, cuda_device)
    assert oracle.rel_frobenius(c, oracle.gemm_ref(a, b)) <= TOL


def test_config1_fp16_1024(cuda_device):
    """fp16 1024^3, A, B ~ N(0,1)*0.1 from seed 0; also through the reference-facing op."""
    from b200k import inputs
    import gemm_unified
    a, b = inputs.gemm_c1()
    ref = oracle.gemm_ref(a, b)
    for idx in (0, 8, 9, 10, 11, 12):
        c = gemm_unified.ops.fine_gemm(a.to(cuda_device), b.to(cuda_device), idx)
        assert c.dtype == torch.float16 and c.shape == (1024, 1024)
        err = oracle.rel_frobenius(c, ref)
        assert err <= TOL, (idx, err)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M", [1, 16, 128, 2048])
def test_config2_llm_shapes_rows(cuda_device, M, dtype):
    """LLM projection shapes: full CPU check for M <= 128, a row sample for larger M."""
    from b200k import inputs
    for (K, N) in inputs.LLAMA7B_KN:
        a, w = inputs.gemm_llm(M, K, N, dtype)
        c = _run(a, w, 0, cuda_device)
        rows = torch.arange(M) if M <= 128 else torch.tensor([0, 1, 127, 128, 129, M // 2, M - 2, M - 1])
        ref = oracle.gemm_ref(a[rows], w)
        err = oracle.rel_frobenius(c[rows], ref)
        assert err <= TOL, (M, K, N, err)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("KN", [(4096, 4096), (4096, 11008), (11008, 4096), (4096, 12288)])
def test_config2_m8192_all_weights(cuda_device, KN, dtype):
    """M = 8192 tokens against each of the four Llama-2-7B-shaped weights, both dtypes, at full size:
    operands drawn on the device (activations N(0,1), weights N(0,0.02)), a sample of rows (tile edges,
    first and last) copied back and checked on the CPU against the fp32 matmul over all N columns; the
    reference-facing op gives the same bits as the C-ABI wrapper."""
    from b200k import gemm, inputs
    import gemm_unified
    K, N = KN
    M = 8192
    a = inputs.device_randn16((M, K), 500 + K, 1.0, dtype, cuda_device)
    w = inputs.device_randn16((K, N), 600 + N, 0.02, dtype, cuda_device)
    c = gemm.gemm(a, w)
    rows = torch.tensor([0, 127, 128, 255, 256, 4095, 4096, 8000, 8190, 8191])
    ref = oracle.gemm_ref(a[rows].cpu(), w.cpu())
    err = oracle.rel_frobenius(c[rows], ref)
    assert err <= TOL, err
    assert torch.equal(gemm_unified.ops.fine_gemm(a, w, 12), c)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(1, 128, 64), (16, 256, 4096), (64, 4096, 4096), (128, 1000, 2048), (7, 136, 200),
                                   (33, 11008, 4096), (100, 520, 11008)])
def test_skinny_split_k_clusters(cuda_device, shape, dtype):
    """M <= 128: split-K inside clusters of 1..8 CTAs with the reduction through distributed
    shared memory; ragged N and K; bit-identical reruns (fixed summation order)."""
    M, N, K = shape
    a, b = _inputs(M, N, K, dtype, seed=M + N + K, std_b=0.05)
    c1 = _run(a, b, 3, cuda_device)
    c2 = _run(a, b, 3, cuda_device)
    assert torch.equal(c1, c2)
    err = oracle.rel_frobenius(c1, oracle.gemm_ref(a, b))
    assert err <= TOL, err


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("splits", [1, 2, 5, 8])
@pytest.mark.parametrize("shape", [(1, 136, 192), (7, 264, 200), (16, 512, 1024), (33, 1096, 520), (64, 2048, 512),
                                   (100, 520, 264), (128, 384, 640)])
def test_skinny_cluster_sizes_and_epilogues(cuda_device, skinny_splits, shape, splits, dtype):
    """Every cluster size the heuristic can pick, forced through the documented override, with all
    three epilogues: a cluster of one stores C straight from the accumulators (odd row counts, ragged
    N), larger ones reduce through distributed shared memory (uneven column shares at 5 and 8)."""
    from b200k import gemm
    skinny_splits(splits)
    M, N, K = shape
    a, b = _inputs(M, N, K, dtype, seed=M + N + K + splits, std_b=0.1)
    ad, bd = a.to(cuda_device), b.to(cuda_device)
    ref = oracle.gemm_ref(a, b)
    assert oracle.rel_frobenius(gemm.gemm(ad, bd, variant=3), ref) <= TOL
    g = torch.Generator().manual_seed(5)
    r = torch.randn(M, N, generator=g).to(dtype)
    assert oracle.rel_frobenius(gemm.gemm_add(ad, bd, r.to(cuda_device)), ref + r.float()) <= TOL
    if N % 16 == 0:
        got = gemm.gemm_swiglu(ad, bd)
        want = torch.nn.functional.silu(ref[:, 0::2]) * ref[:, 1::2]
        assert got.shape == (M, N // 2) and oracle.rel_frobenius(got, want) <= TOL


@pytest.mark.parametrize("splits", [0, 1, 3])
@pytest.mark.parametrize("M", [5, 64, 128])
def test_skinny_strided_operands(cuda_device, skinny_splits, M, splits):
    """Row-strided A, B and C (views into wider tensors, as the column-slab sharding produces them): the
    weight-streaming kernel honours all three leading dimensions on its direct-store, push and pull
    paths, and leaves the columns outside the output view untouched."""
    from b200k import gemm
    skinny_splits(splits)
    K, N = 520, 392
    g = torch.Generator().manual_seed(M + splits)
    a_big = torch.randn(M, K + 24, generator=g).to(torch.bfloat16).to(cuda_device)
    b_big = (torch.randn(K, N + 40, generator=g) * 0.1).to(torch.bfloat16).to(cuda_device)
    c_big = torch.full((M, N + 64), 7.0, dtype=torch.bfloat16, device=cuda_device)
    a, b, c = a_big[:, 8:8 + K], b_big[:, 16:16 + N], c_big[:, 32:32 + N]
    gemm.gemm(a, b, out=c, variant=3)
    ref = oracle.gemm_ref(a.cpu(), b.cpu())
    assert oracle.rel_frobenius(c, ref) <= TOL
    assert bool((c_big[:, :32] == 7.0).all()) and bool((c_big[:, 32 + N:] == 7.0).all())


@pytest.mark.parametrize("splits", [1, 3])
@pytest.mark.parametrize("N", [130, 134, 263, 517])
@pytest.mark.parametrize("M", [3, 64, 128])
def test_skinny_column_window_ragged_n(cuda_device, skinny_splits, M, N, splits):
    """C (and the residual R) as the first N columns of a wider tensor with N not a multiple of 4 (nor
    of 2): the weight-streaming kernel's 4-wide (split-K) and 2-wide (single CTA) stores must stop at
    column N, and the fused add must not read R beyond it."""
    from b200k import gemm
    skinny_splits(splits)
    K = 264
    a, b = _inputs(M, N, K, torch.bfloat16, seed=M + N, std_b=0.1)
    wide = (N + 15) // 8 * 8 + 8
    bd = torch.zeros(K, wide, dtype=torch.bfloat16, device=cuda_device)
    bd[:, :N] = b.to(cuda_device)
    big = torch.full((M, wide), 7.0, dtype=torch.bfloat16, device=cuda_device)
    gemm.gemm(a.to(cuda_device), bd[:, :N], out=big[:, :N], variant=3)
    ref = oracle.gemm_ref(a, b)
    assert oracle.rel_frobenius(big[:, :N], ref) <= TOL
    assert bool((big[:, N:] == 7.0).all())
    rbig = torch.full((M, wide), float("nan"), dtype=torch.bfloat16, device=cuda_device)
    g = torch.Generator().manual_seed(N)
    r = torch.randn(M, N, generator=g).to(torch.bfloat16)
    rbig[:, :N] = r.to(cuda_device)
    big.fill_(7.0)
    gemm.gemm_add(a.to(cuda_device), bd[:, :N], rbig[:, :N], out=big[:, :N])
    assert not torch.isnan(big).any()
    assert oracle.rel_frobenius(big[:, :N], ref + r.float()) <= TOL
    assert bool((big[:, N:] == 7.0).all())


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(1, 256, 512), (16, 264, 520), (33, 1160, 1024), (64, 1288, 4096), (64, 11008, 4096),
                                   (7, 12288, 576), (48, 384, 8192)])
def test_skinny_two_slabs_per_cluster(cuda_device, shape, dtype):
    """The paired-slab decomposition of the weight-streaming GEMM (clusters of three CTAs over two 128-column
    slabs, the middle CTA holding two accumulators), forced on wherever it can run: even and odd slab
    counts (an odd last slab is paired with columns beyond N), ragged N and K, all three epilogues,
    bit-identical reruns, and the same result as the one-slab-per-cluster decomposition within rounding."""
    from b200k import _lib, gemm
    M, N, K = shape
    a, b = _inputs(M, N, K, dtype, seed=M + N + K, std_b=0.05)
    ad, bd = a.to(cuda_device), b.to(cuda_device)
    ref = oracle.gemm_ref(a, b)
    n0 = _lib.launch_count()
    with _lib.option(_lib.OPT_SKINNY_PAIR, 1):
        c1 = gemm.gemm(ad, bd, variant=3)
        c2 = gemm.gemm(ad, bd, variant=3)
        g = torch.Generator().manual_seed(5)
        r = torch.randn(M, N, generator=g).to(dtype)
        cadd = gemm.gemm_add(ad, bd, r.to(cuda_device))
        cswi = gemm.gemm_swiglu(ad, bd) if N % 16 == 0 else None
    with _lib.option(_lib.OPT_SKINNY_PAIR, 2):
        c0 = gemm.gemm(ad, bd, variant=3)
    assert torch.equal(c1, c2)
    assert oracle.rel_frobenius(c1, ref) <= TOL
    assert oracle.rel_frobenius(c1, c0.float().cpu()) <= 2e-3     # same products, other summation split
    assert oracle.rel_frobenius(cadd, ref + r.float()) <= TOL
    if cswi is not None:
        assert oracle.rel_frobenius(cswi, torch.nn.functional.silu(ref[:, 0::2]) * ref[:, 1::2]) <= TOL
    # a column window of a wider output: nothing outside it is written
    big = torch.full((M, N + 24), 7.0, dtype=dtype, device=cuda_device)
    with _lib.option(_lib.OPT_SKINNY_PAIR, 1):
        gemm.gemm(ad, bd, out=big[:, 8:8 + N], variant=3)
    assert torch.equal(big[:, 8:8 + N], c1) and bool((big[:, :8] == 7.0).all()) and bool((big[:, 8 + N:] == 7.0).all())


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_skinny_dependent_launch_chain(cuda_device, mode):
    """Programmatic dependent launch of the weight-streaming GEMM: a launch may begin while the kernel
    before it in the stream still runs and must wait for it before it reads its activations or writes C.
    A chain in which every GEMM consumes the previous one's output (as the projections of a decode step
    do), launched back to back without host synchronisation and also replayed from a CUDA graph, gives
    the bits of the same chain with plain launches (mode 2); mode 1 additionally requests the first weight
    tiles before the wait (weights here are constants).  In the default mode the weight itself may have
    been written by the kernel just before (filled on the device, then multiplied at once)."""
    from b200k import _lib, gemm
    M, K = 48, 1024
    g = torch.Generator().manual_seed(9)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(cuda_device)
    ws = [(torch.randn(K, K, generator=g) * 0.03).to(torch.bfloat16).to(cuda_device) for _ in range(6)]

    def chain():
        y = x
        for w in ws:
            y = gemm.gemm(y, w, variant=3)
        return y

    with _lib.option(_lib.OPT_PDL, 2):
        want = chain()
    torch.cuda.synchronize()
    with _lib.option(_lib.OPT_PDL, mode):
        got = [chain() for _ in range(5)]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            chain()
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out = chain()
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        assert all(torch.equal(y, want) for y in got) and torch.equal(out, want)
        if mode != 1:
            # the weight is produced by the kernel right before the GEMM, again and again
            w = torch.empty(K, 1536, dtype=torch.bfloat16, device=cuda_device)
            for i in range(8):
                w.fill_(0.001 * (i + 1))
                y = gemm.gemm(x, w, variant=3)
                ref = x.float().sum(dim=1, keepdim=True) * (torch.tensor(0.001 * (i + 1)).bfloat16().float())
                assert torch.allclose(y.float(), ref.expand(-1, 1536), rtol=2e-2, atol=2e-2), i
    ref = x.float().cpu()
    for w in ws:
        ref = (ref @ w.float().cpu()).to(torch.bfloat16).float()
    assert oracle.rel_frobenius(want, ref) <= 2e-2


def test_skinny_rejects_large_m(cuda_device):
    from b200k import _lib, gemm
    a = torch.zeros(256, 64, dtype=torch.float16, device=cuda_device)
    b = torch.zeros(64, 128, dtype=torch.float16, device=cuda_device)
    with pytest.raises(_lib.B200KError) as e:
        gemm.gemm(a, b, variant=3)
    assert e.value.code == -2


def test_determinism(cuda_device):
    a, b = _inputs(512, 1024, 2048, torch.bfloat16, seed=3)
    outs = [_run(a, b, 1, cuda_device) for _ in range(3)]
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])


def test_linearity_full_size(cuda_device):
    """Full-size property check (M=8192, K=4096, N=11008): (2A).B == 2(A.B) exactly in
    binary floating point, and column slabs computed alone equal the same slabs of
    the full product bit for bit (the N-tile sharding used across GPUs)."""
    from b200k import gemm, inputs
    a = inputs.device_randn16((8192, 4096), 1, 1.0, torch.bfloat16, cuda_device)
    w = inputs.device_randn16((4096, 11008), 2, 0.02, torch.bfloat16, cuda_device)
    c = gemm.gemm(a, w)
    c2 = gemm.gemm(a * 2, w)
    assert torch.equal(c2, c * 2)
    slab = gemm.gemm(a, w[:, 2752:5504])
    assert torch.equal(slab, c[:, 2752:5504])
    # spot check of 8 rows against the CPU oracle
    rows = torch.tensor([0, 127, 128, 4095, 4096, 8000, 8190, 8191])
    ref = oracle.gemm_ref(a[rows].cpu(), w.cpu())
    assert oracle.rel_frobenius(c[rows], ref) <= TOL


@pytest.mark.parametrize("N", [1408, 5504, 1472, 1288])
def test_large_m_partly_filled_last_tile(cuda_device, N):
    """M = 8192, K = 4096 against column slabs whose last tile is half full or less (1408 = 5.5 tiles of
    256 columns and 5504 = 21.5 are the slabs of the 4096x11008 weight on 8 and 2 GPUs; 1472 = 11.5 tiles
    of 128; 1288 leaves 8 columns): chunks of the last tile that lie outside C store nothing, and the
    epilogue's two staging buffers must still not be overwritten while an earlier store reads them - a
    race that only shows on a GEMM large enough to keep the stores in flight.  Every element is
    checked against the fp32 CPU product, and all tensor-core variants agree to the bit."""
    from b200k import gemm, inputs
    M, K = 8192, 4096
    a = inputs.device_randn16((M, K), 700 + N, 1.0, torch.bfloat16, cuda_device)
    w = inputs.device_randn16((K, 11008), 800 + N, 0.02, torch.bfloat16, cuda_device)
    ws = w[:, 2816:2816 + N]          # a view into the wider weight, as the sharding produces it
    ref = oracle.gemm_ref(a.cpu(), ws.cpu())
    first = None
    for variant in (0, 2, 1, 4, 6, 7):
        for rep in range(2):
            c = gemm.gemm(a, ws, variant=variant)
            host = c.cpu().float()
            assert torch.allclose(host, ref, rtol=2.0 ** -7, atol=1e-2), (variant, rep, float((host - ref).abs().max()))
            if first is None:
                first = c
            assert torch.equal(c, first), (variant, rep)


def test_error_codes(cuda_device):
    from b200k import gemm
    a = torch.zeros(8, 8, dtype=torch.float16, device=cuda_device)
    with pytest.raises(RuntimeError):
        gemm.gemm(a, torch.zeros(16, 8, dtype=torch.float16, device=cuda_device))
    with pytest.raises(RuntimeError):
        gemm.gemm(a, a.float())
    with pytest.raises(RuntimeError):
        gemm.gemm(a.cpu(), a.cpu())
    with pytest.raises(RuntimeError):  # tensor-core variant on a misaligned leading dimension
        gemm.gemm(torch.zeros(8, 9, dtype=torch.float16, device=cuda_device)[:, :8],
                  torch.zeros(8, 9, dtype=torch.float16, device=cuda_device)[:, :8], variant=1)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(128, 256, 64), (300, 520, 200), (1024, 4096, 512), (4096, 4096, 1024),
                                   (1, 256, 192), (8, 4096, 1024), (33, 1024, 2112), (64, 2048, 4096), (100, 520, 200),
                                   (100, 11008, 520)])
def test_fused_residual_add(cuda_device, shape, dtype):
    """C = A.B + R with the add in the epilogue (fp32 before the single rounding): M <= 128 takes the
    weight-streaming kernel (split-K in clusters, every row padding 16..128), larger shapes the 128x128
    kernel, (4096, 4096) the CTA-pair kernel; ragged edges included."""
    from b200k import gemm
    M, N, K = shape
    a, b = _inputs(M, N, K, dtype, seed=M + N + K, std_b=0.1)
    g = torch.Generator().manual_seed(77)
    r = torch.randn(M, N, generator=g).to(dtype)
    c = gemm.gemm_add(a.to(cuda_device), b.to(cuda_device), r.to(cuda_device))
    ref = oracle.gemm_ref(a, b) + r.float()
    assert oracle.rel_frobenius(c, ref) <= TOL


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(128, 128, 64), (300, 264, 200), (512, 2048, 512), (4096, 2048, 1024),
                                   (1, 128, 192), (8, 5504, 1024), (33, 520, 2112), (64, 1024, 4096), (100, 264, 200),
                                   (128, 5504, 512)])
def test_fused_swiglu(cuda_device, shape, dtype):
    """C = silu(A.Wg) * (A.Wu) from one GEMM over the column-interleaved [Wg|Wu] weight; decode-shaped
    row counts (M <= 128) go through the weight-streaming kernel's epilogue."""
    from b200k import gemm
    M, F, K = shape
    g = torch.Generator().manual_seed(M + F + K)
    a = torch.randn(M, K, generator=g).to(dtype)
    wg = (torch.randn(K, F, generator=g) * 0.1).to(dtype)
    wu = (torch.randn(K, F, generator=g) * 0.1).to(dtype)
    w = gemm.interleave_gate_up(wg, wu)
    assert torch.equal(w[:, 0::2], wg) and torch.equal(w[:, 1::2], wu)
    c = gemm.gemm_swiglu(a.to(cuda_device), w.to(cuda_device))
    assert c.shape == (M, F)
    gate, up = oracle.gemm_ref(a, wg), oracle.gemm_ref(a, wu)
    ref = torch.nn.functional.silu(gate) * up
    assert oracle.rel_frobenius(c, ref) <= TOL


def test_fused_argument_errors(cuda_device):
    from b200k import _lib, gemm
    a = torch.zeros(128, 64, dtype=torch.float16, device=cuda_device)
    b = torch.zeros(64, 72, dtype=torch.float16, device=cuda_device)
    with pytest.raises(_lib.B200KError) as e:          # N = 72 is not a multiple of 16
        gemm.gemm_swiglu(a, b)
    assert e.value.code == -2
    with pytest.raises(RuntimeError):
        gemm.gemm_add(a, b, torch.zeros(128, 64, dtype=torch.float16, device=cuda_device))
