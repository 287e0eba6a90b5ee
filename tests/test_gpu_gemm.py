"""tcgen05/TMA GEMM against fp32 PyTorch matmul for every operand-major combination, odd sizes,
batched heads and K segments."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _k():
    from loomformer_paraplex_b200.ops import kernels
    return kernels


def _rel(a, b):
    return float((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-6))


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (2048, 768, 768), (300, 200, 136), (128, 3072, 768)])
@pytest.mark.parametrize("bn", [64, 128, 256])
def test_kmajor_linear(M, N, K, bn):
    k = _k()
    torch.manual_seed(0)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(N, device="cuda")
    c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    k.gemm([x], [K], w, c, M=M, N=N, bias=bias, bn=bn)
    ref = x.float() @ w.float().t() + bias
    k.check_status(c.device)
    assert _rel(c, ref) < 1e-2


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (2048, 768, 768), (300, 200, 136), (4096, 3072, 768), (520, 1160, 200)])
@pytest.mark.parametrize("bn", [128, 256])
def test_pair_tiles_kmajor_linear(M, N, K, bn):
    """256-row tiles computed by clusters of two CTAs (tcgen05 cta_group::2), ragged edges in both directions, more
    tiles than SM pairs (the persistent loop and both accumulator buffers are exercised), bias and accumulate."""
    k = _k()
    torch.manual_seed(0)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(N, device="cuda")
    c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    k.gemm([x], [K], w, c, M=M, N=N, bias=bias, bn=bn, pair=1)
    ref = x.float() @ w.float().t() + bias
    k.check_status(c.device)
    assert _rel(c, ref) < 1e-2
    c32 = torch.ones(M, N, device="cuda")
    k.gemm([x], [K], w, c32, M=M, N=N, bn=bn, pair=1, accumulate=True)
    k.check_status(c.device)
    assert _rel(c32, ref - bias + 1.0) < 1e-2


@pytest.mark.parametrize("pair", [0, 1])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_output_the_tma_unit_cannot_describe_takes_the_direct_epilogue(pair, dtype):
    """A row pitch that is not a multiple of 16 bytes (a column slice of a wider buffer) cannot go through the staged
    TMA epilogue; the per-row store path must give the same numbers and touch nothing outside the slice."""
    k = _k()
    torch.manual_seed(8)
    M, N, K = 520, 200, 136
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    wide = torch.full((M, N + (3 if dtype == torch.float32 else 2)), 7.0, device="cuda", dtype=dtype)
    c = wide[:, :N]
    k.gemm([x], [K], w, c, M=M, N=N, bn=128, pair=pair)
    k.check_status(c.device)
    assert _rel(c, x.float() @ w.float().t()) < 1e-2
    assert bool((wide[:, N:] == 7.0).all())


@pytest.mark.parametrize("a_mn,b_mn", [(False, True), (True, True), (True, False)])
def test_pair_tiles_other_operand_layouts(a_mn, b_mn):
    k = _k()
    torch.manual_seed(4)
    M, N, K = 776, 392, 264
    a = torch.randn(K, M, device="cuda", dtype=torch.bfloat16) if a_mn else torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(K, N, device="cuda", dtype=torch.bfloat16) if b_mn else torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    c = torch.zeros(M, N, device="cuda")
    k.gemm([a], [K], b, c, M=M, N=N, a_mn=a_mn, b_mn=b_mn, bn=128, pair=1)
    k.check_status(c.device)
    ref = (a.float().t() if a_mn else a.float()) @ (b.float() if b_mn else b.float().t())
    assert _rel(c, ref) < 1e-2


def test_pair_tiles_batched_heads_and_segments():
    """Per-head batched operands with two K segments on pair tiles."""
    k = _k()
    torch.manual_seed(6)
    M, heads, N, K1, K2 = 512, 4, 384, 96, 200
    a1 = torch.randn(M, heads, K1, device="cuda", dtype=torch.bfloat16)
    a2 = torch.randn(M, K2, device="cuda", dtype=torch.bfloat16)            # shared by all heads
    w = (torch.randn(N, heads, K1 + K2, device="cuda") * 0.1).to(torch.bfloat16)
    c = torch.empty(M, heads, N, device="cuda", dtype=torch.bfloat16)
    k.gemm([a1, a2], [K1, K2], w, c, M=M, N=N, heads=heads, b_k0=[0, K1], bn=128, pair=1)
    k.check_status(c.device)
    ref = torch.einsum("mhk,nhk->mhn", a1.float(), w.float()[:, :, :K1]) + torch.einsum("mk,nhk->mhn", a2.float(), w.float()[:, :, K1:])
    assert _rel(c, ref) < 1.5e-2


@pytest.mark.parametrize("M,N,K", [(256, 128, 128), (2048, 768, 3072), (264, 200, 136)])
def test_dgrad_mn_major_b(M, N, K):
    k = _k()
    torch.manual_seed(1)
    dy = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)          # reduction over K
    w = torch.randn(K, N, device="cuda", dtype=torch.bfloat16)           # [reduction, out] -> MN-major B
    c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    k.gemm([dy], [K], w, c, M=M, N=N, b_mn=True)
    k.check_status(c.device)
    assert _rel(c, dy.float() @ w.float()) < 1e-2


@pytest.mark.parametrize("M,N,K", [(128, 128, 256), (3072, 768, 2048), (200, 136, 264)])
def test_wgrad_both_mn_major_fp32_accumulate(M, N, K):
    k = _k()
    torch.manual_seed(2)
    dy = torch.randn(K, M, device="cuda", dtype=torch.bfloat16)          # [reduction, out rows]
    x = torch.randn(K, N, device="cuda", dtype=torch.bfloat16)           # [reduction, out cols]
    g = torch.randn(M, N, device="cuda")
    ref = g + dy.float().t() @ x.float()
    k.gemm([dy], [K], x, g, M=M, N=N, a_mn=True, b_mn=True, accumulate=True)
    k.check_status(g.device)
    assert _rel(g, ref) < 1e-2


def test_segmented_batched_imag_projection():
    from types import SimpleNamespace
    from loomformer_paraplex_b200.ops.twins import TorchKernels
    k = _k()
    for open_sectors in (False, True):
        qh, hd, hpq = 8, 96, 384
        n = qh * hd
        d = SimpleNamespace(qh=qh, hd=hd, hpq=hpq, n=n, hidden=qh * hpq, open_sectors=open_sectors,
                            imag_in=(4 * n + hd) if open_sectors else (n + 4 * hd))
        M = 384
        torch.manual_seed(3)
        qkc = torch.randn(M, 3, qh, hd, device="cuda", dtype=torch.bfloat16)
        u = torch.randn(M, n, device="cuda", dtype=torch.bfloat16)
        m2 = torch.randn(M, qh, hd, device="cuda", dtype=torch.bfloat16)
        w = (torch.randn(d.hidden, d.imag_in, device="cuda") * 0.05).to(torch.bfloat16)
        ck, tk = k.CudaKernels(), TorchKernels()
        out = ck.imag_fwd(d, qkc, u, m2, w)
        ref = tk.imag_fwd(d, qkc.float(), u.float(), m2.float(), w.float())
        assert _rel(out, ref) < 1.5e-2
        dbeta = torch.randn(M, d.hidden, device="cuda", dtype=torch.bfloat16)
        g1 = torch.zeros(d.hidden, d.imag_in, device="cuda")
        g2 = torch.zeros_like(g1)
        a1 = ck.imag_bwd(d, dbeta, qkc, u, m2, w, g1)
        ck.flush_wgrads()
        a2 = tk.imag_bwd(d, dbeta.float(), qkc.float(), u.float(), m2.float(), w.float(), g2)
        k.check_status(u.device)
        assert not ck.fallbacks, ck.fallbacks
        assert _rel(g1, g2) < 1.5e-2
        for x1, x2 in zip(a1, a2):
            assert _rel(x1, x2) < 1.5e-2


def test_grouped_wgrad_queue_equals_per_chunk_products():
    """Sixteen queued chunk products leave as one launch with per-segment operands; a ragged queue flushes on demand."""
    k = _k()
    torch.manual_seed(5)
    for chunks, rows in ((16, 256), (5, 200)):
        ck = k.CudaKernels()
        out, n_in = 384, 264
        g = torch.randn(out, n_in, device="cuda")
        ref = g.clone()
        g3 = torch.zeros(48, 8, 72, device="cuda")           # batched (per-head) gradient view
        ref3 = g3.clone()
        for c in range(chunks):
            dy = torch.randn(rows, out, device="cuda", dtype=torch.bfloat16)
            x = torch.randn(rows, n_in, device="cuda", dtype=torch.bfloat16)
            ck.linear_wgrad(dy, x, g)
            ref += dy.float().t() @ x.float()
            dyh = torch.randn(rows, 8, 48, device="cuda", dtype=torch.bfloat16)
            xh = torch.randn(rows, 8, 72, device="cuda", dtype=torch.bfloat16)
            ck._wgrad(dyh, xh, g3, 48, 72, 8)
            ref3 += torch.einsum("rhm,rhn->mhn", dyh.float(), xh.float())
        if chunks == 16:
            assert not ck._wq                                  # a full group left by itself
        ck.flush_wgrads()
        k.check_status(g.device)
        assert not ck.fallbacks and not ck._wq
        assert _rel(g, ref) < 1e-2 and _rel(g3, ref3) < 1e-2


@pytest.mark.parametrize("qh,kvh,hd,B,Tc,T,s", [(8, 2, 96, 4, 128, 384, 128), (15, 5, 64, 3, 100, 300, 200), (4, 2, 128, 2, 192, 192, 0),
                                               (8, 2, 96, 16, 128, 2048, 1920)])
def test_qkv_projection_with_rope_epilogue(qh, kvh, hd, B, Tc, T, s, monkeypatch):
    """The [Q | K | V] projection whose epilogue rotates Q and K and writes the attention operand and the caches, against
    the projection followed by the PyTorch statement of RoPE + cache write.  Rows of the caches outside [s, s+Tc) and
    the other two sectors of the operand buffer must stay untouched."""
    from types import SimpleNamespace
    from loomformer_paraplex_b200.ops.twins import TorchKernels
    monkeypatch.setenv("LOOM_QKV_ROPE", "1")
    k = _k()
    torch.manual_seed(9)
    n, kv = qh * hd, kvh * hd
    d = SimpleNamespace(qh=qh, kvh=kvh, hd=hd, n=n, kv_dim=kv)
    M, K_in = B * Tc, 256
    x = torch.randn(M, K_in, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(n + 2 * kv, K_in, device="cuda") * 0.06).to(torch.bfloat16)
    cos, sin = torch.randn(B, Tc, hd, device="cuda"), torch.randn(B, Tc, hd, device="cuda")
    ck, tk = k.CudaKernels(), TorchKernels()
    qkc1 = torch.full((M, 3, qh, hd), 7.0, device="cuda", dtype=torch.bfloat16)
    kc1 = torch.full((B, T, kvh, hd), 5.0, device="cuda", dtype=torch.bfloat16)
    vc1 = torch.full((B, T, kvh, hd), 3.0, device="cuda", dtype=torch.bfloat16)
    before = k.native.launches() if hasattr(k.native, "launches") else None
    ck.qkv_rope(d, x, w, cos, sin, qkc1, kc1, vc1, s)
    k.check_status(x.device)
    assert not ck.fallbacks, ck.fallbacks
    if before is not None:
        assert k.native.launches() - before == 1            # one launch: the fused path ran
    qkc2, kc2, vc2 = torch.full_like(qkc1, 7.0).float(), torch.full_like(kc1, 5.0).float(), torch.full_like(vc1, 3.0).float()
    tk.qkv_rope(d, x.float(), w.float(), cos, sin, qkc2, kc2, vc2, s)
    assert _rel(qkc1[:, 0], qkc2[:, 0]) < 1.5e-2
    assert _rel(kc1[:, s:s + Tc], kc2[:, s:s + Tc]) < 1.5e-2 and _rel(vc1[:, s:s + Tc], vc2[:, s:s + Tc]) < 1.5e-2
    assert bool((qkc1[:, 1:] == 7.0).all())
    keep = torch.ones(T, dtype=torch.bool, device="cuda"); keep[s:s + Tc] = False
    assert bool((kc1[:, keep] == 5.0).all()) and bool((vc1[:, keep] == 3.0).all())


@pytest.mark.parametrize("M,N,K", [(2048, 1152, 768), (520, 200, 136), (256, 1600, 960)])
def test_pair_tiles_192_wide(M, N, K):
    k = _k()
    torch.manual_seed(10)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(N, device="cuda")
    c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    k.gemm([x], [K], w, c, M=M, N=N, bias=bias, bn=192, pair=1)
    k.check_status(c.device)
    assert _rel(c, x.float() @ w.float().t() + bias) < 1e-2
