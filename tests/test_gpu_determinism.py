"""Race and overrun detection without a sanitizer: kernels documented as free of atomics must give bit-identical
output when repeated, and kernels that write a caller's buffer must leave guard rows on both sides of it untouched."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _K():
    from loomformer_paraplex_b200.ops import kernels
    return kernels, kernels.CudaKernels()


def _dims():
    from loomformer_paraplex_b200.ops.microbench import dims
    return dims()


def bf(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


def _guarded(rows, cols, dtype=torch.bfloat16, guard=8):
    """A [rows, cols] view in the middle of a buffer whose first and last `guard` rows are NaN canaries."""
    buf = torch.full((rows + 2 * guard, cols), float("nan"), device="cuda", dtype=dtype)
    return buf, buf[guard:guard + rows]


def _canaries_intact(buf, rows, guard=8):
    return bool(torch.isnan(buf[:guard]).all()) and bool(torch.isnan(buf[guard + rows:]).all())


@pytest.mark.parametrize("pair", [0, 1])
@pytest.mark.parametrize("M,N,K", [(300, 200, 136), (2048, 768, 768)])
def test_gemm_writes_only_its_output_and_repeats_bit_exactly(M, N, K, pair):
    kernels, _ = _K()
    torch.manual_seed(0)
    x, w = bf(M, K), bf(N, K, scale=0.05)
    outs = []
    for _ in range(3):
        buf, c = _guarded(M, N)
        kernels.gemm([x], [K], w, c, M=M, N=N, bn=128, pair=pair)
        torch.cuda.synchronize()
        assert _canaries_intact(buf, M)
        assert bool(torch.isfinite(c.float()).all())
        outs.append(c.clone())
    kernels.check_status(x.device)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])


def test_attention_backward_slabs_are_deterministic():
    """dK / dV come out of per-head slabs summed in a fixed order: three runs, identical bits."""
    kernels, K = _K()
    from loomformer_paraplex_b200.ops.microbench import _attn_inputs
    torch.manual_seed(1)
    d, B, s, kc, vc, qkc = _attn_inputs(1024, 128, 512)
    lse = K.attn_fwd(d, qkc, kc, vc, s, 512, None)
    dqkc = bf(1024, 3, d.qh, d.hd, scale=0.3)
    res = []
    for _ in range(3):
        dk, dv = K.alloc_kv_grad(d, B, 512, qkc.device), K.alloc_kv_grad(d, B, 512, qkc.device)
        dq = K.attn_bwd(d, dqkc, qkc, kc, vc, lse, s, 512, None, dk, dv)
        torch.cuda.synchronize()
        res.append((dk.clone(), dv.clone(), None if dq is None else dq.clone()))
    kernels.check_status(qkc.device)
    for a, b in zip(res[0], res[1]):
        assert a is None or torch.equal(a, b)
    for a, b in zip(res[0], res[2]):
        assert a is None or torch.equal(a, b)


def test_attention_forward_is_deterministic():
    kernels, K = _K()
    from loomformer_paraplex_b200.ops.microbench import _attn_inputs
    torch.manual_seed(2)
    d, B, s, kc, vc, qkc = _attn_inputs(1024, 128, 512)
    outs = []
    for _ in range(3):
        q = qkc.clone()
        lse = K.attn_fwd(d, q, kc, vc, s, 512, None)
        torch.cuda.synchronize()
        outs.append((q, lse.clone()))
    kernels.check_status(qkc.device)
    assert all(torch.equal(outs[0][0], o[0]) and torch.equal(outs[0][1], o[1]) for o in outs[1:])


def test_depth_read_slot_backward_is_deterministic():
    kernels, K = _K()
    d = _dims()
    torch.manual_seed(3)
    S, M, slot = 8, 1024, 2
    hist = bf(S, M, 2, d.qh, d.hd)
    hk, hv = hist[:, :, 0], hist[:, :, 1]
    q_all = torch.randn(S, d.qh, d.hd, device="cuda")
    dm, lse, dd = bf(S, M, d.qh, d.hd, scale=0.3), torch.randn(S, M, d.qh, device="cuda") + 3, torch.randn(S, M, d.qh, device="cuda")
    outs = []
    for _ in range(3):
        gq = torch.zeros(S, d.qh, d.hd, device="cuda")
        outs.append(K.dread_slot_bwd(d, slot, q_all, hk, hv, dm, lse, dd, gq).clone())
    kernels.check_status(hist.device)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])


def test_add_layernorm_round_trip_is_deterministic():
    """Forward and the data gradient of add + LayerNorm repeat bit-exactly (the parameter gradients go through
    atomics and are excluded)."""
    kernels, K = _K()
    torch.manual_seed(4)
    M, N = 2048, 768
    a, b = bf(M, N), bf(M, N)
    w, bias = torch.randn(N, device="cuda"), torch.randn(N, device="cuda")
    outs = []
    for _ in range(3):
        r = K.add_ln_fwd(a, b, w, bias, None)
        outs.append(tuple(t.clone() for t in r if torch.is_tensor(t)))
    kernels.check_status(a.device)
    for o in outs[1:]:
        assert all(torch.equal(x, y) for x, y in zip(outs[0], o))
