"""PyTorch twins of the grouped small-batch products and of the fused QKV + RoPE launch: the CPU statements that the
CUDA kernels are tested against must themselves equal the plain composition of the ops they stand for."""
from types import SimpleNamespace

import torch
import torch.nn.functional as F

from loomformer_paraplex_b200.ops import reference as R
from loomformer_paraplex_b200.ops.twins import TorchKernels


def test_linear_multi_twin_equals_separate_linears():
    torch.manual_seed(0)
    tk = TorchKernels()
    M = 3
    x1, x2 = torch.randn(M, 16), torch.randn(M, 2, 8)
    w1, w2 = torch.randn(5, 16), torch.randn(7, 16 + 8)
    b2 = torch.randn(7)
    y1 = torch.empty(M, 5)
    wide = torch.full((M, 9), 3.0)
    tk.linear_multi([([x1], w1, None, y1), ([x1, x2[:, 1]], w2, b2, wide[:, :7])], static_weights=True)
    assert torch.allclose(y1, F.linear(x1, w1), atol=1e-6)
    assert torch.allclose(wide[:, :7], F.linear(torch.cat((x1, x2[:, 1]), -1), w2, b2), atol=1e-6)
    assert bool((wide[:, 7:] == 3.0).all())


def test_qkv_rope_twin_equals_projection_then_rope_store():
    torch.manual_seed(1)
    tk = TorchKernels()
    qh, kvh, hd, B, Tc, T, s = 4, 2, 8, 2, 5, 12, 3
    n, kv = qh * hd, kvh * hd
    d = SimpleNamespace(qh=qh, kvh=kvh, hd=hd, n=n, kv_dim=kv)
    x, w = torch.randn(B * Tc, 12), torch.randn(n + 2 * kv, 12)
    cos, sin = torch.randn(B, Tc, hd), torch.randn(B, Tc, hd)
    qkc, kc, vc = torch.zeros(B * Tc, 3, qh, hd), torch.zeros(B, T, kvh, hd), torch.zeros(B, T, kvh, hd)
    tk.qkv_rope(d, x, w, cos, sin, qkc, kc, vc, s)
    qkv = F.linear(x, w).view(B, Tc, -1)
    q, k, v = qkv.split((n, kv, kv), -1)
    c, s_ = cos.unsqueeze(2), sin.unsqueeze(2)
    assert torch.allclose(qkc.view(B, Tc, 3, qh, hd)[:, :, 0], R.apply_rope(q.view(B, Tc, qh, hd), c, s_), atol=1e-6)
    assert torch.allclose(kc[:, s:s + Tc], R.apply_rope(k.view(B, Tc, kvh, hd), c, s_), atol=1e-6)
    assert torch.allclose(vc[:, s:s + Tc], v.view(B, Tc, kvh, hd), atol=1e-6)
    assert float(kc[:, :s].abs().sum()) == 0.0 and float(qkc[:, 1:].abs().sum()) == 0.0
