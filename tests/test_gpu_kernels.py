"""Each native bandwidth-bound kernel against its PyTorch twin evaluated in fp32 on the same bf16 inputs."""
from types import SimpleNamespace

import pytest
import torch

pytestmark = pytest.mark.gpu


def _sets():
    from loomformer_paraplex_b200.ops.kernels import CudaKernels
    from loomformer_paraplex_b200.ops.twins import TorchKernels
    return CudaKernels(), TorchKernels()


def _close(a, b, tol=2e-2, name=""):
    a, b = a.float(), b.float()
    err = float((a - b).abs().max())
    ref = float(b.abs().max()) + 1e-6
    assert err <= tol * ref + 1e-5, (name, err, ref)


def _dims(qh=8, hd=96, kvh=2, hidden=3072, **kw):
    base = dict(qh=qh, hd=hd, kvh=kvh, group=qh // kvh, n=qh * hd, kv_dim=kvh * hd, hidden=hidden, hpq=hidden // qh,
                activation="pvpowlu", powlu_m=3.0, phase_floor=0.05, phase_secant=True)
    base.update(kw)
    return SimpleNamespace(**base)


def bf(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


@pytest.mark.parametrize("hd", [32, 96])
def test_rope_store_and_bwd(hd):
    ck, tk = _sets()
    d = _dims(hd=hd)
    B, Tc, T, s = 3, 40, 100, 24
    torch.manual_seed(0)
    qkv = bf(B, Tc, d.n + 2 * d.kv_dim)
    ang = torch.rand(B, Tc, hd // 2, device="cuda") * 6
    cos, sin = torch.cat((ang.cos(), ang.cos()), -1) * 1.1, torch.cat((ang.sin(), ang.sin()), -1) * 1.1
    outs = []
    for k in (ck, tk):
        qkc = torch.zeros(B * Tc, 3, d.qh, hd, device="cuda", dtype=torch.bfloat16)
        kc = torch.zeros(B, T, d.kvh, hd, device="cuda", dtype=torch.bfloat16)
        vc = torch.zeros_like(kc)
        k.rope_store(d, qkv, cos, sin, qkc, kc, vc, s)
        outs.append((qkc, kc, vc))
    for x, y in zip(*outs):
        _close(x, y, 1e-2)
    dq = bf(B, Tc, d.qh, hd); dqkc = bf(B * Tc, 3, d.qh, hd)
    dkc, dvc = torch.randn(B, T, d.kvh, hd, device="cuda"), torch.randn(B, T, d.kvh, hd, device="cuda")
    a = ck.rope_bwd(d, dq, dqkc, dkc, dvc, s, s + Tc, cos, sin, torch.bfloat16)
    b = tk.rope_bwd(d, dq, dqkc, dkc, dvc, s, s + Tc, cos, sin, torch.float32)
    _close(a, b, 1e-2)


@pytest.mark.parametrize("hd,qh", [(32, 4), (64, 15), (96, 8), (128, 2), (48, 4), (24, 6), (40, 2)])
def test_depth_read(hd, qh):
    ck, tk = _sets()
    d = _dims(qh=qh, hd=hd, kvh=1)
    S, M, n = 7, 333, 5
    torch.manual_seed(1)
    hk, hv = bf(S, M, qh, hd), bf(S, M, qh, hd)
    q = torch.randn(qh, hd, device="cuda")
    m1, l1 = ck.dread_fwd(d, q, hk, hv, n)
    m2, l2 = tk.dread_fwd(d, q, hk.float(), hv.float(), n)
    _close(m1, m2); _close(l1, l2, 1e-3)
    dm = bf(M, qh, hd)
    g1 = [torch.randn(S, M, qh, hd, device="cuda") for _ in range(2)] + [torch.zeros(qh, hd, device="cuda")]
    g2 = [x.clone() for x in g1]
    ck.dread_bwd(d, dm, m1, l1, q, hk, hv, n, *g1)
    tk.dread_bwd(d, dm.float(), m1.float(), l1, q, hk.float(), hv.float(), n, *g2)
    for x, y, nm in zip(g1, g2, ("dk", "dv", "gq")):
        _close(x, y, 2e-2, nm)
    # K and V interleaved as [K | V] rows of one buffer (the layout the training plan keeps)
    both = torch.stack((hk, hv), 2).contiguous()
    m3, l3 = ck.dread_fwd(d, q, both[:, :, 0], both[:, :, 1], n)
    _close(m3, m2); _close(l3, l2, 1e-3)
    assert not ck.fallbacks, ck.fallbacks


@pytest.mark.parametrize("N", [128, 768, 960])
def test_add_layernorm(N):
    ck, tk = _sets()
    M = 517
    torch.manual_seed(2)
    a, b = bf(M, N), bf(M, N)
    w, bias = torch.randn(N, device="cuda"), torch.randn(N, device="cuda")
    y1, x1, mu1, rs1 = ck.add_ln_fwd(a, b, w, bias, None)
    y2, x2, mu2, rs2 = tk.add_ln_fwd(a, b, w, bias, None)
    _close(y1, y2, 1e-2); _close(mu1, mu2, 1e-3); _close(rs1, rs2, 1e-3)
    dy = bf(M, N)
    gw1, gb1, gw2, gb2 = (torch.zeros(N, device="cuda") for _ in range(4))
    d1, _ = ck.add_ln_bwd(dy, x1, mu1, rs1, w, gw1, gb1, None, None, None)
    d2, _ = tk.add_ln_bwd(dy.float(), x1.float(), mu1, rs1, w, gw2, gb2, None, None, None)
    _close(d1, d2, 1e-2); _close(gw1, gw2, 1e-3); _close(gb1, gb2, 1e-3)
    g1, g2 = torch.zeros(N, device="cuda"), torch.zeros(N, device="cuda")
    ck.colsum_add(dy, g1); tk.colsum_add(dy, g2)
    _close(g1, g2, 1e-3)
    assert not ck.fallbacks, ck.fallbacks


@pytest.mark.parametrize("N", [128, 768, 960, 2048])
@pytest.mark.parametrize("cap", [None, 1.0])
def test_add_layernorm_few_rows(N, cap):
    """Up to 64 rows (a decode step) take the block-per-row kernel: same numbers as the PyTorch statement, with and
    without the RMS cap on the addends."""
    ck, tk = _sets()
    torch.manual_seed(22)
    for M in (1, 5, 64):
        a, b = bf(M, N, scale=2.0), bf(M, N, scale=0.5)
        w, bias = torch.rand(N, device="cuda") + 0.5, torch.randn(N, device="cuda") * 0.1
        y1, x1, mu1, rs1 = ck.add_ln_fwd(a, b, w, bias, cap)
        y2, x2, mu2, rs2 = tk.add_ln_fwd(a.float(), b.float(), w, bias, cap)
        _close(y1, y2, 2e-2, "y"); _close(x1, x2, 1e-2, "x"); _close(mu1, mu2, 1e-2, "mean"); _close(rs1, rs2, 1e-2, "rstd")
    assert not ck.fallbacks, ck.fallbacks


def test_cross_entropy():
    ck, tk = _sets()
    torch.manual_seed(3)
    M, V = 300, 8192
    logits = bf(M, V, scale=3.0)
    tgt = torch.randint(0, V, (M,), device="cuda")
    tgt[:17] = -100
    l2, g2 = tk.ce_fwd_bwd(logits.float(), tgt, -100, 0.5)
    l1, g1 = ck.ce_fwd_bwd(logits.clone(), tgt, -100, 0.5)
    assert abs(float(l1) - float(l2)) < 2e-3
    _close(g1, g2, 1e-2)
    # small vocabulary, many rows: every thread's first (and only) column group is written back right after the second
    # reduction, so a loss formed from the row after that point would pick up gradient values instead of logits
    M, V = 8192, 512
    logits = bf(M, V, scale=3.0)
    tgt = torch.randint(0, V, (M,), device="cuda")
    ref = torch.nn.functional.cross_entropy(logits.float(), tgt)
    for _ in range(3):
        l1, _ = ck.ce_fwd_bwd(logits.clone(), tgt, -100, 1.0)
        assert abs(float(l1) - float(ref)) < 2e-5 * float(ref), (float(l1), float(ref))


def _core_case(ck, tk, d, B, Tc, *, p_in, c_prev, seed, gate_lin, gate_w, trace, reset, axis):
    M, H = B * Tc, d.hidden
    x_real, beta_lin = bf(M, H), bf(M, H, scale=1.5)
    pin = bf(M, H, scale=0.5) if p_in else None
    glin = bf(M, H) if gate_lin else None
    alpha = torch.tensor(0.17, device="cuda")
    b_real, b_imag, w_tr = (torch.randn(H, device="cuda") * 0.3 for _ in range(3))
    tr_in = torch.rand(B, H, device="cuda") * 2 - 1 if trace else None
    rs = (torch.rand(M, device="cuda") < 0.05) if reset else None
    cp_t = torch.randn(M, H, 9, device="cuda").to(torch.bfloat16) if c_prev else None
    sd = torch.randn(B, H, 9, device="cuda") if seed else None
    sv = (torch.rand(B, device="cuda") < 0.6) if seed else None
    gw = torch.softmax(torch.randn(9, device="cuda"), 0) if gate_w else None
    anchor = torch.tensor(0.8, device="cuda") if d.phase_secant else None
    planes = lambda t: None if t is None else t.permute(2, 0, 1).contiguous()
    o1 = ck.ffn_core_fwd(d, x_real, pin, alpha, b_real, glin, beta_lin, b_imag, w_tr, tr_in, rs, None, planes(cp_t),
                         sd, sv, gw, axis, 0.05, B)
    f = lambda t: None if t is None else t.float()
    o2 = tk.ffn_core_fwd(d, f(x_real), f(pin), alpha, b_real, f(glin), f(beta_lin), b_imag, w_tr, tr_in, rs, None,
                         f(cp_t), sd, sv, gw, axis, 0.05, B)
    _close(o1["o"], o2["o"], 2e-2, "o"); _close(o1["trace_out"], o2["trace_out"], 1e-3, "trace")
    assert abs(float(o1["beta_sq_sum"]) / float(o2["beta_sq_sum"]) - 1) < 1e-3
    if axis is not None:
        _close(o1["c"].permute(1, 2, 0), o2["c"], 2e-2, "c")
        if gw is not None:
            _close(o1["p_out"], o2["p_out"], 2e-2, "p_out")
    # backward
    do = bf(M, H, scale=0.1)
    dc_t = (torch.randn(M, H, 9, device="cuda") * 0.1).to(torch.bfloat16) if axis is not None else None
    dpo = bf(M, H, scale=0.1) if (axis is not None and gw is not None) else None
    dtr = torch.randn(B, H, device="cuda") * 0.1
    saved = {"x_real": x_real, "p_in": pin, "alpha_gate": alpha, "b_real": b_real, "gate_lin": glin, "beta_lin": beta_lin,
             "b_imag": b_imag, "w_trace": w_tr, "trace_in": tr_in, "reset": rs, "anchor": anchor, "c_prev": planes(cp_t),
             "seed": sd, "seed_valid": sv, "gate_w": gw, "axis": axis, "tria_alpha": 0.05, "B": B,
             "g_b_real": torch.zeros(H, device="cuda"), "g_b_imag": torch.zeros(H, device="cuda"),
             "g_w_trace": torch.zeros(H, device="cuda")}
    g1 = ck.ffn_core_bwd(d, saved, do, planes(dc_t), dpo, dtr)
    saved2 = dict(saved, c_prev=cp_t)
    g2 = tk.ffn_core_bwd(d, saved2, do, dc_t, dpo, dtr)
    for k in ("d_x_real", "d_p_in", "d_gate_lin", "d_beta_lin", "d_trace_in", "d_seed"):
        if g2.get(k) is not None:
            _close(g1[k], g2[k], 3e-2, k)
    if cp_t is not None:
        _close(g1["d_c_prev"].permute(1, 2, 0), g2["d_c_prev"], 3e-2, "d_c_prev")
    _close(saved["g_b_real"], g2["d_b_real"], 2e-2, "g_b_real")
    _close(saved["g_b_imag"], g2["d_b_imag"], 2e-2, "g_b_imag")
    _close(saved["g_w_trace"], g2["d_w_trace"], 2e-2, "g_w_trace")
    if pin is not None:
        assert abs(float(g1["d_alpha_gate"]) - float(g2["d_alpha_gate"])) <= 2e-2 * abs(float(g2["d_alpha_gate"])) + 1e-2
    if gw is not None and axis is not None:
        _close(g1["d_gate_w"], g2["d_gate_w"], 2e-2, "d_gate_w")


@pytest.mark.parametrize("secant", [True, False])
def test_ffn_core_variants(secant):
    ck, tk = _sets()
    d = _dims(hidden=256, phase_secant=secant)
    torch.manual_seed(4)
    _core_case(ck, tk, d, 3, 20, p_in=False, c_prev=False, seed=False, gate_lin=False, gate_w=True, trace=False, reset=False, axis=0)
    _core_case(ck, tk, d, 3, 20, p_in=True, c_prev=True, seed=False, gate_lin=False, gate_w=True, trace=True, reset=True, axis=1)
    _core_case(ck, tk, d, 3, 20, p_in=False, c_prev=False, seed=True, gate_lin=True, gate_w=True, trace=True, reset=True, axis=0)
    _core_case(ck, tk, d, 3, 20, p_in=True, c_prev=True, seed=False, gate_lin=True, gate_w=False, trace=True, reset=False, axis=2)
    _core_case(ck, tk, d, 2, 16, p_in=False, c_prev=False, seed=False, gate_lin=False, gate_w=False, trace=True, reset=True, axis=None)
    assert not ck.fallbacks, ck.fallbacks


@pytest.mark.parametrize("Tc", [128, 70])
def test_temporal_endpoint(Tc):
    ck, tk = _sets()
    torch.manual_seed(5)
    B, H = 3, 64
    from loomformer_paraplex_b200.ops import reference as R
    carr = None                      # realistic carriers: a depth chain of near-orthogonal Tria operators
    for layer in range(4):
        r, i, o = (torch.randn(B, Tc, H, device="cuda") for _ in range(3))
        carr, _ = R.tria_compose(r, i, o, 0.05, layer % 3, prev=carr)
    depth_t = carr.reshape(B * Tc, H, 9).to(torch.bfloat16)
    reset = torch.rand(B, Tc, device="cuda") < 0.02
    state = R.normalize9(torch.eye(3, device="cuda").reshape(1, 1, 3, 3) + 0.05 * torch.randn(B, H, 3, 3, device="cuda")).reshape(B, H, 9)
    fired = torch.tensor([True, False, True], device="cuda")
    planes = depth_t.permute(2, 0, 1).contiguous()
    for st, fr in ((state, fired), (None, None)):
        s1, aux = ck.temporal_fwd(planes, B, Tc, H, reset, st, fr, 0.1)
        s2, _ = tk.temporal_fwd(depth_t.float(), B, Tc, H, reset, st, fr, 0.1)
        _close(s1, s2, 2e-3, "state")
        g = torch.randn(B, H, 9, device="cuda")
        d1, p1 = ck.temporal_bwd(g, planes, B, Tc, H, reset, st, fr, 0.1, aux)
        d2, p2 = tk.temporal_bwd(g, depth_t.float(), B, Tc, H, reset, st, fr, 0.1, None)
        _close(d1.permute(1, 2, 0), d2, 3e-2, "ddepth")
        if st is not None:
            _close(p1, p2, 3e-2, "dstate_in")


# the last three: windows wider than one 128-row query tile (cfg/alt.yaml 192, cfg/mini.yaml 256), head dim 24
# (cfg/alt2.yaml) and a whole 512-token sequence as one chunk (the unchunked forward)
@pytest.mark.parametrize("hd,qh,kvh,Tc,s", [(96, 8, 2, 128, 256), (64, 4, 2, 128, 0), (32, 4, 4, 100, 128), (96, 8, 2, 40, 88),
                                            (96, 8, 2, 192, 192), (24, 4, 2, 256, 0), (64, 4, 2, 512, 0)])
def test_attention_forward(hd, qh, kvh, Tc, s):
    from loomformer_paraplex_b200.ops import kernels
    ck, tk = _sets()
    d = _dims(qh=qh, hd=hd, kvh=kvh)
    B, T = 3, 512
    e = s + Tc
    torch.manual_seed(6)
    kc, vc = bf(B, T, kvh, hd), bf(B, T, kvh, hd)
    kc[:, e:] = 0; vc[:, e:] = 0
    q = bf(B * Tc, qh, hd)
    for seg in (None, (torch.arange(T, device="cuda") // 150).view(1, T).expand(B, T).contiguous()):
        qkc1 = torch.zeros(B * Tc, 3, qh, hd, device="cuda", dtype=torch.bfloat16); qkc1[:, 0] = q
        qkc2 = qkc1.float()
        l1 = ck.attn_fwd(d, qkc1, kc, vc, s, e, seg)
        l2 = tk.attn_fwd(d, qkc2, kc.float(), vc.float(), s, e, seg)
        kernels.check_status(torch.device("cuda"))
        assert not ck.fallbacks, ck.fallbacks
        _close(l1, l2, 2e-3, "lse")
        _close(qkc1[:, 1], qkc2[:, 1], 2e-2, "kctx")
        _close(qkc1[:, 2], qkc2[:, 2], 2e-2, "ctx")


# the last three: windows wider than one 128-row query tile (cfg/alt.yaml 192, cfg/mini.yaml 256), head dim 24
# (cfg/alt2.yaml) and a whole 512-token sequence as one chunk (the unchunked forward)
@pytest.mark.parametrize("hd,qh,kvh,Tc,s", [(96, 8, 2, 128, 256), (64, 4, 2, 128, 0), (32, 4, 4, 100, 128), (96, 8, 2, 40, 88),
                                            (96, 8, 2, 192, 192), (24, 4, 2, 256, 0), (64, 4, 2, 512, 0)])
def test_attention_backward(hd, qh, kvh, Tc, s):
    from loomformer_paraplex_b200.ops import kernels
    ck, tk = _sets()
    d = _dims(qh=qh, hd=hd, kvh=kvh)
    B, T = 2, 512
    e = s + Tc
    torch.manual_seed(7)
    kc, vc = bf(B, T, kvh, hd), bf(B, T, kvh, hd)
    kc[:, e:] = 0; vc[:, e:] = 0
    seg = (torch.arange(T, device="cuda") // 170).view(1, T).expand(B, T).contiguous()
    qkc = torch.zeros(B * Tc, 3, qh, hd, device="cuda", dtype=torch.bfloat16); qkc[:, 0] = bf(B * Tc, qh, hd)
    lse = ck.attn_fwd(d, qkc, kc, vc, s, e, seg)
    dqkc = bf(B * Tc, 3, qh, hd, scale=0.3)
    dk1, dv1 = ck.alloc_kv_grad(d, B, T, qkc.device), ck.alloc_kv_grad(d, B, T, qkc.device)
    dk1 += 1.0                                  # accumulation must preserve what is already there
    dq1 = ck.attn_bwd(d, dqkc, qkc, kc, vc, lse, s, e, seg, dk1, dv1)
    kernels.check_status(torch.device("cuda"))
    assert not ck.fallbacks, ck.fallbacks
    dk2, dv2 = tk.alloc_kv_grad(d, B, T, qkc.device), tk.alloc_kv_grad(d, B, T, qkc.device)
    dq2 = tk.attn_bwd(d, dqkc.float(), qkc.float(), kc.float(), vc.float(), lse, s, e, seg, dk2, dv2)
    _close(dq1, dq2.reshape(dq1.shape), 3e-2, "dq")
    g = qh // kvh
    _close((dk1 - 1.0).view(B, T, kvh, g, hd).sum(3), dk2, 3e-2, "dk")
    _close(dv1.view(B, T, kvh, g, hd).sum(3), dv2, 3e-2, "dv")


@pytest.mark.parametrize("hd,qh,S", [(96, 8, 6), (32, 4, 6), (64, 3, 65), (96, 8, 20), (64, 15, 20), (128, 2, 8), (48, 4, 6), (24, 6, 9),
                                     (40, 2, 5)])
def test_depth_read_backward_per_slot(hd, qh, S):
    """Staged per-slot backward equals the sum of per-sublayer contributions evaluated in fp32 (S=65 is the 32-layer
    stack, which takes the 20-pairs-per-thread instantiation of the 8-dims-per-lane kernel; head widths 96 / 64 / 128 /
    48 / 32 / 24 take the kernel whose lanes own 12, 8 or 16 dims; 40 has no such split)."""
    ck, tk = _sets()
    d = _dims(qh=qh, hd=hd, kvh=qh)
    M = 200
    torch.manual_seed(9)
    hk, hv = bf(S, M, qh, hd), bf(S, M, qh, hd)
    if S == 65:                                  # interleaved [K | V] rows, as the training plan stores them
        both = torch.stack((hk, hv), 2).contiguous()
        hk, hv = both[:, :, 0], both[:, :, 1]
    q_all = torch.randn(S, qh, hd, device="cuda")
    mk = lambda dt: {"q": q_all, "dm": torch.zeros(S, M, qh, hd, dtype=dt, device="cuda"),
                     "lse": torch.zeros(S, M, qh, device="cuda"), "dd": torch.zeros(S, M, qh, device="cuda"),
                     "gq": torch.zeros(S, qh, hd, device="cuda")}
    d1, d2 = mk(torch.bfloat16), mk(torch.float32)
    for sub in range(S):
        m_out, lse = tk.dread_fwd(d, q_all[sub], hk.float(), hv.float(), sub + 1)
        a, b = bf(M, qh, hd, scale=0.3), (bf(M, qh, hd, scale=0.3) if sub % 2 else None)
        ck.dread_stage(d, a, b, m_out.to(torch.bfloat16), lse, d1, sub)
        tk.dread_stage(d, a.float(), None if b is None else b.float(), m_out.to(torch.bfloat16).float(), lse, d2, sub)
    _close(d1["dm"], d2["dm"], 1e-2, "dm"); _close(d1["dd"], d2["dd"], 2e-2, "dd"); _close(d1["lse"], d2["lse"], 1e-5, "lse")
    for slot in (0, 3, S - 1):
        kv1 = ck.dread_slot_bwd(d, slot, q_all, hk, hv, d1["dm"], d1["lse"], d1["dd"], d1["gq"])
        kv2 = tk.dread_slot_bwd(d, slot, q_all, hk.float(), hv.float(), d2["dm"], d2["lse"], d2["dd"], d2["gq"])
        _close(kv1[:, 0], kv2[:, 0], 2e-2, "dk"); _close(kv1[:, 1], kv2[:, 1], 2e-2, "dv")
    _close(d1["gq"], d2["gq"], 2e-2, "gq")
    assert not ck.fallbacks, ck.fallbacks


def test_slot_pool_forward_backward():
    ck, tk = _sets()
    torch.manual_seed(11)
    B, Kn, H = 3, 5, 700
    keys = torch.randn(B, Kn, H, 9, device="cuda")
    w9 = torch.randn(9, device="cuda") * 2
    p1, p2 = ck.slot_pool_fwd(keys, w9), tk.slot_pool_fwd(keys, w9)
    _close(p1, p2, 1e-4, "pooled")
    dp = torch.randn(B, Kn, 9, device="cuda")
    (dk1, dw1), (dk2, dw2) = ck.slot_pool_bwd(dp, keys, w9), tk.slot_pool_bwd(dp, keys, w9)
    _close(dk1, dk2, 1e-3, "dkeys"); _close(dw1, dw2, 1e-3, "dw9")
    assert not ck.fallbacks, ck.fallbacks


@pytest.mark.parametrize("N,Kn,T", [(768, 16, 256), (256, 3, 100), (1024, 40, 64)])
def test_sparse_cross_attention(N, Kn, T):
    ck, tk = _sets()
    torch.manual_seed(12)
    B = 2
    q, k, v = bf(B, T, N, scale=0.3), bf(B, Kn, N, scale=0.3), bf(B, Kn, N)
    key_pos = torch.sort(torch.randperm(T, device="cuda")[:Kn]).values
    allowed = key_pos.view(1, 1, Kn) <= torch.arange(T, device="cuda").view(1, T, 1)
    allowed = allowed & (torch.rand(B, 1, Kn, device="cuda") < 0.8)
    scale = N ** -0.5
    o1 = ck.cross_attn_fwd(q, k, v, allowed, scale)
    o2 = tk.cross_attn_fwd(q.float(), k.float(), v.float(), allowed, scale)
    _close(o1, o2, 2e-2, "out")
    none = ~allowed.any(-1)
    assert bool(none.any()) and float(o1[none].abs().max()) == 0.0        # rows without a key give exactly zero
    dout = bf(B, T, N, scale=0.2)
    g1 = ck.cross_attn_bwd(dout, q, k, v, allowed, scale)
    g2 = tk.cross_attn_bwd(dout.float(), q.float(), k.float(), v.float(), allowed, scale)
    for a, b_, nm in zip(g1, g2, ("dq", "dk", "dv")):
        _close(a, b_, 3e-2, nm)
    assert not ck.fallbacks, ck.fallbacks


def test_rms_type_norms():
    ck, tk = _sets()
    torch.manual_seed(13)
    M, qh, hd = 300, 8, 96
    kv = bf(M, 2 * qh * hd)
    xv = kv[:, qh * hd:].view(M, qh, hd)                       # strided view, as the depth K/V projection produces it
    y1, y2 = ck.fixed_rms_fwd(xv, 0.88), tk.fixed_rms_fwd(xv.float(), 0.88)
    _close(y1, y2, 1e-2, "fixed_rms")
    dy = bf(M, qh, hd, scale=0.3)
    _close(ck.fixed_rms_bwd(dy, xv, 0.88), tk.fixed_rms_bwd(dy.float(), xv.float(), 0.88), 2e-2, "fixed_rms_bwd")
    x, w = bf(M, 768), torch.rand(768, device="cuda") + 0.5
    _close(ck.rms_norm_fwd(x, w), tk.rms_norm_fwd(x.float(), w), 1e-2, "rms_norm")
    g = bf(M, 768, scale=0.3)
    gw1, gw2 = torch.zeros(768, device="cuda"), torch.zeros(768, device="cuda")
    _close(ck.rms_norm_bwd(g, x, w, gw1), tk.rms_norm_bwd(g.float(), x.float(), w, gw2), 2e-2, "rms_norm_bwd")
    _close(gw1, gw2, 2e-2, "rms_norm_gw")
    assert not ck.fallbacks, ck.fallbacks


@pytest.mark.parametrize("B,S,pos,ns,qh,kvh,hd", [(1, 700, 650, 16, 8, 2, 96), (5, 300, 299, 3, 8, 2, 96), (3, 128, 0, 1, 8, 2, 96),
                                                   (2, 2048, 1500, 1, 8, 2, 96), (1, 769, 30, 32, 8, 2, 96),
                                                   (2, 400, 333, 5, 15, 5, 64), (3, 200, 150, 4, 16, 2, 128), (2, 90, 77, 2, 4, 4, 24),
                                                   (1, 769, 768, 7, 8, 2, 96), (64, 769, 600, 7, 8, 2, 96), (3, 100, 99, 1, 8, 2, 96),
                                                   (2, 128, 127, 1, 15, 5, 64), (2, 1000, 5, 8, 16, 2, 128)])
def test_decode_attention_kernel(B, S, pos, ns, qh, kvh, hd):
    """KV-cache attention with the merge done by the last block of each (sequence, KV head): run twice on one workspace
    (the ticket counters must come back to zero), slices that are empty, partial tiles, several tiles.  Slices of at most
    128 positions take the tcgen05 variant, longer ones the CUDA-core variant."""
    from loomformer_paraplex_b200.ops import kernels, native
    torch.manual_seed(14)
    G = qh // kvh
    q, kc, vc = bf(B, qh, hd), bf(B, S, kvh, hd), bf(B, S, kvh, hd)
    kc[:, pos + 1:] = float("nan"); vc[:, pos + 1:] = float("nan")     # rows past the position must never be read into a sum
    p = torch.tensor([pos], device="cuda", dtype=torch.long)
    ws = torch.zeros(B * kvh * ns * (2 * G + 2 * G * hd) + B * kvh, device="cuda")
    kk = kc[:, :pos + 1].float().repeat_interleave(G, dim=2)          # [B,n,QH,HD]
    vv = vc[:, :pos + 1].float().repeat_interleave(G, dim=2)
    a = torch.softmax(torch.einsum("bhd,bshd->bhs", q.float(), kk) / hd ** 0.5, -1)
    for _ in range(2):
        c, k_ctx = torch.zeros_like(q), torch.zeros_like(q)
        native.ext().decode_attn(q, kc, vc, p, c, k_ctx, ws, B, S, qh, kvh, hd, ns, kernels.status_word(q.device))
        kernels.check_status(q.device)
        _close(c, torch.einsum("bhs,bshd->bhd", a, vv), 2e-2, "ctx")
        _close(k_ctx, torch.einsum("bhs,bshd->bhd", a, kk), 2e-2, "kctx")
    assert int(ws[-B * kvh:].view(torch.int32).abs().sum()) == 0


@pytest.mark.parametrize("hidden,batch,carry", [(256, 3, None), (172, 3, None), (256, 20, None), (172, 40, None), (256, 2, 7)])
def test_decode_engine_graph_matches_model_step_on_gpu(hidden, batch, carry):
    """Graph-replayed decode with the fused kernels follows the fp32 composed step (bf16 tolerance).
    ``hidden=172`` is 43 neurons per head: the fused step pads every sector to 48 inert-padded neurons.  Twenty and forty
    rows take the weight-stationary tensor-core kernel instead of the weight-streaming one; a carry token makes boundary keys fire from
    the token stream as well as from the window."""
    from loomformer_paraplex_b200.config import Config
    from loomformer_paraplex_b200.models.loomformer import Model
    from loomformer_paraplex_b200.serve.decode import DecodeEngine
    torch.manual_seed(0)
    cfg = Config(vocab=256, seq_len=96, model_dim=128, n_q_heads=4, head_dim=32, n_kv_heads=2, hidden=hidden, layers=2,
                 activation="pvpowlu", tria_carry_enabled=True, tria_temporal_auto=False, tria_temporal_window=16)
    model = Model(cfg).cuda().eval()
    model.carry_token_id = carry
    eng = DecodeEngine(model, batch=batch, use_graph=True)
    assert eng._native_attn and eng._fused and eng._dk.hpq == (64 if hidden == 256 else 48)
    assert eng.ca_cap == (eng.S if carry is not None else eng.S // 16 + 1)
    prompt = torch.randint(8, 256, (batch, 40), device="cuda")
    fp = DecodeEngine(model, batch=batch, use_graph=False, dtype=torch.float32)
    l1, l2 = eng.prefill(prompt).clone(), fp.prefill(prompt).clone()
    _close(l1, l2, 6e-2, "prefill logits")
    toks = torch.randint(8, 256, (12, batch), device="cuda")
    if carry is not None:
        toks[2, 0] = carry; toks[5] = carry                  # one sequence fires alone, then all of them
    for t in toks:                                           # same forced tokens on both engines; crosses a window fire
        l1, l2 = eng.step(t).clone(), fp.step(t).clone()
        _close(l1, l2, 6e-2, "step logits")
    assert int(eng.ca_len) == int(fp.ca_len) and int(eng.ca_len) >= 3
    n = int(eng.ca_len)
    assert torch.equal(eng.ca_valid[:, :n], fp.ca_valid[:, :n]) and torch.equal(eng.pending, fp.pending)
    # recurrent state: bf16 carriers against fp32 ones; a few near-degenerate 3x3 products amplify the rounding, so the
    # bound is on the bulk of the entries and on the mean, not on the single worst entry
    for name, a, b in (("temporal state", eng.carry, fp.carry), ("phase traces", eng.trace, fp.trace)):
        err, ref = (a.float() - b.float()).abs(), float(b.abs().max())
        assert float(err.mean()) <= 0.01 * ref, (name, float(err.mean()), ref)
        assert float((err > 0.06 * ref).float().mean()) < 5e-3, (name, float(err.max()), ref)
    assert not eng._K.fallbacks, dict(eng._K.fallbacks)


@pytest.mark.parametrize("static", [False, True])
def test_multi_segment_small_batch_linear(static):
    """Several products in one launch: own inputs (one gathered from strided pieces, one of them 96 wide so that a
    k-block straddles two pieces), weights, biases, output views of different dtypes; thirteen segments take two
    launches.  Up to 16 rows run on the weight-streaming kernel, 17..128 on the weight-stationary tcgen05 kernel."""
    from loomformer_paraplex_b200.ops import kernels
    ck = kernels.CudaKernels(defer_wgrad=False)
    torch.manual_seed(21)
    for M in (1, 3, 16, 17, 20, 64, 100, 128):
        x1, x2, x3 = bf(M, 768), bf(M, 3, 4, 32), bf(M, 2, 96)
        w1, w2, w3 = bf(1152, 768, scale=0.05), bf(200, 768 + 32 + 96 + 128, scale=0.05), bf(64, 768, scale=0.05)
        w4 = bf(300, 3072, scale=0.03)
        x4 = bf(M, 3072)
        b2 = torch.randn(200, device="cuda")
        y1 = torch.empty(M, 1152, device="cuda", dtype=torch.bfloat16)
        y4 = torch.empty(M, 300, device="cuda", dtype=torch.bfloat16)
        wide = torch.full((M, 208), 7.0, device="cuda")                       # fp32, strided view
        pieces = [x1, x2[:, 1, 2], x3[:, 1], x2[:, 2].reshape(M, 128)]
        segs = [([x1], w1, None, y1), (pieces, w2, b2, wide[:, :200]), ([x4], w4, None, y4)]
        outs = [torch.empty(M, 64, device="cuda", dtype=torch.bfloat16) for _ in range(10)]
        segs += [([x1], w3, None, o) for o in outs]
        torch.cuda.synchronize()
        ck.linear_multi(segs, static_weights=static)
        kernels.check_status(x1.device)
        _close(y1, x1.float() @ w1.float().t(), 2e-2, "seg 0")
        xc = torch.cat(pieces, -1).float()
        _close(wide[:, :200], xc @ w2.float().t() + b2, 3e-3, "gathered fp32 seg")
        assert bool((wide[:, 200:] == 7.0).all())
        _close(y4, x4.float() @ w4.float().t(), 2e-2, "long-K seg")
        for o in outs:
            _close(o, x1.float() @ w3.float().t(), 2e-2, "small seg")
        if M <= 16:
            # a launch whose segments all have few columns and a long reduction: several warps share a column
            w5, b5 = bf(768, 3072, scale=0.03), torch.randn(768, device="cuda")
            y5 = torch.empty(M, 768, device="cuda", dtype=torch.bfloat16)
            y6 = torch.empty(M, 300, device="cuda")
            ck.linear_multi([([x4], w5, b5, y5), ([x4[:, :1536], x4[:, 1536:]], w4, None, y6)], static_weights=static)
            _close(y5, x4.float() @ w5.float().t() + b5, 2e-2, "split-K seg")
            _close(y6, x4.float() @ w4.float().t(), 3e-3, "split-K seg, two pieces, fp32")
    assert not ck.fallbacks, ck.fallbacks


def test_decode_step_flags_and_boundary_append():
    from loomformer_paraplex_b200.ops import native
    ext = native.ext()
    dev = "cuda"
    B, cap, N, W, seq = 5, 4, 64, 16, 96
    flags = [torch.zeros(B, dtype=torch.bool, device=dev) for _ in range(4)]
    pending = torch.tensor([1, 0, 1, 0, 0], dtype=torch.bool, device=dev)
    tok = torch.tensor([3, 7, 9, 7, 1], device=dev)
    for pos, have, carry_tok, temporal in [(0, 1, 7, True), (15, 1, -1, True), (31, 0, 7, True), (20, 1, 7, False), (95, 1, -1, True)]:
        p = torch.tensor([pos], device=dev)
        hc = torch.tensor([bool(have)], device=dev)
        ext.decode_step_flags(p, tok, pending, hc, *flags, W, seq, True, carry_tok, temporal)
        hard = (pos + 1) % W == 0 and pos + 1 < seq
        fire = torch.full((B,), hard, device=dev) | (tok.eq(carry_tok) if carry_tok >= 0 else torch.zeros(B, dtype=torch.bool, device=dev))
        bos = pos == 0
        assert torch.equal(flags[0], fire)
        assert torch.equal(flags[1], pending | bos | (not temporal) | (not have))
        assert bool((flags[2] == bos).all())
        assert torch.equal(flags[3], pending & (not bos) & bool(have))
    # append: nobody fires -> nothing changes; some fire -> every row written, valid where fired; full store -> last slot
    ca_k, ca_v = torch.zeros(B, cap, N, device=dev, dtype=torch.bfloat16), torch.zeros(B, cap, N, device=dev, dtype=torch.bfloat16)
    valid = torch.zeros(B, cap, dtype=torch.bool, device=dev)
    ca_len, any_out = torch.zeros(1, dtype=torch.long, device=dev), torch.zeros(1, dtype=torch.long, device=dev)
    allowed = torch.zeros(B, cap, dtype=torch.uint8, device=dev)
    pend, have = torch.zeros(B, dtype=torch.bool, device=dev), torch.zeros(1, dtype=torch.bool, device=dev)
    ref_k, ref_valid, ref_len = ca_k.clone(), valid.clone(), 0
    for step, fire in enumerate([[0, 0, 0, 0, 0], [1, 0, 1, 0, 0], [1, 1, 1, 1, 1], [0, 0, 0, 0, 1], [0, 1, 0, 0, 0], [1, 0, 0, 0, 0]]):
        f = torch.tensor(fire, dtype=torch.bool, device=dev)
        nk, nv = bf(B, N), bf(B, N)
        ext.decode_ca_append(nk, nv, f, ca_k, ca_v, valid, ca_len, allowed, any_out, pend, have)
        ca_len.add_(any_out)
        if any(fire):
            slot = min(ref_len, cap - 1)
            ref_k[:, slot] = nk; ref_valid[:, slot] = f; ref_len += 1
        assert int(ca_len) == ref_len and int(any_out) == int(any(fire))
        assert torch.equal(ca_k, ref_k) and torch.equal(valid, ref_valid)
        want = ref_valid & (torch.arange(cap, device=dev).view(1, cap) < ref_len)
        assert torch.equal(allowed.bool(), want)
        assert torch.equal(pend, f) and bool(have)


def test_add_layernorm_with_rms_cap():
    ck, tk = _sets()
    torch.manual_seed(15)
    M, N = 200, 768
    a, b = bf(M, N, scale=2.0), bf(M, N, scale=0.5)          # a is clipped by the cap, b is not
    w, bias = torch.rand(N, device="cuda") + 0.5, torch.randn(N, device="cuda") * 0.1
    y1, x1, mu1, rs1 = ck.add_ln_fwd(a, b, w, bias, 1.0)
    y2, x2, mu2, rs2 = tk.add_ln_fwd(a.float(), b.float(), w, bias, 1.0)
    _close(y1, y2, 2e-2, "y"); _close(x1, x2, 1e-2, "x")
    dy = bf(M, N, scale=0.3)
    gw1, gb1, gw2, gb2 = (torch.zeros(N, device="cuda") for _ in range(4))
    da1, db1 = ck.add_ln_bwd(dy, x1, mu1, rs1, w, gw1, gb1, 1.0, a, b)
    da2, db2 = tk.add_ln_bwd(dy.float(), x2, mu2, rs2, w, gw2, gb2, 1.0, a.float(), b.float())
    _close(da1, da2, 3e-2, "da"); _close(db1, db2, 3e-2, "db"); _close(gw1, gw2, 2e-2, "gw")
    assert not ck.fallbacks, ck.fallbacks


def test_step_bookkeeping_helpers():
    """The per-cell helpers of the training plan: running-radius kernel, zero pool, GEMM output into a given buffer."""
    ck, tk = _sets()
    dev = torch.device("cuda")
    # running radius: in-place EMA + snapshot, against the PyTorch statement
    bsq = torch.tensor(3.7e5, device=dev)
    a1, a2 = torch.tensor(1.25, device=dev), torch.tensor(1.25, device=dev)
    s1 = ck.anchor_update(bsq, 2048.0 * 3072.0, a1, 0.99)
    s2 = tk.anchor_update(bsq, 2048.0 * 3072.0, a2, 0.99)
    assert torch.allclose(a1, a2, rtol=1e-6) and torch.allclose(s1, s2, rtol=1e-6) and s1.data_ptr() != a1.data_ptr()
    tiny = ck.anchor_update(torch.zeros((), device=dev), 10.0, torch.zeros((), device=dev), 0.0)
    assert abs(float(tiny) - 1e-4) < 1e-9                                   # the floor of the radius
    # zero pool: disjoint, aligned, zero slices; ordinary allocation once it is used up
    ck.begin_step(64 + 5 * 7 + 64, dev)
    z1, z2 = ck.zeros(1, device=dev), ck.zeros(5, 7, device=dev)
    z3 = ck.zeros(1000, device=dev)
    assert z1.data_ptr() % 256 == 0 and z2.data_ptr() % 256 == 0 and z2.data_ptr() - z1.data_ptr() == 256
    assert z2.shape == (5, 7) and float(z2.abs().sum()) == 0.0 and float(z3.abs().sum()) == 0.0
    z2.add_(1.0)
    assert float(z1.sum()) == 0.0
    # GEMM storing into a caller's packed buffer (a depth-history slot)
    x, w = bf(300, 256), bf(192, 256, scale=0.1)
    hist = torch.zeros(3, 300, 2, 6, 16, dtype=torch.bfloat16, device=dev)
    out = hist[1].view(300, 192)
    y = ck.linear(x, w, out=out)
    assert y.data_ptr() == out.data_ptr()
    _close(hist[1].view(300, 192), x.float() @ w.float().t(), 2e-2, "linear out=")
    assert float(hist[0].abs().sum()) == 0.0 and float(hist[2].abs().sum()) == 0.0
    assert not ck.fallbacks, ck.fallbacks


def test_per_op_switch_routes_to_the_twin(monkeypatch):
    """LOOM_DISABLE_OPS sends one named operation of a new kernel set to its PyTorch twin and counts it."""
    from loomformer_paraplex_b200.ops import kernels
    monkeypatch.setenv("LOOM_DISABLE_OPS", "add_ln_fwd")
    ck = kernels.CudaKernels()
    monkeypatch.delenv("LOOM_DISABLE_OPS")
    a, b = bf(64, 256), bf(64, 256)
    w, bias = torch.randn(256, device="cuda"), torch.randn(256, device="cuda")
    y1 = ck.add_ln_fwd(a, b, w, bias, None)[0]
    assert ck.fallbacks["add_ln_fwd"] == 1
    y2 = kernels.CudaKernels().add_ln_fwd(a, b, w, bias, None)[0]
    _close(y1, y2, 2e-2, "add_ln via twin")
    monkeypatch.setenv("LOOM_DISABLE_OPS", "no_such_op")
    with pytest.raises(ValueError):
        kernels.CudaKernels()


@pytest.mark.parametrize("M,N,K", [(1, 3072, 768), (3, 1536, 768), (8, 768, 3072), (16, 200, 136), (64, 1152, 768)])
def test_small_batch_linear(M, N, K):
    """The weight-streaming linear of the decode step (up to 16 rows; more rows take the tensor-core GEMM), with bias,
    fp32 output and a row-strided output view."""
    from loomformer_paraplex_b200.ops import kernels
    ck = kernels.CudaKernels(defer_wgrad=False)
    torch.manual_seed(9)
    x, w = bf(M, K), bf(N, K, scale=0.05)
    bias = torch.randn(N, device="cuda")
    ref = x.float() @ w.float().t() + bias
    y = ck.linear_small(x, w, bias)
    _close(y, ref, 2e-2, "bf16 out")
    wide = torch.full((M, N + 8), 7.0, device="cuda", dtype=torch.bfloat16)
    ck.linear_small(x, w, bias, out=wide[:, :N])
    _close(wide[:, :N], ref, 2e-2, "strided out")
    assert bool((wide[:, N:] == 7.0).all())
    if M <= 16:
        y32 = ck.linear_small(x, w, None, out_dtype=torch.float32)
        _close(y32, x.float() @ w.float().t(), 2e-3, "fp32 out")
    kernels.check_status(x.device)


@pytest.mark.parametrize("hd,qh,kvh", [(96, 8, 2), (64, 15, 5), (24, 4, 2)])
def test_decode_rope_store(hd, qh, kvh):
    """RoPE of one new token's Q / K at a device-side position with the KV-cache append, against the PyTorch statement."""
    from loomformer_paraplex_b200.ops import native
    from loomformer_paraplex_b200.ops import reference as R
    torch.manual_seed(10)
    B, S, rows = 3, 40, 64
    n, kv = qh * hd, kvh * hd
    qkv = bf(B, n + 2 * kv)
    cos, sin = torch.randn(rows, hd, device="cuda"), torch.randn(rows, hd, device="cuda")
    kc = torch.zeros(B, S, kvh, hd, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    qkc = torch.zeros(B, 3, qh, hd, device="cuda", dtype=torch.bfloat16)
    for p in (0, 17, 39):
        pos = torch.tensor([p], device="cuda", dtype=torch.long)
        native.ext().decode_rope_store(qkv, cos, sin, pos, qkc[:, 0].view(B, n), kc, vc, qh, kvh, hd)
        c, s_ = cos[p].view(1, 1, hd), sin[p].view(1, 1, hd)
        q_ref = R.apply_rope(qkv[:, :n].float().view(B, qh, hd), c, s_)
        k_ref = R.apply_rope(qkv[:, n:n + kv].float().view(B, kvh, hd), c, s_)
        _close(qkc[:, 0], q_ref, 2e-2, "q")
        _close(kc[:, p], k_ref, 2e-2, "k")
        assert torch.equal(vc[:, p].reshape(B, kv), qkv[:, n + kv:])
    assert float(qkc[:, 1:].abs().sum()) == 0.0
