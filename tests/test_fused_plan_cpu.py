"""The hand-written forward/backward of the fused plan (run with the PyTorch kernel twins on CPU, fp32)
must reproduce the composed model's loss and autograd gradients."""
import pytest
import torch
import torch.nn.functional as F

from loomformer_paraplex_b200.config import Config
from loomformer_paraplex_b200.models.loomformer import Model
from loomformer_paraplex_b200.ops.fused_plan import FusedPlan
from loomformer_paraplex_b200.ops.twins import TorchKernels

BASE = dict(vocab=61, seq_len=20, model_dim=None, n_q_heads=4, head_dim=8, n_kv_heads=2, hidden=None,
            hidden_mult=3.0, layers=4, activation="pvpowlu", tied_embeddings=False, tria_carry_enabled=True,
            tria_temporal_auto=False, tria_temporal_window=6, tria_carrier_alpha=0.05, tria_gamma_max=0.8,
            tria_raw_gamma_init=0.25)
VARIANTS = {
    "head_secant": dict(phase_grad_mode="secant"),
    "head_floor": dict(),
    "open_rich": dict(phase_sectors="open", paraplex_gate_proj=True, depth_attn_readout="per-sublayer",
                      depth_attn_qkv_rms=True, residual_branch_rms_cap=1.0, final_norm=True, tied_embeddings=True,
                      phase_grad_mode="secant"),
    "no_tria": dict(tria_carry_enabled=False),
}


def _model(extra):
    kw = dict(BASE); kw.update(extra)
    torch.manual_seed(0)
    m = Model(Config(**kw))
    with torch.no_grad():
        for _, p in m.named_parameters():
            if p.abs().max() == 0:
                p.normal_(0.0, 0.2)
    return m


@pytest.mark.parametrize("name", list(VARIANTS))
def test_fused_plan_matches_autograd(name):
    _check(name, _model(VARIANTS[name]))


@pytest.mark.parametrize("name", ["head_secant", "open_rich"])
def test_fused_plan_padded_sectors(name):
    """Five neurons per head, executed with every head's sector padded to eight: the padded neurons must change
    neither the loss nor any gradient (the GPU plan pads this way when a sector is not a multiple of 8 wide)."""
    m = _model(dict(VARIANTS[name], hidden=20, hidden_mult=None))
    assert m.d.hpq == 5
    plan = _check(name, m, pad_hidden=True)
    assert plan.d.hpq == 8 and plan.d.hidden == 32 and plan.d_true.hidden == 20


@pytest.mark.parametrize("name", ["head_secant", "open_rich"])
def test_fused_plan_with_chunk_checkpointing(name):
    """With ``grad_checkpointing`` the plan keeps only what crosses chunk boundaries and rebuilds each chunk's tape in
    the backward sweep; loss, gradients and the running radii must be what the stored-tape run gives."""
    m = _model(dict(VARIANTS[name], grad_checkpointing=True))
    assert m.d.grad_checkpointing
    _check(name, m)


def _check(name, m, **plan_kw):
    m.train()
    torch.manual_seed(1)
    x = torch.randint(0, 61, (3, 20))
    y = torch.randint(0, 61, (3, 20))
    y[0, :3] = -100
    pos = torch.arange(20).view(1, 20).expand(3, 20).contiguous()
    seg = None
    if name == "head_floor":       # packed rows: two segments per row
        pos = torch.cat((torch.arange(9), torch.arange(11))).view(1, 20).expand(3, 20).contiguous()
        seg = torch.cat((torch.zeros(9), torch.ones(11))).long().view(1, 20).expand(3, 20).contiguous()
    anchors0 = [b.ffn.beta_anchor.clone() for b in m.blocks]
    # composed plan + autograd
    mask = None
    if seg is not None:
        mask = ((seg[:, :, None] == seg[:, None, :]) & torch.ones(20, 20, dtype=torch.bool).tril()).unsqueeze(1)
    logits = m(x, attn_mask=mask, position_ids=pos)
    loss_ref = F.cross_entropy(logits.reshape(-1, 61), y.reshape(-1), ignore_index=-100)
    loss_ref.backward()
    ref = {n: p.grad.clone() for n, p in m.named_parameters() if p.grad is not None}
    anchors_ref = [b.ffn.beta_anchor.clone() for b in m.blocks]
    for p in m.parameters():
        p.grad = None
    for b, a in zip(m.blocks, anchors0):
        b.ffn.beta_anchor.copy_(a)
    # fused plan with torch twins
    plan = FusedPlan(m, kernels=TorchKernels(), compute_dtype=torch.float32, **plan_kw)
    with torch.no_grad():
        loss, _ = plan.run(x, y, pos, seg, want_grad=True)
    assert abs(float(loss) - float(loss_ref)) < 1e-5
    for b, a in zip(m.blocks, anchors_ref):
        assert torch.allclose(b.ffn.beta_anchor, a, atol=1e-6)
    for n, p in m.named_parameters():
        if n not in ref:
            assert p.grad is None or float(p.grad.abs().max()) == 0.0 or not p.requires_grad, n
            continue
        assert p.grad is not None, n
        scale = float(ref[n].abs().max()) + 1e-8
        err = float((p.grad - ref[n]).abs().max())
        assert err <= 3e-4 * scale + 1e-7, (n, err, scale)
    return plan


def test_fused_forward_logits_match():
    m = _model(dict(phase_grad_mode="secant")).eval()
    x = torch.randint(0, 61, (2, 20))
    with torch.no_grad():
        ref = m(x)
        plan = FusedPlan(m, kernels=TorchKernels(), compute_dtype=torch.float32)
        _, logits = plan.run(x, None, None, None, want_grad=False)
    assert torch.allclose(ref, logits, atol=2e-5, rtol=1e-4)


def test_per_op_switch_names_are_checked(monkeypatch):
    """``LOOM_DISABLE_OPS`` is validated against the kernel interface (the routing itself needs the native set)."""
    from loomformer_paraplex_b200.ops.twins import TorchKernels
    for name in ("attn_fwd", "attn_bwd", "ffn_core_fwd", "ffn_core_bwd", "imag_fwd", "linear", "dread_fwd", "add_ln_fwd"):
        assert callable(getattr(TorchKernels, name))
