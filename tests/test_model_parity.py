"""Model-level parity with the reference on CPU fp32: same state_dict -> same logits, same
gradients, and forward == token-by-token step."""
import copy

import pytest
import torch

from loomformer_paraplex_b200.config import Config
from loomformer_paraplex_b200.models.loomformer import Model
from tests.oracle import load_reference, ref_config

TOY = dict(vocab=97, seq_len=24, batch_size=2, model_dim=None, n_q_heads=4, head_dim=8, n_kv_heads=2,
           hidden=None, hidden_mult=3.0, layers=4, activation="pvpowlu", tied_embeddings=False,
           tria_carry_enabled=True, tria_temporal_auto=False, tria_temporal_window=6,
           tria_carrier_alpha=0.05, tria_gamma_max=0.8, tria_raw_gamma_init=0.25)

VARIANTS = {
    "head_floor": dict(),
    "head_secant": dict(phase_grad_mode="secant"),
    "open_rich": dict(phase_sectors="open", paraplex_gate_proj=True, depth_attn_readout="per-sublayer",
                      depth_attn_qkv_rms=True, phase_grad_mode="secant", final_norm=True, tied_embeddings=True),
    "no_tria": dict(tria_carry_enabled=False),
    "capped": dict(residual_branch_rms_cap=1.0, phase_sectors="open"),
    "ckpt": dict(grad_checkpointing=True, phase_grad_mode="secant"),
}


def _pair(extra):
    lf = load_reference()
    kw = dict(TOY); kw.update(extra)
    rcfg = ref_config(lf, **kw)
    lf.CARRY_TOKEN_ID = None
    lf.apply_config(rcfg)
    torch.manual_seed(0)
    ref = lf.Model(rcfg)
    # move the zero-initialised parameters off zero so every path carries signal
    with torch.no_grad():
        for name, p in ref.named_parameters():
            if p.abs().max() == 0:
                p.normal_(0.0, 0.2)
    mine = Model(Config(**kw))
    missing = mine.load_state_dict(ref.state_dict(), strict=True)
    return lf, ref, mine


@pytest.mark.parametrize("name", list(VARIANTS))
def test_forward_and_grads_match_reference(name):
    lf, ref, mine = _pair(VARIANTS[name])
    ref.train(); mine.train()
    torch.manual_seed(1)
    idx = torch.randint(0, 97, (2, 24))
    out_r = ref(idx)
    out_m = mine(idx)
    assert out_m.shape == out_r.shape
    assert torch.allclose(out_m, out_r, atol=2e-5, rtol=1e-4), float((out_m - out_r).abs().max())
    tgt = torch.randint(0, 97, (2, 24))
    torch.nn.functional.cross_entropy(out_r.reshape(-1, 97), tgt.reshape(-1)).backward()
    torch.nn.functional.cross_entropy(out_m.reshape(-1, 97), tgt.reshape(-1)).backward()
    gr = {n: p.grad for n, p in ref.named_parameters()}
    for n, p in mine.named_parameters():
        if gr[n] is None:
            assert p.grad is None or float(p.grad.abs().max()) == 0.0, n
            continue
        assert p.grad is not None, n
        scale = float(gr[n].abs().max()) + 1e-8
        assert float((p.grad - gr[n]).abs().max()) <= 2e-4 * scale + 1e-7, (n, scale)
    # the anchor EMA moved identically
    for br, bm in zip(ref.blocks, mine.blocks):
        assert torch.allclose(br.ffn.beta_anchor, bm.ffn.beta_anchor, atol=1e-6)


def test_packed_mask_and_position_ids_match_reference():
    lf, ref, mine = _pair(dict())
    ref.eval(); mine.eval()
    torch.manual_seed(2)
    idx = torch.randint(0, 97, (2, 24))
    pos = torch.cat((torch.arange(10), torch.arange(14))).view(1, 24).expand(2, 24).contiguous()
    seg = torch.cat((torch.zeros(10), torch.ones(14))).long()
    mask = (seg[:, None] == seg[None, :]) & torch.ones(24, 24, dtype=torch.bool).tril()
    mask = mask.view(1, 1, 24, 24).expand(2, 1, 24, 24)
    with torch.no_grad():
        a, b = ref(idx, attn_mask=mask, position_ids=pos), mine(idx, attn_mask=mask, position_ids=pos)
    assert torch.allclose(a, b, atol=2e-5, rtol=1e-4)


@pytest.mark.parametrize("name", ["head_floor", "open_rich", "no_tria"])
def test_step_matches_forward_and_reference_step(name):
    lf, ref, mine = _pair(VARIANTS[name])
    ref.eval(); mine.eval()
    torch.manual_seed(3)
    idx = torch.randint(0, 97, (2, 20))
    with torch.no_grad():
        full = mine(idx)
        st_m = st_r = None
        for t in range(20):
            lm, st_m = mine.step(idx[:, t], t, st_m)
            lr, st_r = ref.step(idx[:, t], t, st_r)
            assert torch.allclose(lm, lr, atol=3e-5, rtol=1e-4), (t, float((lm - lr).abs().max()))
            assert torch.allclose(lm, full[:, t], atol=5e-5, rtol=1e-4), (t, float((lm - full[:, t]).abs().max()))
