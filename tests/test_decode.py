"""Decode engine: token-by-token equals Model.step, and batched prefill through the fused plan hands over a state
from which decoding continues exactly as if every prompt token had been stepped."""
import pytest
import torch

from loomformer_paraplex_b200.config import Config
from loomformer_paraplex_b200.models.loomformer import Model
from loomformer_paraplex_b200.ops.fused_plan import FusedPlan
from loomformer_paraplex_b200.ops.twins import TorchKernels
from loomformer_paraplex_b200.serve.decode import DecodeEngine

KW = dict(vocab=61, seq_len=40, model_dim=None, n_q_heads=4, head_dim=8, n_kv_heads=2, hidden=None, hidden_mult=3.0,
          layers=3, activation="pvpowlu", tied_embeddings=False, tria_carry_enabled=True, tria_temporal_auto=False,
          tria_temporal_window=6, tria_carrier_alpha=0.05, tria_gamma_max=0.8, tria_raw_gamma_init=0.25)


def _model(**extra):
    torch.manual_seed(0)
    m = Model(Config(**dict(KW, **extra))).eval()
    with torch.no_grad():
        for _, p in m.named_parameters():
            if p.abs().max() == 0:
                p.normal_(0.0, 0.2)
    return m


@pytest.mark.parametrize("extra", [dict(), dict(phase_sectors="open", paraplex_gate_proj=True, depth_attn_qkv_rms=True,
                                                depth_attn_readout="per-sublayer", final_norm=True)])
def test_engine_step_equals_model_step(extra):
    m = _model(**extra)
    x = torch.randint(0, 61, (2, 25))
    eng = DecodeEngine(m, batch=2, use_graph=False)
    st = None
    for t in range(25):
        ref, st = m.step(x[:, t], t, st)
        got = eng.step(x[:, t])
        assert torch.allclose(ref, got, atol=3e-5, rtol=1e-4), (t, float((ref - got).abs().max()))


@pytest.mark.parametrize("T0", [11, 12, 18, 7])
def test_prefill_then_decode_matches_stepping(T0):
    m = _model()
    x = torch.randint(0, 61, (2, 30))
    ref = DecodeEngine(m, batch=2, use_graph=False)
    for t in range(T0):
        last = ref.step(x[:, t]).clone()
    m.ops = FusedPlan(m, kernels=TorchKernels(), compute_dtype=torch.float32)
    eng = DecodeEngine(m, batch=2, use_graph=False)
    got = eng.prefill(x[:, :T0])
    assert torch.allclose(last, got, atol=5e-5, rtol=1e-4), float((last - got).abs().max())
    for t in range(T0, 30):
        a, b = ref.step(x[:, t]), eng.step(x[:, t])
        assert torch.allclose(a, b, atol=5e-5, rtol=1e-4), (t, float((a - b).abs().max()))


def test_sector_padding_helpers_round_trip():
    """The fused decode step pads every head's hidden sector to a multiple of 8 neurons: padding places sector j of
    head g at g * padded_width + j, leaves zeros behind it, and un-padding restores the tensor (any axis)."""
    cfg = Config(vocab=64, seq_len=16, model_dim=32, n_q_heads=4, head_dim=8, n_kv_heads=2, hidden=20, layers=1,
                 activation="pvpowlu", tria_carry_enabled=True, tria_temporal_auto=False, tria_temporal_window=4)
    eng = DecodeEngine(Model(cfg).eval(), batch=2, use_graph=False)
    assert (eng.d.hpq, eng._dk.hpq, eng._dk.hidden) == (5, 8, 32)
    x = torch.arange(2 * 20 * 3, dtype=torch.float32).view(2, 20, 3) + 1.0
    p = eng._pad(x, 1)
    assert p.shape == (2, 32, 3)
    assert torch.equal(p.view(2, 4, 8, 3)[:, :, :5], x.view(2, 4, 5, 3)) and float(p.view(2, 4, 8, 3)[:, :, 5:].abs().sum()) == 0
    assert torch.equal(eng._unpad(p, 1), x)
    w = torch.randn(20, 7)
    assert torch.equal(eng._unpad(eng._pad(w, 0), 0), w) and eng._pad(w, 0).shape == (32, 7)
    w2 = torch.randn(6, 20)
    assert torch.equal(eng._unpad(eng._pad(w2, 1), 1), w2) and eng._pad(w2, 1).shape == (6, 32)


def test_decode_requests_beyond_the_cache_are_refused_on_the_host():
    """A prompt + continuation that would pass the KV cache / RoPE table must raise before anything is launched."""
    from loomformer_paraplex_b200.serve import decode as dec
    with pytest.raises(ValueError):
        dec.check_request(100, 30, 128)
    dec.check_request(100, 29, 128)
    with pytest.raises(ValueError):
        dec.check_request(0, 4, 128)
    with pytest.raises(ValueError):
        dec.check_request(4, 0, 128)
    model = _model()
    with pytest.raises(ValueError):
        dec.DecodeEngine(model, batch=1, max_len=41, use_graph=False)
    eng = dec.DecodeEngine(model, batch=1, max_len=8, use_graph=False)
    prompt = torch.randint(0, 61, (1, 6))
    with pytest.raises(ValueError):
        eng.generate(prompt, 4)                  # needs 9 positions
    out = eng.generate(prompt, 3)                # needs exactly 8
    assert out.shape == (1, 3)
    with pytest.raises(ValueError):
        eng.step(out[:, -1])                     # position 8 does not exist
    with pytest.raises(ValueError):
        eng.prefill(torch.randint(0, 61, (1, 9)))


def test_boundary_key_store_is_sized_by_what_can_fire():
    """Without a carry token only window boundaries append keys (one per window); with one, any token may.  A carry
    token given to the model after the engine was built grows the store at the next reset, and the engine then follows
    the module's own step through token-triggered boundaries."""
    m = _model()
    eng = DecodeEngine(m, batch=2, use_graph=False)
    assert eng.ca_cap == eng.S // 6 + 1 and eng.ca_k.shape[1] == eng.ca_cap
    x = torch.randint(1, 61, (2, 30))
    x[0, 4] = 0; x[:, 9] = 0; x[1, 10] = 0                     # token 0 becomes the carry token below
    m.carry_token_id = 0
    try:
        eng.reset()
        assert eng.ca_cap == eng.S and eng.ca_k.shape[1] == eng.S and eng.ca_valid.shape[1] == eng.S
        st = None
        for t in range(30):
            ref, st = m.step(x[:, t], t, st)
            got = eng.step(x[:, t])
            assert torch.allclose(ref, got, atol=3e-5, rtol=1e-4), (t, float((ref - got).abs().max()))
        assert int(eng.ca_len) >= 30 // 6 + 2                   # window fires plus the token-triggered ones
    finally:
        m.carry_token_id = None
