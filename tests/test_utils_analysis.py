"""Research tooling: weight spectra, carrier geometry audit, slot-pool audit (tiny model, CPU)."""
import json
import os

import pytest
import torch

from loomformer_paraplex_b200.config import Config
from loomformer_paraplex_b200.data.tokenizers import BPETokenizer, train_tokenizer
from loomformer_paraplex_b200.models.loomformer import Model
from loomformer_paraplex_b200.train import checkpoint as ckpt
from loomformer_paraplex_b200.utils import geometry, slots, spectra

WORDS = "alpha beta gamma delta epsilon zeta eta theta iota kappa lambda mu".split()


@pytest.fixture(scope="module")
def probe(tmp_path_factory):
    d = tmp_path_factory.mktemp("an")
    tokp = str(d / "tok.json")
    train_tokenizer("", 300, tokp, texts=[" ".join(WORDS)] * 50)
    tok = BPETokenizer.load(tokp)
    import numpy as np
    rng = np.random.default_rng(0)
    with open(d / "text.jsonl", "w") as fh:
        for _ in range(200):
            fh.write(json.dumps({"text": " ".join(rng.choice(WORDS, 40))}) + "\n")
    cfg = Config(vocab=tok.vocab_size, tokenizer=tokp, seq_len=64, model_dim=32, n_q_heads=4, n_kv_heads=2, hidden=48,
                 layers=3, activation="pvpowlu", tria_carry_enabled=True, tria_temporal_auto=False,
                 tria_temporal_window=16, paraplex_gate_proj=True)
    torch.manual_seed(0)
    ckpt.save_checkpoint(str(d / "a.pt"), cfg, Model(cfg), None, "adamw", 0, 0)
    torch.manual_seed(1)
    ckpt.save_checkpoint(str(d / "b.pt"), cfg, Model(cfg), None, "adamw", 5, 0)
    return d


def test_spectra_report(probe):
    blob = torch.load(str(probe / "b.pt"), weights_only=True)
    init = torch.load(str(probe / "a.pt"), weights_only=True)["model"]
    lines = []
    out = spectra.analyze(blob, init, "cpu", log=lines.append)
    assert len(out["layers"]) == 3 and out["flags"]
    r = out["layers"][0]
    assert 1.0 <= r["qk_erank_mean"] <= 8.0 and abs(sum(r["imag_sector_share"].values()) - 1.0) < 1e-5
    assert any("[4] depth-attn" in ln for ln in lines) and any("axis 2" in ln for ln in lines)
    # batched per-head ranks equal the one-matrix-at-a-time definition
    qkv = blob["model"]["blocks.0.attn.qkv_weight"].float()
    q0, k0 = qkv[:8], qkv[32:40]
    s = torch.linalg.svdvals(q0.t() @ k0); p = s / s.sum()
    er0 = float(torch.exp(-(p * p.clamp_min(1e-12).log()).sum()))
    wq = qkv[:32].view(4, 8, 32); wk = qkv[32:48].view(2, 8, 32).repeat_interleave(2, 0)
    assert abs(float(spectra.spectrum(wq.transpose(1, 2) @ wk)["erank"][0]) - er0) < 1e-4


def test_geometry_metrics_on_known_matrices():
    th = torch.tensor(0.3)
    rz = torch.tensor([[torch.cos(th), -torch.sin(th), 0.0], [torch.sin(th), torch.cos(th), 0.0], [0.0, 0.0, 1.0]])
    d = geometry.Decomposition((2.0 * rz).view(1, 1, 1, 3, 3), 3.0, 2.7)
    assert abs(float(d.condition) - 1.0) < 1e-5 and abs(float(d.erank) - 3.0) < 1e-4 and bool(d.passed)
    assert abs(float(d.angle) - 0.3) < 1e-5 and not bool(d.reflected)
    axis, ok = geometry.rotation_axis(d.rotation)
    assert bool(ok) and torch.allclose(axis.flatten().abs(), torch.tensor([0.0, 0.0, 1.0]), atol=1e-5)
    flat = torch.diag(torch.tensor([1.0, 1.0, 1e-3])).view(1, 1, 1, 3, 3)
    d2 = geometry.Decomposition(flat, 3.0, 2.7)
    assert not bool(d2.passed) and float(d2.erank) < 2.1
    passed = torch.tensor([[[True], [True], [False], [True]]])
    assert int(geometry.first_failure_horizon(passed)) == 3
    assert int(geometry.first_failure_horizon(torch.ones(1, 4, 1, dtype=torch.bool))) == 5


def test_geometry_and_slots_end_to_end(probe):
    out = str(probe / "geo.json")
    rep = geometry.run(str(probe / "b.pt"), str(probe / "text.jsonl"), init=str(probe / "a.pt"), tokens=64, raw_tokens=48,
                       sequences=2, device="cpu", output=out, log=lambda *_: None)
    assert rep["window"] == 16 and len(rep["trained"]["operational"]["by_chunk"]) == 4
    assert rep["trained"]["boundary_state"]["keys"] == 3
    assert len(rep["trained"]["temporal"]["condition_mean"]) == 48
    assert "16" in rep["trained_vs_init_operational"]["selected_horizons"]
    assert 0.0 <= rep["trained"]["temporal"]["selected_horizons"]["16"]["population_pass"] <= 1.0
    assert json.load(open(out))["thresholds"]["max_condition"] == 3.0
    out2 = str(probe / "slots.json")
    rep2 = slots.run(str(probe / "b.pt"), str(probe / "text.jsonl"), tokens=64, sequences=3, device="cpu", output=out2,
                     log=lambda *_: None)
    assert len(rep2["chunks"]) == 3 and rep2["sequences"] == 3
    c = rep2["chunks"][1]
    assert 1.0 <= c["slot_population"]["covariance_effective_rank"] <= 9.0
    assert 0.0 < c["pool"]["normalized_entropy"]["mean"] <= 1.0 + 1e-6
    with pytest.raises(ValueError):
        geometry.run(str(probe / "b.pt"), str(probe / "text.jsonl"), tokens=60, device="cpu", output=out)
