"""End-to-end workflows on CPU through the public entry points: tokenizer training, pre-training with run-points and
resume, full evaluation, greedy inference, and checkpoint interchange with the reference implementation."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch
import yaml

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORDS = "the quick brown fox jumps over a lazy dog while loom threads weave phase carriers through depth".split()


def run(args, cwd):
    env = dict(os.environ, PYTHONPATH=ROOT, OMP_NUM_THREADS="2")
    r = subprocess.run([sys.executable] + args, cwd=cwd, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return r.stdout + r.stderr


@pytest.fixture(scope="module")
def workdir(tmp_path_factory):
    d = tmp_path_factory.mktemp("wf")
    (d / "data").mkdir()
    rng = np.random.default_rng(0)
    with open(d / "data" / "a.jsonl", "w") as fh:
        for i in range(300):
            fh.write(json.dumps({"text": " ".join(rng.choice(WORDS, 60))}) + "\n")
    cfg = dict(vocab=300, tokenizer="tok.json", tied_embeddings=False, seq_len=48, batch_size=4, model_dim=32, n_q_heads=4,
               head_dim=8, n_kv_heads=2, hidden=None, hidden_mult=3.0, layers=2, activation="pvpowlu",
               phase_grad_mode="secant", tria_carry_enabled=True, tria_temporal_auto=False, tria_temporal_window=16,
               tria_carrier_alpha=0.05, steps=6, lr=3e-3, warmup_steps=2, log_every=2, eval_every=3, eval_batches=1,
               save_every=4, device="cpu", dataset_format="jsonl", train_dataset="data", auto_val_split_pct=5.0,
               prefetch_batches=4, gpu_prefetch_batches=2, optimizer="adamw", amp_dtype="fp32")
    with open(d / "cfg.yaml", "w") as fh:
        yaml.safe_dump(cfg, fh)
    return d


def test_pretrain_resume_eval_infer(workdir):
    d = str(workdir)
    loom = os.path.join(ROOT, "loomformer.py")
    out = run([loom, "--train-tokenizer", "data", "--tokenizer-out", "tok.json", "--vocab", "300", "--config", "cfg.yaml"], d)
    assert os.path.exists(os.path.join(d, "tok.json"))
    out = run([loom, "--train", "--config", "cfg.yaml", "--checkpoint", "m.pt"], d)
    assert "[LoomFormer-paraplex] step      6" in out and "saved LoomFormer-paraplex -> m.pt" in out
    assert os.path.exists(os.path.join(d, "m.runpoint_step4.pt"))
    blob = torch.load(os.path.join(d, "m.pt"), weights_only=True)
    assert blob["step"] == 6 and blob["model_kind"] == "loomformer" and blob["tokens_seen"] == 6 * 4 * 48
    out = run([loom, "--train", "--config", "cfg.yaml", "--checkpoint", "m2.pt", "--resume", "m.runpoint_step4.pt"], d)
    assert "continuing from step 4/6" in out and "restored adamw optimizer state" in out
    out = run([loom, "--eval", "--checkpoint", "m.pt", "--dataset", os.path.join("data", "val", "val_split.jsonl"),
               "--config", "cfg.yaml", "--device", "cpu"], d)
    assert "bpb" in out and "eval_loss" in out
    out = run([loom, "--infer", "--checkpoint", "m.pt", "--prompt", "the quick", "--max-new", "5", "--device", "cpu"], d)
    assert out.strip()


def test_checkpoint_loads_in_reference_and_back(workdir):
    from tests.oracle import load_reference
    lf = load_reference()
    d = str(workdir)
    path = os.path.join(d, "m.pt")
    if not os.path.exists(path):
        pytest.skip("training test did not run")
    blob = torch.load(path, weights_only=True)
    cwd = os.getcwd()
    os.chdir(d)
    try:
        rcfg = lf.Config.from_checkpoint_dict(blob["cfg"])
        for k in ("use_cuda_phase_sin", "use_cuda_beta_space", "use_cuda_pvpowlu", "use_cuda_depth_attn", "use_cuda_tria"):
            setattr(rcfg, k, False)
        lf.build_tokenizer(rcfg)
        lf.apply_config(rcfg)
        ref = lf.Model(rcfg)
        lf.load_model_blob_into(ref, blob, ablation=False)       # strict load inside
        from loomformer_paraplex_b200.serve.runtime import load_model
        mine, _, _, _ = load_model(path, torch.device("cpu"))
    finally:
        os.chdir(cwd)
    x = torch.randint(0, 300, (2, 40))
    with torch.no_grad():
        assert torch.allclose(ref.eval()(x), mine(x), atol=3e-5, rtol=1e-4)


def test_sft_train_and_resume(workdir):
    """Fine-tune the pre-trained checkpoint on chat records, stop at a run-point, resume from it."""
    d = str(workdir)
    if not os.path.exists(os.path.join(d, "m.pt")):
        pytest.skip("training test did not run")
    rng = np.random.default_rng(1)
    with open(os.path.join(d, "chat.jsonl"), "w") as fh:
        for i in range(40):
            fh.write(json.dumps({"messages": [
                {"role": "user", "content": " ".join(rng.choice(WORDS, 5))},
                {"role": "assistant", "content": " ".join(rng.choice(WORDS, 6))}]}) + "\n")
    sft = os.path.join(ROOT, "loomsft.py")
    out = run([sft, "--smoke-test"], d)
    assert "[loomsft smoke] OK" in out
    out = run([sft, "--config", "cfg.yaml", "--sft-dataset", "chat.jsonl", "--val-dataset", "chat.jsonl",
               "--init-checkpoint", "m.pt", "--checkpoint", "s.pt", "--device", "cpu"], d)
    assert "[loomsft] step      4" in out and "eval_loss" in out and "[loomsft] saved -> s.pt" in out
    assert os.path.exists(os.path.join(d, "s.runpoint_step4.pt"))
    out = run([sft, "--config", "cfg.yaml", "--sft-dataset", "chat.jsonl", "--resume", "s.runpoint_step4.pt",
               "--checkpoint", "s2.pt", "--device", "cpu"], d)
    assert "continuing from step 4/6" in out
    assert torch.load(os.path.join(d, "s2.pt"), weights_only=True)["step"] == 6
