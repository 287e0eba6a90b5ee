"""The command-line workflows on a GPU: pre-training through the graph-replayed fused plan with document resets,
run-points and resume, full evaluation, greedy inference, SFT, packaging and a scripted chat turn."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch
import yaml

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORDS = "the quick brown fox jumps over a lazy dog while loom threads weave phase carriers through depth".split()


def run(args, cwd, stdin=None):
    env = dict(os.environ, PYTHONPATH=ROOT, OMP_NUM_THREADS="2")
    r = subprocess.run([sys.executable] + args, cwd=cwd, env=env, capture_output=True, text=True, timeout=900, input=stdin)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return r.stdout + r.stderr


def test_cli_workflows_on_gpu(tmp_path):
    d = str(tmp_path)
    os.makedirs(os.path.join(d, "data"))
    rng = np.random.default_rng(0)
    with open(os.path.join(d, "data", "a.jsonl"), "w") as fh:
        for _ in range(400):
            fh.write(json.dumps({"text": " ".join(rng.choice(WORDS, 70))}) + "\n")
    cfg = dict(vocab=320, tokenizer="tok.json", tied_embeddings=False, seq_len=256, batch_size=4, model_dim=128, n_q_heads=4,
               head_dim=32, n_kv_heads=2, hidden=None, hidden_mult=4.0, layers=2, activation="pvpowlu",
               phase_grad_mode="secant", tria_carry_enabled=True, tria_temporal_auto=False, tria_temporal_window=64,
               tria_carrier_alpha=0.05, steps=12, lr=2e-3, warmup_steps=2, log_every=3, eval_every=6, eval_batches=1,
               save_every=8, device="cuda:0", dataset_format="jsonl", train_dataset="data", auto_val_split_pct=5.0,
               prefetch_batches=4, gpu_prefetch_batches=2, optimizer="adamw", amp_dtype="bf16")
    with open(os.path.join(d, "cfg.yaml"), "w") as fh:
        yaml.safe_dump(cfg, fh)
    loom = os.path.join(ROOT, "loomformer.py")
    run([loom, "--train-tokenizer", "data", "--tokenizer-out", "tok.json", "--vocab", "320", "--config", "cfg.yaml"], d)
    out = run([loom, "--train", "--config", "cfg.yaml", "--checkpoint", "m.pt"], d)
    assert "step     12" in out and os.path.exists(os.path.join(d, "m.runpoint_step8.pt"))
    losses = [float(ln.split("train_loss")[1].split()[0]) for ln in out.splitlines() if "train_loss" in ln]
    assert losses and losses[-1] < losses[0]
    out = run([loom, "--train", "--config", "cfg.yaml", "--checkpoint", "m2.pt", "--resume", "m.runpoint_step8.pt"], d)
    assert "continuing from step 8/12" in out
    out = run([loom, "--eval", "--checkpoint", "m.pt", "--dataset", os.path.join("data", "val", "val_split.jsonl"),
               "--config", "cfg.yaml", "--device", "cuda:0"], d)
    assert "bpb" in out
    out = run([loom, "--infer", "--checkpoint", "m.pt", "--prompt", "the quick", "--max-new", "8", "--device", "cuda:0"], d)
    assert out.strip()
    with open(os.path.join(d, "chat.jsonl"), "w") as fh:
        for _ in range(60):
            fh.write(json.dumps({"messages": [{"role": "user", "content": " ".join(rng.choice(WORDS, 8))},
                                              {"role": "assistant", "content": " ".join(rng.choice(WORDS, 10))}]}) + "\n")
    out = run([os.path.join(ROOT, "loomsft.py"), "--config", "cfg.yaml", "--sft-dataset", "chat.jsonl", "--init-checkpoint",
               "m.pt", "--checkpoint", "s.pt", "--device", "cuda:0", "--steps", "6"], d)
    assert "[loomsft] saved -> s.pt" in out
    run([os.path.join(ROOT, "loompack.py"), "pack", "s.pt", "--tokenizer", "tok.json", "--template",
         os.path.join(ROOT, "chat_template.jinja"), "-o", "s.aio", "--quant", "bf16"], d)
    out = run([os.path.join(ROOT, "loomchat.py"), "s.aio", "--device", "cuda:0", "--temperature", "0", "--max-new", "6"], d,
              stdin="/settings\nthe quick brown\n/exit\n")
    assert "loom>" in out and "temperature" in out


@pytest.mark.parametrize("sync", ["p2p", "fsdp"])
def test_cli_multi_gpu_training_saves_complete_checkpoints(tmp_path, sync):
    """`--device cudas` self-launches one rank per GPU; the fused / sharded gradient paths write checkpoints whose
    parameters and optimizer moments are complete (owners' shards gathered), and resume continues from them."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    d = str(tmp_path)
    os.makedirs(os.path.join(d, "data"))
    rng = np.random.default_rng(0)
    with open(os.path.join(d, "data", "a.jsonl"), "w") as fh:
        for _ in range(400):
            fh.write(json.dumps({"text": " ".join(rng.choice(WORDS, 70))}) + "\n")
    cfg = dict(vocab=320, tokenizer="tok.json", tied_embeddings=False, seq_len=256, batch_size=4, model_dim=128, n_q_heads=4,
               head_dim=32, n_kv_heads=2, hidden=None, hidden_mult=4.0, layers=2, activation="pvpowlu",
               phase_grad_mode="secant", tria_carry_enabled=True, tria_temporal_auto=False, tria_temporal_window=64,
               tria_carrier_alpha=0.05, steps=8, lr=2e-3, warmup_steps=2, log_every=2, eval_every=4, eval_batches=1,
               save_every=4, device="cuda:0,cuda:1", dataset_format="jsonl", train_dataset="data", auto_val_split_pct=5.0,
               prefetch_batches=4, gpu_prefetch_batches=2, optimizer="adamw", amp_dtype="bf16")
    with open(os.path.join(d, "cfg.yaml"), "w") as fh:
        yaml.safe_dump(cfg, fh)
    loom = os.path.join(ROOT, "loomformer.py")
    run([loom, "--train-tokenizer", "data", "--tokenizer-out", "tok.json", "--vocab", "320", "--config", "cfg.yaml"], d)
    out = run([loom, "--train", "--config", "cfg.yaml", "--checkpoint", "m.pt", "--grad-sync", sync], d)
    assert "step      8" in out, out[-2000:]
    blob = torch.load(os.path.join(d, "m.pt"), weights_only=True)
    assert all(torch.isfinite(v).all() for v in blob["model"].values() if torch.is_tensor(v) and v.is_floating_point())
    st = blob["optimizer"]["state"]
    moved = [float(s["exp_avg_sq"].abs().sum()) > 0 for s in st.values() if s["exp_avg_sq"].numel() > 4096]
    assert moved and all(moved)                   # no big tensor is left with another rank's (zero) moments
    out = run([loom, "--train", "--config", "cfg.yaml", "--checkpoint", "m2.pt", "--resume", "m.runpoint_step4.pt",
               "--grad-sync", sync], d)
    assert "continuing from step 4/8" in out
