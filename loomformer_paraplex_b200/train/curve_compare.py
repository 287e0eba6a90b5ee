"""Loss curves of this repository and of the unmodified reference, from one shared initial state, on learnable
synthetic data.

``python -m loomformer_paraplex_b200.train.curve_compare --steps 200 --out curves.md``

Both arms train the 113M architecture (dims of ``cfg/nano.yaml``) in bf16 with AdamW, the same learning-rate schedule
and the same batches: every row is a random pattern of 64 tokens repeated to the sequence length, so the loss falls
quickly once the model copies from one period back -- unlike uniform-random tokens, on which every model sits at
ln(vocab).  The reference arm imports ``baseline/_ref/loomformer.py`` and runs the body of its training loop
(``loomformer.py:5071-5170``); its weights are loaded from this repository's initial ``state_dict`` (the layouts are the
same), which replaces matching two random-number streams.  Prints mean loss per block of steps for both arms.
"""
from __future__ import annotations

import argparse
import math
import os
import sys
import time

import torch
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def model_kw(seq_len: int, steps: int, lr: float, warmup: int) -> dict:
    sys.path.insert(0, ROOT)
    import bench
    return dict(bench.MODEL_KW, seq_len=seq_len, steps=steps, lr=lr, warmup_steps=warmup, min_lr_frac=0.1)


def batches(vocab: int, batch: int, seq_len: int, steps: int, kind: str = "pool", period: int = 64, seed: int = 11):
    """``periodic``: every row a fresh random 64-token pattern repeated (learnable by copying one period back);
    ``pool``: rows drawn in a fixed order from a pool of 16 fixed random rows (learnable by memorising them, which a
    113M model does within a few hundred steps)."""
    g = torch.Generator().manual_seed(seed)
    if kind == "periodic":
        reps = -(-(seq_len + 1) // period)
        return [torch.randint(0, vocab, (batch, period), generator=g).repeat(1, reps)[:, :seq_len + 1].contiguous()
                for _ in range(steps)]
    pool = torch.randint(0, vocab, (16, seq_len + 1), generator=g)
    return [pool[[(i * batch + j) % 16 for j in range(batch)]].contiguous() for i in range(steps)]


def run_ours(kw, data, dev):
    from ..config import Config
    from ..models.loomformer import Model
    from .engine import TrainEngine
    cfg = Config(**kw, batch_size=data[0].shape[0])
    torch.manual_seed(cfg.seed)
    model = Model(cfg).to(dev)
    init = {k: v.detach().clone().cpu() for k, v in model.state_dict().items()}
    eng = TrainEngine(cfg, model, dev, optimizer="adamw")
    losses = []
    for b in data:
        losses.append(eng.step(b.to(dev)))
    out = [float(x) for x in torch.stack(losses).float().cpu()]
    eng.check_finite(losses[-1])
    return out, init


def run_reference(kw, data, dev, init):
    sys.path.insert(0, ROOT)
    import bench
    ref = bench.reference_dir()                     # the path its extensions were built under, when it still fits
    if not os.path.isfile(os.path.join(ref, "loomformer.py")):
        return None
    bench.adopt_reference_toolchain(ref)
    bench.settle_reference_mtimes(ref)
    sys.dont_write_bytecode = True
    sys.path.insert(0, ref)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    import importlib
    lf = importlib.import_module("loomformer")              # baseline/_ref is first on sys.path
    cfg = lf.Config(**{k: v for k, v in kw.items() if k in lf.Config.__dataclass_fields__}, batch_size=data[0].shape[0])
    cfg.device = str(dev)
    lf.CARRY_TOKEN_ID = None
    lf.device_auto(str(dev))
    lf.apply_config(cfg)
    model = lf.Model(cfg).to(dev)
    missing = model.load_state_dict({k: v.to(dev) for k, v in init.items()}, strict=True)
    params = [p for p in model.parameters() if p.requires_grad]
    nodecay = {id(model.tria_agg.pool.logit_scale_raw)} if model.tria_agg is not None else set()
    groups = {}
    for p in params:
        groups.setdefault(0.0 if id(p) in nodecay else cfg.weight_decay, []).append(p)
    opt = torch.optim.AdamW([{"params": ps, "weight_decay": wd} for wd, ps in groups.items()], lr=cfg.lr,
                            weight_decay=cfg.weight_decay)
    model.train()
    losses = []
    for step, b in enumerate(data):
        b = b.to(dev)
        x, y = b[:, :-1], b[:, 1:]
        opt.zero_grad(set_to_none=True)
        position_ids, attn_mask = lf.build_doc_reset_state(x, None)
        with lf.amp_autocast(dev):
            logits = model(x, attn_mask=attn_mask, position_ids=position_ids)
        loss = F.cross_entropy(logits.float().reshape(-1, lf.VOCAB), y.reshape(-1))
        loss.backward()
        if cfg.grad_clip and cfg.grad_clip > 0:
            torch.nn.utils.clip_grad_norm_(params, cfg.grad_clip)
        lr = lf.lr_at(cfg, step)
        for grp in opt.param_groups:
            grp["lr"] = lr
        opt.step()
        losses.append(float(loss.detach()))
    return losses


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--lr", type=float, default=6e-4)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--block", type=int, default=10, help="steps averaged per table row")
    ap.add_argument("--data", default="pool", choices=["pool", "periodic"])
    ap.add_argument("--out", default=None, help="write the table (markdown) here as well")
    a = ap.parse_args(argv)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    kw = model_kw(a.seq_len, a.steps, a.lr, a.warmup)
    data = batches(kw["vocab"], a.batch, a.seq_len, a.steps, a.data)
    t0 = time.time()
    ours, init = run_ours(kw, data, dev)
    t1 = time.time()
    ref = run_reference(kw, data, dev, init)
    t2 = time.time()
    what = ("a random 64-token pattern repeated per row" if a.data == "periodic"
            else "rows cycling through a pool of 16 fixed random rows")
    lines = [f"113M architecture, bf16, AdamW lr {a.lr:g} (warm-up {a.warmup}, cosine), batch {a.batch} x {a.seq_len}, data = {what}; "
             f"one shared initial state; ln(vocab) = {math.log(kw['vocab']):.3f}.",
             f"Wall time: this repository {t1 - t0:.0f} s, reference {t2 - t1:.0f} s for {a.steps} steps.", "",
             "| steps | this repository | reference | difference |", "| --- | --- | --- | --- |"]
    worst = 0.0
    for lo in range(0, a.steps, a.block):
        mo = sum(ours[lo:lo + a.block]) / len(ours[lo:lo + a.block])
        if ref is None:
            lines.append(f"| {lo + 1}-{min(a.steps, lo + a.block)} | {mo:.4f} | unavailable | |")
            continue
        mr = sum(ref[lo:lo + a.block]) / len(ref[lo:lo + a.block])
        worst = max(worst, abs(mo - mr))
        lines.append(f"| {lo + 1}-{min(a.steps, lo + a.block)} | {mo:.4f} | {mr:.4f} | {mo - mr:+.4f} |")
    if ref is not None:
        lines += ["", f"First step: {ours[0]:.4f} vs {ref[0]:.4f}; last step: {ours[-1]:.4f} vs {ref[-1]:.4f}; largest "
                      f"block-mean difference {worst:.4f}."]
    text = "\n".join(lines)
    print(text)
    if a.out:
        with open(a.out, "w") as fh:
            fh.write(text + "\n")


if __name__ == "__main__":
    main()
