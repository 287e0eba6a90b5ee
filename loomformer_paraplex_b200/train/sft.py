"""Supervised fine-tuning workflow (reference ``loomsft.py:354-499`` is single-device; this one also runs under
``torch.distributed`` with per-rank packers and the same gradient paths as pre-training).  Loss is taken on
assistant spans only; packed examples are isolated by per-token segment ids."""
from __future__ import annotations

import os
import time
from typing import Optional

import torch

from ..config import Config, resolve
from ..data import sft as sd
from ..data.chat import ChatTemplate
from ..data.tokenizers import build_tokenizer
from ..models.loomformer import Model
from ..parallel import dist as pdist
from ..parallel.dist import rank0_print
from . import checkpoint as ckpt
from .console import GracefulInterrupt, RunpointWatcher
from .engine import TrainEngine
from .schedule import lr_at


@torch.no_grad()
def eval_sft(model, packer: sd.Packer, batch_size: int, device, n_batches: int = 8) -> float:
    from .evaluate import model_nll
    was = model.training
    model.eval()
    tot, ntok = 0.0, 0
    for _ in range(n_batches):
        b = packer.sample_batch(batch_size, device)
        nll, n = model_nll(model, b["x"], b["y"], b["segment_ids"], b["position_ids"])
        tot += float(nll); ntok += n
    model.train(was)
    return tot / max(1, ntok)


def train_sft(cfg: Config, train_path: str, val_path: Optional[str], init_checkpoint: Optional[str], device,
              ckpt_out: str, resume: Optional[str] = None, resume_step: Optional[int] = None,
              grad_sync: str = "collective", pool=None, tokenizer=None) -> dict:
    world, rank = pdist.world_size(), pdist.rank()
    torch.manual_seed(cfg.seed)
    tok = tokenizer
    carry = None
    if tok is None:
        tok, carry = build_tokenizer(cfg)
    source = resume or init_checkpoint
    ckpt.report_tria_geometry(cfg, source)
    dims = resolve(cfg)
    chat = ChatTemplate(tok)
    pad_id = sd.need_pad_id(tok)
    start = 0
    blob = None
    if resume:
        blob = torch.load(resume, map_location="cpu", weights_only=True)
        start = int(resume_step if resume_step is not None else (blob.get("step") or 0))
        if start >= int(cfg.steps):
            print(f"[resume] start_step={start} >= cfg.steps={cfg.steps} -- nothing to do, exiting.")
            return {"skipped": 1.0}
    model = Model(cfg, dims=dims).to(device)
    model.carry_token_id = carry
    if source:
        ckpt.load_model_checkpoint(model, source, ablation=False, device=device)
    train_pool = pool if pool is not None else sd.preprocess_dataset(train_path, chat, cfg.seq_len, verbose=pdist.is_main())
    packer = sd.Packer(train_pool, cfg.seq_len, pad_id, shuffle=True, seed=cfg.seed + 7919 * rank)
    val_packer = None
    if val_path:
        val_packer = sd.Packer(sd.preprocess_dataset(val_path, chat, cfg.seq_len, verbose=pdist.is_main()), cfg.seq_len,
                               pad_id, shuffle=False, seed=cfg.seed)
    if pdist.is_main():
        rule = "=" * 64
        print(rule); print(f" LoomSFT  ·  {device}  ·  amp={cfg.amp_dtype}  ·  init={source}  ·  ranks={world}"); print(rule)
        print(f"  shape    d_model={dims.n}  heads={dims.qh}q/{dims.kvh}kv(x{dims.group})  head_dim={dims.hd}  layers={dims.layers}")
        print(f"  train    {train_path}")
        print(f"  val      {val_path}" if val_path else "  val      (none -- training loss only)")
        pool_tok = int(sum(len(e.ids) for e in train_pool)); loss_tok = int(sum(int(e.mask.sum()) for e in train_pool))
        accum0 = max(1, int(cfg.grad_accum_steps or 1))
        run_tok = int(cfg.steps) * int(cfg.batch_size) * world * int(cfg.seq_len) * accum0
        print(f"  budget   {run_tok:,} tokens over {cfg.steps:,} steps ({run_tok / max(1, pool_tok):.3f} epochs of "
              f"{pool_tok:,} pool tokens, {len(train_pool):,} examples)")
        print(f"           pool: {loss_tok:,} loss-carrying tokens ({loss_tok / max(1, pool_tok):.1%} of pool)")
        print(rule)
    accum = max(1, int(cfg.grad_accum_steps or 1))
    if resume and start > 0:
        n = start * accum * int(cfg.batch_size)
        rank0_print(f"[resume] fast-forwarding Packer RNG by {n} row draws to skip already-seen data...")
        packer.fast_forward(n)
        rank0_print(f"[resume] continuing from step {start}/{cfg.steps} -- LR schedule/log step numbering continue.")
    engine = TrainEngine(cfg, model, device, grad_sync=grad_sync, train_lr=False)
    engine.step_idx = start
    if resume:
        ckpt.restore_optimizer(engine.opt, blob, engine.opt_name, resume)

    def save(path: Optional[str], at: int) -> None:
        opt_obj = engine.checkpoint_view()          # collective in sharded mode: every rank takes part
        if pdist.is_main():
            ckpt.save_checkpoint(path or ckpt_out, cfg, model, opt_obj, engine.opt_name, at, 0)
            print(f"[loomsft] saved -> {path or ckpt_out}")

    def runpoint(at: int) -> None:
        root, ext = os.path.splitext(ckpt_out)
        ext = ext or ".pt"
        if cfg.runpoints_path:
            os.makedirs(cfg.runpoints_path, exist_ok=True)
            p = os.path.join(cfg.runpoints_path, f"{os.path.basename(root)}.runpoint_step{at}{ext}")
        else:
            p = f"{root}.runpoint_step{at}{ext}"
        rank0_print(f"\n[runpoint] step {at}/{cfg.steps} -- saving, training continues.")
        save(p, at)

    pre = sd.BatchPrefetcher(packer, cfg.batch_size, device, depth=max(2, accum // 4 + 1))
    step, t0, loss = start, time.time(), None
    try:
        ctl = pdist.StepControl(device)
        with GracefulInterrupt() as intr, RunpointWatcher() as rp:
            while step < int(cfg.steps):
                loss = engine.step([pre.next() for _ in range(accum)])
                # rank 0's keyboard and Ctrl-C decide for every rank (saving is a collective)
                bits = ctl.agree((ctl.INTERRUPT if intr.requested else 0) | (ctl.RUNPOINT if rp.consume() else 0))
                if step % max(1, int(cfg.log_every)) == 0:
                    engine.check_finite(loss)
                    tl = pdist.mean_float(float(loss), device)
                    trias = pdist.sum_int(int(engine.last_fire_count), device)
                    engine.last_fire_count.zero_()
                    msg = (f"[loomsft] step {step:6d}  train_loss {tl:.4f}  trias: {trias:d}  lr {lr_at(cfg, step):.2e}  "
                           f"({time.time() - t0:.0f}s)")
                    if val_packer is not None and step % (max(1, int(cfg.log_every)) * 5) == 0:
                        msg += f"  eval_loss {eval_sft(model, val_packer, cfg.batch_size, device):.4f}"
                    rank0_print(msg)
                if (bits & ctl.RUNPOINT) or (cfg.save_every and (step + 1) % int(cfg.save_every) == 0):
                    runpoint(step + 1)
                if bits & ctl.INTERRUPT:
                    rank0_print(f"\n[interrupt] Ctrl-C at step {step}/{cfg.steps} -- saving a runpoint and stopping.")
                    runpoint(step + 1)
                    step += 1
                    break
                step += 1
    finally:
        pre.stop()
    save(None, step)
    return {"final_train_loss": float(loss) if loss is not None else float("nan"), "steps": step}
