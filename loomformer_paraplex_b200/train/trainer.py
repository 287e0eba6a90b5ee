"""Pre-training workflow: data stream, resume (weights, optimizer, step, tokens seen, data cursor), engine, the step
loop with logging / evaluation / run-points / graceful interrupt, final checkpoint and optional full evaluation
(reference ``loomformer.py:4681-5286``).  Log lines keep the reference's content and add tokens/s."""
from __future__ import annotations

import math
import os
import time
from typing import Dict, Optional

import torch

from ..config import Config, resolve
from ..data.streams import ShardStream, doc_reset_state, make_stream
from ..data.tokenizers import build_tokenizer, special_id
from ..data.valsplit import maybe_auto_val_split
from ..models.loomformer import Model
from ..parallel import dist as pdist
from ..parallel.dist import rank0_print
from . import checkpoint as ckpt
from . import evaluate as ev
from .console import GracefulInterrupt, RunpointWatcher
from .engine import TrainEngine
from .schedule import lr_at


def big(n: int) -> str:
    return f"{int(n):,}"


def print_architecture(cfg: Config, d, device, ablation: bool, dataset: str, val_dataset: Optional[str]) -> None:
    rule = "=" * 64
    rank0_print(rule)
    rank0_print(f" LoomFormer  ·  {device}  ·  amp={cfg.amp_dtype}  ·  ablation={ablation}")
    rank0_print(rule)
    rank0_print(f"  shape    d_model={d.n}  heads={d.qh}q/{d.kvh}kv(x{d.group})  head_dim={d.hd}  layers={d.layers}")
    rank0_print(f"  ffn      hidden={d.hidden}  phase={'open' if d.open_sectors else 'head'}  attn=fused-dual-context")
    cap = "off" if d.branch_rms_cap is None else f"{d.branch_rms_cap:g}"
    rank0_print(f"  depth    readout={'per-sublayer' if d.depth_readout_per_sublayer else 'shared'}  "
                f"qkv_rms={d.depth_qkv_rms}  branch_rms_cap={cap}")
    rank0_print(f"  memory   activation_checkpoint={'temporal-chunk' if d.grad_checkpointing else 'off'}")
    rank0_print(f"  rope     yarn  theta={d.rope_theta:g}  factor={d.rope_factor:g}x  orig_len={d.rope_original_seq_len}")
    if d.hd < 8:
        rank0_print(f"  WARNING: head_dim={d.hd} is extremely small for LM attention.")
    rank0_print(f"  data     {dataset}")
    rank0_print(f"  val      {val_dataset}" if val_dataset else "  val      (none -- training loss only)")


def train(cfg: Config, dataset: str, device: torch.device, ckpt_out: Optional[str], ablation: bool = False,
          resume: Optional[str] = None, resume_step: Optional[int] = None, grad_sync: str = "collective",
          stream=None, max_seconds: Optional[float] = None) -> Dict[str, float]:
    world, rank = pdist.world_size(), pdist.rank()
    torch.manual_seed(int(cfg.seed) + 1000003 * rank)
    import random
    import numpy as np
    random.seed(int(cfg.seed) + 1000003 * rank); np.random.seed((int(cfg.seed) + 1000003 * rank) % (2 ** 32))
    cfg.train_dataset = dataset
    tok, carry_id = build_tokenizer(cfg)
    ckpt.report_tria_geometry(cfg, resume)
    if stream is None:
        if pdist.is_main():
            maybe_auto_val_split(cfg, dataset)
        pdist.barrier()
        if not pdist.is_main() and not cfg.val_dataset:
            maybe_auto_val_split(cfg, dataset)
    val_dataset = str(cfg.val_dataset).strip() if cfg.val_dataset else None
    own_stream = stream is None
    if stream is None:
        stream = make_stream(dataset, cfg, device, tokenizer=tok)

    start_step, tokens_seen, blob = 0, 0, {}
    if resume:
        blob = torch.load(resume, map_location="cpu", weights_only=True)
        start_step = int(resume_step if resume_step is not None else (blob.get("step") or 0))
        if resume_step is None and blob.get("step") is None:
            rank0_print(f"[resume] WARNING: {resume!r} has no saved 'step' (older checkpoint) -- defaulting to "
                        "start_step=0. Pass --resume-step N to hard-set it.")
        if start_step >= int(cfg.steps):
            rank0_print(f"[resume] start_step={start_step} >= cfg.steps={cfg.steps} -- nothing to do, exiting.")
            return {"final_eval_loss": float("nan"), "best_eval_loss": float("nan"), "full_eval_loss": float("nan"),
                    "full_eval_bpb": float("nan"), "seconds": 0.0, "skipped": 1.0, "start_step": float(start_step)}
        tokens_seen, exact = ckpt.tokens_seen_of(blob, start_step)
        rank0_print(f"[resume] restored cumulative tokens_seen={big(tokens_seen)}" if exact else
                    f"[resume] checkpoint has no tokens_seen; estimated {big(tokens_seen)} processed tokens "
                    "from its saved step/batch/sequence config.")
        replay, why = ckpt.should_replay_data(cfg, dataset, blob.get("cfg", {}))
        rank0_print(f"[resume] data cursor policy: {why}.")
        accum = max(1, int(cfg.grad_accum_steps or 1))
        if replay and start_step > 0:
            rank0_print(f"[resume] fast-forwarding the data stream by {start_step * accum} batch draws "
                        f"(start_step={start_step} * grad_accum_steps={accum}) to skip already-seen data...")
            stream.fast_forward(start_step * accum)
            rank0_print("[resume] fast-forward done.")
        elif start_step > 0:
            rank0_print("[resume] restarting data stream while preserving checkpoint step/LR schedule.")
        rank0_print(f"[resume] continuing from step {start_step}/{cfg.steps} -- LR schedule/log step numbering continue.")
    stream.prime()
    eval_path = val_dataset or dataset
    same_eval = os.path.abspath(eval_path) == os.path.abspath(dataset)
    eval_stream = stream if same_eval else make_stream(eval_path, cfg, device, tokenizer=tok)
    eos_id = getattr(stream, "eos_id", None) if cfg.doc_reset_attn else None
    eval_eos = getattr(eval_stream, "eos_id", None) if cfg.doc_reset_attn else None
    train_bpt = ev.ensure_bytes_per_token(dataset, cfg, tok, 4096) if os.path.exists(dataset) else 1.0
    eval_bpt = train_bpt if same_eval else ev.ensure_bytes_per_token(eval_path, cfg, tok, None)
    pdist.barrier()
    rank0_print("[data] all ranks ready")

    dims = resolve(cfg)
    print_architecture(cfg, dims, device, ablation, dataset, val_dataset)
    tag = "LoomFormer-ablation-s1" if ablation else "LoomFormer-paraplex"
    model = Model(cfg, ablation=ablation, dims=dims)
    model.carry_token_id = carry_id
    if pdist.is_main() and os.path.exists(dataset):
        try:
            data_tokens = ev.dataset_token_count(dataset, cfg, tok)
            gbs = int(getattr(cfg, "_global_batch_size", cfg.batch_size))
            per_step = gbs * int(cfg.seq_len) * max(1, int(cfg.grad_accum_steps or 1))
            run_tokens = max(0, int(cfg.steps) - start_step) * per_step
            label = "budget" if start_step == 0 else "remaining"
            print(f"  {label:<10}{big(run_tokens)} tokens over {max(0, int(cfg.steps) - start_step):,} steps "
                  f"({run_tokens / max(1, data_tokens):.3f} epochs of {big(data_tokens)})")
            n_par = model.num_params()
            print(f"           paraplex: {big(n_par)} params  ·  {run_tokens / max(1, n_par):.1f} tok/param  ·  "
                  f"{data_tokens / max(1, n_par):.1f} data-tok/param")
        except Exception as exc:          # budget display is informational only
            print(f"  budget   (unavailable: {exc})")
    rank0_print("=" * 64)
    model = model.to(device)
    if resume:
        ckpt.load_model_blob(model, blob, ablation)
        rank0_print(f"[resume] loaded paraplex weights from {resume}")
    if cfg.save_initial_checkpoint and resume:
        raise ValueError("save_initial_checkpoint requires a fresh run without resume")
    engine = TrainEngine(cfg, model, device, grad_sync=grad_sync)
    if world > 1:
        rank0_print(f"[ddp] world_size={world} grad_sync={grad_sync} flat_buffer={big(engine.flat.total)} elements")
    engine.step_idx = start_step
    opt_name = engine.opt_name
    if resume:
        ckpt.restore_optimizer(engine.opt, blob, opt_name, resume)

    def save(path: Optional[str] = None, step_override: Optional[int] = None) -> None:
        if not ckpt_out:
            return
        opt_obj = engine.checkpoint_view()          # collective in sharded mode: every rank takes part
        if pdist.is_main():
            p = path or ckpt_out
            ckpt.save_checkpoint(p, cfg, model, opt_obj, opt_name, step if step_override is None else step_override,
                                 tokens_seen, ablation)
            print(f"[train] saved {tag} -> {p}")

    def save_runpoint(at: int) -> None:
        if not ckpt_out:
            return
        root, ext = os.path.splitext(ckpt_out)
        ext = ext or ".pt"
        if cfg.runpoints_path:
            os.makedirs(cfg.runpoints_path, exist_ok=True)
            p = os.path.join(cfg.runpoints_path, f"{os.path.basename(root)}.runpoint_step{at}{ext}")
        else:
            p = f"{root}.runpoint_step{at}{ext}"
        rank0_print(f"\n[runpoint] step {at}/{cfg.steps} -- saving, training continues.", flush=True)
        save(p, at)

    if cfg.save_initial_checkpoint and ckpt_out:
        root, ext = os.path.splitext(ckpt_out)
        opt_obj = engine.checkpoint_view()          # collective in the fused / sharded modes: every rank takes part
        if pdist.is_main():
            ckpt.save_checkpoint(f"{root}.init{ext or '.pt'}", cfg, model, opt_obj, opt_name, 0, 0, ablation)
            print(f"[train] saved initial {tag} with optimizer state -> {root}.init{ext or '.pt'}")

    note = f"{train_bpt:.3f} bytes/token" if same_eval else f"{train_bpt:.3f} train bytes/token  ·  {eval_bpt:.3f} eval bytes/token"
    rank0_print(f"--- {tag}: {model.num_params():,} params  ·  optimizer={opt_name}  ·  {note} ---")
    t0 = time.time()
    final_eval, best_eval = float("nan"), float("inf")
    accum = max(1, int(cfg.grad_accum_steps or 1))
    log_every = max(1, int(cfg.log_every))
    eval_every = log_every if cfg.eval_every is None else max(1, int(cfg.eval_every))
    data_wait, step, tokens_at_log, t_log = 0.0, start_step, tokens_seen, time.time()
    # multi-rank runs: notice a rank that disappeared on the host, before the next launch, instead of inside a
    # collective (LOOM_HEARTBEAT=0 turns the check off)
    hb = None
    if world > 1 and os.environ.get("LOOM_HEARTBEAT", "1") != "0":
        from ..parallel.health import Heartbeat
        hb = Heartbeat(interval=1.0, max_silence=float(os.environ.get("LOOM_HEARTBEAT_SILENCE", "90")))
    ctl = pdist.StepControl(device)
    stop_now = False
    with GracefulInterrupt() as intr, RunpointWatcher() as rp:
        for step in range(start_step + 1, int(cfg.steps) + 1):
            if hb is not None:
                hb.check()
            # rank 0 decides, every rank acts: a checkpoint is a collective, so the keyboard, Ctrl-C and the wall
            # clock of one rank must never send that rank into it alone
            bits = ctl.agree((ctl.INTERRUPT if intr.requested else 0) | (ctl.RUNPOINT if rp.consume() else 0) |
                             (ctl.STOP if stop_now else 0))
            if bits & ctl.STOP:
                step -= 1
                break
            if bits & ctl.INTERRUPT:
                flag = 0
                if pdist.is_main():
                    print(f"\n[interrupt] Ctrl-C at step {step}/{cfg.steps} ({tag}, {time.time() - t0:.0f}s elapsed).", flush=True)
                    rp.pause()
                    try:
                        flag = 1 if input("[interrupt] save a checkpoint at this step before exiting? [y/N] ").strip().lower() in ("y", "yes") else 0
                    except EOFError:
                        flag = 0
                    finally:
                        rp.resume()
                flag = pdist.broadcast_int(flag, device)
                if flag:
                    save(step_override=step - 1)
                    rank0_print("[interrupt] saved.")
                else:
                    rank0_print("[interrupt] not saving -- exiting without a checkpoint.")
                pdist.barrier()
                pdist.shutdown()
                raise SystemExit(130)
            if bits & ctl.RUNPOINT:
                save_runpoint(step - 1)
            w0 = time.time()
            micro = [stream.next_batch() for _ in range(accum)]
            data_wait += time.time() - w0
            packed = []
            for mb in micro:
                mb = engine.to_device(mb)
                pos, seg = doc_reset_state(mb[:, :-1], eos_id)
                packed.append({"x": mb[:, :-1], "y": mb[:, 1:], "position_ids": pos if seg is not None else None,
                               "segment_ids": seg})
            loss = engine.step(packed)
            tokens_step = sum(int(b[:, 1:].numel()) for b in micro)
            if step == 1 or step % log_every == 0 or step == int(cfg.steps):
                engine.check_finite(loss)
                train_loss = pdist.mean_float(float(loss), device)
                refeeds = pdist.sum_int(int(engine.last_fire_count), device)
                engine.last_fire_count.zero_()
            tokens_seen += tokens_step * world
            if step == 1 or step % log_every == 0:
                elapsed = time.time() - t0
                wait_pct = 100.0 * data_wait / elapsed if elapsed > 0 else 0.0
                lr = lr_at(cfg, step - 1)
                tps = (tokens_seen - tokens_at_log) / max(1e-9, time.time() - t_log)
                tokens_at_log, t_log = tokens_seen, time.time()
                tail = (f"refeeds: {refeeds:d}  lr {lr:.2e}  tokens {big(tokens_seen)}  tok/s {tps:,.0f}  "
                        f"data_wait {data_wait:.0f}s({wait_pct:.0f}%)  ({elapsed:.0f}s)")
                if step == 1 or step % eval_every == 0:
                    final_eval = pdist.mean_float(ev.sampled_eval_loss(model, eval_stream, cfg, eval_eos), device)
                    best_eval = min(best_eval, final_eval)
                    bits, bpb = ev.loss_to_bits(final_eval, eval_bpt)
                    rank0_print(f"[{tag}] step {step:6d}  train_loss {train_loss:.4f}  eval_loss {final_eval:.4f}  "
                                f"bits/tok {bits:.4f}  bpb {bpb:.4f}  {tail}")
                else:
                    rank0_print(f"[{tag}] step {step:6d}  train_loss {train_loss:.4f}  {tail}")
            if cfg.save_every and step % int(cfg.save_every) == 0:
                save_runpoint(step)
            if max_seconds is not None and time.time() - t0 > max_seconds:
                if world == 1:
                    break
                stop_now = True                     # published by rank 0 before the next step; all ranks leave together
    seconds = time.time() - t0
    save()
    out = {"final_eval_loss": final_eval, "best_eval_loss": best_eval, "full_eval_loss": float("nan"),
           "full_eval_bpb": float("nan"), "seconds": seconds, "final_train_loss": float(loss)}
    if val_dataset:
        full = ev.eval_full_model(model, cfg, val_dataset, device, tok)
        out["full_eval_loss"] = pdist.mean_float(full["loss_nats"], device)
        out["full_eval_bpb"] = pdist.mean_float(full["bpb"], device)
        rank0_print(f"[{tag}] full_eval {val_dataset}  eval_loss {out['full_eval_loss']:.4f}  "
                    f"bits/tok {full['bits_tok']:.4f}  bpb {out['full_eval_bpb']:.4f}  tokens {int(full['total_tokens'])}")
    if own_stream:
        stream.close()
    return out
