#!/usr/bin/env python3
"""Headline benchmark: pre-training throughput (tokens/s) of the 113M LoomFormer architecture.

Config: the 113M reference architecture (dims of the reference's ``cfg/nano.yaml``: d=768, 8x96 heads,
2 KV heads, hidden 3072, 10 layers, vocab 8192 untied, Tria window 128), bf16 compute with fp32 master
weights, micro-batch 16 x sequence 2048 per GPU (weak scaling), uniform-random token ids, random
initial weights, AdamW (``--optimizer atom`` switches both arms to ATOM).

``python bench.py --gpus N --steps K --warmup W`` prints ONE JSON line on rank 0.  ``--impl reference``
runs the unmodified reference from ``baseline/_ref`` (its own Model, kernels, DDP wrapper and training
step) on the same config.

Timing: W untimed warm-up steps, then K steps bracketed by barrier + synchronize, device-timed with
CUDA events, max over ranks.  Each step's working set (hundreds of MB of activations) is far larger
than the 126 MB L2, so no explicit flush is needed.  ``value`` times the step on device-resident
inputs; ``e2e`` repeats the measurement through the public ``TrainEngine.step`` call with the batch
copied from pinned host memory and the loss read back every step.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL_KW = dict(
    vocab=8192, tied_embeddings=False, seq_len=2048, model_dim=768, n_q_heads=8, head_dim=96,
    n_kv_heads=None, gqa_group_size=4, hidden=None, hidden_mult=4.0, layers=10, phase_sectors="head",
    residual_init="beta", activation="pvpowlu", powlu_m=3.0, phase_grad_floor=0.05, phase_grad_mode="secant",
    rope_theta=10000.0, rope_original_seq_len=1024, rope_factor=4.0, amp_dtype="bf16",
    tria_carry_enabled=True, use_cuda_tria=True, tria_gamma_max=0.80, tria_raw_gamma_init=0.25,
    tria_temporal_enabled=True, tria_temporal_auto=False, tria_temporal_window=128, tria_carrier_alpha=0.025,
    lr=2e-4, weight_decay=0.01, grad_clip=1.55, warmup_steps=1500, steps=150000, min_lr_frac=0.1, seed=1,
)
PUBLISHED_TOK_S = 27300.0     # reference README: 1x L40S, seq 1024 (other hardware; context only)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, index: int) -> None:
        self.index, self.rows, self.proc = index, [], None

    def start(self) -> None:
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "200"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self) -> None:
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        mhz = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i].lower().startswith("active")
                                                          for r in self.rows)]
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(mhz)}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--optimizer", default="adamw", choices=["adamw", "atom"])
    ap.add_argument("--model", default="113m", choices=["113m", "smol360"],
                    help="113m: the headline architecture (cfg/nano.yaml dims); smol360: cfg/smol360.yaml (SmolLM2 "
                         "transplant shape, 467M parameters), default micro-batch 8")
    ap.add_argument("--micro-batch", type=int, default=None)
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=None, help="debug only: a non-default value makes the number invalid")
    ap.add_argument("--grad-sync", default="auto", choices=["auto", "collective", "p2p", "fsdp"])
    ap.add_argument("--workload", default="pretrain", choices=["pretrain", "sft"],
                    help="sft: synthetic multi-turn chats rendered through the chat template, packed to seq_len, "
                         "assistant-only loss (a secondary benchmark; the headline metric is pretrain)")
    a = ap.parse_args()
    if a.micro_batch is None:
        a.micro_batch = 8 if a.model == "smol360" else 16
    return a


def sft_batches(vocab, micro_batch, seq_len, rank, n=4):
    """Packed SFT batches: conversations with turn lengths uniform in 16..512 rendered through chat_template.jinja,
    packed greedily to seq_len with per-segment positions and segment ids, loss on assistant spans only."""
    import tempfile
    from loomformer_paraplex_b200.data import sft as sd
    from loomformer_paraplex_b200.data.chat import ChatTemplate
    from loomformer_paraplex_b200.data.tokenizers import BPETokenizer, train_tokenizer
    import io, contextlib
    words = [f"w{i:03d}" for i in range(400)]
    with tempfile.TemporaryDirectory() as tmp, contextlib.redirect_stdout(io.StringIO()):
        path = os.path.join(tmp, "tok.json")
        train_tokenizer("", min(vocab, 2048), path, texts=[" ".join(words)] * 20)
        tok = BPETokenizer.load(path)
    chat = ChatTemplate(tok, template_path=os.path.join(ROOT, "chat_template.jinja"))
    convs = sd.synthetic_conversations(600, words, seed=17 + rank, min_len=16, max_len=512)
    pool, _, _ = sd.tokenize_examples(convs, chat, seq_len)
    packer = sd.Packer(pool, seq_len, sd.need_pad_id(tok), shuffle=True, seed=3 + rank)
    import torch
    out = []
    for _ in range(n):
        b = packer.sample_batch(micro_batch, torch.device("cpu"))
        out.append({k: (v.pin_memory() if (torch.is_tensor(v) and torch.cuda.is_available()) else v) for k, v in b.items()})
    return out


def timed_loop(torch, dist, step_fn, steps, warmup, world, before=None):
    """Warm up, then time exactly `steps` calls of step_fn on the device; max over ranks (ms per step)."""
    for _ in range(max(3, warmup)):
        step_fn()
    if before is not None:
        before()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(torch.cuda.current_device() if "CUDA_VISIBLE_DEVICES" not in os.environ else 0)
    sampler.start()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        step_fn()
    b.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    clocks = sampler.stop()
    ms = a.elapsed_time(b) / steps
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms, clocks


def emit(args, impl, ms, clocks, world, extra):
    tokens = args.micro_batch * args.seq_len * world
    value = tokens / (ms / 1000.0)
    line = {
        "metric": "train tokens/s (113M LoomFormer-Paraplex, bf16, seq 2048)", "impl": impl,
        "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": value / PUBLISHED_TOK_S, "dtype": "bf16", "data": "synthetic uniform-random tokens, random-init weights",
        "clocks": clocks,
        "config": {"model": "113M reference architecture (cfg/nano.yaml dims; BASELINE names it cfg/chk.yaml)",
                   "global_batch": args.micro_batch * world, "seq_len": args.seq_len,
                   "parallelism": (f"fsdp{world}" if getattr(args, "grad_sync", "") == "fsdp" else f"dp{world}"),
                   "grad_sync": getattr(args, "grad_sync", "auto"), "optimizer": args.optimizer,
                   "l2": "per-step working set >> 126 MB L2, no explicit flush",
                   "layers": MODEL_KW["layers"] if args.layers is None else args.layers},
    }
    if getattr(args, "model", "113m") == "smol360":
        line["metric"] = "train tokens/s (cfg/smol360.yaml, 467M LoomFormer-Paraplex, bf16, seq 2048)"
        line["config"]["model"] = "cfg/smol360.yaml (SmolLM2-360M transplant shape)"
        line["config"]["layers"] = 32 if args.layers is None else args.layers
        line["vs_baseline"] = None
    if getattr(args, "workload", "pretrain") == "sft":
        line["metric"] = "SFT train tokens/s (113M LoomFormer-Paraplex, bf16, packed chats, seq 2048)"
        line["data"] = "synthetic multi-turn chats through chat_template.jinja, packed, assistant-only loss; random-init weights"
        line["vs_baseline"] = None
    line.update(extra)
    print(json.dumps(line), flush=True)


def run_ours(args):
    import torch
    import torch.distributed as dist
    from loomformer_paraplex_b200.config import Config
    from loomformer_paraplex_b200.data.synthetic import SyntheticTokens
    from loomformer_paraplex_b200.models.loomformer import Model
    from loomformer_paraplex_b200.ops import native
    from loomformer_paraplex_b200.parallel import dist as pdist
    from loomformer_paraplex_b200.train.engine import TrainEngine

    dev, world, rank = pdist.init("cuda")
    if args.model == "smol360":
        cfg = Config.from_yaml(os.path.join(ROOT, "cfg", "smol360.yaml"))
        cfg.batch_size, cfg.seq_len, cfg.optimizer, cfg.tokenizer = args.micro_batch, args.seq_len, args.optimizer, None
        cfg.grad_checkpointing = False            # 180 GB of HBM holds the activations of 8 x 2048 tokens
        if args.layers is not None:
            cfg.layers = args.layers
    else:
        kw = dict(MODEL_KW, batch_size=args.micro_batch, seq_len=args.seq_len, optimizer=args.optimizer)
        if args.layers is not None:
            kw["layers"] = args.layers
        cfg = Config(**kw)
    torch.manual_seed(cfg.seed)
    model = Model(cfg).to(dev)
    # auto: one GPU needs no exchange; several GPUs use the fused NVLink step (reduce-scatter + optimizer + all-gather
    # over peer memory) and fall back to the NCCL all-reduce only if peer-mapped buffers cannot be set up here
    sync = ("p2p" if world > 1 else "collective") if args.grad_sync == "auto" else args.grad_sync
    try:
        engine = TrainEngine(cfg, model, dev, optimizer=args.optimizer, grad_sync=sync)
    except Exception as e:
        if args.grad_sync != "auto" or sync == "collective":
            raise
        print(f"[bench] fused NVLink step unavailable ({type(e).__name__}: {e}); using the NCCL all-reduce", file=sys.stderr)
        sync = "collective"
        torch.manual_seed(cfg.seed)
        model = Model(cfg).to(dev)
        engine = TrainEngine(cfg, model, dev, optimizer=args.optimizer, grad_sync=sync)
    args.grad_sync = sync
    state = {"i": 0}
    loss_host = torch.zeros((), dtype=torch.float32).pin_memory()
    if args.workload == "sft":
        host = sft_batches(cfg.vocab, args.micro_batch, args.seq_len, rank)
        to_dev = lambda b: {k: v.to(dev, non_blocking=True) for k, v in b.items() if torch.is_tensor(v)}
        resident = [to_dev(b) for b in host]
        h2d = sum(v.numel() * v.element_size() for v in host[0].values() if torch.is_tensor(v))

        def step_device():
            engine.step([resident[state["i"] % len(resident)]])
            state["i"] += 1

        def step_e2e():
            loss = engine.step([to_dev(host[state["i"] % len(host)])])
            state["i"] += 1
            loss_host.copy_(loss, non_blocking=True)
            torch.cuda.current_stream().synchronize()
    else:
        src = SyntheticTokens(cfg.vocab, args.micro_batch, args.seq_len, seed=cfg.seed, rank=rank, pin=True, pool=4)
        resident = [b.to(dev) for b in src.batches]
        h2d = int(src.batches[0].numel() * src.batches[0].element_size())

        def step_device():
            engine.step(resident[state["i"] % len(resident)])
            state["i"] += 1

        def step_e2e():
            loss = engine.step(src.next())
            loss_host.copy_(loss, non_blocking=True)
            torch.cuda.current_stream().synchronize()

    ms, clocks = timed_loop(torch, dist, step_device, args.steps, args.warmup, world, before=native.reset_launches)
    launches = native.launches()
    ms_e2e, _ = timed_loop(torch, dist, step_e2e, args.steps, 3, world)
    engine.check_finite(loss_host)
    from loomformer_paraplex_b200.ops import kernels
    kernels.check_status(dev)
    if rank == 0:
        tokens = args.micro_batch * args.seq_len * world
        fb = dict(getattr(engine.plan.K, "fallbacks", {})) if engine.plan is not None else {}
        emit(args, "ours", ms, clocks, world, {
            "e2e": {"value": tokens / (ms_e2e / 1000.0), "unit": "tokens/s",
                    "h2d_bytes_per_step": int(h2d),
                    "d2h_bytes_per_step": 4, "ms_per_step": ms_e2e},
            "gpu_launches": int(launches),
            "library_fallback_calls": fb, "final_loss": float(loss_host)})
    pdist.shutdown()


def run_reference(args):
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isfile(os.path.join(ref_dir, "loomformer.py")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is absent (the reference is a script "
                          "tree without setup.py/pyproject.toml; it is installed by copying it there)"}))
        return
    sys.dont_write_bytecode = True
    sys.path.insert(0, ref_dir)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    import math
    import contextlib
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F
    import loomformer as lf            # the reference's module (baseline/_ref is first on sys.path)
    from torch.nn.parallel import DistributedDataParallel as DDP

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    lf.device_auto(f"cuda:{local}")
    cfg = lf.Config.from_yaml(os.path.join(ref_dir, "cfg", "smol360.yaml" if args.model == "smol360" else "nano.yaml"))
    cfg.seq_len, cfg.batch_size, cfg.optimizer, cfg.device = args.seq_len, args.micro_batch, args.optimizer, f"cuda:{local}"
    if args.layers is not None:
        cfg.layers = args.layers
    lf.CARRY_TOKEN_ID = None
    lf.set_seed(int(cfg.seed) + 1000003 * rank)
    lf.apply_config(cfg)
    base = lf.Model(cfg).to(dev)
    model = base
    if world > 1:           # same wrapper arguments as the reference trainer
        model = DDP(base, device_ids=[local], output_device=local, find_unused_parameters=False,
                    bucket_cap_mb=64, gradient_as_bucket_view=True, static_graph=True)
    named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
    params = [p for _, p in named]
    Opt, opt_name = lf.optimizer_class_from_name(cfg.optimizer)
    nodecay = {id(base.tria_agg.pool.logit_scale_raw)} if base.tria_agg is not None else set()
    groups = {}
    for p in params:
        groups.setdefault((0.0 if id(p) in nodecay else cfg.weight_decay, 1.0), []).append(p)
    opt = Opt([{"params": ps, "weight_decay": wd, "lr_mult": mult} for (wd, mult), ps in groups.items()],
              lr=cfg.lr, weight_decay=cfg.weight_decay)
    g = torch.Generator().manual_seed(int(cfg.seed) + 1000003 * rank)
    host = [torch.randint(0, lf.VOCAB, (args.micro_batch, args.seq_len + 1), generator=g).pin_memory() for _ in range(4)]
    resident = [b.to(dev) for b in host]
    state = {"i": 0, "step": 0, "loss": 0.0}

    def nonfinite(which):
        for _, p in named:
            t = p.grad if which == "grad" else p
            if t is not None and not torch.isfinite(t.detach()).all():
                return True
        return False

    def one_step(batch):
        # body of the reference training loop (loomformer.py:5071-5170), one micro-batch per step
        opt.zero_grad(set_to_none=True)
        x, y = batch[:, :-1], batch[:, 1:]
        position_ids, attn_mask = lf.build_doc_reset_state(x, None)
        with lf.amp_autocast(dev):
            logits = model(x, attn_mask=attn_mask, position_ids=position_ids)
        loss = F.cross_entropy(logits.float().reshape(-1, lf.VOCAB), y.reshape(-1), reduction="none").mean()
        before = float(loss.detach().item())
        loss.backward()
        after = float(loss.detach().item())
        if not (math.isfinite(before) and math.isfinite(after)) or nonfinite("grad"):
            raise RuntimeError("reference arm: non-finite loss or gradient")
        if cfg.grad_clip and cfg.grad_clip > 0:
            torch.nn.utils.clip_grad_norm_(params, cfg.grad_clip)
        lr = lf.lr_at(cfg, state["step"])
        for grp in opt.param_groups:
            grp["lr"] = lr * float(grp.get("lr_mult", 1.0))
        opt.step()
        if nonfinite("param"):
            raise RuntimeError("reference arm: non-finite parameter")
        state["step"] += 1
        state["loss"] = before

    def step_device():
        one_step(resident[state["i"] % 4]); state["i"] += 1

    def step_e2e():
        one_step(host[state["i"] % 4].to(dev, non_blocking=True)); state["i"] += 1

    model.train()
    ms, clocks = timed_loop(torch, dist, step_device, args.steps, args.warmup, world)
    ms_e2e, _ = timed_loop(torch, dist, step_e2e, args.steps, 3, world)
    if rank == 0:
        tokens = args.micro_batch * args.seq_len * world
        emit(args, "reference", ms, clocks, world, {
            "e2e": {"value": tokens / (ms_e2e / 1000.0), "unit": "tokens/s",
                    "h2d_bytes_per_step": int(host[0].numel() * 8), "d2h_bytes_per_step": 8, "ms_per_step": ms_e2e},
            "gpu_launches": None, "final_loss": state["loss"],
            "note": "unmodified reference Model/DDP/optimizer from baseline/_ref; loop body replicated from its trainer"})
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gpus > 1 and world == 1:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", os.environ.get("MASTER_PORT", "29517"),
               os.path.abspath(__file__)] + sys.argv[1:]
        raise SystemExit(subprocess.call(cmd))
    if args.impl == "reference":
        try:
            run_reference(args)
        except Exception as e:          # the reference arm must never take the bench down
            if int(os.environ.get("RANK", "0")) == 0:
                print(json.dumps({"impl": "reference", "unavailable": f"{type(e).__name__}: {str(e)[:300]}"}))
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
