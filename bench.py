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
    ap.add_argument("--secondary", default="auto", choices=["auto", "on", "off"],
                    help="after the headline, measure the other benchmark configurations in the same process and report "
                         "them under 'secondary' (smol360 training, decode at batch 1 and 64, SFT); auto: on for the "
                         "default headline run")
    ap.add_argument("--secondary-budget", type=float, default=240.0,
                    help="wall-clock seconds the secondary measurements may take in total; what does not fit is "
                         "reported as unavailable")
    ap.add_argument("--workload", default="pretrain", choices=["pretrain", "sft"],
                    help="sft: synthetic multi-turn chats rendered through the chat template, packed to seq_len, "
                         "assistant-only loss (a secondary benchmark; the headline metric is pretrain)")
    a = ap.parse_args()
    if a.micro_batch is None:
        a.micro_batch = 8 if a.model == "smol360" else 16
    if a.secondary == "auto":
        a.secondary = "on" if (a.model == "113m" and a.workload == "pretrain" and a.layers is None) else "off"
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
                   "parallelism": f"dp{world}", "optimizer": args.optimizer,
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


def make_cfg(args, model_name):
    from loomformer_paraplex_b200.config import Config
    if model_name == "smol360":
        cfg = Config.from_yaml(os.path.join(ROOT, "cfg", "smol360.yaml"))
        cfg.batch_size, cfg.seq_len, cfg.optimizer, cfg.tokenizer = args.micro_batch, args.seq_len, args.optimizer, None
        cfg.grad_checkpointing = False            # 180 GB of HBM holds the activations of 8 x 2048 tokens
        if args.layers is not None:
            cfg.layers = args.layers
        return cfg
    kw = dict(MODEL_KW, batch_size=args.micro_batch, seq_len=args.seq_len, optimizer=args.optimizer)
    if args.layers is not None:
        kw["layers"] = args.layers
    return Config(**kw)


def make_engine(args, cfg, dev, world):
    """Model + engine.  auto: one GPU needs no exchange; several GPUs use the fused NVLink step (reduce-scatter +
    optimizer + all-gather over peer memory) and fall back to the NCCL all-reduce only if peer-mapped buffers cannot
    be set up here.  Returns (engine, name of the gradient path)."""
    import torch
    from loomformer_paraplex_b200.models.loomformer import Model
    from loomformer_paraplex_b200.train.engine import TrainEngine
    sync = ("p2p" if world > 1 else "collective") if args.grad_sync == "auto" else args.grad_sync
    torch.manual_seed(cfg.seed)
    model = Model(cfg).to(dev)
    try:
        return TrainEngine(cfg, model, dev, optimizer=args.optimizer, grad_sync=sync), sync
    except Exception as e:
        if args.grad_sync != "auto" or sync == "collective":
            raise
        print(f"[bench] fused NVLink step unavailable ({type(e).__name__}: {e}); using the NCCL all-reduce", file=sys.stderr)
        torch.manual_seed(cfg.seed)
        model = Model(cfg).to(dev)
        return TrainEngine(cfg, model, dev, optimizer=args.optimizer, grad_sync="collective"), "collective"


def measure_training(args, cfg, engine, dev, world, rank, workload, steps, warmup):
    """Device-timed and end-to-end step time of `engine` on `workload`; returns a dict of raw figures."""
    import torch
    import torch.distributed as dist
    from loomformer_paraplex_b200.data.synthetic import SyntheticTokens
    from loomformer_paraplex_b200.ops import kernels, native
    state = {"i": 0}
    loss_host = torch.zeros((), dtype=torch.float32).pin_memory()
    if workload == "sft":
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

    ms, clocks = timed_loop(torch, dist, step_device, steps, warmup, world, before=native.reset_launches)
    launches = native.launches()
    ms_e2e, _ = timed_loop(torch, dist, step_e2e, steps, 3, world)
    engine.check_finite(loss_host)
    kernels.check_status(dev)
    fb = dict(getattr(engine.plan.K, "fallbacks", {})) if engine.plan is not None else {}
    return {"ms": ms, "ms_e2e": ms_e2e, "clocks": clocks, "launches": int(launches), "h2d": int(h2d),
            "fallbacks": fb, "loss": float(loss_host), "peak_gb": torch.cuda.max_memory_allocated(dev) / 2 ** 30}


def measure_decode(cfg_kw, dev, world, batch, prompt_len, new):
    """Greedy decode under CUDA-graph replay: `batch` prompts of `prompt_len` uniform-random tokens, `new` steps.
    One replica per rank; device-timed, max over ranks; tokens/s summed over replicas."""
    import torch
    import torch.distributed as dist
    from loomformer_paraplex_b200.config import Config
    from loomformer_paraplex_b200.models.loomformer import Model
    from loomformer_paraplex_b200.serve.decode import DecodeEngine
    cfg = Config(**cfg_kw)
    torch.manual_seed(1)
    model = Model(cfg).to(dev).eval()
    eng = DecodeEngine(model, batch=batch, max_len=prompt_len + new + 1, use_graph=True)
    g = torch.Generator(device="cpu").manual_seed(5 + int(os.environ.get("RANK", "0")))
    prompt_host = torch.randint(0, cfg.vocab, (batch, prompt_len), generator=g).pin_memory()
    prompt = prompt_host.to(dev)
    for _ in range(3):                                        # warm-up incl. graph capture
        eng.generate(prompt, 4)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    e0.record()
    logits = eng.prefill(prompt)
    tok = logits.argmax(-1)
    e1.record()
    for _ in range(new):
        eng.step(tok)
        tok = eng.next_tok
    e2.record()
    torch.cuda.synchronize()
    # end to end through the public call: prompt from pinned host memory, generated ids back to the host
    t0 = time.perf_counter()
    out = eng.generate(prompt_host.to(dev, non_blocking=True), new).cpu()
    wall = time.perf_counter() - t0
    t = torch.tensor([e0.elapsed_time(e1), e1.elapsed_time(e2), wall * 1e3], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    pre_ms, dec_ms, e2e_ms = (float(x) for x in t.tolist())
    del eng, model
    return {"replicas": world, "batch_per_replica": batch, "prompt": prompt_len, "new": new,
            "prefill_tok_s": world * batch * prompt_len / (pre_ms / 1e3),
            "decode_tok_s": world * batch * new / (dec_ms / 1e3), "ms_per_decode_step": dec_ms / new,
            "e2e_generate_tok_s": world * batch * new / (e2e_ms / 1e3),
            "h2d_bytes": int(prompt_host.numel() * 8), "d2h_bytes": int(out.numel() * 8),
            "unit": "tokens/s", "graph_replay": True}


def measure_tp_ops(dev, world, rank):
    """The two fused tensor-parallel GEMMs over all ranks of the job on the 113M FFN shape (2048 tokens): all-gather of
    the row-sharded activations inside the column-parallel up-projection, reduce-scatter inside the row-parallel
    down-projection's epilogue.  Device-timed with the bracketing barriers, max over ranks; roofline = the slower of
    the per-rank FLOPs at the measured GEMM peak and the bytes that cross NVLink at 770 GB/s per direction."""
    import torch
    import torch.distributed as dist
    from loomformer_paraplex_b200.ops import kernels
    from loomformer_paraplex_b200.parallel.tp import TensorParallel
    tp = TensorParallel(device=dev)
    M, K, H = 2048, 768, 3072
    per, hl = M // world, H // world
    g = torch.Generator(device="cpu").manual_seed(11)
    x_rows = torch.randn(per, K, generator=g).to(torch.bfloat16).to(dev)
    w_up = (torch.randn(hl, K, generator=g) * 0.03).to(torch.bfloat16).to(dev)
    w_dn = (torch.randn(K, hl, generator=g) * 0.03).to(torch.bfloat16).to(dev)
    o_l = torch.randn(M, hl, generator=g).to(torch.bfloat16).to(dev)

    def timed(fn, iters=20):
        for _ in range(3):
            fn()
        torch.cuda.synchronize(); dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record(); torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)
    t_up = timed(lambda: tp.column_parallel("x", x_rows, w_up, M))
    t_dn = timed(lambda: tp.row_parallel("z", o_l, w_dn))
    kernels.check_status(dev)
    peak = 1608.7e12
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            peak = float(json.load(fh)["bf16_tflops"]) * 1e12
    except Exception:
        pass
    flops = 2.0 * M * K * hl
    up_bytes, dn_bytes = (world - 1) * per * K * 2, (world - 1) * per * K * 4
    roof_up = max(flops / peak, up_bytes / 770e9) * 1e3
    roof_dn = max(flops / peak, dn_bytes / 770e9) * 1e3
    return {"world": world, "shape": "2048 tokens, 768 -> 3072/world -> 768", "ms_all_gather_up_gemm": t_up,
            "ms_down_gemm_reduce_scatter": t_dn, "roofline_ms": [roof_up, roof_dn],
            "fraction_of_roofline": [roof_up / t_up, roof_dn / t_dn],
            "note": "op-level: the model itself is not tensor-parallel"}


class LineGuard:
    """Guarantees that the one JSON line is printed.  The secondary measurements run after the headline; should one of
    them block (a rank lost inside a collective), a timer prints the headline with whatever secondary results exist,
    marks the line, and ends the process, instead of leaving the caller without a number."""

    def __init__(self, rank, limit_s, emit_fn):
        self.rank, self.emit_fn, self.done = rank, emit_fn, threading.Lock()
        self.timer = threading.Timer(limit_s, self._expire)
        self.timer.daemon = True
        self.timer.start()

    def _expire(self):
        if self.done.acquire(blocking=False):
            if self.rank == 0:
                self.emit_fn(True)
            sys.stdout.flush()
            os._exit(0)

    def finish(self):
        if self.done.acquire(blocking=False):
            self.timer.cancel()
            if self.rank == 0:
                self.emit_fn(False)


def secondary_ours(args, dev, world, rank, deadline, out):
    """The benchmark configurations that are not the headline, measured after it in the same process."""
    import copy
    import gc
    import torch

    def guarded(name, fn):
        skip = deadline - time.time() < 20.0
        if world > 1:
            from loomformer_paraplex_b200.parallel import dist as pdist
            skip = bool(pdist.max_float(1.0 if skip else 0.0, dev) > 0.5)       # one decision for all ranks
        if skip:
            out[name] = {"unavailable": f"secondary time budget used up before this measurement ({args.secondary_budget:.0f}s)"}
            return
        try:
            out[name] = fn()
        except Exception as e:
            out[name] = {"unavailable": f"{type(e).__name__}: {str(e)[:200]}"}
        gc.collect()
        torch.cuda.empty_cache()

    for batch in (1, 64):
        guarded(f"decode_b{batch}", lambda: measure_decode(dict(MODEL_KW), dev, world, batch, 512, 256))
    torch.cuda.reset_peak_memory_stats(dev)

    def smol(grad_sync=None):
        a = copy.copy(args)
        a.model, a.micro_batch = "smol360", 8
        if grad_sync is not None:
            a.grad_sync = grad_sync
        cfg = make_cfg(a, "smol360")
        engine, path = make_engine(a, cfg, dev, world)
        r = measure_training(a, cfg, engine, dev, world, rank, "pretrain", 5, 3)
        tokens = a.micro_batch * a.seq_len * world
        return {"metric": "train tokens/s (cfg/smol360.yaml, 467M parameters, bf16, micro-batch 8 x seq 2048 per GPU)",
                "value": tokens / (r["ms"] / 1e3), "unit": "tokens/s", "ms_per_step": r["ms"], "steps": 5, "warmup": 3,
                "e2e_value": tokens / (r["ms_e2e"] / 1e3), "grad_path": path, "gpu_launches": r["launches"],
                "library_fallback_calls": r["fallbacks"], "final_loss": r["loss"], "peak_memory_gib": round(r["peak_gb"], 2)}
    guarded("smol360", smol)
    if world > 1:
        # sharded data parallelism (owner-only update, weights fetched from their owners inside the consuming GEMM)
        guarded("smol360_fsdp", lambda: smol("fsdp"))
        guarded("tp_fused_gemms", lambda: measure_tp_ops(dev, world, rank))

    def sft():
        a = copy.copy(args)
        cfg = make_cfg(a, "113m")
        engine, path = make_engine(a, cfg, dev, world)
        r = measure_training(a, cfg, engine, dev, world, rank, "sft", 6, 3)
        tokens = a.micro_batch * a.seq_len * world
        return {"metric": "SFT train tokens/s (113M, packed synthetic chats, assistant-only loss, seq 2048)",
                "value": tokens / (r["ms"] / 1e3), "unit": "tokens/s", "ms_per_step": r["ms"], "steps": 6, "warmup": 3,
                "e2e_value": tokens / (r["ms_e2e"] / 1e3), "grad_path": path, "gpu_launches": r["launches"],
                "library_fallback_calls": r["fallbacks"], "final_loss": r["loss"]}
    guarded("sft", sft)


def run_ours(args):
    import gc
    import torch
    from loomformer_paraplex_b200.parallel import dist as pdist

    dev, world, rank = pdist.init("cuda")
    cfg = make_cfg(args, args.model)
    engine, path = make_engine(args, cfg, dev, world)
    r = measure_training(args, cfg, engine, dev, world, rank, args.workload, args.steps, args.warmup)
    sec = {}
    tokens = args.micro_batch * args.seq_len * world

    def emit_line(aborted):
        extra = {"secondary": dict(sec)} if args.secondary == "on" else {}
        if aborted:
            extra["secondary_aborted"] = "a secondary measurement did not return in time; the headline above is complete"
        emit(args, "ours", r["ms"], r["clocks"], world, dict({
            "e2e": {"value": tokens / (r["ms_e2e"] / 1000.0), "unit": "tokens/s", "h2d_bytes_per_step": r["h2d"],
                    "d2h_bytes_per_step": 4, "ms_per_step": r["ms_e2e"]},
            "gpu_launches": r["launches"], "grad_path": path, "peak_memory_gib": round(r["peak_gb"], 2),
            "library_fallback_calls": r["fallbacks"], "final_loss": r["loss"]}, **extra))

    guard = LineGuard(rank, args.secondary_budget + 150.0, emit_line)
    if args.secondary == "on":
        del engine
        gc.collect()
        torch.cuda.empty_cache()
        secondary_ours(args, dev, world, rank, time.time() + args.secondary_budget, sec)
    guard.finish()
    pdist.shutdown()


def reference_dir():
    """Where the unmodified reference tree lives.  Its own loader rebuilds an extension whenever the absolute source
    paths recorded in its ninja files change, so when those files name a path that still points at this tree (a
    symbolic link to the same folder) that path is used: the pre-built objects are then reused instead of compiled
    again (several minutes per fresh machine otherwise)."""
    here = os.path.join(ROOT, "baseline", "_ref")
    ninja = os.path.join(here, "kernels", "build", "loomformer_pvpowlu", "build.ninja")
    try:
        with open(ninja) as fh:
            for line in fh:
                if "cuda_compile" in line and line.startswith("build "):
                    built = line.split("cuda_compile", 1)[1].strip()
                    cand = built.split(os.sep + "kernels" + os.sep)[0]
                    if os.path.isdir(cand) and os.path.samefile(cand, here):
                        return cand
    except OSError:
        pass
    return here


def adopt_reference_toolchain(ref_dir):
    """The command lines in the reference's ninja files name the host compiler its extensions were built with (torch
    takes it from CC / CXX) and the GPU target (from TORCH_CUDA_ARCH_LIST).  With different values in the environment
    every command line changes and ninja compiles everything again (about a minute per extension), so the recorded
    values are put back into the environment; the compilers only when they exist here."""
    ninja = os.path.join(ref_dir, "kernels", "build", "loomformer_pvpowlu", "build.ninja")
    try:
        with open(ninja) as fh:
            text = fh.read()
    except OSError:
        return
    for line in text.splitlines():
        if line.startswith("cxx = "):
            cxx = line.split("=", 1)[1].strip()
            if os.path.isfile(cxx):
                os.environ["CXX"] = cxx
        if line.startswith("cuda_cflags = ") and "-ccbin " in line:
            cc = line.split("-ccbin ", 1)[1].split()[0]
            if os.path.isfile(cc):
                os.environ["CC"] = cc
        if line.startswith("cuda_cflags = ") and "-gencode=arch=compute_" in line:
            # the target the objects were compiled for: torch derives the -gencode flag from TORCH_CUDA_ARCH_LIST, and a
            # value inherited from the environment (e.g. 10.0a instead of 10.0) changes every nvcc command line
            arch = line.split("-gencode=arch=compute_", 1)[1].split(",")[0]          # "100" or "100a"
            digits = "".join(ch for ch in arch if ch.isdigit())
            suffix = arch[len(digits):]
            if len(digits) >= 2:
                os.environ["TORCH_CUDA_ARCH_LIST"] = f"{digits[:-1]}.{digits[-1]}{suffix}"


def settle_reference_mtimes(ref_dir):
    """A copy of the tree to another machine may scramble file times; ninja compares them.  Order them the way a
    finished build leaves them (sources < objects < libraries).  File contents are untouched."""
    kdir = os.path.join(ref_dir, "kernels")
    now = time.time()
    try:
        for base, dirs, files in os.walk(kdir):
            in_build = os.sep + "build" in base[len(kdir):]
            for f in files:
                path = os.path.join(base, f)
                if not in_build:
                    stamp = now - 3 * 86400
                elif f.endswith(".o"):
                    stamp = now - 2 * 86400
                elif f.endswith(".so"):
                    stamp = now - 86400
                else:
                    continue
                os.utime(path, (stamp, stamp))
    except OSError:
        pass


def run_reference(args):
    ref_dir = reference_dir()
    if not os.path.isfile(os.path.join(ref_dir, "loomformer.py")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is absent (the reference is a script "
                          "tree without setup.py/pyproject.toml; it is installed by copying it there)"}))
        return
    sys.dont_write_bytecode = True
    sys.path.insert(0, ref_dir)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    adopt_reference_toolchain(ref_dir)
    if int(os.environ.get("LOCAL_RANK", "0")) == 0:
        settle_reference_mtimes(ref_dir)
    import math
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F
    t_start = time.time()
    import loomformer as lf            # the reference's module (baseline/_ref is first on sys.path)
    from torch.nn.parallel import DistributedDataParallel as DDP

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl")
        dist.barrier(device_ids=[local])        # rank 0 of the node has settled the file times
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    lf.device_auto(f"cuda:{local}")

    def train_arm(model_name, micro_batch, workload, steps, warmup, deadline=None):
        """Body of the reference training loop (loomformer.py:5071-5170) on its own Model, DDP wrapper and optimizer."""
        cfg = lf.Config.from_yaml(os.path.join(ref_dir, "cfg", "smol360.yaml" if model_name == "smol360" else "nano.yaml"))
        cfg.seq_len, cfg.batch_size, cfg.optimizer, cfg.device = args.seq_len, micro_batch, args.optimizer, f"cuda:{local}"
        if args.layers is not None:
            cfg.layers = args.layers
        lf.CARRY_TOKEN_ID = None
        lf.set_seed(int(cfg.seed) + 1000003 * rank)
        lf.apply_config(cfg)
        if rank == 0:
            print(f"[bench] reference: extensions loaded and config applied {time.time() - t_start:.0f}s after start "
                  f"({model_name}, {workload})", file=sys.stderr, flush=True)
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
        if workload == "sft":
            packed = sft_batches(lf.VOCAB, micro_batch, args.seq_len, rank)
            host = packed
            h2d = sum(v.numel() * v.element_size() for v in host[0].values() if torch.is_tensor(v))
            put = lambda b: {k: v.to(dev, non_blocking=True) for k, v in b.items() if torch.is_tensor(v)}
        else:
            g = torch.Generator().manual_seed(int(cfg.seed) + 1000003 * rank)
            host = [torch.randint(0, lf.VOCAB, (micro_batch, args.seq_len + 1), generator=g).pin_memory() for _ in range(4)]
            h2d = int(host[0].numel() * 8)
            put = lambda b: b.to(dev, non_blocking=True)
        resident = [put(b) for b in host]
        state = {"i": 0, "step": 0, "loss": 0.0}

        def nonfinite(which):
            for _, p in named:
                t = p.grad if which == "grad" else p
                if t is not None and not torch.isfinite(t.detach()).all():
                    return True
            return False

        def one_step(batch):
            opt.zero_grad(set_to_none=True)
            if workload == "sft":          # packed rows: per-segment positions, block-diagonal causal mask, masked targets
                x, y, position_ids = batch["x"], batch["y"], batch["position_ids"]
                seg = batch["segment_ids"]
                T = x.shape[1]
                attn_mask = ((seg[:, :, None] == seg[:, None, :]) &
                             torch.ones(T, T, dtype=torch.bool, device=x.device).tril()).unsqueeze(1)
            else:
                x, y = batch[:, :-1], batch[:, 1:]
                position_ids, attn_mask = lf.build_doc_reset_state(x, None)
            with lf.amp_autocast(dev):
                logits = model(x, attn_mask=attn_mask, position_ids=position_ids)
            if workload == "sft":
                loss = F.cross_entropy(logits.float().reshape(-1, lf.VOCAB), y.reshape(-1), ignore_index=-100)
            else:
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
            one_step(put(host[state["i"] % 4])); state["i"] += 1

        model.train()
        ms, clocks = timed_loop(torch, dist, step_device, steps, warmup, world)
        ms_e2e, _ = timed_loop(torch, dist, step_e2e, steps, 3, world)
        return {"ms": ms, "ms_e2e": ms_e2e, "clocks": clocks, "h2d": h2d, "loss": state["loss"]}

    def decode_arm(batch, prompt_len, new, budget_s):
        """The reference's own decode path: Model.step token by token (it has no batched prefill), bf16 autocast."""
        kw = {k: v for k, v in MODEL_KW.items() if k in lf.Config.__dataclass_fields__}
        cfg = lf.Config(**kw)
        lf.CARRY_TOKEN_ID = None
        lf.apply_config(cfg)
        torch.manual_seed(1)
        model = lf.Model(cfg).to(dev).eval()
        g = torch.Generator(device="cpu").manual_seed(5 + rank)
        prompt = torch.randint(0, cfg.vocab, (batch, prompt_len), generator=g).to(dev)
        t_end = time.time() + budget_s
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        with torch.inference_mode(), torch.autocast("cuda", dtype=torch.bfloat16):
            st = None
            for t in range(8):
                lg, st = model.step(prompt[:, t], t, st)
            torch.cuda.synchronize()
            st, done_p, done_n = None, 0, 0
            e0.record()
            for t in range(prompt_len):
                lg, st = model.step(prompt[:, t], t, st)
                done_p += 1
                if time.time() > t_end:
                    break
            e1.record()
            tok = lg.argmax(-1)
            if done_p == prompt_len:
                for i in range(new):
                    lg, st = model.step(tok, prompt_len + i, st)
                    tok = lg.argmax(-1)
                    done_n += 1
                    if time.time() > t_end:
                        break
            e2.record()
            torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1), e1.elapsed_time(e2), float(done_p), float(done_n)], device=dev)
        if world > 1:
            mx = t.clone(); dist.all_reduce(mx, op=dist.ReduceOp.MAX)
            mn = t.clone(); dist.all_reduce(mn, op=dist.ReduceOp.MIN)
            t = torch.stack((mx[0], mx[1], mn[2], mn[3]))
        pre_ms, dec_ms, done_p, done_n = float(t[0]), float(t[1]), int(t[2]), int(t[3])
        res = {"replicas": world, "batch_per_replica": batch, "prompt": done_p, "new": done_n,
               "prefill_tok_s": world * batch * done_p / (pre_ms / 1e3), "unit": "tokens/s", "graph_replay": False,
               "note": "Model.step loop of the reference, prompt ingested token by token"}
        if done_n:
            res["decode_tok_s"] = world * batch * done_n / (dec_ms / 1e3)
            res["ms_per_decode_step"] = dec_ms / done_n
        if done_p < prompt_len or done_n < new:
            res["truncated"] = f"stopped by the {budget_s:.0f}s guard after {done_p} prompt and {done_n} new tokens"
        return res

    def agree_skip(flag):
        if world <= 1:
            return bool(flag)
        t = torch.tensor([1 if flag else 0], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return bool(t.item())

    r = train_arm(args.model, args.micro_batch, args.workload, args.steps, args.warmup)
    sec = {}
    tokens_head = args.micro_batch * args.seq_len * world

    def emit_line(aborted):
        extra = {"secondary": dict(sec)} if args.secondary == "on" else {}
        if aborted:
            extra["secondary_aborted"] = "a secondary measurement did not return in time; the headline above is complete"
        emit(args, "reference", r["ms"], r["clocks"], world, dict({
            "e2e": {"value": tokens_head / (r["ms_e2e"] / 1000.0), "unit": "tokens/s",
                    "h2d_bytes_per_step": r["h2d"], "d2h_bytes_per_step": 8, "ms_per_step": r["ms_e2e"]},
            "gpu_launches": None, "final_loss": r["loss"],
            "note": "unmodified reference Model/DDP/optimizer from baseline/_ref; loop body replicated from its trainer"},
            **extra))

    guard = LineGuard(rank, args.secondary_budget + 240.0, emit_line)
    if args.secondary == "on":
        import gc
        deadline = time.time() + args.secondary_budget

        def guarded(name, fn):
            if agree_skip(deadline - time.time() < 30.0):
                sec[name] = {"unavailable": f"secondary time budget used up before this measurement ({args.secondary_budget:.0f}s)"}
                return
            try:
                sec[name] = fn()
            except Exception as e:
                sec[name] = {"unavailable": f"{type(e).__name__}: {str(e)[:200]}"}
            gc.collect()
            torch.cuda.empty_cache()

        guarded("decode_b1", lambda: decode_arm(1, 512, 256, 45.0))
        guarded("decode_b64", lambda: decode_arm(64, 512, 256, 45.0))

        def smol():
            q = train_arm("smol360", 8, "pretrain", 3, 3)
            tokens = 8 * args.seq_len * world
            return {"metric": "train tokens/s (cfg/smol360.yaml, 467M parameters, bf16, micro-batch 8 x seq 2048 per GPU)",
                    "value": tokens / (q["ms"] / 1e3), "unit": "tokens/s", "ms_per_step": q["ms"], "steps": 3, "warmup": 3,
                    "e2e_value": tokens / (q["ms_e2e"] / 1e3), "grad_path": "its DistributedDataParallel wrapper",
                    "final_loss": q["loss"], "note": "cfg/smol360.yaml as shipped (activation checkpointing on)"}
        guarded("smol360", smol)
        if world > 1:
            sec["smol360_fsdp"] = {"unavailable": "the reference has no sharded data parallelism (its only strategy is DDP)"}
            sec["tp_fused_gemms"] = {"unavailable": "the reference has no tensor parallelism"}

        def sft():
            q = train_arm("113m", args.micro_batch, "sft", 3, 3)
            tokens = args.micro_batch * args.seq_len * world
            return {"metric": "SFT train tokens/s (113M, packed synthetic chats, assistant-only loss, seq 2048)",
                    "value": tokens / (q["ms"] / 1e3), "unit": "tokens/s", "ms_per_step": q["ms"], "steps": 3, "warmup": 3,
                    "e2e_value": tokens / (q["ms_e2e"] / 1e3), "final_loss": q["loss"],
                    "note": "the reference's Model under its DDP wrapper on this repository's packed batches (its own SFT "
                            "script is single-device)"}
        guarded("sft", sft)
    guard.finish()
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
