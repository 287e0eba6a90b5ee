"""Decode throughput: prompts of uniform-random tokens, greedy continuation under CUDA-graph replay.

``python -m loomformer_paraplex_b200.serve.bench_decode --batch 64 --prompt 512 --new 256`` prints one JSON line with
prefill and decode tokens/s (device-timed).  ``--impl reference`` times the reference implementation's own
``Model.step`` loop (from ``baseline/_ref``) on the same shapes.  With ``--replicas N`` (or under torchrun) every rank
serves its own batch -- data-parallel serving -- and the line reports the sum over ranks, timed as the max over ranks.
``--histogram`` instead prints, per kernel, launches and device time of one decode step run eagerly under the PyTorch
profiler (shares only: the step itself is timed by the plain run, under graph replay)."""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def model_kw():
    sys.path.insert(0, ROOT)
    import bench
    return dict(bench.MODEL_KW)


def run_ours(a, dev):
    from ..config import Config
    from ..models.loomformer import Model
    from .decode import DecodeEngine
    cfg = Config(**model_kw())
    torch.manual_seed(1)
    model = Model(cfg).to(dev).eval()
    eng = DecodeEngine(model, batch=a.batch, max_len=a.prompt + a.new + 1, use_graph=True)
    g = torch.Generator(device="cpu").manual_seed(5 + int(os.environ.get("RANK", "0")))
    prompt = torch.randint(0, cfg.vocab, (a.batch, a.prompt), generator=g).to(dev)
    for _ in range(2):                                        # warm-up incl. graph capture
        eng.generate(prompt, 4)
    torch.cuda.synchronize()
    e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    e0.record()
    logits = eng.prefill(prompt)
    tok = logits.argmax(-1)
    e1.record()
    for _ in range(a.new):
        eng.step(tok)
        tok = eng.next_tok
    e2.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1), e1.elapsed_time(e2)


def histogram(a, dev, top: int = 30) -> None:
    """Kernel histogram of one eager decode step at position ``a.prompt`` (three steps, averaged)."""
    import collections
    from torch.profiler import ProfilerActivity, profile
    from ..config import Config
    from ..models.loomformer import Model
    from .decode import DecodeEngine
    cfg = Config(**model_kw())
    torch.manual_seed(1)
    model = Model(cfg).to(dev).eval()
    eng = DecodeEngine(model, batch=a.batch, max_len=a.prompt + a.new + 1, use_graph=False)
    prompt = torch.randint(0, cfg.vocab, (a.batch, a.prompt), device=dev)
    eng.generate(prompt, 4)
    tok = eng.next_tok.clone()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        for _ in range(3):
            eng.step(tok)
        torch.cuda.synchronize()
    cnt, tim = collections.Counter(), collections.Counter()
    for e in prof.events():
        if e.device_type == torch.autograd.DeviceType.CUDA:
            name = e.name.replace("(anonymous namespace)::", "").replace("void ", "")[:64]
            cnt[name] += 1
            tim[name] += e.device_time
    print(f"batch {a.batch}, position {a.prompt}: {sum(cnt.values()) / 3:.0f} launches per step, "
          f"{sum(tim.values()) / 3:.0f} us of kernel time per step (eager; the replayed graph overlaps launches)")
    for k, v in tim.most_common(top):
        print(f"  {v / 3:8.1f} us {cnt[k] / 3:6.1f} x  {k}")


def run_reference(a, dev):
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(ref):
        return None
    sys.path.insert(0, ref)
    os.chdir(ref)
    import loomformer as lf
    kw = {k: v for k, v in model_kw().items() if k in lf.Config.__dataclass_fields__}
    cfg = lf.Config(**kw)
    lf.apply_config(cfg)
    torch.manual_seed(1)
    model = lf.Model(cfg).to(dev).eval()
    g = torch.Generator(device="cpu").manual_seed(5)
    prompt = torch.randint(0, cfg.vocab, (a.batch, a.prompt), generator=g).to(dev)
    e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    with torch.inference_mode(), torch.autocast("cuda", dtype=torch.bfloat16):
        st = None
        for t in range(8):                                    # warm-up
            lg, st = model.step(prompt[:, t], t, st)
        torch.cuda.synchronize()
        st = None
        e0.record()
        for t in range(a.prompt):                             # the reference prefills token by token
            lg, st = model.step(prompt[:, t], t, st)
        e1.record()
        tok = lg.argmax(-1)
        for i in range(a.new):
            lg, st = model.step(tok, a.prompt + i, st)
            tok = lg.argmax(-1)
        e2.record()
        torch.cuda.synchronize()
    return e0.elapsed_time(e1), e1.elapsed_time(e2)


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--new", type=int, default=256)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--histogram", action="store_true", help="kernel histogram of one eager decode step instead of timing")
    a = ap.parse_args(argv)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if a.histogram:
        histogram(a, dev)
        return
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    res = run_ours(a, dev) if a.impl == "ours" else run_reference(a, dev)
    if res is None:
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not present"}))
        return
    pre_ms, dec_ms = res
    if world > 1:
        t = torch.tensor([pre_ms, dec_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        pre_ms, dec_ms = float(t[0]), float(t[1])
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"metric": "decode tokens/s (113M LoomFormer-Paraplex, bf16, greedy, KV cache + Tria carry)",
                          "impl": a.impl, "replicas": world, "batch_per_replica": a.batch, "prompt": a.prompt, "new": a.new,
                          "prefill_ms": pre_ms, "decode_ms": dec_ms,
                          "prefill_tok_s": world * a.batch * a.prompt / (pre_ms / 1e3),
                          "decode_tok_s": world * a.batch * a.new / (dec_ms / 1e3),
                          "ms_per_decode_step": dec_ms / a.new, "data": "uniform-random prompt tokens, random-init weights"}))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
