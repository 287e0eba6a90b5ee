#!/usr/bin/env python3
"""LoomFormer-Paraplex on B200: tokenizer training, corpus preparation, pre-training, evaluation, inference, export.

Command-line surface of the reference entry point (``loomformer.py:5515-5668`` there): same flags, same YAML schema,
same checkpoint format.  ``--device cudas`` (or a comma list) re-launches under ``torch.distributed.run`` with one
process per GPU."""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def smoke_test() -> None:
    import torch
    import torch.nn.functional as F
    from loomformer_paraplex_b200.config import Config
    from loomformer_paraplex_b200.models.loomformer import Model
    from loomformer_paraplex_b200.ops.opset import force_composed
    dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    cfg = Config(vocab=64, model_dim=12, n_q_heads=6, n_kv_heads=3, hidden=66, layers=2, seq_len=16, batch_size=2, steps=2)
    torch.manual_seed(cfg.seed)
    force_composed(True)
    model = Model(cfg).to(dev)
    x = torch.randint(0, 64, (2, 16), device=dev)
    logits = model(x)
    assert logits.shape == (2, 16, 64) and model.head.weight is model.emb.weight
    loss = F.cross_entropy(logits.reshape(-1, 64).float(), torch.randint(0, 64, (32,), device=dev))
    loss.backward()
    force_composed(False)
    print(f"[smoke] forward/backward OK logits={tuple(logits.shape)} loss={loss.item():.4f} "
          f"logit_std={float(logits.float().std()):.4f} emb_std={float(model.emb.weight.float().std()):.4f} "
          f"tied={model.head.weight is model.emb.weight}")


def prepare(raw_dir: str, cfg, out: str) -> None:
    import numpy as np
    from loomformer_paraplex_b200.data.corpus import RawCorpus
    from loomformer_paraplex_b200.data.tokenizers import build_tokenizer
    tok, _ = build_tokenizer(cfg)
    corpus = RawCorpus(raw_dir, fmt=cfg.dataset_format, text_field=cfg.text_field)
    ids, nbytes = [], 0
    for fi, key, n in corpus.docs:
        text = corpus.read_doc(fi, key, n)
        nbytes += len(text.encode("utf-8"))
        ids.extend(tok.encode(text))
    assert cfg.vocab <= 65536, "uint16 storage requires vocab <= 65536"
    arr = np.array(ids, dtype=np.uint16)
    arr.tofile(out)
    bpt = nbytes / max(1, len(arr))
    with open(out + ".meta.json", "w", encoding="utf-8") as fh:
        json.dump({"tokens": len(arr), "bytes": nbytes, "bytes_per_token": bpt, "vocab": cfg.vocab}, fh)
    print(f"[prepare] {len(arr)} tokens, {nbytes} bytes, {bpt:.3f} bytes/token -> {out} ({cfg.summary()})")


def main() -> None:
    ap = argparse.ArgumentParser(description="LoomFormer: GQA Transformer LM with Paraplex FFN (B200-native)")
    ap.add_argument("--config", type=str, default=None)
    ap.add_argument("--dataset", type=str, default=None)
    ap.add_argument("--output", type=str, default=None)
    ap.add_argument("--device", type=str, default=None)
    ap.add_argument("--prepare", type=str, default=None, metavar="RAWDIR")
    ap.add_argument("--train-tokenizer", type=str, default=None, metavar="RAWDIR")
    ap.add_argument("--tokenizer-out", type=str, default="tokenizer.json")
    ap.add_argument("--vocab", type=int, default=8192)
    ap.add_argument("--train", action="store_true")
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--amp-dtype", type=str, default=None, choices=("bf16", "fp32", "off", "fp16"))
    ap.add_argument("--infer", action="store_true")
    ap.add_argument("--eval", action="store_true", help="full sequential eval on --dataset, or config/checkpoint val_dataset")
    ap.add_argument("--eval-batch-size", type=int, default=None)
    ap.add_argument("--eval-data-cache", type=str, default="ram", choices=("mmap", "ram", "gpu"))
    ap.add_argument("--checkpoint", type=str, default=None)
    ap.add_argument("--export-aoti", type=str, default=None, metavar="OUT.pt2")
    ap.add_argument("--export-batch-size", type=int, default=1)
    ap.add_argument("--resume", type=str, default=None)
    ap.add_argument("--resume-step", type=int, default=None)
    ap.add_argument("--resume-data", type=str, default=None, choices=("auto", "continue", "restart"))
    ap.add_argument("--prompt", type=str, default="")
    ap.add_argument("--max-new", type=int, default=64)
    ap.add_argument("--smoke-test", action="store_true")
    ap.add_argument("--ablation", action="store_true", help="diagnostic: skip imag/phase and use s=1")
    ap.add_argument("--quiet", action="store_true", help="--train only: detach into the background, log to a file")
    ap.add_argument("--grad-sync", type=str, default="auto", choices=("auto", "collective", "p2p", "fsdp"),
                    help="multi-GPU gradient path: NCCL all-reduce or the fused NVLink reduce-scatter+AdamW+all-gather kernel")
    args = ap.parse_args()

    if args.smoke_test:
        smoke_test()
        return
    if args.quiet and args.train and "WORLD_SIZE" not in os.environ:
        ts = time.strftime("%Y%m%d_%H%M%S")
        log_path = f"log_{ts}.log"
        child = [a for a in sys.argv[1:] if a != "--quiet"]
        with open(log_path, "a", encoding="utf-8") as log:
            proc = subprocess.Popen([sys.executable, os.path.abspath(__file__)] + child, stdout=log, stderr=log,
                                    stdin=subprocess.DEVNULL, start_new_session=True)
        time.sleep(3.0)
        if proc.poll() is not None and proc.returncode != 0:
            print(f"[quiet] background process exited immediately (code {proc.returncode}) -- see {log_path} for why:")
            print(open(log_path, encoding="utf-8").read()[-2000:])
            raise SystemExit(proc.returncode)
        with open(f"{log_path}.pid", "w") as fh:
            fh.write(str(proc.pid))
        print(f"[quiet] training running in background, pid={proc.pid}")
        print(f"[quiet] use: tail -f {log_path}   (kill with: kill {proc.pid})")
        return

    import torch
    from loomformer_paraplex_b200.config import Config, resolve
    from loomformer_paraplex_b200.parallel import dist as pdist
    cfg = Config.from_yaml(args.config) if args.config else Config()
    if args.steps is not None:
        cfg.steps = args.steps
    if args.amp_dtype is not None:
        cfg.amp_dtype = args.amp_dtype
    if args.resume_data is not None:
        cfg.resume_data_stream = args.resume_data
    pref = args.device if args.device is not None else cfg.device
    if args.train:
        pdist.maybe_self_launch(pref, os.path.abspath(__file__), sys.argv[1:])
    dev, world, rank = pdist.init(pref)
    if dev.type == "cuda" and world == 1:
        idx = 0 if dev.index is None else int(dev.index)
        if idx >= torch.cuda.device_count():
            raise RuntimeError(f"Requested {dev}, but only {torch.cuda.device_count()} CUDA device(s) are visible. "
                               f"CUDA_VISIBLE_DEVICES={os.environ.get('CUDA_VISIBLE_DEVICES')!r}.")
    gbs = int(cfg.batch_size)
    if world > 1:
        if gbs < world or gbs % world:
            raise ValueError(f"batch_size={gbs} is global in DDP mode and must be a multiple of world_size={world}")
        cfg._global_batch_size, cfg.batch_size = gbs, gbs // world
        pdist.rank0_print(f"[ddp] world_size={world} backend={'nccl' if dev.type == 'cuda' else 'gloo'}")
        pdist.rank0_print(f"[ddp] batch_size(global)={gbs} -> batch_size(local)={cfg.batch_size}")
        pdist.rank0_print(f"[ddp] grad_accum_steps={cfg.grad_accum_steps} -> effective_global_batch={gbs * int(cfg.grad_accum_steps)}")
    else:
        cfg._global_batch_size = gbs
    if args.quiet and args.train:
        ts = time.strftime("%Y%m%d_%H%M%S")
        log_path = f"log_{ts}_rank{rank}.log"
        pdist.rank0_print(f"[quiet] rank {rank}: logging to {log_path}  ·  use: tail -f {log_path}")
        sys.stdout = sys.stderr = open(log_path, "a", buffering=1, encoding="utf-8")
        print(f"[quiet] --- log started {ts} (rank {rank}/{world}) ---")

    if args.train_tokenizer:
        from loomformer_paraplex_b200.data.tokenizers import train_tokenizer
        train_tokenizer(args.train_tokenizer, args.vocab, args.tokenizer_out, dataset_format=cfg.dataset_format,
                        text_field=cfg.text_field)
    elif args.prepare:
        prepare(args.prepare, cfg, args.output or "prep.bin")
    elif args.train:
        from loomformer_paraplex_b200.train.trainer import train
        dataset = args.dataset or cfg.train_dataset
        assert dataset, "--train needs --dataset or train_dataset in config"
        sync = args.grad_sync
        if sync == "auto":
            sync = "p2p" if (world > 1 and dev.type == "cuda") else "collective"      # fused NVLink step (AdamW and ATOM)
        res = train(cfg, dataset, dev, args.checkpoint or "loomformer.pt", args.ablation,
                    args.resume if args.resume is not None else cfg.resume, args.resume_step, grad_sync=sync)
        pdist.rank0_print("\nSummary:")
        if res.get("skipped"):
            pdist.rank0_print(f"paraplex: skipped -- checkpoint step {int(res['start_step'])} >= cfg.steps")
        else:
            extra = ""
            if res["full_eval_loss"] == res["full_eval_loss"]:
                extra = f" | full_eval_loss {res['full_eval_loss']:.4f} | full_bpb {res['full_eval_bpb']:.4f}"
            pdist.rank0_print(f"paraplex: final_eval_loss {res['final_eval_loss']:.4f} | best_eval_loss "
                              f"{res['best_eval_loss']:.4f}{extra} | time {res['seconds']:.0f}s")
        pdist.shutdown()
    elif args.export_aoti:
        from loomformer_paraplex_b200.serve.runtime import export_package
        assert args.checkpoint, "--export-aoti needs --checkpoint"
        export_package(args.checkpoint, args.export_aoti, dev, args.export_batch_size)
    elif args.infer:
        from loomformer_paraplex_b200.serve.runtime import infer
        assert args.checkpoint, "--infer needs --checkpoint"
        infer(args.checkpoint, args.prompt, args.max_new, dev)
    elif args.eval:
        from loomformer_paraplex_b200.serve.runtime import eval_full
        assert args.checkpoint, "--eval needs --checkpoint"
        eval_full(args.checkpoint, args.dataset or cfg.val_dataset, dev, args.eval_batch_size, args.eval_data_cache)
    else:
        ap.print_help()


if __name__ == "__main__":
    main()
