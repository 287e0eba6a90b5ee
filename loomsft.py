#!/usr/bin/env python3
"""loomsft: supervised fine-tuning of a LoomFormer checkpoint on chat data (JSONL ``messages`` records or an Arrow
``messages`` column), packed to ``seq_len`` with assistant-only loss.  Flags follow the reference tool
(``loomsft.py:598-632`` there); ``--device cudas`` additionally fine-tunes data-parallel on all GPUs."""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def smoke_test() -> None:
    """Tokenizer with the chat specials, schema validation, rendering, tool-call parsing, packing shapes, a packed
    forward, and cross-segment isolation (perturbing segment 0 must not move later segments' logits)."""
    import tempfile
    import torch
    from loomformer_paraplex_b200.config import Config
    from loomformer_paraplex_b200.data import sft as sd
    from loomformer_paraplex_b200.data.chat import ChatTemplate
    from loomformer_paraplex_b200.data.streams import dense_mask
    from loomformer_paraplex_b200.data.tokenizers import BPETokenizer, train_tokenizer
    from loomformer_paraplex_b200.models.loomformer import Model
    words = "alpha beta gamma delta epsilon zeta eta theta iota kappa lambda mu".split()
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "tok.json")
        train_tokenizer("", 320, path, texts=[" ".join(words)] * 50)
        tok = BPETokenizer.load(path)
    chat = ChatTemplate(tok)
    ex = {"messages": [{"role": "user", "content": "alpha?"},
                       {"role": "assistant", "content": None, "tool_calls": [
                           {"id": "c0", "type": "function", "function": {"name": "f", "arguments": "{}"}}]},
                       {"role": "tool", "tool_call_id": "c0", "content": "beta"},
                       {"role": "assistant", "content": "gamma"}]}
    sd.validate_example(ex)
    assert chat.parse_tool_calls(chat.render_text(ex["messages"]))[0]["function"]["name"] == "f"
    pool, _, _ = sd.tokenize_examples(sd.synthetic_conversations(30, words, min_len=2, max_len=8), chat, 96)
    packer = sd.Packer(pool, 96, sd.need_pad_id(tok), shuffle=True, seed=0)
    b = packer.sample_batch(2, torch.device("cpu"))
    cfg = Config(vocab=tok.vocab_size, seq_len=96, model_dim=32, n_q_heads=4, n_kv_heads=2, hidden=64, layers=2,
                 activation="pvpowlu", tria_carry_enabled=True, tria_temporal_auto=False, tria_temporal_window=32)
    torch.manual_seed(0)
    model = Model(cfg).eval()
    mask = dense_mask(b["segment_ids"])
    with torch.no_grad():
        base = model(b["x"], attn_mask=mask, position_ids=b["position_ids"])
        x2 = b["x"].clone()
        seg0 = b["segment_ids"][0] == 0
        x2[0, seg0] = (x2[0, seg0] + 1) % tok.vocab_size
        moved = model(x2, attn_mask=mask, position_ids=b["position_ids"])
    later = b["segment_ids"][0] > 0
    leak = float((base[0, later] - moved[0, later]).abs().max()) if bool(later.any()) else 0.0
    # Tria's temporal carrier crosses segments only through fired keys, which the packing mask hides
    assert leak < 1e-4, f"cross-segment leak {leak}"
    print(f"[loomsft smoke] OK  rows={tuple(b['x'].shape)}  loss tokens={int((b['y'] != -100).sum())}  leak={leak:.2e}")


def main() -> None:
    ap = argparse.ArgumentParser(description="loomsft: SFT training for LoomFormer (B200-native)")
    ap.add_argument("--config", type=str, default=None)
    ap.add_argument("--sft-dataset", type=str, default=None)
    ap.add_argument("--val-dataset", type=str, default=None)
    ap.add_argument("--init-checkpoint", type=str, default=None)
    ap.add_argument("--checkpoint", type=str, default="loomsft.pt")
    ap.add_argument("--resume", type=str, default=None)
    ap.add_argument("--resume-step", type=int, default=None)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--device", type=str, default=None)
    ap.add_argument("--grad-sync", type=str, default="collective", choices=("collective", "p2p", "fsdp"))
    ap.add_argument("--smoke-test", action="store_true")
    args = ap.parse_args()
    if args.smoke_test:
        smoke_test()
        return
    from loomformer_paraplex_b200.config import Config
    from loomformer_paraplex_b200.parallel import dist as pdist
    from loomformer_paraplex_b200.train.sft import train_sft
    cfg = Config.from_yaml(args.config) if args.config else Config()
    if args.steps is not None:
        cfg.steps = args.steps
    pref = args.device if args.device is not None else cfg.device
    pdist.maybe_self_launch(pref, os.path.abspath(__file__), sys.argv[1:])
    dev, world, _ = pdist.init(pref)
    if world > 1:
        if int(cfg.batch_size) % world:
            raise ValueError(f"batch_size={cfg.batch_size} must be divisible by world_size={world}")
        cfg._global_batch_size, cfg.batch_size = int(cfg.batch_size), int(cfg.batch_size) // world
    assert args.sft_dataset, "--sft-dataset is required"
    assert args.init_checkpoint or args.resume, ("--init-checkpoint is required (SFT starts from a pretrained LoomFormer "
                                                 "checkpoint), unless --resume points at an existing SFT runpoint")
    train_sft(cfg, args.sft_dataset, args.val_dataset, args.init_checkpoint, dev, args.checkpoint, resume=args.resume,
              resume_step=args.resume_step, grad_sync=args.grad_sync)
    pdist.shutdown()


if __name__ == "__main__":
    main()
