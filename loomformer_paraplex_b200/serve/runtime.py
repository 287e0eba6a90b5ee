"""Model loading for inference / evaluation and the minimal greedy ``infer`` workflow
(reference ``loomformer.py:5289-5311, 5457-5487``)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ..config import Config, resolve
from ..data.tokenizers import build_tokenizer
from ..models.loomformer import Model
from ..train import checkpoint as ckpt
from ..train import evaluate as ev
from .decode import DecodeEngine


def load_model(path: str, device: torch.device, tokenizer=None) -> Tuple[Model, Config, object, dict]:
    blob = torch.load(path, map_location=device, weights_only=True)
    cfg = Config.from_checkpoint_dict(blob["cfg"])
    carry = None
    if tokenizer is None:
        tokenizer, carry = build_tokenizer(cfg)
    ablation = bool(blob.get("ablation", False))
    model = Model(cfg, ablation=ablation, dims=resolve(cfg, calibrate=False)).to(device)
    model.carry_token_id = carry
    ckpt.load_model_blob(model, blob, ablation)
    return model.eval(), cfg, tokenizer, blob


@torch.no_grad()
def infer(ckpt_path: str, prompt: str, max_new: int, device: torch.device) -> str:
    model, cfg, tok, _ = load_model(ckpt_path, device)
    ids = tok.encode(prompt) or [0]
    eng = DecodeEngine(model, batch=1, use_graph=(device.type == "cuda"))
    room = max(0, min(max_new, model.d.seq_len - len(ids)))
    out = list(ids)
    if room > 0:
        out += eng.generate(torch.tensor([ids], device=device), room)[0].tolist()
    text = tok.decode(out)
    print(text)
    return text


@torch.no_grad()
def eval_full(ckpt_path: str, dataset: Optional[str], device: torch.device, eval_batch_size: Optional[int] = None,
              eval_data_cache: str = "ram"):
    model, cfg, tok, _ = load_model(ckpt_path, device)
    dataset = dataset or cfg.val_dataset
    if not dataset:
        raise ValueError("--eval needs --dataset, or val_dataset in config/checkpoint")
    out = ev.eval_full_model(model, cfg, dataset, device, tok, eval_batch_size, eval_data_cache)
    print(f"dataset {dataset}")
    print(f"total_tokens {int(out['total_tokens'])}")
    print(f"total_nll {out['total_nll']:.6f}")
    print(f"eval_loss {out['loss_nats']:.6f}")
    print(f"bits/token {out['bits_tok']:.6f}")
    print(f"bpb {out['bpb']:.6f}")
    return out


def export_package(ckpt_path: str, out_path: str, device: torch.device, batch_size: int = 1) -> str:
    """Self-contained forward package at a fixed ``[batch, seq_len]`` shape.

    The reference exports through ``torch.export`` + AOTInductor (``loomformer.py:5314-5341``).  The same route is
    tried first on the composed plan; if the compiler tool-chain is unavailable the ``ExportedProgram`` itself is
    saved (``torch.export.save``), which loads with ``torch.export.load`` and needs no model code either."""
    from ..ops.opset import force_composed
    model, cfg, _, _ = load_model(ckpt_path, device)
    x = torch.randint(0, model.d.vocab, (batch_size, model.d.seq_len), device=device)
    force_composed(True)
    try:
        with torch.no_grad():
            exported = torch.export.export(model, (x,))
            try:
                path = torch._inductor.aoti_compile_and_package(exported, package_path=out_path)
                kind = "AOTInductor package"
            except Exception as exc:
                torch.export.save(exported, out_path)
                path, kind = out_path, f"ExportedProgram (AOTInductor unavailable: {type(exc).__name__})"
    finally:
        force_composed(False)
    print(f"[export-aoti] wrote {path} ({kind})")
    print(f"[export-aoti] shape baked in: batch_size={batch_size}, seq_len={model.d.seq_len}, vocab={model.d.vocab}")
    return str(path)
