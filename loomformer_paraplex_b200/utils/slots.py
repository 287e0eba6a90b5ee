"""Audit of the boundary-slot population and the slot pool (reference ``utils/analyze_tria_slots_pool.py:59-202``):
for every temporal endpoint, the covariance ranks of the per-stream 9-vectors, how similar slots are across contexts,
how peaked the pool's softmax over streams is, and how the aggregated memory keys of adjacent boundaries relate."""
from __future__ import annotations

import json
import math
from typing import Any, Dict, List, Optional

import torch
import torch.nn.functional as F

from .geometry import amp, build_rows, load_probe_model, override_config, rope_report, tensor_quantiles


def pairwise_context_cosines(v: torch.Tensor) -> torch.Tensor:
    """``v`` [S, ..., D]: cosine between every pair of contexts, flattened."""
    u = F.normalize(v.float(), dim=-1, eps=1e-12)
    n = u.shape[0]
    if n < 2:
        return u.new_empty(0)
    iu = torch.triu_indices(n, n, offset=1)
    return (u[iu[0]] * u[iu[1]]).sum(-1).flatten()


def covariance_ranks(slots: torch.Tensor):
    x = slots.float().reshape(-1, 9)
    x = x - x.mean(0, keepdim=True)
    ev = torch.linalg.eigvalsh(x.t() @ x / max(x.shape[0] - 1, 1)).clamp_min(0).flip(0)
    p = ev / ev.sum().clamp_min(1e-12)
    return ev, torch.exp(-(p * p.clamp_min(1e-12).log()).sum()), ev.sum().square() / ev.square().sum().clamp_min(1e-12)


def chunk_report(carry: torch.Tensor, model, index: int):
    """``carry`` [S, H, 3, 3] at one boundary -> (report, slots [S, H, 9], aggregated key [S, N])."""
    slots = carry.reshape(carry.shape[0], carry.shape[1], 9).float()
    ev, erank, prank = covariance_ranks(slots)
    cos = pairwise_context_cosines(slots)
    agg = model.tria_agg
    score_w = agg.reader.make_score_w(agg.pool.query, agg.pool.logit_scale()).float()
    w = torch.softmax((slots * score_w).sum(-1), dim=-1)
    ent = -(w * w.clamp_min(1e-12).log()).sum(-1)
    pooled = (w.unsqueeze(-1) * slots).sum(1)
    lin = lambda x, m: F.linear(x, m.weight.float(), None if m.bias is None else m.bias.float())
    key = lin(lin(pooled, agg.reader.proj), agg.up)
    rep = {"chunk_index": index,
           "slot_population": {"covariance_eigenvalues": [float(x) for x in ev], "covariance_effective_rank": float(erank),
                               "covariance_participation_rank": float(prank), "context_cosine": tensor_quantiles(cos),
                               "context_abs_cosine": tensor_quantiles(cos.abs()), "slot_norm": tensor_quantiles(slots.norm(dim=-1))},
           "pool": {"normalized_entropy": tensor_quantiles(ent / math.log(slots.shape[1])),
                    "effective_streams": tensor_quantiles(ent.exp()), "max_weight": tensor_quantiles(w.amax(-1))},
           "aggregated_key": {"norm": tensor_quantiles(key.norm(dim=-1)),
                              "context_cosine": tensor_quantiles(pairwise_context_cosines(key.unsqueeze(1)))}}
    return rep, slots, key


def run(checkpoint: str, data: str, tokenizer: Optional[str] = None, tokens: int = 1536, window: Optional[int] = None,
        alpha: Optional[float] = None, polarm_beta: Optional[float] = None, sequences: int = 4, device: str = "cuda",
        output: str = "tria_slots_pool.json", tokenizer_obj=None, log=print) -> Dict[str, Any]:
    blob = torch.load(checkpoint, map_location="cpu", weights_only=True)
    cfg = override_config(blob, tokens, tokenizer, window, alpha, polarm_beta)
    dev = torch.device(device)
    W = int(cfg.tria_temporal_window)
    rows = build_rows(cfg, data, tokens, sequences, tokenizer_obj)
    model = load_probe_model(cfg, blob, dev)
    pos = torch.arange(tokens, device=dev).view(1, tokens)
    ends: List[torch.Tensor] = []
    with torch.inference_mode():
        for i, row in enumerate(rows, 1):
            with amp(dev):
                model(row.view(1, tokens).to(dev), position_ids=pos)
            if model.last_tria_document_carry is None:
                raise RuntimeError("actual Tria boundary-state capture failed")
            ends.append(model.last_tria_document_carry.detach().float().cpu())
            log(f"sequence {i}/{len(rows)}")
    endpoints = torch.cat(ends, 0)
    model.cpu()
    reports, slot_c, key_c = [], [], []
    for k in range(endpoints.shape[1]):
        rep, s, key = chunk_report(endpoints[:, k], model, k)
        reports.append(rep); slot_c.append(s); key_c.append(key)
    adj = lambda xs: (torch.cat([(F.normalize(a, dim=-1, eps=1e-12) * F.normalize(b, dim=-1, eps=1e-12)).sum(-1).flatten()
                                 for a, b in zip(xs[:-1], xs[1:])]) if len(xs) > 1 else torch.zeros(1))
    a_s, a_k = adj(slot_c), adj(key_c)
    report = {"checkpoint": checkpoint, "step": int(blob.get("step", 0) or 0), "dataset": data, "window": W,
              "tokens_analyzed": tokens, "sequences": len(rows), "polarm_beta": float(cfg.tria_polarm_beta),
              "rope": rope_report(cfg, tokens), "chunks": reports,
              "adjacent_boundary_slot_cosine": tensor_quantiles(a_s),
              "adjacent_boundary_slot_abs_cosine": tensor_quantiles(a_s.abs()),
              "adjacent_aggregated_key_cosine": tensor_quantiles(a_k)}
    with open(output, "w", encoding="utf-8") as fh:
        json.dump(report, fh, indent=2)
    log(f"JSON saved to {output}")
    return report


def main(argv=None) -> None:
    import argparse
    ap = argparse.ArgumentParser(description="boundary-slot population and slot-pool audit")
    ap.add_argument("checkpoint")
    ap.add_argument("--data", required=True)
    ap.add_argument("--tokenizer")
    ap.add_argument("--tokens", type=int, default=1536)
    ap.add_argument("--window", type=int)
    ap.add_argument("--alpha", type=float)
    ap.add_argument("--polarm-beta", type=float)
    ap.add_argument("--sequences", type=int, default=4)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--output", default="tria_slots_pool.json")
    a = ap.parse_args(argv)
    run(a.checkpoint, a.data, a.tokenizer, a.tokens, a.window, a.alpha, a.polarm_beta, a.sequences, a.device, a.output)


if __name__ == "__main__":
    main()
