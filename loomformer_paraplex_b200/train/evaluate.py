"""Evaluation: sampled eval loss during training and the full sequential evaluation (non-overlapping windows plus
the tail) reporting nats/token, bits/token and bits/byte (reference ``loomformer.py:4114-4255, 5344-5487``)."""
from __future__ import annotations

import json
import math
import os
from typing import Dict, Optional, Tuple

import numpy as np
import torch
import torch.nn.functional as F

from ..data.corpus import RawCorpus
from ..data.streams import doc_reset_state, dense_mask
from ..parallel import dist as pdist


def is_prepared(dataset: str, cfg=None) -> bool:
    fmt = str(getattr(cfg, "dataset_format", "auto") or "auto").lower() if cfg is not None else "auto"
    return fmt == "bin" or (fmt == "auto" and os.path.isfile(dataset) and dataset.endswith(".bin"))


def load_bytes_per_token(dataset: str) -> Tuple[float, str, bool]:
    meta = dataset + ".meta.json"
    if not os.path.exists(meta):
        return 1.0, meta, False
    with open(meta, encoding="utf-8") as fh:
        bpt = float(json.load(fh).get("bytes_per_token", 1.0))
    if not math.isfinite(bpt) or bpt <= 0.0:
        raise ValueError(f"bad bytes_per_token={bpt!r} in {meta}")
    return bpt, meta, True


def compute_bytes_per_token(dataset: str, cfg, tok, max_docs: Optional[int] = None) -> Tuple[float, str]:
    meta = dataset + ".meta.json"
    if is_prepared(dataset, cfg):
        return 1.0, meta
    corpus = RawCorpus(dataset, fmt=cfg.dataset_format, text_field=cfg.text_field)
    docs, exact, stride = corpus.docs, True, 1
    if max_docs and len(docs) > max_docs:
        exact, stride = False, max(1, len(docs) // int(max_docs))
        docs = docs[::stride][:int(max_docs)]
    nbytes = ntok = ndocs = 0
    for text in corpus.iter_sampled_texts(docs):
        if text:
            nbytes += len(text.encode("utf-8")); ntok += len(tok.encode(text)); ndocs += 1
    if ntok <= 0:
        raise ValueError(f"cannot compute bytes/token for empty corpus: {dataset}")
    payload = {"tokens": ntok, "bytes": nbytes, "bytes_per_token": nbytes / ntok, "vocab": int(cfg.vocab),
               "format": corpus.fmt, "text_field": cfg.text_field, "docs": ndocs, "total_docs": len(corpus),
               "total_chars": corpus.total_chars, "exact": exact, "sample_stride": stride,
               "source": "computed_from_raw_corpus" if exact else "estimated_from_raw_corpus_sample"}
    tmp = meta + f".tmp.{os.getpid()}"
    with open(tmp, "w", encoding="utf-8") as fh:
        json.dump(payload, fh, ensure_ascii=False, indent=2)
    os.replace(tmp, meta)
    return payload["bytes_per_token"], meta


def ensure_bytes_per_token(dataset: str, cfg, tok, max_docs: Optional[int]) -> float:
    bpt, meta, ok = load_bytes_per_token(dataset)
    if ok or is_prepared(dataset, cfg):
        return bpt
    if pdist.is_main():
        print(f"[meta] {meta} missing; computing bytes/token from {dataset} with active tokenizer"
              + (f" (sample_docs={max_docs})" if max_docs else "") + "...")
        bpt, _ = compute_bytes_per_token(dataset, cfg, tok, max_docs)
        print(f"[meta] wrote {meta} bytes/token={bpt:.6f} exact={'false' if max_docs else 'true'}")
    pdist.barrier()
    return load_bytes_per_token(dataset)[0]


def loss_to_bits(loss_nats: float, bytes_per_token: float) -> Tuple[float, float]:
    bits = float(loss_nats) / math.log(2.0)
    return bits, bits / bytes_per_token


def dataset_token_count(dataset: str, cfg, tok) -> int:
    if is_prepared(dataset, cfg):
        n = os.path.getsize(dataset)
        if n % 2:
            raise ValueError(f"prepared dataset byte size is not uint16-aligned: {dataset} has {n} bytes")
        return n // 2
    corpus = RawCorpus(dataset, fmt=cfg.dataset_format, text_field=cfg.text_field)
    sample = corpus.docs[::max(1, len(corpus.docs) // 50)][:50]
    chars = toks = 0
    for text in corpus.iter_sampled_texts(sample):
        chars += len(text); toks += len(tok.encode(text))
    return int(corpus.total_chars / max(1e-6, chars / max(1, toks)))


@torch.no_grad()
def model_nll(model, x, y, segment_ids=None, position_ids=None, amp: str = "fp32") -> Tuple[torch.Tensor, int]:
    """Summed NLL of ``y`` given ``x`` (fp32 log-softmax) and the number of scored tokens."""
    plan = model._opset(model.emb.weight) if not model.ablation else None
    if plan is not None:
        _, logits = plan.run(x, None, position_ids, segment_ids, want_grad=False)
    else:
        mask = None if segment_ids is None else dense_mask(segment_ids)
        logits = model(x, attn_mask=mask, position_ids=position_ids)
    V = logits.shape[-1]
    nll = F.cross_entropy(logits.float().reshape(-1, V), y.reshape(-1), reduction="sum", ignore_index=-100)
    return nll, int((y != -100).sum())


@torch.no_grad()
def sampled_eval_loss(model, stream, cfg, eos_id: Optional[int] = None) -> float:
    was = model.training
    model.eval()
    losses = []
    for _ in range(max(1, int(cfg.eval_batches))):
        b = stream.next_batch()
        x, y = b[:, :-1], b[:, 1:]
        pos, seg = doc_reset_state(x, eos_id)
        nll, n = model_nll(model, x, y, seg, pos)
        losses.append(float(nll) / max(1, n))
    model.train(was)
    return float(np.mean(losses))


@torch.no_grad()
def eval_full_model(model, cfg, dataset: str, device, tok=None, eval_batch_size: Optional[int] = None,
                    eval_data_cache: str = "ram") -> Dict[str, float]:
    model.eval()
    if is_prepared(dataset, cfg):
        bpt = load_bytes_per_token(dataset)[0]
        data = np.memmap(dataset, dtype=np.uint16, mode="r")
    else:
        corpus = RawCorpus(dataset, fmt=cfg.dataset_format, text_field=cfg.text_field)
        ids, nbytes = [], 0
        for fi, key, n in corpus.docs:
            text = corpus.read_doc(fi, key, n)
            nbytes += len(text.encode("utf-8"))
            ids.extend(tok.encode(text))
        data = np.array(ids, dtype=np.uint16)
        bpt = nbytes / max(1, len(data))
    if len(data) < 2:
        raise ValueError(f"dataset too short for eval: {dataset}")
    cache = str(eval_data_cache or "ram").lower()
    if cache not in ("mmap", "ram", "gpu"):
        raise ValueError(f"eval_data_cache must be 'mmap', 'ram', or 'gpu', got {eval_data_cache!r}")
    T = int(cfg.seq_len)
    B = max(1, int(eval_batch_size if eval_batch_size is not None else cfg.batch_size))
    n = int(len(data))
    n_full = (n - 1) // T
    if cache != "mmap":
        data = np.array(data, dtype=np.uint16, copy=True)
    total_nll, total_tok = 0.0, 0

    def score(arr):
        nonlocal total_nll, total_tok
        batch = torch.from_numpy(np.asarray(arr, dtype=np.int64))
        if device.type == "cuda":
            batch = batch.pin_memory()
        batch = batch.to(device, non_blocking=True)
        nll, k = model_nll(model, batch[:, :-1], batch[:, 1:])
        total_nll += float(nll); total_tok += k

    if n_full > 0:
        s = data.strides[0]
        windows = np.lib.stride_tricks.as_strided(data, shape=(n_full, T + 1), strides=(T * s, s), writeable=False)
        for i in range(0, n_full, B):
            score(windows[i:i + B])
    if n_full * T < n - 1:
        score(data[n_full * T:n][None, :])
    loss = total_nll / max(1, total_tok)
    bits, bpb = loss_to_bits(loss, bpt)
    return {"total_tokens": float(total_tok), "total_nll": float(total_nll), "loss_nats": float(loss),
            "bits_tok": float(bits), "bpb": float(bpb)}
