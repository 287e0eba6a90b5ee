"""Supervised fine-tuning data: schema validation, one-off rendering + tokenisation, greedy packing of examples
into fixed-length rows (per-segment position ids, segment ids, loss mask restricted to assistant spans and to
targets inside the same segment) and a background prefetcher (reference ``loomsft.py:32-61, 108-325``).

Batches carry ``segment_ids`` instead of a dense ``[B,1,T,T]`` mask; ``dense_mask`` builds the latter on demand.
"""
from __future__ import annotations

import json
import queue
import random
import threading
import time
from typing import Dict, Iterator, List, Optional, Tuple

import numpy as np
import torch

from .streams import dense_mask
from .tokenizers import special_id

IGNORE_INDEX = -100
ROLES = {"system", "user", "assistant", "tool"}


def validate_example(ex: Dict, where: str = "") -> None:
    msgs = ex.get("messages")
    if not isinstance(msgs, list) or not msgs:
        raise ValueError(f"{where}messages must be a non-empty list")
    if msgs[0].get("role") not in ("system", "user"):
        raise ValueError(f"{where}first turn role must be system/user, got {msgs[0].get('role')!r}")
    pending = set()
    for i, m in enumerate(msgs):
        role, content, calls = m.get("role"), m.get("content"), m.get("tool_calls")
        if role not in ROLES:
            raise ValueError(f"{where}turn {i}: unknown role {role!r}")
        if role == "assistant":
            if content is None and not calls:
                raise ValueError(f"{where}turn {i}: assistant content is null with no tool_calls")
            for tc in calls or []:
                if "id" not in tc or "function" not in tc:
                    raise ValueError(f"{where}turn {i}: malformed tool_calls entry {tc!r}")
                pending.add(tc["id"])
            continue
        if calls:
            raise ValueError(f"{where}turn {i}: tool_calls only allowed on assistant turns")
        if role == "tool":
            ref = m.get("tool_call_id")
            if ref not in pending:
                raise ValueError(f"{where}turn {i}: tool_call_id {ref!r} has no matching preceding tool_calls entry")
            pending.discard(ref)
        elif content is None:
            raise ValueError(f"{where}turn {i}: {role} turn must have non-null content")


def iter_examples(path: str) -> Iterator[Tuple[int, Dict]]:
    """Numbered examples from a JSONL file or from the ``messages`` column of an Arrow file."""
    if path.endswith((".arrow", ".feather")):
        from .corpus import read_arrow_table
        table, _ = read_arrow_table(path)
        if "messages" not in table.column_names:
            raise ValueError(f"{path}: expected a 'messages' column, got {table.column_names}")
        for i, row in enumerate(table.column("messages").to_pylist(), 1):
            yield i, {"messages": row}
        return
    with open(path, "r", encoding="utf-8") as fh:
        for n, raw in enumerate(fh, 1):
            raw = raw.strip()
            if raw:
                yield n, json.loads(raw)


class TokenizedExample:
    __slots__ = ("ids", "mask")

    def __init__(self, ids, mask) -> None:
        self.ids, self.mask = np.asarray(ids, dtype=np.int32), np.asarray(mask, dtype=np.int8)


def tokenize_examples(examples, chat, seq_len: int, where: str = "") -> Tuple[List[TokenizedExample], int, int]:
    out, too_long, no_loss = [], 0, 0
    for n, ex in examples:
        validate_example(ex, where=f"{where}{n}: ")
        ids, mask = chat.render_training_ids(ex["messages"], tools=ex.get("tools"))
        if len(ids) > seq_len - 1:
            too_long += 1
        elif not any(mask):
            no_loss += 1
        else:
            out.append(TokenizedExample(ids, mask))
    return out, too_long, no_loss


def preprocess_dataset(path: str, chat, seq_len: int, verbose: bool = True) -> List[TokenizedExample]:
    t0 = time.time()
    out, too_long, no_loss = tokenize_examples(iter_examples(path), chat, seq_len, where=f"{path}:")
    if not out:
        raise ValueError(f"{path}: no examples fit within seq_len={seq_len} after validation/rendering")
    if verbose:
        print(f"[loomsft] preprocessed {path}: {len(out)} kept, {too_long} dropped (> seq_len-1={seq_len - 1} tokens), "
              f"{no_loss} dropped (no loss-carrying tokens) -- {time.time() - t0:.0f}s total", flush=True)
    return out


def need_pad_id(tok) -> int:
    pad = special_id(tok, "<pad>")
    if pad is None:
        raise ValueError("tokenizer is missing <pad>. Retrain it with data.tokenizers.train_tokenizer "
                         "(its default special tokens include <pad>).")
    return pad


class Packer:
    """Greedy first-fit packing of a reusable example pool into rows of ``seq_len`` tokens."""

    def __init__(self, pool: List[TokenizedExample], seq_len: int, pad_id: int, shuffle: bool, seed: int = 0) -> None:
        if not pool:
            raise ValueError("empty example pool")
        self.pool, self.T, self.pad_id, self.shuffle = pool, seq_len, pad_id, shuffle
        self._rng = random.Random(seed)
        self._order = list(range(len(pool)))
        if shuffle:
            self._rng.shuffle(self._order)
        self._cursor = 0

    def _next(self) -> TokenizedExample:
        if self._cursor >= len(self._order):
            self._cursor = 0
            if self.shuffle:
                self._rng.shuffle(self._order)
        ex = self.pool[self._order[self._cursor]]
        self._cursor += 1
        return ex

    def fast_forward(self, rows: int) -> None:
        for _ in range(rows):
            used = 0
            while used < self.T:
                n = len(self._next().ids)
                if used + n > self.T:
                    break
                used += n

    def pack_row(self):
        T = self.T
        ids = np.full(T, self.pad_id, dtype=np.int64)
        loss = np.zeros(T, dtype=np.int64)
        pos = np.zeros(T, dtype=np.int64)
        seg = np.full(T, -1, dtype=np.int64)
        used = s = 0
        while used < T:
            ex = self._next()
            n = len(ex.ids)
            if used + n > T:
                break
            ids[used:used + n], loss[used:used + n] = ex.ids, ex.mask
            pos[used:used + n], seg[used:used + n] = np.arange(n), s
            used += n
            s += 1
        return ids, loss, pos, seg

    def sample_batch(self, batch_size: int, device: torch.device, want_dense_mask: bool = False) -> Dict[str, torch.Tensor]:
        rows = [self.pack_row() for _ in range(batch_size)]
        ids, loss, pos, seg = (torch.from_numpy(np.stack([r[i] for r in rows])) for i in range(4))
        x, y = ids[:, :-1], ids[:, 1:]
        valid = loss[:, 1:].bool() & (seg[:, :-1] == seg[:, 1:])
        batch = {"x": x, "y": torch.where(valid, y, torch.full_like(y, IGNORE_INDEX)),
                 "position_ids": pos[:, :-1], "segment_ids": seg[:, :-1]}
        batch = {k: v.contiguous().to(device, non_blocking=True) for k, v in batch.items()}
        if want_dense_mask:
            batch["attn_mask"] = dense_mask(batch["segment_ids"])
        return batch


class BatchPrefetcher:
    """Builds packed batches on a background thread; producer errors surface in the consumer."""

    def __init__(self, packer: Packer, batch_size: int, device: torch.device, depth: int = 2, **kw) -> None:
        self.packer, self.batch_size, self.device, self.kw = packer, batch_size, device, kw
        self._q: "queue.Queue" = queue.Queue(maxsize=max(1, depth))
        self._stop = threading.Event()
        self._err: Optional[BaseException] = None
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def _run(self) -> None:
        try:
            while not self._stop.is_set():
                b = self.packer.sample_batch(self.batch_size, self.device, **self.kw)
                while not self._stop.is_set():
                    try:
                        self._q.put(b, timeout=0.2)
                        break
                    except queue.Full:
                        pass
        except BaseException as exc:
            self._err = exc
            try:
                self._q.put_nowait(None)
            except queue.Full:
                pass

    def next(self) -> Dict[str, torch.Tensor]:
        b = self._q.get()
        if b is None and self._err is not None:
            raise RuntimeError("BatchPrefetcher background thread failed") from self._err
        return b

    def stop(self) -> None:
        self._stop.set()


def synthetic_conversations(n: int, vocab_words: List[str], seed: int = 0, min_len: int = 16, max_len: int = 512):
    """Random multi-turn conversations (user/assistant alternation, optional system turn) whose turn lengths are
    uniform in ``[min_len, max_len]`` words -- the synthetic SFT workload of the benchmark configs."""
    rng = random.Random(seed)
    for i in range(n):
        msgs = []
        if rng.random() < 0.3:
            msgs.append({"role": "system", "content": " ".join(rng.choices(vocab_words, k=rng.randint(min_len, max_len)))})
        for t in range(rng.randint(1, 4)):
            msgs.append({"role": "user", "content": " ".join(rng.choices(vocab_words, k=rng.randint(min_len, max_len)))})
            msgs.append({"role": "assistant", "content": " ".join(rng.choices(vocab_words, k=rng.randint(min_len, max_len)))})
        yield i + 1, {"messages": msgs}
