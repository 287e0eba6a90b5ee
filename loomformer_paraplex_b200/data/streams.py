"""Training data streams.

``TokenStream``  random ``T+1`` windows from a prepared ``.bin`` (uint16) file.
``ShardStream``  streaming tokenisation of raw shards: the global row range is split by rank, a background
                 thread tokenises documents (joined by ``<eos>``), cuts ``[B, T+1]`` batches (``<bos>`` first when
                 the tokenizer has one), pins them and feeds a bounded queue; the consumer stacks several batches
                 into one host->device copy (reference ``loomformer.py:1241-1285, 1784-1971``).
Both expose ``next_batch()`` (device tensor), ``batches(n)`` (iterator) and ``fast_forward(n)``.
``doc_reset_state`` turns ``<eos>`` positions into per-document position ids and segment ids; the fused kernels
take segment ids directly and the dense ``[B,1,T,T]`` mask is only built for the composed plan.
"""
from __future__ import annotations

import json
import os
import queue
import threading
from typing import Iterator, List, Optional, Tuple

import numpy as np
import torch

from ..parallel import dist as pdist
from .corpus import infer_format, read_arrow_table, resolve_files
from .tokenizers import build_tokenizer, special_id


def doc_reset_state(x: torch.Tensor, eos_id: Optional[int]) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Returns ``(position_ids [B,T], segment_ids [B,T] or None)``.  A document ends WITH its ``<eos>``."""
    B, T = x.shape
    idx = torch.arange(T, device=x.device).unsqueeze(0).expand(B, T)
    if eos_id is None:
        return idx, None
    boundary = (x == eos_id).long()
    seg = torch.cumsum(boundary, dim=1) - boundary
    new_seg = torch.ones_like(seg, dtype=torch.bool)
    new_seg[:, 1:] = seg[:, 1:] != seg[:, :-1]
    start = torch.cummax(torch.where(new_seg, idx, torch.zeros_like(idx)), dim=1).values
    return idx - start, seg


def dense_mask(segment_ids: torch.Tensor) -> torch.Tensor:
    """Block-diagonal AND causal boolean mask ``[B,1,T,T]`` for the composed plan."""
    T = segment_ids.shape[1]
    causal = torch.ones(T, T, dtype=torch.bool, device=segment_ids.device).tril()
    return ((segment_ids.unsqueeze(2) == segment_ids.unsqueeze(1)) & causal).unsqueeze(1)


class TokenStream:
    def __init__(self, path: str, cfg, device: torch.device, bos_id: Optional[int] = None, seed: Optional[int] = None):
        cache = str(cfg.dataset_cache or "mmap").lower()
        if cache not in ("mmap", "ram"):
            raise ValueError(f"dataset_cache must be 'mmap' or 'ram', got {cache!r}")
        mm = np.memmap(path, dtype=np.uint16, mode="r")
        self.data = np.array(mm, dtype=np.uint16, copy=True) if cache == "ram" else mm
        self.cfg, self.device, self.bos_id, self.eos_id = cfg, device, bos_id, None
        if len(self.data) <= cfg.seq_len + 1:
            raise ValueError(f"dataset too short: {len(self.data)} tokens for seq_len={cfg.seq_len}")
        self.rng = np.random.default_rng(cfg.seed + 1000003 * pdist.rank() if seed is None else seed)

    def sample_host_batch(self) -> torch.Tensor:
        B, T = int(self.cfg.batch_size), int(self.cfg.seq_len)
        need = T + 1 - (1 if self.bos_id is not None else 0)
        ix = self.rng.integers(0, len(self.data) - need - 1, size=B)
        rows = np.stack([self.data[i:i + need].astype(np.int64) for i in ix])
        if self.bos_id is not None:
            rows = np.concatenate((np.full((B, 1), self.bos_id, dtype=np.int64), rows), axis=1)
        t = torch.from_numpy(rows)
        return t.pin_memory() if self.device.type == "cuda" else t

    def next_batch(self) -> torch.Tensor:
        return self.sample_host_batch().to(self.device, non_blocking=True)

    def fast_forward(self, n: int) -> None:
        for _ in range(n):
            self.sample_host_batch()

    def batches(self, n: int) -> Iterator[torch.Tensor]:
        for _ in range(n):
            yield self.next_batch()

    def prime(self) -> None:
        pass

    def close(self) -> None:
        pass


class ShardStream:
    CHUNK_DOCS = 20000

    def __init__(self, path: str, cfg, device: torch.device, tokenizer=None) -> None:
        self.cfg, self.device = cfg, device
        self.tok = tokenizer if tokenizer is not None else build_tokenizer(cfg)[0]
        self.bos_id, self.eos_id = special_id(self.tok, "<bos>"), special_id(self.tok, "<eos>")
        fmt = str(cfg.dataset_format or "auto")
        self.files = resolve_files(path, fmt)
        if not self.files:
            raise ValueError(f"no corpus files found at {path!r} (format={fmt!r})")
        self.fmt = fmt if fmt != "auto" else infer_format(self.files[0])
        self.text_field = cfg.text_field
        self.rank, self.world = pdist.rank(), pdist.world_size()
        counts = [self._row_count(p) for p in self.files]
        total = int(sum(counts))
        lo, hi = total * self.rank // self.world, total * (self.rank + 1) // self.world
        self.plan: List[Tuple[int, int, int]] = []
        cur = 0
        for fi, n in enumerate(counts):
            a, b = max(lo, cur) - cur, min(hi, cur + n) - cur
            if a < b:
                self.plan.append((fi, int(a), int(b)))
            cur += n
        self.rows = hi - lo
        if self.rows <= 0 or not self.plan:
            raise ValueError(f"rank {self.rank} received no rows")
        self.need = int(cfg.seq_len) + 1 - (1 if self.bos_id is not None else 0)
        self._q: "queue.Queue" = queue.Queue(maxsize=max(1, int(cfg.prefetch_batches)))
        self._stop = threading.Event()
        self._error: Optional[BaseException] = None
        self._dev_chunk: Optional[torch.Tensor] = None
        self._dev_pos = 0
        self._thread = threading.Thread(target=self._produce, daemon=True, name=f"data-rank-{self.rank}")
        self._thread.start()
        desc = ", ".join(f"{os.path.basename(self.files[i])}[{a}:{b}]" for i, a, b in self.plan)
        self._report("rows={:,} plan={}".format(self.rows, desc))

    def _report(self, msg: str) -> None:
        if pdist.initialized():
            import torch.distributed as dist
            got = [None] * self.world
            dist.all_gather_object(got, (self.rank, msg))
            if pdist.is_main():
                for r, m in sorted(got):
                    print(f"[data] rank={r} {m}", flush=True)
        else:
            print(f"[data] rank=0 {msg}", flush=True)

    def _row_count(self, p: str) -> int:
        if self.fmt == "parquet":
            import pyarrow.parquet as pq
            return int(pq.ParquetFile(p).metadata.num_rows)
        if self.fmt == "arrow":
            return int(read_arrow_table(p)[0].num_rows)
        if self.fmt == "jsonl":
            with open(p, "rb") as fh:
                return sum(1 for line in fh if line.strip())
        if self.fmt == "txt":
            return 1
        raise ValueError(f"unsupported raw dataset format {self.fmt!r}")

    def _text_chunks(self, p: str, a: int, b: int):
        if self.fmt in ("parquet", "arrow"):
            if self.fmt == "parquet":
                import pyarrow.parquet as pq
                table = pq.read_table(p, columns=[self.text_field])
            else:
                table = read_arrow_table(p)[0]
            col = table.column(self.text_field).slice(a, b - a)
            for s in range(0, len(col), self.CHUNK_DOCS):
                yield col.slice(s, min(self.CHUNK_DOCS, len(col) - s)).to_pylist()
        elif self.fmt == "jsonl":
            chunk, row = [], 0
            with open(p, "rb") as fh:
                for line in fh:
                    if not line.strip():
                        continue
                    if row >= b:
                        break
                    if row >= a:
                        chunk.append(json.loads(line.decode("utf-8", errors="replace")).get(self.text_field, ""))
                        if len(chunk) >= self.CHUNK_DOCS:
                            yield chunk
                            chunk = []
                    row += 1
            if chunk:
                yield chunk
        else:
            with open(p, "r", encoding="utf-8", errors="replace") as fh:
                yield [fh.read()]

    def _produce(self) -> None:
        try:
            B = int(self.cfg.batch_size)
            carry = np.zeros(0, dtype=np.int64)
            eos = None if self.eos_id is None else np.array([self.eos_id], dtype=np.int64)
            while not self._stop.is_set():
                first = True
                for fi, a, b in self.plan:
                    for texts in self._text_chunks(self.files[fi], a, b):
                        pieces = []
                        for ids in self.tok.encode_batch(texts):
                            if not first and eos is not None:
                                pieces.append(eos)
                            pieces.append(np.asarray(ids, dtype=np.int64))
                            first = False
                        if pieces:
                            carry = np.concatenate([carry] + pieces) if carry.size else np.concatenate(pieces)
                        per = B * self.need
                        while carry.size >= per and not self._stop.is_set():
                            block, carry = carry[:per].reshape(B, self.need), carry[per:]
                            batch = torch.from_numpy(block.copy())
                            if self.bos_id is not None:
                                batch = torch.cat((torch.full((B, 1), int(self.bos_id), dtype=torch.int64), batch), dim=1)
                            if self.device.type == "cuda":
                                batch = batch.pin_memory()
                            self._put(batch)
        except BaseException as exc:        # forwarded to the consumer
            self._error = exc
            try:
                self._q.put_nowait(None)
            except queue.Full:
                pass

    def _put(self, batch) -> None:
        while not self._stop.is_set():
            try:
                self._q.put(batch, timeout=0.2)
                return
            except queue.Full:
                continue

    def host_batch(self) -> torch.Tensor:
        b = self._q.get()
        if b is None:
            raise RuntimeError("data producer failed") from self._error
        return b

    def _load_chunk(self, count: int) -> None:
        host = torch.stack([self.host_batch() for _ in range(count)])
        self._dev_chunk, self._dev_pos = host.to(self.device, non_blocking=True), 0

    def chunk_size(self) -> int:
        return min(int(self.cfg.gpu_prefetch_batches), int(self.cfg.prefetch_batches))

    def prime(self) -> None:
        n = self.chunk_size()
        self._load_chunk(n)
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        self._report(f"ready: RAM={int(self.cfg.prefetch_batches)} batches, GPU={n} batches")

    def next_batch(self) -> torch.Tensor:
        if self._dev_chunk is None or self._dev_pos >= self._dev_chunk.shape[0]:
            self._load_chunk(self.chunk_size())
        b = self._dev_chunk[self._dev_pos]
        self._dev_pos += 1
        return b

    def fast_forward(self, n: int) -> None:
        for _ in range(n):
            self.host_batch()

    def batches(self, n: int) -> Iterator[torch.Tensor]:
        for _ in range(n):
            yield self.next_batch()

    def close(self) -> None:
        self._stop.set()


def make_stream(path: str, cfg, device: torch.device, tokenizer=None):
    fmt = str(cfg.dataset_format or "auto").lower()
    if fmt == "bin" or (fmt == "auto" and os.path.isfile(path) and path.endswith(".bin")):
        tok = tokenizer if tokenizer is not None else build_tokenizer(cfg)[0]
        return TokenStream(path, cfg, device, bos_id=special_id(tok, "<bos>"))
    return ShardStream(path, cfg, device, tokenizer=tokenizer)
