"""Raw text corpora: one index over txt / jsonl / parquet / arrow files with per-document character lengths,
sequential iteration and random character-window sampling (reference ``loomformer.py:1288-1451``)."""
from __future__ import annotations

import glob
import json
import os
from typing import Dict, Iterator, List, Tuple

import numpy as np

EXTENSIONS = {"txt": (".txt",), "jsonl": (".jsonl", ".ndjson"), "parquet": (".parquet",), "arrow": (".arrow", ".feather")}


def read_arrow_table(path: str):
    """Read an Arrow IPC file, IPC stream or Feather file; returns ``(table, container_kind)``."""
    import pyarrow as pa
    if os.path.splitext(path)[1].lower() == ".feather":
        import pyarrow.feather as feather
        return feather.read_table(path), "feather"
    with pa.memory_map(path, "rb") as src:
        try:
            return pa.ipc.open_file(src).read_all(), "file"
        except Exception:
            src.seek(0)
            return pa.ipc.open_stream(src).read_all(), "stream"


def resolve_files(path: str, fmt: str = "auto") -> List[str]:
    if os.path.isfile(path):
        return [path]
    exts = EXTENSIONS.get(fmt) or [e for v in EXTENSIONS.values() for e in v]
    found = set()
    for e in exts:
        found.update(glob.glob(os.path.join(path, f"*{e}")))
    return sorted(found)


def infer_format(path: str) -> str:
    ext = os.path.splitext(path)[1].lower()
    for fmt, exts in EXTENSIONS.items():
        if ext in exts:
            return fmt
    raise ValueError(f"cannot infer corpus format from extension {ext!r} ({path!r})")


class RawCorpus:
    def __init__(self, path: str, fmt: str = "auto", text_field: str = "text") -> None:
        self.text_field = text_field
        self.files = resolve_files(path, fmt)
        if not self.files:
            raise ValueError(f"no corpus files found at {path!r} (format={fmt!r})")
        self.fmt = fmt if fmt != "auto" else infer_format(self.files[0])
        self._tables: Dict[int, object] = {}
        self.docs: List[Tuple[int, object, int]] = []           # (file index, row / byte offset, chars)
        for fi, p in enumerate(self.files):
            self.docs.extend(getattr(self, "_index_" + self.fmt)(fi, p))
        if not self.docs:
            raise ValueError(f"corpus at {path!r} indexed to zero documents")
        self._cum = np.cumsum([d[2] for d in self.docs])
        self.total_chars = int(self._cum[-1])

    def __len__(self) -> int:
        return len(self.docs)

    # -- indexers -------------------------------------------------------------------------
    def _index_txt(self, fi, p):
        return [(fi, None, os.path.getsize(p))]

    def _index_jsonl(self, fi, p):
        out, offset = [], 0
        with open(p, "rb") as fh:
            for line in fh:
                s = line.decode("utf-8", errors="replace").strip()
                if s:
                    try:
                        txt = json.loads(s).get(self.text_field, "")
                        if txt:
                            out.append((fi, offset, len(txt)))
                    except Exception:
                        pass
                offset += len(line)
        return out

    def _index_parquet(self, fi, p):
        import pyarrow.compute as pc
        import pyarrow.parquet as pq
        pf, out, base = pq.ParquetFile(p), [], 0
        for rg in range(pf.num_row_groups):
            col = pf.read_row_group(rg, columns=[self.text_field]).column(self.text_field)
            lens = pc.utf8_length(col).to_numpy(zero_copy_only=False)
            out.extend((fi, base + i, int(n)) for i, n in enumerate(lens) if n > 0)
            base += len(lens)
        return out

    def _index_arrow(self, fi, p):
        import pyarrow.compute as pc
        table, _ = read_arrow_table(p)
        lens = pc.utf8_length(table.column(self.text_field)).to_numpy(zero_copy_only=False)
        return [(fi, i, int(n)) for i, n in enumerate(lens) if n > 0]

    # -- access ---------------------------------------------------------------------------
    def read_doc(self, fi: int, key, length: int = 0) -> str:
        p = self.files[fi]
        if self.fmt == "txt":
            with open(p, "r", encoding="utf-8", errors="replace") as fh:
                return fh.read()
        if self.fmt == "jsonl":
            with open(p, "rb") as fh:
                fh.seek(key)
                return json.loads(fh.readline().decode("utf-8", errors="replace")).get(self.text_field, "")
        table = self._tables.get(fi)
        if table is None:
            if self.fmt == "parquet":
                import pyarrow.parquet as pq
                table = pq.read_table(p, columns=[self.text_field])
            else:
                table, _ = read_arrow_table(p)
            self._tables[fi] = table
        return str(table.column(self.text_field)[key])

    def iter_texts(self) -> Iterator[str]:
        for fi, key, n in self.docs:
            txt = self.read_doc(fi, key, n)
            if txt:
                yield txt

    def iter_sampled_texts(self, docs) -> Iterator[str]:
        """Texts of a document subset; parquet reads touch only the row groups that hold wanted rows."""
        if self.fmt != "parquet":
            for fi, key, n in docs:
                yield self.read_doc(fi, key, n)
            return
        import pyarrow.parquet as pq
        by_file: Dict[int, List[int]] = {}
        for fi, key, _ in docs:
            by_file.setdefault(fi, []).append(int(key))
        for fi, rows in by_file.items():
            pf = pq.ParquetFile(self.files[fi])
            it = iter(sorted(rows))
            want, base = next(it, None), 0
            for rg in range(pf.num_row_groups):
                end = base + pf.metadata.row_group(rg).num_rows
                if want is not None and want < end:
                    col = pf.read_row_group(rg, columns=[self.text_field]).column(self.text_field)
                    while want is not None and want < end:
                        yield str(col[want - base])
                        want = next(it, None)
                base = end
                if want is None:
                    break

    def sample_window_spans(self, min_chars: int, rng: np.random.Generator) -> List[str]:
        """Text spans starting at a uniformly random character position, continued over following documents
        until ``min_chars`` characters are available."""
        pos = int(rng.integers(0, self.total_chars))
        di = min(int(np.searchsorted(self._cum, pos, side="right")), len(self.docs) - 1)
        fi, key, n = self.docs[di]
        spans = [self.read_doc(fi, key, n)[max(0, pos - (int(self._cum[di]) - n)):]]
        total, j = len(spans[0]), di + 1
        while total < min_chars and j < len(self.docs):
            t = self.read_doc(*self.docs[j])
            spans.append(t)
            total += len(t)
            j += 1
        return spans
