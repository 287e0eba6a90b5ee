"""Destructive hold-out split: cuts the tail ``pct`` percent of every top-level shard of a training directory into
``<dir>/val/val_split.<ext>`` (rewriting the shards as train-only) and records a manifest.  Runs once; an existing
split is reused (reference ``loomformer.py:1550-1775``)."""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional

import numpy as np

from ..parallel.dist import rank0_print
from .corpus import infer_format, read_arrow_table, resolve_files


def split_count(n: int, pct: float) -> int:
    if n <= 1:
        return 0
    return min(max(1, int(round(n * pct / 100.0))), n - 1)


def _replace(path: str, writer) -> None:
    tmp = path + ".tmp"
    writer(tmp)
    os.replace(tmp, path)


def _split_tables(files: List[str], val_path: str, pct: float, kind: str) -> Dict[str, int]:
    import pyarrow as pa
    import pyarrow.parquet as pq
    vals, ntrain, nval = [], 0, 0
    for p in files:
        if kind == "parquet":
            table, container = pq.read_table(p), "parquet"
        else:
            table, container = read_arrow_table(p)
        n = int(table.num_rows)
        k = split_count(n, pct)
        if k <= 0:
            ntrain += n
            continue
        train, val = table.slice(0, n - k), table.slice(n - k, k)
        if container == "parquet":
            _replace(p, lambda t: pq.write_table(train, t))
        elif container == "feather":
            import pyarrow.feather as feather
            _replace(p, lambda t: feather.write_feather(train, t))
        else:
            def write(t, train=train, container=container):
                with pa.OSFile(t, "wb") as sink:
                    mk = pa.ipc.new_stream if container == "stream" else pa.ipc.new_file
                    with mk(sink, train.schema) as w:
                        w.write_table(train)
            _replace(p, write)
        vals.append(val)
        ntrain += int(train.num_rows)
        nval += int(val.num_rows)
    if not vals:
        raise ValueError("auto val split produced no validation rows")
    try:
        merged = pa.concat_tables(vals, promote_options="default")
    except TypeError:
        merged = pa.concat_tables(vals, promote=True)
    if kind == "parquet":
        pq.write_table(merged, val_path)
    else:
        def write_val(t):
            with pa.OSFile(t, "wb") as sink:
                with pa.ipc.new_file(sink, merged.schema) as w:
                    w.write_table(merged)
        _replace(val_path, write_val)
    return {"train_rows": ntrain, "val_rows": nval}


def _split_lines(files: List[str], val_path: str, pct: float) -> Dict[str, int]:
    ntrain = nval = 0
    with open(val_path + ".tmp", "wb") as vf:
        for p in files:
            with open(p, "rb") as fh:
                lines = fh.readlines()
            k = split_count(len(lines), pct)
            keep, held = lines[:len(lines) - k], (lines[len(lines) - k:] if k > 0 else [])
            _replace(p, lambda t: open(t, "wb").writelines(keep))
            vf.writelines(held)
            ntrain += len(keep)
            nval += len(held)
    os.replace(val_path + ".tmp", val_path)
    return {"train_rows": ntrain, "val_rows": nval}


def _split_text(files: List[str], val_path: str, pct: float) -> Dict[str, int]:
    ntrain = nval = 0
    with open(val_path + ".tmp", "wb") as vf:
        for p in files:
            with open(p, "rb") as fh:
                data = fh.read()
            n = len(data)
            if n <= 1:
                train, val = data, b""
            else:
                cut = n - min(max(1, int(round(n * pct / 100.0))), n - 1)
                nl = data.rfind(b"\n", 0, cut)
                if nl > 0:
                    cut = nl + 1
                train, val = data[:cut], data[cut:]
            _replace(p, lambda t: open(t, "wb").write(train))
            vf.write(val)
            ntrain += len(train)
            nval += len(val)
    os.replace(val_path + ".tmp", val_path)
    return {"train_bytes": ntrain, "val_bytes": nval}


def _split_bin(files: List[str], val_path: str, pct: float) -> Dict[str, int]:
    vals, ntrain, nval = [], 0, 0
    for p in files:
        arr = np.fromfile(p, dtype=np.uint16)
        k = split_count(int(arr.shape[0]), pct)
        train, val = arr[:arr.shape[0] - k], (arr[arr.shape[0] - k:] if k > 0 else arr[:0])
        _replace(p, lambda t: train.tofile(t))
        vals.append(val)
        ntrain += int(train.shape[0])
        nval += int(val.shape[0])
    np.concatenate(vals).astype(np.uint16, copy=False).tofile(val_path)
    return {"train_tokens": ntrain, "val_tokens": nval}


def maybe_auto_val_split(cfg, dataset: str) -> Optional[str]:
    if cfg.val_dataset:
        return str(cfg.val_dataset)
    pct = float(cfg.auto_val_split_pct or 0.0)
    if pct <= 0.0:
        return None
    if not (0.0 < pct < 100.0):
        raise ValueError(f"auto_val_split_pct must be in (0,100), got {pct}")
    if not os.path.isdir(dataset):
        raise ValueError("auto_val_split_pct only works when the training dataset is a directory of shards")
    fmt = str(cfg.dataset_format or "auto").lower()
    files = resolve_files(dataset, fmt) if fmt != "bin" else sorted(
        os.path.join(dataset, f) for f in os.listdir(dataset) if f.endswith(".bin"))
    if not files:
        raise ValueError(f"auto_val_split_pct found no top-level corpus files in {dataset!r} (format={fmt!r})")
    kind = fmt if fmt != "auto" else infer_format(files[0])
    if kind != "bin" and any(infer_format(p) != kind for p in files):
        raise ValueError("auto_val_split_pct requires one dataset format per folder; found mixed extensions")
    ext = {"arrow": ".arrow", "parquet": ".parquet", "jsonl": ".jsonl", "txt": ".txt", "bin": ".bin"}.get(kind)
    if ext is None:
        raise ValueError(f"auto_val_split_pct unsupported dataset_format={kind!r}")
    os.makedirs(os.path.join(dataset, "val"), exist_ok=True)
    val_path = os.path.join(dataset, "val", "val_split" + ext)
    if os.path.exists(val_path):
        rank0_print(f"[auto-val-split] existing {val_path}; using it and NOT splitting again")
        cfg.val_dataset = val_path
        return val_path
    rank0_print(f"[auto-val-split] destructive split: pct={pct:.6g}% format={kind} files={len(files)} -> {val_path}")
    if kind in ("arrow", "parquet"):
        stats = _split_tables(files, val_path, pct, kind)
    elif kind == "jsonl":
        stats = _split_lines(files, val_path, pct)
    elif kind == "txt":
        stats = _split_text(files, val_path, pct)
    else:
        stats = _split_bin(files, val_path, pct)
    with open(val_path + ".manifest.json", "w", encoding="utf-8") as fh:
        json.dump({"dataset": os.path.abspath(dataset), "format": kind, "pct": pct, "files": files,
                   "val_dataset": val_path, "stats": stats}, fh, ensure_ascii=False, indent=2)
    rank0_print(f"[auto-val-split] done: {stats} | manifest={val_path}.manifest.json")
    cfg.val_dataset = val_path
    return val_path
