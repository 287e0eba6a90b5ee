"""Single-file inference packages (``.aio``): checkpoint + tokenizer JSON + chat template in one ``torch.save`` blob.

Layout (interchangeable with the reference tool, ``loompack.py:198-272`` there)::

    {"format": "loom.aio", "version": 1, "manifest": {...}, "checkpoint": {...inference-only checkpoint...},
     "tokenizer_json": bytes, "chat_template_jinja": bytes}

"Quantisation" is a storage cast: large matrices go to bf16/fp16, while anything whose precision matters for the
carriers, norms, gates and phase statistics stays fp32.  Tensors that alias one storage (tied embeddings) stay aliased
in the package."""
from __future__ import annotations

import hashlib
import json
import os
import time
from collections import Counter
from pathlib import Path
from typing import Any, Dict, Mapping, Optional, Tuple

import torch

FORMAT_NAME = "loom.aio"
FORMAT_VERSION = 1
DEFAULT_MIN_QUANT_ELEMENTS = 65536

# substrings of parameter names that are never stored below fp32
PRECISION_CRITICAL = ("layernorm", "layer_norm", ".ln_", ".norm", "beta_anchor", "raw_gamma", "raw_alpha", "logit_scale",
                      "gate_selector", "identity_gate", "tria_agg.reader", "tria_agg.pool")
_QUANT = {"none": None, "off": None, "keep": None, "fp32": torch.float32, "float32": torch.float32,
          "bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "fp16": torch.float16, "float16": torch.float16,
          "half": torch.float16}
_SHORT = {torch.float32: "fp32", torch.float16: "fp16", torch.bfloat16: "bf16", torch.float64: "fp64",
          torch.int64: "int64", torch.int32: "int32", torch.int16: "int16", torch.int8: "int8", torch.uint8: "uint8",
          torch.bool: "bool"}
MANIFEST_CFG_KEYS = ("vocab", "model_dim", "n_q_heads", "n_kv_heads", "head_dim", "hidden", "layers", "seq_len",
                     "tied_embeddings", "activation", "phase_sectors", "tria_carry_enabled", "tria_temporal_window",
                     "tria_carrier_alpha", "tria_polarm_beta")


def dtype_name(dt: torch.dtype) -> str:
    return _SHORT.get(dt, str(dt).replace("torch.", ""))


def parse_quant(name: str) -> Optional[torch.dtype]:
    key = str(name).strip().lower()
    if key not in _QUANT:
        raise ValueError(f"unsupported --quant {name!r}; use none, fp32, bf16, or fp16")
    return _QUANT[key]


def storage_class(name: str, t: torch.Tensor, min_elements: int) -> str:
    """Why a tensor keeps fp32 (``non-floating``/``fp64``/``scalar/vector``/``small``/``bias``/``critical``) or
    ``matrix`` when it may be cast down."""
    low = name.lower()
    if not t.is_floating_point():
        return "non-floating"
    if t.dtype == torch.float64:
        return "fp64"
    if t.ndim < 2:
        return "scalar/vector"
    if t.numel() < min_elements:
        return "small"
    if low == "bias" or low.endswith(".bias"):
        return "bias"
    if any(m in low for m in PRECISION_CRITICAL):
        return "critical"
    return "matrix"


def _alias_key(t: torch.Tensor):
    if t.device.type != "cpu" or t.layout != torch.strided:
        return None
    return (t.untyped_storage().data_ptr(), t.storage_offset(), tuple(t.shape), tuple(t.stride()), t.dtype)


def convert_state(state: Mapping[str, Any], target: Optional[torch.dtype], min_elements: int) -> Tuple[Dict[str, Any], Dict]:
    out: Dict[str, Any] = {}
    seen: Dict[Any, torch.Tensor] = {}
    why = Counter()
    src_bytes = dst_bytes = changed = kept = 0
    nbytes = lambda t: int(t.numel()) * int(t.element_size())
    for name, val in state.items():
        if not torch.is_tensor(val):
            out[name] = val
            continue
        t = val.detach().cpu()
        src_bytes += nbytes(t)
        key = _alias_key(t)
        if key is not None and key in seen:
            out[name] = seen[key]
            dst_bytes += nbytes(seen[key])
            why["alias"] += 1
            continue
        cls = storage_class(name, t, min_elements)
        if target is None:
            new, cls = t.contiguous(), "unchanged"
        elif cls != "matrix":
            new = t.float().contiguous() if (t.is_floating_point() and t.dtype != torch.float64) else t.contiguous()
            kept += 1
        else:
            new = t.to(target).contiguous()
            changed += int(new.dtype != t.dtype)
        out[name] = new
        dst_bytes += nbytes(new)
        why[cls] += 1
        if key is not None:
            seen[key] = new
    report = {"target_dtype": "none" if target is None else dtype_name(target), "min_quant_elements": int(min_elements),
              "source_bytes": int(src_bytes), "packed_tensor_bytes": int(dst_bytes), "changed_tensors": int(changed),
              "kept_fp32_tensors": int(kept), "decisions": dict(sorted(why.items()))}
    return out, report


def _digest(b: bytes) -> Dict[str, Any]:
    return {"bytes": len(b), "sha256": hashlib.sha256(b).hexdigest()}


def read_checkpoint(path: str) -> Dict[str, Any]:
    blob = torch.load(path, map_location="cpu", weights_only=True)
    if not isinstance(blob, dict):
        raise TypeError("checkpoint must be a mapping")
    if not isinstance(blob.get("model"), Mapping):
        raise ValueError("checkpoint must contain a model state dict under key 'model'")
    if not isinstance(blob.get("cfg"), Mapping):
        raise ValueError("checkpoint must contain configuration under key 'cfg'")
    return blob


def build_package(model_path: str, tokenizer_path: str, template_path: str, output_path: str, quant: str = "none",
                  min_quant_elements: int = DEFAULT_MIN_QUANT_ELEMENTS) -> Dict[str, Any]:
    if min_quant_elements < 1:
        raise ValueError("--min-quant-elements must be positive")
    blob = read_checkpoint(model_path)
    state, report = convert_state(blob["model"], parse_quant(quant), min_quant_elements)
    ck: Dict[str, Any] = {"model_kind": blob.get("model_kind", "loomformer"), "ffn_type": blob.get("ffn_type", "paraplex"),
                          "cfg": dict(blob["cfg"]), "ablation": bool(blob.get("ablation", False)), "model": state}
    for k in ("step", "tokens_seen", "train_loss", "eval_loss"):     # optimizer state is dropped
        if k in blob and (blob[k] is None or isinstance(blob[k], (str, int, float, bool))):
            ck[k] = blob[k]
    tok_bytes, tpl_bytes = Path(tokenizer_path).read_bytes(), Path(template_path).read_bytes()
    cfg = ck["cfg"]
    manifest = {
        "format": FORMAT_NAME, "version": FORMAT_VERSION, "created_unix": int(time.time()),
        "model_kind": ck["model_kind"], "ffn_type": ck["ffn_type"], "ablation": ck["ablation"], "quantization": report,
        "model": {"source_name": os.path.basename(model_path), "state_keys": len(state),
                  "parameters": int(sum(v.numel() for v in state.values() if torch.is_tensor(v))),
                  "step": ck.get("step"), "config": {k: cfg.get(k) for k in MANIFEST_CFG_KEYS if k in cfg}},
        "assets": {"tokenizer": {"name": os.path.basename(tokenizer_path), **_digest(tok_bytes)},
                   "chat_template": {"name": os.path.basename(template_path), **_digest(tpl_bytes)}},
    }
    out = Path(output_path)
    out.parent.mkdir(parents=True, exist_ok=True)
    tmp = out.with_name(out.name + ".tmp")
    torch.save({"format": FORMAT_NAME, "version": FORMAT_VERSION, "manifest": manifest, "checkpoint": ck,
                "tokenizer_json": tok_bytes, "chat_template_jinja": tpl_bytes}, tmp)
    os.replace(tmp, out)
    manifest["archive_bytes"] = out.stat().st_size
    return manifest


def load_aio(path: str, map_location="cpu") -> Dict[str, Any]:
    pkg = torch.load(path, map_location=map_location, weights_only=True)
    if not isinstance(pkg, dict):
        raise TypeError("AIO package is not a mapping")
    if pkg.get("format") != FORMAT_NAME:
        raise ValueError(f"not a {FORMAT_NAME} package")
    if int(pkg.get("version", -1)) != FORMAT_VERSION:
        raise ValueError(f"unsupported AIO version {pkg.get('version')!r}")
    return pkg


def inspect_package(path: str, show_keys: bool = False) -> None:
    pkg = load_aio(path)
    print(json.dumps(pkg["manifest"], ensure_ascii=False, indent=2, sort_keys=True))
    if show_keys:
        for name, v in pkg["checkpoint"]["model"].items():
            if torch.is_tensor(v):
                print(f"{name:72s} {str(tuple(v.shape)):24s} {dtype_name(v.dtype)}")
            else:
                print(f"{name:72s} {type(v).__name__}")


def extract_package(path: str, directory: str) -> None:
    pkg = load_aio(path)
    out = Path(directory)
    out.mkdir(parents=True, exist_ok=True)
    torch.save(pkg["checkpoint"], out / "model.pt")
    (out / "tokenizer.json").write_bytes(pkg["tokenizer_json"])
    (out / "chat_template.jinja").write_bytes(pkg["chat_template_jinja"])
    (out / "manifest.json").write_text(json.dumps(pkg["manifest"], ensure_ascii=False, indent=2, sort_keys=True) + "\n",
                                       encoding="utf-8")


def size_text(n: int) -> str:
    x = float(n)
    for unit in ("B", "KiB", "MiB", "GiB", "TiB"):
        if x < 1024.0 or unit == "TiB":
            return f"{x:.1f} {unit}"
        x /= 1024.0
    return f"{n} B"
