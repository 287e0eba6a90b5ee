"""Checkpoint I/O, bit-compatible with the reference layout.

A checkpoint is one ``torch.save`` dict: ``cfg`` (dataclass dict with the GLOBAL batch size and
``tria_temporal_auto=False`` once a window is resolved), ``model_kind="loomformer"``, ``ffn_type="paraplex"``,
``ablation``, ``model`` (state_dict), ``optimizer_name``, ``optimizer``, ``step``, ``tokens_seen``.
Loading validates kind / FFN type / ablation, canonicalises legacy key spellings (separate q/k/v and depth k/v
weights, ``_tria_reader.*`` aliases) and is strict (reference ``loomformer.py:4363-4432, 4481-4523, 4981-5018``).
"""
from __future__ import annotations

import os
from typing import Any, Dict, Optional, Tuple

import torch

from ..parallel.dist import rank0_print


def canonicalize_state_dict(state: dict, layers: int) -> dict:
    state = dict(state)
    for old, new in (("_tria_reader.proj.weight", "tria_agg.reader.proj.weight"),
                     ("_tria_reader.proj.bias", "tria_agg.reader.proj.bias"),
                     ("_tria_reader.key_proj.weight", "tria_agg.reader.key_proj.weight")):
        v = state.pop(old, None)
        if v is None:
            continue
        cur = state.get(new)
        if cur is not None and not torch.equal(v, cur):
            raise ValueError(f"checkpoint reader aliases disagree: {old!r} != {new!r}")
        state.setdefault(new, v)
    for i in range(layers):
        pre = f"blocks.{i}.attn."
        parts = [state.get(pre + k) for k in ("q.weight", "k.weight", "v.weight")]
        if any(p is not None for p in parts):
            if not all(p is not None for p in parts):
                raise ValueError(f"incomplete QKV checkpoint group for layer {i}")
            merged = torch.cat(parts, dim=0)
            cur = state.get(pre + "qkv_weight")
            if cur is not None and not torch.equal(cur, merged):
                raise ValueError(f"packed QKV disagrees with legacy weights at layer {i}")
            state[pre + "qkv_weight"] = merged
            for k in ("q.weight", "k.weight", "v.weight"):
                state.pop(pre + k)
    parts = [state.get(k) for k in ("depth_attn.w_k.weight", "depth_attn.w_v.weight")]
    if any(p is not None for p in parts):
        if not all(p is not None for p in parts):
            raise ValueError("incomplete depth K/V checkpoint group")
        merged = torch.cat(parts, dim=0)
        cur = state.get("depth_attn.kv_weight")
        if cur is not None and not torch.equal(cur, merged):
            raise ValueError("packed depth K/V disagrees with legacy weights")
        state["depth_attn.kv_weight"] = merged
        state.pop("depth_attn.w_k.weight"); state.pop("depth_attn.w_v.weight")
    return state


def load_model_blob(model, blob: dict, ablation: bool = False, assign: bool = False) -> None:
    if blob.get("model_kind") != "loomformer":
        raise ValueError(f"checkpoint kind mismatch: expected model_kind='loomformer', got {blob.get('model_kind')!r}")
    if blob.get("ffn_type") != "paraplex":
        raise ValueError(f"checkpoint uses removed FFN type: {blob.get('ffn_type')!r}")
    if bool(blob.get("ablation", False)) != bool(ablation):
        raise ValueError(f"checkpoint ablation mismatch: checkpoint={blob.get('ablation', False)!r}, model={bool(ablation)!r}")
    state = canonicalize_state_dict(blob["model"], model.d.layers)
    if assign:
        model.load_state_dict(state, strict=True, assign=True)
    else:
        # copy into the existing storages so flat-buffer views stay valid
        own = model.state_dict()
        missing = sorted(set(own) - set(state)); extra = sorted(set(state) - set(own))
        if missing or extra:
            raise RuntimeError(f"state_dict mismatch: missing={missing} unexpected={extra}")
        with torch.no_grad():
            for k, v in own.items():
                if v.shape != state[k].shape:
                    raise RuntimeError(f"size mismatch for {k}: checkpoint {tuple(state[k].shape)} vs model {tuple(v.shape)}")
                v.copy_(state[k])


def load_model_checkpoint(model, path: str, ablation: bool, device) -> dict:
    if not os.path.exists(path):
        raise FileNotFoundError(f"resume checkpoint not found: {path}")
    blob = torch.load(path, map_location=device, weights_only=True)
    load_model_blob(model, blob, ablation)
    rank0_print(f"[resume] loaded paraplex weights from {path}")
    return blob


def checkpoint_cfg(cfg) -> Dict[str, Any]:
    d = cfg.to_dict()
    d["batch_size"] = int(getattr(cfg, "_global_batch_size", cfg.batch_size))
    if d.get("tria_temporal_window") is not None:
        d["tria_temporal_auto"] = False
    return d


def save_checkpoint(path: str, cfg, model, optimizer, optimizer_name: str, step: int, tokens_seen: int,
                    ablation: bool = False) -> None:
    # parameters are views into one flat buffer: clone each so the file holds tensors, not the whole buffer per
    # entry, while tensors that alias each other (tied embeddings) stay one tensor in the file
    copies: Dict[Any, torch.Tensor] = {}
    state = {}
    for k, v in model.state_dict().items():
        key = (v.data_ptr(), tuple(v.shape), tuple(v.stride()), v.dtype)
        if key not in copies:
            copies[key] = v.detach().clone().cpu()
        state[k] = copies[key]
    blob = {"cfg": checkpoint_cfg(cfg), "model_kind": "loomformer", "ffn_type": "paraplex", "ablation": bool(ablation),
            "model": state,
            "optimizer_name": optimizer_name, "optimizer": None if optimizer is None else optimizer.state_dict(),
            "step": int(step), "tokens_seen": int(tokens_seen)}
    tmp = path + f".tmp.{os.getpid()}"
    torch.save(blob, tmp)
    os.replace(tmp, path)


def restore_optimizer(optimizer, blob: dict, optimizer_name: str, path: str = "") -> bool:
    """Tensor history comes from the checkpoint; learning rate / weight decay / lr multipliers stay those of the
    active config.  A different optimizer kind starts fresh."""
    saved = blob.get("optimizer")
    if saved is None:
        rank0_print(f"[resume] WARNING: {path!r} has no optimizer state (legacy checkpoint); optimizer starts fresh.")
        return False
    saved_name = str(blob.get("optimizer_name", optimizer_name)).strip().lower()
    if saved_name != str(optimizer_name).strip().lower():
        rank0_print(f"[resume] WARNING: checkpoint optimizer={saved_name!r}, active config optimizer="
                    f"{optimizer_name!r}; optimizer starts fresh.")
        return False
    optimizer.load_state_dict(saved)
    rank0_print(f"[resume] restored {optimizer_name} optimizer state from {path}")
    return True


def tokens_seen_of(blob: dict, completed_steps: int) -> Tuple[int, bool]:
    if blob.get("tokens_seen") is not None:
        return max(0, int(blob["tokens_seen"])), True
    c = blob.get("cfg", {})
    b, t, a = int(c.get("batch_size", 0) or 0), int(c.get("seq_len", 0) or 0), max(1, int(c.get("grad_accum_steps", 1) or 1))
    if b <= 0 or t <= 0:
        return 0, False
    return max(0, int(completed_steps)) * b * t * a, False


def should_replay_data(cfg, dataset: str, saved_cfg: dict) -> Tuple[bool, str]:
    policy = str(cfg.resume_data_stream or "auto").lower()
    if policy not in ("auto", "continue", "restart"):
        raise ValueError(f"resume_data_stream must be auto, continue, or restart; got {policy!r}")
    if policy == "continue":
        return True, "forced by resume_data_stream=continue"
    if policy == "restart":
        return False, "forced by resume_data_stream=restart"
    saved = saved_cfg.get("train_dataset")
    if not saved:
        return True, ("checkpoint has no train_dataset metadata; auto keeps legacy replay "
                      "(use resume_data_stream=restart to force a fresh stream)")
    if os.path.abspath(str(saved)) == os.path.abspath(dataset):
        return True, "train_dataset matches checkpoint"
    return False, f"train_dataset changed ({saved!r} -> {dataset!r})"


def report_tria_geometry(cfg, path: Optional[str]) -> bool:
    """The active config owns the Tria geometry on resume; checkpoint values are only reported."""
    if not path:
        return False
    saved = torch.load(path, map_location="cpu", weights_only=True).get("cfg", {})
    keys = ("tria_temporal_window", "tria_carrier_alpha", "tria_polarm_beta")
    found = {k: saved[k] for k in keys if saved.get(k) is not None}
    if not found:
        return False
    diff = {k: (v, getattr(cfg, k)) for k, v in found.items()
            if getattr(cfg, k) is not None and float(v) != float(getattr(cfg, k))}
    if diff:
        rank0_print("[resume] Tria geometry differs; keeping config SSOT (" +
                    ", ".join(f"{k}: checkpoint={a:g} config={b:g}" for k, (a, b) in diff.items()) + ")")
    else:
        rank0_print("[resume] Tria geometry matches active config")
    return True
