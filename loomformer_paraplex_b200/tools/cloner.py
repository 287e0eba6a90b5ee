"""Donor transplant: read a Hugging Face decoder checkpoint, emit a LoomFormer YAML whose shapes receive it (``scan``),
then build a LoomFormer checkpoint carrying the donor's matrices (``clone``).  Which donor tensor goes where, and which
learning rate each transplanted tensor gets, is data: a ``mappings/<family>.json`` file
(reference ``loomcloner.py:24-66, 73-93, 264-372, 387-434``)."""
from __future__ import annotations

import json
import mmap
import os
import struct
from pathlib import Path
from typing import Any, Dict, List, Optional, Tuple

import torch
import yaml

from ..config import Config, resolve

BOOKKEEPING = ("cloned", "cloned_from", "cloned_mapping", "train_lr")
# which axis of an FFN matrix is the hidden width (zero-padded when the donor's width is not a multiple of n_q_heads)
HIDDEN_AXIS = {"ffn.w1_real.weight": 0, "ffn.gate_proj.weight": 0, "ffn.w2.weight": 1}
_ST_DTYPES = {"F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "F64": torch.float64,
              "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
              "BOOL": torch.bool}


# ------------------------------------------------------------------ donor files
def load_json(path: str) -> Dict[str, Any]:
    with open(path, encoding="utf-8") as fh:
        return json.load(fh)


def donor_config(donor_dir: str) -> Dict[str, Any]:
    return load_json(os.path.join(donor_dir, "config.json"))


def safetensors_header(path: str) -> Tuple[Dict[str, Any], int]:
    """The JSON header of a safetensors file and the byte offset where tensor data starts (no tensor bytes read)."""
    with open(path, "rb") as fh:
        n = struct.unpack("<Q", fh.read(8))[0]
        head = json.loads(fh.read(n))
    head.pop("__metadata__", None)
    return head, 8 + n


def safetensors_files(donor_dir: str) -> List[str]:
    one = os.path.join(donor_dir, "model.safetensors")
    if os.path.exists(one):
        return [one]
    shards = sorted(str(p) for p in Path(donor_dir).glob("model-*-of-*.safetensors"))
    if not shards:
        raise FileNotFoundError(f"no model.safetensors or sharded safetensors files found in {donor_dir}")
    return shards


def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    """All tensors of one file, copied out of a read-only memory map."""
    head, base = safetensors_header(path)
    out: Dict[str, torch.Tensor] = {}
    with open(path, "rb") as fh, mmap.mmap(fh.fileno(), 0, access=mmap.ACCESS_READ) as mm:
        for name, meta in head.items():
            lo, hi = meta["data_offsets"]
            dt = _ST_DTYPES[meta["dtype"]]
            buf = bytearray(mm[base + lo: base + hi])
            t = torch.frombuffer(buf, dtype=dt) if hi > lo else torch.empty(0, dtype=dt)
            out[name] = t.reshape(meta["shape"])
    return out


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor]) -> None:
    """Minimal writer (used to fabricate donors in tests and to export weights)."""
    names = {v: k for k, v in _ST_DTYPES.items()}
    head, blobs, at = {}, [], 0
    for k, t in tensors.items():
        raw = t.detach().contiguous().cpu().view(torch.uint8).numpy().tobytes() if t.numel() else b""
        head[k] = {"dtype": names[t.dtype], "shape": list(t.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    js = json.dumps(head, separators=(",", ":")).encode()
    js += b" " * (-len(js) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(js)))
        fh.write(js)
        for b in blobs:
            fh.write(b)


def detect_mapping(cfg: Dict[str, Any], mappings_dir: str) -> str:
    archs = set(cfg.get("architectures", []))
    for p in sorted(Path(mappings_dir).glob("*.json")):
        if archs & set(load_json(str(p)).get("detect", {}).get("any_of", [])):
            return str(p)
    raise ValueError(f"no mapping in {mappings_dir} declares support for architectures={sorted(archs)}; "
                     f"pass --mapping explicitly or add a mappings/*.json for this family")


# ------------------------------------------------------------------ scan: donor config -> YAML
def derive_fields(donor: Dict[str, Any], mapping: Dict[str, Any]) -> Dict[str, Any]:
    out = {ours: donor[theirs] for theirs, ours in mapping.get("config_map", {}).items() if theirs in donor}
    ratio = mapping.get("hidden_from")
    if ratio:
        out[ratio["target_field"]] = donor[ratio["numerator"]] / donor[ratio["denominator"]]      # exact, unrounded
    hd = mapping.get("head_dim_from")
    if hd:
        num, den = donor[hd["numerator"]], donor[hd["denominator"]]
        if num % den:
            raise ValueError(f"head_dim would be non-integer: {num}/{den} -- donor shape assumption violated")
        out["head_dim"] = num // den
    return out


def hidden_width(model_dim: int, hidden_mult: float, n_q_heads: int) -> int:
    """Smallest multiple of ``n_q_heads`` not below ``round(model_dim * hidden_mult)``."""
    return -(-round(model_dim * hidden_mult) // n_q_heads) * n_q_heads


def scan_to_yaml(donor: Dict[str, Any], mapping: Dict[str, Any], donor_dir: str, tokenizer_path: str, dataset: str,
                 steps: int, lr: float, gate_proj: bool, final_norm: bool) -> str:
    f = derive_fields(donor, mapping)
    n, qh, hd, layers = int(f["model_dim"]), int(f["n_q_heads"]), int(f["head_dim"]), int(f["layers"])
    kvh = int(f.get("n_kv_heads", qh))
    mult = float(f["hidden_mult"])
    ctx = int(f.get("rope_original_seq_len", 2048))
    hidden = hidden_width(n, mult, qh)
    donor_hidden = donor.get(mapping.get("hidden_from", {}).get("numerator", ""))
    name = donor.get("_name_or_path") or os.path.basename(os.path.normpath(donor_dir))
    family = mapping.get("family", "?")
    sections: List[Tuple[Optional[str], Dict[str, Any]]] = [
        (None, dict(optimizer="atom", steps=steps, lr=float(f"{lr:g}"), weight_decay=0.01, grad_clip=1.55,
                    warmup_steps=max(1, steps // 30), min_lr_frac=0.1, seed=1, log_every=10, eval_every=50, eval_batches=4,
                    device="cuda:0", grad_accum_steps=1, grad_checkpointing=False, graph=False, save_graph=False,
                    amp_dtype="bf16", save_every=500, runpoints_path=None)),
        (None, dict(seq_len=ctx, batch_size=8, prefetch_batches=256)),
        (None, dict(rope_theta=float(f.get("rope_theta", 10000.0)), rope_original_seq_len=ctx, rope_factor=1.0,
                    rope_beta_fast=32.0, rope_beta_slow=1.0, rope_attention_factor=None)),
        (None, dict(tria_carry_enabled=True, use_cuda_tria=True, tria_gamma_max=0.80, tria_raw_gamma_init=0.25,
                    tria_temporal_enabled=True, tria_temporal_auto=False, tria_temporal_window=128,
                    tria_temporal_window_min=32, tria_target_refeeds_per_sequence=7, tria_min_refeeds_per_sequence=1,
                    tria_carrier_alpha=0.0375, tria_polarm_beta=0.1,
                    tria_carrier_alpha_candidates=[0.0125, 0.025, 0.0375, 0.05, 0.0625, 0.075],
                    tria_temporal_max_condition=3.0, tria_temporal_min_effective_rank=2.70,
                    tria_temporal_population_pass_fraction=0.90, tria_temporal_calib_seeds=1, tria_temporal_calib_batch=1,
                    tria_temporal_calib_tokens=512, tria_temporal_calib_device="auto",
                    tria_temporal_calib_parallel_sweep=2)),
        ("the donor's own tokenizer: with any other one the embedding and head matrices could not be transplanted",
         dict(tokenizer=tokenizer_path, vocab=int(f["vocab"]), tied_embeddings=bool(f.get("tied_embeddings", False)))),
        ("train_dataset is a placeholder: point it at a real corpus before training",
         dict(train_dataset=dataset, val_dataset=None, auto_val_split_pct=1.0, dataset_format="arrow", text_field="text",
              dataset_cache=None)),
        (f"d_model = {qh} * {hd} = {qh * hd}; hidden = round_up(model_dim * hidden_mult, n_q_heads); hidden_mult is the "
         f"donor's intermediate_size / hidden_size, unrounded",
         dict(model_dim=n, n_q_heads=qh, head_dim=hd, n_kv_heads=kvh, gqa_group_size=None, hidden=hidden,
              hidden_mult=float(f"{mult:.6f}"), layers=layers)),
    ]
    if donor_hidden is not None and donor_hidden != hidden:
        sections.append((f"NOTE: donor intermediate_size={donor_hidden} is not divisible by n_q_heads={qh}; the per-head phase "
                         f"sectors need hidden % n_q_heads == 0, so hidden is rounded up to {hidden} and --clone zero-pads "
                         f"up_proj/gate_proj/down_proj by {hidden - donor_hidden} channel(s). Zero channels contribute "
                         f"nothing until trained; truncating would discard trained donor weights.", {}))
    sections += [
        ("LoomFormer-only parts (depth attention, residual cap, phase machinery) have no donor counterpart and keep "
         "their own initialisation",
         dict(phase_sectors="head", residual_init="beta", depth_attn_readout="per-sublayer", depth_attn_qkv_rms=True,
              residual_branch_rms_cap=1.0, activation="pvpowlu", powlu_m=3.0, phase_grad_floor=0.05,
              phase_grad_mode="secant", attn_impl="sdpa")),
        ("gate_proj: " + ("transplanted from the donor's SwiGLU gate" if gate_proj else "donor gate_proj is DROPPED")
         + "; final_norm: " + ("model.norm.weight lands on ln_final (exact RMSNorm match)" if final_norm
                               else "donor model.norm.weight is DROPPED"),
         dict(paraplex_gate_proj=bool(gate_proj), final_norm=bool(final_norm))),
        (None, dict(use_cuda_beta_space=True, use_cuda_phase_sin=True, use_cuda_pvpowlu=True, use_cuda_depth_attn=True)),
        ("===AUTO GENERATED=== clone bookkeeping. train_lr entries use LoomFormer parameter names with the blocks.N. "
         "prefix removed (one entry covers every layer) or exact global names; the trainer turns them into "
         "requires_grad flags and per-tensor learning rates",
         dict(cloned=True, cloned_from=name, cloned_mapping=family)),
    ]
    lines = [f"# {name} -- clone", f"# ===AUTO GENERATED=== by loomcloner.py --scan, from {os.path.join(donor_dir, 'config.json')}",
             f"# mapping: {family}"]
    for note, body in sections:
        lines.append("")
        if note:
            lines += [f"# {ln}" for ln in _wrap(note, 100)]
        if body:
            lines += [f"{k}: {_scalar(v)}" for k, v in body.items()]
    lines.append("train_lr:")
    for ov in mapping.get("train_lr_overrides", []):
        tail = f"  # {ov['note']}" if ov.get("note") else ""
        lines += [f"  - name: {ov['pattern']}", f"    train: {'yes' if ov.get('train', True) else 'no'}",
                  f"    lr: {lr * float(ov.get('lr_scale', 1.0)):.2e}{tail}"]
    return "\n".join(lines) + "\n"


def _scalar(v: Any) -> str:
    """One-line YAML for a scalar or a flat list."""
    text = yaml.safe_dump(v, default_flow_style=True, width=1000).strip()
    return text[:-3].strip() if text.endswith("...") else text


def _wrap(text: str, width: int) -> List[str]:
    out, cur = [], ""
    for w in text.split():
        if cur and len(cur) + 1 + len(w) > width:
            out.append(cur)
            cur = w
        else:
            cur = f"{cur} {w}".strip()
    return out + ([cur] if cur else [])


# ------------------------------------------------------------------ clone: donor tensors -> LoomFormer state
def pad_axis(t: torch.Tensor, size: int, axis: int) -> torch.Tensor:
    have = t.shape[axis]
    if have == size:
        return t
    if have > size:
        raise ValueError(f"donor hidden width {have} > target {size} on axis {axis} -- this function only pads up, never "
                         f"truncates; check the --scan-computed 'hidden' value")
    shape = list(t.shape)
    shape[axis] = size - have
    return torch.cat([t, t.new_zeros(shape)], dim=axis)


def _rule_applies(rule: Dict[str, Any], cfg: Config) -> bool:
    need = rule.get("requires_config") or {}
    return all(bool(getattr(cfg, k, False)) == v for k, v in need.items())


def remap(donor: Dict[str, torch.Tensor], mapping: Dict[str, Any], cfg: Config, verbose: bool = True) -> Dict[str, torch.Tensor]:
    out: Dict[str, torch.Tensor] = {}
    dropped: List[str] = []
    hidden = int(cfg.hidden) if cfg.hidden else None
    for i in range(int(cfg.layers)):
        qkv: Dict[str, torch.Tensor] = {}
        for suffix, rule in mapping.get("per_layer", {}).items():
            key = f"model.layers.{i}.{suffix}"
            if key not in donor:
                continue
            op = rule["op"]
            if op == "drop" or not _rule_applies(rule, cfg):
                dropped.append(key)
            elif op == "copy":
                t = donor[key]
                if rule["to"] in HIDDEN_AXIS and hidden is not None:
                    t = pad_axis(t, hidden, HIDDEN_AXIS[rule["to"]])
                out[f"blocks.{i}.{rule['to']}"] = t
            elif op == "qkv_concat":
                qkv[rule["part"]] = donor[key]
            else:
                raise ValueError(f"unknown op {op!r} for {key}")
        if qkv:
            if sorted(qkv) != ["k", "q", "v"]:
                raise ValueError(f"layer {i}: incomplete qkv parts collected: {sorted(qkv)}")
            out[f"blocks.{i}.attn.qkv_weight"] = torch.cat([qkv["q"], qkv["k"], qkv["v"]], dim=0)
    for key, rule in mapping.get("global", {}).items():
        if key not in donor:
            if verbose and not rule.get("optional", False) and rule.get("op") != "drop":
                print(f"[loomcloner] WARNING: global key {key!r} not found in donor, and not marked optional")
        elif rule["op"] == "drop" or not _rule_applies(rule, cfg):
            dropped.append(key)
        else:
            out[rule["to"]] = donor[key]
    if dropped and verbose:
        print(f"[loomcloner] dropped {len(dropped)} donor tensor(s) with no LoomFormer destination:")
        for k in dropped[:10]:
            print(f"  - {k}")
        if len(dropped) > 10:
            print(f"  ... and {len(dropped) - 10} more")
    return out


def set_resume_field(yaml_path: str, value: str) -> None:
    """Set the top-level ``resume:`` line of a YAML file in place, leaving comments and ordering alone."""
    with open(yaml_path, encoding="utf-8") as fh:
        lines = fh.readlines()
    new = f"resume: {value}\n"
    at = next((i for i, ln in enumerate(lines) if ln.startswith("resume:")), None)
    if at is not None:
        lines[at] = new
    else:
        anchor = next((i for i, ln in enumerate(lines) if ln.startswith("optimizer:")), len(lines))
        lines.insert(anchor, new)
    with open(yaml_path, "w", encoding="utf-8") as fh:
        fh.writelines(lines)


def clone(config_path: str, donor_dir: str, mapping_path: str, out_path: str) -> Dict[str, int]:
    from ..models.loomformer import Model
    with open(config_path, encoding="utf-8") as fh:
        cfg_dict = yaml.safe_load(fh)
    cfg = Config.from_dict({k: v for k, v in cfg_dict.items() if k not in BOOKKEEPING})
    mapping = load_json(mapping_path)
    donor: Dict[str, torch.Tensor] = {}
    for shard in safetensors_files(donor_dir):
        donor.update(read_safetensors(shard))
    donor_dtype = next(iter(donor.values())).dtype
    state = remap(donor, mapping, cfg)
    del donor
    # build in the donor's dtype: a transplant gains nothing from fp32 storage, and the checkpoint stays donor-sized
    prev = torch.get_default_dtype()
    torch.set_default_dtype(donor_dtype if donor_dtype.is_floating_point else prev)
    try:
        model = Model(cfg, dims=resolve(cfg, calibrate=False))
    finally:
        torch.set_default_dtype(prev)
    missing, unexpected = model.load_state_dict(state, strict=False)
    print(f"[loomcloner] built model in {donor_dtype} (matching donor -- not upcast to fp32)")
    print(f"[loomcloner] loaded {len(state) - len(unexpected)} tensors from donor, {len(missing)} LoomFormer-only params "
          f"kept at their own init, {len(unexpected)} unexpected (ignored)")
    if unexpected:
        print(f"[loomcloner] unexpected keys (not in Model, check the mapping): {unexpected[:10]}")
    torch.save({"cfg": cfg_dict, "model_kind": "loomformer", "ffn_type": "paraplex", "ablation": False,
                "model": model.state_dict(), "step": 0, "cloned": True, "cloned_from": cfg_dict.get("cloned_from"),
                "cloned_mapping": cfg_dict.get("cloned_mapping")}, out_path)
    print(f"[loomcloner] saved -> {out_path}")
    set_resume_field(config_path, out_path)
    print(f"[loomcloner] {config_path} updated with resume: {out_path} -- `--train --config {config_path}` alone now "
          f"resumes it, no --resume needed")
    return {"loaded": len(state) - len(unexpected), "missing": len(missing), "unexpected": len(unexpected)}
