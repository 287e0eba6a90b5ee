"""Configuration schema and resolved model geometry.

Two objects live here:

* :class:`Config` -- the user-facing YAML schema.  Field names, defaults and the
  "unknown keys are rejected / float strings are coerced / legacy checkpoint keys
  are migrated" behaviour follow the reference schema
  (``loomformer.py:214-450`` in the reference project) so every ``cfg/*.yaml`` written
  for it loads unchanged and checkpoints stay interchangeable.
* :class:`Dims` -- an immutable, fully resolved description of the model geometry
  (``loomformer.py:904-1133`` derives the same quantities into module globals).  Every
  module of this framework receives a ``Dims`` explicitly; there is no process-global
  shape state, so several differently shaped models can coexist in one process
  (calibration sweeps, tests, serving replicas).
"""
from __future__ import annotations

import dataclasses
import json
import math
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

FANIN_GAIN = 0.88


@dataclass
class Config:
    # --- tokenizer / data -------------------------------------------------------
    vocab: int = 256
    tokenizer: Optional[str] = None
    tied_embeddings: bool = True
    doc_reset_attn: bool = True
    device: Optional[str] = None
    train_dataset: Optional[str] = None
    val_dataset: Optional[str] = None
    auto_val_split_pct: float = 0.0
    dataset_format: str = "auto"
    text_field: str = "text"
    seq_len: int = 128
    batch_size: int = 32
    # --- model shape ------------------------------------------------------------
    model_dim: Optional[int] = 12
    n_q_heads: int = 6
    head_dim: Optional[int] = None
    n_kv_heads: Optional[int] = 3
    gqa_group_size: Optional[int] = None
    hidden: Optional[int] = 66
    hidden_mult: Optional[float] = None
    layers: int = 3
    phase_sectors: str = "head"
    residual_init: str = "beta"
    depth_attn_readout: str = "shared"
    depth_attn_qkv_rms: bool = False
    residual_branch_rms_cap: Optional[float] = None
    activation: str = "gelu"
    powlu_m: float = 3.0
    phase_grad_floor: float = 0.05
    phase_grad_mode: str = "floor"
    use_cuda_phase_sin: bool = True
    use_cuda_beta_space: bool = True
    use_cuda_pvpowlu: bool = True
    use_cuda_depth_attn: bool = True
    amp_dtype: str = "fp32"
    dataset_cache: str = "mmap"
    attn_impl: str = "sdpa"
    attn_sdpa_compute_dtype: str = "auto"
    attn_sdpa_value_fusion: bool = True
    attn_sdpa_recompute_backward: bool = False
    rope_theta: float = 10000.0
    rope_factor: float = 4.0
    rope_original_seq_len: Optional[int] = None
    rope_beta_fast: float = 32.0
    rope_beta_slow: float = 1.0
    rope_attention_factor: Optional[float] = None
    # --- training ---------------------------------------------------------------
    steps: int = 2000
    lr: float = 2e-3
    weight_decay: float = 0.01
    grad_clip: float = 1.0
    grad_accum_steps: int = 1
    prefetch_batches: int = 256
    gpu_prefetch_batches: int = 8
    grad_checkpointing: bool = False
    save_every: int = 0
    runpoints_path: Optional[str] = None
    save_initial_checkpoint: bool = False
    tria_carry_enabled: bool = False
    cloned: bool = False
    cloned_from: Optional[str] = None
    cloned_mapping: Optional[str] = None
    train_lr: Optional[List[Dict[str, Any]]] = None
    resume: Optional[str] = None
    resume_data_stream: str = "auto"
    paraplex_gate_proj: bool = False
    final_norm: bool = False
    use_cuda_tria: bool = False
    graph: bool = False
    save_graph: bool = False
    tria_temporal_enabled: bool = True
    tria_temporal_window: Optional[int] = None
    tria_temporal_window_min: int = 32
    tria_temporal_window_max: Optional[int] = None
    tria_temporal_calibration: Optional[str] = None
    tria_temporal_auto: bool = True
    tria_carrier_alpha: float = 0.05
    tria_carrier_alpha_candidates: Optional[List[float]] = None
    tria_polarm_beta: float = 0.1
    tria_min_refeeds_per_sequence: int = 1
    tria_temporal_max_condition: float = 3.0
    tria_temporal_min_effective_rank: float = 2.70
    tria_temporal_population_pass_fraction: float = 0.90
    tria_temporal_calib_seeds: int = 3
    tria_temporal_calib_batch: int = 4
    tria_temporal_calib_tokens: Optional[int] = None
    tria_temporal_calib_device: str = "auto"
    tria_temporal_calib_parallel_sweep: int = 1
    tria_target_refeeds_per_sequence: int = 3
    tria_gamma_max: float = 0.25
    tria_raw_gamma_init: float = 0.0
    warmup_steps: int = 100
    min_lr_frac: float = 0.1
    seed: int = 1
    log_every: int = 100
    eval_every: Optional[int] = None
    eval_batches: int = 4
    optimizer: str = "adamw"

    # ------------------------------------------------------------------ builders
    def summary(self) -> str:
        hd = "auto" if self.head_dim is None else self.head_dim
        grp = "auto" if self.gqa_group_size is None else self.gqa_group_size
        return (f"LoomFormer [V={self.vocab} d_model={self.model_dim} qh={self.n_q_heads} "
                f"head_dim={hd} kvh={self.n_kv_heads} group={grp} "
                f"H={self.hidden} D={self.layers} T={self.seq_len} B={self.batch_size}]")

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "Config":
        fields = {f.name: f for f in dataclasses.fields(cls)}
        extra = sorted(k for k in raw if k not in fields)
        if extra:
            raise ValueError(f"unknown config field(s): {extra}")
        vals = dict(raw)
        for name, f in fields.items():
            if "float" in str(f.type) and isinstance(vals.get(name), str):
                vals[name] = float(vals[name])
        return cls(**vals)

    @classmethod
    def from_yaml(cls, path: str) -> "Config":
        import yaml
        with open(path, encoding="utf-8") as fh:
            return cls.from_dict(yaml.safe_load(fh) or {})

    @classmethod
    def from_checkpoint_dict(cls, raw: Dict[str, Any]) -> "Config":
        """Accept a ``cfg`` dict stored in a checkpoint, including older key spellings."""
        vals = dict(raw)
        old_w = vals.pop("tria_temporal_deadline", None)
        new_w = vals.get("tria_temporal_window")
        if old_w is not None and new_w is not None and int(old_w) != int(new_w):
            raise ValueError("checkpoint has conflicting tria_temporal_window/tria_temporal_deadline values: "
                             f"{new_w!r} vs {old_w!r}")
        if new_w is None and old_w is not None:
            vals["tria_temporal_window"] = int(old_w)
        if vals.pop("baseline_hidden", None) is not None:
            raise ValueError("checkpoint requests removed GeluFFN baseline_hidden")
        if bool(vals.pop("train_baseline", False)):
            raise ValueError("checkpoint requests removed GeluFFN baseline training")
        vals = {k: v for k, v in vals.items() if not k.startswith("_")}
        return cls.from_dict(vals)

    def to_dict(self) -> Dict[str, Any]:
        return {k: v for k, v in dataclasses.asdict(self).items() if not k.startswith("_")}


def _norm_choice(value: Any, default: str) -> str:
    return str(value or default).strip().lower()


_AMP_ALIASES = {"float32": "fp32", "bfloat16": "bf16", "float16": "fp16", "half": "fp16",
                "none": "off", "false": "off", "0": "off", "no": "off"}
_SDPA_ALIASES = {"none": "model", "native": "model", "float32": "fp32", "float16": "fp16",
                 "half": "fp16", "bfloat16": "bf16"}


@dataclass(frozen=True)
class Dims:
    """Resolved model geometry (all derived quantities, validated)."""

    vocab: int
    seq_len: int
    n: int                 # model width
    qh: int                # query heads
    kvh: int               # key/value heads
    group: int             # query heads per kv head
    hd: int                # head dim
    hidden: int            # FFN hidden width (multiple of qh)
    hpq: int               # hidden neurons per query head
    kv_dim: int
    imag_in: int           # live fan-in of one w1_imag row
    layers: int
    tied: bool
    open_sectors: bool
    residual_init: str
    depth_readout_per_sublayer: bool
    depth_qkv_rms: bool
    branch_rms_cap: Optional[float]
    activation: str
    powlu_m: float
    phase_floor: float
    phase_secant: bool
    gate_proj: bool
    final_norm: bool
    tria: bool
    tria_temporal: bool
    tria_window: int
    tria_alpha: float
    tria_polarm_beta: float
    tria_gamma_max: float
    tria_raw_gamma_init: float
    rope_theta: float
    rope_factor: float
    rope_original_seq_len: int
    rope_beta_fast: float
    rope_beta_slow: float
    rope_attention_factor: Optional[float]
    grad_checkpointing: bool
    amp_dtype: str
    attn_impl: str
    deepnorm_beta: float

    @property
    def n_sub(self) -> int:
        return 2 * self.layers

    def fanin_std(self, fan_in: int) -> float:
        if fan_in <= 0:
            raise ValueError(f"fan_in must be positive, got {fan_in}")
        return FANIN_GAIN / math.sqrt(float(fan_in))

    def residual_std(self, fan_in: int) -> float:
        return self.fanin_std(fan_in) * (self.deepnorm_beta if self.residual_init == "beta" else 1.0)


def resolve(cfg: Config, *, calibrate: bool = True) -> Dims:
    """Validate ``cfg``, write the resolved values back into it and return the geometry.

    Mirrors the validation messages and derivations of the reference's ``apply_config``
    (``loomformer.py:904-1133``) without touching global state.  ``calibrate=False`` skips
    the Tria start-up sweep (used by the sweep itself and by tools that only need shapes).
    """
    qh, layers, vocab, seq = int(cfg.n_q_heads), int(cfg.layers), int(cfg.vocab), int(cfg.seq_len)
    if qh <= 0 or layers <= 0 or vocab <= 0 or seq <= 0:
        raise ValueError("model/data dimensions must be positive")
    if int(cfg.prefetch_batches) <= 0 or int(cfg.gpu_prefetch_batches) <= 0:
        raise ValueError("prefetch_batches and gpu_prefetch_batches must be positive")
    tria_on = bool(cfg.tria_carry_enabled)
    temporal = bool(cfg.tria_temporal_enabled)
    if tria_on and not temporal:
        raise ValueError("tria_carry_enabled requires tria_temporal_enabled")
    cfg.use_cuda_tria = bool(cfg.use_cuda_tria)

    if cfg.head_dim is not None:
        hd = int(cfg.head_dim)
        if hd <= 0:
            raise ValueError("head_dim must be positive")
        n = qh * hd
        if cfg.model_dim is not None and int(cfg.model_dim) != n:
            raise ValueError(f"inconsistent shape: model_dim={int(cfg.model_dim)} but "
                             f"n_q_heads*head_dim={qh}*{hd}={n}")
    elif cfg.model_dim is None:
        hd, n = 32, qh * 32
    else:
        n = int(cfg.model_dim)
        if n <= 0:
            raise ValueError("model_dim must be positive")
        if n % qh:
            raise ValueError("model_dim must be divisible by n_q_heads, or set head_dim")
        hd = n // qh

    if cfg.gqa_group_size is not None and cfg.n_kv_heads is not None:
        group, kvh = int(cfg.gqa_group_size), int(cfg.n_kv_heads)
        if group * kvh != qh:
            raise ValueError(f"inconsistent GQA: n_kv_heads*group={kvh}*{group} != n_q_heads={qh}")
    elif cfg.gqa_group_size is not None:
        group = int(cfg.gqa_group_size)
        if group <= 0 or qh % group:
            raise ValueError("gqa_group_size must divide n_q_heads")
        kvh = qh // group
    elif cfg.n_kv_heads is not None:
        kvh = int(cfg.n_kv_heads)
        if kvh <= 0 or qh % kvh:
            raise ValueError("n_kv_heads must divide n_q_heads")
        group = qh // kvh
    else:
        group = 4 if qh % 4 == 0 else (2 if qh % 2 == 0 else 1)
        kvh = qh // group

    if cfg.hidden is None:
        mult = 4.0 if cfg.hidden_mult is None else float(cfg.hidden_mult)
        want = max(qh, int(round(n * mult)))
        hidden = -(-want // qh) * qh
    else:
        hidden = int(cfg.hidden)
    if hidden <= 0:
        raise ValueError("hidden must be positive")
    if hidden % qh:
        raise ValueError("hidden must be divisible by n_q_heads")
    if hd % 2:
        raise ValueError("head_dim must be even for rotary attention")

    attn_impl = _norm_choice(cfg.attn_impl, "sdpa")
    if attn_impl not in ("sdpa", "manual"):
        raise ValueError(f"attn_impl must be 'sdpa' or 'manual', got {attn_impl!r}")

    theta = 10000.0 if cfg.rope_theta is None else float(cfg.rope_theta)
    factor = 4.0 if cfg.rope_factor is None else float(cfg.rope_factor)
    orig = seq if cfg.rope_original_seq_len is None else int(cfg.rope_original_seq_len)
    bfast = 32.0 if cfg.rope_beta_fast is None else float(cfg.rope_beta_fast)
    bslow = 1.0 if cfg.rope_beta_slow is None else float(cfg.rope_beta_slow)
    attn_factor = None if cfg.rope_attention_factor is None else float(cfg.rope_attention_factor)
    if theta <= 0.0 or factor <= 0.0 or orig <= 0:
        raise ValueError("rope_theta, rope_factor and rope_original_seq_len must be positive")
    if bfast <= 0.0 or bslow <= 0.0:
        raise ValueError("rope_beta_fast and rope_beta_slow must be positive")
    cfg.rope_theta, cfg.rope_factor, cfg.rope_original_seq_len = theta, factor, orig
    cfg.rope_beta_fast, cfg.rope_beta_slow, cfg.rope_attention_factor = bfast, bslow, attn_factor

    res_init = _norm_choice(cfg.residual_init, "beta")
    if res_init not in ("beta", "fanin"):
        raise ValueError(f"residual_init must be 'beta' or 'fanin', got {res_init!r}")
    readout = _norm_choice(cfg.depth_attn_readout, "shared")
    if readout not in ("shared", "per-sublayer"):
        raise ValueError(f"depth_attn_readout must be 'shared' or 'per-sublayer', got {readout!r}")
    cap = None if cfg.residual_branch_rms_cap is None else float(cfg.residual_branch_rms_cap)
    if cap is not None and cap <= 0.0:
        raise ValueError("residual_branch_rms_cap must be positive or null")
    act = _norm_choice(cfg.activation, "gelu")
    if act not in ("gelu", "powlu", "pvpowlu"):
        raise ValueError(f"activation must be 'gelu', 'powlu' or 'pvpowlu', got {act!r}")
    mode = _norm_choice(cfg.phase_grad_mode, "floor")
    if mode not in ("floor", "secant"):
        raise ValueError(f"phase_grad_mode must be 'floor' or 'secant', got {mode!r}")
    amp = _norm_choice(cfg.amp_dtype, "fp32")
    amp = _AMP_ALIASES.get(amp, amp)
    if amp not in ("bf16", "fp32", "fp16", "off"):
        raise ValueError(f"amp_dtype must be bf16, fp32/off, or fp16, got {amp!r}")
    cfg.amp_dtype = amp
    sdpa_dt = _norm_choice(cfg.attn_sdpa_compute_dtype, "auto")
    sdpa_dt = _SDPA_ALIASES.get(sdpa_dt, sdpa_dt)
    if sdpa_dt not in ("auto", "model", "fp32", "fp16", "bf16"):
        raise ValueError("attn_sdpa_compute_dtype must be auto, model, fp32, fp16, or bf16; "
                         f"got {sdpa_dt!r}")
    cfg.attn_impl, cfg.attn_sdpa_compute_dtype = attn_impl, sdpa_dt
    sectors = _norm_choice(cfg.phase_sectors, "head")
    if sectors not in ("head", "open"):
        raise ValueError(f"phase_sectors must be 'head' or 'open', got {sectors!r}")
    imag_in = (n + 4 * hd) if sectors == "head" else (4 * n + hd)

    cfg.model_dim, cfg.head_dim, cfg.n_kv_heads, cfg.gqa_group_size, cfg.hidden = n, hd, kvh, group, hidden

    alpha = float(cfg.tria_carrier_alpha)
    if not math.isfinite(alpha) or alpha <= 0.0:
        raise ValueError(f"tria_carrier_alpha must be finite and > 0, got {alpha}")
    pbeta = float(cfg.tria_polarm_beta)
    if not math.isfinite(pbeta) or pbeta < 0.0 or pbeta >= 1.0:
        raise ValueError(f"tria_polarm_beta must be finite and in [0, 1), got {pbeta}")
    cfg.tria_carrier_alpha, cfg.tria_polarm_beta = alpha, pbeta

    if tria_on and temporal and calibrate:
        from .models.calibration import apply_temporal_calibration
        apply_temporal_calibration(cfg)
        alpha = float(cfg.tria_carrier_alpha)
    window = cfg.tria_temporal_window
    if tria_on and window is None:
        raise ValueError("tria_temporal_auto=false requires tria_temporal_window; "
                         "auto mode selects it during startup calibration")
    window = int(window or seq)
    if window <= 0:
        raise ValueError("tria_temporal_window must be positive")
    if calibrate or cfg.tria_temporal_window is not None:
        cfg.tria_temporal_window = window

    return Dims(
        vocab=vocab, seq_len=seq, n=n, qh=qh, kvh=kvh, group=group, hd=hd, hidden=hidden,
        hpq=hidden // qh, kv_dim=kvh * hd, imag_in=imag_in, layers=layers,
        tied=bool(cfg.tied_embeddings), open_sectors=(sectors == "open"), residual_init=res_init,
        depth_readout_per_sublayer=(readout == "per-sublayer"), depth_qkv_rms=bool(cfg.depth_attn_qkv_rms),
        branch_rms_cap=cap, activation=act, powlu_m=float(cfg.powlu_m or 3.0),
        phase_floor=max(float(cfg.phase_grad_floor or 0.0), 0.0), phase_secant=(mode == "secant"),
        gate_proj=bool(cfg.paraplex_gate_proj), final_norm=bool(cfg.final_norm),
        tria=tria_on, tria_temporal=temporal, tria_window=window, tria_alpha=alpha, tria_polarm_beta=pbeta,
        tria_gamma_max=float(cfg.tria_gamma_max), tria_raw_gamma_init=float(cfg.tria_raw_gamma_init),
        rope_theta=theta, rope_factor=factor, rope_original_seq_len=orig, rope_beta_fast=bfast,
        rope_beta_slow=bslow, rope_attention_factor=attn_factor,
        grad_checkpointing=bool(cfg.grad_checkpointing), amp_dtype=amp, attn_impl=attn_impl,
        deepnorm_beta=(8.0 * max(1, layers)) ** -0.25,
    )


def imag_live_columns(d: Dims, head: int) -> List[int]:
    """Columns of the virtual dense ``[Q | Kctx | C | U | D]`` operand (width 5N) that one
    ``w1_imag`` row of query-head group ``head`` reads, in storage order.

    head sectors: ``[Q_g | Kctx_g | C_g | U(0..N) | D_g]``; open sectors:
    ``[Q_g | Kctx(all) | C(all) | U | D(all)]`` (reference ``loomformer.py:871-900``).
    """
    n, hd = d.n, d.hd
    own = range(head * hd, (head + 1) * hd)
    full = range(n)
    parts = [own, full if d.open_sectors else own, full if d.open_sectors else own, full,
             full if d.open_sectors else own]
    cols: List[int] = []
    for sector, part in enumerate(parts):
        cols.extend(sector * n + c for c in part)
    assert len(cols) == d.imag_in
    return cols


def load_calibration_json(path: str) -> Dict[str, Any]:
    with open(path, encoding="utf-8") as fh:
        blob = json.load(fh)
    src = blob.get("recommended", blob)
    if "tria_temporal_window" not in src:
        raise ValueError(f"{path!r} is missing temporal Tria calibration keys: ['tria_temporal_window']")
    return src
