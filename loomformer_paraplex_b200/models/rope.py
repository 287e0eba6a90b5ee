"""YaRN rotary tables (rotate-half convention).

The inverse frequencies blend position interpolation and extrapolation with a linear ramp
between two "correction" dimensions, and the cos/sin tables are pre-multiplied by the YaRN
attention factor ``0.1*ln(factor)+1``; see the reference ``loomformer.py:2899-2985``.
One table is built per model and shared by all layers (the reference keeps a copy per layer).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from ..config import Dims


def yarn_mscale(scale: float, mscale: float = 1.0) -> float:
    return 1.0 if scale <= 1.0 else 0.1 * mscale * math.log(scale) + 1.0


def _correction_dim(rotations: float, dim: int, base: float, max_pos: int) -> float:
    return dim * math.log(max_pos / (rotations * 2.0 * math.pi)) / (2.0 * math.log(base))


def yarn_inv_freq(d: Dims) -> Tuple[torch.Tensor, float]:
    hd = d.hd
    freqs = d.rope_theta ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd)
    extrap, interp = 1.0 / freqs, 1.0 / (d.rope_factor * freqs)
    lo = max(math.floor(_correction_dim(d.rope_beta_fast, hd, d.rope_theta, d.rope_original_seq_len)), 0)
    hi = min(math.ceil(_correction_dim(d.rope_beta_slow, hd, d.rope_theta, d.rope_original_seq_len)), hd - 1)
    hi_f = float(hi) + (0.001 if lo == hi else 0.0)
    ramp = ((torch.arange(hd // 2, dtype=torch.float32) - lo) / (hi_f - lo)).clamp(0.0, 1.0)
    keep = 1.0 - ramp
    inv = interp * (1.0 - keep) + extrap * keep
    factor = d.rope_attention_factor if d.rope_attention_factor is not None else yarn_mscale(d.rope_factor)
    return inv, float(factor)


def build_tables(d: Dims, length: Optional[int] = None, device=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 ``cos``/``sin`` tables of shape ``[length, HD]`` (already scaled by the attention factor)."""
    inv, factor = yarn_inv_freq(d)
    t = torch.arange(length or d.seq_len, dtype=torch.float32)
    ang = torch.outer(t, inv)
    ang = torch.cat((ang, ang), dim=-1)
    cos, sin = ang.cos() * factor, ang.sin() * factor
    if device is not None:
        cos, sin = cos.to(device), sin.to(device)
    return cos, sin
