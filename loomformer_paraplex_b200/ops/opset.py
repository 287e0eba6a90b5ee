"""Selection of the operator implementation a model runs with.

``select_opset`` returns ``None`` for the composed pure-PyTorch plan (CPU tensors, or when the
caller forces it) and the fused sm_100a plan for CUDA tensors.  A CUDA model never falls back
silently: if the native extension cannot be loaded the error propagates.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

_FORCE_COMPOSED = False


def force_composed(flag: bool = True) -> None:
    """Run CUDA models through the composed PyTorch plan (used to A/B the fused kernels)."""
    global _FORCE_COMPOSED
    _FORCE_COMPOSED = bool(flag)


def select_opset(model, probe: torch.Tensor):
    if _FORCE_COMPOSED or os.environ.get("LOOM_COMPOSED", "0") == "1":
        return None
    if not probe.is_cuda:
        return getattr(model, "ops", None)      # a plan bound explicitly (tests run the fused plan on CPU twins)
    if getattr(model, "ops", None) is None:
        from .fused_plan import FusedPlan
        model.ops = FusedPlan(model)
    return model.ops
