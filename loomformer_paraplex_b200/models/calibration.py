"""Start-up calibration of the Tria temporal window and carrier gain.

For each candidate gain ``alpha`` a few randomly initialised models are run once (flat plan) on
random tokens; the last-layer depth carriers are composed over time and, per position, the
fraction of (batch, neuron) carriers whose singular values satisfy ``cond <= max_condition`` and
``effective_rank >= min_effective_rank`` is measured.  The *stable horizon* of a gain is the
first position where that fraction drops below the required pass fraction.  The largest gain
whose horizon reaches the target window ``seq_len // (target_refeeds + 1)`` wins
(reference ``loomformer.py:483-674``).
"""
from __future__ import annotations

import dataclasses
import math
from typing import Any, Dict, List

import torch

from ..config import Config, load_calibration_json
from ..ops import reference as R


def _log(msg: str) -> None:
    from ..parallel.dist import rank0_print
    rank0_print(msg)


def alpha_candidates(cfg: Config) -> List[float]:
    raw = cfg.tria_carrier_alpha_candidates
    vals = [0.025, 0.0375, 0.05] if raw is None else [float(x) for x in raw]
    vals.append(float(cfg.tria_carrier_alpha))
    out = sorted({x for x in vals if math.isfinite(x) and x > 0.0})
    if not out:
        raise ValueError("tria_carrier_alpha_candidates must contain a positive finite value")
    return out


@torch.no_grad()
def calibrate_from_init(cfg: Config, carry_token_id=None) -> Dict[str, Any]:
    from .loomformer import Model
    seq = int(cfg.seq_len)
    pref = str(cfg.tria_temporal_calib_device or "auto").lower()
    if pref == "auto":
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    else:
        device = torch.device(pref)
        if device.type == "cuda" and not torch.cuda.is_available():
            raise ValueError("tria_temporal_calib_device requests CUDA, but CUDA is unavailable")
    seeds = max(1, int(cfg.tria_temporal_calib_seeds))
    batch = max(1, int(cfg.tria_temporal_calib_batch))
    min_refeeds = max(1, int(cfg.tria_min_refeeds_per_sequence))
    target_refeeds = max(max(1, int(cfg.tria_target_refeeds_per_sequence)), min_refeeds)
    window_min = max(2, int(cfg.tria_temporal_window_min))
    if max(0, (seq - 1) // 2) < min_refeeds:
        raise ValueError(f"seq_len={seq} cannot contain tria_min_refeeds_per_sequence={min_refeeds}; "
                         "increase seq_len or lower the minimum")
    target_w = max(2, seq // (target_refeeds + 1))
    if cfg.tria_temporal_window_max is not None:
        target_w = min(target_w, int(cfg.tria_temporal_window_max))
    T = int(target_w if cfg.tria_temporal_calib_tokens is None else min(seq, int(cfg.tria_temporal_calib_tokens)))
    if T <= 1:
        raise ValueError(f"temporal Tria calibration needs at least 2 tokens, got usable T={T}")
    target_w = min(T, target_w)
    if target_w < window_min:
        _log(f"[tria] requested target refeeds cap W at {target_w}, below "
             f"tria_temporal_window_min={window_min}; preserving the refeed target")
    else:
        target_w = max(window_min, target_w)
    max_cond = float(cfg.tria_temporal_max_condition)
    min_rank = float(cfg.tria_temporal_min_effective_rank)
    need = float(cfg.tria_temporal_population_pass_fraction)
    if max_cond <= 1.0 or not (1.0 <= min_rank <= 3.0):
        raise ValueError("bad Tria stability thresholds")
    if not (0.0 < need <= 1.0):
        raise ValueError("tria_temporal_population_pass_fraction must be in (0,1]")

    results = []
    for alpha in alpha_candidates(cfg):
        ok_sum = torch.zeros(T, device=device)
        cond_sum = torch.zeros(T, device=device)
        rank_sum = torch.zeros(T, device=device)
        count = 0
        for s in range(seeds):
            torch.manual_seed(int(cfg.seed) + 9176 + s)
            trial = dataclasses.replace(cfg, tria_carrier_alpha=float(alpha), tria_temporal_auto=False,
                                        tria_temporal_calibration=None, tria_temporal_window=target_w)
            from ..config import resolve
            model = Model(trial, dims=resolve(trial, calibrate=False)).to(device).eval()
            model.capture_tria_depth_carry = True
            idx = torch.randint(0, int(cfg.vocab), (batch, T), device=device)
            if carry_token_id is not None:
                idx = torch.where(idx.eq(int(carry_token_id)), (idx + 1) % int(cfg.vocab), idx)
            from ..ops.opset import force_composed
            model._forward_flat(idx)
            depth = model.last_tria_depth_carry
            if depth is None:
                raise RuntimeError("temporal Tria auto-calibration requires tria_carry_enabled with paraplex")
            reset = torch.zeros(batch, T, dtype=torch.bool, device=device)
            reset[:, 0] = True
            doc = R.temporal_scan(depth.float(), reset)
            Bc, Tc, H = doc.shape[:3]
            sv = torch.linalg.svdvals(doc.reshape(Bc * Tc, H, 3, 3))
            cond = (sv[..., 0] / sv[..., -1].clamp_min(1e-12)).reshape(Bc, Tc, H)
            prob = sv / sv.sum(-1, keepdim=True).clamp_min(1e-12)
            erank = torch.exp(-(prob * prob.clamp_min(1e-12).log()).sum(-1)).reshape(Bc, Tc, H)
            good = (cond <= max_cond) & (erank >= min_rank)
            ok_sum += good.float().sum(dim=(0, 2))
            cond_sum += cond.sum(dim=(0, 2))
            rank_sum += erank.sum(dim=(0, 2))
            count += Bc * H
            del model
        frac = ok_sum / max(count, 1)
        bad = torch.nonzero(frac < need)
        horizon = T if bad.numel() == 0 else max(1, int(bad[0, 0]))
        results.append({"alpha": float(alpha), "stable_horizon": int(horizon),
                        "pass_fraction": frac.cpu().tolist(),
                        "condition_mean": (cond_sum / max(count, 1)).cpu().tolist(),
                        "effective_rank_mean": (rank_sum / max(count, 1)).cpu().tolist()})
    eligible = [x for x in results if x["stable_horizon"] >= target_w]
    if eligible:
        best = max(eligible, key=lambda x: x["alpha"])
        window, censored = target_w, best["stable_horizon"] >= T
    else:
        best = max(results, key=lambda x: (x["stable_horizon"], -x["alpha"]))
        window, censored = max(2, min(target_w, best["stable_horizon"])), False
    window = max(2, window)
    passed = float(best["pass_fraction"][window - 1])
    if passed < need:
        raise RuntimeError(
            "temporal Tria calibration found no valid window: "
            f"best alpha={best['alpha']:g}, W={window}, condition={best['condition_mean'][window - 1]:.3f}, "
            f"effective_rank={best['effective_rank_mean'][window - 1]:.3f}, "
            f"population_pass={passed:.3f} < {need:.3f}")
    out = {
        "source": "forward_init_carrier", "tria_temporal_window": int(window),
        "tria_carrier_alpha": float(best["alpha"]), "target_window": int(target_w),
        "expected_refeeds_per_sequence": int((seq - 1) // window),
        "target_refeeds_per_sequence": target_refeeds, "stable_horizon": int(best["stable_horizon"]),
        "condition_at_window": float(best["condition_mean"][window - 1]),
        "effective_rank_at_window": float(best["effective_rank_mean"][window - 1]),
        "population_pass_at_window": passed, "max_condition": max_cond, "min_effective_rank": min_rank,
        "required_population_pass": need, "calib_tokens": T, "calib_seeds": seeds, "calib_batch": batch,
        "calib_device": str(device), "censored": censored, "candidates": results,
    }
    _log("[tria] carrier auto-calibration: "
         f"device={device} H={cfg.hidden} L={cfg.layers} T={T} -> alpha={out['tria_carrier_alpha']:g} "
         f"W={window} refeeds={out['expected_refeeds_per_sequence']} cond={out['condition_at_window']:.3f} "
         f"erank={out['effective_rank_at_window']:.3f} pass={passed:.3f}")
    return out


def apply_temporal_calibration(cfg: Config) -> None:
    """Fill ``cfg.tria_temporal_window`` / ``tria_carrier_alpha`` from a JSON file or a sweep."""
    if cfg.tria_temporal_calibration:
        src = load_calibration_json(cfg.tria_temporal_calibration)
        cfg.tria_temporal_window = int(src["tria_temporal_window"])
        if "tria_carrier_alpha" in src:
            cfg.tria_carrier_alpha = float(src["tria_carrier_alpha"])
        _log(f"[tria] temporal calibration loaded {cfg.tria_temporal_calibration}: "
             f"W={cfg.tria_temporal_window} alpha={cfg.tria_carrier_alpha:g}")
        return
    if not bool(cfg.tria_temporal_auto):
        return
    result = calibrate_from_init(cfg)
    cfg.tria_temporal_window = result["tria_temporal_window"]
    cfg.tria_carrier_alpha = result["tria_carrier_alpha"]
    cfg._tria_temporal_auto_result = result
