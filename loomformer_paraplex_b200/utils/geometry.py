"""Geometry audit of the Tria carriers on real text (reference ``utils/analyze_tria_geometry.py:235-330, 511-698,
889-1061``).

For every position, stream (hidden unit) and sequence the 3x3 depth carrier and the temporal carrier built from it are
decomposed by SVD: condition number, entropy effective rank, the proper polar rotation (angle, axis, incremental path
length), finite-time Lyapunov gaps and the first position where a stream leaves the "stable" regime.  Three views are
reported: the raw un-chunked forward, the operational chunked forward (per chunk and pooled), and the actual boundary
states written at the temporal endpoints.  With ``--init`` the same audit runs on an initial checkpoint and the two are
paired stream by stream.

Accumulators live on the analysis device and cross to the host once, in ``finish``.  Runs on CUDA (bf16 autocast, the
fused plan) and on CPU (fp32)."""
from __future__ import annotations

import contextlib
import gc
import json
import math
from pathlib import Path
from typing import Any, Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F

from ..config import Config, resolve
from ..data.corpus import RawCorpus
from ..data.tokenizers import build_tokenizer, special_id
from ..models.loomformer import Model
from ..models.rope import yarn_mscale
from ..ops import reference as R
from ..train import checkpoint as ckpt

QUANTILES = (("p10", 0.10), ("p50", 0.50), ("p90", 0.90), ("p99", 0.99))


def tensor_quantiles(v: torch.Tensor) -> Dict[str, float]:
    v = v.float().flatten()
    if v.numel() > 8_000_000:                        # torch.quantile has an input-size limit; subsample evenly
        v = v[:: v.numel() // 4_000_000]
    out = {"mean": float(v.mean())}
    qs = torch.quantile(v, torch.tensor([q for _, q in QUANTILES], device=v.device))
    out.update({name: float(x) for (name, _), x in zip(QUANTILES, qs)})
    return out


class Decomposition:
    """SVD-derived quantities of a batch of 3x3 carriers ``[..., 3, 3]``."""

    def __init__(self, m: torch.Tensor, max_condition: float, min_rank: float) -> None:
        u, s, vh = torch.linalg.svd(m.float(), full_matrices=False)
        self.u, self.s, self.vh = u, s, vh
        self.condition = s[..., 0] / s[..., -1].clamp_min(1e-12)
        self.prob = s / s.sum(-1, keepdim=True).clamp_min(1e-12)
        self.erank = torch.exp(-(self.prob * self.prob.clamp_min(1e-12).log()).sum(-1))
        self.passed = (self.condition <= max_condition) & (self.erank >= min_rank)
        rot = u @ vh
        self.reflected = torch.linalg.det(rot) < 0
        fix = torch.where(self.reflected, -1.0, 1.0)
        u2 = u.clone()
        u2[..., :, -1] *= fix[..., None]
        self.rotation = u2 @ vh                      # nearest proper rotation
        self.angle = rotation_angle(self.rotation)


def rotation_angle(r: torch.Tensor) -> torch.Tensor:
    tr = r.diagonal(dim1=-2, dim2=-1).sum(-1)
    return torch.acos(((tr - 1.0) * 0.5).clamp(-1.0, 1.0))


def rotation_axis(r: torch.Tensor):
    """Unit rotation axis via the quaternion of ``r`` and a validity mask (axis undefined near the identity)."""
    d0, d1, d2 = r[..., 0, 0], r[..., 1, 1], r[..., 2, 2]
    half = lambda x: 0.5 * torch.sqrt(x.clamp_min(0.0))
    q = torch.stack((half(1 + d0 + d1 + d2),
                     torch.copysign(half(1 + d0 - d1 - d2), r[..., 2, 1] - r[..., 1, 2]),
                     torch.copysign(half(1 - d0 + d1 - d2), r[..., 0, 2] - r[..., 2, 0]),
                     torch.copysign(half(1 - d0 - d1 + d2), r[..., 1, 0] - r[..., 0, 1])), dim=-1)
    v = F.normalize(q, dim=-1, eps=1e-12)[..., 1:]
    nrm = v.norm(dim=-1, keepdim=True)
    return v / nrm.clamp_min(1e-12), nrm[..., 0] > 1e-5


def projector_concentration(vectors: torch.Tensor, valid: Optional[torch.Tensor] = None) -> Dict[str, Any]:
    """Eigenvalues of the second-moment matrix of unit vectors: 1/3 each when isotropic, (1,0,0) when aligned."""
    v = vectors.float().reshape(-1, 3)
    if valid is not None:
        v = v[valid.reshape(-1)]
    if v.numel() == 0:
        return {"valid_count": 0, "projector_eigenvalues": [float("nan")] * 3, "concentration": float("nan")}
    ev = torch.linalg.eigvalsh(v.t() @ v / v.shape[0]).flip(0)
    return {"valid_count": int(v.shape[0]), "projector_eigenvalues": [float(x) for x in ev], "concentration": float(ev[0])}


def context_frame_coherence(vectors: torch.Tensor) -> Optional[Dict[str, float]]:
    """Mean squared overlap of one stream's frame vector between every pair of sequences."""
    v = vectors.float()
    n = v.shape[0]
    if n < 2:
        return None
    g = torch.einsum("ahi,bhi->abh", v, v).square()
    iu = torch.triu_indices(n, n, offset=1)
    return tensor_quantiles(g[iu[0], iu[1]].mean(0))


def first_failure_horizon(passed: torch.Tensor) -> torch.Tensor:
    """``passed`` [S, T, H] -> first failing position (1-based) per sequence and stream, ``T + 1`` if none."""
    s, t, h = passed.shape
    bad = ~passed
    first = bad.float().argmax(1) + 1
    return torch.where(bad.any(1), first, torch.full_like(first, t + 1)).reshape(s, h)


def regime_fractions(cond: torch.Tensor, er: torch.Tensor, max_condition: float, min_rank: float) -> Dict[str, float]:
    stable = (cond <= max_condition) & (er >= min_rank)
    f = lambda m: float(m.float().mean())
    return {"stable": f(stable), "directional_full_rank": f(~stable & (er >= min_rank)),
            "plane_like": f((er < min_rank) & (er >= 1.8)), "line_like": f(er < 1.8)}


def boundary_state_report(m: torch.Tensor, max_condition: float, min_rank: float) -> Dict[str, Any]:
    """``m`` [S, K, H, 3, 3]: the carriers actually written at the K temporal endpoints."""
    d = Decomposition(m, max_condition, min_rank)

    def view(k: Optional[int]):
        pick = (lambda x: x) if k is None else (lambda x: x[:, k])
        c, e, p = pick(d.condition), pick(d.erank), pick(d.prob)
        return {"condition": tensor_quantiles(c), "effective_rank": tensor_quantiles(e),
                "population_pass": float(pick(d.passed).float().mean()),
                "regimes": regime_fractions(c, e, max_condition, min_rank),
                "normalized_singular_values_mean": [float(x) for x in p.reshape(-1, 3).mean(0)],
                "rotation_angle": tensor_quantiles(pick(d.angle)),
                "polar_reflection_fraction": float(pick(d.reflected).float().mean())}

    return {"keys": int(m.shape[1]), "all": view(None), "by_key": [{"key_index": k, **view(k)} for k in range(m.shape[1])]}


class GeometryAccumulator:
    """Running per-position means plus full samples at selected horizons, over calls of ``add([S, T, H, 3, 3])``."""

    CURVES = ("condition", "effective_rank", "population_pass", "rotation_angle", "incremental_rotation_angle",
              "rotation_path_length", "finite_time_lyapunov_gap_12", "finite_time_lyapunov_gap_23", "polar_reflection")
    KEEP = ("condition", "effective_rank", "singular_probability", "rotation_angle", "rotation_axis", "rotation_axis_valid",
            "dominant_input", "weak_input", "dominant_output", "weak_output", "rotation", "path_length")

    def __init__(self, tokens: int, horizons: Sequence[int], window: int, max_condition: float, min_rank: float,
                 population_pass: float) -> None:
        self.T, self.horizons, self.window = int(tokens), [int(h) for h in horizons], int(window)
        self.max_condition, self.min_rank, self.population_pass = max_condition, min_rank, population_pass
        self.sums: Optional[torch.Tensor] = None          # [len(CURVES), T] float64 on the data's device
        self.count = 0
        self.kept = {h: {k: [] for k in self.KEEP} for h in self.horizons}
        self.failure: List[torch.Tensor] = []
        self.step_overlap = {"dominant": [], "weak": []}
        self.window_conc = {"dominant": {}, "weak": {}}

    def add(self, m: torch.Tensor) -> None:
        d = Decomposition(m, self.max_condition, self.min_rank)
        S, T, H = d.condition.shape
        assert T == self.T, (T, self.T)
        eye = torch.eye(3, device=m.device).expand(S, 1, H, 3, 3)
        prev = torch.cat((eye, d.rotation[:, :-1]), dim=1)
        inc = rotation_angle(d.rotation @ prev.transpose(-1, -2))
        path = inc.cumsum(1)
        hz = torch.arange(1, T + 1, device=m.device, dtype=torch.float32).view(1, T, 1)
        gap12 = (d.s[..., 0] / d.s[..., 1].clamp_min(1e-12)).log() / hz
        gap23 = (d.s[..., 1] / d.s[..., 2].clamp_min(1e-12)).log() / hz
        curves = torch.stack([x.double().sum(dim=(0, 2)) for x in (d.condition, d.erank, d.passed, d.angle, inc, path,
                                                                    gap12, gap23, d.reflected)])
        self.sums = curves if self.sums is None else self.sums + curves
        self.count += S * H
        self.failure.append(first_failure_horizon(d.passed))
        frames = {"dominant": d.vh[..., 0, :], "weak": d.vh[..., -1, :]}
        outs = {"dominant": d.u[..., :, 0], "weak": d.u[..., :, -1]}
        for name, v in frames.items():
            if T > 1:
                self.step_overlap[name].append((v[:, 1:] * v[:, :-1]).sum(-1).square().mean(1))
            for lo in range(0, T, self.window):
                hi = min(lo + self.window, T)
                mom = torch.einsum("sthi,sthj->shij", v[:, lo:hi], v[:, lo:hi]) / (hi - lo)
                self.window_conc[name].setdefault(f"{lo}:{hi}", []).append(torch.linalg.eigvalsh(mom)[..., -1])
        axis, axis_ok = rotation_axis(d.rotation)
        for h in self.horizons:
            i, k = h - 1, self.kept[h]
            k["condition"].append(d.condition[:, i].flatten()); k["effective_rank"].append(d.erank[:, i].flatten())
            k["singular_probability"].append(d.prob[:, i].reshape(-1, 3)); k["rotation_angle"].append(d.angle[:, i].flatten())
            k["rotation_axis"].append(axis[:, i].reshape(-1, 3)); k["rotation_axis_valid"].append(axis_ok[:, i].flatten())
            k["dominant_input"].append(frames["dominant"][:, i]); k["weak_input"].append(frames["weak"][:, i])
            k["dominant_output"].append(outs["dominant"][:, i]); k["weak_output"].append(outs["weak"][:, i])
            k["rotation"].append(d.rotation[:, i]); k["path_length"].append(path[:, i].flatten())

    def finish(self) -> Dict[str, Any]:
        mean = (self.sums / self.count).cpu()
        curves = {n: mean[i] for i, n in enumerate(self.CURVES)}
        below = torch.nonzero(curves["population_pass"] < self.population_pass)
        stable_h = self.T if below.numel() == 0 else max(1, int(below[0, 0]))
        selected, tensors = {}, {}
        for h in self.horizons:
            k = {n: torch.cat(v, dim=0).cpu() for n, v in self.kept[h].items()}
            c, e = k["condition"], k["effective_rank"]
            selected[str(h)] = {
                "condition": tensor_quantiles(c), "effective_rank": tensor_quantiles(e),
                "population_pass": float(((c <= self.max_condition) & (e >= self.min_rank)).float().mean()),
                "regimes": regime_fractions(c, e, self.max_condition, self.min_rank),
                "normalized_singular_values_mean": [float(x) for x in k["singular_probability"].mean(0)],
                "rotation_angle": tensor_quantiles(k["rotation_angle"]),
                "rotation_axis_global": projector_concentration(k["rotation_axis"], k["rotation_axis_valid"]),
                "rotation_path_length": tensor_quantiles(k["path_length"]),
                "dominant_input_global": projector_concentration(k["dominant_input"]),
                "weak_input_global": projector_concentration(k["weak_input"]),
                "dominant_output_global": projector_concentration(k["dominant_output"]),
                "weak_output_global": projector_concentration(k["weak_output"]),
                "dominant_input_context_coherence": context_frame_coherence(k["dominant_input"]),
                "weak_input_context_coherence": context_frame_coherence(k["weak_input"]),
            }
            tensors[str(h)] = {n: k[n] for n in ("rotation", "dominant_input", "weak_input", "singular_probability")}
        fail = torch.cat(self.failure, 0).cpu().float()
        by_w = fail <= self.window
        cat = lambda xs: torch.cat([x.flatten() for x in xs]).cpu() if xs else torch.zeros(1)
        report = {
            "stable_horizon": stable_h,
            "condition_mean": curves["condition"].tolist(), "effective_rank_mean": curves["effective_rank"].tolist(),
            "population_pass": curves["population_pass"].tolist(), "rotation_angle_mean": curves["rotation_angle"].tolist(),
            "incremental_rotation_angle_mean": curves["incremental_rotation_angle"].tolist(),
            "rotation_path_length_mean": curves["rotation_path_length"].tolist(),
            "finite_time_lyapunov_gap_12_mean": curves["finite_time_lyapunov_gap_12"].tolist(),
            "finite_time_lyapunov_gap_23_mean": curves["finite_time_lyapunov_gap_23"].tolist(),
            "polar_reflection_fraction": curves["polar_reflection"].tolist(),
            "selected_horizons": selected,
            "per_stream_first_failure": {
                "all": tensor_quantiles(fail), "channel_mean": tensor_quantiles(fail.mean(0)),
                "channel_context_std": tensor_quantiles(fail.std(0, unbiased=False)),
                "fraction_always_stable": float((fail > self.T).float().mean()),
                "fraction_failed_by_window": float(by_w.float().mean()),
                "channels_failed_by_window_all_contexts": float(by_w.all(0).float().mean()),
                "channels_failed_by_window_some_context": float(by_w.any(0).float().mean())},
            "singular_frame_dynamics": {
                "dominant_step_overlap": tensor_quantiles(cat(self.step_overlap["dominant"])),
                "weak_step_overlap": tensor_quantiles(cat(self.step_overlap["weak"])),
                "dominant_window_projector_concentration": {k: tensor_quantiles(cat(v)) for k, v in self.window_conc["dominant"].items()},
                "weak_window_projector_concentration": {k: tensor_quantiles(cat(v)) for k, v in self.window_conc["weak"].items()}},
        }
        return {"report": report, "selected_tensors": tensors, "first_failure": fail}


# ------------------------------------------------------------------ data and model plumbing
def build_rows(cfg: Config, data_path: str, tokens: int, sequences: int, tokenizer=None) -> List[torch.Tensor]:
    """``sequences`` rows of ``tokens`` ids cut from the corpus stream (documents joined by <eos>, rows opened by <bos>
    when the tokenizer has one)."""
    tok = tokenizer or build_tokenizer(cfg)[0]
    bos, eos = special_id(tok, "<bos>"), special_id(tok, "<eos>")
    body = tokens - (1 if bos is not None else 0)
    need = sequences * body
    stream: List[int] = []
    for i, text in enumerate(RawCorpus(data_path, fmt="auto", text_field=cfg.text_field).iter_texts()):
        if i and eos is not None:
            stream.append(eos)
        stream.extend(tok.encode(text))
        if len(stream) >= need:
            break
    if len(stream) < need:
        raise RuntimeError(f"need {need} tokens, got {len(stream)}")
    head = [bos] if bos is not None else []
    return [torch.tensor(head + stream[i * body:(i + 1) * body], dtype=torch.long) for i in range(sequences)]


def override_config(blob: Dict[str, Any], tokens: int, tokenizer: Optional[str], window: Optional[int],
                    alpha: Optional[float], polarm_beta: Optional[float]) -> Config:
    cfg = Config.from_checkpoint_dict(dict(blob["cfg"]))
    if tokens <= 0:
        raise ValueError("tokens must be positive")
    cfg.seq_len = int(tokens)
    if tokenizer is not None:
        cfg.tokenizer = tokenizer
    if window is not None:
        cfg.tria_temporal_window = int(window)
    if alpha is not None:
        cfg.tria_carrier_alpha = float(alpha)
    if polarm_beta is not None:
        cfg.tria_polarm_beta = float(polarm_beta)
    cfg.grad_checkpointing = False
    cfg.device = None
    if int(tokens) % int(cfg.tria_temporal_window):
        raise ValueError("tokens must be divisible by the temporal window")
    return cfg


def load_probe_model(cfg: Config, blob: Dict[str, Any], device: torch.device) -> Model:
    """The checkpoint's model with the vocabulary head removed and carrier capture switched on."""
    model = Model(cfg, dims=resolve(cfg, calibrate=False))
    ckpt.load_model_blob(model, blob, False)
    model.to(device).eval().requires_grad_(False)
    model.head = torch.nn.Identity()
    model.ops = None                                     # introspection needs the composed forward
    model.capture_tria_depth_carry = True
    return model


def amp(device: torch.device):
    return torch.autocast("cuda", dtype=torch.bfloat16) if device.type == "cuda" else contextlib.nullcontext()


def rope_report(cfg: Config, tokens: int) -> Dict[str, Any]:
    af = cfg.rope_attention_factor
    return {"original_seq_len": int(cfg.rope_original_seq_len or cfg.seq_len), "factor": float(cfg.rope_factor),
            "attention_factor": float(af) if af is not None else float(yarn_mscale(cfg.rope_factor)), "cache_seq_len": tokens}


def analyze_checkpoint(label: str, path: str, blob: Dict[str, Any], rows: List[torch.Tensor], cfg: Config,
                       device: torch.device, tokens: int, raw_tokens: int, horizons: List[int], max_condition: float,
                       min_rank: float, population_pass: float, log=print):
    log(f"loading {label}: {path}")
    model = load_probe_model(cfg, blob, device)
    W = int(cfg.tria_temporal_window)
    mk = lambda t, hs: GeometryAccumulator(t, hs, W, max_condition, min_rank, population_pass)
    raw_h = [h for h in horizons if h <= raw_tokens]
    op_h = sorted({h for h in horizons if h <= W} | {W})
    raw_depth, raw_temporal = mk(raw_tokens, raw_h), mk(raw_tokens, raw_h)
    op_depth, op_temporal = mk(W, op_h), mk(W, op_h)
    chunks = tokens // W
    op_depth_c = [mk(W, op_h) for _ in range(chunks)]
    op_temporal_c = [mk(W, op_h) for _ in range(chunks)]
    pos = torch.arange(tokens, device=device).view(1, tokens)
    first = lambda t: torch.zeros(1, t, dtype=torch.bool, device=device).index_fill_(1, torch.tensor([0], device=device), True)
    boundaries = []
    with torch.inference_mode():
        for i, row in enumerate(rows, 1):                 # un-chunked forward: how long would carriers last unaided
            with amp(device):
                model._forward_flat(row[:raw_tokens].view(1, -1).to(device), attn_mask=None, position_ids=pos[:, :raw_tokens])
            depth = model.last_tria_depth_carry
            if depth is None:
                raise RuntimeError("Tria depth carry capture failed")
            raw_depth.add(depth)
            raw_temporal.add(R.temporal_scan(depth.float(), first(raw_tokens)))
            log(f"  {label}: sequence {i}/{len(rows)}")
        inner = model._run_chunk_stack
        for i, row in enumerate(rows, 1):                 # operational forward: chunked, with endpoint refeed
            seen: List[torch.Tensor] = []

            def tap(*a, **kw):
                h, carry, states = inner(*a, **kw)
                seen.append(carry.detach())
                return h, carry, states

            model._run_chunk_stack = tap
            try:
                with amp(device):
                    model(row.view(1, tokens).to(device), position_ids=pos)
            finally:
                model._run_chunk_stack = inner
            if model.last_tria_document_carry is None:
                raise RuntimeError("actual Tria boundary-state capture failed")
            boundaries.append(model.last_tria_document_carry.detach().float().cpu())
            depth = torch.cat(seen, dim=1)
            if depth.shape[1] != tokens:
                raise RuntimeError(f"captured {depth.shape[1]} chunked tokens, expected {tokens}")
            for c in range(chunks):
                dc = depth[:, c * W:(c + 1) * W]
                tc = R.temporal_scan(dc.float(), first(W))
                for acc, x in ((op_depth, dc), (op_temporal, tc), (op_depth_c[c], dc), (op_temporal_c[c], tc)):
                    acc.add(x)
            log(f"  {label}: operational sequence {i}/{len(rows)} chunks={chunks}")
    raw_t, op_t = raw_temporal.finish(), op_temporal.finish()
    report = {
        "step": int(blob.get("step", 0) or 0),
        "depth": raw_depth.finish()["report"], "temporal": raw_t["report"],
        "operational": {"window": W, "chunks": chunks * len(rows), "depth": op_depth.finish()["report"],
                        "temporal": op_t["report"],
                        "by_chunk": [{"chunk_index": c, "start": c * W, "end": (c + 1) * W, "receives_refeed": c > 0,
                                      "depth": op_depth_c[c].finish()["report"], "temporal": op_temporal_c[c].finish()["report"]}
                                     for c in range(chunks)]},
        "boundary_state": boundary_state_report(torch.cat(boundaries, 0), max_condition, min_rank),
    }
    del model
    gc.collect()
    if device.type == "cuda":
        torch.cuda.empty_cache()
    return report, raw_t, op_t


def paired_report(init: Dict[str, Any], trained: Dict[str, Any], horizons: Sequence[int], tokens: int) -> Dict[str, Any]:
    """Stream-by-stream change from the initial to the trained checkpoint."""
    out = {}
    for h in horizons:
        a, b = init["selected_tensors"][str(h)], trained["selected_tensors"][str(h)]
        out[str(h)] = {
            "relative_polar_rotation_angle": tensor_quantiles(rotation_angle(b["rotation"] @ a["rotation"].transpose(-1, -2))),
            "dominant_input_frame_overlap_squared": tensor_quantiles((a["dominant_input"] * b["dominant_input"]).sum(-1).square()),
            "weak_input_frame_overlap_squared": tensor_quantiles((a["weak_input"] * b["weak_input"]).sum(-1).square()),
            "normalized_stretch_delta_l2": tensor_quantiles((a["singular_probability"] - b["singular_probability"]).norm(dim=-1)),
        }
    fa, fb = init["first_failure"].clamp_max(tokens + 1), trained["first_failure"].clamp_max(tokens + 1)
    delta = fb - fa
    ca, cb = fa.flatten() - fa.mean(), fb.flatten() - fb.mean()
    corr = float((ca * cb).mean() / (ca.square().mean().sqrt() * cb.square().mean().sqrt()).clamp_min(1e-12))
    return {"selected_horizons": out, "first_failure_delta_trained_minus_init": tensor_quantiles(delta),
            "fraction_streams_shortened": float((delta < 0).float().mean()),
            "fraction_streams_lengthened": float((delta > 0).float().mean()), "first_failure_correlation": corr}


def print_checkpoint_summary(label: str, rep: Dict[str, Any], window: int, horizons: Sequence[int], log=print) -> None:
    t = rep["temporal"]
    log(f"{label}: temporal stable horizon={t['stable_horizon']} depth stable horizon={rep['depth']['stable_horizon']}")
    for h in horizons:
        m = t["selected_horizons"][str(h)]
        sv = "/".join(f"{v:.3f}" for v in m["normalized_singular_values_mean"])
        log(f"  h={h:4d} pass={m['population_pass']:.4f} cond={m['condition']['mean']:.3f} rank={m['effective_rank']['mean']:.3f} "
            f"rot={math.degrees(m['rotation_angle']['mean']):6.1f}deg path={m['rotation_path_length']['mean']:.1f}rad sv={sv}")
    ff, dyn = t["per_stream_first_failure"], t["singular_frame_dynamics"]
    log(f"  first-failure median={ff['all']['p50']:.1f} p10={ff['all']['p10']:.1f} p90={ff['all']['p90']:.1f} "
        f"failed_by_W={ff['fraction_failed_by_window']:.4f}")
    log(f"  weak-frame lag1 overlap={dyn['weak_step_overlap']['mean']:.4f} "
        f"dominant-frame lag1 overlap={dyn['dominant_step_overlap']['mean']:.4f}")
    op = rep["operational"]["temporal"]
    b = op["selected_horizons"][str(window)]
    log(f"  operational W={window}: pass={b['population_pass']:.4f} cond={b['condition']['mean']:.3f} "
        f"rank={b['effective_rank']['mean']:.3f} failed_by_W={op['per_stream_first_failure']['fraction_failed_by_window']:.4f}")
    parts = []
    for c in rep["operational"]["by_chunk"]:
        cb = c["temporal"]["selected_horizons"][str(window)]
        parts.append(f"c{c['chunk_index']}:{cb['population_pass']:.3f}/{cb['condition']['mean']:.2f}/{cb['effective_rank']['mean']:.2f}")
    log("  operational chunks pass/cond/rank: " + " ".join(parts))
    bs = rep["boundary_state"]
    a = bs["all"]
    log(f"  actual post-PolARM boundaries={bs['keys']}: pass={a['population_pass']:.4f} cond={a['condition']['mean']:.3f}/"
        f"{a['condition']['p50']:.3f}/{a['condition']['p90']:.3f}/{a['condition']['p99']:.3f} rank={a['effective_rank']['mean']:.3f}")


def run(checkpoint: str, data: str, init: Optional[str] = None, tokenizer: Optional[str] = None, tokens: int = 768,
        raw_tokens: int = 768, window: Optional[int] = None, alpha: Optional[float] = None,
        polarm_beta: Optional[float] = None, sequences: int = 4, device: str = "cuda",
        output: str = "tria_geometry_analysis.json", max_condition: float = 3.0, min_effective_rank: float = 2.70,
        population_pass: float = 0.90, tokenizer_obj=None, log=print) -> Dict[str, Any]:
    blob = torch.load(checkpoint, map_location="cpu", weights_only=True)
    init_blob = torch.load(init, map_location="cpu", weights_only=True) if init else None
    cfg = override_config(blob, tokens, tokenizer, window, alpha, polarm_beta)
    dev = torch.device(device)
    raw_tokens = min(int(raw_tokens), tokens)
    W = int(cfg.tria_temporal_window)
    horizons = sorted({h for h in (1, 8, 16, 32, 64, 96, 128, W, 2 * W, 3 * W, 4 * W, tokens) if 1 <= h <= tokens})
    raw_h = [h for h in horizons if h <= raw_tokens]
    rows = build_rows(cfg, data, tokens, sequences, tokenizer_obj)
    log(f"T={tokens} W={W} alpha={cfg.tria_carrier_alpha:g} sequences={len(rows)} horizons={horizons} "
        f"rope_original={cfg.rope_original_seq_len} rope_factor={cfg.rope_factor:g}")
    args = (rows, cfg, dev, tokens, raw_tokens, horizons, max_condition, min_effective_rank, population_pass, log)
    report: Dict[str, Any] = {"checkpoint": checkpoint}
    if init_blob is not None:
        report["init_checkpoint"] = init
    report.update({"dataset": data, "native_alpha": float(cfg.tria_carrier_alpha), "polarm_beta": float(cfg.tria_polarm_beta),
                   "window": W, "tokens_analyzed": tokens, "raw_tokens_analyzed": raw_tokens, "sequences": len(rows),
                   "rope": rope_report(cfg, tokens),
                   "thresholds": {"max_condition": max_condition, "min_effective_rank": min_effective_rank,
                                  "population_pass": population_pass}})
    log_summary = []
    if init_blob is None:
        rep, _, _ = analyze_checkpoint("checkpoint", checkpoint, blob, *args)
        report["analysis"] = rep
        log_summary.append(("checkpoint", rep))
    else:
        irep, iraw, iop = analyze_checkpoint("init", init, init_blob, *args)
        trep, traw, top = analyze_checkpoint("trained", checkpoint, blob, *args)
        report.update({"init": irep, "trained": trep, "trained_vs_init": paired_report(iraw, traw, raw_h, raw_tokens),
                       "trained_vs_init_operational": paired_report(iop, top, [h for h in raw_h if h <= W], W)})
        log_summary += [("init", irep), ("trained", trep)]
    Path(output).write_text(json.dumps(report, indent=2), encoding="utf-8")
    log("\n=== Rotation-aware summary ===")
    for label, rep in log_summary:
        print_checkpoint_summary(label, rep, W, raw_h, log)
    if init_blob is not None:
        p = report["trained_vs_init"]
        log("\n=== Learned change ===")
        log(f"streams shortened={p['fraction_streams_shortened']:.4f} lengthened={p['fraction_streams_lengthened']:.4f} "
            f"horizon correlation={p['first_failure_correlation']:.4f}")
        for h in raw_h:
            m = p["selected_horizons"][str(h)]
            log(f"  h={h:4d} relative rotation={math.degrees(m['relative_polar_rotation_angle']['mean']):6.1f}deg "
                f"dominant overlap={m['dominant_input_frame_overlap_squared']['mean']:.3f} "
                f"weak overlap={m['weak_input_frame_overlap_squared']['mean']:.3f} "
                f"stretch delta={m['normalized_stretch_delta_l2']['mean']:.3f}")
    log(f"\nJSON saved to {output}")
    return report


def main(argv=None) -> None:
    import argparse
    ap = argparse.ArgumentParser(description="SVD geometry audit of Tria depth/temporal carriers")
    ap.add_argument("checkpoint")
    ap.add_argument("--init")
    ap.add_argument("--data", required=True)
    ap.add_argument("--tokenizer")
    ap.add_argument("--tokens", type=int, default=768)
    ap.add_argument("--raw-tokens", type=int, default=768)
    ap.add_argument("--window", type=int)
    ap.add_argument("--alpha", type=float)
    ap.add_argument("--polarm-beta", type=float)
    ap.add_argument("--sequences", type=int, default=4)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--output", default="tria_geometry_analysis.json")
    ap.add_argument("--max-condition", type=float, default=3.0)
    ap.add_argument("--min-effective-rank", type=float, default=2.70)
    ap.add_argument("--population-pass", type=float, default=0.90)
    a = ap.parse_args(argv)
    run(a.checkpoint, a.data, a.init, a.tokenizer, a.tokens, a.raw_tokens, a.window, a.alpha, a.polarm_beta, a.sequences,
        a.device, a.output, a.max_condition, a.min_effective_rank, a.population_pass)


if __name__ == "__main__":
    main()
