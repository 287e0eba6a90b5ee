"""Checkpoint anatomy from weights alone -- no data, no forward pass (reference ``utils/spectra.py:1-120``).

Sections of the report: [1] per-layer circuits (QK / OV effective rank per head, FFN skeleton ``w2 @ w1_real``,
spectral norms of the residual writers), [2] ``w1_imag`` energy per input sector (Q/K/C/U/D), [3] hidden-unit
degeneracies (duplicate rows, dead units, ``gate_proj`` collapsing onto ``w1_real``), [4] depth attention (Gram of the
per-sublayer queries, value-circuit ranks), [5] embedding / memory head / norm gains, [6] aggregates per carrier axis
(``layer % 3``), [7] anomaly flags.  All per-head SVDs of a layer are one batched call."""
from __future__ import annotations

import json
import math
from typing import Any, Dict, List, Optional

import torch
import torch.nn.functional as F

SECTORS = ("Q", "K", "C", "U", "D")


def spectrum(w: torch.Tensor) -> Dict[str, torch.Tensor]:
    """Batched singular-value summary of ``[..., m, n]``: largest value, entropy effective rank, stable rank, share of
    the top value."""
    s = torch.linalg.svdvals(w.float())
    p = s / s.sum(-1, keepdim=True).clamp_min(1e-12)
    erank = torch.exp(-(p * p.clamp_min(1e-12).log()).sum(-1))
    return {"smax": s[..., 0], "erank": erank, "stable_rank": s.square().sum(-1) / s[..., 0].square().clamp_min(1e-24),
            "top1": p[..., 0], "full": min(w.shape[-2:])}


def spectrum1(w: torch.Tensor) -> Dict[str, float]:
    d = spectrum(w)
    out = {k: float(v) for k, v in d.items() if k != "full"}
    out["full"] = d["full"]
    out["erank_frac"] = out["erank"] / d["full"]
    return out


def duplicate_rows(w: torch.Tensor, hi: float = 0.98, lo: float = 0.90) -> Dict[str, Any]:
    """Largest |cosine| of each row against any other row."""
    u = F.normalize(w.float(), dim=1, eps=1e-9)
    g = (u @ u.t()).abs_().fill_diagonal_(0)
    mx = g.max(1).values
    return {"cos_p50": float(mx.median()), "cos_p99": float(torch.quantile(mx, 0.99)), "dup98": int((mx > hi).sum()),
            "dup90": int((mx > lo).sum())}


def drift(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.float(), b.to(a.device).float()
    return float((a - b).norm() / b.norm().clamp_min(1e-12))


def vector_stats(v: torch.Tensor) -> Dict[str, Any]:
    v = v.float()
    return {"mean": float(v.mean()), "std": float(v.std()), "min": float(v.min()), "max": float(v.max()),
            "near_zero": int((v.abs() < 0.05).sum())}


def analyze(blob: Dict[str, Any], init: Optional[Dict[str, torch.Tensor]] = None, device: str = "cpu",
            log=print) -> Dict[str, Any]:
    sd = {k: v.to(device) for k, v in blob["model"].items() if torch.is_tensor(v)}
    cfg = blob["cfg"]
    L, qh, hd = int(cfg["layers"]), int(cfg["n_q_heads"]), int(cfg["head_dim"])
    n = qh * hd
    group = int(cfg.get("gqa_group_size") or (qh // int(cfg["n_kv_heads"])))
    kvh = qh // group
    kv = kvh * hd
    head_mode = str(cfg.get("phase_sectors", "head")) == "head"
    hidden = sd["blocks.0.ffn.w1_real.weight"].shape[0]
    log(f"step={blob.get('step', '?')}  L={L} d={n} H={hidden} qh={qh} kvh={kvh} hd={hd} "
        f"phase={'head' if head_mode else 'open'}  device={device}")
    sizes = [hd, hd, hd, n, hd] if head_mode else [hd, n, n, n, n]
    edges = [0]
    for s in sizes:
        edges.append(edges[-1] + s)
    out: Dict[str, Any] = {"layers": [], "step": blob.get("step")}
    log("\n=== [1-3] per-layer: circuits / phase sectors / degeneracies ===")
    log(" L | QK_er OV_er | ffn_er sk_smax | o_smax w2_smax | imag% Q/K/C/U/D | dup98 dead | g~w1 | drift(w1/w2/o)")
    for li in range(L):
        p = f"blocks.{li}."
        qkv = sd[p + "attn.qkv_weight"].float()
        wq = qkv[:n].view(qh, hd, n)
        wk = qkv[n:n + kv].view(kvh, hd, n).repeat_interleave(group, 0)
        wv = qkv[n + kv:].view(kvh, hd, n).repeat_interleave(group, 0)
        o = sd[p + "attn.o.weight"].float()
        oh = o.view(n, qh, hd).permute(1, 0, 2)                                   # [qh, n, hd]
        qk_er = spectrum(wq.transpose(1, 2) @ wk)["erank"]                        # all heads at once
        ov_er = spectrum(oh @ wv)["erank"]
        w1, w2 = sd[p + "ffn.w1_real.weight"].float(), sd[p + "ffn.w2.weight"].float()
        skeleton = spectrum1(w2 @ w1)
        e = sd[p + "ffn.w1_imag"].float().square()
        shares = [float(e[:, edges[i]:edges[i + 1]].sum() / e.sum().clamp_min(1e-30)) for i in range(5)]
        dup = duplicate_rows(w1)
        gain = w1.norm(dim=1) * w2.norm(dim=0)
        dead = int((gain < 0.05 * gain.median()).sum())
        gp = sd.get(p + "ffn.gate_proj.weight")
        gcos = float((F.normalize(gp.float(), dim=1) * F.normalize(w1, dim=1)).sum(1).abs().mean()) if gp is not None else float("nan")
        dr = ""
        if init is not None:
            dr = "/".join(f"{drift(sd[p + k], init[p + k]):.2f}" for k in ("ffn.w1_real.weight", "ffn.w2.weight", "attn.o.weight"))
        row = {"layer": li, "qk_erank_mean": float(qk_er.mean()), "qk_erank_min": float(qk_er.min()),
               "ov_erank_mean": float(ov_er.mean()), "ov_erank_min": float(ov_er.min()), "ffn_skeleton": skeleton,
               "o_smax": float(spectrum(o)["smax"]), "w2_smax": float(spectrum(w2)["smax"]),
               "imag_sector_share": dict(zip(SECTORS, shares)), "dup": dup, "dead_hidden": dead, "gate_w1_cos": gcos}
        out["layers"].append(row)
        log(f"{li:3d} | {row['qk_erank_mean']:5.1f} {row['ov_erank_mean']:5.1f} | {skeleton['erank']:6.1f} {skeleton['smax']:7.3f} "
            f"| {row['o_smax']:6.3f} {row['w2_smax']:7.3f} | {'/'.join(f'{100 * s:.0f}' for s in shares):>14s} "
            f"| {dup['dup98']:5d} {dead:4d} | {gcos:4.2f} | {dr}")

    out["depth"] = _depth_section(sd, n, log)
    out["embedding"] = _embedding_section(sd, init, L, log)
    out["axes"] = _axis_section(sd, out["layers"], L, log)
    out["flags"] = _flag_section(out["layers"], {"hd": hd, "n": n, "hidden": hidden}, log)
    return out


# ---------------------------------------------------------------------------------------------- report sections 4-7
def _depth_section(sd, n: int, log) -> Dict[str, Any]:
    """[4] How distinct the per-sublayer depth queries are, and how much rank the depth value circuit keeps."""
    log("\n=== [4] depth-attn ===")
    q = F.normalize(sd["depth_attn.q_params"].float(), dim=-1)                  # [2L, qh, hd]
    cos = torch.einsum("ahd,bhd->hab", q, q).abs().mean(0)                      # head-averaged |cos| between sublayers
    off = cos[~torch.eye(cos.shape[0], dtype=torch.bool, device=cos.device)]
    close = int((off > 0.9).sum()) // 2
    res: Dict[str, Any] = {"gram_mean": float(cos.fill_diagonal_(0).mean())}
    log(f"  {cos.shape[0]} sublayer queries, |cos| between different sublayers: mean {res['gram_mean']:.3f}, "
        f"99th pct {float(torch.quantile(off, 0.99)):.3f}, near-parallel pairs (>0.9): {close}")
    w_o = sd.get("depth_attn.w_o_weight")
    if w_o is None:
        return res
    w_o = w_o.float()
    w_o = w_o[None] if w_o.dim() == 2 else w_o
    value_rows = sd["depth_attn.kv_weight"].float()[n:]
    res["vc_erank"] = spectrum(w_o @ value_rows)["erank"].tolist()
    res["wo_smax"] = spectrum(w_o)["smax"].tolist()
    for label, vals, fmt in (("readout @ value projection, effective rank", res["vc_erank"], "{:.0f}"),
                             ("readout spectral norm", res["wo_smax"], "{:.2f}")):
        log(f"  {label} by sublayer: " + ", ".join(fmt.format(v) for v in vals))
    return res


_MEMORY_HEAD = ("tria_final_ca.w_qk.weight", "tria_final_ca.w_v.weight", "tria_agg.up.weight",
                "tria_agg.reader.proj.weight", "tria_agg.reader.key_proj.weight")


def _embedding_section(sd, init, L: int, log) -> Dict[str, Any]:
    """[5] Token embedding geometry, the matrices of the boundary-memory read-out, and normalisation gains."""
    log("\n=== [5] embedding / memory head / norms ===")
    emb = sd["emb.weight"].float()
    spec = spectrum1(emb)
    norms = emb.norm(dim=1)
    res = {"spectrum": spec, "cone": float(emb.mean(0).norm() / norms.mean().clamp_min(1e-12)),
           "low_norm_tokens": int((norms < 0.25 * norms.median()).sum())}
    log(f"  embedding table: effective rank {spec['erank']:.1f} of {spec['full']}, leading share {spec['top1']:.3f}, "
        f"common direction {res['cone']:.3f} of a row norm, {res['low_norm_tokens']} rows under a quarter of the median norm")
    for name in _MEMORY_HEAD:
        if name not in sd:
            continue
        sp = spectrum1(sd[name])
        moved = f", moved {drift(sd[name], init[name]):.3f} from init" if init is not None and name in init else ""
        log(f"  {name:34s} rank {sp['erank']:.1f}/{sp['full']}  norm {sp['smax']:.3f}  leading share {sp['top1']:.3f}{moved}")
    per_norm = [f"blocks.{li}.{which}" for li in range(L) for which in ("ln_attn", "ln_ffn")]
    g = vector_stats(torch.cat([sd[k + ".weight"].float() for k in per_norm]))
    log(f"  block LayerNorm gains: {g['mean']:.3f} +- {g['std']:.3f}, range [{g['min']:.3f}, {g['max']:.3f}], "
        f"{g['near_zero']} with magnitude under 0.05")
    shifts = [sd[k + ".bias"].float() for k in per_norm if k + ".bias" in sd]
    if shifts:
        b = torch.cat(shifts)
        log(f"  block LayerNorm shifts: rms {float(b.square().mean().sqrt()):.3f}, largest {float(b.abs().max()):.3f}")
    if "ln_final.weight" in sd:
        f = vector_stats(sd["ln_final.weight"])
        log(f"  final norm gains: {f['mean']:.3f} +- {f['std']:.3f}, range [{f['min']:.3f}, {f['max']:.3f}]")
    return res


def _axis_section(sd, layer_rows: List[Dict[str, Any]], L: int, log) -> List[Dict[str, Any]]:
    """[6] Layers share a carrier rotation axis every third layer; average a few per-layer figures per axis."""
    log("\n=== [6] axis aggregates (layer % 3: 0=Rz 1=Rx 2=Ry) ===")
    res = []
    for axis, name in enumerate(("Rz", "Rx", "Ry")):
        members = list(range(axis, L, 3))
        if not members:
            continue
        mean = lambda vals: float(sum(vals) / len(vals))
        imag = [sd[f"blocks.{li}.ffn.w1_imag"].float() for li in members]
        ibias = [sd[f"blocks.{li}.ffn.w1_imag_bias"].float() for li in members]
        agg = {"axis": axis, "layers": members,
               "U": mean([layer_rows[li]["imag_sector_share"]["U"] for li in members]),
               "D": mean([layer_rows[li]["imag_sector_share"]["D"] for li in members]),
               "ffn_sk_erank": mean([layer_rows[li]["ffn_skeleton"]["erank"] for li in members]),
               "imag_bias_rms": mean([float(b.square().mean().sqrt()) for b in ibias]),
               "imag_std": mean([float(w.std()) for w in imag])}
        res.append(agg)
        log(f"  axis {axis} ({name}), layers {members}: phase input energy from the block input {100 * agg['U']:.1f}% and "
            f"from the depth read {100 * agg['D']:.1f}%; skeleton rank {agg['ffn_sk_erank']:.1f}; "
            f"phase bias rms {agg['imag_bias_rms']:.4f}; phase weight std {agg['imag_std']:.4f}")
    return res


# One rule per line: (what it looks at, predicate over (row, sizes), message).  A rule fires per layer.
_LAYER_RULES = (
    ("qk", lambda r, z: r["qk_erank_min"] < z["hd"] / 4,
     lambda r, z: f"a query-key head has collapsed: smallest effective rank {r['qk_erank_min']:.0f} of {z['hd']}"),
    ("ov", lambda r, z: r["ov_erank_min"] < z["hd"] / 4,
     lambda r, z: f"an output-value head has collapsed: smallest effective rank {r['ov_erank_min']:.0f} of {z['hd']}"),
    ("skeleton", lambda r, z: r["ffn_skeleton"]["erank_frac"] < 0.2,
     lambda r, z: f"w2 @ w1_real spans few directions: effective rank {r['ffn_skeleton']['erank']:.0f} of {z['n']}"),
    ("duplicates", lambda r, z: r["dup"]["dup98"] > z["hidden"] / 200,
     lambda r, z: f"{r['dup']['dup98']} hidden units nearly repeat another one (|cos| above 0.98)"),
    ("dead", lambda r, z: r["dead_hidden"] > z["hidden"] / 100,
     lambda r, z: f"{r['dead_hidden']} hidden units carry almost no signal"),
    ("gate", lambda r, z: (not math.isnan(r["gate_w1_cos"])) and r["gate_w1_cos"] > 0.9,
     lambda r, z: f"gate_proj rows line up with w1_real rows (mean |cos| {r['gate_w1_cos']:.2f})"),
)


def _flag_section(layer_rows: List[Dict[str, Any]], sizes: Dict[str, int], log) -> List[str]:
    """[7] Degeneracy checks over the per-layer table, plus a z-score test for one outlying ``w2`` norm."""
    log("\n=== [7] flags ===")
    found = [f"layer {r['layer']}: {message(r, sizes)}"
             for r in layer_rows for _, fires, message in _LAYER_RULES if fires(r, sizes)]
    norms = torch.tensor([r["w2_smax"] for r in layer_rows])
    if norms.numel() > 1:
        z = (norms - norms.mean()) / norms.std().clamp_min(1e-9)
        found += [f"layer {li}: w2 spectral norm {float(norms[li]):.2f} stands {float(z[li]):+.1f} sigma from the other layers"
                  for li in range(norms.numel()) if abs(float(z[li])) > 3]
    if not found:
        found = ["nothing flagged"]
    for line in found:
        log("  - " + line)
    return found


def main(argv=None) -> None:
    import argparse
    ap = argparse.ArgumentParser(description="weight-space anatomy of a LoomFormer checkpoint")
    ap.add_argument("ckpt")
    ap.add_argument("--init", default=None)
    ap.add_argument("--device", default="auto")
    ap.add_argument("--json", default=None)
    a = ap.parse_args(argv)
    dev = ("cuda" if torch.cuda.is_available() else "cpu") if a.device == "auto" else a.device
    blob = torch.load(a.ckpt, map_location="cpu", weights_only=True)
    init = torch.load(a.init, map_location="cpu", weights_only=True)["model"] if a.init else None
    out = analyze(blob, init, dev)
    if a.json:
        with open(a.json, "w") as fh:
            json.dump(out, fh, indent=1, default=float)
        print(f"\n[json] -> {a.json}")


if __name__ == "__main__":
    main()
