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

    log("\n=== [4] depth-attn ===")
    qp = F.normalize(sd["depth_attn.q_params"].float(), dim=-1).permute(1, 0, 2)      # [qh, 2L, hd]
    gram = (qp @ qp.transpose(1, 2)).abs().mean(0).fill_diagonal_(0)
    nsub = gram.shape[0]
    log(f"  query Gram over {nsub} sublayers (mean over heads): offdiag |cos| mean={float(gram.mean()):.3f} "
        f"p99={float(torch.quantile(gram.flatten(), 0.99)):.3f} pairs>0.9={int((gram > 0.9).sum()) // 2}")
    out["depth"] = {"gram_mean": float(gram.mean())}
    wo = sd.get("depth_attn.w_o_weight")
    if wo is not None:
        wvd = sd["depth_attn.kv_weight"].float()[n:]
        wo = wo.float()
        if wo.dim() == 2:
            wo = wo.unsqueeze(0)
        ers = spectrum(wo @ wvd)["erank"].tolist()
        smx = spectrum(wo)["smax"].tolist()
        log("  value-circuit erank per sublayer:\n  " + " ".join(f"{v:.0f}" for v in ers))
        log("  w_o smax per sublayer:\n  " + " ".join(f"{v:.2f}" for v in smx))
        out["depth"].update(vc_erank=ers, wo_smax=smx)

    log("\n=== [5] embedding / memory head / norms ===")
    emb = sd["emb.weight"].float()
    es = spectrum1(emb)
    rows = emb.norm(dim=1)
    cone = float(emb.mean(0).norm() / rows.mean().clamp_min(1e-12))
    low = int((rows < 0.25 * rows.median()).sum())
    log(f"  emb: erank={es['erank']:.1f}/{es['full']} top1={es['top1']:.3f} cone(|mean|/|row|)={cone:.3f} low-norm tokens={low}")
    out["embedding"] = {"spectrum": es, "cone": cone, "low_norm_tokens": low}
    for name in ("tria_final_ca.w_qk.weight", "tria_final_ca.w_v.weight", "tria_agg.up.weight", "tria_agg.reader.proj.weight",
                 "tria_agg.reader.key_proj.weight"):
        if name in sd:
            s = spectrum1(sd[name])
            d = f" drift={drift(sd[name], init[name]):.3f}" if init is not None and name in init else ""
            log(f"  {name}: erank={s['erank']:.1f}/{s['full']} smax={s['smax']:.3f} top1={s['top1']:.3f}{d}")
    gains = torch.cat([sd[f"blocks.{li}.{ln}.weight"].float() for li in range(L) for ln in ("ln_attn", "ln_ffn")])
    gs = vector_stats(gains)
    log(f"  LN gains overall: mean={gs['mean']:.3f} std={gs['std']:.3f} min={gs['min']:.3f} max={gs['max']:.3f} "
        f"|g|<0.05: {gs['near_zero']}")
    biases = [sd[k].float() for li in range(L) for ln in ("ln_attn", "ln_ffn") if (k := f"blocks.{li}.{ln}.bias") in sd]
    if biases:
        b = torch.cat(biases)
        log(f"  LN biases: rms={float(b.square().mean().sqrt()):.3f} absmax={float(b.abs().max()):.3f}")
    if "ln_final.weight" in sd:
        log(f"  ln_final: {vector_stats(sd['ln_final.weight'])}")

    log("\n=== [6] axis aggregates (layer % 3: 0=Rz 1=Rx 2=Ry) ===")
    out["axes"] = []
    for ax in range(3):
        idx = [li for li in range(L) if li % 3 == ax]
        if not idx:
            continue
        rows_ = [out["layers"][li] for li in idx]
        agg = {"axis": ax, "layers": idx,
               "U": sum(r["imag_sector_share"]["U"] for r in rows_) / len(idx),
               "D": sum(r["imag_sector_share"]["D"] for r in rows_) / len(idx),
               "ffn_sk_erank": sum(r["ffn_skeleton"]["erank"] for r in rows_) / len(idx),
               "imag_bias_rms": float(torch.stack([sd[f"blocks.{li}.ffn.w1_imag_bias"].float().square().mean().sqrt() for li in idx]).mean()),
               "imag_std": float(torch.stack([sd[f"blocks.{li}.ffn.w1_imag"].float().std() for li in idx]).mean())}
        out["axes"].append(agg)
        log(f"  axis {ax}: layers={idx}\n          U%={100 * agg['U']:.1f} D%={100 * agg['D']:.1f} "
            f"ffn_sk_erank={agg['ffn_sk_erank']:.1f} imag_bias_rms={agg['imag_bias_rms']:.4f} imag_std={agg['imag_std']:.4f}")

    log("\n=== [7] flags ===")
    flags: List[str] = []
    for r in out["layers"]:
        li = r["layer"]
        if r["qk_erank_min"] < 0.25 * hd:
            flags.append(f"L{li}: degenerate QK head (min erank {r['qk_erank_min']:.0f}/{hd})")
        if r["ov_erank_min"] < 0.25 * hd:
            flags.append(f"L{li}: degenerate OV head (min erank {r['ov_erank_min']:.0f}/{hd})")
        if r["ffn_skeleton"]["erank_frac"] < 0.2:
            flags.append(f"L{li}: low-rank FFN skeleton ({r['ffn_skeleton']['erank']:.0f}/{n})")
        if r["dup"]["dup98"] > 0.005 * hidden:
            flags.append(f"L{li}: {r['dup']['dup98']} duplicate hidden units (cos>0.98)")
        if r["dead_hidden"] > 0.01 * hidden:
            flags.append(f"L{li}: {r['dead_hidden']} dead hidden units")
        if not math.isnan(r["gate_w1_cos"]) and r["gate_w1_cos"] > 0.9:
            flags.append(f"L{li}: gate_proj collapsed onto w1_real (cos {r['gate_w1_cos']:.2f})")
    sm = torch.tensor([r["w2_smax"] for r in out["layers"]])
    if sm.numel() > 1:
        z = (sm - sm.mean()) / sm.std().clamp_min(1e-9)
        for li in torch.nonzero(z.abs() > 3).flatten().tolist():
            flags.append(f"L{li}: w2 spectral-norm outlier ({float(sm[li]):.2f}, z={float(z[li]):+.1f})")
    out["flags"] = flags or ["none -- no degeneracy criteria triggered"]
    for f in out["flags"]:
        log("  * " + f)
    return out


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
