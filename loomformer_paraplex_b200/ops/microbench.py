"""Per-kernel microbenchmarks with roofline fractions.

``python -m loomformer_paraplex_b200.ops.microbench --op ffn_core_bwd --tokens 8192`` times one native op on
113M-model shapes with CUDA events (warm-up, L2 flushed between iterations by writing a buffer larger than L2) and
reports achieved bytes/s and FLOP/s against the measured peaks of the machine (``MEASURED_PEAKS.json`` at the
repository root when present: STREAM-style copy bandwidth and cuBLAS bf16 throughput).  ``--op all`` prints a table.
The same entry is what profiler captures run, so a capture and a timing describe the same launch."""
from __future__ import annotations

import argparse
import json
import os
from types import SimpleNamespace
from typing import Callable, Dict, Tuple

import torch

from . import kernels as kmod

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks() -> Tuple[Dict[str, float], str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            p = json.load(fh)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"])}, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def dims(qh=8, hd=96, kvh=2, hidden=3072) -> SimpleNamespace:
    return SimpleNamespace(qh=qh, hd=hd, kvh=kvh, group=qh // kvh, n=qh * hd, kv_dim=kvh * hd, hidden=hidden,
                           hpq=hidden // qh, activation="pvpowlu", powlu_m=3.0, phase_floor=0.05, phase_secant=True)


def bf(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


def nbytes(*ts) -> int:
    return sum(t.numel() * t.element_size() for t in ts if t is not None)


# every builder returns (callable, algorithmic bytes, algorithmic flops)
def case_linear(K, M, n_in=768, n_out=3072):
    x, w = bf(M, n_in), bf(n_out, n_in, scale=0.03)
    y = K.linear(x, w)
    return (lambda: K.linear(x, w)), nbytes(x, w, y), 2.0 * M * n_in * n_out


def case_wgrad(K, M, n_in=768, n_out=3072):
    x, dy = bf(M, n_in), bf(M, n_out, scale=0.1)
    g = torch.zeros(n_out, n_in, device="cuda")
    def run():
        K.linear_wgrad(dy, x, g)
        K.flush_wgrads()
    return run, nbytes(x, dy, g) + nbytes(g), 2.0 * M * n_in * n_out


def case_wgrad_grouped(K, M, n_in=768, n_out=3072, chunks=16):
    """The same product cut into 16 chunk-sized pieces and issued as one grouped launch."""
    rows = M // chunks
    xs, dys = [bf(rows, n_in) for _ in range(chunks)], [bf(rows, n_out, scale=0.1) for _ in range(chunks)]
    g = torch.zeros(n_out, n_in, device="cuda")
    def run():
        for dy, x in zip(dys, xs):
            K.linear_wgrad(dy, x, g)
        K.flush_wgrads()
    return run, nbytes(*xs, *dys, g) + nbytes(g), 2.0 * M * n_in * n_out


def case_dgrad(K, M, n_in=768, n_out=3072):
    dy, w = bf(M, n_out, scale=0.1), bf(n_out, n_in, scale=0.03)
    dx = K.linear_dgrad(dy, w)
    return (lambda: K.linear_dgrad(dy, w)), nbytes(dy, w, dx), 2.0 * M * n_in * n_out


def case_imag_bwd(K, M):
    """Backward of the per-head imaginary projection (head sectors): four batched per-head data-gradient GEMMs
    (N = head dim), the shared-sector one, and their queued weight gradients."""
    d = dims()
    d.open_sectors, d.imag_in = False, d.n + 4 * d.hd
    qkc, u, m2 = bf(M, 3, d.qh, d.hd), bf(M, d.n), bf(M, d.qh, d.hd)
    w = bf(d.hidden, d.imag_in, scale=0.05)
    dbeta = bf(M, d.hidden, scale=0.1)
    gw = torch.zeros(d.hidden, d.imag_in, device="cuda")
    def run():
        K.imag_bwd(d, dbeta, qkc, u, m2, w, gw)
        K.flush_wgrads()
    flops = 2 * 2.0 * M * d.hidden * d.imag_in // d.qh * 1.0          # data + weight gradient of the per-head product
    return run, nbytes(qkc, u, m2, w, dbeta, gw) + nbytes(qkc, u, m2, gw), flops


def _core_inputs(M, B, H):
    x_real, beta_lin, pin = bf(M, H), bf(M, H, scale=1.5), bf(M, H, scale=0.5)
    alpha = torch.tensor(0.17, device="cuda")
    b_real, b_imag, w_tr = (torch.randn(H, device="cuda") * 0.3 for _ in range(3))
    tr_in = torch.rand(B, H, device="cuda") * 2 - 1
    cp = bf(9, M, H)
    gw = torch.softmax(torch.randn(9, device="cuda"), 0)
    return x_real, beta_lin, pin, alpha, b_real, b_imag, w_tr, tr_in, cp, gw


def case_ffn_core_fwd(K, M, Tc=128):
    d = dims()
    B, H = M // Tc, d.hidden
    x_real, beta_lin, pin, alpha, b_real, b_imag, w_tr, tr_in, cp, gw = _core_inputs(M, B, H)
    run = lambda: K.ffn_core_fwd(d, x_real, pin, alpha, b_real, None, beta_lin, b_imag, w_tr, tr_in, None, None, cp, None,
                                 None, gw, 1, 0.05, B)
    o = run()
    return run, nbytes(x_real, beta_lin, pin, cp, o["o"], o["c"], o["p_out"]), 0.0


def case_ffn_core_bwd(K, M, Tc=128):
    d = dims()
    B, H = M // Tc, d.hidden
    x_real, beta_lin, pin, alpha, b_real, b_imag, w_tr, tr_in, cp, gw = _core_inputs(M, B, H)
    saved = {"x_real": x_real, "p_in": pin, "alpha_gate": alpha, "b_real": b_real, "gate_lin": None, "beta_lin": beta_lin,
             "b_imag": b_imag, "w_trace": w_tr, "trace_in": tr_in, "reset": None, "anchor": torch.tensor(0.8, device="cuda"),
             "c_prev": cp, "seed": None, "seed_valid": None, "gate_w": gw, "axis": 1, "tria_alpha": 0.05, "B": B,
             "g_b_real": torch.zeros(H, device="cuda"), "g_b_imag": torch.zeros(H, device="cuda"),
             "g_w_trace": torch.zeros(H, device="cuda")}
    do, dc, dpo = bf(M, H, scale=0.1), bf(9, M, H, scale=0.1), bf(M, H, scale=0.1)
    dtr = torch.randn(B, H, device="cuda") * 0.1
    run = lambda: K.ffn_core_bwd(d, saved, do, dc, dpo, dtr)
    g = run()
    return run, nbytes(x_real, beta_lin, pin, cp, do, dc, dpo, g["d_x_real"], g["d_p_in"], g["d_beta_lin"], g["d_c_prev"]), 0.0


def _attn_inputs(M, Tc, T):
    d = dims()
    B = M // Tc
    s = T - Tc
    kc, vc = bf(B, T, d.kvh, d.hd), bf(B, T, d.kvh, d.hd)
    qkc = torch.zeros(M, 3, d.qh, d.hd, device="cuda", dtype=torch.bfloat16)
    qkc[:, 0] = bf(M, d.qh, d.hd)
    return d, B, s, kc, vc, qkc


def case_attn_fwd(K, M, Tc=128, T=1024):
    d, B, s, kc, vc, qkc = _attn_inputs(M, Tc, T)
    run = lambda: K.attn_fwd(d, qkc, kc, vc, s, T, None)
    # S = Q K^T, then [A V | A K]: 3 products of 2*Tc*T*hd per head; causal tail of the chunk ignored
    return run, nbytes(qkc, kc, vc), 3 * 2.0 * B * d.qh * Tc * T * d.hd


def case_attn_fwd_library(K, M, Tc=128, T=1024):
    """What the native forward replaced, timed the same way: PyTorch SDPA with value = [K ; V] (one call returns both
    contexts), keys and values repeated to the query heads, an explicit boolean mask (reference
    ``loomformer.py:3085-3114``).  Not an operation of this repository: a yardstick."""
    import torch.nn.functional as F
    d, B, s, kc, vc, qkc = _attn_inputs(M, Tc, T)
    q = qkc[:, 0].view(B, Tc, d.qh, d.hd).transpose(1, 2)                               # [B, QH, Tc, HD]
    k = kc.repeat_interleave(d.group, dim=2).transpose(1, 2)                            # [B, QH, T, HD]
    v = torch.cat((kc, vc), -1).repeat_interleave(d.group, dim=2).transpose(1, 2)       # [B, QH, T, 2 HD]
    mask = (torch.arange(T, device="cuda").view(1, T) <= (s + torch.arange(Tc, device="cuda")).view(Tc, 1)).view(1, 1, Tc, T)
    run = lambda: F.scaled_dot_product_attention(q, k, v, attn_mask=mask)
    run()
    return run, nbytes(qkc, kc, vc), 3 * 2.0 * B * d.qh * Tc * T * d.hd


def case_attn_bwd(K, M, Tc=128, T=1024):
    d, B, s, kc, vc, qkc = _attn_inputs(M, Tc, T)
    lse = K.attn_fwd(d, qkc, kc, vc, s, T, None)
    dqkc = bf(M, 3, d.qh, d.hd, scale=0.3)
    dk, dv = K.alloc_kv_grad(d, B, T, qkc.device), K.alloc_kv_grad(d, B, T, qkc.device)
    run = lambda: K.attn_bwd(d, dqkc, qkc, kc, vc, lse, s, T, None, dk, dv)
    # S, dP (two contexts), dQ, dK (two terms), dV: 7 products
    return run, nbytes(qkc, dqkc, kc, vc) + 2 * nbytes(dk, dv), 7 * 2.0 * B * d.qh * Tc * T * d.hd


def case_dread_slot_bwd(K, M, S=20, slot=5):
    """Gradient of one depth-history slot over the 15 sublayers that read it (10-layer model)."""
    d = dims()
    hist = bf(S, M, 2, d.qh, d.hd)                        # rows [K | V], as the training plan keeps the history
    hk, hv = hist[:, :, 0], hist[:, :, 1]
    q_all = torch.randn(S, d.qh, d.hd, device="cuda")
    dm, lse, dd = bf(S, M, d.qh, d.hd, scale=0.3), torch.randn(S, M, d.qh, device="cuda") + 3, torch.randn(S, M, d.qh, device="cuda")
    gq = torch.zeros(S, d.qh, d.hd, device="cuda")
    run = lambda: K.dread_slot_bwd(d, slot, q_all, hk, hv, dm, lse, dd, gq)
    dkv = run()                                           # [M, 2, QH, HD]: rows [dK | dV]
    return run, nbytes(hist[slot], dkv) + nbytes(dm[slot:], lse[slot:], dd[slot:]), 0.0


def case_dread_fwd(K, M, S=20, n=11):
    d = dims()
    hist = bf(S, M, 2, d.qh, d.hd)
    hk, hv = hist[:, :, 0], hist[:, :, 1]
    q = torch.randn(d.qh, d.hd, device="cuda")
    run = lambda: K.dread_fwd(d, q, hk, hv, n)
    out, lse = run()
    return run, nbytes(hk[:n], hv[:n], out, lse), 0.0


def case_optimizer(K, M):
    from ..optim.flat import FlatOptimizer, FlatParams
    lin = torch.nn.Linear(4096, max(256, M // 4), bias=False).cuda()        # ~M*1024 parameters
    flat = FlatParams(lin, want_bf16_shadow=True)
    opt = FlatOptimizer(flat, "adamw", lr=1e-3, weight_decay=0.01, grad_clip=1.0)
    flat.grads.normal_()
    n = flat.params.numel()
    return (lambda: opt.step()), n * (4 * 7 + 2) + n * 4, 0.0     # norm pass reads g; update reads p,g,m,v writes p,m,v,shadow


CASES: Dict[str, Callable] = {"imag_bwd": case_imag_bwd, "linear": case_linear, "dgrad": case_dgrad, "wgrad": case_wgrad,
                              "wgrad_grouped": case_wgrad_grouped, "ffn_core_fwd": case_ffn_core_fwd,
                              "ffn_core_bwd": case_ffn_core_bwd, "attn_fwd": case_attn_fwd, "attn_fwd_library": case_attn_fwd_library, "attn_bwd": case_attn_bwd,
                              "dread_slot_bwd": case_dread_slot_bwd, "dread_fwd": case_dread_fwd,
                              "optimizer": case_optimizer}


def time_op(fn, iters: int, warmup: int, flush: torch.Tensor) -> float:
    """Median milliseconds over ``iters`` launches, each preceded by an L2 flush outside the timed events."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        flush.add_(1)                                   # evicts L2 (buffer larger than L2)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    times.sort()
    return times[len(times) // 2]


def run(op: str, tokens: int, iters: int, warmup: int) -> Dict[str, float]:
    K = kmod.CudaKernels()
    fn, byts, flops = CASES[op](K, tokens)
    flush = torch.zeros(160 * 1024 * 1024 // 4, device="cuda")
    ms = time_op(fn, iters, warmup, flush)
    kmod.check_status(torch.device("cuda"))
    assert not K.fallbacks, f"library fallback used: {dict(K.fallbacks)}"
    pk, kind = peaks()
    gbs, tfl = byts / ms / 1e6, flops / ms / 1e9
    return {"op": op, "tokens": tokens, "ms": ms, "GB/s": gbs, "TFLOP/s": tfl, "frac_hbm": gbs / pk["hbm_gbs"],
            "frac_bf16": tfl / pk["bf16_tflops"], "peaks": kind}


GEMM_SHAPES = [(2048, 768, 3072), (2048, 768, 768), (2048, 1152, 768), (2048, 3072, 768), (2048, 8192, 768),
               (32768, 3072, 768)]          # (M, N, K): the linear layers of the 113M training step + one large case


def time_burst(fn, n: int = 20) -> float:
    """Milliseconds per launch over ``n`` back-to-back launches (operands stay in L2: what a graph replay sees)."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(n):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / n


def gemm_table(iters: int, warmup: int, variants=("auto", "cta64", "cta128", "cta256", "pair128", "pair192", "pair256")) -> None:
    """Every forward-linear shape of the step: this repository's kernel with each tile shape, and the library GEMM
    (``torch.nn.functional.linear`` -> cuBLAS) timed in the same run the same way.  Two timings per entry: one launch
    after an L2 flush (cold), and back-to-back launches (warm)."""
    import torch.nn.functional as F
    K = kmod.CudaKernels()
    flush = torch.zeros(160 * 1024 * 1024 // 4, device="cuda")
    pk, kind = peaks()
    print(f"{'M,N,K':>18s} " + " ".join(f"{v:>15s}" for v in variants) + f" {'library':>15s}   us cold/warm; best ours "
          f"as TFLOP/s warm and fraction of {kind} bf16 peak")
    for (M, N, Kd) in GEMM_SHAPES:
        x, w = bf(M, Kd), bf(N, Kd, scale=0.03)
        ref = F.linear(x, w)
        cells, best = [], 1e9
        for v in variants:
            if v == "auto":
                os.environ.pop("LOOM_GEMM_TILE", None)
            else:
                os.environ["LOOM_GEMM_TILE"] = v
            y = K.linear(x, w)
            err = float((y.float() - ref.float()).abs().max() / (ref.float().abs().max() + 1e-6))
            assert err < 2e-2, (M, N, Kd, v, err)
            cold = time_op(lambda: K.linear(x, w), iters, warmup, flush) * 1e3
            warm = time_burst(lambda: K.linear(x, w)) * 1e3
            best = min(best, warm)
            cells.append(f"{cold:7.1f}/{warm:7.1f}")
        os.environ.pop("LOOM_GEMM_TILE", None)
        lib_cold = time_op(lambda: F.linear(x, w), iters, warmup, flush) * 1e3
        lib_warm = time_burst(lambda: F.linear(x, w)) * 1e3
        tfl = 2.0 * M * N * Kd / best / 1e6
        print(f"{M:6d},{N:5d},{Kd:5d} " + " ".join(cells) + f" {lib_cold:7.1f}/{lib_warm:7.1f}   {tfl:7.1f} "
              f"{tfl / pk['bf16_tflops']:.2f}")
    kmod.check_status(torch.device("cuda"))


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--op", default="all", choices=["all", "gemm_shapes"] + sorted(CASES))
    ap.add_argument("--vs", default=None, choices=[None, "library"],
                    help="with --op gemm_shapes: also time the library GEMM on every shape (always on for that op)")
    ap.add_argument("--tokens", type=int, default=32768, help="rows M = batch x chunk tokens")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args(argv)
    torch.manual_seed(0)
    if a.op == "gemm_shapes":
        gemm_table(a.iters, a.warmup)
        return
    print(f"{'op':14s} {'tokens':>7s} {'ms':>9s} {'GB/s':>9s} {'of HBM':>7s} {'TFLOP/s':>9s} {'of bf16':>8s}")
    for op in (sorted(CASES) if a.op == "all" else [a.op]):
        r = run(op, a.tokens, a.iters, a.warmup)
        print(f"{r['op']:14s} {r['tokens']:7d} {r['ms']:9.4f} {r['GB/s']:9.1f} {r['frac_hbm']:7.3f} {r['TFLOP/s']:9.1f} "
              f"{r['frac_bf16']:8.3f}   ({r['peaks']} peaks)")
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
