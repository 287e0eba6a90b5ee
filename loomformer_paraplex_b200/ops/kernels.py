"""CUDA kernel set: the sm_100a implementations behind the fused plan's kernel interface.

``CudaKernels`` derives from the PyTorch twins, so an operation that has no native kernel yet (or a
shape the native kernel does not cover, e.g. a row pitch that is not 16-byte aligned) runs through
PyTorch on the GPU.  Which operations ran natively is visible in ``native.launches()`` and in
``CudaKernels.fallbacks`` -- nothing is hidden.
"""
from __future__ import annotations

from collections import Counter
from typing import List, Optional

import torch

from . import native
from .twins import TorchKernels

_STATUS = {}


def status_word(device) -> torch.Tensor:
    """Device word that bounded waits inside kernels set when they give up (0 = healthy)."""
    key = str(device)
    if key not in _STATUS:
        _STATUS[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _STATUS[key]


def check_status(device) -> None:
    code = int(status_word(device).item())
    if code != 0:
        status_word(device).zero_()
        raise RuntimeError(f"a kernel gave up a bounded wait (code {code}); results of this step are invalid")


def _tma_ok(t: torch.Tensor) -> bool:
    return (t.is_cuda and t.dtype == torch.bfloat16 and t.stride(-1) == 1 and t.data_ptr() % 16 == 0
            and all((s * 2) % 16 == 0 for s in t.stride()[:-1]))


def _pick_bn(M: int, N: int, heads: int = 1) -> int:
    tiles_m = -(-M // 128)
    for bn in (256, 128, 64):
        if N >= bn and tiles_m * (-(-N // bn)) * heads >= 120:
            return bn
    return 64 if N <= 64 else 128


def gemm(a_list: List[torch.Tensor], k_len: List[int], b: torch.Tensor, c: torch.Tensor, *, M: int, N: int,
         heads: int = 1, a_mn: bool = False, b_mn: bool = False, a_k0: Optional[List[int]] = None,
         b_k0: Optional[List[int]] = None, bias: Optional[torch.Tensor] = None, accumulate: bool = False,
         bn: Optional[int] = None, swap_mn: bool = False) -> None:
    ext = native.ext()
    n = len(a_list)
    ext.gemm(a_list, k_len, a_k0 or [0] * n, b_k0 or [0] * n, b, a_mn, b_mn, c, bias, M, N, heads, accumulate,
             bn or _pick_bn(M, N, heads), swap_mn, status_word(c.device))
    native.count()


def optimizer_step(opt) -> None:
    """Native flat optimizer step (norm -> clip -> AdamW/ATOM -> bf16 shadow), three launches."""
    ext = native.ext()
    f = opt.flat
    dev = f.device
    if not hasattr(opt, "_hyper_dev"):
        opt._hyper_ring = [torch.zeros(8, dtype=torch.float32).pin_memory() for _ in range(8)]
        opt._hyper_dev = torch.zeros(8, dtype=torch.float32, device=dev)
        opt._partial = torch.zeros(1024, dtype=torch.float32, device=dev)
    t = opt.step_count
    b1, b2 = opt.betas
    h = opt._hyper_ring[t % 8]      # rotating pinned buffers: the async copy of an older step may still be queued
    h[0], h[1], h[2], h[3] = opt.lr, b1, b2, opt.eps
    h[4], h[5] = 1.0 - b1 ** t, 1.0 - b2 ** t
    h[6] = 1.0 if (opt.kind == "atom" and t <= opt.bootstrap_steps) else 0.0
    opt._hyper_dev.copy_(h, non_blocking=True)
    atom_out = opt.atom_out if opt.kind == "atom" else None
    ext.grad_norm(f.grads, opt.grad_clip, opt._partial, opt.stats, atom_out)
    if opt.kind == "adamw":
        ext.adamw_flat(f.params, f.grads, opt.m, opt.v, f.shadow, opt.lr_mult_blk, opt.wd_blk, opt.active_blk,
                       opt.stats, opt._hyper_dev)
    else:
        ext.atom_flat(f.params, f.grads, opt.m, opt.v, f.shadow, opt.lr_mult_blk, opt.wd_blk, opt.cnt_blk,
                      opt.gprev_blk, opt.pnode_blk, opt.trust_blk, opt.stats, opt._hyper_dev, opt.atom_out)
    native.count(3)


class CudaKernels(TorchKernels):
    name = "cuda"

    def __init__(self) -> None:
        native.ext()
        self.fallbacks: Counter = Counter()

    # ------------------------------------------------------------------ GEMMs
    def linear(self, x, w, bias=None, out_dtype=None):
        M, Kd = x.shape
        N = w.shape[0]
        if not (_tma_ok(x) and _tma_ok(w)) or (out_dtype not in (None, torch.bfloat16, torch.float32)):
            self.fallbacks["linear"] += 1
            return super().linear(x, w, bias, out_dtype)
        c = torch.empty(M, N, dtype=out_dtype or torch.bfloat16, device=x.device)
        b32 = None if bias is None else bias.float().contiguous()
        gemm([x], [Kd], w, c, M=M, N=N, bias=b32)
        return c

    def linear_dgrad(self, dy, w):
        M, N = dy.shape
        Kd = w.shape[1]
        if not (_tma_ok(dy) and _tma_ok(w)):
            self.fallbacks["linear_dgrad"] += 1
            return super().linear_dgrad(dy, w)
        c = torch.empty(M, Kd, dtype=torch.bfloat16, device=dy.device)
        gemm([dy], [N], w, c, M=M, N=Kd, b_mn=True)
        return c

    def linear_wgrad(self, dy, x, gw):
        dy2, x2 = dy.reshape(-1, dy.shape[-1]), x.reshape(-1, x.shape[-1])
        if not (_tma_ok(dy2) and _tma_ok(x2) and gw.dtype == torch.float32 and gw.stride(-1) == 1 and gw.dim() == 2):
            self.fallbacks["linear_wgrad"] += 1
            return super().linear_wgrad(dy, x, gw)
        gemm([dy2], [dy2.shape[0]], x2, gw, M=dy2.shape[1], N=x2.shape[1], a_mn=True, b_mn=True, accumulate=True)

    # ------------------------------------------------------------------ imaginary projection
    def imag_fwd(self, d, qkc, u, m2, w_imag):
        M = u.shape[0]
        if not (_tma_ok(qkc) and _tma_ok(u) and _tma_ok(m2) and _tma_ok(w_imag) and d.hd % 8 == 0 and d.hpq % 8 == 0):
            self.fallbacks["imag_fwd"] += 1
            return super().imag_fwd(d, qkc, u, m2, w_imag)
        hd, n = d.hd, d.n
        beta = torch.empty(M, d.hidden, dtype=torch.bfloat16, device=u.device)
        w3 = w_imag.view(d.qh, d.hpq, d.imag_in).transpose(0, 1)             # [HPQ, QH, IMAG_IN]
        c3 = beta.view(M, d.qh, d.hpq)
        if d.open_sectors:
            segs = [qkc[:, 0], qkc[:, 1].reshape(M, n), qkc[:, 2].reshape(M, n), u, m2.reshape(M, n)]
            lens = [hd, n, n, n, n]
        else:
            segs = [qkc[:, 0], qkc[:, 1], qkc[:, 2], u, m2.view(M, d.qh, hd)]
            lens = [hd, hd, hd, n, hd]
        offs = [0]
        for k in lens[:-1]:
            offs.append(offs[-1] + k)
        gemm(segs, lens, w3, c3, M=M, N=d.hpq, heads=d.qh, b_k0=offs)
        return beta

    def imag_bwd(self, d, dbeta, qkc, u, m2, w_imag, gw_imag):
        M = u.shape[0]
        ok = (_tma_ok(qkc) and _tma_ok(u) and _tma_ok(m2) and _tma_ok(w_imag) and _tma_ok(dbeta)
              and d.hd % 8 == 0 and d.hpq % 8 == 0 and gw_imag.dtype == torch.float32)
        if not ok:
            self.fallbacks["imag_bwd"] += 1
            return super().imag_bwd(d, dbeta, qkc, u, m2, w_imag, gw_imag)
        hd, n, H = d.hd, d.n, d.hidden
        dev = u.device
        w3 = w_imag.view(d.qh, d.hpq, d.imag_in).transpose(0, 1)             # [HPQ, QH, IMAG_IN]
        g3 = gw_imag.view(d.qh, d.hpq, d.imag_in).transpose(0, 1)
        db3 = dbeta.view(M, d.qh, d.hpq)
        dqkc = torch.empty_like(qkc)
        du = torch.empty(M, n, dtype=torch.bfloat16, device=dev)
        dm2 = torch.empty(M, d.qh, hd, dtype=torch.bfloat16, device=dev)
        m2v = m2.view(M, d.qh, hd)

        def per_head(col0, a_src, c_dst):
            # data gradient of a head-local sector and its weight gradient
            gemm([db3], [d.hpq], w3[:, :, col0:col0 + hd], c_dst, M=M, N=hd, heads=d.qh, b_mn=True)
            gemm([db3], [M], a_src, g3[:, :, col0:col0 + hd], M=d.hpq, N=hd, heads=d.qh, a_mn=True, b_mn=True,
                 accumulate=True)

        def shared(col0, a_src2d, c_dst2d):
            gemm([dbeta], [H], w_imag[:, col0:col0 + n], c_dst2d, M=M, N=n, b_mn=True)
            gemm([dbeta], [M], a_src2d, gw_imag[:, col0:col0 + n], M=H, N=n, a_mn=True, b_mn=True, accumulate=True)

        if d.open_sectors:
            per_head(0, qkc[:, 0], dqkc[:, 0])
            shared(hd, qkc[:, 1].reshape(M, n), dqkc[:, 1].reshape(M, n))
            shared(hd + n, qkc[:, 2].reshape(M, n), dqkc[:, 2].reshape(M, n))
            shared(hd + 2 * n, u, du)
            shared(hd + 3 * n, m2v.reshape(M, n), dm2.view(M, n))
        else:
            per_head(0, qkc[:, 0], dqkc[:, 0])
            per_head(hd, qkc[:, 1], dqkc[:, 1])
            per_head(2 * hd, qkc[:, 2], dqkc[:, 2])
            shared(3 * hd, u, du)
            per_head(3 * hd + n, m2v, dm2)
        return dqkc, du, dm2
