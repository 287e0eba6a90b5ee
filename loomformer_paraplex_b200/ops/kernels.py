"""CUDA kernel set: the sm_100a implementations behind the fused plan's kernel interface.

``CudaKernels`` derives from the PyTorch twins, so an operation that has no native kernel yet (or a
shape the native kernel does not cover, e.g. a row pitch that is not 16-byte aligned) runs through
PyTorch on the GPU.  Which operations ran natively is visible in ``native.launches()`` and in
``CudaKernels.fallbacks`` -- nothing is hidden.
"""
from __future__ import annotations

from collections import Counter
from typing import List, Optional

import os

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


def has_status_word(device) -> bool:
    return str(device) in _STATUS


def check_status(device) -> None:
    code = int(status_word(device).item())
    if code != 0:
        status_word(device).zero_()
        raise RuntimeError(f"a kernel gave up a bounded wait (code {code}); results of this step are invalid")


def _tma_ok(t: torch.Tensor) -> bool:
    return (t.is_cuda and t.dtype == torch.bfloat16 and t.stride(-1) == 1 and t.data_ptr() % 16 == 0
            and all((s * 2) % 16 == 0 for s in t.stride()[:-1]))


def _pick_bn(M: int, N: int, heads: int = 1) -> int:
    """Tile width.  Measured on B200 (M = 2048 rows, the chunk size): 128-wide tiles beat 64-wide ones whenever the
    output is at least 128 wide (a 64-wide tile reads 192 B of shared memory per tensor-core clock, more than the
    128 B/clk an SM delivers), and 256-wide tiles pay off only when they still give about three waves of CTAs."""
    tiles_m = -(-M // 128)
    if N >= 256 and tiles_m * (-(-N // 256)) * heads >= 3 * 148:
        return 256
    return 128 if N >= 128 else 64


_FORCED_TILE = {"cta64": (64, 0), "cta128": (128, 0), "cta256": (256, 0), "pair128": (128, 1), "pair192": (192, 1),
                "pair256": (256, 1)}


def _pick_tile(M: int, N: int, heads: int = 1, plain: bool = True, K: int = 0):
    """``(tile width, pair)``.  ``pair`` selects 256-row tiles computed by clusters of two CTAs
    (``tcgen05.mma.cta_group::2``): each SM stages 128 rows of A and only half of the tile's B columns per k-block.
    Measured on B200 against the single-CTA tiles (back-to-back launches, M = 2048): pair tiles are as fast or faster
    on every linear shape of the training step, 256-wide ones unless the reduction is long and only the 128-wide ones
    give enough tiles to occupy the 74 SM pairs.  ``LOOM_GEMM_TILE`` (cta64|cta128|cta256|pair128|pair192|pair256) forces one
    shape for sweeps; ``LOOM_GEMM_PAIR=0`` turns pair tiles off."""
    forced = os.environ.get("LOOM_GEMM_TILE")
    if forced in _FORCED_TILE:
        bn, pair = _FORCED_TILE[forced]
        if not pair or (plain and N > 64 and M >= 256):
            return bn, pair
    small_n = int(os.environ.get("LOOM_GEMM_PAIR_MIN_N", "65"))      # narrowest output that still takes pair tiles
    if plain and M >= 256 and N >= small_n and os.environ.get("LOOM_GEMM_PAIR", "1") != "0":
        rows = -(-M // 256)
        t256 = rows * (-(-N // 256)) * heads
        # 256-wide pair tiles when they occupy at least half of the 74 SM pairs (a long reduction wants all of them)
        if N >= 256 and (t256 >= 74 or (K < 4096 and t256 >= 37)):
            return 256, 1
        return 128, 1
    return _pick_bn(M, N, heads), 0


def gemm(a_list: List[torch.Tensor], k_len: List[int], b, c: torch.Tensor, *, M: int, N: int,
         heads: int = 1, a_mn: bool = False, b_mn: bool = False, a_k0: Optional[List[int]] = None,
         b_k0: Optional[List[int]] = None, bias: Optional[torch.Tensor] = None, accumulate: bool = False,
         bn: Optional[int] = None, swap_mn: bool = False, peer_ptrs: Optional[List[int]] = None,
         gather_rank: int = 0, a_peer_ptrs: Optional[List[int]] = None, a_rows_per_rank: int = 0,
         rs_out_ptrs: Optional[List[int]] = None, rs_rows_per_rank: int = 0, rs_rank: int = 0,
         pair: Optional[int] = None) -> None:
    ext = native.ext()
    n = len(a_list)
    plain = not (peer_ptrs or a_peer_ptrs or rs_out_ptrs)
    if pair is None:
        if bn:
            pair = 0
        else:
            bn, pair = _pick_tile(M, N, heads, plain, sum(int(k) for k in k_len))
    if bn == 192 and (a_mn or b_mn or not pair):
        bn = 128                                     # 192-wide tiles exist for K-major operands on pair tiles only
    ext.gemm(a_list, k_len, a_k0 or [0] * n, b_k0 or [0] * n, b if isinstance(b, (list, tuple)) else [b], a_mn, b_mn,
             c, bias, M, N, heads, accumulate,
             bn or _pick_bn(M, N, heads), swap_mn, status_word(c.device), peer_ptrs or [], gather_rank,
             a_peer_ptrs or [], a_rows_per_rank, rs_out_ptrs or [], rs_rows_per_rank, rs_rank, int(pair))
    native.count()


def upload_hyper(opt) -> torch.Tensor:
    """Step-dependent optimizer scalars -> device array (async copy from a rotating pinned buffer)."""
    dev = opt.flat.device
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
    return opt._hyper_dev


def optimizer_step(opt) -> None:
    """Native flat optimizer step (norm -> clip -> status gate -> AdamW/ATOM -> bf16 shadow), four launches."""
    ext = native.ext()
    f = opt.flat
    upload_hyper(opt)
    atom_out = opt.atom_out if opt.kind == "atom" else None
    ext.grad_norm(f.grads, opt.grad_clip, opt._partial, opt.stats, atom_out)
    ext.status_gate(status_word(f.device), opt.stats)     # a timed-out wait skips the update like a NaN does
    if opt.kind == "adamw":
        ext.adamw_flat(f.params, f.grads, opt.m, opt.v, f.shadow, opt.lr_mult_blk, opt.wd_blk, opt.active_blk,
                       opt.stats, opt._hyper_dev)
    else:
        ext.atom_flat(f.params, f.grads, opt.m, opt.v, f.shadow, opt.lr_mult_blk, opt.wd_blk, opt.cnt_blk,
                      opt.gprev_blk, opt.pnode_blk, opt.trust_blk, opt.stats, opt._hyper_dev, opt.atom_out)
    native.count(4)


class CudaKernels(TorchKernels):
    name = "cuda"

    # weight-gradient products of this many chunks go out as one launch (LOOM_WGRAD_GROUP overrides, 1..16)
    WGRAD_GROUP = max(1, min(16, int(os.environ.get("LOOM_WGRAD_GROUP", "16"))))

    def __init__(self, defer_wgrad: bool = True) -> None:
        native.ext()
        self.fallbacks: Counter = Counter()
        self.defer_wgrad = defer_wgrad
        self._wq: dict = {}
        # grouped weight-gradient launches go to a second stream (nothing reads a weight gradient before the end of
        # the backward pass); their operands stay referenced until the join in flush_wgrads.  LOOM_WGRAD_STREAM=0
        # keeps them on the launching stream.
        self._wg_side = None
        self._wg_inflight: list = []
        self._wg_overlap = defer_wgrad and os.environ.get("LOOM_WGRAD_STREAM", "1") != "0"

    # ------------------------------------------------------------------ grouped weight gradients
    def _wgrad(self, dy, x, gw, M, N, heads=1):
        """gw[M, (heads,) N] += dy^T x.  The chunk-serial backward produces one such product per chunk for every
        weight; with a reduction length of only B*Tc rows each is a short, poorly filled GEMM.  They are queued
        instead (the operands stay alive in the queue) and issued as ONE launch whose reduction runs over all
        queued chunks -- same arithmetic, one pass over the fp32 gradient instead of sixteen."""
        if not self.defer_wgrad:
            gemm([dy], [dy.shape[0]], x, gw, M=M, N=N, heads=heads, a_mn=True, b_mn=True, accumulate=True)
            return
        key = (gw.data_ptr(), M, N, heads, tuple(gw.stride()))
        ent = self._wq.get(key)
        if ent is None:
            ent = self._wq[key] = ([], [], gw)
        ent[0].append(dy)
        ent[1].append(x)
        if len(ent[0]) >= self.WGRAD_GROUP:
            self._flush_one(key)

    def _flush_one(self, key):
        dys, xs, gw = self._wq.pop(key)
        _, M, N, heads, _ = key
        if not self._wg_overlap:
            gemm(dys, [t.shape[0] for t in dys], xs, gw, M=M, N=N, heads=heads, a_mn=True, b_mn=True, accumulate=True)
            return
        dev = gw.device
        if self._wg_side is None:
            self._wg_side = torch.cuda.Stream(device=dev)
        side = self._wg_side
        side.wait_stream(torch.cuda.current_stream(dev))       # the operands were produced on the launching stream
        with torch.cuda.stream(side):
            gemm(dys, [t.shape[0] for t in dys], xs, gw, M=M, N=N, heads=heads, a_mn=True, b_mn=True, accumulate=True)
        self._wg_inflight.append((dys, xs, gw))                # keep the memory from being reused before the join

    def flush_wgrads(self) -> None:
        """Issue what is still queued and make the launching stream wait for every weight-gradient launch."""
        for key in list(self._wq):
            self._flush_one(key)
        if self._wg_inflight:
            torch.cuda.current_stream(self._wg_inflight[0][2].device).wait_stream(self._wg_side)
            self._wg_inflight.clear()

    # ------------------------------------------------------------------ small per-cell bookkeeping
    def begin_step(self, zero_floats: int, device) -> None:
        """One fill per step instead of one per accumulator: the step's fp32 zero-initialised buffers are slices of
        this pool (a slice is handed out once; when the pool runs out ``zeros`` allocates as usual)."""
        self._zpool = torch.zeros(max(int(zero_floats), 0), dtype=torch.float32, device=device)
        self._zoff = 0

    def zeros(self, *shape, device=None):
        n = 1
        for v in shape:
            n *= int(v)
        pool = getattr(self, "_zpool", None)
        span_ = (n + 63) // 64 * 64                      # keep every slice 256-byte aligned
        dv = torch.device(device)
        same = pool is not None and pool.device.type == dv.type and dv.index in (None, pool.device.index)
        if not same or self._zoff + span_ > pool.numel():
            return torch.zeros(*shape, dtype=torch.float32, device=device)
        out = pool[self._zoff:self._zoff + n].view(*shape)
        self._zoff += span_
        return out

    def anchor_update(self, beta_sq_sum, n_el, anchor, decay):
        if not (anchor.is_cuda and anchor.dtype == torch.float32 and beta_sq_sum.dtype == torch.float32):
            self.fallbacks["anchor_update"] += 1
            return super().anchor_update(beta_sq_sum, n_el, anchor, decay)
        snap = torch.empty((), dtype=torch.float32, device=anchor.device)
        native.ext().anchor_ema(beta_sq_sum, 1.0 / float(n_el), float(decay), anchor, snap)
        native.count()
        return snap

    # ------------------------------------------------------------------ GEMMs
    def linear(self, x, w, bias=None, out_dtype=None, gather=None, out=None):
        """``gather=(peer_ptrs, rank)``: ``w`` is this rank's copy of a row-sharded weight; the launch fetches every
        64-row block from the rank that owns it and completes the local copy on the way.  ``out``: a packed bf16
        [M, N] buffer the epilogue stores into (saves the copy into a pre-allocated slot)."""
        M, Kd = x.shape
        N = w.shape[0]
        out_ok = out is None or (out.dtype == torch.bfloat16 and out.is_contiguous() and tuple(out.shape) == (M, N)
                                 and out.data_ptr() % 16 == 0 and out_dtype in (None, torch.bfloat16))
        if not (_tma_ok(x) and _tma_ok(w) and out_ok) or (out_dtype not in (None, torch.bfloat16, torch.float32)):
            if gather is not None:
                raise RuntimeError("a sharded weight needs the TMA path (16-byte aligned bf16 rows)")
            self.fallbacks["linear"] += 1
            return super().linear(x, w, bias, out_dtype, out)
        c = out if out is not None else torch.empty(M, N, dtype=out_dtype or torch.bfloat16, device=x.device)
        b32 = None if bias is None else bias.float().contiguous()
        if gather is not None:
            gemm([x], [Kd], w, c, M=M, N=N, bias=b32, peer_ptrs=list(gather[0]), gather_rank=int(gather[1]))
        else:
            gemm([x], [Kd], w, c, M=M, N=N, bias=b32)
        return c

    def qkv_rope(self, d, x, w, cos, sin, qkc, kcache, vcache, s):
        """The projection and the rotation as one launch: 192- or 256-wide CTA-pair tiles hold whole heads, and the
        epilogue rotates Q and K in fp32 straight from the accumulator and writes the attention operand and the caches
        (``csrc/gemm.cu: store_tile_rope``).  Off unless ``LOOM_QKV_ROPE=1``: on the 113M training step the per-row
        stores of this epilogue cost what the separate rotation launch costs (145.8 against 145.2 ms per step)."""
        B, Tc = cos.shape[:2]
        M = x.shape[0]
        bn = 192 if 192 % d.hd == 0 else (256 if 256 % d.hd == 0 else 0)
        ok = (bn and d.hd in (64, 96, 128) and M >= 256 and M == B * Tc and _tma_ok(x) and _tma_ok(w)
              and qkc.dtype == torch.bfloat16 and qkc.is_contiguous() and kcache.dtype == torch.bfloat16
              and kcache.is_contiguous() and vcache.is_contiguous() and kcache.shape[0] == B
              and os.environ.get("LOOM_QKV_ROPE", "0") == "1" and os.environ.get("LOOM_GEMM_PAIR", "1") != "0")
        if not ok:
            return super().qkv_rope(d, x, w, cos, sin, qkc, kcache, vcache, s)
        native.ext().gemm_qkv_rope(x, w, None, _f32c(cos).view(M, d.hd), _f32c(sin).view(M, d.hd), qkc[:, 0].view(M, d.n),
                                   kcache, vcache, Tc, int(s), d.qh, d.kvh, d.hd, bn, status_word(x.device))
        native.count()

    def linear_small(self, x, w, bias=None, out=None, out_dtype=None):
        """``x @ w^T (+ bias)`` for a handful of rows (the decode step): up to 16 rows go through the weight-streaming
        kernel (``csrc/decode_step.cu``), more through the tensor-core GEMM.  ``out`` may be a row-strided bf16 / fp32
        view (a history slot), which saves the copy."""
        M, Kd = x.shape
        N = w.shape[0]
        ok = (x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1 and w.stride(1) == 1
              and Kd % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
              and w.data_ptr() % 16 == 0)
        if M > 16 or not ok:
            if out is not None and not (out.is_contiguous() and out.dtype == torch.bfloat16):
                out.copy_(self.linear(x, w, bias, out_dtype))
                return out
            return self.linear(x, w, bias, out_dtype, out=out)
        y = out if out is not None else torch.empty(M, N, dtype=out_dtype or torch.bfloat16, device=x.device)
        native.ext().skinny_linear(x, w, None if bias is None else _f32c(bias), y)
        native.count()
        return y

    def linear_multi(self, segs, static_weights=False):
        """Several small-batch products in one launch, at most 12 segments each: up to 16 rows through the
        weight-streaming kernel (``csrc/decode_step.cu``), up to 128 through the weight-stationary tensor-core kernel
        (``csrc/decode_gemm.cu``: weight rows as the M side of the MMA, batch as N); more rows fall back to one GEMM
        per segment.  ``static_weights``: nothing earlier in the stream writes the weights or biases (an inference
        engine's copies), so the kernels may fetch them while their predecessor runs."""
        M = segs[0][3].shape[0]

        def piece_ok(t):
            return (t.dtype == torch.bfloat16 and t.dim() == 2 and t.stride(1) == 1 and t.shape[1] % 8 == 0
                    and (M == 1 or (t.stride(0) % 8 == 0 and t.stride(0) >= t.shape[1])) and t.data_ptr() % 16 == 0)

        ok = M <= 128 and all(all(piece_ok(x) for x in pieces) and piece_ok(w) and out.stride(1) == 1
                              and out.dtype in (torch.bfloat16, torch.float32) for pieces, w, _, out in segs)
        if not ok:
            for pieces, w, bias, out in segs:
                x = pieces[0] if len(pieces) == 1 else torch.cat(list(pieces), -1)
                self.linear_small(x.contiguous(), w, bias, out=out)
            return
        packed = [(list(pieces), w, None if bias is None else _f32c(bias), out) for pieces, w, bias, out in segs]
        for i in range(0, len(packed), 12):
            if M <= 16:
                native.ext().skinny_multi(packed[i:i + 12], bool(static_weights))
            else:
                native.ext().decode_gemm(packed[i:i + 12], bool(static_weights), status_word(segs[0][3].device))
            native.count()

    def linear_dgrad(self, dy, w, out=None, accumulate=False):
        """``dy @ w``; with ``out`` the product is written (or, with ``accumulate``, added) into that bf16 buffer by
        the GEMM's epilogue, which saves the separate add that sums gradient branches."""
        M, N = dy.shape
        Kd = w.shape[1]
        if not (_tma_ok(dy) and _tma_ok(w)) or (out is not None and (out.dtype != torch.bfloat16 or out.stride(-1) != 1)):
            self.fallbacks["linear_dgrad"] += 1
            return super().linear_dgrad(dy, w, out, accumulate)
        c = out if out is not None else torch.empty(M, Kd, dtype=torch.bfloat16, device=dy.device)
        gemm([dy], [N], w, c, M=M, N=Kd, b_mn=True, accumulate=bool(accumulate and out is not None))
        return c

    def linear_dgrad_multi(self, segs):
        """``sum_i dy_i @ w_i`` as ONE launch: the reduction runs over the concatenation of the segments, each with its
        own weight operand, so gradient branches that end in the same tensor need neither separate launches nor
        read-modify-write accumulation.  Segments ``(None, value)`` are added afterwards."""
        prod = [(dy, w) for dy, w in segs if dy is not None]
        vals = [w for dy, w in segs if dy is None]
        if not prod or len(prod) > 16 or not all(_tma_ok(dy) and _tma_ok(w) for dy, w in prod):
            self.fallbacks["linear_dgrad_multi"] += 1
            return super().linear_dgrad_multi(segs)
        M, N = prod[0][0].shape[0], prod[0][1].shape[1]
        c = torch.empty(M, N, dtype=torch.bfloat16, device=prod[0][0].device)
        if len(prod) == 1:
            gemm([prod[0][0]], [prod[0][0].shape[1]], prod[0][1], c, M=M, N=N, b_mn=True)
        else:
            gemm([dy for dy, _ in prod], [dy.shape[1] for dy, _ in prod], [w for _, w in prod], c, M=M, N=N, b_mn=True)
        for v in vals:
            c += v.to(c.dtype)
        return c

    def linear_wgrad(self, dy, x, gw):
        dy2, x2 = dy.reshape(-1, dy.shape[-1]), x.reshape(-1, x.shape[-1])
        if not (_tma_ok(dy2) and _tma_ok(x2) and gw.dtype == torch.float32 and gw.stride(-1) == 1 and gw.dim() == 2):
            self.fallbacks["linear_wgrad"] += 1
            return super().linear_wgrad(dy, x, gw)
        self._wgrad(dy2, x2, gw, dy2.shape[1], x2.shape[1])

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

    def imag_bwd(self, d, dbeta, qkc, u, m2, w_imag, gw_imag, du_acc=None, defer_u=False):
        """``du_acc``: an existing bf16 ``[M, N]`` gradient of ``u`` to add this projection's share into (returned as
        ``du``) instead of allocating a new one.  ``defer_u``: leave the data gradient of the shared ``u`` sector to
        the caller: ``du`` is ``None`` and a fourth element ``(dbeta, weight slice)`` is returned, a segment for
        :meth:`linear_dgrad_multi`."""
        M = u.shape[0]
        ok = (_tma_ok(qkc) and _tma_ok(u) and _tma_ok(m2) and _tma_ok(w_imag) and _tma_ok(dbeta)
              and d.hd % 8 == 0 and d.hpq % 8 == 0 and gw_imag.dtype == torch.float32)
        if not ok:
            self.fallbacks["imag_bwd"] += 1
            return super().imag_bwd(d, dbeta, qkc, u, m2, w_imag, gw_imag, du_acc, defer_u)
        hd, n, H = d.hd, d.n, d.hidden
        dev = u.device
        w3 = w_imag.view(d.qh, d.hpq, d.imag_in).transpose(0, 1)             # [HPQ, QH, IMAG_IN]
        g3 = gw_imag.view(d.qh, d.hpq, d.imag_in).transpose(0, 1)
        db3 = dbeta.view(M, d.qh, d.hpq)
        dqkc = torch.empty_like(qkc)
        acc_u = du_acc is not None and du_acc.dtype == torch.bfloat16 and du_acc.stride(-1) == 1
        du = None if defer_u else (du_acc if acc_u else torch.empty(M, n, dtype=torch.bfloat16, device=dev))
        u_seg = None
        dm2 = torch.empty(M, d.qh, hd, dtype=torch.bfloat16, device=dev)
        m2v = m2.view(M, d.qh, hd)

        def per_head(col0, a_src, c_dst):
            # data gradient of a head-local sector and its weight gradient
            gemm([db3], [d.hpq], w3[:, :, col0:col0 + hd], c_dst, M=M, N=hd, heads=d.qh, b_mn=True)
            self._wgrad(db3, a_src, g3[:, :, col0:col0 + hd], d.hpq, hd, d.qh)

        def shared(col0, a_src2d, c_dst2d, accumulate=False):
            if c_dst2d is not None:
                gemm([dbeta], [H], w_imag[:, col0:col0 + n], c_dst2d, M=M, N=n, b_mn=True, accumulate=accumulate)
            self._wgrad(dbeta, a_src2d, gw_imag[:, col0:col0 + n], H, n)

        if d.open_sectors:
            per_head(0, qkc[:, 0], dqkc[:, 0])
            shared(hd, qkc[:, 1].reshape(M, n), dqkc[:, 1].reshape(M, n))
            shared(hd + n, qkc[:, 2].reshape(M, n), dqkc[:, 2].reshape(M, n))
            shared(hd + 2 * n, u, du, acc_u)
            u_seg = (dbeta, w_imag[:, hd + 2 * n:hd + 3 * n])
            shared(hd + 3 * n, m2v.reshape(M, n), dm2.view(M, n))
        else:
            # the three attention sectors of a head are adjacent columns of its weight block: one batched data-gradient
            # GEMM with N = 3 * head_dim into [M, QH, 3, HD], then one strided copy into the [M, 3, QH, HD] order the
            # attention backward reads (two launches instead of three GEMMs); the weight gradients stay per sector
            # because their inputs are the sectors of qkc
            tmp = torch.empty(M, d.qh, 3 * hd, dtype=torch.bfloat16, device=dev)
            gemm([db3], [d.hpq], w3[:, :, 0:3 * hd], tmp, M=M, N=3 * hd, heads=d.qh, b_mn=True)
            if dqkc.is_contiguous():
                native.ext().sector_fold(tmp, dqkc, M, d.qh, hd)
            else:
                dqkc.copy_(tmp.view(M, d.qh, 3, hd).transpose(1, 2))
            native.count()
            for s_ in range(3):
                self._wgrad(db3, qkc[:, s_], g3[:, :, s_ * hd:(s_ + 1) * hd], d.hpq, hd, d.qh)
            shared(3 * hd, u, du, acc_u)
            u_seg = (dbeta, w_imag[:, 3 * hd:3 * hd + n])
            per_head(3 * hd + n, m2v, dm2)
        if defer_u:
            return dqkc, None, dm2, u_seg
        if du_acc is not None and not acc_u:
            du = du_acc + du
        return dqkc, du, dm2


def _bf16c(t: torch.Tensor) -> torch.Tensor:
    return t if (t.dtype == torch.bfloat16 and t.is_contiguous()) else t.to(torch.bfloat16).contiguous()


def _f32c(t: torch.Tensor) -> torch.Tensor:
    return t if (t.dtype == torch.float32 and t.is_contiguous()) else t.float().contiguous()


def _opt(t, fn):
    return None if t is None else fn(t)


class _ElementwiseMixin:
    """Native versions of the bandwidth-bound operations (see csrc/elementwise.cu, ffn_core.cu, temporal.cu)."""

    # ------------------------------------------------------------------ rope
    def rope_store(self, d, qkv, cos, sin, qkc, kcache, vcache, s):
        B, Tc, _ = qkv.shape
        if qkv.dtype != torch.bfloat16 or d.hd % 2:
            self.fallbacks["rope_store"] += 1
            return super().rope_store(d, qkv, cos, sin, qkc, kcache, vcache, s)
        native.ext().rope_store(qkv.contiguous(), _f32c(cos).view(B * Tc, d.hd), _f32c(sin).view(B * Tc, d.hd), qkc,
                                kcache, vcache, B * Tc, Tc, kcache.shape[1], s, d.qh, d.kvh, d.hd)
        native.count()

    def rope_bwd(self, d, dq_attn, dqkc, dkc, dvc, s, e, cos, sin, out_dtype):
        B, Tc = dq_attn.shape[:2]
        if out_dtype != torch.bfloat16:
            self.fallbacks["rope_bwd"] += 1
            return super().rope_bwd(d, dq_attn, dqkc, dkc, dvc, s, e, cos, sin, out_dtype)
        out = torch.empty(B, Tc, d.n + 2 * d.kv_dim, dtype=torch.bfloat16, device=dq_attn.device)
        native.ext().rope_bwd(_bf16c(dq_attn), _bf16c(dqkc), dkc, dvc, _f32c(cos).view(B * Tc, d.hd),
                              _f32c(sin).view(B * Tc, d.hd), out, B * Tc, Tc, dkc.shape[1], s, d.qh, d.kvh, d.hd,
                              dkc.shape[2] // d.kvh)
        native.count()
        return out

    # ------------------------------------------------------------------ attention
    def _attn_ok(self, d, qkc, s, e):
        # any chunk length (the kernels walk 128-row query tiles) and any head dim that keeps rows 16-byte aligned
        return qkc.dtype == torch.bfloat16 and d.hd % 8 == 0 and d.hd <= 128 and e > s

    def attn_fwd(self, d, qkc, kcache, vcache, s, e, seg):
        if not self._attn_ok(d, qkc, s, e):
            self.fallbacks["attn_fwd"] += 1
            return super().attn_fwd(d, qkc, kcache, vcache, s, e, seg)
        B, T = kcache.shape[0], kcache.shape[1]
        Tc = e - s
        lse = torch.empty(B, d.qh, Tc, dtype=torch.float32, device=qkc.device)
        seg32 = None if seg is None else (seg if seg.dtype == torch.int32 else seg.to(torch.int32)).contiguous()
        native.ext().attn(False, qkc, kcache, vcache, lse, seg32, None, None, None, None, B, d.qh, d.kvh, d.hd, Tc, T,
                          s, e, status_word(qkc.device))
        native.count()
        return lse

    def alloc_kv_grad(self, d, B, T, device):
        """Per-query-head key/value gradient slabs (the GQA group sum happens in rope_bwd)."""
        if d.hd % 8 or d.hd > 128:
            return super().alloc_kv_grad(d, B, T, device)
        return torch.zeros(B, T, d.qh, d.hd, dtype=torch.float32, device=device)

    def attn_bwd(self, d, dqkc, qkc, kcache, vcache, lse, s, e, seg, dkcache, dvcache):
        if not self._attn_ok(d, qkc, s, e) or dkcache.shape[2] != d.qh:
            self.fallbacks["attn_bwd"] += 1
            if dkcache.shape[2] != d.kvh:
                raise RuntimeError("attention backward fallback needs kv-head shaped gradient buffers")
            return super().attn_bwd(d, dqkc, qkc, kcache, vcache, lse, s, e, seg, dkcache, dvcache)
        B, T = kcache.shape[0], kcache.shape[1]
        Tc = e - s
        dq = torch.empty(B * Tc, d.qh, d.hd, dtype=torch.bfloat16, device=qkc.device)
        seg32 = None if seg is None else (seg if seg.dtype == torch.int32 else seg.to(torch.int32)).contiguous()
        native.ext().attn(True, qkc, kcache, vcache, lse, seg32, _bf16c(dqkc), dq, dkcache, dvcache, B, d.qh, d.kvh, d.hd,
                          Tc, T, s, e, status_word(qkc.device))
        native.count()
        return dq

    # ------------------------------------------------------------------ depth attention
    def _dread_ok(self, d, hist_k, hist_v=None, dense=False):
        """History is [slots, M, QH, HD] bf16 with unit strides inside a row; K and V may interleave as [K | V] rows of
        one buffer (slot and row strides multiples of 8 elements).  ``dense``: the kernel wants a packed tensor."""
        if not (hist_k.dtype == torch.bfloat16 and d.hd % 8 == 0 and d.hd <= 128 and hist_k.dim() == 4):
            return False
        if dense:
            return hist_k.is_contiguous()
        ok = (hist_k.stride(3) == 1 and hist_k.stride(2) == d.hd and hist_k.stride(1) % 8 == 0
              and hist_k.stride(0) % 8 == 0 and hist_k.data_ptr() % 16 == 0)
        if ok and hist_v is not None:
            ok = hist_v.stride() == hist_k.stride() and hist_v.data_ptr() % 16 == 0
        return ok

    def dread_fwd(self, d, q_row, hist_k, hist_v, n):
        if not self._dread_ok(d, hist_k, hist_v):
            self.fallbacks["dread_fwd"] += 1
            return super().dread_fwd(d, q_row, hist_k, hist_v, n)
        M = hist_k.shape[1]
        out = torch.empty(M, d.qh, d.hd, dtype=torch.bfloat16, device=hist_k.device)
        lse = torch.empty(M, d.qh, dtype=torch.float32, device=hist_k.device)
        native.ext().dread(False, _f32c(q_row), hist_k, hist_v, out, lse, None, None, None, None, n, M * d.qh, d.qh, d.hd)
        native.count()
        return out, lse

    def dread_bwd(self, d, dm, m, lse, q_row, hist_k, hist_v, n, dhist_k, dhist_v, gq):
        if not (self._dread_ok(d, hist_k, dense=True) and hist_v.is_contiguous()):
            self.fallbacks["dread_bwd"] += 1
            return super().dread_bwd(d, dm, m, lse, q_row, hist_k, hist_v, n, dhist_k, dhist_v, gq)
        M = hist_k.shape[1]
        native.ext().dread(True, _f32c(q_row), hist_k, hist_v, _bf16c(m), lse, _bf16c(dm), dhist_k, dhist_v, gq, n,
                           M * d.qh, d.qh, d.hd)
        native.count()

    def dread_stage(self, d, a, b, m, lse, dst, sub):
        dm_all = dst["dm"]
        if not (dm_all.dtype == torch.bfloat16 and d.hd % 8 == 0 and d.hd <= 128):
            self.fallbacks["dread_stage"] += 1
            return super().dread_stage(d, a, b, m, lse, dst, sub)
        M = dm_all.shape[1]
        native.ext().dread_stage(_bf16c(a), _opt(b, _bf16c), _bf16c(m), dm_all[sub], dst["dd"][sub], _f32c(lse),
                                 dst["lse"][sub], M * d.qh, d.hd)
        native.count()

    def dread_slot_bwd(self, d, slot, q_all, hist_k, hist_v, dm_all, lse_all, dd_all, gq_all):
        pairs = (dm_all.shape[0] - slot) * d.hd          # the kernel keeps at most 20 (sublayer, dim) pairs per thread
        if not (self._dread_ok(d, hist_k, hist_v) and dm_all.dtype == torch.bfloat16 and pairs <= 256 * 20):
            self.fallbacks["dread_slot_bwd"] += 1
            return super().dread_slot_bwd(d, slot, q_all, hist_k, hist_v, dm_all, lse_all, dd_all, gq_all)
        S, M = dm_all.shape[0], dm_all.shape[1]
        dkv = torch.empty(M, 2, d.qh, d.hd, dtype=torch.bfloat16, device=hist_k.device)     # rows [dK | dV]
        native.ext().dread_slot_bwd(q_all, hist_k[slot], hist_v[slot], dm_all, lse_all, dd_all, dkv[:, 0], dkv[:, 1],
                                    gq_all, slot, S, M, d.qh, d.hd)
        native.count()
        return dkv

    # ------------------------------------------------------------------ add + LayerNorm
    def add_ln_fwd(self, a, b, w, bias, cap, eps=1e-5):
        M, N = a.shape
        if N % 8 or N > 2048 or a.dtype != torch.bfloat16:
            self.fallbacks["add_ln_fwd"] += 1
            return super().add_ln_fwd(a, b, w, bias, cap, eps)
        y, x = torch.empty_like(a), torch.empty_like(a)
        mean = torch.empty(M, dtype=torch.float32, device=a.device)
        rstd = torch.empty(M, dtype=torch.float32, device=a.device)
        native.ext().add_ln_fwd(a.contiguous(), _bf16c(b), w, bias, y, x, mean, rstd, M, N, eps,
                                float(cap) if cap is not None else 0.0)
        native.count()
        return y, x, mean, rstd

    def add_ln_bwd(self, dy, x, mean, rstd, w, gw, gb, cap, a, b):
        M, N = x.shape
        if N % 8 or N > 2048 or x.dtype != torch.bfloat16:
            self.fallbacks["add_ln_bwd"] += 1
            return super().add_ln_bwd(dy, x, mean, rstd, w, gw, gb, cap, a, b)
        dx = torch.empty_like(x)
        native.ext().add_ln_bwd(_bf16c(dy), x, mean, rstd, w, dx, gw, gb, M, N)
        native.count()
        if cap is None:
            return dx, dx
        da, db = torch.empty_like(x), torch.empty_like(x)
        native.ext().cap_bwd(dx, _bf16c(a), da, M, N, float(cap))
        native.ext().cap_bwd(dx, _bf16c(b), db, M, N, float(cap))
        native.count(2)
        return da, db

    def colsum_add(self, dy, gb):
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.dtype != torch.bfloat16 or dy2.shape[1] % 2 or dy2.stride(1) != 1 or not gb.is_contiguous():
            self.fallbacks["colsum_add"] += 1
            return super().colsum_add(dy, gb)
        native.ext().colsum(dy2, gb, dy2.shape[0], dy2.shape[1])
        native.count()

    # ------------------------------------------------------------------ loss
    def ce_fwd_bwd(self, logits, targets, ignore_index, grad_scale):
        if logits.dtype != torch.bfloat16 or logits.shape[1] % 8 or not logits.is_contiguous():
            self.fallbacks["ce"] += 1
            return super().ce_fwd_bwd(logits, targets, ignore_index, grad_scale)
        M = logits.shape[0]
        targets = targets.contiguous()
        n = targets.ne(ignore_index).sum().clamp(min=1).float()
        nll = torch.empty(M, dtype=torch.float32, device=logits.device)
        scale = ((grad_scale if grad_scale is not None else 0.0) / n).reshape(1)
        native.ext().ce(logits, targets, nll, scale, ignore_index, grad_scale is not None)
        native.count()
        return nll.sum() / n, (logits if grad_scale is not None else None)

    # ------------------------------------------------------------------ paraplex core + tria
    def _core_ok(self, d, x_real):
        return x_real.dtype == torch.bfloat16 and d.hidden % 2 == 0 and d.activation == "pvpowlu"

    def ffn_core_fwd(self, d, x_real, p_in, alpha_gate, b_real, gate_lin, beta_lin, b_imag, w_trace, trace_in,
                     reset, anchor, c_prev, seed, seed_valid, gate_w, axis, tria_alpha, B, trace_out=None, bsq=None):
        if not self._core_ok(d, x_real):
            self.fallbacks["ffn_core_fwd"] += 1
            return super().ffn_core_fwd(d, x_real, p_in, alpha_gate, b_real, gate_lin, beta_lin, b_imag, w_trace,
                                        trace_in, reset, anchor, c_prev, seed, seed_valid, gate_w, axis, tria_alpha, B,
                                        trace_out, bsq)
        M, H = x_real.shape
        dev = x_real.device
        o = torch.empty(M, H, dtype=torch.bfloat16, device=dev)
        c = torch.empty(9, M, H, dtype=torch.bfloat16, device=dev) if axis is not None else None
        p_out = torch.empty(M, H, dtype=torch.bfloat16, device=dev) if (axis is not None and gate_w is not None) else None
        if trace_out is None:
            trace_out = torch.empty(B, H, dtype=torch.float32, device=dev)
        if bsq is None:
            bsq = self.zeros(1, device=dev)
        native.ext().ffn_core(
            False, B, M // B, H, -1 if axis is None else axis, bool(d.phase_secant), d.powlu_m, tria_alpha, d.phase_floor,
            _opt(alpha_gate if p_in is not None else None, lambda t: _f32c(t).reshape(1)), None,
            x_real, _opt(p_in, _bf16c), _f32c(b_real), _opt(gate_lin, _bf16c), _bf16c(beta_lin), _f32c(b_imag),
            _f32c(w_trace), _opt(trace_in, _f32c), _opt(reset, lambda t: t.contiguous()), c_prev,
            _opt(seed, _f32c), _opt(seed_valid, lambda t: t.contiguous()), _opt(gate_w, _f32c),
            o, c, p_out, trace_out, bsq, None, None, None, None, None, None, None, None, None, None, None, None,
            None, None, None, None)
        native.count()
        return {"r": None, "gsrc": None, "o": o, "i": None, "trace_out": trace_out, "beta_sq_sum": bsq[0], "c": c,
                "p_out": p_out}

    def ffn_core_bwd(self, d, saved, do, dc, dp_out, dtrace_out):
        x_real = saved["x_real"]
        if not self._core_ok(d, x_real):
            self.fallbacks["ffn_core_bwd"] += 1
            return super().ffn_core_bwd(d, saved, do, dc, dp_out, dtrace_out)
        M, H = x_real.shape
        B, dev = saved["B"], x_real.device
        p_in, gate_lin, c_prev, seed, trace_in = (saved.get(k) for k in ("p_in", "gate_lin", "c_prev", "seed", "trace_in"))
        axis = saved.get("axis")
        bf = dict(dtype=torch.bfloat16, device=dev)
        dx = torch.empty(M, H, **bf)
        dpin = torch.empty(M, H, **bf) if p_in is not None else None
        dgl = torch.empty(M, H, **bf) if gate_lin is not None else None
        dbeta = torch.empty(M, H, **bf)
        gz = torch.empty(M, H, dtype=torch.float32, device=dev)
        dcp = torch.empty(9, M, H, **bf) if (c_prev is not None and axis is not None) else None
        dseed = self.zeros(B, H, 9, device=dev) if (seed is not None and axis is not None) else None
        dtr = self.zeros(B, H, device=dev) if trace_in is not None else None
        acc = saved.get("gsc_acc")
        gsc = acc if acc is not None else torch.zeros(10, dtype=torch.float32, device=dev)
        gate_w = saved.get("gate_w")
        native.ext().ffn_core(
            True, B, M // B, H, -1 if axis is None else axis, bool(d.phase_secant), d.powlu_m, saved.get("tria_alpha") or 0.0,
            d.phase_floor,
            _opt(saved.get("alpha_gate") if p_in is not None else None, lambda t: _f32c(t).reshape(1)),
            _opt(saved.get("anchor"), lambda t: _f32c(t).reshape(1)),
            x_real, _opt(p_in, _bf16c), _f32c(saved["b_real"]), _opt(gate_lin, _bf16c), _bf16c(saved["beta_lin"]),
            _f32c(saved["b_imag"]), _f32c(saved["w_trace"]), _opt(trace_in, _f32c),
            _opt(saved.get("reset"), lambda t: t.contiguous()), c_prev, _opt(seed, _f32c),
            _opt(saved.get("seed_valid"), lambda t: t.contiguous()), _opt(gate_w, _f32c),
            None, None, None, None, None,
            _bf16c(do), _opt(dc, _bf16c), _opt(dp_out if gate_w is not None else None, _bf16c), _opt(dtrace_out, _f32c),
            dx, dpin, dgl, dbeta, gz, dcp, dseed, dtr,
            saved["g_b_real"], saved["g_w_trace"], saved["g_b_imag"], gsc)
        native.count(2)
        return {"d_x_real": dx, "d_p_in": dpin, "d_gate_lin": dgl, "d_beta_lin": dbeta, "d_trace_in": dtr,
                "d_c_prev": dcp, "d_seed": dseed, "d_b_real": None, "d_b_imag": None, "d_w_trace": None,
                "d_alpha_gate": gsc[0] if (p_in is not None and acc is None) else None,
                "d_gate_w": gsc[1:10] if (gate_w is not None and acc is None) else None}

    # ------------------------------------------------------------------ readout: slot pool and sparse cross attention
    def slot_pool_fwd(self, keys, score_w):
        if not (keys.dtype == torch.float32 and keys.is_contiguous() and keys.dim() == 4):
            self.fallbacks["slot_pool_fwd"] += 1
            return super().slot_pool_fwd(keys, score_w)
        B, Kn, H, _ = keys.shape
        pooled = torch.empty(B, Kn, 9, dtype=torch.float32, device=keys.device)
        self._pool_stats = torch.empty(B * Kn, 2, dtype=torch.float32, device=keys.device)
        self._pool_out = pooled
        native.ext().slot_pool(False, keys, _f32c(score_w), pooled, self._pool_stats, None, None, None, B * Kn, H)
        native.count()
        return pooled

    def slot_pool_bwd(self, dpooled, keys, score_w):
        st = getattr(self, "_pool_stats", None)
        if st is None or not (keys.dtype == torch.float32 and keys.is_contiguous()) or st.shape[0] != keys.shape[0] * keys.shape[1]:
            self.fallbacks["slot_pool_bwd"] += 1
            return super().slot_pool_bwd(dpooled, keys, score_w)
        B, Kn, H, _ = keys.shape
        dkeys = torch.empty_like(keys)
        part = torch.empty(B * Kn, 9, dtype=torch.float32, device=keys.device)
        native.ext().slot_pool(True, keys, _f32c(score_w), self._pool_out, st, _f32c(dpooled), dkeys, part, B * Kn, H)
        native.count()
        return dkeys, part.sum(0)

    def cross_attn_fwd(self, q, k, v, allowed, scale):
        B, T, N = q.shape
        Kn = k.shape[1]
        if not (q.dtype == torch.bfloat16 and N % 8 == 0 and N <= 2048 and 1 <= Kn <= 1024):
            self.fallbacks["cross_attn_fwd"] += 1
            return super().cross_attn_fwd(q, k, v, allowed, scale)
        out = torch.empty_like(q)
        self._ca_prob = torch.empty(B, T, Kn, dtype=torch.float32, device=q.device)
        native.ext().cross_attn(False, q.contiguous(), k.contiguous(), v.contiguous(), allowed.to(torch.uint8).contiguous(),
                                out, self._ca_prob, None, None, None, B, T, Kn, N, float(scale))
        native.count()
        return out

    def cross_attn_bwd(self, dout, q, k, v, allowed, scale):
        B, T, N = q.shape
        Kn = k.shape[1]
        prob = getattr(self, "_ca_prob", None)
        if prob is None or prob.shape != (B, T, Kn) or q.dtype != torch.bfloat16:
            self.fallbacks["cross_attn_bwd"] += 1
            return super().cross_attn_bwd(dout, q, k, v, allowed, scale)
        ds = torch.empty_like(prob)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        native.ext().cross_attn(True, q.contiguous(), k.contiguous(), v.contiguous(), _bf16c(dout), dq, prob, ds, dk, dv,
                                B, T, Kn, N, float(scale))
        native.count(2)
        return dq, dk, dv

    # ------------------------------------------------------------------ RMS-type norms
    @staticmethod
    def _rows_view(x):
        """[M, heads, HD] bf16 view with contiguous heads -> (rows, heads, HD, row pitch) or None."""
        if x.dim() != 3 or x.dtype != torch.bfloat16 or x.stride(2) != 1 or x.stride(1) != x.shape[2]:
            return None
        if x.shape[2] % 8 or x.shape[2] > 128 or x.data_ptr() % 16 or (x.stride(0) * 2) % 16:
            return None
        return x.shape[0] * x.shape[1], x.shape[1], x.shape[2], x.stride(0)

    def fixed_rms_fwd(self, x, target):
        rv = self._rows_view(x)
        if rv is None:
            if x.numel() > 65536:
                self.fallbacks["fixed_rms_fwd"] += 1
            return super().fixed_rms_fwd(x, target)
        rows, heads, hd, ld = rv
        y = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device)
        native.ext().fixed_rms(False, None, x, y, rows, heads, hd, ld, float(target), 1e-6)
        native.count()
        return y

    def fixed_rms_bwd(self, dy, x, target, eps=1e-6):
        rv = self._rows_view(x)
        if rv is None or dy.dtype != torch.bfloat16 or not dy.is_contiguous():
            if x.numel() > 65536:
                self.fallbacks["fixed_rms_bwd"] += 1
            return super().fixed_rms_bwd(dy, x, target, eps)
        rows, heads, hd, ld = rv
        dx = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device)
        native.ext().fixed_rms(True, dy, x, dx, rows, heads, hd, ld, float(target), float(eps))
        native.count()
        return dx

    def rms_norm_fwd(self, x, w, eps=1e-6):
        N = x.shape[-1]
        if not (x.dtype == torch.bfloat16 and x.is_contiguous() and N % 8 == 0 and N <= 2048):
            self.fallbacks["rms_norm_fwd"] += 1
            return super().rms_norm_fwd(x, w, eps)
        y = torch.empty_like(x)
        native.ext().rms_norm(False, None, x, _f32c(w), y, None, x.numel() // N, N, float(eps))
        native.count()
        return y

    def rms_norm_bwd(self, dy, x, w, gw, eps=1e-6):
        N = x.shape[-1]
        if not (x.dtype == torch.bfloat16 and x.is_contiguous() and N % 8 == 0 and N <= 2048):
            self.fallbacks["rms_norm_bwd"] += 1
            return super().rms_norm_bwd(dy, x, w, gw, eps)
        M = x.numel() // N
        dx = torch.empty_like(x)
        part = torch.empty(min(296, -(-M // 8)), N, dtype=torch.float32, device=x.device)
        native.ext().rms_norm(True, _bf16c(dy), x, _f32c(w), dx, part, M, N, float(eps))
        gw.add_(part.sum(0))
        native.count()
        return dx

    # ------------------------------------------------------------------ temporal endpoint
    def temporal_fwd(self, depth, B, Tc, H, reset, state, fired, polarm_beta):
        if not (depth.dim() == 3 and depth.shape[0] == 9):          # carriers came from the PyTorch twin
            self.fallbacks["temporal_fwd"] += 1
            return super().temporal_fwd(depth, B, Tc, H, reset, state, fired, polarm_beta)
        dev = depth.device
        out = torch.empty(B, H, 9, dtype=torch.float32, device=dev)
        raw = torch.empty(B, H, 9, dtype=torch.float32, device=dev)
        nck = Tc // 16          # must match CKPT in csrc/temporal.cu
        ck = torch.empty(nck, B, H, 9, dtype=torch.float32, device=dev) if nck > 0 else None
        native.ext().temporal_fwd(depth, reset.contiguous(), _opt(state, _f32c), _opt(fired, lambda t: t.contiguous()),
                                  polarm_beta, out, raw, ck, B, Tc, H)
        native.count()
        return out, {"raw": raw, "ckpt": ck}

    def temporal_bwd(self, dstate, depth, B, Tc, H, reset, state, fired, polarm_beta, aux):
        if aux is None or "raw" not in aux:
            self.fallbacks["temporal_bwd"] += 1
            return super().temporal_bwd(dstate, depth, B, Tc, H, reset, state, fired, polarm_beta, aux)
        dev = depth.device
        ddepth = torch.empty_like(depth)
        dprev = torch.empty(B, H, 9, dtype=torch.float32, device=dev) if state is not None else None
        native.ext().temporal_bwd(depth, reset.contiguous(), _opt(state, _f32c), _opt(fired, lambda t: t.contiguous()),
                                  polarm_beta, aux["raw"], aux["ckpt"], _f32c(dstate.reshape(B, H, 9)), ddepth, dprev,
                                  B, Tc, H)
        native.count()
        return ddepth, dprev


class CudaKernels(_ElementwiseMixin, CudaKernels):      # noqa: F811  (final kernel set = GEMMs + element-wise kernels)
    """``LOOM_DISABLE_OPS=attn_fwd,attn_bwd,ffn_core_fwd,...`` (or ``all``) sends the named operations of a new kernel set
    to their PyTorch twins, for bisecting a numerical difference to one kernel; each such call is counted in
    ``fallbacks`` like any other library fallback.  The reference has per-op switches of the same kind
    (``LOOM_TRIA_DISABLE_OPS``, reference ``tria.py:104-109``)."""

    def __init__(self, *args, **kw) -> None:
        super().__init__(*args, **kw)
        names = [n.strip() for n in os.environ.get("LOOM_DISABLE_OPS", "").split(",") if n.strip()]
        if not names:
            return
        if names == ["all"]:
            names = [n for n in dir(TorchKernels) if not n.startswith("_") and callable(getattr(TorchKernels, n))]
        for n in names:
            twin = getattr(TorchKernels, n, None)
            if twin is None or not callable(twin) or n in ("flush_wgrads",):
                raise ValueError(f"LOOM_DISABLE_OPS: {n!r} is not an operation of the kernel set")

            def routed(*a, _twin=twin, _n=n, **k):
                self.fallbacks[_n] += 1
                return _twin(self, *a, **k)
            setattr(self, n, routed)
