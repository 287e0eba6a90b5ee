"""Pure-PyTorch definitions of every LoomFormer operator.

These functions *are the numerics contract*: the sm_100a kernels in ``ops/csrc`` are tested
against them in fp32, and they are the execution path on CPU (gloo plumbing runs, unit tests,
tools).  They are written against explicit arguments (no module-global shapes) and are fully
differentiable through ordinary autograd, except where the model defines a custom gradient
(the bounded phase nonlinearity).

Formulas follow the reference implementation's fallbacks
(``loomformer.py:2013-2056, 2212-2248, 2621-2638, 3433-3449``; ``tria.py:35-93, 128-166,
989-1123, 1346-1389, 1444-1455``).
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

HALF_PI = math.pi / 2.0
_LOWP = (torch.float16, torch.bfloat16)


def _up(x: torch.Tensor) -> torch.Tensor:
    return x.float() if x.dtype in _LOWP else x


# --------------------------------------------------------------------------- norms
def fixed_rms(x: torch.Tensor, target: float = 1.0, eps: float = 1e-6) -> torch.Tensor:
    """``x * target / sqrt(mean(x^2) + eps)`` over the last dim (statistics in fp32)."""
    s = torch.rsqrt(_up(x).square().mean(-1, keepdim=True) + eps) * float(target)
    return x * s.to(x.dtype)


def capped_rms(x: torch.Tensor, cap: float = 1.0, eps: float = 1e-6) -> torch.Tensor:
    """Shrink vectors whose RMS exceeds ``cap``; never amplify."""
    rms = torch.sqrt(_up(x).square().mean(-1, keepdim=True) + eps)
    return x * (float(cap) / rms).clamp(max=1.0).to(x.dtype)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * weight


# --------------------------------------------------------------------------- phase
def phase_angle(beta: torch.Tensor) -> torch.Tensor:
    return HALF_PI * beta * torch.rsqrt(1.0 + beta * beta)


class _PhaseSin(torch.autograd.Function):
    """``sin(pi/2 * b/sqrt(1+b^2))`` with the model's surrogate slope.

    floor mode: ``max(cos x, floor) * dx/db``.  secant mode: slope of the chord from the
    anchor point ``a`` to ``b`` (true slope when ``|b-a| < near``).
    """

    @staticmethod
    def forward(ctx, beta, anchor, floor: float, near: float):
        ctx.save_for_backward(beta, anchor if anchor is not None else beta.new_empty(0))
        ctx.secant = anchor is not None
        ctx.floor, ctx.near = float(floor), float(near)
        return torch.sin(phase_angle(beta))

    @staticmethod
    def backward(ctx, g):
        beta, anchor = ctx.saved_tensors
        x = phase_angle(beta)
        dx = HALF_PI * (1.0 + beta * beta).pow(-1.5)
        if ctx.secant:
            gap = beta - anchor
            near = gap.abs() < ctx.near
            chord = (torch.sin(x) - torch.sin(phase_angle(anchor))) / torch.where(near, torch.ones_like(gap), gap)
            slope = torch.where(near, torch.cos(x) * dx, chord)
        else:
            slope = torch.cos(x).clamp(min=ctx.floor) * dx
        return g * slope, None, None, None


def phase_sin(beta: torch.Tensor, anchor: Optional[torch.Tensor] = None, floor: float = 0.05,
              near: float = 1e-4) -> torch.Tensor:
    """Bounded phase nonlinearity.  ``anchor`` (a detached scalar snapshot) selects secant mode."""
    if anchor is not None:
        anchor = anchor.detach().clone()
    return _PhaseSin.apply(beta, anchor, floor, near)


def phase_radius(beta: torch.Tensor, floor: float = 1e-4) -> torch.Tensor:
    """Detached fp32 RMS of ``beta`` over all elements, clamped below by ``floor``."""
    return beta.detach().float().square().mean().sqrt().clamp_min(float(floor))


def shift_trace(s0: torch.Tensor, carried: Optional[torch.Tensor], reset: Optional[torch.Tensor]) -> torch.Tensor:
    """Previous-token phase of the same neuron: ``[carried, s0[:, :-1]]`` zeroed at resets."""
    B, T, H = s0.shape
    first = s0.new_zeros(B, 1, H) if carried is None else carried.to(s0.dtype).view(B, 1, H)
    prev = torch.cat((first, s0[:, :-1]), dim=1)
    if reset is not None:
        prev = prev.masked_fill(reset.to(torch.bool).unsqueeze(-1), 0)
    return prev


def squash(z: torch.Tensor) -> torch.Tensor:
    return z * torch.rsqrt(1.0 + z * z)


# --------------------------------------------------------------------------- activations
def powlu(x: torch.Tensor, m: float = 3.0) -> torch.Tensor:
    xp = x.clamp(min=1e-12)
    pos = xp.pow(1.0 + m / (xp.sqrt() + 1.0)) * torch.sigmoid(x)
    return torch.where(x > 0, pos, x.pow(2) * torch.sigmoid(x))


def powlu_gate(a: torch.Tensor, m: float = 3.0) -> torch.Tensor:
    """``a^(m/(sqrt(a)+1)) * sigmoid(a)`` for strictly positive ``a`` (a softplus output)."""
    return a.pow(m / (a.sqrt() + 1.0)) * torch.sigmoid(a)


def paraplex_core(
    r: torch.Tensor, gate_src: torch.Tensor, beta_lin: torch.Tensor, bias: torch.Tensor,
    trace_w: torch.Tensor, carried: Optional[torch.Tensor], reset: Optional[torch.Tensor],
    anchor: Optional[torch.Tensor], *, floor: float, m: float, activation: str = "pvpowlu",
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Everything between the up-projections and ``w2``.

    Returns ``(O, I, next_trace)`` where ``I`` is the squashed phase and ``next_trace`` the raw
    phase of the last token (what the next chunk / decode step consumes).
    """
    beta = beta_lin + bias
    s0 = phase_sin(beta, anchor, floor)
    prev = shift_trace(s0, carried, reset)
    i_sq = squash(s0 + prev * trace_w.view(1, 1, -1))
    amp = F.softplus(gate_src)
    p = torch.addcmul(r, amp, i_sq)
    if activation == "pvpowlu":
        out = p * powlu_gate(amp, m)
    elif activation == "gelu":
        out = F.gelu(p)
    else:
        out = powlu(p, m)
    return out, i_sq, s0[:, -1, :]


# --------------------------------------------------------------------------- attention
def rotate_half(x: torch.Tensor) -> torch.Tensor:
    a, b = x.chunk(2, dim=-1)
    return torch.cat((-b, a), dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """``x``: [B,T,heads,HD]; ``cos``/``sin``: [B or 1, T, 1, HD]."""
    return x * cos + rotate_half(x) * sin


def dual_context_attention(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, allowed: torch.Tensor, group: int,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Softmax attention that returns both ``A@K`` and ``A@V`` per query head.

    q: [B,Tq,QH,HD]; k, v: [B,Tk,KVH,HD]; ``allowed``: bool broadcastable to [B,1,Tq,Tk].
    Softmax is evaluated in fp32.  Returns ``(k_ctx, v_ctx)``, each [B,Tq,QH,HD].
    """
    B, Tq, QH, HD = q.shape
    kq = k.repeat_interleave(group, dim=2).transpose(1, 2)
    vq = v.repeat_interleave(group, dim=2).transpose(1, 2)
    s = torch.matmul(q.transpose(1, 2), kq.transpose(-1, -2)) / math.sqrt(HD)
    s = s.masked_fill(~allowed, float("-inf"))
    a = torch.softmax(s.float(), dim=-1).to(vq.dtype)
    return torch.matmul(a, kq).transpose(1, 2).contiguous(), torch.matmul(a, vq).transpose(1, 2).contiguous()


def depth_read(q_row: torch.Tensor, hist_k: torch.Tensor, hist_v: torch.Tensor) -> torch.Tensor:
    """One learned query per head against ``S`` stored depth states.

    q_row: [QH,HD]; hist_k/hist_v: [S,B,T,QH,HD].  Returns [B,T,QH,HD] (fp32 softmax over S).
    """
    hd = q_row.shape[-1]
    s = (hist_k.float() * q_row.float()).sum(-1) / math.sqrt(hd)          # [S,B,T,QH]
    w = torch.softmax(s, dim=0)
    return (w.unsqueeze(-1) * hist_v.float()).sum(0).to(hist_v.dtype)


# --------------------------------------------------------------------------- Tria (3x3 carriers)
def normalize9(m: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """Divide each 3x3 matrix by ``sqrt(mean of its 9 squared entries + eps)``."""
    w = _up(m)
    out = w / torch.sqrt(w.square().mean(dim=(-1, -2), keepdim=True) + eps)
    return out.to(m.dtype)


def build_tria(r: torch.Tensor, i: torch.Tensor, o: torch.Tensor, alpha: float, axis: int,
               eps: float = 1e-6) -> torch.Tensor:
    """``(I + alpha*K(a,b,c)) @ R_axis`` with ``(a,b,c) = tanh(x / rms(x))``, ``x = (ri, ro, io)``."""
    if axis not in (0, 1, 2):
        raise ValueError(f"axis must be 0(z), 1(x), or 2(y), got {axis}")
    x = torch.stack((r * i, r * o, i * o), dim=-1)
    x = torch.tanh(x / torch.sqrt(x.square().mean(-1, keepdim=True) + eps)) * float(alpha)
    a, b, c = x.unbind(-1)
    one = torch.ones_like(a)
    if axis == 0:
        rows = ((-c, -one, b), (one, -c, -a), (a, b, one))
    elif axis == 1:
        rows = ((one, b, c), (c, -a, -one), (-b, one, -a))
    else:
        rows = ((-b, -c, one), (a, one, c), (-one, a, -b))
    return torch.stack([torch.stack(row, dim=-1) for row in rows], dim=-2)


def tria_compose(
    r: torch.Tensor, i: torch.Tensor, o: torch.Tensor, alpha: float, axis: int,
    prev: Optional[torch.Tensor] = None, seed: Optional[torch.Tensor] = None,
    seed_valid: Optional[torch.Tensor] = None, gate_w: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """One depth step of the carrier chain.

    ``prev`` [B,T,H,3,3]: ``C = N(T_l @ prev)``.  Without ``prev``: ``C = N(T_l)`` except that the
    first token of rows with ``seed_valid`` uses ``N(T_l @ seed)`` (``seed`` [B,H,3,3]).
    ``gate_w`` [9] (already soft-maxed) additionally returns ``p = <gate_w, vec(C)>``.
    """
    t = build_tria(r, i, o, alpha, axis)
    if prev is not None:
        pre = torch.matmul(t, prev.to(t.dtype))
    elif seed is not None:
        first = torch.matmul(t[:, 0], seed.to(t.dtype))
        first = torch.where(seed_valid.to(torch.bool)[:, None, None, None], first, t[:, 0])
        pre = torch.cat((first.unsqueeze(1), t[:, 1:]), dim=1)
    else:
        pre = t
    c = normalize9(pre)
    p = None
    if gate_w is not None:
        p = (c.reshape(*c.shape[:3], 9) * gate_w).sum(-1)
    return c, p


def temporal_endpoint(depth: torch.Tensor, reset: torch.Tensor, state: Optional[torch.Tensor] = None,
                      eps: float = 1e-6) -> torch.Tensor:
    """Run ``acc = N(D_t @ acc)`` over a chunk and return only the final accumulator.

    depth: [B,T,H,3,3]; reset: [B,T] restarts ``acc = N(D_t)``; ``state`` [B,H,3,3] is the
    accumulator entering the chunk (``None`` = start fresh).  Works in fp32.
    """
    w = _up(depth)
    reset = reset.to(torch.bool)
    acc = None if state is None else state.to(w.dtype)
    for t in range(w.shape[1]):
        d = w[:, t]
        if acc is None:
            pre = d
        else:
            pre = torch.where(reset[:, t, None, None, None], d, torch.matmul(d, acc))
        acc = normalize9(pre, eps)
    return acc


def temporal_scan(depth: torch.Tensor, reset: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """Full trajectory of the temporal recurrence, [B,T,H,3,3] in fp32 (index 0 always restarts)."""
    w = _up(depth)
    reset = reset.to(torch.bool)
    outs, acc = [], None
    for t in range(w.shape[1]):
        d = w[:, t]
        pre = d if acc is None else torch.where(reset[:, t, None, None, None], d, torch.matmul(d, acc))
        acc = normalize9(pre, eps)
        outs.append(acc)
    return torch.stack(outs, dim=1)


def polarm(m: torch.Tensor, beta: float, eps: float = 1e-6) -> torch.Tensor:
    """One Gram-correction step toward a scaled orthogonal matrix: ``M (I - beta/2 (G^ - I))``."""
    if not math.isfinite(beta) or beta < 0.0 or beta >= 1.0:
        raise ValueError(f"PolARM beta must be finite and in [0, 1), got {beta}")
    w = _up(m)
    g = w.transpose(-1, -2) @ w
    scale = g.diagonal(dim1=-2, dim2=-1).mean(-1, keepdim=True).unsqueeze(-1).clamp_min(eps)
    eye = torch.eye(3, device=w.device, dtype=w.dtype)
    return (w @ (eye - 0.5 * beta * (g / scale - eye))).to(m.dtype)


def slot_pool(carry: torch.Tensor, score_w: torch.Tensor) -> torch.Tensor:
    """Softmax over neurons of ``<score_w, vec(C_h)>`` then the pooled 9-vector.  [B,K,H,3,3] -> [B,K,9]."""
    slots = carry.reshape(*carry.shape[:3], 9)
    w = torch.softmax((slots * score_w.to(slots.dtype)).sum(-1), dim=-1)
    return (w.unsqueeze(-1) * slots).sum(2)


def masked_cross_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, allowed: torch.Tensor,
                           scale: float) -> torch.Tensor:
    """q [B,T,D] vs few keys k,v [B,K,D]; rows with no allowed key return exactly zero."""
    s = torch.bmm(q, k.transpose(1, 2)) * float(scale)
    any_key = allowed.any(-1, keepdim=True)
    w = torch.softmax(s.masked_fill(~(allowed | ~any_key), float("-inf")), dim=-1)
    return torch.bmm(w, v) * any_key.to(q.dtype)
