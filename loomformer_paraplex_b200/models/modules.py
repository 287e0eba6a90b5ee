"""Parameter-holding building blocks of LoomFormer.

Attribute names reproduce the reference ``state_dict`` layout exactly (``emb.weight``,
``blocks.{i}.attn.qkv_weight``, ``blocks.{i}.ffn.w1_imag`` ...; reference
``loomformer.py:2666-2718, 3215-3229, 3367-3389`` and ``tria.py:1257-1603``) so checkpoints are
interchangeable.  The modules only own parameters, initialisation and the small pieces of math
that are not performance relevant; the model's execution plans (``models/loomformer.py``) decide
which operator implementation consumes them.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config import Dims, imag_live_columns
from ..ops import reference as R


def _normal(t: torch.Tensor, std: float) -> None:
    nn.init.normal_(t, mean=0.0, std=std)


class Attention(nn.Module):
    """Causal grouped-query attention parameters: packed ``qkv_weight`` and output ``o``."""

    def __init__(self, d: Dims) -> None:
        super().__init__()
        self.d = d
        self.qkv_weight = nn.Parameter(torch.empty(d.n + 2 * d.kv_dim, d.n))
        self.o = nn.Linear(d.n, d.n, bias=False)
        n, kv = d.n, d.kv_dim
        with torch.no_grad():
            _normal(self.qkv_weight[:n + kv], d.fanin_std(n))
            _normal(self.qkv_weight[n + kv:], d.residual_std(n))
            _normal(self.o.weight, d.residual_std(n))


class DepthAttn(nn.Module):
    """Softmax read over earlier-depth states: shared K/V projection, one query per sublayer."""

    def __init__(self, d: Dims) -> None:
        super().__init__()
        self.d = d
        n = d.n
        self.kv_weight = nn.Parameter(torch.empty(2 * n, n))
        if d.depth_readout_per_sublayer:
            self.w_o_weight = nn.Parameter(torch.empty(d.n_sub, n, n))
            self.w_o = None
        else:
            self.register_parameter("w_o_weight", None)
            self.w_o = nn.Linear(n, n, bias=False)
        self.q_params = nn.Parameter(torch.empty(d.n_sub, d.qh, d.hd))
        with torch.no_grad():
            _normal(self.kv_weight[:n], d.fanin_std(n))
            _normal(self.kv_weight[n:], d.residual_std(n))
            _normal(self.w_o_weight if self.w_o is None else self.w_o.weight, d.residual_std(n))
            _normal(self.q_params, d.fanin_std(d.hd))

    def query(self, sub: int) -> torch.Tensor:
        q = self.q_params[sub]
        return R.fixed_rms(q, self.d.fanin_std(self.d.hd)) if self.d.depth_qkv_rms else q

    def readout_weight(self, sub: int) -> torch.Tensor:
        return self.w_o_weight[sub] if self.w_o is None else self.w_o.weight

    def project(self, h: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        d = self.d
        B, T, _ = h.shape
        k, v = F.linear(h, self.kv_weight).split((d.n, d.n), dim=-1)
        k, v = k.view(B, T, d.qh, d.hd), v.view(B, T, d.qh, d.hd)
        if d.depth_qkv_rms:
            from ..config import FANIN_GAIN
            k, v = R.fixed_rms(k, FANIN_GAIN), R.fixed_rms(v, FANIN_GAIN * d.deepnorm_beta)
        return k, v


class GateSelector(nn.Module):
    def __init__(self) -> None:
        super().__init__()
        self.logits = nn.Parameter(torch.zeros(9))

    def weights(self) -> torch.Tensor:
        return torch.softmax(self.logits, dim=0)

    def forward(self, carry: torch.Tensor) -> torch.Tensor:
        return (carry.reshape(*carry.shape[:3], 9) * self.weights()).sum(-1)


class IdentityAnchoredGate(nn.Module):
    """``wx * (1 + alpha * p) + bias`` with ``alpha = alpha_max * tanh(raw_alpha)`` (zero at init)."""

    def __init__(self, alpha_max: float = 0.25) -> None:
        super().__init__()
        self.alpha_max = float(alpha_max)
        self.raw_alpha = nn.Parameter(torch.zeros(()))

    def alpha(self) -> torch.Tensor:
        return self.alpha_max * torch.tanh(self.raw_alpha)

    def forward(self, wx: torch.Tensor, bias: torch.Tensor, p: Optional[torch.Tensor]) -> torch.Tensor:
        if p is None:
            return wx + bias
        return wx * (1.0 + self.alpha() * p) + bias


class ParaplexFFN(nn.Module):
    """Real projection + sector-masked imaginary projection -> bounded phase -> PvPowLU -> w2.

    ``w1_imag`` stores only the live fan-in of every neuron, ``[H, IMAG_IN]`` in the column
    order given by :func:`config.imag_live_columns`.
    """

    def __init__(self, d: Dims, ablation: bool = False) -> None:
        super().__init__()
        self.d, self.ablation = d, bool(ablation)
        n, h = d.n, d.hidden
        self.w1_real = nn.Linear(n, h)
        self.w1_imag = nn.Parameter(torch.empty(h, d.imag_in))
        self.w1_imag_trace = nn.Parameter(torch.zeros(h))
        self.w1_imag_bias = nn.Parameter(torch.zeros(h))
        self.w2 = nn.Linear(h, n)
        self.register_buffer("beta_anchor", torch.tensor(1.0), persistent=True)
        self.beta_anchor_decay = 0.99
        if d.tria:
            self.gate_selector: Optional[GateSelector] = GateSelector()
            self.identity_gate: Optional[IdentityAnchoredGate] = IdentityAnchoredGate()
        else:
            self.gate_selector = None
            self.identity_gate = None
        self.gate_proj = nn.Linear(n, h) if d.gate_proj else None
        with torch.no_grad():
            _normal(self.w1_real.weight, d.fanin_std(n)); self.w1_real.bias.zero_()
            _normal(self.w1_imag, d.fanin_std(d.imag_in))
            _normal(self.w2.weight, d.residual_std(h)); self.w2.bias.zero_()
            if self.gate_proj is not None:
                _normal(self.gate_proj.weight, d.fanin_std(n)); self.gate_proj.bias.zero_()

    # -- imaginary projection, reference form ------------------------------------------
    def beta_linear(self, u, q, kctx, c, dsel) -> torch.Tensor:
        """``W_imag . [Q;Kctx;C;u;D]`` evaluated per head group without a dense scatter."""
        d = self.d
        B, T, _ = u.shape
        w = self.w1_imag.view(d.qh, d.hpq, d.imag_in)
        if d.open_sectors:
            shared = torch.cat((kctx.reshape(B, T, d.n), c.reshape(B, T, d.n), u, dsel.reshape(B, T, d.n)), -1)
            outs = []
            for g in range(d.qh):
                a = torch.cat((q[:, :, g], shared), dim=-1)
                outs.append(F.linear(a, w[g].to(a.dtype)))
            return torch.cat(outs, dim=-1)
        a = torch.cat((q, kctx, c, u.unsqueeze(2).expand(B, T, d.qh, d.n), dsel), dim=-1)   # [B,T,QH,IMAG_IN]
        out = torch.einsum("btgk,ghk->btgh", a, w.to(a.dtype))
        return out.reshape(B, T, d.hidden)

    def dense_imag_weight(self) -> torch.Tensor:
        """Scatter the compact rows into the virtual dense ``[H, 5N]`` matrix (analysis tools)."""
        d = self.d
        dense = self.w1_imag.new_zeros(d.hidden, 5 * d.n)
        for g in range(d.qh):
            cols = torch.tensor(imag_live_columns(d, g), device=dense.device)
            dense[g * d.hpq:(g + 1) * d.hpq, cols] = self.w1_imag[g * d.hpq:(g + 1) * d.hpq]
        return dense

    def update_anchor(self, beta: torch.Tensor) -> None:
        with torch.no_grad():
            self.beta_anchor.mul_(self.beta_anchor_decay).add_(
                R.phase_radius(beta).to(self.beta_anchor.dtype), alpha=1.0 - self.beta_anchor_decay)


class SharedTriaReader(nn.Module):
    def __init__(self, k: int = 32) -> None:
        super().__init__()
        self.k = k
        self.proj = nn.Linear(9, k)
        self.key_proj = nn.Linear(9, k, bias=False)
        with torch.no_grad():
            self.key_proj.weight.normal_(mean=0.0, std=1.5)

    def forward(self, carry: torch.Tensor) -> torch.Tensor:
        return self.proj(carry.reshape(*carry.shape[:3], 9).to(self.proj.weight.dtype))

    def make_score_w(self, query: torch.Tensor, logit_scale: torch.Tensor) -> torch.Tensor:
        raw = torch.mv(self.key_proj.weight.t(), query)
        return F.normalize(raw, dim=0, eps=1e-6) * logit_scale


class AttentionPool(nn.Module):
    def __init__(self, k: int, init_logit_scale: float = 1.0) -> None:
        super().__init__()
        self.query = nn.Parameter(torch.zeros(k))
        self.logit_scale_raw = nn.Parameter(torch.tensor(math.log(math.expm1(float(init_logit_scale)))))

    def logit_scale(self) -> torch.Tensor:
        return F.softplus(self.logit_scale_raw)


class TriaAggregator(nn.Module):
    """Pool the per-neuron temporal carriers of each boundary key into one ``N``-vector."""

    def __init__(self, reader: SharedTriaReader, d_model: int) -> None:
        super().__init__()
        self.reader = reader
        self.pool = AttentionPool(reader.k)
        self.up = nn.Linear(reader.k, d_model)

    def score_w(self) -> torch.Tensor:
        return self.reader.make_score_w(self.pool.query, self.pool.logit_scale())

    def forward(self, carry: torch.Tensor, pool_fn=None) -> torch.Tensor:
        w = self.score_w()
        pooled = (pool_fn or R.slot_pool)(carry, w.to(carry.dtype))
        z = self.reader.proj(pooled.to(self.reader.proj.weight.dtype))
        return self.up(z.to(self.up.weight.dtype))


class TriaFinalCrossAttention(nn.Module):
    """Sparse cross-attention from every token to the fired boundary keys, added with a bounded gain."""

    def __init__(self, d_model: int, gamma_max: float = 0.25, raw_gamma_init: float = 0.0) -> None:
        super().__init__()
        self.w_qk = nn.Linear(d_model, d_model, bias=False)
        self.w_v = nn.Linear(d_model, d_model, bias=False)
        self.gamma_max = float(gamma_max)
        self.raw_gamma = nn.Parameter(torch.tensor(float(raw_gamma_init)))
        self.scale = d_model ** -0.5

    def gamma(self) -> torch.Tensor:
        return self.gamma_max * torch.tanh(self.raw_gamma)

    def forward(self, a: torch.Tensor, b: torch.Tensor, allowed: torch.Tensor, attend_fn=None) -> torch.Tensor:
        """a: keys [B,K,N]; b: stream [B,T,N]; allowed: bool [B,T,K]."""
        q, k, v = self.w_qk(b), self.w_qk(a.to(b.dtype)), self.w_v(a.to(b.dtype))
        out = (attend_fn or R.masked_cross_attention)(q, k, v, allowed, self.scale)
        return b + self.gamma().to(out.dtype) * out


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6) -> None:
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return R.rms_norm(x, self.weight, self.eps)


class Block(nn.Module):
    def __init__(self, d: Dims, ablation: bool = False) -> None:
        super().__init__()
        self.ln_attn = nn.LayerNorm(d.n)
        self.attn = Attention(d)
        self.ln_ffn = nn.LayerNorm(d.n)
        self.ffn = ParaplexFFN(d, ablation=ablation)
