"""ATOM and AdamW of this repository against the reference's own optimizer classes on identical gradients, and the
optimizer entry of a checkpoint exchanged in both directions.

The reference's CPU path of ATOM (``atom/atom.py:912-974``) is the oracle.  It never updates the per-block accept
rate ``pnode_blk`` (its CUDA kernel does, ``atom.py:238-242``), so trust values agree only inside the bootstrap window
(the first 20 steps, where trust is clamped from below); moments and the block gradient means agree at every step."""
import importlib.util
import os
import sys

import pytest
import torch

from loomformer_paraplex_b200.optim.flat import FlatOptimizer, FlatParams

REF_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")


def _ref_atom():
    path = os.path.join(REF_DIR, "atom", "atom.py")
    if not os.path.isfile(path):
        pytest.skip("reference copy not present under baseline/_ref")
    if "ref_atom" in sys.modules:
        return sys.modules["ref_atom"]
    sys.dont_write_bytecode = True
    spec = importlib.util.spec_from_file_location("ref_atom", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["ref_atom"] = mod
    spec.loader.exec_module(mod)
    return mod


class _Net(torch.nn.Module):
    def __init__(self):
        super().__init__()
        torch.manual_seed(0)
        self.a = torch.nn.Parameter(torch.randn(37, 29))          # 1073 elements: 4 full blocks + a ragged one
        self.b = torch.nn.Parameter(torch.randn(256))             # exactly one block
        self.c = torch.nn.Parameter(torch.randn(5))               # a lone partial block
        self.nodecay = torch.nn.Parameter(torch.randn(3, 100))


def _pair(kind):
    ours, theirs = _Net(), _Net()
    flat = FlatParams(ours, want_bf16_shadow=False)
    opt = FlatOptimizer(flat, kind, lr=3e-3, weight_decay=0.05, grad_clip=0.0, no_decay={"nodecay"})
    groups = [{"params": [theirs.a, theirs.b, theirs.c], "weight_decay": 0.05, "lr_mult": 1.0},
              {"params": [theirs.nodecay], "weight_decay": 0.0, "lr_mult": 1.0}]
    if kind == "atom":
        ref = _ref_atom().ATOM(groups, lr=3e-3, weight_decay=0.05)
    else:
        ref = torch.optim.AdamW(groups, lr=3e-3, weight_decay=0.05)
    return ours, flat, opt, theirs, ref


def _feed(ours, flat, theirs, step):
    g = torch.Generator().manual_seed(100 + step)
    for (n, p), q in zip(ours.named_parameters(), theirs.parameters()):
        grad = torch.randn(p.shape, generator=g) * (0.5 + 0.1 * (step % 7))
        if step % 5 == 0:
            grad = grad + 0.3                   # a drifting mean exercises the block-mean predictor
        q.grad = grad.clone()
        seg = next(s for s in flat.segments if s.name == n)
        flat.grads[seg.offset:seg.offset + seg.numel] = grad.reshape(-1)


def _seg(flat, name):
    return next(s for s in flat.segments if s.name == name)


def test_atom_matches_reference_class_through_bootstrap_and_beyond():
    ours, flat, opt, theirs, ref = _pair("atom")
    for step in range(1, 51):
        _feed(ours, flat, theirs, step)
        opt.step()
        ref.step()
        for (n, p), q in zip(ours.named_parameters(), theirs.parameters()):
            st = ref.state[q]
            s = _seg(flat, n)
            sl = slice(s.offset, s.offset + s.numel)
            bs = slice(s.offset // 256, (s.offset + s.padded) // 256)
            assert torch.allclose(opt.m[sl].view_as(q), st["m"], rtol=1e-5, atol=1e-7), (step, n)
            assert torch.allclose(opt.v[sl].view_as(q), st["v"], rtol=1e-5, atol=1e-7), (step, n)
            assert torch.allclose(opt.gprev_blk[bs], st["gprev_blk"].float(), rtol=1e-4, atol=1e-6), (step, n)
            if step <= 20:                       # bootstrap window: trust is clamped identically on both sides
                assert torch.allclose(p.detach(), q.detach(), rtol=1e-5, atol=1e-6), (step, n)
    stats = opt.atom_refresh_stats()
    assert 0.0 <= stats["commit_frac"] <= 1.0 and stats["params_tensors"] == 4.0


def test_adamw_matches_torch_adamw():
    ours, flat, opt, theirs, ref = _pair("adamw")
    for step in range(1, 31):
        _feed(ours, flat, theirs, step)
        opt.step()
        ref.step()
    for p, q in zip(ours.parameters(), theirs.parameters()):
        assert torch.allclose(p.detach(), q.detach(), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("kind", ["adamw", "atom"])
def test_optimizer_state_dict_round_trips_through_the_reference_classes(kind, tmp_path):
    """A state dict written here loads into the reference's optimizer (what its ``load_optimizer_checkpoint`` does,
    ``loomformer.py:4481-4523``) and continues identically for the steps where both sides share one formula; a state
    dict written by the reference loads here."""
    ours, flat, opt, theirs, ref = _pair(kind)
    for step in range(1, 6):
        _feed(ours, flat, theirs, step)
        opt.step()
        ref.step()
    # ours -> reference class
    path = tmp_path / "opt.pt"
    torch.save({"optimizer": opt.state_dict(), "optimizer_name": kind}, path)
    blob = torch.load(path, weights_only=True)
    fresh = _Net()
    with torch.no_grad():
        for q, p in zip(fresh.parameters(), ours.parameters()):
            q.copy_(p)
    groups = [{"params": [fresh.a, fresh.b, fresh.c], "weight_decay": 0.05, "lr_mult": 1.0},
              {"params": [fresh.nodecay], "weight_decay": 0.0, "lr_mult": 1.0}]
    ref2 = _ref_atom().ATOM(groups, lr=3e-3, weight_decay=0.05) if kind == "atom" else \
        torch.optim.AdamW(groups, lr=3e-3, weight_decay=0.05)
    ref2.load_state_dict(blob["optimizer"])
    for step in range(6, 11):
        _feed(ours, flat, fresh, step)
        opt.step()
        ref2.step()
    for p, q in zip(ours.parameters(), fresh.parameters()):
        assert torch.allclose(p.detach(), q.detach(), rtol=1e-5, atol=1e-6)
    # reference -> ours
    ours3 = _Net()
    with torch.no_grad():
        for q, p in zip(ours3.parameters(), theirs.parameters()):
            q.copy_(p)
    flat3 = FlatParams(ours3, want_bf16_shadow=False)
    opt3 = FlatOptimizer(flat3, kind, lr=3e-3, weight_decay=0.05, grad_clip=0.0, no_decay={"nodecay"})
    sd = ref.state_dict()
    torch.save({"optimizer": sd}, path)
    opt3.load_state_dict(torch.load(path, weights_only=True)["optimizer"])
    assert opt3.step_count == 5
    for step in range(6, 11):
        _feed(ours3, flat3, theirs, step)
        opt3.step()
        ref.step()
    for p, q in zip(ours3.parameters(), theirs.parameters()):
        assert torch.allclose(p.detach(), q.detach(), rtol=1e-5, atol=1e-6)
