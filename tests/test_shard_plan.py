"""Ownership maps of the sharded data-parallel mode, checked on the host for every world size the peer kernels
accept (1..8): each 256-element block of the flat buffer has exactly one owner, row-sharded weights are owned in runs
of 64 rows, compact <-> full round-trips, and the FFN weights of a model whose hidden sectors get padded stay
replicated."""
import pytest
import torch

from loomformer_paraplex_b200.config import Config
from loomformer_paraplex_b200.models.loomformer import Model
from loomformer_paraplex_b200.optim.flat import FlatParams
from loomformer_paraplex_b200.parallel.fsdp import BLOCK, ShardPlan, row_block_owner

CFG = dict(vocab=128, seq_len=32, model_dim=64, n_q_heads=4, head_dim=16, n_kv_heads=2, hidden=None, hidden_mult=8.0,
           layers=2, activation="pvpowlu", tied_embeddings=False, tria_carry_enabled=True, tria_temporal_auto=False,
           tria_temporal_window=8, tria_carrier_alpha=0.05, tria_gamma_max=0.8, tria_raw_gamma_init=0.25)


@pytest.mark.parametrize("world", [1, 2, 3, 4, 5, 8])
def test_every_block_has_one_owner(world):
    torch.manual_seed(0)
    model = Model(Config(**CFG))
    flat = FlatParams(model)
    plans = [ShardPlan(flat, model, world, r) for r in range(world)]
    owned = torch.zeros(flat.nblk, dtype=torch.int32)
    for r, sp in enumerate(plans):
        assert torch.equal(sp.owner_blk, plans[0].owner_blk)            # every rank derives the same map
        mine = sp.owner_blk.eq(r)
        assert int(mine.sum()) == sp.owned_blocks == sp.owned_index.numel()
        owned += mine.int()
        full = torch.arange(flat.total, dtype=torch.float32)
        back = sp.expand(sp.compact(full), reduce=False)
        assert torch.equal(back.view(-1, BLOCK)[mine], full.view(-1, BLOCK)[mine])
        assert float(back.view(-1, BLOCK)[~mine].abs().sum()) == 0.0
    assert torch.equal(owned, torch.ones_like(owned))
    # weights fetched on use: owned in runs of 64 rows, in rank order
    sp = plans[0]
    for seg in flat.segments:
        if id(seg.param) not in sp.gathered:
            continue
        rows, cols = seg.param.shape
        per, blocks = row_block_owner(rows, world)
        assert blocks == sorted(blocks) and max(blocks) <= world - 1 and len(blocks) == -(-rows // 64)
        per64 = 64 * cols // BLOCK
        b0 = seg.offset // BLOCK
        for rb, owner in enumerate(blocks):
            got = sp.owner_blk[b0 + rb * per64:b0 + min((rb + 1) * per64, (seg.numel + BLOCK - 1) // BLOCK)]
            assert bool(got.eq(owner).all()), (seg.name, rb)
    if world > 1:
        assert sp.gathered, "the linear weights of this shape should be fetched on use"


def test_padded_sector_model_keeps_ffn_weights_replicated():
    torch.manual_seed(0)
    model = Model(Config(**dict(CFG, hidden=4 * 171, hidden_mult=None)))     # 171 neurons per head, as in smol360
    assert model.d.hpq % 8 != 0
    flat = FlatParams(model)
    sp = ShardPlan(flat, model, 2, 0)
    names = set(sp.gathered.values())
    assert not any(n.endswith(("ffn.w1_real.weight", "ffn.gate_proj.weight", "ffn.w2.weight")) for n in names)
    assert any(n.endswith("attn.qkv_weight") for n in names)


def test_sharded_mode_with_atom_selects_the_replicated_fused_step(capsys):
    """The sharded update exists for AdamW only; asking for it with ATOM must not fail at the first optimizer step but
    select the replicated fused step when the engine is built."""
    from loomformer_paraplex_b200.train.engine import TrainEngine
    cfg = Config(**dict(CFG, batch_size=2, optimizer="atom"))
    torch.manual_seed(0)
    eng = TrainEngine(cfg, Model(cfg), torch.device("cpu"), grad_sync="fsdp")
    assert eng.grad_sync == "p2p" and eng.opt_name == "atom" and eng.sync.shard is None
    assert "replicated" in capsys.readouterr().out
    eng2 = TrainEngine(cfg, Model(cfg), torch.device("cpu"), optimizer="adamw", grad_sync="fsdp")
    assert eng2.grad_sync == "fsdp"
