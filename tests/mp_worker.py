"""Multi-process worker used by the multi-GPU / multi-rank tests (launched through torch.distributed.run)."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from loomformer_paraplex_b200.config import Config
from loomformer_paraplex_b200.data.synthetic import SyntheticTokens
from loomformer_paraplex_b200.models.loomformer import Model
from loomformer_paraplex_b200.parallel import dist as pdist
from loomformer_paraplex_b200.train.engine import TrainEngine

CFG = dict(vocab=512, seq_len=128, model_dim=128, n_q_heads=4, head_dim=32, gqa_group_size=2, n_kv_heads=None,
           hidden=None, hidden_mult=4.0, layers=2, activation="pvpowlu", phase_grad_mode="secant",
           tied_embeddings=False, tria_carry_enabled=True, tria_temporal_auto=False, tria_temporal_window=64,
           tria_carrier_alpha=0.05, amp_dtype="bf16", lr=1e-3, warmup_steps=2, steps=20, grad_clip=1.0)


def main():
    mode, out, device_kind = sys.argv[1], sys.argv[2], sys.argv[3]
    dev, world, rank = pdist.init(device_kind)
    torch.manual_seed(0)
    cfg = Config(**CFG)
    model = Model(cfg).to(dev)
    eng = TrainEngine(cfg, model, dev, optimizer="adamw", grad_sync=mode)
    src = SyntheticTokens(cfg.vocab, 2, cfg.seq_len, seed=3, rank=rank, pool=4, pin=False)
    losses = [float(eng.step(src.next())) for _ in range(4)]
    if dev.type == "cuda":
        from loomformer_paraplex_b200.ops import kernels
        kernels.check_status(dev)
    # every rank must hold identical parameters
    flat = eng.flat.params.detach().float().cpu()
    gathered = [torch.zeros_like(flat) for _ in range(world)] if rank == 0 else None
    import torch.distributed as dist
    if dev.type == "cuda":
        t = eng.flat.params.detach().clone()
        lst = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(lst, t)
        same = all(torch.equal(lst[0], x) for x in lst)
    else:
        lst = [torch.zeros_like(flat) for _ in range(world)]
        dist.all_gather(lst, flat)
        same = all(torch.equal(lst[0], x) for x in lst)
    if rank == 0:
        torch.save({"params": flat, "losses": losses, "same": same}, out)
    pdist.shutdown()


if __name__ == "__main__":
    main()
