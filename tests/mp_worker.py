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


def gather_gemm_case(out, dev, world, rank):
    """A row-sharded weight: every rank holds valid data only in the 64-row blocks it owns.  The gathering linear
    layer must produce x @ W^T from the owners' rows and leave a complete local copy behind."""
    import torch.distributed as dist
    from loomformer_paraplex_b200.ops import kernels
    from loomformer_paraplex_b200.parallel.fsdp import row_block_owner
    from loomformer_paraplex_b200.parallel.symm import SymmetricBuffers
    res = {}
    symm = SymmetricBuffers()
    K = kernels.CudaKernels()
    for name, (n_out, k_in, m) in {"qkv": (1152, 768, 512), "wide": (3072, 768, 300), "ragged": (200, 136, 130)}.items():
        g = torch.Generator(device="cpu").manual_seed(7)
        w_true = (torch.randn(n_out, k_in, generator=g) * 0.05).to(torch.bfloat16).to(dev)
        x = torch.randn(m, k_in, generator=g).to(torch.bfloat16).to(dev)
        buf = symm.alloc(f"w_{name}", n_out * k_in, torch.bfloat16, dev).view(n_out, k_in)
        _, owners = row_block_owner(n_out, world)
        buf.fill_(float("nan"))
        for b, o in enumerate(owners):
            if o == rank:
                buf[b * 64:(b + 1) * 64] = w_true[b * 64:(b + 1) * 64]
        torch.cuda.synchronize(); dist.barrier()
        y = K.linear(x, buf, gather=(symm.peer_ptrs(f"w_{name}"), rank))
        torch.cuda.synchronize(); dist.barrier()
        kernels.check_status(dev)
        ref = x.float() @ w_true.float().t()
        res[name] = {"out_err": float((y.float() - ref).abs().max() / ref.abs().max()),
                     "copy_equal": bool(torch.equal(buf, w_true)), "finite": bool(torch.isfinite(y.float()).all())}
    ok = torch.tensor([float(all(v["copy_equal"] and v["finite"] and v["out_err"] < 2e-2 for v in res.values()))], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if rank == 0:
        torch.save({"cases": res, "all_ranks_ok": bool(ok.item() > 0.5)}, out)
    pdist.shutdown()


def main():
    mode, out, device_kind = sys.argv[1], sys.argv[2], sys.argv[3]
    dev, world, rank = pdist.init(device_kind)
    torch.manual_seed(0)
    if mode == "gather":
        return gather_gemm_case(out, dev, world, rank)
    cfg = Config(**CFG)
    model = Model(cfg).to(dev)
    eng = TrainEngine(cfg, model, dev, optimizer="adamw", grad_sync=mode)
    src = SyntheticTokens(cfg.vocab, 2, cfg.seq_len, seed=3, rank=rank, pool=4, pin=False)
    losses = [float(eng.step(src.next())) for _ in range(4)]
    if dev.type == "cuda":
        from loomformer_paraplex_b200.ops import kernels
        kernels.check_status(dev)
    eng.complete_master()                       # sharded mode: owners' values -> every rank (no-op otherwise)
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
