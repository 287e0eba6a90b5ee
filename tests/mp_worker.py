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


def tensor_parallel_case(out, dev, world, rank):
    """Column-parallel up projection (all-gather inside the GEMM) and row-parallel down projection (reduce-scatter in
    the epilogue) of an MLP against the single-device result; also times both fused GEMMs (max over ranks)."""
    import torch.distributed as dist
    from loomformer_paraplex_b200.ops import kernels
    from loomformer_paraplex_b200.parallel.tp import TensorParallel
    tp = TensorParallel(device=dev)
    M, K, H = 2048, 768, 3072
    g = torch.Generator(device="cpu").manual_seed(11)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(dev)
    w_up = (torch.randn(H, K, generator=g) * 0.03).to(torch.bfloat16).to(dev)
    w_dn = (torch.randn(K, H, generator=g) * 0.03).to(torch.bfloat16).to(dev)
    per, hl = M // world, H // world
    x_rows = x[rank * per:(rank + 1) * per].contiguous()
    w_up_l = w_up[rank * hl:(rank + 1) * hl].contiguous()
    w_dn_l = w_dn[:, rank * hl:(rank + 1) * hl].contiguous()
    y_l = tp.column_parallel("x", x_rows, w_up_l, M)
    o_l = torch.tanh(y_l.float()).to(torch.bfloat16)
    z = tp.row_parallel("z", o_l, w_dn_l)
    torch.cuda.synchronize(); dist.barrier()
    kernels.check_status(dev)
    y_ref = x.float() @ w_up.float().t()
    o_ref = torch.tanh(y_ref[:, rank * hl:(rank + 1) * hl].to(torch.bfloat16).float()).to(torch.bfloat16)
    up_err = float((y_l.float() - y_ref[:, rank * hl:(rank + 1) * hl]).abs().max() / y_ref.abs().max())
    o_full = torch.tanh(y_ref.to(torch.bfloat16).float()).to(torch.bfloat16).float()
    z_ref = (o_full @ w_dn.float().t())[rank * per:(rank + 1) * per]
    dn_err = float((z - z_ref).abs().max() / z_ref.abs().max())
    # timing: device events around each fused op (barriers included), max over ranks
    def timed(fn, iters=20):
        for _ in range(3):
            fn()
        torch.cuda.synchronize(); dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record(); torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)
    t_up = timed(lambda: tp.column_parallel("x", x_rows, w_up_l, M))
    t_dn = timed(lambda: tp.row_parallel("z", o_l, w_dn_l))
    ok = torch.tensor([float(up_err < 2e-2 and dn_err < 2e-2)], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if rank == 0:
        flops = 2.0 * M * K * hl
        torch.save({"up_err": up_err, "dn_err": dn_err, "all_ranks_ok": bool(ok.item() > 0.5), "ms_up": t_up, "ms_down": t_dn,
                    "flops_per_rank": flops, "nvlink_bytes_up": (world - 1) * per * K * 2,
                    "nvlink_bytes_down": (world - 1) * per * K * 4, "world": world}, out)
    pdist.shutdown()


def control_case(out, dev, world, rank):
    """Only rank 0 sees the run-point key / Ctrl-C / the wall clock; every rank must act on rank 0's value at the same
    step, and flags raised on other ranks must not leak into the decision."""
    import torch.distributed as dist
    ctl = pdist.StepControl(dev)
    seen = []
    for it in range(8):
        if rank == 0:
            local = (ctl.RUNPOINT if it == 3 else 0) | (ctl.STOP if it == 6 else 0)
        else:
            local = ctl.INTERRUPT if it == 2 else 0          # must be ignored: only rank 0 decides
        seen.append(ctl.agree(local))
    fallback = pdist.StepControl(dev, use_store=False)
    seen.append(fallback.agree(ctl.RUNPOINT if rank == 0 else ctl.INTERRUPT))
    t = torch.tensor(seen, dtype=torch.long)
    lst = [torch.zeros_like(t) for _ in range(world)]
    dist.all_gather(lst, t)
    if rank == 0:
        torch.save({"per_rank": [x.tolist() for x in lst]}, out)
    pdist.shutdown()


def main():
    mode, out, device_kind = sys.argv[1], sys.argv[2], sys.argv[3]
    dev, world, rank = pdist.init(device_kind)
    torch.manual_seed(0)
    if mode == "control":
        return control_case(out, dev, world, rank)
    if mode == "gather":
        return gather_gemm_case(out, dev, world, rank)
    if mode == "tp":
        return tensor_parallel_case(out, dev, world, rank)
    cfg = Config(**CFG)
    model = Model(cfg).to(dev)
    optimizer = "adamw"
    if mode.endswith("+atom"):
        mode, optimizer = mode.split("+")[0], "atom"
    eng = TrainEngine(cfg, model, dev, optimizer=optimizer, grad_sync=mode)
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
