"""Tracing and profiling helpers.

* ``span(name)``: an NVTX range when ``LOOM_NVTX=1`` (per chunk / layer / phase in the fused plan and the engine), a
  no-op otherwise, so timeline tools show the step's structure without costing anything in normal runs.
* ``kernel_breakdown(...)`` / ``python -m loomformer_paraplex_b200.utils.tracing``: device time per kernel and per
  kernel family over one training step of the benchmark model (torch profiler, eager launches so kernels keep their
  names).  The reference has three ``record_function`` labels and a wall-clock data-wait percentage
  (reference ``loomformer.py:3095,3282,3355,5075-5077``)."""
from __future__ import annotations

import contextlib
import os
import sys
from typing import Dict, List, Tuple

import torch

_NVTX = os.environ.get("LOOM_NVTX", "0") == "1"

FAMILIES = (("GEMMs (gemm_kernel / gemm_pair_kernel: forward, data gradient, grouped weight gradient)",
             ("gemm_kernel", "gemm_pair_kernel")),
            ("fused Paraplex core + Tria step (ffn_core_*)", ("ffn_core",)),
            ("attention (attn_fwd, attn_bwd)", ("attn_fwd", "attn_bwd")),
            ("depth attention (dread_*)", ("dread",)),
            ("add + LayerNorm", ("add_ln", "cap_bwd")),
            ("temporal endpoint + PolARM", ("temporal_",)),
            ("RoPE / cache write", ("rope_",)),
            ("readout (slot pool, sparse cross attention)", ("slot_pool", "cross_attn")),
            ("optimizer / gradient norm", ("adamw_flat", "atom_flat", "sumsq", "norm_finalize", "rs_reduce", "update_allgather")),
            ("cross-entropy", ("::ce_kernel",)))


@contextlib.contextmanager
def span(name: str):
    if _NVTX and torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


def kernel_breakdown(steps_warm: int = 3, micro_batch: int = 16, seq_len: int = 2048) -> Tuple[List[Tuple[float, int, str]], Dict[str, Tuple[float, int]]]:
    """One profiled training step of the benchmark model -> (per-kernel rows (ms, launches, name), per-family totals)."""
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    if root not in sys.path:
        sys.path.insert(0, root)
    import bench
    from torch.profiler import ProfilerActivity, profile
    from ..config import Config
    from ..data.synthetic import SyntheticTokens
    from ..models.loomformer import Model
    from ..train.engine import TrainEngine
    dev = torch.device("cuda", torch.cuda.current_device())
    cfg = Config(**dict(bench.MODEL_KW, batch_size=micro_batch, seq_len=seq_len))
    torch.manual_seed(cfg.seed)
    model = Model(cfg).to(dev)
    eng = TrainEngine(cfg, model, dev, optimizer="adamw", cuda_graph=False)       # eager: kernels keep their names
    src = SyntheticTokens(cfg.vocab, micro_batch, seq_len, pool=2)
    res = [b.to(dev) for b in src.batches]
    for i in range(steps_warm):
        eng.step(res[i % 2])
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        eng.step(res[0])
        torch.cuda.synchronize()
    rows = sorted(((r.device_time_total / 1000.0, r.count, r.key) for r in prof.key_averages() if r.device_time_total > 0),
                  reverse=True)
    fam: Dict[str, Tuple[float, int]] = {}
    rest_ms, rest_n = 0.0, 0
    for ms, n, name in rows:
        for title, keys in FAMILIES:
            if any(k in name for k in keys):
                a, b = fam.get(title, (0.0, 0))
                fam[title] = (a + ms, b + n)
                break
        else:
            rest_ms, rest_n = rest_ms + ms, rest_n + n
    fam["everything else (PyTorch copies / adds / fills, small kernels)"] = (rest_ms, rest_n)
    return rows, fam


def main(argv=None) -> None:
    import argparse
    ap = argparse.ArgumentParser(description="device time per kernel family over one training step of the benchmark model")
    ap.add_argument("--micro-batch", type=int, default=16)
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--top", type=int, default=30)
    a = ap.parse_args(argv)
    rows, fam = kernel_breakdown(3, a.micro_batch, a.seq_len)
    total = sum(ms for ms, _ in fam.values())
    print(f"{'family':78s} {'launches':>9s} {'ms':>9s} {'share':>6s}")
    for title, (ms, n) in sorted(fam.items(), key=lambda kv: -kv[1][0]):
        print(f"{title:78s} {n:9d} {ms:9.2f} {ms / total:6.2f}")
    print(f"{'total device time':78s} {'':9s} {total:9.2f}")
    print()
    for ms, n, name in rows[:a.top]:
        print(f"{ms:10.2f} ms  x{n:6d}  {name[:120]}")


if __name__ == "__main__":
    main()
