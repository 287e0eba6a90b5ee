"""Failure detection without touching a GPU fault: a rank that leaves between steps is noticed on the host; a step
that overruns trips the watchdog; a device wait that can never be satisfied returns an error code (GPU test)."""
import os
import subprocess
import sys
import time

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_heartbeat_reports_a_rank_that_left(tmp_path):
    out = str(tmp_path / "hb.pt")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29641", os.path.join(ROOT, "tests", "health_worker.py"), out]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=180)
    assert os.path.exists(out), r.stdout[-2000:] + r.stderr[-2000:]
    res = torch.load(out)
    assert res["detected"] == [1] and res["after_s"] < 10.0
    assert res["collective_error"] is not None          # the collective failed fast instead of hanging


def test_step_watchdog_fires_and_disarms():
    from loomformer_paraplex_b200.parallel.health import StepWatchdog
    hits = []
    wd = StepWatchdog(0.2, on_timeout=lambda limit: hits.append(limit))
    with wd.step():
        time.sleep(0.05)
    assert not wd.fired and not hits
    with wd.step():
        time.sleep(0.5)
    assert wd.fired and hits == [0.2]


@pytest.mark.gpu
def test_bounded_device_wait_reports_instead_of_hanging():
    """A cross-rank barrier whose peer never arrives (its flag word is never written) gives up after its cycle budget,
    records the caller's code in the status word and returns; the context stays usable."""
    from loomformer_paraplex_b200.ops import kernels, native
    dev = torch.device("cuda")
    mine = torch.zeros(64, dtype=torch.int32, device=dev)
    absent = torch.zeros(64, dtype=torch.int32, device=dev)       # stands for a peer that never signals
    status = kernels.status_word(dev)
    status.zero_()
    t0 = time.time()
    native.ext().tp_barrier([mine.data_ptr(), absent.data_ptr()], 0, 1, status, 777)
    torch.cuda.synchronize()
    assert time.time() - t0 < 30.0
    with pytest.raises(RuntimeError, match="777"):
        kernels.check_status(dev)
    assert int(status.item()) == 0                                 # cleared by the check; later work is unaffected
    assert float((torch.ones(8, device=dev) * 2).sum()) == 16.0


def _tiny_engine():
    from loomformer_paraplex_b200.config import Config
    from loomformer_paraplex_b200.models.loomformer import Model
    from loomformer_paraplex_b200.train.engine import TrainEngine
    torch.manual_seed(0)
    cfg = Config(vocab=64, seq_len=16, model_dim=None, n_q_heads=2, head_dim=8, n_kv_heads=1, hidden=None,
                 hidden_mult=2.0, layers=2, tied_embeddings=False, tria_carry_enabled=True, tria_temporal_auto=False,
                 tria_temporal_window=8, tria_carrier_alpha=0.05, lr=1e-3, warmup_steps=1, steps=4, grad_clip=1.0,
                 amp_dtype="fp32")
    dev = torch.device("cpu")
    return TrainEngine(cfg, Model(cfg), dev, optimizer="adamw"), cfg


def test_training_loop_raises_when_a_kernel_gave_up_a_wait():
    """The status word that bounded device waits set must surface in the training loop's own guard (log cadence and
    before every checkpoint), not only in benchmarks."""
    from loomformer_paraplex_b200.ops import kernels
    eng, cfg = _tiny_engine()
    batch = torch.randint(0, cfg.vocab, (2, cfg.seq_len + 1))
    loss = eng.step(batch)
    eng.check_finite(loss)                                   # healthy step passes
    word = kernels.status_word(eng.device)
    try:
        word.fill_(401)
        with pytest.raises(RuntimeError, match="bounded wait"):
            eng.check_finite(loss)
        assert int(word.item()) == 0                         # reported once, then cleared
        word.fill_(103)
        with pytest.raises(RuntimeError, match="bounded wait"):
            eng.checkpoint_view()
    finally:
        word.zero_()
        kernels._STATUS.pop(str(eng.device), None)


def test_skipped_updates_between_log_lines_are_reported():
    """A non-finite step is skipped on the device; the next guard call must say so even if later steps were fine."""
    eng, cfg = _tiny_engine()
    batch = torch.randint(0, cfg.vocab, (2, cfg.seq_len + 1))
    before = eng.flat.params.clone()
    eng.flat.grads.fill_(float("nan"))
    eng.opt.step()                                           # skipped: parameters untouched
    assert torch.equal(before, eng.flat.params)
    loss = eng.step(batch)                                   # a healthy step afterwards
    with pytest.raises(RuntimeError, match="skipped"):
        eng.check_finite(loss)
    eng.check_finite(eng.step(batch))                        # counted once
