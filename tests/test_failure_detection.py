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
