"""Worker for the failure-detection test: two gloo ranks; rank 1 leaves between steps; rank 0 must notice on the host
(heartbeat) before its next collective, and a collective attempted anyway must end with an error, not hang."""
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from loomformer_paraplex_b200.parallel import dist as pdist
from loomformer_paraplex_b200.parallel.health import Heartbeat, PeerLost


def main():
    out = sys.argv[1]
    dev, world, rank = pdist.init("cpu", timeout_s=8.0)
    import torch.distributed as dist
    hb = Heartbeat(interval=0.2, max_silence=2.0)
    x = torch.ones(4)
    for step in range(3):                      # healthy steps
        hb.check()
        dist.all_reduce(x)
    if rank == 1:
        hb.stop()
        os._exit(0)                            # leaves between steps, nothing in flight
    t0 = time.monotonic()
    detected, after = None, None
    while time.monotonic() - t0 < 15.0:
        try:
            hb.check()
        except PeerLost as e:
            detected, after = e.ranks, time.monotonic() - t0
            break
        time.sleep(0.2)
    collective_error = None
    try:                                       # what would have happened without the check: a bounded failure
        dist.all_reduce(x)
    except Exception as e:                     # noqa: BLE001 - any backend error type counts
        collective_error = type(e).__name__
    torch.save({"detected": detected, "after_s": after, "collective_error": collective_error}, out)
    os._exit(0)


if __name__ == "__main__":
    main()
