"""Worker (gloo, CPU): rank 1 stops between steps (raises, reports the error and exits); the other ranks learn of it from
the heartbeat monitor on the host before their next step and leave cleanly. Exit code 0 = expected behaviour."""
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mindformers_b200.fault import HeartbeatMonitor, RankFailure  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    mode = sys.argv[1] if len(sys.argv) > 1 else "error"
    store = dist.TCPStore(os.environ["MASTER_ADDR"], int(os.environ["MASTER_PORT"]) + 1, world, rank == 0, wait_for_workers=True)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    mon = HeartbeatMonitor(store, rank, world, interval=0.1, timeout=1.0).start()
    x = torch.ones(4)
    noticed = False
    try:
        for step in range(200):
            mon.check()                          # host-side check before launching the step's collective
            if rank == 1 and step == 3:
                if mode == "error":
                    mon.report_error("synthetic failure between steps")
                mon.stop()                       # "silent" mode: the rank just stops beating
                dist.destroy_process_group()
                return 0
            if step < 3:
                dist.all_reduce(x)               # all ranks still alive
            time.sleep(0.05)
            mon.beat()
    except RankFailure as e:
        noticed = 1 in e.ranks
    mon.stop()
    if rank == 0:
        time.sleep(0.5)                          # keep the store alive until the others have read it
    return 0 if noticed else 1


if __name__ == "__main__":
    sys.exit(main())
