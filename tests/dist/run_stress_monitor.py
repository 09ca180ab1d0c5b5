"""Worker (torchrun, gloo, CPU): the stress-test monitor agrees on healthy ranks and names the rank whose result was
perturbed on the host (a stand-in for a GPU that computes wrong numbers; no device is faulted)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mindformers_b200.core.callback import RunContext, StressTestModelMonitor  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank = dist.get_rank()
    mon = StressTestModelMonitor(interval_steps=2, stress_steps=3, hidden_size=64)
    mon.on_step_end(RunContext(global_step=1))
    assert not mon.reports                                   # not a multiple of the interval
    mon.on_step_end(RunContext(global_step=2))
    assert mon.reports[-1]["ok"] and mon.reports[-1]["max_spread"] == 0.0
    healthy = mon.run_stress_job()
    if rank == 1:
        healthy = healthy.clone()
        healthy[1] += 1e-3                                   # one loss value off on this rank only
    report = mon.compare(healthy)
    assert not report["ok"] and report["suspects"] == [1], report
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
