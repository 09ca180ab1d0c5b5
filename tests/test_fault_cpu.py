"""Failure detection and restart supervision, host side only (gloo ranks on CPU; no GPU is faulted or hung)."""
import os
import socket
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("mode", ["error", "silent"])
def test_peer_failure_is_noticed_between_steps(mode):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=3", "--master-addr", "127.0.0.1",
           "--master-port", str(_port()), os.path.join(ROOT, "tests", "dist", "run_heartbeat.py"), mode]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=120, env=dict(os.environ, OMP_NUM_THREADS="1"))
    assert r.returncode == 0, r.stderr[-2000:]


def test_run_with_restarts_resumes_and_gives_up():
    from mindformers_b200.fault import RankFailure, run_with_restarts
    calls = []

    def train(attempt, resume):
        calls.append((attempt, resume))
        if attempt < 2:
            raise RankFailure([1], "no heartbeat")
        return "done"
    assert run_with_restarts(train, "/ckpt", max_restarts=3, backoff_s=0.0) == "done"
    assert calls == [(0, None), (1, "/ckpt"), (2, "/ckpt")]
    with pytest.raises(ValueError):
        run_with_restarts(lambda a, r: (_ for _ in ()).throw(ValueError("bad config")), "/ckpt", backoff_s=0.0)
    with pytest.raises(RuntimeError):
        run_with_restarts(lambda a, r: (_ for _ in ()).throw(RuntimeError("TREError spike")), "/ckpt", max_restarts=1, backoff_s=0.0)


def test_heartbeat_with_hash_store():
    import time
    import torch.distributed as dist
    from mindformers_b200.fault import HeartbeatMonitor, RankFailure
    store = dist.HashStore()
    a = HeartbeatMonitor(store, 0, 2, interval=0.05, timeout=0.3).start()
    b = HeartbeatMonitor(store, 1, 2, interval=0.05, timeout=0.3).start()
    time.sleep(0.3)
    a.check()
    b.stop()                        # rank 1 goes silent
    time.sleep(0.8)
    with pytest.raises(RankFailure):
        a.check()
    a.stop()


def test_stress_test_monitor_names_the_deviating_rank():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=3", "--master-addr", "127.0.0.1",
           "--master-port", str(_port()), os.path.join(ROOT, "tests", "dist", "run_stress_monitor.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=180, env=dict(os.environ, OMP_NUM_THREADS="1"))
    assert r.returncode == 0, r.stderr[-2000:]


def test_step_pause_holds_the_loop_until_the_request_is_cleared(tmp_path):
    """TSP: a ``{"Pause": 1}`` file holds training at a step boundary; clearing it (from another thread, as an operator
    would) resumes; a request that is never cleared ends at ``max_pause_seconds``."""
    import json
    import threading
    import time
    from types import SimpleNamespace
    from mindformers_b200.core.callback import StepPauseCallback
    path = tmp_path / "step_pause.json"
    cb = StepPauseCallback(pause_path=str(path), poll_seconds=0.05, max_pause_seconds=5.0)
    ctx = SimpleNamespace(global_step=3)
    t0 = time.time()
    cb.on_step_end(ctx)                                   # no file: nothing happens
    assert time.time() - t0 < 0.05 and cb.pauses == 0
    path.write_text(json.dumps({"Pause": 1}))
    threading.Timer(0.3, lambda: path.write_text(json.dumps({"Pause": 0}))).start()
    t0 = time.time()
    cb.on_step_end(ctx)
    held = time.time() - t0
    assert 0.25 < held < 2.0 and cb.pauses == 1 and abs(cb.paused_seconds - held) < 0.1
    path.write_text(json.dumps({"Pause": 1}))
    short = StepPauseCallback(pause_path=str(path), poll_seconds=0.05, max_pause_seconds=0.2)
    t0 = time.time()
    short.on_step_end(ctx)
    assert 0.15 < time.time() - t0 < 1.0
