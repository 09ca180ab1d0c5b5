"""Multi-GPU checks (2 ranks): each spawns a ``torchrun`` worker from ``tests/dist`` and asserts on its exit code.
Skipped on boxes with fewer than two GPUs. NVLS is switched off; the kernels use plain peer loads/stores."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(script, *args, nproc=2, timeout=900):
    if torch.cuda.device_count() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", "29611", os.path.join(ROOT, "tests", "dist", script), *args]
    r = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=timeout)
    assert r.returncode == 0, (r.stdout[-3000:], r.stderr[-3000:])
    return r.stdout


def test_fused_tensor_parallel_gemms():
    _run("run_fused_tp.py", "--bench", "0")


def test_fused_data_parallel_optimizer():
    _run("run_fused_dp.py", "--big", "0")


def test_fused_moe_expert_parallel_exchange():
    _run("run_fused_moe.py", "--bench", "0")


def test_fused_context_parallel_attention():
    _run("run_fused_cp.py", "--bench", "0")


def test_tp_attention_ep_moe_inference_bf16_and_fp8():
    _run("run_tp_ep_inference.py")


def test_low_latency_all_reduce():
    _run("run_ll_allreduce.py")
