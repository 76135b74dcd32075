"""Multi-GPU checks, run as child processes (one per GPU) when at least two GPUs are visible."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _need(n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


def _torchrun(n, script_args, timeout=600):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", "29641"] + script_args
    return subprocess.run(cmd, cwd=REPO, env=env, capture_output=True, text=True, timeout=timeout)


def test_fused_zero1_matches_nccl_zero1_two_gpus():
    _need(2)
    res = _torchrun(2, ["-m", "cppmega_mlx_b200.parallel.selftest", "zero1"])
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    line = [l for l in res.stdout.splitlines() if l.startswith("{")][-1]
    out = json.loads(line)
    assert out["max_param_diff"] < 2e-2, out
    assert all(abs(a - b) < 5e-2 for a, b in zip(out["loss_fused"], out["loss_nccl"])), out
