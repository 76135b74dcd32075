"""Trainer CLI as a subprocess: JSON receipt, dry run, fail-closed errors, checkpoint + resume == uninterrupted run."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BASE = ["--batch-size", "2", "--seq-len", "12", "--hidden-size", "32", "--num-attention-heads", "2", "--mamba-head-dim", "8",
        "--mamba-state-dim", "8", "--json"]


def _run(*args, env=None):
    e = dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="")
    e.update(env or {})
    r = subprocess.run([sys.executable, "-m", "cppmega_mlx_b200.cli.train_hybrid_tiny", *args], capture_output=True, text=True,
                       env=e, cwd=ROOT, timeout=300)
    line = r.stdout.strip().splitlines()[-1] if r.stdout.strip() else "{}"
    return r.returncode, json.loads(line), r


@pytest.fixture()
def shard(tmp_path):
    p = tmp_path / "train.npz"
    rng = np.random.default_rng(0)
    np.savez(p, tokens=rng.integers(4, 96, size=13 * 2 * 40, dtype=np.int32))
    return str(p)


def test_receipt_and_dry_run(shard):
    rc, out, _ = _run("--npz-path", shard, "--steps", "3", "--eval-batches", "2", *BASE)
    assert rc == 0 and out["status"] == "ok" and out["steps_completed"] == 3 and len(out["metrics"]) == 3
    assert out["dataset"]["format"] == "npz" and out["route_symbols"] == list("AEMR") and out["parameter_count"] > 0
    assert out["eval"]["batches"] == 2 and out["optimizer"]["source"] == "default"
    assert {"config", "model_config", "environment", "memory", "kernel_dispatch", "tokenizer_contract"} <= set(out)
    rc, dry, _ = _run("--steps", "3", "--dry-run", *BASE)
    assert rc == 0 and dry["status"] == "dry_run" and "metrics" not in dry and dry["dataset"]["source"] == "synthetic"


def test_fail_closed_json_and_env_override(shard):
    rc, out, _ = _run("--steps", "2", "--optimizer", "sgd", *BASE)
    assert rc == 2 and out["status"] == "error" and "optimizer" in out["error"]
    rc, out, _ = _run("--npz-path", "/nonexistent/x.npz", "--steps", "1", *BASE)
    assert rc == 2 and out["status"] == "error"
    rc, out, _ = _run("--npz-path", shard, "--steps", "1", "--vocab-size", "16", *BASE)
    assert rc == 2 and "vocab" in out["error"]
    rc, out, _ = _run("--steps", "2", *BASE, env={"CPPMEGA_OPTIMIZER": "lion8bit"})
    assert rc == 0 and out["optimizer"]["name"] == "lion8bit" and out["optimizer"]["source"].startswith("env:")


@pytest.mark.parametrize("opt", ["adamw", "muon"])
def test_resume_through_cli_equals_uninterrupted(shard, tmp_path, opt):
    common = ["--npz-path", shard, "--optimizer", opt, "--grad-accum-steps", "2", "--shuffle", *BASE]
    rc, full, _ = _run("--steps", "6", *common)
    assert rc == 0
    ckdir = str(tmp_path / "ck")
    rc, first, _ = _run("--steps", "3", "--checkpoint-dir", ckdir, "--checkpoint-save-interval", "3", *common)
    assert rc == 0 and first["checkpoints"][0]["step"] == 3
    rc, second, r = _run("--steps", "6", "--resume-from", ckdir, *common)
    assert rc == 0, r.stdout + r.stderr
    assert second["resume"]["step"] == 3 and second["resume"]["consumed_batches"] == 6
    a = [m["loss"] for m in full["metrics"]]
    b = [m["loss"] for m in first["metrics"]] + [m["loss"] for m in second["metrics"]]
    assert a == b
