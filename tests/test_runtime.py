"""Runtime: kernel policy, seed/RNG snapshots, environment report, memory plan, audit, host-side failure detection."""
import random
import time

import numpy as np
import pytest
import torch

from cppmega_mlx_b200.runtime import kernel_policy as kp
from cppmega_mlx_b200.runtime import memory, seed
from cppmega_mlx_b200.runtime.env import detect_runtime_environment
from cppmega_mlx_b200.runtime.memory_audit import audit_memory
from cppmega_mlx_b200.runtime.watchdog import (FileStore, Heartbeat, PeerFailure, StepWatchdog, find_stalled_ranks,
                                               require_all_alive)


def test_kernel_path_env(monkeypatch):
    assert kp.selected_path() is kp.KernelPath.AUTO
    monkeypatch.setenv("CPPMEGA_KERNEL_PATH", "reference")
    assert kp.selected_path() is kp.KernelPath.REFERENCE and not kp.selected_path().uses_kernels
    monkeypatch.setenv("CPPMEGA_KERNEL_PATH__MAMBA3", "path_c")
    assert kp.selected_path("mamba3") is kp.KernelPath.PATH_C and kp.selected_path("mamba3").uses_kernels
    assert kp.selected_path("m2rnn") is kp.KernelPath.REFERENCE
    monkeypatch.setenv("CPPMEGA_KERNEL_PATH", "bogus")
    with pytest.raises(ValueError):
        kp.selected_path()


def test_dispatch_log_is_a_ring():
    kp.clear_dispatch_log()
    for i in range(kp.DISPATCH_LOG_CAPACITY + 10):
        kp.record_dispatch(f"op{i}", kp.KernelPath.AUTO, "kernels")
    log = kp.get_dispatch_log()
    assert len(log) == kp.DISPATCH_LOG_CAPACITY and log[0]["op"] == "op10" and log[-1]["requested"] == "auto"
    kp.clear_dispatch_log()
    assert kp.get_dispatch_log() == []


def test_apply_policy_switches_backend(monkeypatch):
    from cppmega_mlx_b200.ops import _backend as B
    monkeypatch.setenv("CPPMEGA_KERNEL_PATH", "reference")
    try:
        kp.apply_policy_from_env()
        assert not B.kernels_enabled()
    finally:
        B.set_kernels_enabled(True)


def test_seed_and_snapshot_round_trip():
    seed.seed_all(11)
    snap = seed.capture_rng_state()
    a = (random.random(), float(np.random.rand()), torch.rand(3))
    seed.restore_rng_state(snap)
    b = (random.random(), float(np.random.rand()), torch.rand(3))
    assert a[0] == b[0] and a[1] == b[1] and torch.equal(a[2], b[2])
    with pytest.raises(ValueError):
        seed.seed_all(-1)
    with pytest.raises(ValueError):
        seed.restore_rng_state({"python": snap["python"]})


def test_environment_report_is_read_only_dict():
    env = detect_runtime_environment().to_dict()
    assert env["torch"] == torch.__version__ and env["hardware_tier"] in ("cpu", "b200", "cuda-other")


def test_memory_plan_and_receipt():
    plan = memory.memory_limit_plan(1000, allocator_fraction=0.9, peak_fraction=0.5)
    assert plan.allocator_limit_bytes == 900 and plan.peak_target_bytes == 500
    with pytest.raises(ValueError):
        memory.memory_limit_plan(1000, allocator_fraction=0.5, peak_fraction=0.9)
    with pytest.raises(ValueError):
        memory.memory_limit_plan(0)
    rec = memory.memory_limit_receipt(plan, [memory.MemorySnapshot(1, 400, 2), memory.MemorySnapshot(1, 600, 2)])
    assert rec["peak_bytes"] == 600 and not rec["within_peak_target"] and rec["within_allocator_limit"]
    assert memory.apply_memory_limit_plan(plan)["applied"] == torch.cuda.is_available()
    assert memory.ClearCachePolicy(every_n_steps=2).maybe_clear_cache(2) == torch.cuda.is_available()


def test_memory_audit_categories():
    from cppmega_mlx_b200.recipes.model_factory import build_local_gb10_quarter_tiny_smoke_model
    from cppmega_mlx_b200.training.optimizers import make_adamw
    m = build_local_gb10_quarter_tiny_smoke_model()
    opt = make_adamw(m)
    for _, p in m.named_parameters():
        p.grad = torch.zeros_like(p)
    opt.step()
    rep = audit_memory(m, opt)
    total = sum(p.numel() * p.element_size() for p in m.parameters())
    assert rep["parameter_bytes"] == total
    assert set(rep["by_category"]) >= {"embedding", "muon", "adamw"}
    assert rep["optimizer_state_bytes"] == 2 * sum(p.numel() * 4 for p in m.parameters())
    assert len(rep["largest_leaves"]) == 10


def test_heartbeat_detects_a_silent_rank(tmp_path):
    store = FileStore(tmp_path)
    hb0, hb1 = Heartbeat(store, 0, 0.05).start(), Heartbeat(store, 1, 0.05).start()
    time.sleep(0.15)
    assert find_stalled_ranks(store, 2, deadline_s=1.0) == []
    hb1.stop()                      # rank 1 "dies" on the host: its stamps stop
    time.sleep(0.4)
    assert find_stalled_ranks(store, 2, deadline_s=0.2) == [1]
    with pytest.raises(PeerFailure):
        require_all_alive(store, 2, 0.2, rank=0)
    assert find_stalled_ranks(store, 3, deadline_s=10.0) == [2]   # a rank that never joined
    hb0.stop()


def test_step_watchdog():
    w = StepWatchdog(timeout_s=5.0)
    w.progress(1)
    w.check(now=w.last_time + 1.0)
    with pytest.raises(TimeoutError):
        w.check(now=w.last_time + 6.0)
    w.progress(2)
    w.check()


def test_lint_rules_fire_and_the_package_is_clean(tmp_path):
    import os
    from cppmega_mlx_b200.runtime.lint import lint_paths, lint_source
    hot = tmp_path / "nn"
    hot.mkdir()
    bad = hot / "layer.py"
    bad.write_text(
        "import triton\n"
        "import torch\n"
        "class L:\n"
        "    def forward(self, x):\n"
        "        n = x.sum().item()\n"
        "        m = x.max().item()  # lint: allow HS001 needed for the test\n"
        "        torch.cuda.synchronize()\n"
        "        return x * n * m\n"
        "    def helper(self, x):\n"
        "        return x.tolist()\n"
        "def f():\n"
        "    try:\n"
        "        pass\n"
        "    except:\n"
        "        pass\n"
        "    import os, subprocess\n"
        "    os.environ['MASTER_ADDR'] = 'localhost'\n"
        "    subprocess.run(['pkill', '-f', 'python'])\n"
        "    return torch.compile(f)\n")
    rules = sorted((v.rule, v.line) for v in lint_paths([str(tmp_path)]))
    assert rules == [("CL001", 1), ("CL001", 19), ("EX001", 14), ("HS001", 5), ("HS001", 7), ("PK001", 18), ("RZ001", 17)]
    # the same sync outside a hot directory, or outside a hot function, is not flagged
    assert not lint_source("def forward(x):\n    return x.item()\n", "cli/tool.py")
    assert not lint_source("import torch.distributed as d\nd.init_process_group('gloo', init_method='tcp://127.0.0.1:29500')\n", "x.py")
    assert [v.rule for v in lint_source("import torch.distributed as d\nd.init_process_group('gloo', init_method='tcp://myhost:1')\n", "x.py")] == ["RZ001"]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    found = lint_paths([os.path.join(root, "cppmega_mlx_b200"), os.path.join(root, "bench.py"), os.path.join(root, "__graft_entry__.py")])
    assert not found, "\n".join(map(str, found))
