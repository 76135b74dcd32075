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


def _free_port() -> int:
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _torchrun(n, script_args, timeout=600, extra_env=None):
    # NVLS off and plain peer loads / stores in our own kernels: a rank that died while bound to a multicast object would
    # fault its peers; a free port, so concurrent jobs on a shared machine cannot collide.
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1", **(extra_env or {}))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port())] + script_args
    return subprocess.run(cmd, cwd=REPO, env=env, capture_output=True, text=True, timeout=timeout)


def _selftest(case, n=2, extra_env=None):
    _need(n)
    res = _torchrun(n, ["-m", "cppmega_mlx_b200.parallel.selftest", case], extra_env=extra_env)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    return json.loads([l for l in res.stdout.splitlines() if l.startswith("{")][-1])


def test_fused_zero1_matches_nccl_zero1_two_gpus():
    out = _selftest("zero1")
    # Muon's orthogonalised update has unit scale, so one differently rounded bf16 gradient sum can move a single element by about
    # the learning rate (2e-2 here) per step; the mean over all parameters is the tight bound
    assert out["max_param_diff"] < 5e-2, out
    assert out["mean_param_diff"] < 2e-3, out
    assert out["rank_spread"] == 0.0, out
    assert all(abs(a - b) < 5e-2 for a, b in zip(out["loss_fused"], out["loss_nccl"])), out


def test_fused_zero1_multimem_form_matches_nccl_two_gpus():
    """The same step with the gradients reduced in the switch (multimem.ld_reduce) and the parameters pushed by one multicast
    store (multimem.st).  Skipped where the symmetric buffers have no multicast binding."""
    out = _selftest("zero1", extra_env={"CPPMEGA_ZERO1_MULTIMEM": "1"})
    if not out["multimem"]:
        pytest.skip("symmetric memory has no multicast binding on this machine")
    assert out["max_param_diff"] < 5e-2, out
    assert out["mean_param_diff"] < 2e-3, out
    assert out["rank_spread"] == 0.0, out
    assert all(abs(a - b) < 5e-2 for a, b in zip(out["loss_fused"], out["loss_nccl"])), out


def test_symmetric_memory_all_reduce_matches_nccl_two_gpus():
    """Stand-alone all-reduce over one symmetric buffer, peer form and (where bound) multimem form, fp32 and bf16, ragged lengths."""
    out = _selftest("allreduce")
    assert out["fp32_peer"]["max_rel_err"] < 1e-5 and out["bf16_peer"]["max_rel_err"] < 2e-2, out
    for k in ("fp32_multimem", "bf16_multimem"):
        if isinstance(out[k], dict):
            assert out[k]["max_rel_err"] < (1e-5 if k.startswith("fp32") else 2e-2), out


def test_fused_zero1_is_bitwise_deterministic_two_gpus():
    out = _selftest("zero1det")
    assert out["bitwise_equal"] and out["finite"], out
    assert out["rank_spread"] == 0.0, out


def test_fused_tp_pairs_match_nccl_two_gpus():
    """GEMM → reduce-scatter and all-gather → GEMM over peer memory against the NCCL pairs (small shape)."""
    out = _selftest("tp", extra_env={"CMB_TP_SMALL": "1"})
    assert all(e < 3e-2 for e in out["rel_err_vs_nccl[y,dx,dw_up,dw_down]"]), out
    assert out["rel_err_vs_fp32_single_gpu"] < 3e-2, out


def test_fused_tp_all_reduce_ffn_matches_nccl_two_gpus():
    """The replicated-activation FFN (what ``bench.py --tp 2 --tp-fused`` runs): fused GEMM → reduce-scatter + gather vs NCCL all-reduce."""
    out = _selftest("tpar", extra_env={"CMB_TP_SMALL": "1"})
    assert all(e < 3e-2 for e in out["rel_err_vs_nccl[y,dx,dw_up,dw_down]"]), out


def test_fused_ep_dispatch_combine_matches_all_to_all_two_gpus():
    out = _selftest("ep", extra_env={"CMB_EP_SMALL": "1"})
    assert all(e < 5e-2 for e in out["rel_err_vs_nccl[y,dx,dw_gate_up,dw_down,dw_router]"]), out


def test_fused_ep_overflow_is_dropped_not_written_two_gpus():
    out = _selftest("epdrop")
    assert out["dropped_total"] > 0, out
    assert all(e < 5e-2 for e in out["rel_err_vs_nccl[y,dx,dw_down]"]), out


def test_head_parallel_cached_decode_matches_unsharded_session_two_gpus():
    """Prefill + one-token steps on the head-parallel stack (Mamba3, MLA, M2RNN; every rank keeps its share of the caches) against the
    unsharded model's own decode session, bf16 with the kernels on."""
    out = _selftest("tpdecode")
    assert out["finite"] and out["sharded_mixers"]["mamba3"] == 1 and out["sharded_mixers"]["mla"] == 1 and out["sharded_mixers"]["m2rnn"] == 1, out
    assert out["rel_err_prefill"] < 4e-2 and out["rel_err_decode_steps"] < 4e-2, out

