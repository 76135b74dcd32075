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


def _run_main(mod, argv, capsys):
    rc = mod.main(argv)
    out = capsys.readouterr().out.strip().splitlines()
    return rc, out


def test_check_environment_and_data_smoke_and_audit(capsys, tmp_path):
    import json

    import numpy as np

    from cppmega_mlx_b200.cli import audit_memory, check_environment, data_smoke
    rc, out = _run_main(check_environment, ["--json"], capsys)
    rep = json.loads("\n".join(out))
    assert rc == 0 and rep["distributed_backends"]["gloo"] and "kernel_library" in rep and "environment" in rep
    rc, out = _run_main(data_smoke, ["--synthetic", "--seq-len", "16", "--batch-size", "3"], capsys)
    rep = json.loads(out[-1])
    assert rc == 0 and rep["status"] == "ok" and rep["batches"][0]["inputs"] == [3, 16] and rep["cursor_after"]["global"] == 2
    bad = tmp_path / "bad.npz"
    np.savez(bad, tokens=np.arange(400, dtype=np.int32))
    rc, out = _run_main(data_smoke, [str(bad), "--seq-len", "16", "--vocab-size", "100"], capsys)
    assert rc == 2 and json.loads(out[-1])["ids_within_vocab"] is False           # ids beyond the vocabulary fail closed
    rc, out = _run_main(audit_memory, ["--profile", "hybrid_1b", "--dp", "8"], capsys)
    rep = json.loads(out[-1])
    assert rc == 0 and rep["parameters"] == 1756904002 and 0 < rep["zero1"]["fraction_of_b200_hbm"] < 1


def test_train_tiny_npz_and_optimizer_receipts(capsys, tmp_path):
    import json

    from cppmega_mlx_b200.cli import bench_optimizers, train_tiny_npz
    rc, out = _run_main(train_tiny_npz, ["--steps", "25", "--json"], capsys)
    rep = json.loads(out[-1])
    assert rc == 0 and rep["status"] == "ok" and rep["last_loss"] < rep["first_loss"] - 0.5
    rc, out = _run_main(train_tiny_npz, ["--data", str(tmp_path / "missing.npz"), "--json"], capsys)
    assert rc == 2 and json.loads(out[-1])["status"] == "error"
    rc, out = _run_main(bench_optimizers, ["--matrices", "2", "--rows", "64", "--cols", "128", "--steps", "2"], capsys)
    rows = {r["optimizer"]: r for r in map(json.loads, out)}
    assert rc == 0 and rows["adam8bit_symmetric"]["state_vs_adamw_fp32"] < 0.3 and rows["lion8bit_symmetric"]["state_vs_adamw_fp32"] < 0.15
    assert rows["muon_quantized_momentum"]["state_bytes"] < 0.35 * rows["muon_fp32_carrier"]["state_bytes"]
    assert rows["muon_bf16_carrier"]["max_param_drift_vs_family_fp32"] < 1e-3


def test_zero1_loopback_receipt(capsys):
    import json

    from cppmega_mlx_b200.cli import bench_zero1_loopback
    rc, out = _run_main(bench_zero1_loopback, ["--steps", "3", "--port", "29741"], capsys)
    rep = json.loads(out[-1])
    assert rc == 0 and rep["status"] == "ok" and rep["max_loss_gap"] < 1e-4 and rep["state_fraction_largest_rank"] < 0.6


def test_bench_tiny_archives_and_refuses_unmatched_comparisons(capsys, tmp_path):
    import json

    from cppmega_mlx_b200.cli import bench_tiny
    arch = str(tmp_path / "rows")
    rc, out = _run_main(bench_tiny, ["--steps", "5", "--warmup", "2", "--pattern", "AM", "--archive", arch], capsys)
    rep = json.loads(out[-1])
    assert rc == 0 and rep["row"]["value"] > 0 and (tmp_path / "rows" / "index.json").exists()
    rc, out = _run_main(bench_tiny, ["--steps", "5", "--warmup", "2", "--pattern", "AM", "--compare-to", arch, "--min-ratio", "0.05"], capsys)
    cmp = json.loads(out[-1])["comparisons"]
    assert rc == 0 and cmp[0]["status"] == "ok" and cmp[0]["ratio"] > 0.05
    rc, out = _run_main(bench_tiny, ["--steps", "5", "--warmup", "2", "--pattern", "AM", "--batch-size", "4", "--compare-to", arch,
                                     "--min-ratio", "0.05"], capsys)
    cmp = json.loads(out[-1])["comparisons"]
    assert rc == 3 and cmp[0]["status"] == "refused" and "global_batch" in cmp[0]["reason"]   # no matched row → gate fails closed


def test_bench_matrix_runs_cells_in_fresh_processes_and_renders(tmp_path):
    from cppmega_mlx_b200.cli import bench_matrix as BM
    dry = subprocess.run([sys.executable, "-m", "cppmega_mlx_b200.cli.bench_matrix", "--dry-run", "--optimizers", "adamw,lion"],
                         capture_output=True, text=True, cwd=ROOT)
    rep = json.loads(dry.stdout.strip().splitlines()[-1])
    assert rep["status"] == "dry_run" and rep["cells"] == 4 and all("bench_tiny" in c for c in rep["commands"])
    out = tmp_path / "m"
    run = subprocess.run([sys.executable, "-m", "cppmega_mlx_b200.cli.bench_matrix", "--optimizers", "adamw,nonsense", "--paths", "eager",
                          "--pattern", "AM", "--steps", "4", "--warmup", "1", "--out-dir", str(out)], capture_output=True, text=True, cwd=ROOT)
    rep = json.loads(run.stdout.strip().splitlines()[-1])
    assert run.returncode == 1 and rep["status"] == "partial" and rep["failed"] == 1      # the bad cell is kept, with its error
    good, bad = rep["matrix"]
    assert good["status"] == "ok" and good["tokens_per_second"] > 0 and bad["status"] == "error" and "optimizer" in bad["error"]
    assert "| float32 | adamw | cross_entropy | eager |" in (out / "matrix.md").read_text()
    page = (out / "matrix.html").read_text()
    assert page.startswith("<!doctype html>") and "adamw" in page and 'class="bad"' in page
    cells = [{"dtype": "f", "optimizer": "o", "loss_backend": "l", "path": "kernels", "status": "ok", "tokens_per_second": 30.0},
             {"dtype": "f", "optimizer": "o", "loss_backend": "l", "path": "eager", "status": "ok", "tokens_per_second": 10.0}]
    BM.add_ratios(cells)
    assert cells[0]["ratio_vs_eager"] == 3.0 and "ratio_vs_eager" not in cells[1]


def test_v4_parquet_smoke_runs_the_whole_block_cohort_and_writes_a_receipt(capsys, tmp_path):
    """The V4 smoke builds engram + GDN + KDA + attention + NSA + CSA/HCA + MoE + MLP from the reference's template parameters
    (head_dim, intermediate_size, use_short_conv, …), reads a token parquet and returns finite losses and timings."""
    from cppmega_mlx_b200.cli import v4_parquet_smoke as S
    pq = tmp_path / "tokens.parquet"
    S.write_synthetic_parquet(pq, rows=6, row_len=49, vocab_size=300)
    rc = S.main(["--parquet", str(pq), "--hidden-size", "128", "--layers", "6", "--vocab-size", "300", "--seq-len", "48", "--steps", "2",
                 "--device", "cpu", "--out", str(tmp_path / "reports")])
    assert rc == 0
    rec = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rec["total_blocks"] == 8 and rec["steps"] == 2 and len(rec["per_step"]) == 2
    assert all(np.isfinite(s["loss"]) and s["total_ms"] > 0 for s in rec["per_step"])
    assert rec["tokens_per_sec"] > 0
    assert len(list((tmp_path / "reports").glob("v4_parquet_smoke_h128_L6_*.json"))) == 1
    assert S.main(["--parquet", str(tmp_path / "missing.parquet"), "--device", "cpu"]) == 1
    with pytest.raises(ValueError):          # token ids must fit the vocabulary
        S.main(["--parquet", str(pq), "--hidden-size", "128", "--layers", "6", "--vocab-size", "100", "--seq-len", "48", "--steps", "1", "--device", "cpu"])


def test_train_step_receipt_harness_gates_and_optimizer_table(capsys, tmp_path):
    """The receipt harness on a synthetic shard: steps run, the throughput and acceptance gates are evaluated (a synthetic, shallow,
    3-step fp32 run can never be accepted), the optimizer table lists all eight choices, and --require-acceptance turns the
    refusal into a non-zero exit code."""
    from cppmega_mlx_b200.cli import m04_train_step as M
    common = ["--synthetic", "--model-profile", "custom", "--vocab-size", "256", "--hidden-size", "32", "--pattern", "MA", "--depth", "2",
              "--num-attention-heads", "2", "--steps", "3", "--batch-size", "2", "--seq-len", "16", "--dtype", "float32", "--device", "cpu",
              "--json"]
    out = tmp_path / "receipt.json"
    assert M.main(common + ["--output", str(out)]) == 0
    rec = json.loads(out.read_text())
    assert rec["status"] == "ok" and len(rec["steps"]) == 3 and np.isfinite(rec["final_loss"])
    assert rec["acceptance_gate"]["accepted"] is False and "real_parquet_source" in rec["acceptance_gate"]["failed"]
    assert rec["throughput_claim_gate"]["status"] == "pass" and len(rec["optimizer"]["table"]) == 8
    assert "kernel_dispatch" in rec
    capsys.readouterr()
    assert M.main(common + ["--output", str(tmp_path / "r2.json"), "--require-acceptance"]) != 0
    assert M.main(common + ["--output", str(tmp_path / "dry.json"), "--dry-run-json"]) == 0
    assert json.loads((tmp_path / "dry.json").read_text())["status"] == "dry_run"


def test_parity_manifest_cli_is_fail_closed_without_an_artifact(capsys, tmp_path):
    from cppmega_mlx_b200.cli import parity_manifest as P
    out = tmp_path / "mtp.json"
    rc = P.main(["mtp", "--tiny", "--no-artifact", "--device", "cpu", "--output", str(out), "--json"])
    man = json.loads(out.read_text())
    assert man["status"] == "blocked" and man["reference"]["artifact_preflight_status"] == "not_supplied"
    assert np.isfinite(man["local"]["loss_values"]["total_loss"])
    assert rc != 0 or man["status"] == "blocked"
    out2 = tmp_path / "fwd.json"
    P.main(["forward", "--tiny", "--no-artifact", "--device", "cpu", "--output", str(out2)])
    assert json.loads(out2.read_text())["status"] in ("blocked", "refused")


def test_cut_ce_receipt_and_route_gradient_probe(capsys, tmp_path):
    import json

    from cppmega_mlx_b200.cli import bench_cce, probe_route_grad
    out_file = tmp_path / "cce.jsonl"
    rc, out = _run_main(bench_cce, ["--batch-size", "2", "--seq-len", "48", "--vocab-size", "512", "--hidden", "32", "--row-chunk", "16",
                                    "--iters", "2", "--warmup", "1", "--output", str(out_file)], capsys)
    rows = [json.loads(l) for l in out]
    assert rc == 0 and [r.get("form") for r in rows[:2]] == ["materialized", "cut"] and rows[2]["status"] == "ok"
    assert rows[1]["loss_abs_diff_vs_materialized"] < 1e-5 and rows[1]["max_grad_abs_diff_vs_materialized"] < 1e-6
    assert rows[2]["memory_ratio_cut_vs_materialized"] == pytest.approx(16 * 4 / (96 * 8))      # one chunk of fp32 logits against all rows twice
    assert len(out_file.read_text().splitlines()) == 3
    rc, out = _run_main(bench_cce, ["--seq-len", "0"], capsys)
    assert rc == 2 and json.loads(out[-1])["status"] == "error"

    rc, out = _run_main(probe_route_grad, ["--tiny", "--seq-len", "16", "--batch-size", "2", "--model-profile", "nam56r_56l"], capsys)
    rep = json.loads(out[-1])
    assert rc == 0 and rep["status"] == "ok" and [r["route"] for r in rep["routes"]] == ["reference", "kernels"]
    ref, ker = rep["routes"]
    assert ref["loss_finite"] and ref["grad_norm"] > 0 and not ref["nonfinite_gradients"] and ref["total_kernel_calls"] == 0
    assert ker["loss_abs_diff_vs_reference"] < 1e-5 and ker["max_grad_rel_diff_vs_reference"]["value"] < 1e-4     # no GPU here: both routes are the restatements
    assert set("".join(rep["pattern"])) >= set("AMER")
    rc, out = _run_main(probe_route_grad, ["--routes", "metal"], capsys)
    assert rc == 2 and "routes must be taken from" in json.loads(out[-1])["error"]
    rc, out = _run_main(probe_route_grad, ["--model-profile", "nope"], capsys)
    assert rc == 2 and "unknown model profile" in json.loads(out[-1])["error"]


def test_trainer_context_parallel_two_processes_match_one(tmp_path):
    """``--context-parallel 2`` under the launcher: two processes share every sequence and reproduce the single-process losses
    (Mamba3 scans on both ranks at once with the boundary terms exchanged, M2RNN continues from the first rank's state, attention
    gathers the keys: the split evaluation equals the whole one)."""
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    args = ["--batch-size", "2", "--seq-len", "12", "--hidden-size", "32", "--num-attention-heads", "2", "--pattern", "MAR", "--depth", "3",
            "--mamba-head-dim", "8", "--mamba-state-dim", "8", "--mamba-chunk-size", "4",
            "--steps", "3", "--vocab-size", "64", "--loss-backend", "cross_entropy", "--eval-batches", "1", "--json"]
    rc, one, r = _run(*args)
    assert rc == 0, r.stderr[-2000:]
    env = dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), "-m", "cppmega_mlx_b200.cli.train_hybrid_tiny", *args, "--context-parallel", "2"]
    p = subprocess.run(cmd, capture_output=True, text=True, env=env, cwd=ROOT, timeout=600)
    assert p.returncode == 0, p.stderr[-3000:]
    two = json.loads([l for l in p.stdout.splitlines() if l.startswith("{")][-1])          # rank 0 prints the receipt
    assert two["context_parallel"] == {"size": 2, "data_parallel": 1, "tokens_per_rank": 6} and two["world_size"] == 2
    l1, l2 = [m["loss"] for m in one["metrics"]], [m["loss"] for m in two["metrics"]]
    assert len(l1) == len(l2) == 3
    # rank 0 reports the mean over its half of the tokens; the parameters (and so the later losses) follow the whole-sequence gradient
    assert all(abs(a - b) < 0.15 for a, b in zip(l1, l2)), (l1, l2)
    assert abs(one["eval"]["loss"] - two["eval"]["loss"]) < 2e-4, (one["eval"], two["eval"])
    rc, rep, _ = _run(*args, "--context-parallel", "5")
    assert rc == 2 and "divide seq_len" in rep["error"]


@pytest.mark.parametrize("sp", [False, True])
def test_trainer_tensor_parallel_two_processes_match_one(sp, tmp_path):
    """``--tensor-parallel 2`` (and ``--sequence-parallel``) under the launcher: every mixer kind head- / expert-parallel on two
    processes trains like one process, and the checkpoint it writes is the logical (unsharded) one: a single process resumes from it."""
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    args = ["--batch-size", "2", "--seq-len", "12", "--hidden-size", "32", "--num-attention-heads", "4", "--pattern", "MAER", "--depth", "4",
            "--mamba-head-dim", "16", "--mamba-state-dim", "8", "--mamba-groups", "2", "--mamba-chunk-size", "4", "--mamba-expand", "2",
            "--moe-num-experts", "4", "--moe-top-k", "2", "--moe-expert-hidden-size", "16", "--m2rnn-k-head-dim", "4", "--m2rnn-v-head-dim", "4", "--m2rnn-num-v-heads", "4", "--m2rnn-num-f-heads", "4",
            "--ffn-hidden-size", "48", "--steps", "3", "--vocab-size", "64", "--loss-backend", "cross_entropy", "--eval-batches", "1", "--json"]
    rc, one, r = _run(*args)
    assert rc == 0, r.stderr[-2000:]
    env = dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="")
    ckpt = tmp_path / "tp_ckpt"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), "-m", "cppmega_mlx_b200.cli.train_hybrid_tiny", *args, "--tensor-parallel", "2",
           "--checkpoint-path", str(ckpt)] + (["--sequence-parallel"] if sp else [])
    p = subprocess.run(cmd, capture_output=True, text=True, env=env, cwd=ROOT, timeout=600)
    assert p.returncode == 0, p.stderr[-3000:]
    two = json.loads([l for l in p.stdout.splitlines() if l.startswith("{")][-1])
    info = two["tensor_parallel"]
    assert info["size"] == 2 and info["data_parallel"] == 1 and info["sequence_parallel"] == sp and sum(info["sharded_mixers"].values()) == 4
    l1, l2 = [m["loss"] for m in one["metrics"]], [m["loss"] for m in two["metrics"]]
    assert all(abs(a - b) < 2e-4 for a, b in zip(l1, l2)), (l1, l2)
    assert abs(one["eval"]["loss"] - two["eval"]["loss"]) < 2e-4
    rc, again, r = _run(*args, "--resume-from", str(ckpt), "--steps", "4")           # one process continues from the two-process checkpoint
    assert rc == 0 and again["resume"]["step"] == 3 and again["steps_completed"] == 4, r.stderr[-2000:]
    rc, rep, _ = _run(*args, "--sequence-parallel")
    assert rc == 2 and "needs tensor_parallel" in rep["error"]


def test_trainer_expert_parallel_two_processes_and_logical_checkpoint(tmp_path):
    """``--expert-parallel 2`` under the launcher: the routed experts are spread over both processes, the dense part is ZeRO-1 data
    parallel, and the checkpoint holds all experts: one process resumes from it with the whole bank."""
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    args = ["--batch-size", "2", "--seq-len", "12", "--hidden-size", "32", "--num-attention-heads", "4", "--pattern", "AE", "--depth", "2",
            "--moe-num-experts", "4", "--moe-top-k", "2", "--moe-expert-hidden-size", "16", "--vocab-size", "64", "--loss-backend", "cross_entropy",
            "--learning-rate", "0.01", "--json"]
    env = dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="")
    ckpt = tmp_path / "ep_ckpt"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), "-m", "cppmega_mlx_b200.cli.train_hybrid_tiny", *args, "--steps", "8", "--expert-parallel", "2",
           "--checkpoint-path", str(ckpt)]
    p = subprocess.run(cmd, capture_output=True, text=True, env=env, cwd=ROOT, timeout=600)
    assert p.returncode == 0, p.stderr[-3000:]
    two = json.loads([l for l in p.stdout.splitlines() if l.startswith("{")][-1])
    assert two["expert_parallel"] == {"size": 2, "experts_per_rank": 2} and two["optimizer"]["class"]
    losses = [m["loss"] for m in two["metrics"]]
    import math
    assert len(losses) == 8 and all(math.isfinite(l) and l < 6.0 for l in losses)          # synthetic tokens are random: the loss stays near ln(64)
    rc, again, r = _run(*args, "--resume-from", str(ckpt), "--steps", "9")
    assert rc == 0 and again["resume"]["step"] == 8 and again["steps_completed"] == 9, r.stderr[-2000:]
    assert abs(again["metrics"][0]["loss"] - losses[-1]) < 1.0                      # continues from the trained weights, not from scratch
    rc, rep, _ = _run(*args, "--expert-parallel", "2")
    assert rc == 2 and "must equal the world size" in rep["error"]
