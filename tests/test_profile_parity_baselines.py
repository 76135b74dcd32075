import json

import pytest
import torch

from cppmega_mlx_b200.training import baselines as BL
from cppmega_mlx_b200.training import parity as PA
from cppmega_mlx_b200.training import profile as PR
from cppmega_mlx_b200.training import safetensors_io as st


def test_step_profiler_and_layer_timer():
    from cppmega_mlx_b200.recipes.model_factory import build_local_gb10_quarter_tiny_smoke_model
    m = build_local_gb10_quarter_tiny_smoke_model()
    x = torch.randint(4, 100, (2, 16))
    out, met = PR.profile_step(lambda: m(x), label="fwd", tokens=32)
    assert out.shape[0] == 2 and met.seconds > 0 and met.tokens_per_second > 0 and met.label == "fwd"
    assert json.dumps(met.to_dict())
    sink = []
    with PR.profile_context("ctx", sink, tokens=8):
        m(x)
    assert len(sink) == 1 and sink[0].label == "ctx"
    with PR.LayerTimer(m) as lt:
        m(x)
    assert len(lt.seconds) == len(m.layers) and all(v >= 0 for v in lt.seconds.values())


def test_kernel_adoption_gate():
    hot = PR.HotspotEvidence("mamba3_scan", 0.030, 0.100, differentiable=True, vjp_covered=True)
    assert PR.assess_kernel_adoption("mamba3_scan_sm100", [hot]).allowed
    assert not PR.assess_kernel_adoption("k", []).allowed
    assert not PR.assess_kernel_adoption("k", [PR.HotspotEvidence("x", 0.005, 0.100)]).allowed                 # 5 % of the window
    assert not PR.assess_kernel_adoption("k", [PR.HotspotEvidence("x", 0.0005, 0.001)]).allowed                # under 1 ms
    assert not PR.assess_kernel_adoption("k", [PR.HotspotEvidence("x", 0.03, 0.1, local_profile=False)]).allowed
    assert not PR.assess_kernel_adoption("k", [PR.HotspotEvidence("x", 0.03, 0.1, differentiable=True)]).allowed
    with pytest.raises(RuntimeError):
        PR.require_kernel_hotspot_evidence("k", [])
    with pytest.raises(ValueError):
        PR.HotspotEvidence("x", 2.0, 1.0)
    rows = PR.summarize_hotspots([hot, PR.HotspotEvidence("y", 0.05, 0.1)])
    assert rows[0]["name"] == "y"


def test_parity_receipts_fail_closed(tmp_path):
    ours = {"a": torch.ones(3, 4), "b": torch.zeros(2)}
    man = PA.parity_against_artifact("fwd", ours, tmp_path / "missing.safetensors")
    assert man.status == "refused" and all(r.status == "refused" for r in man.receipts)
    st.save_file({"a": torch.ones(3, 4) + 0.01, "b": torch.ones(2)}, tmp_path / "art.safetensors")
    man = PA.parity_against_artifact("fwd", ours, tmp_path / "art.safetensors")
    by = {r.name: r for r in man.receipts}
    assert by["a"].status == "pass" and by["b"].status == "fail" and man.status == "fail"
    assert PA.compare_tensors("s", torch.ones(2), torch.ones(3)).status == "fail"
    assert PA.compare_tensors("n", torch.tensor([float("nan")]), torch.ones(1)).status == "fail"
    man.write(tmp_path / "m.json")
    assert json.loads((tmp_path / "m.json").read_text())["status"] == "fail"


def test_baseline_archive_and_matched_comparison(tmp_path):
    wl = dict(model="hybrid_1b", global_batch=4, seq_len=4096, dtype="bf16", optimizer="muon_adamw", n_gpus=1, parallelism="dp1")
    base = BL.BaselineRow("eager", "tokens/s", 8551.0, "tokens/s", wl, hardware="B200")
    ours = BL.BaselineRow("ours", "tokens/s", 33784.0, "tokens/s", wl, hardware="B200")
    BL.archive_baseline(base, tmp_path)
    BL.archive_baseline(ours, tmp_path)
    idx = json.loads((tmp_path / "index.json").read_text())
    assert idx["count"] == 2 and len(BL.load_rows(tmp_path)) == 2
    cmp = BL.compare_rows(ours, base)
    assert cmp["status"] == "ok" and cmp["ratio"] == pytest.approx(3.95, abs=0.01)
    other = BL.BaselineRow("o", "tokens/s", 1.0, "tokens/s", {**wl, "seq_len": 2048}, hardware="B200")
    assert BL.compare_rows(other, base)["status"] == "refused"
    with pytest.raises(ValueError):
        BL.BaselineRow("x", "m", 1.0, "u", {"model": "a"})
    with pytest.raises(ValueError):
        BL.BaselineRow("x", "m", float("nan"), "u", wl)
