"""Checkpoint layout, fail-closed validation, reference tensor naming, exact resume (mid-accumulation included)."""
import json

import pytest
import torch

from cppmega_mlx_b200.data.batch import synthetic_token_batch
from cppmega_mlx_b200.recipes.model_factory import build_local_gb10_quarter_tiny_smoke_model
from cppmega_mlx_b200.training import checkpoint as ck
from cppmega_mlx_b200.training import safetensors_io as st
from cppmega_mlx_b200.training.compiled import PretrainingStep
from cppmega_mlx_b200.training.optimizers import make_adamw, make_muon


def _setup(seed=0, accum=2, opt="muon"):
    torch.manual_seed(seed)
    m = build_local_gb10_quarter_tiny_smoke_model()
    o = make_muon(m) if opt == "muon" else make_adamw(m)
    return m, o, PretrainingStep(m, o, grad_accum_steps=accum)


def _batches(m, n):
    return [synthetic_token_batch(2, 16, vocab_size=m.config.vocab_size, seed=100 + i) for i in range(n)]


def test_safetensors_round_trip_and_third_party_reader(tmp_path):
    ts = {"b": torch.randn(3, 4).bfloat16(), "a": torch.arange(5), "s": torch.tensor(3.5), "e": torch.empty(0, 3)}
    p = tmp_path / "x.safetensors"
    st.save_file(ts, p, {"format": "mlx"})
    back = st.load_file(p)
    assert all(torch.equal(back[k], ts[k]) for k in ts) and st.file_metadata(p) == {"format": "mlx"}
    sft = pytest.importorskip("safetensors.torch")
    other = sft.load_file(str(p))
    assert all(torch.equal(other[k], ts[k]) for k in ts)


def test_safetensors_rejects_corruption(tmp_path):
    p = tmp_path / "x.safetensors"
    st.save_file({"a": torch.arange(10)}, p)
    raw = p.read_bytes()
    (tmp_path / "short.safetensors").write_bytes(raw[:-20])
    with pytest.raises(ValueError):
        st.load_file(tmp_path / "short.safetensors")
    (tmp_path / "hdr.safetensors").write_bytes(b"\xff" * 8 + raw[8:])
    with pytest.raises(ValueError):
        st.load_file(tmp_path / "hdr.safetensors")


def test_parallel_range_writers(tmp_path):
    ts = {f"t{i}": torch.randn(7, i + 1) for i in range(4)}
    head, ranges, total = st.plan_layout(ts, {"format": "mlx"})
    p = tmp_path / "r.safetensors"
    st.create_sized(p, head, total)
    st.write_ranges(p, {k: ts[k] for k in ("t0", "t2")}, ranges)   # "rank 0"
    st.write_ranges(p, {k: ts[k] for k in ("t1", "t3")}, ranges)   # "rank 1"
    back = st.load_file(p)
    assert all(torch.equal(back[k], ts[k]) for k in ts)


def test_layout_and_reference_names(tmp_path):
    m, o, step = _setup()
    step(_batches(m, 1)[0])
    meta = ck.save_checkpoint(m, tmp_path / "c", optimizer=o, training_step=step)
    files = {f.name for f in (tmp_path / "c").iterdir()}
    assert {"model.safetensors", "optimizer.safetensors", "metadata.json", "gradient_accumulator.safetensors"} <= files
    assert meta["format"] == "cppmega_mlx_checkpoint_v1" and meta["version"] == 1 and meta["sharding"]["mode"] == "single_file"
    assert st.file_metadata(tmp_path / "c" / "model.safetensors") == {"format": "mlx"}
    names = set(meta["tensors"])
    assert "layers.1.block.experts.0.gate_proj.weight" in names and "layers.1.block.experts.3.down_proj.weight" in names
    assert "layers.1.block.shared_expert.up_proj.weight" in names
    assert not any("w_gate_up" in n or "gate_up_proj" in n for n in names)
    assert meta["model_config"]["pattern"] == m.config.pattern
    assert meta["rng"]["mode"] == "snapshot" and meta["training_state"]["gradient_accumulator"]["present"]


def test_name_mapping_is_invertible():
    m, _, _ = _setup()
    w = {n: p.detach() for n, p in m.named_parameters()}
    back = ck.from_reference_names(ck.to_reference_names(w), {n: p.shape for n, p in w.items()})
    assert all(torch.equal(back[n], w[n]) for n in w)


@pytest.mark.parametrize("opt", ["muon", "adamw"])
def test_resume_equals_uninterrupted(tmp_path, opt):
    m, o, step = _setup(opt=opt)
    bs = _batches(m, 12)
    losses = []
    for i, b in enumerate(bs):
        if i == 5:  # odd micro-step: saved in the middle of an accumulation window
            ck.save_checkpoint(m, tmp_path / "c", optimizer=o, training_step=step, metadata={"batch_cursor": {"offset": i}})
        losses.append(step(b).loss)
    m2, o2, step2 = _setup(seed=9, opt=opt)
    meta = ck.load_checkpoint(m2, tmp_path / "c", optimizer=o2, training_step=step2)
    assert meta["batch_cursor"]["offset"] == 5 and step2.state.micro_step == 5
    resumed = [step2(b).loss for b in bs[5:]]
    assert resumed == losses[5:]
    for (n, p), (_, q) in zip(m.named_parameters(), m2.named_parameters()):
        assert torch.equal(p, q), n


def test_validation_happens_before_mutation(tmp_path):
    m, o, step = _setup()
    step(_batches(m, 1)[0])
    ck.save_checkpoint(m, tmp_path / "c", optimizer=o, training_step=step)
    mp = tmp_path / "c" / "metadata.json"
    good = json.loads(mp.read_text())
    m2, o2, _ = _setup(seed=4)
    before = {n: p.clone() for n, p in m2.named_parameters()}

    def expect_fail(mutate):
        bad = json.loads(json.dumps(good))
        mutate(bad)
        mp.write_text(json.dumps(bad))
        with pytest.raises(ck.CheckpointError):
            ck.load_checkpoint(m2, tmp_path / "c", optimizer=o2)
        assert all(torch.equal(before[n], p) for n, p in m2.named_parameters())

    expect_fail(lambda d: d.update(format="other"))
    expect_fail(lambda d: d.update(version=7))
    expect_fail(lambda d: d.update(tp_rank=0))
    expect_fail(lambda d: d["optimizer"].update(parallel_state={"x": 1}))
    expect_fail(lambda d: d.update(num_tensors=3))
    expect_fail(lambda d: d["rng"].update(mode="weird"))
    expect_fail(lambda d: d["sharding"].update(mode="zero3"))
    expect_fail(lambda d: d.update(weights="nope.safetensors"))
    expect_fail(lambda d: d.update(tensors=d["tensors"][:-1], num_tensors=d["num_tensors"] - 1))
    mp.write_text("{not json")
    with pytest.raises(ck.CheckpointError):
        ck.load_checkpoint(m2, tmp_path / "c")
    mp.unlink()
    with pytest.raises(ck.CheckpointError):
        ck.load_checkpoint(m2, tmp_path / "c")


def test_shape_mismatch_and_missing_optimizer(tmp_path):
    m, o, _ = _setup()
    ck.save_checkpoint(m, tmp_path / "w.safetensors")
    assert (tmp_path / "w.json").exists()
    m2 = build_local_gb10_quarter_tiny_smoke_model()
    ck.load_checkpoint(m2, tmp_path / "w.safetensors")
    assert all(torch.equal(p, q) for p, q in zip(m.parameters(), m2.parameters()))
    with pytest.raises(ck.CheckpointError):
        ck.load_checkpoint(m2, tmp_path / "w.safetensors", optimizer=o)
    m3 = build_local_gb10_quarter_tiny_smoke_model(vocab_size=96)
    with pytest.raises(ck.CheckpointError):
        ck.load_checkpoint(m3, tmp_path / "w.safetensors")


def test_indexed_shards_and_latest(tmp_path):
    m, o, step = _setup()
    meta = ck.save_checkpoint(m, tmp_path / "step_3", max_shard_bytes=40_000)
    assert meta["sharding"]["mode"] == "indexed" and len(meta["sharding"]["files"]) > 1
    assert (tmp_path / "step_3" / ck.SHARD_INDEX_NAME).exists()
    (tmp_path / "step_9").mkdir()  # incomplete: no metadata.json
    assert ck.latest_checkpoint(tmp_path).name == "step_3"
    m2 = build_local_gb10_quarter_tiny_smoke_model()
    ck.load_checkpoint(m2, tmp_path / "step_3")
    assert all(torch.equal(p, q) for p, q in zip(m.parameters(), m2.parameters()))
