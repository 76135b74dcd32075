"""Hybrid LM end to end on CPU: every route gets gradients, training reduces the loss, config round trips, MTP / STP losses,
optimizers (Muon split, 8-bit state), quantizers, MoE dispatch vs dense reference."""
import math

import pytest
import torch

from cppmega_mlx_b200.data.batch import synthetic_token_batch
from cppmega_mlx_b200.models.hybrid_lm import HybridTinyConfig, HybridTinyLM
from cppmega_mlx_b200.recipes import model_factory as mf
from cppmega_mlx_b200.recipes.pattern import expand_nam_pattern, expand_symbols, parse_rank_list
from cppmega_mlx_b200.training import loss as L
from cppmega_mlx_b200.training import mtp
from cppmega_mlx_b200.training.compiled import PretrainingStep
from cppmega_mlx_b200.training.loop import one_step_train
from cppmega_mlx_b200.training.optimizers import (is_muon_compatible, make_adamw, make_lion, make_muon, newton_schulz5,
                                                  split_param_groups)
from cppmega_mlx_b200.training.optimizers_quantized import make_adam8bit, make_lion8bit
from cppmega_mlx_b200.training._quantize_8bit import dequantize_blockwise, quantize_blockwise


def _tiny(**kw):
    torch.manual_seed(0)
    return mf.build_local_gb10_quarter_tiny_smoke_model(**kw)


def test_pattern_expansion():
    assert expand_symbols("AEMR", 6) == ("A", "E", "M", "R", "A", "E")
    ex = expand_nam_pattern("AEMEAEMEAEMR", 13, dsa_a_layer_ranks=(1, 3))
    routes = [l.attention_route for l in ex.layers if l.symbol == "A"]
    assert routes.count("dsa") == 2 and len(routes) == 4
    assert parse_rank_list("1, 2,5") == (1, 2, 5)
    with pytest.raises(ValueError):
        expand_symbols("AXQ", 3)


def test_profiles_and_parameter_counts():
    assert set(mf.list_model_profiles()) >= {"local_gb10_quarter", "nam56r_full", "hybrid_1b", "moe_hybrid_ep8"}
    p = mf.get_model_profile("local_gb10_quarter")
    assert p.pattern == "AEMEAEMEAEMR" and p.depth == 13 and p.hidden_size == 3584
    with pytest.raises((KeyError, ValueError)):
        mf.get_model_profile("nope")


def test_config_yaml_round_trip_and_validation():
    cfg = _tiny().config
    again = HybridTinyConfig.from_yaml(cfg.to_yaml())
    assert again == cfg
    with pytest.raises((ValueError, TypeError)):
        HybridTinyConfig.from_dict({**cfg.to_dict(), "bogus_field": 1})
    with pytest.raises(ValueError):
        HybridTinyConfig(**{**cfg.to_dict(), "hidden_size": 0})


def test_every_route_receives_gradients_and_moves():
    m = _tiny()
    b = synthetic_token_batch(2, 16, vocab_size=m.config.vocab_size, seed=1)
    before = {n: p.detach().clone() for n, p in m.named_parameters()}
    opt = make_adamw(m, learning_rate=1e-2)
    out = one_step_train(m, opt, b)
    assert math.isfinite(float(out.loss))
    moved = {n for n, p in m.named_parameters() if not torch.equal(p, before[n])}
    for sentinel in ("layers.0.block.q_proj.weight", "layers.1.block.experts.w_gate_up", "layers.1.block.router.gate.weight",
                     "layers.2.block.in_proj.weight", "layers.2.block.D", "layers.4.block.sparse_kv_proj.weight",
                     "layers.11.block.state_weight", "token_embedding.weight", "lm_head.weight", "mtp_head.proj.weight"):
        assert sentinel in moved, sentinel


def test_training_reduces_loss_fp32_two_optimizers():
    for make in (lambda m: make_adamw(m, learning_rate=3e-3), lambda m: make_muon(m, lr_muon=2e-2, lr_adamw=3e-3)):
        m = _tiny()
        step = PretrainingStep(m, make(m))
        b = synthetic_token_batch(4, 24, vocab_size=m.config.vocab_size, seed=2)
        losses = [step(b).loss for _ in range(8)]
        assert all(math.isfinite(x) for x in losses) and losses[-1] < losses[0] - 0.05, losses


def test_grad_accumulation_equals_big_batch():
    m1, m2 = _tiny(), _tiny()
    big = synthetic_token_batch(4, 16, vocab_size=m1.config.vocab_size, seed=3)
    from cppmega_mlx_b200.data.batch import LMTokenBatch
    halves = [LMTokenBatch(tokens=big.tokens[:2]), LMTokenBatch(tokens=big.tokens[2:])]
    lf = L.make_loss_fn(backend="cross_entropy", mtp=False)
    from cppmega_mlx_b200.training.optimizers import Optimizer

    class SGD(Optimizer):     # Adam's first step is ~lr·sign(g): too sensitive to rounding for an equality test
        def init_single(self, name, p):
            return {}

        def apply_single(self, name, grad, p, st):
            p.add_(grad, alpha=-self.lr)
    s1 = PretrainingStep(m1, SGD(m1, 0.1), loss_fn=lf)
    s2 = PretrainingStep(m2, SGD(m2, 0.1), loss_fn=lf, grad_accum_steps=2)
    s1(big)
    r = [s2(h) for h in halves]
    assert not r[0].applied_update and r[1].applied_update
    for (n, p), (_, q) in zip(m1.named_parameters(), m2.named_parameters()):
        if "router" in n or "experts" in n:
            continue  # aux-loss normalisation is per micro-batch
        assert torch.allclose(p, q, atol=2e-5), n


def test_signature_check_and_document_mask():
    m = _tiny()
    step = PretrainingStep(m, make_adamw(m))
    step(synthetic_token_batch(2, 16, vocab_size=m.config.vocab_size, seed=1))
    with pytest.raises(ValueError):
        step(synthetic_token_batch(2, 12, vocab_size=m.config.vocab_size, seed=1))
    ids = torch.randint(4, 100, (1, 12))
    docs = torch.tensor([[0] * 6 + [1] * 6])
    m.eval()
    with torch.no_grad():
        full = m(ids, document_ids=docs)
        second = m(ids[:, 6:])
    # attention cannot look across the document boundary, but recurrent mixers / learned positions do carry over, so only
    # check that the masked forward runs and differs from the unmasked one
    assert full.shape == (1, 12, m.config.vocab_size) and second.shape[1] == 6
    assert not torch.allclose(full, m(ids))


def test_cce_loss_equals_materialised_loss():
    m = _tiny()
    b = synthetic_token_batch(2, 16, vocab_size=m.config.vocab_size, seed=4)
    a = L.make_loss_fn(backend="cce", mtp=False)(m, b)
    c = L.make_loss_fn(backend="cross_entropy", mtp=False)(m, b)
    assert torch.allclose(a.loss, c.loss, atol=1e-5) and int(a.ntokens) == int(c.ntokens)


def test_mtp_weights_roll_and_stop_gradient():
    w = mtp.compute_mtp_step_weights(3, 0.5)
    assert torch.allclose(w, torch.tensor([1.0, 0.5, 0.25]) / 1.75)
    t = torch.arange(1, 7)[None]
    lab = mtp.roll_and_mask_mtp_labels(t, depth=2)
    assert lab[0][0].tolist() == [2, 3, 4, 5, 6, -1] and lab[1][0].tolist() == [3, 4, 5, 6, -1, -1]
    docs = torch.tensor([[0, 0, 0, 1, 1, 1]])
    lab_d = mtp.roll_and_mask_mtp_labels(t, depth=1, document_ids=docs)
    assert lab_d[0][0].tolist() == [2, 3, -1, 5, 6, -1]
    m = _tiny()
    b = synthetic_token_batch(2, 16, vocab_size=m.config.vocab_size, seed=5)
    out = L.make_loss_fn(backend="cross_entropy", mtp=True)(m, b)
    assert "mtp_loss" in out.components or any("mtp" in k for k in out.components)
    m.zero_grad()
    hidden = m.decoder_hidden_states(b.inputs)
    m.mtp_head.loss(hidden, b.inputs)[0].backward()
    assert m.lm_head.weight.grad is None or float(m.lm_head.weight.grad.abs().max()) == 0.0   # stopped lm_head weight
    assert m.mtp_head.proj.weight.grad is not None


def test_stp_loss_range():
    from cppmega_mlx_b200.training.stp_loss import compute_stp_loss
    h = torch.randn(2, 32, 8, requires_grad=True)
    v = compute_stp_loss(h)
    v = v[0] if isinstance(v, tuple) else v
    assert 0.0 <= float(v) <= 2.0
    v.backward()
    assert h.grad is not None
    line = torch.arange(32.0)[None, :, None] * torch.ones(1, 1, 8)
    s = compute_stp_loss(line)
    s = s[0] if isinstance(s, tuple) else s
    assert float(s) < 1e-5          # straight trajectory → zero curvature penalty


def test_adamw_bias_correction_matches_torch_adamw():
    from cppmega_mlx_b200.training.optimizers import make_adamw
    torch.manual_seed(0)
    w0 = torch.randn(40, 30) * 0.1
    mine = [("w", torch.nn.Parameter(w0.clone()))]
    theirs = torch.nn.Parameter(w0.clone())
    opt = make_adamw(mine, learning_rate=1e-2, weight_decay=0.1, bias_correction=True)
    ref = torch.optim.AdamW([theirs], lr=1e-2, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.1)
    for _ in range(4):
        g = torch.randn(40, 30) * 0.01
        mine[0][1].grad, theirs.grad = g.clone(), g.clone()
        opt.step()
        ref.step()
    assert torch.allclose(mine[0][1], theirs, atol=1e-6, rtol=1e-5)


def test_muon_split_and_newton_schulz():
    m = _tiny()
    muon, other = split_param_groups(m)
    mn, on = {n for n, _ in muon}, {n for n, _ in other}
    assert "layers.0.block.q_proj.weight" in mn and "token_embedding.weight" in on and "lm_head.weight" in on
    assert "layers.2.block.D" in on and not (mn & on)
    assert not is_muon_compatible("layers.2.block.dt_bias", torch.zeros(8))
    g = torch.randn(24, 10)
    o = newton_schulz5(g)
    sv = torch.linalg.svdvals(o)
    assert float(sv.max()) < 1.3 and float(sv.min()) > 0.5          # NS-5 pushes singular values towards 1
    assert newton_schulz5(g.t()).shape == (10, 24)
    b16 = newton_schulz5(g, ns_carrier="bf16")
    assert torch.allclose(b16.float(), o, atol=0.1)


@pytest.mark.parametrize("scheme", ["symmetric_int8_v1", "dynamic_int8_v1"])
def test_blockwise_quantizers(scheme):
    x = torch.randn(1000) * 3
    try:
        q, absmax = quantize_blockwise(x, scheme=scheme)
    except ValueError:
        pytest.skip(f"scheme {scheme} not registered under this name")
    assert q.dtype == torch.uint8 and absmax.numel() == 4
    back = dequantize_blockwise(q, absmax, numel=1000, scheme=scheme)
    err = (back - x).abs().max() / x.abs().max()
    assert float(err) < (0.01 if "symmetric" in scheme else 0.05)
    assert float(dequantize_blockwise(*quantize_blockwise(torch.zeros(300), scheme=scheme), numel=300, scheme=scheme).abs().max()) == 0.0


def test_8bit_optimizers_track_fp32_and_shrink_state():
    torch.manual_seed(1)
    w0 = torch.randn(64, 128)
    tgt = torch.randn(64, 128)

    def run(make, steps=30):
        p = torch.nn.Parameter(w0.clone())
        opt = make([("w", p)])
        for _ in range(steps):
            p.grad = (p.detach() - tgt)
            opt.step()
        return p.detach(), opt
    a32, o32 = run(lambda ps: make_adamw(ps, learning_rate=1e-2, weight_decay=0.0))
    a8, o8 = run(lambda ps: make_adam8bit(ps, learning_rate=1e-2, min_8bit_size=0))
    d0 = float((w0 - tgt).norm())
    # linear int8 loses the small entries of v, so the symmetric scheme takes larger steps than fp32 Adam: check descent
    assert float((a8 - tgt).norm()) < 0.9 * d0 and float((a32 - tgt).norm()) < d0
    ad, _ = run(lambda ps: make_adam8bit(ps, learning_rate=1e-2, quant_scheme="dynamic_int8_v1"))
    assert float((ad - tgt).norm()) < 0.9 * d0
    assert o8.state_bytes() < 0.3 * o32.state_bytes()
    l32, _ = run(lambda ps: make_lion(ps, learning_rate=1e-3))
    l8, ol8 = run(lambda ps: make_lion8bit(ps, learning_rate=1e-3))
    assert float((l32 - l8).abs().max()) < 0.02
    st = o8.state["w"]
    assert {"m_quant", "m_absmax", "v_quant", "v_absmax"} <= set(st)
    small, osm = run(lambda ps: make_adam8bit(ps, learning_rate=1e-2, min_8bit_size=10 ** 9), steps=2)
    assert "m_quant" not in osm.state["w"]                          # fp32 escape for small tensors


def test_moe_sorted_dispatch_equals_dense_reference_and_bias_update():
    from cppmega_mlx_b200.nn.moe import MoE, MoEConfig
    torch.manual_seed(2)
    for scoring, alf in (("softmax", False), ("sigmoid", True), ("sqrtsoftplus", True)):
        cfg = MoEConfig(d_model=16, num_experts=6, top_k=2, expert_hidden_size=8, shared_expert_hidden_size=8, scoring=scoring,
                        aux_loss_free=alf)
        moe = MoE(cfg)
        x = torch.randn(3, 7, 16)
        out = moe(x)
        assert torch.allclose(out.output, moe.dense_reference_forward(x), atol=1e-5), scoring
        assert out.router.top_indices.shape == (3, 7, 2)
        if alf:
            b0 = moe.router.expert_bias.clone()
            moe.update_bias_after_step(out.router.load)
            assert not torch.equal(b0, moe.router.expert_bias)
            # the bias only changes *selection*: gate weights come from the raw scores
            moe.router.expert_bias.fill_(0.0)
            w_a = moe(x).router.top_weights
            assert torch.isfinite(w_a).all()


def test_external_trainer_adapter_probe_batch_mapping_and_refusal():
    import types
    from cppmega_mlx_b200.data.batch import LMTokenBatch
    from cppmega_mlx_b200.training import external_trainer_adapter as X
    # a stand-in trainer module: one API complete, one with a missing parameter, one absent
    fake = types.ModuleType("fake_trainer_mod")
    fake.__version__ = "0.0"
    fake.Trainer = lambda model, args, train_dataset, eval_dataset, data_collator: None
    fake.TrainingArguments = lambda per_device_train_batch_size, max_steps: None
    import sys
    sys.modules["fake_trainer_mod"] = fake
    try:
        info = X.describe_external_trainer_apis("fake_trainer_mod")
    finally:
        del sys.modules["fake_trainer_mod"]
    assert info.available and info.missing_apis == ("DataCollatorForLanguageModeling",) and info.incompatible_apis == ("TrainingArguments",)
    assert "train_dataset" in info.api_signatures["Trainer"] and not info.integration_supported
    assert not X.describe_external_trainer_apis("no_such_trainer_module_anywhere").available
    toks = torch.tensor([[5, 6, 7, 8], [9, 10, 0, 0]])
    mask = torch.tensor([[1, 1, 1, 1], [1, 1, 0, 0]])
    batch = LMTokenBatch(tokens=toks, attention_mask=mask, structure_ids=torch.zeros_like(toks), document_ids=torch.ones_like(toks))
    dense = X.as_dense_trainer_batch(batch)
    assert tuple(dense) == X.DENSE_BATCH_KEYS and torch.equal(dense["input_ids"], toks)
    assert dense["labels"][1].tolist() == [9, 10, -100, -100] and torch.equal(dense["attention_mask"], mask)
    meta = X.describe_batch_route_metadata(batch)
    assert meta.dropped == ("structure_ids", "document_ids") and meta.has_attention_mask and (meta.batch_size, meta.seq_len) == (2, 4)
    with pytest.raises(X.ExternalTrainerIntegrationUnsupported, match="unsupported"):
        X.require_supported_external_trainer_integration(info)
    with pytest.raises(ValueError):
        X.as_dense_trainer_batch({"tokens": torch.tensor([[1, -2, 3]])})


def test_no_grad_forward_with_deferred_residual_adds_equals_the_plain_forward():
    """Without gradients every residual add is handed to the next norm (one fused launch on the GPU); the result must be the
    stack's ordinary output, for blocks with and without an FFN and for the final norm."""
    from cppmega_mlx_b200 import ops
    torch.manual_seed(0)
    for kw in ({}, {"ffn_hidden_size": 48}):
        model = _tiny(**kw).eval()
        ids = torch.randint(0, model.config.vocab_size, (2, 12))
        with torch.enable_grad():
            ref = model(ids)
        with torch.no_grad():
            got = model(ids)
        ref = ref[0] if isinstance(ref, tuple) else ref
        got = got[0] if isinstance(got, tuple) else got
        assert torch.allclose(got, ref.detach(), atol=1e-5, rtol=1e-5)
    h, d, w = torch.randn(3, 16), torch.randn(3, 16), torch.rand(16) + 0.5
    with torch.no_grad():
        s, y = ops.add_rms_norm(h, d, w, 1e-5)
    assert torch.equal(s, h + d) and torch.allclose(y, ops.rms_norm_ref(h + d, w, 1e-5))
