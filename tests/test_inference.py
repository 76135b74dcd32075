"""Inference: caches, generation loops, sampling, infilling, speculative acceptance, quantisation, paged serving."""
import pytest
import torch

from cppmega_mlx_b200 import inference as I
from cppmega_mlx_b200.inference import quantization as Q
from cppmega_mlx_b200.inference import speculative_decode as SD
from cppmega_mlx_b200.inference.serving import OutOfBlocks
from cppmega_mlx_b200.recipes.model_factory import build_local_gb10_quarter_tiny_smoke_model


def _model(pattern="AEMR", **kw):
    torch.manual_seed(0)
    kw.setdefault("dsa_a_layer_ranks", ())
    return build_local_gb10_quarter_tiny_smoke_model(pattern=pattern, depth=len(pattern), **kw).eval()


def test_kv_cache_positions_trim_rollback_clone_fp8():
    c = I.HybridKVCache(2)
    k, v = torch.randn(1, 5, 2, 4), torch.randn(1, 5, 2, 4)
    kk, vv = c.update_and_fetch(0, k, v)
    assert torch.equal(kk, k) and c.position(0) == 5 and c.position(1) == 0 and c.offset == 5
    c.update_and_fetch(1, k, v)
    k2 = torch.randn(1, 1, 2, 4)
    kk, _ = c.update_and_fetch(0, k2, k2)
    assert kk.shape[1] == 6 and torch.equal(kk[:, 5:], k2)
    with pytest.raises(ValueError):
        c.rollback(6)                      # layer 1 is only at 5: strict
    c.rollback(5)
    assert c.position(0) == 5
    d = c.clone()
    d.update_and_fetch(0, k2, k2)
    assert c.position(0) == 5 and d.position(0) == 6
    assert c.trim(2) == 2 and c.position(1) == 3
    c.expand_batch(3)
    assert c.a[0].buf.shape[0] == 3
    f = I.HybridKVCache(1, quantize="fp8")
    lat, _ = f.update_and_fetch_latent(0, torch.randn(2, 7, 16), None)
    lat2, _ = f.update_and_fetch_latent(0, torch.randn(2, 1, 16), None)
    assert lat2.shape == (2, 8, 16) and torch.allclose(lat2[:, :7], lat, atol=0) and f.nbytes() < 2 * 256 * 16 * 4


@pytest.mark.parametrize("pattern,kw", [("AE", {}), ("A", {"dsa_a_layer_ranks": (0,)}), ("M", {}), ("R", {}),
                                        ("A", {"mla_low_rank": True, "dsa_a_layer_ranks": (0,)})])
def test_incremental_decode_equals_full_recompute(pattern, kw):
    m = _model(pattern, **kw)
    ids = torch.randint(4, 100, (2, 14))
    with torch.no_grad():
        s = I.DecodeSession(m)
        got = [s.forward(ids[:, :8])[:, -1]] + [s.forward(ids[:, i:i + 1])[:, -1] for i in range(8, 14)]
        want = [m(ids[:, :n])[:, -1] for n in range(8, 15)]
    for g, w in zip(got, want):
        assert torch.allclose(g, w, atol=2e-5)


def test_generation_paths_agree_and_stream():
    m = _model("AEAR")
    p = torch.randint(4, 100, (2, 9))
    a = I.generate_tokens(m, p, max_new_tokens=5)
    b = I.generate_tokens_with_kv_cache(m, p, max_new_tokens=5)
    assert torch.equal(a, b) and a.shape == (2, 14)
    chunks = list(I.stream_generate_tokens(m, p, max_new_tokens=5))
    assert len(chunks) == 5 and chunks[0].position == 9 and torch.equal(torch.stack([c.token_ids for c in chunks], 1), a[:, 9:])
    stop = int(a[0, 10])
    e = I.generate_tokens_with_kv_cache(m, p[:1], max_new_tokens=5, eos_token_id=stop)
    first = a[0, 9:].tolist().index(stop)
    assert e.shape[1] == 9 + first + 1 and int(e[0, -1]) == stop
    assert m.training is False
    with pytest.raises(ValueError):
        I.generate_tokens(m, torch.zeros(1, 0, dtype=torch.long), max_new_tokens=1)

    class Tup(torch.nn.Module):
        def forward(self, x):
            return (torch.zeros(1, 1, 3), None)
    with pytest.raises(TypeError):
        I.next_token_logits(Tup(), p)


def test_prompt_cache_reuse():
    m = _model("AEMR")
    prefix, rest = list(range(10, 18)), [30, 31, 32]
    entry = I.build_prompt_cache(m, prefix)
    out = I.generate_from_prompt_cache(m, entry, prefix + rest, max_new_tokens=4)
    ref = I.generate_tokens_with_kv_cache(m, prefix + rest, max_new_tokens=4)
    assert out.shape == ref.shape == (1, 15) and entry.hits == 1
    again = I.generate_from_prompt_cache(m, entry, prefix + rest, max_new_tokens=4)      # the entry itself is not consumed
    assert torch.equal(out, again)
    with pytest.raises(ValueError):
        I.generate_from_prompt_cache(m, entry, [1, 2, 3], max_new_tokens=1)


def test_engram_models_fall_back_to_full_recompute():
    m = _model("AN")
    assert not I.supports_incremental_decode(m)
    with pytest.raises(ValueError):
        I.DecodeSession(m)
    p = torch.randint(4, 100, (1, 6))
    assert torch.equal(I.generate_tokens_with_kv_cache(m, p, max_new_tokens=3), I.generate_tokens(m, p, max_new_tokens=3))


def test_sampling_rules():
    logits = torch.tensor([[1.0, 3.0, 2.0, -1.0]])
    assert I.sample_next_token(logits, temperature=0).tolist() == [1]
    assert torch.isinf(I.apply_top_k(logits, 2)[0, [0, 3]]).all()
    tp = I.apply_top_p(logits, 0.5)
    assert torch.isfinite(tp[0, 1]) and torch.isinf(tp[0, [0, 2, 3]]).all()      # the top token always stays
    assert torch.isfinite(I.apply_top_p(logits, 1e-9)[0, 1])
    g = torch.Generator().manual_seed(0)
    draws = torch.stack([I.sample_next_token(logits.expand(2000, 4), temperature=1.0, generator=g)])
    freq = torch.bincount(draws.flatten(), minlength=4).float() / 2000
    assert torch.allclose(freq, torch.softmax(logits[0], -1), atol=0.04)
    only = I.sample_next_token(logits.expand(200, 4), temperature=1.0, top_k=1, generator=g)
    assert (only == 1).all()
    with pytest.raises(ValueError):
        I.sample_next_token(logits, temperature=-1)


def test_infilling_prompt():
    p = I.build_infilling_prompt([10, 11], [20], mode="psm")
    assert p == [4, 10, 11, 6, 20, 5]
    s = I.build_infilling_prompt([10, 11], [20], mode="spm", instruction_ids=[60])
    assert s == [45, 60, 6, 20, 4, 10, 11, 5]
    with pytest.raises(ValueError):
        I.build_infilling_prompt([4], [20])
    assert I.splice_infill([1], [7, 8, 3, 9], [2]) == [1, 7, 8, 2]


def test_leviathan_acceptance_matches_target_distribution():
    g = torch.Generator().manual_seed(1)
    pd = torch.tensor([[0.7, 0.2, 0.1]])
    pt = torch.tensor([[0.2, 0.5, 0.3], [1 / 3, 1 / 3, 1 / 3]])
    counts = torch.zeros(3)
    acc = 0
    n = 6000
    for _ in range(n):
        x = torch.multinomial(pd[0], 1, generator=g)
        r = SD.leviathan_accept(x, pd, pt, generator=g)
        counts[int(r.tokens[0])] += 1
        acc += r.num_accepted
    assert torch.allclose(counts / n, pt[0], atol=0.03)          # first emitted token is distributed as the target
    assert abs(acc / n - (0.2 + 0.2 + 0.1)) < 0.03                # Σ min(p_t, p_d)
    same = SD.leviathan_accept(torch.tensor([1, 2]), torch.tensor([[0, 1.0, 0], [0, 0, 1.0]]),
                               torch.tensor([[0, 1.0, 0], [0, 0, 1.0], [1.0, 0, 0]]), generator=g)
    assert same.all_accepted and same.tokens.tolist() == [1, 2, 0]
    t = SD.typical_accept(torch.tensor([0, 2]), torch.tensor([[0.6, 0.3, 0.1], [0.8, 0.15, 0.05], [1.0, 0, 0]]), generator=g)
    assert t.num_accepted == 1 and not t.all_accepted
    toks, cnt = SD.batched_leviathan_accept(torch.tensor([[1, 2], [0, 0]]), torch.tensor([[[0, 1.0, 0], [0, 0, 1.0]]] * 2),
                                            torch.tensor([[[0, 1.0, 0], [0, 0, 1.0], [1.0, 0, 0]]] * 2), generator=g)
    assert cnt.tolist() == [2, 0] and toks[1, 1:].tolist() == [-1, -1]


def test_speculative_generate_greedy_equals_target_greedy():
    target, draft = _model("AEMR"), _model("AR", hidden_size=64)
    prompt = list(range(10, 19))
    ref = I.generate_tokens_with_kv_cache(target, prompt, max_new_tokens=8)
    out, stats = I.speculative_generate(target, draft, prompt, max_new_tokens=8, num_draft=3, temperature=0.0)
    assert torch.equal(out, ref)                                  # rollback restores SSM / RNN state exactly
    self_out, self_stats = I.speculative_generate(target, target, prompt, max_new_tokens=8, num_draft=3, temperature=0.0)
    assert torch.equal(self_out, ref) and self_stats["acceptance_rate"] == 1.0


def test_weight_quantisation():
    w = torch.randn(8, 128)
    p, s, b = Q.quantize_affine(w)
    assert p.shape == (8, 64) and s.shape == (8, 2)
    assert float((Q.dequantize_affine(p, s, b) - w).abs().max()) < float(w.abs().max()) / 7
    m = _model("AE", hidden_size=128)
    x = torch.randint(4, 100, (1, 8))
    with torch.no_grad():
        before = m(x)
        rep = Q.quantize_model_linears(m)
        after = m(x)
    assert rep.quantized and all("lm_head" not in n and "token_embedding" not in n for n in rep.quantized)
    assert rep.bytes_after < 0.2 * rep.bytes_before
    assert float((before - after).abs().mean()) < 0.1
    assert Q.kv_quantization_for_length(100) is None and Q.kv_quantization_for_length(256) == "fp8"


def test_block_manager_and_paged_attention():
    mgr = I.PagedKVBlockManager(num_blocks=8, num_layers=2, block_size=4, kv_heads=2, head_dim=8, dtype=torch.float32)
    assert mgr.allocate(7, 6) == [0, 1] and mgr.num_free_blocks == 6
    ks, vs = torch.randn(6, 2, 8), torch.randn(6, 2, 8)
    mgr.append(7, 0, ks, vs, advance=False)
    mgr.append(7, 1, ks * 2, vs * 2)
    mgr.allocate(9, 3)
    k9, v9 = torch.randn(3, 2, 8), torch.randn(3, 2, 8)
    mgr.append(9, 1, k9, v9)
    g = mgr.gather(7, 1)
    assert torch.equal(g[0], ks * 2)
    table, lens = I.build_paged_block_table(mgr, [7, 9])
    assert table.tolist() == [[0, 1], [2, -1]] and lens.tolist() == [6, 3]
    q = torch.randn(2, 4, 8)
    out = I.paged_decode_attention(q, mgr, 1, table, lens)
    for i, (kk, vv) in enumerate(((ks * 2, vs * 2), (k9, v9))):
        kx, vx = kk.repeat_interleave(2, 1), vv.repeat_interleave(2, 1)            # GQA: 4 q heads over 2 kv heads
        ref = torch.einsum("hk,khv->hv", torch.softmax(torch.einsum("hd,khd->hk", q[i], kx) * 8 ** -0.5, -1), vx)
        assert torch.allclose(out[i], ref, atol=1e-5)
    mgr.free(7)
    assert mgr.allocate(11, 1) == [0]                                              # LIFO reuse
    with pytest.raises(OutOfBlocks):
        mgr.allocate(12, 100)
    lat = I.PagedKVBlockManager(num_blocks=4, num_layers=1, block_size=4, kv_heads=1, head_dim=12, dtype=torch.float32)
    lat.allocate(0, 7)
    rows = torch.randn(7, 1, 12)
    lat.append(0, 0, rows, rows)
    t, l = I.build_paged_block_table(lat, [0])
    ql = torch.randn(1, 3, 12)
    idx = torch.tensor([[6, 2, 0, -1]])
    o = I.paged_latent_decode_attention(ql, lat, 0, t, l, d_v=8, scale=0.3, topk_idx=idx)
    sel = rows[[6, 2, 0], 0]
    ref = torch.softmax(ql[0] @ sel.t() * 0.3, -1) @ sel[:, :8]
    assert torch.allclose(o[0], ref, atol=1e-5)


def test_scheduler_priority_preemption_and_adapters():
    mgr = I.PagedKVBlockManager(num_blocks=6, num_layers=1, block_size=4, kv_heads=1, head_dim=4, dtype=torch.float32)
    sch = I.ContinuousBatchScheduler(mgr, max_batch_size=2)
    sch.add_request(1, prompt_len=7, max_new_tokens=6, priority=0)
    sch.add_request(2, prompt_len=7, max_new_tokens=6, priority=5)
    sch.add_request(3, prompt_len=3, max_new_tokens=2, priority=9, adapter_key="lora-a")
    st = sch.schedule()
    assert st.adapter_key == "lora-a" and st.prefill == [3]                      # highest priority picks the adapter group
    sch.complete_step(st)
    st = sch.schedule()
    assert st.decode == [3] and st.prefill == []                                   # other adapters wait for the group to drain
    sch.complete_step(st)
    assert sch.finished == [3]
    st = sch.schedule()
    assert st.prefill == [2, 1]                                                    # priority order
    sch.complete_step(st)
    seen_preempt = False
    for _ in range(40):
        if sch.idle():
            break
        st = sch.schedule()
        seen_preempt |= bool(st.preempted)
        if st.preempted:
            assert st.preempted == [1]                                             # lowest priority is the victim
        sch.complete_step(st)
    assert sch.idle() and seen_preempt and sorted(sch.finished) == [1, 2, 3]
    assert sch.requests[1].preemptions >= 1 and mgr.num_free_blocks == 6
    with pytest.raises(ValueError):
        sch.add_request(1, 1, 1)
    with pytest.raises(ValueError):
        sch.add_request(50, 1000, 1)
    fifo = I.ContinuousBatchScheduler(mgr, max_batch_size=1, policy="fifo")
    fifo.add_request(1, 2, 1, priority=0)
    fifo.add_request(2, 2, 1, priority=9)
    assert fifo.schedule().prefill == [1]


@pytest.mark.parametrize("pattern,kw", [("AE", {}), ("A", {"dsa_a_layer_ranks": (0,)}), ("MR", {}),
                                        ("A", {"mla_low_rank": True, "dsa_a_layer_ranks": (0,)}),
                                        ("AM", {"mla_low_rank": True})])
def test_static_cache_steps_equal_growing_cache_steps(pattern, kw):
    """The fixed-capacity, device-position step (the one a CUDA graph replays) produces the same logits as DecodeSession."""
    m = _model(pattern, **kw)
    ids = torch.randint(4, 100, (2, 15))
    with torch.no_grad():
        ref = I.DecodeSession(m)
        want = [ref.forward(ids[:, :9], last_only=True)[:, 0]] + [ref.forward(ids[:, i:i + 1])[:, 0] for i in range(9, 15)]
        g = I.GraphDecodeSession(m, capacity=32, use_graph=False)
        got = [g.prefill(ids[:, :9]).clone()] + [g.step(ids[:, i]).clone() for i in range(9, 15)]
    for a, b in zip(got, want):
        assert torch.allclose(a, b, atol=2e-5)
    assert g.cache.pos.tolist() == [15, 15] and g.tokens_seen == 15
    with pytest.raises(ValueError):
        I.GraphDecodeSession(m, capacity=8).prefill(ids[:, :9])
    out = I.GraphDecodeSession(m, capacity=32, use_graph=False).generate(ids[:, :9], 4)
    assert torch.equal(out, I.generate_tokens_with_kv_cache(m, ids[:, :9], max_new_tokens=4))


def test_graph_session_sampling_and_eos():
    m = _model("AM", mla_low_rank=True)
    ids = torch.randint(4, 100, (2, 9))
    g = torch.Generator().manual_seed(3)
    a = I.GraphDecodeSession(m, capacity=64, use_graph=False).generate(ids, 6, temperature=0.8, top_k=20, top_p=0.9, generator=g)
    g = torch.Generator().manual_seed(3)
    b = I.GraphDecodeSession(m, capacity=64, use_graph=False).generate(ids, 6, temperature=0.8, top_k=20, top_p=0.9, generator=g)
    assert a.shape == (2, 15) and torch.equal(a, b)
    greedy = I.GraphDecodeSession(m, capacity=64, use_graph=False).generate(ids, 6)
    eos = int(greedy[0, 10])
    c = I.GraphDecodeSession(m, capacity=64, use_graph=False).generate(ids, 6, eos_token_id=eos)
    assert torch.equal(c[0, :11], greedy[0, :11]) and bool((c[0, 11:] == eos).all())


@pytest.mark.parametrize("pattern,kw", [("AM", {"mla_low_rank": True, "dsa_a_layer_ranks": (0,)}), ("AER", {})])
def test_serving_engine_continuous_batching_matches_single_request_generation(pattern, kw):
    """Requests of different lengths join and leave two slots at different times; each gets exactly the tokens it would get
    alone (per-slot positions, recurrent state and cache rows never leak between requests)."""
    m = _model(pattern, **kw)
    torch.manual_seed(5)
    prompts = [torch.randint(4, 100, (n,)) for n in (5, 11, 3, 8, 6)]
    budgets = [6, 3, 7, 2, 5]
    eng = I.ServingEngine(m, max_batch=2, capacity=32, use_graph=False)
    ids = [eng.submit(p, b) for p, b in zip(prompts, budgets)]
    out = eng.run()
    assert eng.idle() and all(eng.requests[i].finish_reason == "length" for i in ids)
    for i, p, b in zip(ids, prompts, budgets):
        want = I.generate_tokens_with_kv_cache(m, p[None], max_new_tokens=b)[0, p.numel():].tolist()
        assert out[i] == want
    assert eng.steps < sum(budgets)                  # slots really were shared


def test_serving_engine_with_scheduler_preemption_and_eos():
    from cppmega_mlx_b200.inference.serving import ContinuousBatchScheduler, PagedKVBlockManager
    m = _model("AM")
    torch.manual_seed(6)
    prompts = [torch.randint(4, 100, (n,)) for n in (6, 7, 5)]
    alone = [I.generate_tokens_with_kv_cache(m, p[None], max_new_tokens=8)[0, p.numel():].tolist() for p in prompts]
    # 5 blocks of 4 tokens: not enough for all three to grow, so the scheduler must preempt and the engine must recompute
    mgr = PagedKVBlockManager(num_blocks=7, num_layers=1, block_size=4, kv_heads=1, head_dim=4)
    sch = ContinuousBatchScheduler(mgr, max_batch_size=3)
    eng = I.ServingEngine(m, max_batch=3, capacity=32, use_graph=False, scheduler=sch)
    ids = [eng.submit(p, 8, priority=pr) for p, pr in zip(prompts, (2, 1, 0))]
    out = eng.run(max_steps=200)
    assert eng.idle() and sch.idle()
    assert sum(sch.requests[i].preemptions for i in ids) >= 1
    for i, w in zip(ids, alone):
        assert out[i] == w
    # EOS retires a request early
    eos = alone[0][2]
    eng2 = I.ServingEngine(m, max_batch=2, capacity=32, use_graph=False, eos_token_id=eos)
    r = eng2.submit(prompts[0], 8)
    got = eng2.run()[r]
    assert got == alone[0][:alone[0].index(eos) + 1] and eng2.requests[r].finish_reason == "eos"


@pytest.mark.parametrize("pattern,kw", [("AM", {"mla_low_rank": True, "dsa_a_layer_ranks": (0,)}), ("AA", {})])
def test_serving_engine_paged_cache_with_preemption(pattern, kw):
    """Paged physical cache: attention reads through the page table, requests hold only the pages the block manager gave
    them, and a pool too small for everybody forces preemption + recompute — the tokens still equal single-request generation."""
    m = _model(pattern, **kw)
    torch.manual_seed(7)
    prompts = [torch.randint(4, 100, (n,)) for n in (6, 9, 5, 7)]
    alone = [I.generate_tokens_with_kv_cache(m, p[None], max_new_tokens=9)[0, p.numel():].tolist() for p in prompts]
    eng = I.ServingEngine(m, max_batch=3, capacity=32, use_graph=False, page_size=4, num_pages=10)
    ids = [eng.submit(p, 9, priority=pr) for p, pr in zip(prompts, (3, 2, 1, 0))]
    out = eng.run(max_steps=400)
    assert eng.idle() and isinstance(eng.cache, I.PagedDecodeCache)
    for i, w in zip(ids, alone):
        assert out[i] == w
    sch = eng.scheduler
    assert sum(sch.requests[i].preemptions for i in ids) >= 1                 # 9 usable pages of 4 tokens cannot hold them all
    assert sch.manager.num_free_blocks == sch.manager.num_blocks - 1          # everything returned except the scratch page


def test_paged_decode_cache_addressing_and_errors():
    c = I.PagedDecodeCache(1, 2, num_pages=6, page_size=4, max_pages_per_seq=3, device="cpu")
    assert c.capacity == 12 and c.table().shape == (2, 3)
    c.set_pages(0, [5, 2])
    c.set_pages(1, [1])
    kv = I.HybridKVCache(1)
    rows = torch.arange(6 * 3, dtype=torch.float32).view(1, 6, 3)
    kv.update_and_fetch_latent(0, rows, None)
    c.load_slot(0, kv, 6)                                           # 6 tokens → pages 5 (rows 0-3) and 2 (rows 0-1)
    pool = c.a[0]
    assert torch.equal(pool[5], rows[0, :4]) and torch.equal(pool[2, :2], rows[0, 4:6]) and c.pos.tolist() == [6, 0]
    new = torch.full((2, 1, 3), 7.0)
    c.write_a(0, new)                                               # slot 0 → page 2 row 2; slot 1 → page 1 row 0
    assert torch.equal(pool[2, 2], new[0, 0]) and torch.equal(pool[1, 0], new[1, 0])
    dense = c.dense_rows(pool)
    assert dense.shape == (2, 12, 3) and torch.equal(dense[0, :6], rows[0]) and torch.equal(dense[0, 6], new[0, 0])
    c.advance()
    assert c.pos.tolist() == [7, 1] and c.lengths().tolist() == [8, 2]
    c.active[1] = 0
    c.advance()
    assert c.pos.tolist() == [8, 1]                                 # an inactive row stays where it is
    with pytest.raises(ValueError):
        c.set_pages(0, [0, 1, 2, 3])                                # more pages than a sequence may hold
    with pytest.raises(ValueError):
        c.load_slot(1, kv, 6)                                       # one page published, two needed
    c.clear_pages(0, fill=4)
    assert c.table()[0].tolist() == [4, 4, 4]
    with pytest.raises(NotImplementedError):
        c.load_from(kv)
