"""Split-KV tcgen05 decode attention against the PyTorch fp32 oracle of the same op."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _pools(n_pages, page, kvh, d, dv=None, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    k = torch.randn(n_pages, page, kvh, d, device="cuda", generator=g).bfloat16()
    v = None if dv is None else torch.randn(n_pages, page, kvh, dv, device="cuda", generator=g).bfloat16()
    return k, v


def _check(out, ref):
    from cppmega_mlx_b200.ops import _backend as B
    B.check_status()
    err = (out.float() - ref.float()).abs().max().item()
    assert err <= 2e-2 * max(1.0, ref.float().abs().max().item()), err


@pytest.mark.parametrize("splits", [1, 3, None])
@pytest.mark.parametrize("heads", [16, 32, 8])
def test_latent_paged_dense(splits, heads):
    from cppmega_mlx_b200.ops import decode_attention as D
    torch.manual_seed(1)
    page, n_pages = 64, 40
    k, _ = _pools(n_pages, page, 1, 576)
    lengths = torch.tensor([100, 500, 1, 0], dtype=torch.int32, device="cuda")
    table = torch.randperm(n_pages, device="cuda").int()[:36].view(4, 9)
    q = torch.randn(4, heads, 576, device="cuda").bfloat16()
    out = D.decode_attention(q, k, None, table, lengths, scale=576 ** -0.5, d_v=512, splits=splits)
    ref = D.decode_attention_reference(q, k, None, table, lengths, scale=576 ** -0.5, d_v=512)
    assert out.shape == (4, heads, 512)
    _check(out, ref)
    assert float(out[3].float().abs().max()) == 0.0        # a sequence with no key yields zeros


def test_latent_paged_topk():
    from cppmega_mlx_b200.ops import decode_attention as D
    torch.manual_seed(2)
    page, n_pages = 32, 64
    k, _ = _pools(n_pages, page, 1, 576, seed=3)
    lengths = torch.tensor([1000, 333], dtype=torch.int32, device="cuda")
    table = torch.randperm(n_pages, device="cuda").int().view(2, 32)
    topk = torch.stack([torch.randperm(1024, device="cuda")[:200] for _ in range(2)]).int()   # some entries ≥ length: ignored
    topk[:, 150:] = -1
    q = torch.randn(2, 16, 576, device="cuda").bfloat16() * 3                                   # peaky softmax: exercises the re-referencing
    out = D.decode_attention(q, k, None, table, lengths, scale=576 ** -0.5, topk=topk, d_v=512, splits=2)
    ref = D.decode_attention_reference(q, k, None, table, lengths, scale=576 ** -0.5, topk=topk, d_v=512)
    _check(out, ref)


@pytest.mark.parametrize("dk,dv,kvh,h", [(128, 128, 4, 16), (192, 128, 2, 8), (128, 128, 1, 40)])
def test_gqa_paged_and_contiguous(dk, dv, kvh, h):
    from cppmega_mlx_b200.ops import decode_attention as D
    torch.manual_seed(4)
    page, n_pages = 16, 96
    k, v = _pools(n_pages, page, kvh, dk, dv, seed=5)
    lengths = torch.tensor([500, 17, 64], dtype=torch.int32, device="cuda")
    table = torch.randperm(n_pages, device="cuda").int().view(3, 32)
    q = torch.randn(3, h, dk, device="cuda").bfloat16()
    out = D.decode_attention(q, k, v, table, lengths, scale=dk ** -0.5)
    ref = D.decode_attention_reference(q, k, v, table, lengths, scale=dk ** -0.5)
    _check(out, ref)
    # contiguous cache [B, T, kvh, D], sliced from a larger allocation (non-trivial batch stride)
    kc = torch.randn(3, 600, kvh, dk, device="cuda").bfloat16()[:, :512]
    vc = torch.randn(3, 600, kvh, dv, device="cuda").bfloat16()[:, :512]
    out = D.decode_attention(q, kc, vc, None, lengths, scale=dk ** -0.5, splits=4)
    ref = D.decode_attention_reference(q, kc, vc, None, lengths, scale=dk ** -0.5)
    _check(out, ref)


def test_serving_paged_attention_uses_kernel():
    from cppmega_mlx_b200.inference.serving import PagedKVBlockManager, build_paged_block_table, paged_latent_decode_attention
    from cppmega_mlx_b200.ops import _backend as B
    from cppmega_mlx_b200.ops.decode_attention import decode_attention_reference
    torch.manual_seed(6)
    m = PagedKVBlockManager(num_blocks=32, num_layers=2, block_size=16, kv_heads=1, head_dim=576, device="cuda")
    for sid, n in ((7, 90), (9, 33)):
        m.allocate(sid, n)
        for layer in range(2):
            m.append(sid, layer, torch.randn(n, 1, 576, device="cuda").bfloat16(), torch.zeros(n, 1, 576, device="cuda").bfloat16(),
                     advance=layer == 1)
    table, lengths = build_paged_block_table(m, [7, 9])
    q = torch.randn(2, 16, 576, device="cuda").bfloat16()
    before = B.launch_count("paged_decode")
    out = paged_latent_decode_attention(q, m, 1, table, lengths, d_v=512, scale=576 ** -0.5)
    assert B.launch_count("paged_decode") == before + 1
    ref = decode_attention_reference(q, m.k_pool[:, 1], None, table, lengths, scale=576 ** -0.5, d_v=512)
    _check(out, ref)


@pytest.mark.parametrize("kw", [{"mla_low_rank": True, "dsa_a_layer_ranks": ()}, {"mla_low_rank": True, "dsa_a_layer_ranks": (0, 1)}])
def test_model_decode_steps_use_kernel_and_match_eager(kw):
    """One-token steps of a low-rank-MLA model go through the decode kernel and agree with the PyTorch path on the same cache."""
    from cppmega_mlx_b200 import inference as I
    from cppmega_mlx_b200.ops import _backend as B
    from cppmega_mlx_b200.recipes.model_factory import build_local_gb10_quarter_tiny_smoke_model
    torch.manual_seed(0)
    # latent rows of 512 + 64 columns: the geometry the decode kernel is built for (a toy latent width would legitimately
    # run the PyTorch path, and the launch counter below would say so)
    m = build_local_gb10_quarter_tiny_smoke_model(pattern="AA", depth=2, mla_kv_lora_rank=512, mla_qk_rope_head_dim=64,
                                                  dsa_indexer_head_dim=64, **kw).eval().cuda().bfloat16()
    ids = torch.randint(4, 100, (2, 40), device="cuda")
    with torch.no_grad():
        s = I.DecodeSession(m)
        s.forward(ids[:, :32])
        before = B.launch_count("paged_decode")
        got = [s.forward(ids[:, i:i + 1])[:, -1].float() for i in range(32, 40)]
        assert B.launch_count("paged_decode") >= before + 8 * 2      # one decode-attention launch per A layer per token
        with B.use_kernels(False):
            r = I.DecodeSession(m)
            r.forward(ids[:, :32])
            want = [r.forward(ids[:, i:i + 1])[:, -1].float() for i in range(32, 40)]
    B.check_status()
    for g, w in zip(got, want):
        assert (g - w).abs().max() < 0.08 * max(1.0, float(w.abs().max()))


def test_graph_replay_matches_eager_static_steps():
    """A captured step replayed from the CUDA graph gives the logits of the same static step launched eagerly."""
    from cppmega_mlx_b200 import inference as I
    from cppmega_mlx_b200.ops import _backend as B
    from cppmega_mlx_b200.recipes.model_factory import build_local_gb10_quarter_tiny_smoke_model
    torch.manual_seed(0)
    m = build_local_gb10_quarter_tiny_smoke_model(pattern="AMAR", depth=4, mla_low_rank=True, dsa_a_layer_ranks=(0,)).eval().cuda().bfloat16()
    ids = torch.randint(4, 100, (2, 30), device="cuda")
    with torch.no_grad():
        e = I.GraphDecodeSession(m, capacity=64, use_graph=False)
        want = [e.prefill(ids[:, :20]).float().clone()] + [e.step(ids[:, i]).float().clone() for i in range(20, 30)]
        g = I.GraphDecodeSession(m, capacity=64, use_graph=True)
        got = [g.prefill(ids[:, :20]).float().clone()] + [g.step(ids[:, i]).float().clone() for i in range(20, 30)]
    assert g.graph is not None
    B.check_status()
    for a, b in zip(got, want):
        assert (a - b).abs().max() <= 1e-2 * max(1.0, float(b.abs().max()))
    assert g.cache.pos.tolist() == [30, 30]
    out = I.GraphDecodeSession(m, capacity=64).generate(ids[:, :20], 6)
    assert out.shape == (2, 26)


@pytest.mark.parametrize("paged", [False, True])
def test_serving_engine_graph_replay_with_slot_turnover(paged):
    """Continuous batching on the GPU: the captured step serves a changing mix of requests; results equal the eager engine's."""
    from cppmega_mlx_b200 import inference as I
    from cppmega_mlx_b200.ops import _backend as B
    from cppmega_mlx_b200.recipes.model_factory import build_local_gb10_quarter_tiny_smoke_model
    torch.manual_seed(0)
    m = build_local_gb10_quarter_tiny_smoke_model(pattern="AMAR", depth=4, mla_low_rank=True, dsa_a_layer_ranks=(0,)).eval().cuda().bfloat16()
    prompts = [torch.randint(4, 100, (n,)) for n in (9, 17, 5, 12, 7)]
    budgets = [8, 4, 9, 3, 6]

    def serve(use_graph):
        kw = dict(page_size=16, num_pages=12) if paged else {}
        eng = I.ServingEngine(m, max_batch=2, capacity=64, use_graph=use_graph, **kw)
        ids = [eng.submit(p, b) for p, b in zip(prompts, budgets)]
        out = eng.run()
        return [out[i] for i in ids], eng
    want, _ = serve(False)
    got, eng = serve(True)
    B.check_status()
    assert eng.graphs and eng.idle()
    assert got == want and [len(g) for g in got] == budgets
