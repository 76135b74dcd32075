"""TP (+SP), EP and PP on CPU ranks (gloo): each must reproduce the single-process result."""
import pytest
import torch

from cppmega_mlx_b200.parallel import pp as PP
from cppmega_mlx_b200.parallel import state as PS
from tests._dist_util import run_ranks

pytestmark = pytest.mark.distributed


def test_group_layout_is_a_partition():
    lay = PS.group_ranks(8, tp=2, pp=2, ep=2)
    assert lay["tp"] == [[0, 1], [2, 3], [4, 5], [6, 7]]
    assert lay["dp"] == [[0, 2], [1, 3], [4, 6], [5, 7]]
    assert lay["pp"] == [[0, 4], [1, 5], [2, 6], [3, 7]]
    for kind in lay:
        flat = sorted(r for g in lay[kind] for r in g)
        assert flat == list(range(8)), kind
    assert PS.rank_coordinates(5, 8, 2, 2) == (1, 0, 1)
    with pytest.raises(ValueError):
        PS.group_ranks(8, tp=3, pp=1, ep=1)
    with pytest.raises(ValueError):
        PS.group_ranks(8, tp=2, pp=2, ep=3)
    assert PP.split_layers(7, 3) == [range(0, 3), range(3, 5), range(5, 7)]
    assert PP.one_f_one_b_order(0, 2, 3) == [("F", 0), ("F", 1), ("B", 0), ("F", 2), ("B", 1), ("B", 2)]
    assert PP.one_f_one_b_order(1, 2, 3) == [("F", 0), ("B", 0), ("F", 1), ("B", 1), ("F", 2), ("B", 2)]
    for s in range(4):       # every stage runs each micro-batch once forward and once backward, B after F
        o = PP.one_f_one_b_order(s, 4, 6)
        assert sorted(i for k, i in o if k == "F") == list(range(6)) == sorted(i for k, i in o if k == "B")
        assert all(o.index(("F", i)) < o.index(("B", i)) for i in range(6))


def _tp_rank(rank, world, sp):
    from cppmega_mlx_b200.nn.basic import FeedForward, RMSNorm
    from cppmega_mlx_b200.parallel import tp as TP
    st = PS.init_parallel_state(tp=world)
    torch.manual_seed(0)
    norm, ffn = RMSNorm(16), FeedForward(16, 24, "swiglu")
    x = torch.randn(2, 8, 16)
    ref_in = x.clone().requires_grad_()
    ref = ffn(norm(ref_in))
    ref.square().sum().backward()
    ref_g = {"norm": norm.weight.grad.clone(), "up": ffn.gate_up_proj.weight.grad.clone(), "down": ffn.down_proj.weight.grad.clone(),
             "x": ref_in.grad.clone()}
    norm.weight.grad = None
    tpf = TP.TPFeedForward(ffn, st.tp_group, sequence_parallel=sp)
    xin = x.clone().requires_grad_()
    h = TP.scatter_sequence(xin, st.tp_group) if sp else xin
    out = tpf(norm(h))
    full = TP._all_gather_dim(out.detach(), st.tp_group, 1) if sp else out.detach()
    assert torch.allclose(full, ref.detach(), atol=1e-5)
    out.square().sum().backward()
    if sp:
        TP.allreduce_replicated_grads(torch.nn.ModuleList([norm, tpf]), st.tp_group)
        gx = xin.grad.clone()
        torch.distributed.all_reduce(gx)
    else:
        gx = xin.grad
    assert torch.allclose(gx, ref_g["x"], atol=1e-4)
    assert torch.allclose(norm.weight.grad, ref_g["norm"], atol=1e-4)
    assert torch.allclose(tpf.up.weight.grad, TP.shard_rows(ref_g["up"], st.tp_group, blocks=2), atol=1e-4)
    assert torch.allclose(tpf.down.weight.grad, TP.shard_cols(ref_g["down"], st.tp_group), atol=1e-4)
    return True


@pytest.mark.parametrize("sp", [False, True])
def test_tensor_parallel_ffn_matches_single_rank(sp):
    assert all(run_ranks(_tp_rank, 2, sp))


def _tp_mixers_rank(rank, world):
    """A stack with every mixer kind (M, A, E, R) plus dense FFNs: head- / expert-parallel mixers and column/row-parallel FFNs on two
    ranks reproduce the single-process forward, the input gradient and the (sliced or replicated) parameter gradients."""
    from cppmega_mlx_b200.models.hybrid_lm import HybridTinyConfig, HybridTinyLM
    from cppmega_mlx_b200.parallel import tp as TP
    st = PS.init_parallel_state(tp=world)
    cfg = HybridTinyConfig(vocab_size=64, hidden_size=32, pattern="MAER", depth=4, num_attention_heads=4, max_seq_length=16, mamba_head_dim=16,
                           mamba_state_dim=8, mamba_chunk_size=8, mamba_groups=2, moe_num_experts=4, moe_top_k=2, moe_expert_hidden_size=16,
                           moe_shared_expert_hidden_size=16, m2rnn_k_head_dim=4, m2rnn_v_head_dim=4, m2rnn_num_q_heads=1, m2rnn_num_k_heads=2,
                           m2rnn_num_v_heads=4, m2rnn_num_f_heads=4, m2rnn_num_g_heads=4, mla_low_rank=True, mla_q_lora_rank=16,
                           mla_kv_lora_rank=16, mla_qk_nope_head_dim=8, mla_qk_rope_head_dim=4, mla_v_head_dim=8, ffn_hidden_size=48,
                           position_embedding=False)
    torch.manual_seed(0)
    full = HybridTinyLM(cfg)
    with torch.no_grad():
        for p in full.parameters():
            if p.dim() == 2 and float(p.abs().sum()) == 0:
                p.normal_(std=0.05)             # zero-initialised output projections would hide the mixers
    ids = torch.randint(0, 64, (2, 12))
    ref = full(ids)
    ref.square().mean().backward()
    ref_g = {n: p.grad.clone() for n, p in full.named_parameters() if p.grad is not None}
    full.zero_grad()
    tpm = HybridTinyLM(cfg)
    tpm.load_state_dict(full.state_dict())
    done = TP.tensor_parallelize_mixers(tpm, st.tp_group)
    assert done == {"mla": 1, "moe": 1, "m2rnn": 1, "mamba3": 1}, done
    assert TP.tensor_parallelize_ffn(tpm, st.tp_group) >= 3          # the dense FFNs (and the MoE layer's shared expert)
    out = tpm(ids)
    assert torch.allclose(out, ref.detach(), atol=2e-5), float((out - ref).abs().max())
    out.square().mean().backward()
    g = {n: p.grad for n, p in tpm.named_parameters() if p.grad is not None}
    H, r = 4, rank
    checks = 0
    for n, want in ref_g.items():
        if n in g and g[n].shape == want.shape:                    # replicated parameters: identical full gradients on every rank
            assert torch.allclose(g[n], want, atol=3e-5), (n, float((g[n] - want).abs().max()))
            checks += 1
    a = "layers.1.block."
    assert torch.allclose(g[a + "wo.weight"], ref_g[a + "wo.weight"][:, r * 16:(r + 1) * 16], atol=3e-5)
    assert torch.allclose(g[a + "wq_b.weight"], ref_g[a + "wq_b.weight"][r * 24:(r + 1) * 24], atol=3e-5)
    e = "layers.2.block.experts."
    assert torch.allclose(g[e + "w_down"], ref_g[e + "w_down"][r * 2:(r + 1) * 2], atol=3e-5)
    m = "layers.3.block."
    assert torch.allclose(g[m + "out_proj.weight"], ref_g[m + "out_proj.weight"][:, r * 8:(r + 1) * 8], atol=3e-5)
    assert torch.allclose(g[m + "state_weight"], ref_g[m + "state_weight"], atol=3e-5)          # one shared matrix: replicated, gradient summed
    assert torch.allclose(g[m + "A_log"], ref_g[m + "A_log"][r * 2:(r + 1) * 2], atol=3e-5)
    # Mamba3 (4 heads of 16, 2 groups, d_inner 64): rank r holds heads 2r, 2r+1 and group r; the phase rows (dd_dt of heads 0 and 1)
    # and the angle rows are replicated with gradients summed over the ranks
    k = "layers.0.block."
    w_ref = ref_g[k + "in_proj.weight"]
    d_in, d_bc, Hm, Gm = 64, 16, 4, 2
    base = 2 * d_in + 2 * d_bc
    rep_want = torch.cat([w_ref[base:base + Gm], w_ref[base + 3 * Hm:]], 0)
    assert torch.allclose(g[k + "in_proj_rep.weight"], rep_want, atol=3e-5), float((g[k + "in_proj_rep.weight"] - rep_want).abs().max())
    assert torch.allclose(g[k + "rep_dt_bias"], ref_g[k + "dt_bias"][:Gm], atol=3e-5)
    sl = g[k + "in_proj.weight"]
    assert torch.allclose(sl[:32], w_ref[r * 32:(r + 1) * 32], atol=3e-5)                                  # z rows of this rank
    assert torch.allclose(sl[64:72], w_ref[2 * d_in + r * 8:2 * d_in + (r + 1) * 8], atol=3e-5)            # B rows of this rank's group
    n_own = 2 if r == 0 else 0
    dd_a_local = sl[80 + (2 - n_own):80 + (2 - n_own) + 2]
    assert torch.allclose(dd_a_local, w_ref[base + Hm + 2 * r:base + Hm + 2 * r + 2], atol=3e-5)          # dd_A rows
    assert torch.allclose(g[k + "out_proj.weight"], ref_g[k + "out_proj.weight"][:, r * 32:(r + 1) * 32], atol=3e-5)
    assert torch.allclose(g[k + "D"], ref_g[k + "D"][2 * r:2 * r + 2], atol=3e-5)
    assert torch.allclose(g[k + "B_norm_weight"], ref_g[k + "B_norm_weight"][:, r:r + 1], atol=3e-5)
    assert checks > 10
    return True


def test_tensor_parallel_mixers_match_single_rank():
    assert all(run_ranks(_tp_mixers_rank, 2))


def _tp_decode_rank(rank, world):
    """Cached decode on the head- / expert-parallel stack: prefill + one-token steps through a ``DecodeSession`` give the logits the
    unsharded model gives through its own session (each rank keeps its own share of every cache), and the Mamba3 mixer alone
    continues from a cache in chunks of several tokens as well.  The comparison is piece by piece: the trapezoid rule looks one
    token ahead, so the last position of a piece differs from an uninterrupted run in both forms alike, and the state catches up
    when the next token arrives."""
    from cppmega_mlx_b200.inference import DecodeSession
    from cppmega_mlx_b200.models.hybrid_lm import HybridTinyConfig, HybridTinyLM
    from cppmega_mlx_b200.parallel import tp as TP
    st = PS.init_parallel_state(tp=world)
    cfg = HybridTinyConfig(vocab_size=64, hidden_size=32, pattern="MAER", depth=4, num_attention_heads=4, max_seq_length=16, mamba_head_dim=16,
                           mamba_state_dim=8, mamba_chunk_size=8, mamba_groups=2, moe_num_experts=4, moe_top_k=2, moe_expert_hidden_size=16,
                           moe_shared_expert_hidden_size=16, m2rnn_k_head_dim=4, m2rnn_v_head_dim=4, m2rnn_num_q_heads=1, m2rnn_num_k_heads=2,
                           m2rnn_num_v_heads=4, m2rnn_num_f_heads=4, m2rnn_num_g_heads=4, mla_low_rank=True, mla_q_lora_rank=16,
                           mla_kv_lora_rank=16, mla_qk_nope_head_dim=8, mla_qk_rope_head_dim=4, mla_v_head_dim=8, ffn_hidden_size=48,
                           position_embedding=False)
    torch.manual_seed(0)
    full = HybridTinyLM(cfg).eval()
    with torch.no_grad():
        for p in full.parameters():
            if p.dim() == 2 and float(p.abs().sum()) == 0:
                p.normal_(std=0.05)
    ids = torch.randint(0, 64, (2, 12))
    pieces = [slice(0, 7)] + [slice(t, t + 1) for t in range(7, 12)]
    with torch.no_grad():
        s0 = DecodeSession(full)
        ref = torch.cat([s0.forward(ids[:, p]) for p in pieces], 1)
    tpm = HybridTinyLM(cfg).eval()
    tpm.load_state_dict(full.state_dict())
    assert TP.tensor_parallelize_mixers(tpm, st.tp_group)["mamba3"] == 1
    TP.tensor_parallelize_ffn(tpm, st.tp_group)
    with torch.no_grad():
        sess = DecodeSession(tpm)
        got = torch.cat([sess.forward(ids[:, p]) for p in pieces], 1)
    assert torch.allclose(got, ref, atol=3e-5), float((got - ref).abs().max())
    mam = tpm.layers[0].block
    assert isinstance(mam, TP.Mamba3TP)
    c = mam.config
    assert mam.mamba_state_shapes_per_request() == ((1, mam.R), (2, c.headdim, c.d_state), (1, 2, c.d_state), (2, c.headdim))
    x = torch.randn(2, 11, 32)
    with torch.no_grad():
        blk = full.layers[0].block
        whole, _ = blk(x)
        w0, wc = blk(x[:, :4], return_cache=True)
        w1, wc = blk(x[:, 4:5], cache=wc, return_cache=True)
        w2, wc = blk(x[:, 5:9], cache=wc, return_cache=True)
        want = torch.cat([w0, w1, w2, blk(x[:, 9:], cache=wc)[0]], 1)
        a, cache = mam(x[:, :4], return_cache=True)
        assert cache.ssm.shape == (2, 2, c.headdim, c.d_state) and cache.angle_dt.shape == (2, 1, mam.R) and cache.conv.shape[1] == c.d_conv - 1
        b, cache = mam(x[:, 4:5], cache=cache, return_cache=True)          # one token
        d, cache = mam(x[:, 5:9], cache=cache, return_cache=True)          # a chunk of several
        e, _ = mam(x[:, 9:], cache=cache)                                  # the last piece leaves no cache behind
        z0 = mam.zero_cache_state(2)
        assert z0.k.shape == (2, 1, 2, c.d_state) and z0.conv.shape == (2, c.d_conv - 1, mam.conv_weight.shape[0])
    got = torch.cat([a, b, d, e], 1)
    assert torch.allclose(got, want, atol=3e-5), float((got - want).abs().max())
    assert torch.allclose(got[:, -1], whole[:, -1], atol=3e-5) and torch.allclose(got[:, :3], whole[:, :3], atol=3e-5)
    lo = rank * 2                                                       # the caches are slices of the unsharded block's cache
    assert torch.allclose(cache.ssm, wc.ssm[:, lo:lo + 2], atol=3e-5) and torch.allclose(cache.k, wc.k[:, :, lo:lo + 2], atol=3e-5)
    assert torch.allclose(cache.angle_dt, wc.angle_dt[:, rank:rank + 1], atol=3e-5)      # group r turns with the phase of head r
    with pytest.raises(NotImplementedError, match="through a cache"):
        mam(x, h0=torch.zeros(2, 2, c.headdim, c.d_state))
    mam.sequence_parallel = True
    with pytest.raises(NotImplementedError, match="do not combine"):
        mam(x, return_cache=True)
    return True


def test_tensor_parallel_cached_decode_matches_full_forward():
    assert all(run_ranks(_tp_decode_rank, 2))


def _sp_mixers_rank(rank, world, aux, batch):
    """The same stack with a sequence-parallel residual stream: every rank holds half of the tokens between the blocks; output,
    the gradient of the embeddings (entry of the region), the norm weights (summed over the group afterwards) and the sliced /
    replicated mixer parameters all match the single-process model.  ``aux``: the MoE router's balance loss and the attention
    indexer's distillation loss — both computed identically on every rank from the gathered sequence — are part of the loss."""
    from cppmega_mlx_b200.models.hybrid_lm import HybridTinyConfig, HybridTinyLM
    from cppmega_mlx_b200.parallel import tp as TP
    st = PS.init_parallel_state(tp=world)
    extra = dict(dsa_all_a_layers=True, attention_sparse_topk=4, dsa_indexer_head_dim=8, dsa_indexer_loss_coeff=0.5,
                 moe_aux_loss_free=False) if aux else {}
    cfg = HybridTinyConfig(vocab_size=64, hidden_size=32, pattern="MAER", depth=4, num_attention_heads=4, max_seq_length=16, mamba_head_dim=16,
                           mamba_state_dim=8, mamba_chunk_size=8, mamba_groups=2, moe_num_experts=4, moe_top_k=2, moe_expert_hidden_size=16,
                           moe_shared_expert_hidden_size=16, m2rnn_k_head_dim=4, m2rnn_v_head_dim=4, m2rnn_num_q_heads=1, m2rnn_num_k_heads=2,
                           m2rnn_num_v_heads=4, m2rnn_num_f_heads=4, m2rnn_num_g_heads=4, mla_low_rank=True, mla_q_lora_rank=16,
                           mla_kv_lora_rank=16, mla_qk_nope_head_dim=8, mla_qk_rope_head_dim=4, mla_v_head_dim=8, ffn_hidden_size=48,
                           position_embedding=False, **extra)
    torch.manual_seed(0)
    full = HybridTinyLM(cfg)
    with torch.no_grad():
        for p in full.parameters():
            if p.dim() == 2 and float(p.abs().sum()) == 0:
                p.normal_(std=0.05)
    full.train()
    ids = torch.randint(0, 64, (batch, 12))      # an even batch is split over the ranks, an odd one keeps whole rows and splits the sequence

    def loss_of(m):
        out = m(ids)
        total = out.square().mean()
        if aux:
            a, i = m.aux_losses(), m.indexer_losses()
            assert a is not None and i is not None
            total = total + 0.1 * a + i
        return out, total
    ref, ref_loss = loss_of(full)
    ref_loss.backward()
    ref_g = {n: p.grad.clone() for n, p in full.named_parameters() if p.grad is not None}
    spm = HybridTinyLM(cfg)
    spm.load_state_dict(full.state_dict())
    spm.train()
    assert TP.tensor_parallelize_mixers(spm, st.tp_group) == {"mla": 1, "moe": 1, "m2rnn": 1, "mamba3": 1}
    assert TP.tensor_parallelize_ffn(spm, st.tp_group, sequence_parallel=True) >= 3
    partial = TP.enable_sequence_parallel(spm, st.tp_group)
    assert len(partial) == 2 * 4 + 1                                  # two norm weights per block and the final norm
    out, loss = loss_of(spm)
    assert out.shape == ref.shape and torch.allclose(out, ref.detach(), atol=3e-5), float((out - ref).abs().max())
    # with the indexer loss each rank's teacher is the mean over its own heads: the reported value is the group mean of the per-rank
    # values, an upper bound of the all-heads value; its gradient is exact (checked below on the indexer's parameters)
    assert abs(float(loss.detach()) - float(ref_loss.detach())) < (5e-2 if aux else 1e-5) and (not aux or float(loss.detach()) >= float(ref_loss.detach()) - 1e-6)
    loss.backward()
    TP.allreduce_sequence_parallel_grads(spm)
    g = {n: p.grad for n, p in spm.named_parameters() if p.grad is not None}
    checked = []
    for n, want in ref_g.items():
        if n in g and g[n].shape == want.shape:                       # replicated parameters (norms, embeddings, low-rank projections, router …)
            assert torch.allclose(g[n], want, atol=5e-5), (n, float((g[n] - want).abs().max()))
            checked.append(n)
    for must in ("token_embedding.weight", "norm.weight", "layers.0.norm.weight", "layers.2.ffn_norm.weight", "layers.1.block.wq_a.weight",
                 "layers.2.block.router.gate.weight", "layers.3.block.state_weight"):
        assert must in checked, (must, sorted(checked))
    if aux:
        assert any(n.startswith("layers.1.block.indexer.") for n in checked), sorted(checked)
    r = rank
    assert torch.allclose(g["layers.1.block.wo.weight"], ref_g["layers.1.block.wo.weight"][:, r * 16:(r + 1) * 16], atol=5e-5)
    assert torch.allclose(g["layers.1.block.wq_b.weight"], ref_g["layers.1.block.wq_b.weight"][r * 24:(r + 1) * 24], atol=5e-5)
    assert torch.allclose(g["layers.2.block.experts.w_down"], ref_g["layers.2.block.experts.w_down"][r * 2:(r + 1) * 2], atol=5e-5)
    assert torch.allclose(g["layers.3.block.out_proj.weight"], ref_g["layers.3.block.out_proj.weight"][:, r * 8:(r + 1) * 8], atol=5e-5)
    w_ref = ref_g["layers.0.block.in_proj.weight"]
    base = 2 * 64 + 2 * 16
    rep_want = torch.cat([w_ref[base:base + 2], w_ref[base + 12:]], 0)
    assert torch.allclose(g["layers.0.block.in_proj_rep.weight"], rep_want, atol=5e-5)
    assert torch.allclose(g["layers.0.block.in_proj.weight"][:32], w_ref[r * 32:(r + 1) * 32], atol=5e-5)
    assert torch.allclose(g["layers.0.block.out_proj.weight"], ref_g["layers.0.block.out_proj.weight"][:, r * 32:(r + 1) * 32], atol=5e-5)
    return True


@pytest.mark.parametrize("aux,batch", [(False, 2), (True, 2), (True, 3)])
def test_sequence_parallel_stack_matches_single_rank(aux, batch):
    assert all(run_ranks(_sp_mixers_rank, 2, aux, batch))


def _sp_refusals_rank(rank, world):
    """enable_sequence_parallel refuses a stack whose mixers are not all sharded, and one whose FFNs are tensor parallel without
    sequence parallelism; the gradient scale and the group-mean gradient are identities forward."""
    from cppmega_mlx_b200.models.hybrid_lm import HybridTinyConfig, HybridTinyLM
    from cppmega_mlx_b200.parallel import tp as TP
    st = PS.init_parallel_state(tp=world)
    cfg = HybridTinyConfig(vocab_size=64, hidden_size=32, pattern="MA", depth=2, num_attention_heads=4, max_seq_length=16, mamba_head_dim=16,
                           mamba_state_dim=8, mamba_chunk_size=8, mamba_groups=2, mla_low_rank=True, mla_q_lora_rank=16, mla_kv_lora_rank=16,
                           mla_qk_nope_head_dim=8, mla_qk_rope_head_dim=4, mla_v_head_dim=8, ffn_hidden_size=48, position_embedding=False)
    torch.manual_seed(0)
    m = HybridTinyLM(cfg)
    TP.tensor_parallelize_ffn(m, st.tp_group, sequence_parallel=True)
    with pytest.raises(ValueError, match="not head- / expert-parallel"):
        TP.enable_sequence_parallel(m, st.tp_group)
    m2 = HybridTinyLM(cfg)
    TP.tensor_parallelize_mixers(m2, st.tp_group)
    TP.tensor_parallelize_ffn(m2, st.tp_group, sequence_parallel=False)
    with pytest.raises(ValueError, match="sequence_parallel=True"):
        TP.enable_sequence_parallel(m2, st.tp_group)
    assert getattr(m2, "sp_group", None) is None
    x = torch.randn(3, 5, requires_grad=True)
    y = TP.scale_grad(x, 0.25)
    assert torch.equal(y, x)
    y.sum().backward()
    assert torch.allclose(x.grad, torch.full_like(x, 0.25))
    z = torch.full((4,), float(rank + 1), requires_grad=True)
    (TP.mean_grad_over_tp(z, st.tp_group) * (rank + 1.0)).sum().backward()       # local gradients 1 and 2: every rank ends with 1.5
    assert torch.allclose(z.grad, torch.full((4,), 1.5))
    # leaving the region hands back the local slice of an identical gradient; entering it gathers the slices' gradients
    full = torch.arange(8.0).reshape(1, 8, 1).requires_grad_()
    sl = TP.enter_sequence_parallel(full, st.tp_group, 1)
    assert sl.shape == (1, 4, 1) and float(sl[0, 0, 0]) == 4.0 * rank
    back = TP.leave_sequence_parallel(sl * 2.0, st.tp_group, 1)
    assert torch.equal(back.detach(), full.detach() * 2.0)
    back.sum().backward()
    assert torch.allclose(full.grad, torch.full_like(full, 2.0))
    return True


def test_sequence_parallel_refusals_and_gradient_helpers():
    assert all(run_ranks(_sp_refusals_rank, 2))


def _ep_rank(rank, world):
    from cppmega_mlx_b200.nn.moe import MoE, MoEConfig
    from cppmega_mlx_b200.parallel import ep as EP
    st = PS.init_parallel_state(ep=world)
    cfg = MoEConfig(d_model=16, num_experts=4, top_k=2, expert_hidden_size=8, shared_expert_hidden_size=8, scoring="sigmoid",
                    aux_loss_free=True)
    torch.manual_seed(0)
    full = MoE(cfg)
    torch.manual_seed(100)
    xs = [torch.randn(1, 6 + r, 16) for r in range(world)]            # a different token count per rank
    ref_outs = []
    for x in xs:
        ref_outs.append(full(x).output)
    sum(o.square().sum() for o in ref_outs).backward()
    local = MoE(cfg, ep_group=st.ep_group)
    EP.shard_experts_(full, local)
    assert local.local_experts == 2 and local.experts.w_down.shape[0] == 2
    out = local(xs[rank]).output
    assert torch.allclose(out, ref_outs[rank].detach(), atol=1e-5)
    out.square().sum().backward()
    EP.allreduce_replicated_grads(local, st.ep_group)
    sl = slice(rank * 2, rank * 2 + 2)
    assert torch.allclose(local.experts.w_gate_up.grad, full.experts.w_gate_up.grad[sl], atol=1e-4)
    assert torch.allclose(local.experts.w_down.grad, full.experts.w_down.grad[sl], atol=1e-4)
    assert torch.allclose(local.router.gate.weight.grad, full.router.gate.weight.grad, atol=1e-4)
    assert torch.allclose(local.shared_expert.down_proj.weight.grad, full.shared_expert.down_proj.weight.grad, atol=1e-4)
    return True


def test_expert_parallel_matches_single_rank():
    assert all(run_ranks(_ep_rank, 2))


def test_plan_slots_overflow_is_dropped_and_slots_stay_inside_the_buffer():
    """The fused path's slot computation with a deliberately small receive buffer: every kept slot is inside the buffer and
    unique per destination, every assignment that would not fit is marked −1, and all ranks agree on the layout."""
    from cppmega_mlx_b200.parallel.ep import plan_slots
    torch.manual_seed(0)
    W, Le, A = 3, 2, 700
    es = [torch.randint(0, W * Le, (A,)) for _ in range(W)]
    es[1][:500] = 4                                              # a skewed router: rank 1 sends most rows to one expert
    C = torch.stack([torch.bincount(e, minlength=W * Le).view(W, Le) for e in es])      # [src, dst, expert]
    cap = 512
    seen = [set() for _ in range(W)]
    dropped = 0
    for r in range(W):
        dest, slot, keep, pad_off, pad_end, tot = plan_slots(es[r], C, r, Le, cap)
        full = plan_slots(es[r], C, r, Le, None)[1]
        assert torch.equal(keep, full < cap) and torch.equal(slot[keep], full[keep]) and bool((slot[~keep] == -1).all())
        assert bool((slot[keep] >= 0).all()) and bool((slot[keep] < cap).all())
        assert torch.equal(dest.long(), es[r] // Le)
        for d, sl in zip(dest[keep].tolist(), slot[keep].tolist()):
            assert sl not in seen[d]                             # no two assignments share a row of a receive buffer
            seen[d].add(sl)
        e_local = es[r][keep] % Le
        lo, hi = pad_off[dest[keep].long(), e_local], pad_off[dest[keep].long(), e_local] + tot[dest[keep].long(), e_local]
        assert bool(((slot[keep] >= lo) & (slot[keep] < hi)).all())     # inside its expert's segment
        dropped += int((~keep).sum())
    assert dropped > 0 and int(pad_end[:, -1].max()) > cap       # the case really overflows


def _ep_capacity_rank(rank, world):
    """With a capacity, the all-to-all path drops exactly the assignments ``plan_slots`` marks: the result equals the
    uncapped path with those assignments' gate weights set to zero."""
    from cppmega_mlx_b200.nn.moe import MoE, MoEConfig
    from cppmega_mlx_b200.parallel import ep as EP
    st = PS.init_parallel_state(ep=world)
    cfg = MoEConfig(d_model=16, num_experts=4, top_k=2, expert_hidden_size=8, shared_expert_hidden_size=None, scoring="sigmoid")
    torch.manual_seed(0)
    full = MoE(cfg)
    local = MoE(cfg, ep_group=st.ep_group)
    EP.shard_experts_(full, local)
    torch.manual_seed(7 + rank)
    T = 300
    flat = torch.randn(T, 16)
    top_idx = torch.stack([torch.zeros(T, dtype=torch.long), 1 + torch.randint(0, 3, (T,))], 1)   # every token also picks expert 0
    top_w = torch.rand(T, 2)
    cap = 384
    got = EP.ep_moe_forward(local, flat, top_idx, top_w, capacity_rows=cap)
    mine = torch.bincount(top_idx.reshape(-1), minlength=4).view(world, 2)
    allc = [torch.empty_like(mine) for _ in range(world)]
    torch.distributed.all_gather(allc, mine)
    keep = EP.plan_slots(top_idx.reshape(-1), torch.stack(allc), rank, 2, cap)[2].view(T, 2)
    ref = EP.ep_moe_forward(local, flat, top_idx, top_w * keep)
    assert int((~keep).sum()) > 0 or rank == 0
    assert torch.allclose(got, ref, atol=1e-6)
    return int((~keep).sum())


def test_expert_parallel_capacity_drops_match_plan():
    assert sum(run_ranks(_ep_capacity_rank, 2)) > 0


def _pp_rank(rank, world):
    from cppmega_mlx_b200.ops import linear_cross_entropy
    from cppmega_mlx_b200.recipes.model_factory import build_local_gb10_quarter_tiny_smoke_model
    st = PS.init_parallel_state(pp=world)
    torch.manual_seed(0)
    model = build_local_gb10_quarter_tiny_smoke_model(pattern="AEMR", depth=4, dsa_a_layer_ranks=(), mtp_enabled=False)
    torch.manual_seed(1)
    micro = [torch.randint(4, 100, (2, 9)) for _ in range(3)]

    def loss_of(hidden, lm_head, tgt):
        return linear_cross_entropy(hidden.reshape(-1, hidden.shape[-1]), lm_head.weight, tgt.reshape(-1))
    ref = sum(loss_of(model.decoder_hidden_states(m[:, :-1]), model.lm_head, m[:, 1:]) for m in micro) / 3
    ref.backward()
    ref_grads = {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None}
    model.zero_grad()
    stage = PP.PipelineStage(model, st.pp_rank, world)
    res = PP.run_1f1b(stage, [m[:, :-1] for m in micro], [m[:, 1:] for m in micro], num_micro=3, act_shape=(2, 8, model.config.hidden_size),
                      act_dtype=torch.float32, loss_fn=lambda s, h, t: loss_of(h, s.lm_head, t), prev_rank=st.pp_prev, next_rank=st.pp_next)
    if stage.last:
        assert torch.allclose(res.loss, ref.detach(), atol=1e-5)
    owned = {f"layers.{i}." for i in stage.layer_range}
    checked = 0
    for n, p in model.named_parameters():
        mine = any(n.startswith(o) for o in owned) or (stage.first and n.startswith(("token_embedding", "position_embedding"))) or \
            (stage.last and n.startswith(("norm.", "lm_head")))
        if mine and n in ref_grads:
            assert p.grad is not None and torch.allclose(p.grad, ref_grads[n], atol=1e-4), n
            checked += 1
    return checked


def test_pipeline_1f1b_matches_single_rank():
    counts = run_ranks(_pp_rank, 2)
    assert all(c > 0 for c in counts)


def _ep_zero1_rank(rank, world):
    import torch.distributed as dist
    from cppmega_mlx_b200.data.batch import synthetic_token_batch
    from cppmega_mlx_b200.models.hybrid_lm import HybridTinyLM
    from cppmega_mlx_b200.recipes.model_factory import build_local_gb10_quarter_tiny_smoke_model
    from cppmega_mlx_b200.training.compiled import PretrainingStep
    from cppmega_mlx_b200.training.distributed_optimizer import ExpertParallelZeRO1Optimizer, is_expert_parameter
    from cppmega_mlx_b200.training.optimizers import make_adamw
    torch.manual_seed(0)
    cfg = build_local_gb10_quarter_tiny_smoke_model(pattern="AE", depth=2, dsa_a_layer_ranks=(), mtp_enabled=False).config
    torch.manual_seed(0)
    m = HybridTinyLM(cfg, ep_group=dist.group.WORLD)
    opt = ExpertParallelZeRO1Optimizer(m, lambda ps: make_adamw(ps, learning_rate=1e-2), ep_size=world)
    opt.zero_grad()
    step = PretrainingStep(m, opt)
    b = synthetic_token_batch(2, 16, vocab_size=cfg.vocab_size, seed=rank)
    losses = [step(b).loss for _ in range(4)]
    dense = torch.cat([p.detach().reshape(-1) for n, p in m.named_parameters() if not is_expert_parameter(n)])
    ref = dense.clone()
    dist.broadcast(ref, 0)
    n_local = m.layers[1].block.experts.w_down.shape[0]
    return losses, float((dense - ref).abs().max()), n_local


def test_expert_parallel_zero1_trains_and_keeps_replicas_in_sync():
    out = run_ranks(_ep_zero1_rank, 2)
    for losses, spread, n_local in out:
        assert losses[-1] < losses[0] and spread == 0.0 and n_local == 2      # 4 experts over 2 ranks; dense weights identical everywhere


class _CatCache:
    """A KV cache that grows by concatenation, so autograd runs through it (the serving cache writes in place)."""
    static = False

    def __init__(self):
        self.rows, self.offset = {}, 0

    def position(self, layer_idx):
        return self.offset

    def _grow(self, key, t):
        if t is None:
            return None
        self.rows[key] = t if key not in self.rows else torch.cat([self.rows[key], t], 1)
        return self.rows[key]

    def update_and_fetch(self, layer_idx, k, v):
        return self._grow((layer_idx, "k"), k), self._grow((layer_idx, "v"), v)

    def update_and_fetch_latent(self, layer_idx, latent, idx_k):
        return self._grow((layer_idx, "l"), latent), self._grow((layer_idx, "i"), idx_k)


def _cp_rank(rank, world, parallel):
    """Context parallelism: the sequence split over the ranks (weights replicated) gives the logits, the loss and — after averaging
    over the group — the parameter gradients of the single-process model.  With the Mamba3 layers scanning on all ranks at once
    (``parallel``) that is the plain forward over the whole sequence; with the state hand-off form it is the piecewise evaluation
    cut at the slice boundaries (prefill, then continue from the cache; the graph runs through the cache and the states)."""
    from cppmega_mlx_b200.models.hybrid_lm import HybridDecodeState, HybridTinyConfig, HybridTinyLM
    from cppmega_mlx_b200.parallel import cp as CP
    st = PS.init_parallel_state(tp=1)
    group = torch.distributed.group.WORLD
    for pattern, low_rank in (("MARE", True), ("AMRM", False)):
        cfg = HybridTinyConfig(vocab_size=64, hidden_size=32, pattern=pattern, depth=4, num_attention_heads=4, max_seq_length=24, mamba_head_dim=16,
                               mamba_state_dim=8, mamba_chunk_size=4, mamba_groups=2, moe_num_experts=4, moe_top_k=2, moe_expert_hidden_size=16,
                               moe_shared_expert_hidden_size=16, m2rnn_k_head_dim=4, m2rnn_v_head_dim=4, m2rnn_num_q_heads=1, m2rnn_num_k_heads=2,
                               m2rnn_num_v_heads=4, m2rnn_num_f_heads=4, m2rnn_num_g_heads=4, mla_low_rank=low_rank, mla_q_lora_rank=16,
                               mla_kv_lora_rank=16, mla_qk_nope_head_dim=8, mla_qk_rope_head_dim=4, mla_v_head_dim=8, ffn_hidden_size=48,
                               position_embedding=not low_rank, moe_aux_loss_coeff=0.0)
        torch.manual_seed(0)
        model = HybridTinyLM(cfg)
        with torch.no_grad():
            for p in model.parameters():
                if p.dim() == 2 and float(p.abs().sum()) == 0:
                    p.normal_(std=0.05)
        S = 6 * world
        ids = torch.randint(0, 64, (2, S + 1))
        inp, tgt = ids[:, :-1], ids[:, 1:]
        ce = torch.nn.functional.cross_entropy
        # single process, piecewise with autograd through cache and states
        n = S // world
        model.cp_parallel_mamba = parallel
        if parallel:
            ref = model(inp)
        else:
            kv, state, outs = _CatCache(), HybridDecodeState(), []
            for r in range(world):
                outs.append(model(inp[:, r * n:(r + 1) * n], kv_cache=kv, state=state))
                kv.offset += n
            ref = torch.cat(outs, 1)
        ref_loss = ce(ref.reshape(-1, 64), tgt.reshape(-1))
        ref_loss.backward()
        ref_g = {k: p.grad.clone() for k, p in model.named_parameters() if p.grad is not None}
        model.zero_grad()
        # the pieces on different ranks
        mine = CP.shard_sequence(inp, group)
        assert mine.shape == (2, n) and torch.equal(mine, inp[:, rank * n:(rank + 1) * n])
        logits = CP.context_parallel_forward(model, mine, group)
        assert torch.allclose(logits, ref.detach()[:, rank * n:(rank + 1) * n], atol=3e-5), (pattern, float((logits - ref.detach()[:, rank * n:(rank + 1) * n]).abs().max()))
        loss = ce(logits.reshape(-1, 64), CP.shard_sequence(tgt, group).reshape(-1))
        loss.backward()
        CP.allreduce_context_parallel_grads(model, group)
        total = loss.detach().clone()
        torch.distributed.all_reduce(total)
        assert abs(float(total) / world - float(ref_loss)) < 1e-5
        got = {k: p.grad for k, p in model.named_parameters()}
        assert set(ref_g) <= set(got)
        for k, want in ref_g.items():
            assert torch.allclose(got[k], want, atol=3e-5), (pattern, k, float((got[k] - want).abs().max()))
    # the switch on the model: loss functions and the training step then work on the rank's part of the batch as they are
    from cppmega_mlx_b200.data.batch import LMTokenBatch
    from cppmega_mlx_b200.training.loss import make_loss_fn
    CP.enable_context_parallel(model, group, parallel_mamba=parallel)
    assert torch.allclose(model(mine), logits.detach(), atol=1e-6)
    part = CP.shard_batch(LMTokenBatch(ids), group)
    assert torch.equal(part.inputs, mine) and torch.equal(part.targets, CP.shard_sequence(tgt, group))
    model.zero_grad()
    out = make_loss_fn(backend="cross_entropy")(model, part)
    assert abs(float(out.loss) - float(loss)) < 1e-5
    out.loss.backward()
    CP.allreduce_context_parallel_grads(model, group)
    for k, want in ref_g.items():
        assert torch.allclose(dict(model.named_parameters())[k].grad, want, atol=3e-5), k
    CP.disable_context_parallel(model)
    assert model(inp).shape == (2, S, 64)
    with pytest.raises(ValueError, match="sequence length to divide"):
        CP.shard_batch(LMTokenBatch(ids[:, :-1]), group)
    # refusals: a sequence that does not divide, layers without a state to continue from
    with pytest.raises(ValueError, match="sequence length to divide"):
        CP.shard_sequence(torch.zeros(1, 2 * world + 1), group)
    eng = HybridTinyLM(HybridTinyConfig(vocab_size=64, hidden_size=32, pattern="AN", depth=2, num_attention_heads=4, max_seq_length=24))
    with pytest.raises(NotImplementedError, match="continue from a state"):
        CP.context_parallel_forward(eng, mine, group)
    return True


@pytest.mark.parametrize("world,parallel", [(2, False), (3, False), (2, True), (3, True), (4, True)])
def test_context_parallel_matches_single_rank(world, parallel):
    assert all(run_ranks(_cp_rank, world, parallel))


def _tp_plain_attention_rank(rank, world, mode):
    """Plain q / k / v attention (grouped-query, and the shared sparse key-value form) head-parallel on two ranks: forward, input
    and parameter gradients, the sequence-parallel stack, and cached decode reproduce the single-process model."""
    from cppmega_mlx_b200.inference import DecodeSession
    from cppmega_mlx_b200.models.hybrid_lm import HybridTinyConfig, HybridTinyLM
    from cppmega_mlx_b200.nn.attention import CausalSelfAttention
    from cppmega_mlx_b200.parallel import tp as TP
    st = PS.init_parallel_state(tp=world)
    cfg = HybridTinyConfig(vocab_size=64, hidden_size=32, pattern="AA", depth=2, num_attention_heads=4, num_attention_kv_heads=2, attention_mode=mode,
                           attention_sparse_topk=5, max_seq_length=16, ffn_hidden_size=48, position_embedding=False)
    torch.manual_seed(0)
    full = HybridTinyLM(cfg)
    with torch.no_grad():
        for p in full.parameters():
            if p.dim() == 2 and float(p.abs().sum()) == 0:
                p.normal_(std=0.05)
    ids = torch.randint(0, 64, (2, 12))
    ref = full(ids)
    ref.square().mean().backward()
    ref_g = {n: p.grad.clone() for n, p in full.named_parameters() if p.grad is not None}
    full.zero_grad()

    def sharded(sp):
        m = HybridTinyLM(cfg)
        m.load_state_dict(full.state_dict())
        done = TP.tensor_parallelize_mixers(m, st.tp_group)
        assert done["attention"] == 2 and done["mla"] == 0, done
        assert TP.tensor_parallelize_ffn(m, st.tp_group, sequence_parallel=sp) == 2
        if sp:
            TP.enable_sequence_parallel(m, st.tp_group)
        return m
    r = rank
    kv_name = "sparse_kv_proj" if mode == "dsa" else "k_proj"
    for sp in (False, True):
        m = sharded(sp)
        blk = m.layers[0].block
        assert isinstance(blk, CausalSelfAttention) and blk.config.num_q_heads == 2 and blk.config.kv_heads == 1 and blk.config.q_head_dim == 8
        assert set(blk.tp_index_maps) >= {"q_proj.weight", "out_proj.weight", kv_name + ".weight"}
        out = m(ids)
        assert torch.allclose(out, ref.detach(), atol=3e-5), (sp, float((out - ref).abs().max()))
        out.square().mean().backward()
        if sp:
            TP.allreduce_sequence_parallel_grads(m)
        g = {n: p.grad for n, p in m.named_parameters() if p.grad is not None}
        for n in ("token_embedding.weight", "norm.weight", "layers.1.norm.weight"):
            assert torch.allclose(g[n], ref_g[n], atol=3e-5), (sp, n, float((g[n] - ref_g[n]).abs().max()))
        a = "layers.1.block."
        assert torch.allclose(g[a + "q_proj.weight"], ref_g[a + "q_proj.weight"][r * 16:(r + 1) * 16], atol=3e-5)
        assert torch.allclose(g[a + kv_name + ".weight"], ref_g[a + kv_name + ".weight"][r * 8:(r + 1) * 8], atol=3e-5)
        assert torch.allclose(g[a + "out_proj.weight"], ref_g[a + "out_proj.weight"][:, r * 16:(r + 1) * 16], atol=3e-5)
    # the logical (consolidated) view of the sharded parameters is the unsharded model
    from cppmega_mlx_b200.parallel.sharded_state import consolidated_parameters
    whole = consolidated_parameters(sharded(False))
    want_sd = full.state_dict()
    assert set(whole) == set(want_sd) and all(torch.equal(whole[n], want_sd[n]) for n in want_sd)
    # cached decode: every rank keeps the keys / values of its own heads
    m = sharded(False).eval()
    pieces = [slice(0, 7)] + [slice(t, t + 1) for t in range(7, 12)]
    with torch.no_grad():
        s0, s1 = DecodeSession(full.eval()), DecodeSession(m)
        want = torch.cat([s0.forward(ids[:, p]) for p in pieces], 1)
        got = torch.cat([s1.forward(ids[:, p]) for p in pieces], 1)
    assert torch.allclose(got, want, atol=3e-5), float((got - want).abs().max())
    # a head count the group does not divide stays replicated
    odd = HybridTinyLM(HybridTinyConfig(vocab_size=64, hidden_size=48, pattern="A", depth=1, num_attention_heads=3, max_seq_length=16,
                                        mamba_head_dim=16, position_embedding=False))
    assert TP.tensor_parallelize_mixers(odd, st.tp_group).get("attention", 0) == 0
    with pytest.raises(ValueError, match="must divide"):
        TP._shard_attention(odd.layers[0].block, st.tp_group)
    # an M2RNN mixer with grouped value heads stays replicated too, and still gives the single-process result
    grouped = HybridTinyConfig(vocab_size=64, hidden_size=32, pattern="R", depth=1, num_attention_heads=4, max_seq_length=16, m2rnn_k_head_dim=4,
                               m2rnn_v_head_dim=4, m2rnn_num_v_heads=2, m2rnn_num_f_heads=2, m2rnn_num_g_heads=4, position_embedding=False)
    torch.manual_seed(1)
    g0 = HybridTinyLM(grouped).eval()
    g1 = HybridTinyLM(grouped).eval()
    g1.load_state_dict(g0.state_dict())
    assert TP.tensor_parallelize_mixers(g1, st.tp_group)["m2rnn"] == 0
    with torch.no_grad():
        assert torch.allclose(g1(ids), g0(ids), atol=1e-6)
    with pytest.raises(ValueError, match="needs num_v_heads == num_heads"):
        TP._shard_m2rnn(g0.layers[0].block, st.tp_group)
    return True


@pytest.mark.parametrize("mode", ["gqa", "dsa"])
def test_tensor_parallel_plain_attention_matches_single_rank(mode):
    assert all(run_ranks(_tp_plain_attention_rank, 2, mode))


def _cp_tp_rank(rank, world):
    """Context parallelism over the data-parallel axis combined with head- / expert-parallel mixers (2 × 2 ranks): each
    tensor-parallel pair holds half of the sequence, the recurrent states travel between the ranks with the same tensor-parallel
    index, and the logits are those of the single-process piecewise evaluation."""
    from cppmega_mlx_b200.models.hybrid_lm import HybridDecodeState, HybridTinyConfig, HybridTinyLM
    from cppmega_mlx_b200.parallel import cp as CP
    from cppmega_mlx_b200.parallel import tp as TP
    st = PS.init_parallel_state(tp=2)
    cp_group = st.dp_group
    assert torch.distributed.get_world_size(cp_group) == 2
    cfg = HybridTinyConfig(vocab_size=64, hidden_size=32, pattern="MARE", depth=4, num_attention_heads=4, max_seq_length=16, mamba_head_dim=16,
                           mamba_state_dim=8, mamba_chunk_size=4, mamba_groups=2, moe_num_experts=4, moe_top_k=2, moe_expert_hidden_size=16,
                           moe_shared_expert_hidden_size=16, m2rnn_k_head_dim=4, m2rnn_v_head_dim=4, m2rnn_num_q_heads=1, m2rnn_num_k_heads=2,
                           m2rnn_num_v_heads=4, m2rnn_num_f_heads=4, m2rnn_num_g_heads=4, mla_low_rank=True, mla_q_lora_rank=16,
                           mla_kv_lora_rank=16, mla_qk_nope_head_dim=8, mla_qk_rope_head_dim=4, mla_v_head_dim=8, ffn_hidden_size=48,
                           position_embedding=False, moe_aux_loss_coeff=0.0)
    torch.manual_seed(0)
    full = HybridTinyLM(cfg)
    with torch.no_grad():
        for p in full.parameters():
            if p.dim() == 2 and float(p.abs().sum()) == 0:
                p.normal_(std=0.05)
    ids = torch.randint(0, 64, (2, 12))
    kv, state, outs = _CatCache(), HybridDecodeState(), []
    with torch.no_grad():
        for r in range(2):
            outs.append(full(ids[:, r * 6:(r + 1) * 6], kv_cache=kv, state=state))
            kv.offset += 6
    ref = torch.cat(outs, 1)
    m = HybridTinyLM(cfg)
    m.load_state_dict(full.state_dict())
    assert sum(TP.tensor_parallelize_mixers(m, st.tp_group).values()) == 4
    TP.tensor_parallelize_ffn(m, st.tp_group)
    CP.enable_context_parallel(m, cp_group)
    mine = CP.shard_sequence(ids, cp_group)
    c = torch.distributed.get_rank(cp_group)
    out = m(mine)
    assert torch.allclose(out, ref[:, c * 6:(c + 1) * 6], atol=3e-5), float((out - ref[:, c * 6:(c + 1) * 6]).abs().max())
    out.square().mean().backward()                       # the backward hand-offs pair up as well
    assert all(torch.isfinite(p.grad).all() for p in m.parameters() if p.grad is not None)
    return True


def test_context_parallel_composes_with_tensor_parallel_mixers():
    assert all(run_ranks(_cp_tp_rank, 4))


def _profile_sp_rank(rank, world, name):
    """The routing of a named production profile (pattern, sparse-attention ranks) at toy width: every mixer kind it contains is
    head- / expert-parallel, the residual stream sequence parallel, and the logits are those of the single-process model."""
    from cppmega_mlx_b200.models.hybrid_lm import HybridTinyLM
    from cppmega_mlx_b200.parallel import tp as TP
    from cppmega_mlx_b200.recipes.model_factory import get_model_profile
    st = PS.init_parallel_state(tp=world)
    cfg = get_model_profile(name).tiny_smoke_config(position_embedding=False, dsa_indexer_loss_coeff=0.0)
    torch.manual_seed(0)
    full = HybridTinyLM(cfg).eval()
    with torch.no_grad():
        for p in full.parameters():
            if p.dim() == 2 and float(p.abs().sum()) == 0:
                p.normal_(std=0.05)
    ids = torch.randint(0, cfg.vocab_size, (2, 16))
    with torch.no_grad():
        ref = full(ids)
    m = HybridTinyLM(cfg).eval()
    m.load_state_dict(full.state_dict())
    done = TP.tensor_parallelize_mixers(m, st.tp_group)
    assert sum(done.values()) == cfg.depth, (done, cfg.pattern)              # nothing stayed replicated
    TP.tensor_parallelize_ffn(m, st.tp_group, sequence_parallel=True)
    TP.enable_sequence_parallel(m, st.tp_group)
    with torch.no_grad():
        out = m(ids)
    assert torch.allclose(out, ref, atol=5e-5), (name, float((out - ref).abs().max()))
    return True


@pytest.mark.parametrize("name", ["local_gb10_quarter", "nam56r_56l"])
def test_production_profile_routing_is_fully_tensor_and_sequence_parallel(name):
    assert all(run_ranks(_profile_sp_rank, 2, name))
