"""Checkpoints of sharded runs on CPU ranks (gloo): files hold logical tensors whatever the parallel layout, a run saved at
one world size resumes at another on the same loss trajectory, and a failing writer never leaves the other ranks waiting."""
import pytest
import torch

from tests._dist_util import run_ranks

pytestmark = pytest.mark.distributed


def _moe_cfg():
    from cppmega_mlx_b200.models.hybrid_lm import HybridTinyConfig
    return HybridTinyConfig(vocab_size=64, hidden_size=32, pattern="EA", depth=2, num_attention_heads=2, max_seq_length=16,
                            moe_num_experts=4, moe_top_k=2, moe_expert_hidden_size=16, moe_shared_expert_hidden_size=16,
                            ffn_hidden_size=48)


def _ep_tp_save(rank, world, path, mode):
    """Train two steps with expert-parallel experts (mode 'ep') or tensor-parallel FFNs (mode 'tp'), save, reload into a fresh
    sharded model and into nothing else; returns this rank's view for the parent to compare with a single-process load."""
    from cppmega_mlx_b200.models.hybrid_lm import HybridTinyLM
    from cppmega_mlx_b200.parallel import state as PS
    from cppmega_mlx_b200.parallel import tp as TP
    from cppmega_mlx_b200.parallel.sharded_state import sharded_specs
    from cppmega_mlx_b200.training import checkpoint as ck
    from cppmega_mlx_b200.training.distributed_optimizer import ExpertParallelZeRO1Optimizer
    from cppmega_mlx_b200.training.optimizers import make_adamw
    st = PS.init_parallel_state(ep=world) if mode == "ep" else PS.init_parallel_state(tp=world)

    def build():
        torch.manual_seed(0)
        if mode == "ep":
            return HybridTinyLM(_moe_cfg(), ep_group=st.ep_group)
        m = HybridTinyLM(_moe_cfg())
        assert TP.tensor_parallelize_ffn(m, st.tp_group) > 0
        return m
    model = build()
    assert sharded_specs(model)
    factory = lambda ps: make_adamw(ps, learning_rate=1e-2)
    opt = ExpertParallelZeRO1Optimizer(model, factory, ep_size=world) if mode == "ep" else factory(model)
    torch.manual_seed(5)                                   # tensor-parallel ranks see the same tokens, expert-parallel ranks differ
    ids = torch.randint(0, 64, (2, 9)) if mode == "tp" else torch.randint(0, 64, (world, 2, 9))[rank]
    for _ in range(2):
        opt.zero_grad()
        out = model(ids[:, :-1])
        torch.nn.functional.cross_entropy(out.reshape(-1, 64), ids[:, 1:].reshape(-1)).backward()
        if mode == "ep":
            from cppmega_mlx_b200.parallel import ep as EP
            for mod in model.modules():
                if hasattr(mod, "ep_size") and mod.ep_size > 1:
                    EP.allreduce_replicated_grads(mod, st.ep_group)
        opt.step()
    ck.save_checkpoint(model, path, optimizer=opt)
    fresh = build()
    fopt = ExpertParallelZeRO1Optimizer(fresh, factory, ep_size=world) if mode == "ep" else factory(fresh)
    ck.load_checkpoint(fresh, path, optimizer=fopt)
    for (n, a), (_, b) in zip(model.named_parameters(), fresh.named_parameters()):
        assert torch.equal(a, b), n
    # the restored optimizer continues exactly like the original one
    for o, m in ((opt, model), (fopt, fresh)):
        o.zero_grad()
        out = m(ids[:, :-1])
        torch.nn.functional.cross_entropy(out.reshape(-1, 64), ids[:, 1:].reshape(-1)).backward()
        o.step()
    for (n, a), (_, b) in zip(model.named_parameters(), fresh.named_parameters()):
        assert torch.allclose(a, b, atol=1e-7), n
    return {n: tuple(p.shape) for n, p in model.named_parameters()}


@pytest.mark.parametrize("mode", ["ep", "tp"])
def test_sharded_run_writes_logical_tensors(tmp_path, mode):
    from cppmega_mlx_b200.models.hybrid_lm import HybridTinyLM
    from cppmega_mlx_b200.training import checkpoint as ck
    shapes = run_ranks(_ep_tp_save, 2, str(tmp_path / "c"), mode)[0]
    torch.manual_seed(0)
    single = HybridTinyLM(_moe_cfg())                      # a plain single-process model reads the same files
    meta = ck.load_checkpoint(single, tmp_path / "c")
    assert meta["num_tensors"] > 0
    full = {n: tuple(p.shape) for n, p in single.named_parameters()}
    if mode == "ep":
        assert shapes["layers.0.block.experts.w_down"][0] * 2 == full["layers.0.block.experts.w_down"][0] == 4
    else:
        assert shapes["layers.0.ffn.up.weight"][0] * 2 == full["layers.0.ffn.gate_up_proj.weight"][0]
        assert shapes["layers.0.ffn.down.weight"][1] * 2 == full["layers.0.ffn.down_proj.weight"][1]


def _zero1_run(rank, world, path, load_from, steps, save_at):
    from cppmega_mlx_b200.data.batch import LMTokenBatch, synthetic_token_batch
    from cppmega_mlx_b200.models.hybrid_lm import HybridTinyConfig, HybridTinyLM
    from cppmega_mlx_b200.training import checkpoint as ck
    from cppmega_mlx_b200.training.compiled import PretrainingStep
    from cppmega_mlx_b200.training.distributed_optimizer import DistributedZeRO1Optimizer
    from cppmega_mlx_b200.training.optimizers import make_adamw
    torch.manual_seed(0)
    model = HybridTinyLM(HybridTinyConfig(vocab_size=64, hidden_size=32, pattern="AM", depth=2, num_attention_heads=2, max_seq_length=16,
                                          mamba_head_dim=16, mamba_state_dim=8, mamba_chunk_size=8, ffn_hidden_size=48))
    opt = DistributedZeRO1Optimizer(model, lambda ps: make_adamw(ps, learning_rate=1e-2))
    opt.zero_grad()
    step = PretrainingStep(model, opt)
    first = 0
    if load_from:
        ck.load_checkpoint(model, load_from, optimizer=opt, training_step=step)
        first = save_at
    losses = []
    for i in range(first, steps):
        full = synthetic_token_batch(4, 16, 64, seed=i)     # the same global batch whatever the world size
        per = 4 // world
        m = step(LMTokenBatch(tokens=full.tokens[rank * per:(rank + 1) * per]))
        t = torch.tensor([m.loss])
        if world > 1:
            torch.distributed.all_reduce(t)
            t /= world
        losses.append(float(t))
        if path and i + 1 == save_at:
            ck.save_checkpoint(model, path, optimizer=opt, training_step=step)
    return losses


@pytest.mark.parametrize("w_save,w_resume", [(2, 1), (2, 4), (1, 2)])
def test_zero1_checkpoint_resumes_at_another_world_size(tmp_path, w_save, w_resume):
    """Elastic resume: the optimizer state is stored by parameter name, so the shard layout of the resuming run is free."""
    base = run_ranks(_zero1_run, 1, None, None, 5, 0)[0]
    path = str(tmp_path / "c")
    head = run_ranks(_zero1_run, w_save, path, None, 3, 3)[0]
    tail = run_ranks(_zero1_run, w_resume, None, path, 5, 3)[0]
    for a, b in zip(base, head + tail):
        assert abs(a - b) < 5e-4 * max(1.0, abs(a)), (base, head, tail)


def _failing_writer(rank, world, path):
    from cppmega_mlx_b200.models.tiny_lm import TinyLM, TinyLMConfig
    from cppmega_mlx_b200.training import checkpoint as ck
    model = TinyLM(TinyLMConfig(vocab_size=32, hidden_size=16, num_heads=2, num_layers=1, ffn_hidden_size=16, max_seq_length=8))
    if rank == 0:
        import pathlib
        pathlib.Path(path).write_text("a file where the checkpoint directory should go")   # mkdir fails on the writer only
    torch.distributed.barrier()
    try:
        ck.save_checkpoint(model, path + "/ck")
    except Exception as e:  # noqa: BLE001
        return type(e).__name__
    return "no error"


def test_writer_failure_reaches_every_rank(tmp_path):
    names = run_ranks(_failing_writer, 2, str(tmp_path / "blocked"), timeout=60)
    assert names[0] != "no error" and names[1] == "CheckpointError"


def _all_mixers_cfg():
    from cppmega_mlx_b200.models.hybrid_lm import HybridTinyConfig
    return HybridTinyConfig(vocab_size=64, hidden_size=32, pattern="MAER", depth=4, num_attention_heads=4, max_seq_length=16, mamba_head_dim=16,
                            mamba_state_dim=8, mamba_chunk_size=8, mamba_groups=2, moe_num_experts=4, moe_top_k=2, moe_expert_hidden_size=16,
                            moe_shared_expert_hidden_size=16, m2rnn_k_head_dim=4, m2rnn_v_head_dim=4, m2rnn_num_q_heads=1, m2rnn_num_k_heads=2,
                            m2rnn_num_v_heads=4, m2rnn_num_f_heads=4, m2rnn_num_g_heads=4, mla_low_rank=True, mla_q_lora_rank=16,
                            mla_kv_lora_rank=16, mla_qk_nope_head_dim=8, mla_qk_rope_head_dim=4, mla_v_head_dim=8, ffn_hidden_size=48,
                            position_embedding=False)


def _mixer_tp_roundtrip(rank, world, path):
    """Head- / expert-parallel mixers and tensor-parallel FFNs: two optimizer steps (Muon on the matrices, AdamW on the rest), save,
    reload into a fresh sharded model, continue both identically."""
    from cppmega_mlx_b200.models.hybrid_lm import HybridTinyLM
    from cppmega_mlx_b200.parallel import state as PS
    from cppmega_mlx_b200.parallel import tp as TP
    from cppmega_mlx_b200.training import checkpoint as ck
    from cppmega_mlx_b200.training.optimizers import make_muon
    st = PS.init_parallel_state(tp=world)

    def build(seed):
        torch.manual_seed(seed)
        m = HybridTinyLM(_all_mixers_cfg())
        with torch.no_grad():
            for p in m.parameters():
                if p.dim() == 2 and float(p.abs().sum()) == 0:
                    p.normal_(std=0.05)
        assert TP.tensor_parallelize_mixers(m, st.tp_group) == {"mla": 1, "moe": 1, "m2rnn": 1, "mamba3": 1}
        assert TP.tensor_parallelize_ffn(m, st.tp_group) >= 3
        return m
    model = build(0)
    factory = lambda m: make_muon(m.named_parameters(), lr_muon=1e-2, lr_adamw=1e-2)
    opt = factory(model)
    torch.manual_seed(5)
    ids = torch.randint(0, 64, (2, 9))

    def one_step(m, o):
        o.zero_grad()
        out = m(ids[:, :-1])
        torch.nn.functional.cross_entropy(out.reshape(-1, 64), ids[:, 1:].reshape(-1)).backward()
        o.step()
    for _ in range(2):
        one_step(model, opt)
    ck.save_checkpoint(model, path, optimizer=opt)
    saved_out = model(ids[:, :-1]).detach()
    fresh = build(1)                                        # other initial values: everything must come from the files
    fopt = factory(fresh)
    ck.load_checkpoint(fresh, path, optimizer=fopt)
    for (n, a), (_, b) in zip(model.named_parameters(), fresh.named_parameters()):
        if rank == 0 and n == "layers.0.block.dt_bias":
            a, b = a[2:], b[2:]                             # rank 0 takes the step-size bias of its first ngroups heads from rep_dt_bias
        assert torch.equal(a, b), n
    one_step(model, opt)
    one_step(fresh, fopt)
    for (n, a), (_, b) in zip(model.named_parameters(), fresh.named_parameters()):
        if rank == 0 and n == "layers.0.block.dt_bias":
            a, b = a[2:], b[2:]
        assert torch.allclose(a, b, atol=1e-6), n
    return {n: tuple(p.shape) for n, p in model.named_parameters()}, saved_out


def test_head_parallel_mixers_round_trip_through_logical_tensors(tmp_path):
    """Every mixer kind sharded over two ranks writes the tensors of the single-process model (packed projections reassembled from
    the ranks' per-head slices and the replicated rows), and a single-process model loading them computes what the ranks did."""
    from cppmega_mlx_b200.models.hybrid_lm import HybridTinyLM
    from cppmega_mlx_b200.training import checkpoint as ck
    res = run_ranks(_mixer_tp_roundtrip, 2, str(tmp_path / "c"))
    shapes, out = res[0]
    torch.manual_seed(3)
    single = HybridTinyLM(_all_mixers_cfg())
    ck.load_checkpoint(single, tmp_path / "c")
    full = {n: tuple(p.shape) for n, p in single.named_parameters()}
    assert shapes["layers.0.block.in_proj_rep.weight"][0] + shapes["layers.0.block.in_proj.weight"][0] < full["layers.0.block.in_proj.weight"][0]
    assert "layers.0.block.in_proj_rep.weight" not in full and "layers.0.block.rep_dt_bias" not in full
    torch.manual_seed(5)
    ids = torch.randint(0, 64, (2, 9))
    got = single(ids[:, :-1]).detach()
    assert torch.allclose(got, out, atol=2e-5), float((got - out).abs().max())
    # the optimizer state (Muon momentum of the reassembled matrices, AdamW moments of the rest) fits the single-process optimizer
    from cppmega_mlx_b200.training.optimizers import make_muon
    opt = make_muon(single.named_parameters(), lr_muon=1e-2, lr_adamw=1e-2)
    ck.load_checkpoint(single, tmp_path / "c", optimizer=opt)
    opt.zero_grad()
    torch.nn.functional.cross_entropy(single(ids[:, :-1]).reshape(-1, 64), ids[:, 1:].reshape(-1)).backward()
    opt.step()
    assert all(bool(torch.isfinite(p).all()) for p in single.parameters())


def _unmapped_mixer_refused(rank, world, path):
    from cppmega_mlx_b200.models.hybrid_lm import HybridTinyLM
    from cppmega_mlx_b200.parallel import state as PS
    from cppmega_mlx_b200.parallel import tp as TP
    from cppmega_mlx_b200.training import checkpoint as ck
    st = PS.init_parallel_state(tp=world)
    torch.manual_seed(0)
    model = HybridTinyLM(_moe_cfg())
    assert sum(TP.tensor_parallelize_mixers(model, st.tp_group).values()) > 0
    for m in model.modules():
        if getattr(m, "tp_index_maps", None) is not None:
            m.tp_index_maps = None
    with pytest.raises(ck.CheckpointError, match="cannot be consolidated"):
        ck.save_checkpoint(model, path)


def test_sharded_module_without_an_index_map_is_refused(tmp_path):
    """A tensor-parallel module that brings no gather rule must fail closed on every rank instead of writing rank 0's slice under
    the logical parameter names."""
    run_ranks(_unmapped_mixer_refused, 2, str(tmp_path / "ckpt"))
