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


def _mixer_tp_refused(rank, world, path):
    from cppmega_mlx_b200.models.hybrid_lm import HybridTinyLM
    from cppmega_mlx_b200.parallel import state as PS
    from cppmega_mlx_b200.parallel import tp as TP
    from cppmega_mlx_b200.training import checkpoint as ck
    st = PS.init_parallel_state(tp=world)
    torch.manual_seed(0)
    model = HybridTinyLM(_moe_cfg())
    assert sum(TP.tensor_parallelize_mixers(model, st.tp_group).values()) > 0
    with pytest.raises(ck.CheckpointError, match="cannot be consolidated"):
        ck.save_checkpoint(model, path)


def test_head_parallel_mixers_are_refused_not_written_as_one_rank_slice(tmp_path):
    """No gather rule exists for head- / expert-sharded mixers: saving must fail closed on every rank instead of writing rank 0's
    slice under the logical parameter names."""
    run_ranks(_mixer_tp_refused, 2, str(tmp_path / "ckpt"))
