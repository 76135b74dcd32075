"""ZeRO-1 plumbing on CPU ranks (gloo): W=2 must follow the W=1 loss trajectory and own ~half the state.
Mirrors the reference's parity criterion (tests/test_distributed_zero1.py:208-305, :313-362)."""
import torch

from tests._dist_util import run_ranks


def _tiny_cfg():
    from cppmega_mlx_b200.models.hybrid_lm import HybridTinyConfig
    return HybridTinyConfig(vocab_size=64, hidden_size=128, pattern="AMER", depth=4, num_attention_heads=4,
                            max_seq_length=64, mamba_head_dim=32, mamba_state_dim=16, mamba_chunk_size=16,
                            moe_num_experts=4, moe_top_k=2, moe_expert_hidden_size=256, m2rnn_k_head_dim=32,
                            m2rnn_v_head_dim=16)


def _train(rank, world, steps, opt_name):
    from cppmega_mlx_b200.data.batch import LMTokenBatch, synthetic_token_batch
    from cppmega_mlx_b200.models.hybrid_lm import HybridTinyLM
    from cppmega_mlx_b200.training.compiled import PretrainingStep
    from cppmega_mlx_b200.training.distributed_optimizer import DistributedZeRO1Optimizer
    from cppmega_mlx_b200.training.optimizers import make_adamw, make_muon
    torch.manual_seed(0)
    model = HybridTinyLM(_tiny_cfg())
    factory = (lambda ps: make_adamw(ps, learning_rate=1e-3)) if opt_name == "adamw" else \
        (lambda ps: make_muon(ps, lr_muon=2e-3, lr_adamw=1e-3))
    opt = DistributedZeRO1Optimizer(model, factory)
    opt.zero_grad()
    step = PretrainingStep(model, opt)
    full = synthetic_token_batch(2, 64, 64, seed=0)
    per = 2 // world
    mine = LMTokenBatch(tokens=full.tokens[rank * per:(rank + 1) * per])
    losses = []
    for _ in range(steps):
        m = step(mine)
        t = torch.tensor([m.loss])
        if world > 1:
            torch.distributed.all_reduce(t)
            t /= world
        losses.append(float(t))
    return losses, opt.shard_owned_state_bytes(), float(sum(p.float().sum() for p in model.parameters()))


def test_zero1_world2_matches_world1_adamw():
    base = run_ranks(_train, 1, 3, "adamw")[0]
    two = run_ranks(_train, 2, 3, "adamw")
    for a, b in zip(base[0], two[0][0]):
        assert abs(a - b) < 2e-4 * max(1.0, abs(a))
    # both ranks end with identical parameters and each owns about half of the optimizer state
    assert abs(two[0][2] - two[1][2]) < 1e-3
    assert abs(two[0][2] - base[2]) < 5e-2
    for r in range(2):
        assert 0.35 * base[1] < two[r][1] < 0.65 * base[1]


def test_zero1_world2_matches_world1_muon():
    base = run_ranks(_train, 1, 2, "muon")[0]
    two = run_ranks(_train, 2, 2, "muon")
    for a, b in zip(base[0], two[0][0]):
        assert abs(a - b) < 5e-4 * max(1.0, abs(a))
    assert abs(two[0][2] - two[1][2]) < 1e-3


def test_owner_assignment_is_balanced_and_disjoint():
    from cppmega_mlx_b200.models.hybrid_lm import HybridTinyLM
    from cppmega_mlx_b200.training.distributed_optimizer import assign_owners
    from cppmega_mlx_b200.training.optimizers import named_trainable
    named = named_trainable(HybridTinyLM(_tiny_cfg()))
    owners = assign_owners(named, 4)
    assert set(owners) == {n for n, _ in named}
    load = [0] * 4
    for n, p in named:
        load[owners[n]] += p.numel()
    biggest = max(p.numel() for _, p in named)
    assert max(load) <= max(biggest, 1.5 * (sum(load) / 4))


def _consistency(rank, world, mismatch):
    from cppmega_mlx_b200.parallel.consistency import check_rank_consistency
    torch.manual_seed(0)
    named = [("a.weight", torch.zeros(4, 8)), ("b.weight", torch.zeros(3 if (mismatch and rank == 1) else 5))]
    try:
        return "ok:" + check_rank_consistency(named, slots={"a.weight": (0, 0, 32)})[:8]
    except RuntimeError as e:
        return "error:" + str(e)


def test_rank_consistency_check_passes_and_names_the_first_difference():
    """Every rank must describe the same tensors before a kernel addresses peers' buffers by offset."""
    same = run_ranks(_consistency, 2, False)
    assert same[0] == same[1] and same[0].startswith("ok:")
    diff = run_ranks(_consistency, 2, True)
    for r in diff:                                   # raised on every rank, pointing at the entry
        assert r.startswith("error:") and "b.weight" in r and "entry 1" in r


def test_flat_buffers_alias_nothing_and_the_audit_sees_a_planted_overlap():
    from cppmega_mlx_b200.runtime.memory_audit import audit_grad_buffer_aliasing
    from cppmega_mlx_b200.training.distributed_optimizer import FlatBuffers
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(12, 7), torch.nn.Linear(7, 5), torch.nn.Linear(5, 3))
    named = list(model.named_parameters())
    owners = {n: i % 2 for i, (n, _) in enumerate(named)}
    FlatBuffers(named, owners, 2)
    rep = audit_grad_buffer_aliasing(model)
    assert rep["tensors"] == 12 and rep["overlaps"] == [] and rep["flat_storages"] == 2     # params buffer and grads buffer
    # plant a wrong slot: the second layer's bias now sits on top of the first layer's weight
    w = model[0].weight
    model[1].bias.data = w.data.view(-1)[3:10]
    rep = audit_grad_buffer_aliasing(model)
    assert [(a, b) for a, b, _ in rep["overlaps"]] == [("0.weight", "1.bias")] and rep["overlaps"][0][2] == 7 * 4
    # tied weights are one tensor, not an overlap
    tied = torch.nn.Sequential(torch.nn.Linear(4, 4, bias=False), torch.nn.Linear(4, 4, bias=False))
    tied[1].weight = tied[0].weight
    assert audit_grad_buffer_aliasing(tied)["overlaps"] == []


def test_owner_assignment_by_cost_balances_newton_schulz_work():
    """``assign_owners`` is deterministic, and with ``muon_owner_cost`` the matrices Muon orthogonalises are spread by their
    tensor-core work rather than by size (an embedding-sized AdamW tensor no longer counts like a matrix of the same size)."""
    import torch
    from cppmega_mlx_b200.training.distributed_optimizer import assign_owners, muon_owner_cost
    from cppmega_mlx_b200.training.optimizers import is_muon_compatible
    named = [("embed_tokens.weight", torch.empty(16384, 512, device="meta"))]
    named += [(f"layers.{i}.ffn.up.weight", torch.empty(2048, 1024, device="meta")) for i in range(12)]
    named += [(f"layers.{i}.norm.weight", torch.empty(1024, device="meta")) for i in range(12)]

    def ns(n, p):
        return 0.0 if not is_muon_compatible(n, p) else float(min(p.shape)) ** 2 * max(p.shape)
    by_size, by_cost = assign_owners(named, 4), assign_owners(named, 4, muon_owner_cost)
    assert by_cost == assign_owners(named, 4, muon_owner_cost)
    assert set(by_size) == set(by_cost) == {n for n, _ in named}

    def spread(owners):
        load = [0.0] * 4
        for n, p in named:
            load[owners[n]] += ns(n, p)
        return max(load) - min(load)
    assert spread(by_cost) < spread(by_size)
    assert spread(by_cost) == 0.0          # 12 equal matrices over 4 ranks
