"""The tiny A/M/E/R hybrid LM on CPU: vocab 64, d_model 128, layers A (MLA 4 heads × 32, kv_lora 64, rope 16), M (Mamba3 state 16,
expand 2, chunk 16), E (4 experts top-2 softmax, hidden 256), R (M2RNN); tokens uniform in [0,64) from seed 0, shape [2,65];
cross-entropy, AdamW lr 1e-3, two steps in fp32 — and the same under 2-rank ZeRO-1 on gloo."""
import math

import pytest
import torch

from tests._dist_util import run_ranks


def _build():
    from cppmega_mlx_b200.models.hybrid_lm import HybridTinyConfig, HybridTinyLM
    torch.manual_seed(0)
    cfg = HybridTinyConfig(vocab_size=64, hidden_size=128, pattern="AMER", depth=4, dsa_a_layer_ranks=(), num_attention_heads=4, max_seq_length=64,
                           mla_low_rank=True, mla_q_lora_rank=64, mla_kv_lora_rank=64, mla_qk_nope_head_dim=16, mla_qk_rope_head_dim=16,
                           mla_v_head_dim=32, mamba_state_dim=16, mamba_expand=2, mamba_chunk_size=16, mamba_head_dim=32, mamba_groups=1,
                           moe_num_experts=4, moe_top_k=2, moe_expert_hidden_size=256, moe_shared_expert_hidden_size=None, moe_scoring="softmax",
                           m2rnn_k_head_dim=32, m2rnn_v_head_dim=16, m2rnn_num_v_heads=8, m2rnn_num_f_heads=8, m2rnn_num_g_heads=8,
                           mtp_enabled=False, init_std=0.02)
    return HybridTinyLM(cfg)


def _tokens():
    return torch.randint(0, 64, (2, 65), generator=torch.Generator().manual_seed(0))


def test_two_adamw_steps_reduce_the_loss():
    from cppmega_mlx_b200.data.batch import LMTokenBatch
    from cppmega_mlx_b200.training.compiled import PretrainingStep
    from cppmega_mlx_b200.training.loss import make_loss_fn
    from cppmega_mlx_b200.training.optimizers import make_adamw
    m = _build()
    assert m.route_symbols == ("A", "M", "E", "R") and next(m.parameters()).dtype == torch.float32
    step = PretrainingStep(m, make_adamw(m, learning_rate=1e-3), loss_fn=make_loss_fn(backend="cross_entropy", mtp=False))
    b = LMTokenBatch(tokens=_tokens())
    l0, l1 = step(b).loss, step(b).loss
    assert math.isfinite(l0) and math.isfinite(l1) and abs(l0 - math.log(64)) < 0.5 and l1 < l0


def _rank(rank, world):
    from cppmega_mlx_b200.data.batch import LMTokenBatch
    from cppmega_mlx_b200.training.compiled import PretrainingStep
    from cppmega_mlx_b200.training.distributed_optimizer import DistributedZeRO1Optimizer
    from cppmega_mlx_b200.training.loss import make_loss_fn
    from cppmega_mlx_b200.training.optimizers import make_adamw
    m = _build()
    full_state = sum(p.numel() for p in m.parameters()) * 8
    opt = DistributedZeRO1Optimizer(m, lambda ps: make_adamw(ps, learning_rate=1e-3))
    opt.zero_grad()
    step = PretrainingStep(m, opt, loss_fn=make_loss_fn(backend="cross_entropy", mtp=False))
    b = LMTokenBatch(tokens=_tokens())                      # every rank sees the same batch: the averaged gradient equals the W=1 gradient
    losses = [step(b).loss for _ in range(2)]
    return losses, opt.shard_owned_state_bytes(), full_state


@pytest.mark.distributed
def test_zero1_on_two_gloo_ranks_matches_single_process():
    from cppmega_mlx_b200.data.batch import LMTokenBatch
    from cppmega_mlx_b200.training.compiled import PretrainingStep
    from cppmega_mlx_b200.training.loss import make_loss_fn
    from cppmega_mlx_b200.training.optimizers import make_adamw
    m = _build()
    step = PretrainingStep(m, make_adamw(m, learning_rate=1e-3), loss_fn=make_loss_fn(backend="cross_entropy", mtp=False))
    b = LMTokenBatch(tokens=_tokens())
    single = [step(b).loss for _ in range(2)]
    out = run_ranks(_rank, 2)
    for losses, owned, full in out:
        assert all(abs(a - c) < 1e-4 for a, c in zip(losses, single))
        assert 0.3 * full < owned < 0.7 * full              # each rank holds roughly half of the optimizer state
    assert out[0][1] + out[1][1] == out[0][2]
