"""Skip-step policy for a non-finite loss, with the NaN injected on the host (a loss function that returns NaN on a chosen call).
Single process and two gloo ranks where only one rank sees the bad loss."""
import pytest
import torch

from cppmega_mlx_b200.data.batch import LMTokenBatch, synthetic_token_batch
from cppmega_mlx_b200.recipes import model_factory as mf
from cppmega_mlx_b200.training import loss as L
from cppmega_mlx_b200.training.compiled import PretrainingStep
from cppmega_mlx_b200.training.optimizers import make_adamw
from tests._dist_util import run_ranks


def _poisoned(bad_calls):
    inner = L.make_loss_fn(backend="cross_entropy", mtp=False)
    calls = {"n": 0}

    def fn(model, batch):
        out = inner(model, batch)
        calls["n"] += 1
        if calls["n"] in bad_calls:
            out.loss = out.loss * float("nan")
        return out
    return fn


def _snapshot(model):
    return torch.cat([p.detach().reshape(-1).clone() for p in model.parameters()])


def test_skip_policy_drops_the_window_and_training_continues():
    torch.manual_seed(0)
    model = mf.build_local_gb10_quarter_tiny_smoke_model()
    step = PretrainingStep(model, make_adamw(model, learning_rate=1e-2), loss_fn=_poisoned({3}), grad_accum_steps=2, nonfinite_policy="skip")
    batches = [synthetic_token_batch(2, 16, vocab_size=model.config.vocab_size, seed=s) for s in range(6)]
    r = [step(batches[0]), step(batches[1])]
    assert r[1].applied_update and step.state.step == 1
    before = _snapshot(model)
    r = [step(batches[2]), step(batches[3])]          # the first micro-batch of this window is poisoned
    assert not r[0].applied_update and not r[1].applied_update
    assert step.skipped_updates == 1 and step.state.step == 1
    assert torch.equal(before, _snapshot(model))
    assert all(p.grad is None or float(p.grad.abs().max()) == 0.0 for p in model.parameters())
    r = [step(batches[4]), step(batches[5])]
    assert r[1].applied_update and step.state.step == 2
    assert not torch.equal(before, _snapshot(model))
    assert all(torch.isfinite(p).all() for p in model.parameters())


def test_raise_policy_and_default():
    torch.manual_seed(0)
    model = mf.build_local_gb10_quarter_tiny_smoke_model()
    b = synthetic_token_batch(2, 16, vocab_size=model.config.vocab_size, seed=1)
    step = PretrainingStep(model, make_adamw(model, learning_rate=1e-2), loss_fn=_poisoned({1}), nonfinite_policy="raise")
    with pytest.raises(FloatingPointError):
        step(b)
    with pytest.raises(ValueError):
        PretrainingStep(model, make_adamw(model, learning_rate=1e-2), nonfinite_policy="ignore")


def _rank(rank, world):
    from cppmega_mlx_b200.training.distributed_optimizer import DistributedZeRO1Optimizer
    torch.manual_seed(0)
    model = mf.build_local_gb10_quarter_tiny_smoke_model()
    opt = DistributedZeRO1Optimizer(model, lambda ps: make_adamw(ps, learning_rate=1e-2))
    opt.zero_grad()
    step = PretrainingStep(model, opt, loss_fn=_poisoned({2} if rank == 1 else set()), nonfinite_policy="skip")
    gen = torch.Generator().manual_seed(10 + rank)
    snaps = []
    for _ in range(3):
        step(LMTokenBatch(tokens=torch.randint(0, model.config.vocab_size, (2, 17), generator=gen)))
        snaps.append(_snapshot(model))
    assert step.skipped_updates == 1 and step.state.step == 2          # rank 0 skipped too although its own loss was finite
    assert torch.equal(snaps[0], snaps[1]) and not torch.equal(snaps[1], snaps[2])
    ref = snaps[2].clone()
    torch.distributed.broadcast(ref, 0)
    assert torch.equal(ref, snaps[2])


@pytest.mark.distributed
def test_one_bad_rank_skips_the_update_on_every_rank():
    run_ranks(_rank, 2)
