import pytest
import torch

from cppmega_mlx_b200.nn.basic import FeedForward
from cppmega_mlx_b200.training import plasticity as P
from cppmega_mlx_b200.training.optimizers import make_adamw


def test_fire_newton_schulz_orthogonalises_and_keeps_norm():
    torch.manual_seed(0)
    for shape in ((24, 10), (10, 24), (3, 12, 8)):
        w = torch.randn(*shape)
        o = P.newton_schulz(w)
        assert o.shape == w.shape
        assert torch.allclose(o.flatten(-2).norm(dim=-1), w.flatten(-2).norm(dim=-1), rtol=1e-4)
        sv = torch.linalg.svdvals(o)
        assert float((sv.max(-1).values / sv.min(-1).values).max()) < 1.05       # all singular values equal
    assert float(P.spectral_norm_power_iter(torch.diag(torch.tensor([3.0, 1.0, 0.5])), 30)) == pytest.approx(3.0, rel=1e-3)
    with pytest.raises(ValueError):
        P.newton_schulz(torch.randn(5))


def test_apply_fire_selects_and_resets_optimizer_state():
    torch.manual_seed(1)
    from cppmega_mlx_b200.recipes.model_factory import build_local_gb10_quarter_tiny_smoke_model
    m = build_local_gb10_quarter_tiny_smoke_model()
    opt = make_adamw(m)
    for p in m.parameters():
        p.grad = torch.randn_like(p)
    opt.step()
    emb = m.token_embedding.weight.clone()
    fired = P.apply_fire(m, target_keywords=("q_proj", "experts"))
    assert "layers.0.block.q_proj.weight" in fired and "layers.1.block.experts.w_gate_up" in fired
    assert not any("embedding" in n or "lm_head" in n for n in fired) and torch.equal(emb, m.token_embedding.weight)
    n = P.reset_optimizer_states_for_fired(opt, fired)
    assert n == len(fired)
    assert float(opt.state["layers.0.block.q_proj.weight"]["m"].abs().max()) == 0.0
    assert float(opt.state["layers.0.block.k_proj.weight"]["m"].abs().max()) > 0.0


def test_dash_shrinks_only_aligned_rows():
    w = torch.tensor([[1.0, 0.0], [0.0, 1.0], [1.0, 1.0]])
    g = torch.tensor([[2.0, 0.0], [1.0, 0.0], [-1.0, -1.0]])        # aligned, orthogonal, opposed
    out = P.dash_step(w, g, alpha=0.05, shrink_rate=0.5)
    assert torch.allclose(out[0], w[0] * (1 - 0.5 * 0.95)) and torch.equal(out[1], w[1]) and torch.equal(out[2], w[2])
    assert float(P.dash_step(w, g, shrink_rate=100.0)[0, 0]) == 0.5     # clamp
    with pytest.raises(ValueError):
        P.dash_step(w, g[:2])
    lin = torch.nn.Linear(4, 3)
    lin.weight.grad = lin.weight.detach().clone()
    lin.bias.grad = torch.zeros(3)
    before = lin.weight.detach().clone()
    assert P.dash_step_model(lin, shrink_rate=0.5, skip_muon=False) == 1
    assert torch.allclose(lin.weight, before * (1 - 0.5 * 0.95))


def test_redo_detects_and_recycles_dormant_units():
    torch.manual_seed(2)
    ffn = FeedForward(8, 16, "swiglu")
    with torch.no_grad():
        ffn.gate_up_proj.weight[16 + 3] = 0.0          # unit 3: up row dead → activation always 0
        ffn.gate_up_proj.weight[5] = -50.0             # unit 5: gate saturated off
    diag = P.ReDoDiagnostics(ema_alpha=0.5)
    diag.attach({"ffn": ffn})
    for _ in range(4):
        ffn(torch.rand(32, 8) + 0.1)
    ratio = diag.get_dormant_ratio(tau=0.025)["ffn"]
    assert ratio == pytest.approx(2 / 16)
    w_out_before = ffn.down_proj.weight.detach().clone()
    n = P.recycle_dormant_neurons({"ffn": ffn}, diag.stats, tau=0.025, generator=torch.Generator().manual_seed(0))
    assert n == 2
    changed = (ffn.down_proj.weight != w_out_before).any(0)
    assert changed.nonzero().flatten().tolist() == [3, 5]
    assert float(ffn.gate_up_proj.weight[5].abs().max()) < 10.0 and float(ffn.gate_up_proj.weight[16 + 3].abs().max()) > 0.0
    assert diag.get_dormant_ratio(tau=0.025)["ffn"] == 0.0
    diag.detach()
    assert ffn._redo_probe is None
