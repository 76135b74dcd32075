"""Grouped (MoE) GEMM on the GPU against the per-expert loop; MoE layer forward/backward against the dense reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _loop(xp, w, L, transpose=False):
    out = torch.zeros(L.rows, w.shape[2] if transpose else w.shape[1], device=xp.device)
    for e in range(w.shape[0]):
        a, b = int(L.k_ranges[e, 0]), int(L.k_ranges[e, 1])
        if b > a:
            out[a:b] = xp[a:b].float() @ (w[e].float() if transpose else w[e].float().t())
    return out


@pytest.mark.parametrize("E,A,din,dout", [(4, 1000, 256, 384), (8, 300, 128, 128), (64, 6 * 512, 512, 256)])
def test_grouped_linear_fwd_bwd(E, A, din, dout):
    from cppmega_mlx_b200.ops import _backend as B
    from cppmega_mlx_b200.ops import grouped_gemm_cuda as GG
    torch.manual_seed(0)
    dev = "cuda"
    e = torch.randint(0, E, (A,), device=dev)
    if E == 8:
        e[e == 3] = 2                      # an expert without tokens
    L = GG.build_layout(e, E)
    x = torch.randn(A, din, device=dev).bfloat16()
    tok = torch.arange(A, device=dev)[L.order]
    xp = GG.scatter_to_padded(x, tok, L).requires_grad_()
    w = (torch.randn(E, dout, din, device=dev) * 0.05).bfloat16().requires_grad_()
    y = GG.grouped_linear_padded(xp, w, L)
    ref = _loop(xp.detach(), w.detach(), L)
    valid = torch.zeros(L.rows, dtype=torch.bool, device=dev)
    valid[L.slot] = True
    assert torch.allclose(y.float()[valid], ref[valid], atol=3e-2, rtol=3e-2)
    assert float(y.float()[~valid & (torch.arange(L.rows, device=dev) < int(L.k_ranges[-1, 1]))].abs().max()) == 0.0
    gy = torch.zeros_like(y)
    gy[L.slot] = torch.randn(A, dout, device=dev).bfloat16()
    y.backward(gy)
    gx_ref = _loop(gy, w.detach(), L, transpose=True)
    assert torch.allclose(xp.grad.float()[valid], gx_ref[valid], atol=3e-2, rtol=3e-2)
    gw_ref = torch.zeros(E, dout, din, device=dev)
    for k in range(E):
        a, b = int(L.k_ranges[k, 0]), int(L.k_ranges[k, 1])
        gw_ref[k] = gy[a:b].float().t() @ xp.detach()[a:b].float()
    scale = gw_ref.abs().max().clamp_min(1.0)
    assert float((w.grad.float() - gw_ref).abs().max() / scale) < 2e-2
    if E == 8:
        assert float(w.grad[3].abs().max()) == 0.0
    B.check_status()


def test_moe_layer_matches_dense_reference():
    from cppmega_mlx_b200.nn.moe import MoE, MoEConfig
    from cppmega_mlx_b200.ops import _backend as B
    torch.manual_seed(1)
    cfg = MoEConfig(d_model=256, num_experts=16, top_k=4, expert_hidden_size=128, shared_expert_hidden_size=128, scoring="sigmoid",
                    aux_loss_free=True)
    moe = MoE(cfg).cuda().bfloat16()
    x = (torch.randn(2, 300, 256, device="cuda") * 0.5).bfloat16().requires_grad_()
    out = moe(x).output
    with B.use_kernels(False):
        ref = moe.dense_reference_forward(x.detach())
    assert torch.allclose(out.float(), ref.float(), atol=5e-2, rtol=5e-2)
    out.float().square().mean().backward()
    g_k = {n: p.grad.float().clone() for n, p in moe.named_parameters() if p.grad is not None}
    gx_k = x.grad.float().clone()
    moe.zero_grad()
    x.grad = None
    with B.use_kernels(False):
        moe(x).output.float().square().mean().backward()
    assert torch.allclose(gx_k, x.grad.float(), atol=2e-3, rtol=5e-2)
    for n, p in moe.named_parameters():
        if p.grad is None:
            continue
        ref_g = p.grad.float()
        assert float((g_k[n] - ref_g).abs().max()) <= 5e-2 * float(ref_g.abs().max()) + 1e-4, n
    B.check_status()
