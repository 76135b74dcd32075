"""Whole mixers on the GPU: kernels on (bf16) against the PyTorch restatement in fp32 with the same weights."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def _compare(module, x, call, rel=6e-2, grad_rel=1e-1):
    from cppmega_mlx_b200.ops import _backend as B
    ref = copy.deepcopy(module).float()
    xr = x.detach().float().requires_grad_()
    xk = x.detach().bfloat16().requires_grad_()
    mod = module.bfloat16()
    with B.use_kernels(True):
        before = B.launch_count()
        yk = call(mod, xk)
        g = torch.randn_like(yk)
        yk.backward(g)
        assert B.launch_count() > before
    with B.use_kernels(False):
        yr = call(ref, xr)
        yr.backward(g.float())
    torch.cuda.synchronize()
    B.check_status()

    def close(a, b, name, r):
        err = (a.float() - b.float()).abs().max().item()
        scale = b.float().abs().max().item() + 1e-4
        assert err <= r * scale, f"{name}: err {err:.4g} scale {scale:.4g}"

    close(yk, yr, "output", rel)
    close(xk.grad, xr.grad, "input grad", grad_rel)
    pk, pr = dict(mod.named_parameters()), dict(ref.named_parameters())
    for n, p in pk.items():
        if p.grad is not None and pr[n].grad is not None and p.numel() > 64:
            close(p.grad, pr[n].grad, f"grad {n}", 1.5e-1)


def test_conv_silu_op():
    from cppmega_mlx_b200 import ops
    torch.manual_seed(0)
    proj = torch.randn(2, 77, 40 + 96 + 10, device="cuda").bfloat16().requires_grad_()
    w = (torch.randn(96, 4, 1, device="cuda") * 0.3).bfloat16().requires_grad_()
    bias = (torch.randn(96, device="cuda") * 0.1).bfloat16().requires_grad_()
    head, o1, o2, tail = ops.packed_split_conv_silu(proj, 40, 96, 64, w, bias)
    loss = (o1.float() ** 2).sum() + o2.float().sum() * 0.5 + head.float().sum() + (tail.float() ** 2).sum()
    loss.backward()
    pr, wr, br = (t.detach().float().requires_grad_() for t in (proj, w, bias))
    r1, r2 = ops.conv.causal_conv1d_silu_reference(pr, 40, 96, 64, wr, br)
    lr = (r1 ** 2).sum() + r2.sum() * 0.5 + pr[..., :40].sum() + (pr[..., 136:] ** 2).sum()
    lr.backward()
    assert (o1.float() - r1).abs().max() < 3e-2 and (o2.float() - r2).abs().max() < 3e-2
    assert (proj.grad.float() - pr.grad).abs().max() < 0.1 * pr.grad.abs().max()
    assert (w.grad.float() - wr.grad).abs().max() < 0.05 * wr.grad.abs().max() + 0.05
    assert (bias.grad.float() - br.grad).abs().max() < 0.05 * br.grad.abs().max() + 0.05


def test_mamba3_block():
    from cppmega_mlx_b200.nn.mamba3 import Mamba3Block, Mamba3Config
    torch.manual_seed(0)
    m = Mamba3Block(Mamba3Config(d_model=256, headdim=64, d_state=64, ngroups=2, chunk_size=64, d_conv=4)).cuda()
    x = torch.randn(2, 256, 256, device="cuda") * 0.5
    _compare(m, x, lambda mod, t: mod(t)[0])


def test_feed_forward_block():
    from cppmega_mlx_b200.nn.basic import FeedForward
    torch.manual_seed(0)
    m = FeedForward(256, 512, "swiglu").cuda()
    _compare(m, torch.randn(4, 128, 256, device="cuda"), lambda mod, t: mod(t))


def test_rmsnorm_block():
    from cppmega_mlx_b200.nn.basic import RMSNorm
    torch.manual_seed(0)
    m = RMSNorm(512).cuda()
    with torch.no_grad():
        m.weight.uniform_(0.5, 1.5)
    _compare(m, torch.randn(3, 100, 512, device="cuda"), lambda mod, t: mod(t), rel=2e-2, grad_rel=3e-2)
