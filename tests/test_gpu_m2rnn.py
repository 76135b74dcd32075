"""M2RNN recurrence kernels against the PyTorch recurrence (fp32 autograd) on the GPU."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("K,nq,nk,nv,nw,nf,S", [(64, 4, 4, 4, 4, 4, 70), (64, 1, 1, 4, 2, 4, 33), (32, 2, 2, 2, 1, 2, 128)])
def test_m2rnn_fwd_bwd(K, nq, nk, nv, nw, nf, S):
    from cppmega_mlx_b200.ops import _backend as B
    from cppmega_mlx_b200.ops import m2rnn_cuda
    from cppmega_mlx_b200.ops.m2rnn_scan import m2rnn_scan, m2rnn_scan_reference
    torch.manual_seed(0)
    dev, b, V = "cuda", 2, 16
    packed = (torch.randn(b, S, nq * K + nk * K + nv * V, device=dev) * 0.5).bfloat16().requires_grad_()
    q = packed[..., :nq * K].view(b, S, nq, K)                      # strided views of one packed projection
    k = packed[..., nq * K:(nq + nk) * K].view(b, S, nk, K)
    v = packed[..., (nq + nk) * K:].view(b, S, nv, V)
    W = (torch.randn(nw, V, V, device=dev) * 0.2).bfloat16().requires_grad_()
    f = torch.rand(b, S, nf, device=dev).mul(0.5).add(0.4).bfloat16().requires_grad_()
    H = max(nq, nk, nv, nw, nf)
    h0 = (torch.randn(b, H, K, V, device=dev) * 0.1).bfloat16().requires_grad_()
    assert m2rnn_cuda.supported(q, k, v, W, f)
    y, hl = m2rnn_scan(q, k, v, W, f, h0)
    wy, wh = torch.randn_like(y.float()), torch.randn_like(hl.float())
    ((y.float() * wy).sum() + (hl.float() * wh).sum()).backward()
    got = [t.grad.float().clone() for t in (packed, W, f, h0)]
    for t in (packed, W, f, h0):
        t.grad = None
    with B.use_kernels(False):
        yr, hr = m2rnn_scan_reference(q.float(), k.float(), v.float(), W.float(), f.float(), h0.float())
    ((yr * wy).sum() + (hr * wh).sum()).backward()
    ref = [t.grad.float() for t in (packed, W, f, h0)]
    assert torch.allclose(y.float(), yr, atol=3e-2, rtol=3e-2)
    assert torch.allclose(hl.float(), hr, atol=2e-2, rtol=2e-2)
    for name, a, r in zip(("qkv", "W", "f", "h0"), got, ref):
        err = float((a - r).abs().max()) / max(float(r.abs().max()), 1e-3)
        assert err < 5e-2, (name, err)
    B.check_status()


@pytest.mark.parametrize("nq,nk,nv,nw,nf,S,with_h0", [(2, 2, 2, 2, 2, 70, True), (1, 1, 2, 1, 2, 130, False), (2, 1, 2, 2, 1, 64, True)])
def test_m2rnn_wide_heads_tensor_core_fwd_bwd(nq, nk, nv, nw, nf, S, with_h0):
    """K = 64, V = 128: the tcgen05 time-loop kernels (checkpoint every 64 steps + replay in backward) against the fp32 recurrence,
    over sequence lengths below, at and across checkpoint boundaries, grouped head counts and packed strided inputs."""
    from cppmega_mlx_b200.ops import _backend as B
    from cppmega_mlx_b200.ops import m2rnn_cuda
    from cppmega_mlx_b200.ops.m2rnn_scan import m2rnn_scan, m2rnn_scan_reference
    torch.manual_seed(1)
    dev, b, K, V = "cuda", 2, 64, 128
    packed = (torch.randn(b, S, nq * K + nk * K + nv * V, device=dev) * 0.3).bfloat16().requires_grad_()
    q = packed[..., :nq * K].view(b, S, nq, K)
    k = packed[..., nq * K:(nq + nk) * K].view(b, S, nk, K)
    v = packed[..., (nq + nk) * K:].view(b, S, nv, V)
    W = (torch.randn(nw, V, V, device=dev) * 0.06).bfloat16().requires_grad_()
    f = torch.rand(b, S, nf, device=dev).mul(0.5).add(0.4).bfloat16().requires_grad_()
    H = max(nq, nk, nv, nw, nf)
    h0 = (torch.randn(b, H, K, V, device=dev) * 0.1).bfloat16().requires_grad_() if with_h0 else None
    leaves = [packed, W, f] + ([h0] if with_h0 else [])
    assert m2rnn_cuda.supported(q, k, v, W, f)
    n0, n1 = B.launch_count("m2rnn_tc_fwd"), B.launch_count("m2rnn_tc_bwd")
    y, hl = m2rnn_scan(q, k, v, W, f, h0)
    wy, wh = torch.randn_like(y.float()), torch.randn_like(hl.float())
    ((y.float() * wy).sum() + (hl.float() * wh).sum()).backward()
    assert B.launch_count("m2rnn_tc_fwd") == n0 + 1 and B.launch_count("m2rnn_tc_bwd") == n1 + 1
    torch.cuda.synchronize()
    B.check_status()
    got = [t.grad.float().clone() for t in leaves]
    for t in leaves:
        t.grad = None
    with B.use_kernels(False):
        yr, hr = m2rnn_scan_reference(q.float(), k.float(), v.float(), W.float(), f.float(), None if h0 is None else h0.float())
    ((yr * wy).sum() + (hr * wh).sum()).backward()
    ref = [t.grad.float() for t in leaves]
    assert torch.allclose(y.float(), yr, atol=4e-2, rtol=4e-2)
    assert torch.allclose(hl.float(), hr, atol=3e-2, rtol=3e-2)
    for name, a, r in zip(("qkv", "W", "f", "h0"), got, ref):
        err = float((a - r).abs().max()) / max(float(r.abs().max()), 1e-3)
        assert err < 6e-2, (name, err)


def test_m2rnn_mixer_uses_kernel_and_matches_eager():
    from cppmega_mlx_b200.nn.m2rnn import M2RNNConfig, M2RNNMixer
    from cppmega_mlx_b200.ops import _backend as B
    torch.manual_seed(1)
    mix = M2RNNMixer(M2RNNConfig(d_model=256, k_head_dim=64, v_head_dim=16, num_v_heads=4, num_f_heads=4, num_g_heads=4)).cuda().bfloat16()
    x = (torch.randn(2, 96, 256, device="cuda") * 0.5).bfloat16()
    n0, c0 = B.launch_count("m2rnn_fwd"), B.launch_count("conv_silu_fwd")
    out, _ = mix(x)
    assert B.launch_count("m2rnn_fwd") == n0 + 1 and B.launch_count("conv_silu_fwd") == c0 + 1
    with B.use_kernels(False):
        ref, _ = mix(x)
    assert torch.allclose(out.float(), ref.float(), atol=5e-2, rtol=5e-2)


@pytest.mark.parametrize("H,nv,ng,V", [(4, 4, 4, 16), (4, 2, 1, 16), (2, 2, 2, 128)])
def test_m2rnn_post_gate_kernel_matches_reference(H, nv, ng, V):
    from cppmega_mlx_b200 import ops
    from cppmega_mlx_b200.ops import _backend as B
    torch.manual_seed(2)
    b, s = 2, 37
    y = torch.randn(b, s, H, V, device="cuda").bfloat16().requires_grad_()
    pack = torch.randn(b, s, 3 + nv * V + ng * V, device="cuda").bfloat16().requires_grad_()      # v and g are strided slices
    v = pack[..., 3:3 + nv * V].view(b, s, nv, V)
    g = pack[..., 3 + nv * V:].view(b, s, ng, V)
    D = torch.randn(H, V, device="cuda").bfloat16().requires_grad_()
    n0 = B.launch_count("m2rnn_post_fwd")
    out = ops.m2rnn_post_gate(y, v, g, D)
    assert B.launch_count("m2rnn_post_fwd") == n0 + 1
    w = torch.randn_like(out.float())
    (out.float() * w).sum().backward()
    got = [t.grad.float().clone() for t in (y, pack, D)]
    for t in (y, pack, D):
        t.grad = None
    ref = ops.m2rnn_post_gate_reference(y.float(), v.float(), g.float(), D.float())
    (ref * w).sum().backward()
    assert torch.allclose(out.float(), ref, atol=3e-2, rtol=3e-2)
    for a, t in zip(got, (y, pack, D)):
        r = t.grad.float()
        assert (a - r).abs().max() <= 3e-2 * r.abs().max() + 3e-2


@pytest.mark.parametrize("K,V,nq,nk,nv,nw,nf,with_h0", [(64, 16, 1, 1, 4, 2, 4, True), (32, 16, 2, 2, 2, 1, 2, False), (64, 128, 1, 1, 2, 2, 2, True)])
def test_m2rnn_one_token_step_kernel(K, V, nq, nk, nv, nw, nf, with_h0):
    """Decode: a single token without autograd runs the step kernel (no history, no tensor-memory setup) and matches the recurrence."""
    from cppmega_mlx_b200.ops import _backend as B
    from cppmega_mlx_b200.ops.m2rnn_scan import m2rnn_scan, m2rnn_scan_reference
    torch.manual_seed(1)
    dev, b = "cuda", 3
    packed = (torch.randn(b, 1, nq * K + nk * K + nv * V, device=dev) * 0.5).bfloat16()
    q = packed[..., :nq * K].view(b, 1, nq, K)
    k = packed[..., nq * K:(nq + nk) * K].view(b, 1, nk, K)
    v = packed[..., (nq + nk) * K:].view(b, 1, nv, V)
    W = (torch.randn(nw, V, V, device=dev) * (0.2 if V == 16 else 0.05)).bfloat16()
    f = torch.rand(b, 1, nf, device=dev).mul(0.5).add(0.4).bfloat16()
    H = max(nq, nk, nv, nw, nf)
    h0 = (torch.randn(b, H, K, V, device=dev) * 0.3).float() if with_h0 else None
    n0 = B.launch_count("m2rnn_step")
    with torch.no_grad():
        y, h = m2rnn_scan(q, k, v, W, f, h0)
        y2, h2 = m2rnn_scan(q, k, v, W, f, h)           # a second token from the returned state
    assert B.launch_count("m2rnn_step") == n0 + 2
    yr, hr = m2rnn_scan_reference(q.float(), k.float(), v.float(), W.float(), f.float(), h0)
    yr2, hr2 = m2rnn_scan_reference(q.float(), k.float(), v.float(), W.float(), f.float(), hr)
    assert torch.allclose(y.float(), yr, atol=3e-2, rtol=3e-2)
    assert torch.allclose(h.float(), hr, atol=2e-2, rtol=2e-2)
    assert torch.allclose(y2.float(), yr2, atol=4e-2, rtol=4e-2)
    assert torch.allclose(h2.float(), hr2, atol=3e-2, rtol=3e-2)
    B.check_status()
