"""Whole mixers on the GPU: kernels on (bf16) against the PyTorch restatement in fp32 with the same weights."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def _compare(module, x, call, rel=6e-2, grad_rel=1e-1, expect=()):
    from cppmega_mlx_b200.ops import _backend as B
    ref = copy.deepcopy(module).float()
    xr = x.detach().float().requires_grad_()
    xk = x.detach().bfloat16().requires_grad_()
    mod = module.bfloat16()
    with B.use_kernels(True):
        before = {name: B.launch_count(name) for name in expect}
        yk = call(mod, xk)
        g = torch.randn_like(yk)
        yk.backward(g)
        for name in expect:      # the named entry points of the kernel library ran, not merely some kernel
            assert B.launch_count(name) > before[name], f"{name} was not launched"
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


@pytest.mark.parametrize("S,n_head,C,C1,n_tail", [(77, 40, 96, 64, 10),      # pitch 146: the narrow (4-byte) kernels
                                                  (77, 40, 96, 64, 8),       # everything a multiple of 8: the wide kernels, ragged tiles
                                                  (200, 36, 100, 60, 8),     # multiples of 4 only: narrow forward, wide backward
                                                  (130, 0, 512, 256, 0)])    # two channel blocks per row, several runs
def test_conv_silu_op(S, n_head, C, C1, n_tail):
    from cppmega_mlx_b200 import ops
    torch.manual_seed(0)
    proj = torch.randn(2, S, n_head + C + n_tail, device="cuda").bfloat16().requires_grad_()
    w = (torch.randn(C, 4, 1, device="cuda") * 0.3).bfloat16().requires_grad_()
    bias = (torch.randn(C, device="cuda") * 0.1).bfloat16().requires_grad_()
    head, o1, o2, tail = ops.packed_split_conv_silu(proj, n_head, C, C1, w, bias)
    hc = torch.randn(2, S, n_head, device="cuda").bfloat16()        # a dense head gradient: the pitched-copy kernel packs it
    loss = (o1.float() ** 2).sum() + o2.float().sum() * 0.5 + (head * hc).float().sum() + (tail.float() ** 2).sum()
    loss.backward()
    pr, wr, br = (t.detach().float().requires_grad_() for t in (proj, w, bias))
    r1, r2 = ops.conv.causal_conv1d_silu_reference(pr, n_head, C, C1, wr, br)
    lr = (r1 ** 2).sum() + r2.sum() * 0.5 + (pr[..., :n_head] * hc.float()).sum() + (pr[..., n_head + C:] ** 2).sum()
    lr.backward()
    assert torch.equal(proj.grad[..., :n_head], hc)
    if n_tail:
        gt, rt = proj.grad[..., n_head + C:].float(), pr.grad[..., n_head + C:]
        assert (gt - rt).abs().max() <= 2e-2 * (rt.abs().max() + 1e-6)
    assert (o1.float() - r1).abs().max() < 3e-2 and (o2.float() - r2).abs().max() < 3e-2
    assert (proj.grad.float() - pr.grad).abs().max() < 0.1 * pr.grad.abs().max()
    assert (w.grad.float() - wr.grad).abs().max() < 0.05 * wr.grad.abs().max() + 0.05
    assert (bias.grad.float() - br.grad).abs().max() < 0.05 * br.grad.abs().max() + 0.05


def test_mamba3_block():
    from cppmega_mlx_b200.nn.mamba3 import Mamba3Block, Mamba3Config
    torch.manual_seed(0)
    m = Mamba3Block(Mamba3Config(d_model=256, headdim=64, d_state=64, ngroups=2, chunk_size=64, d_conv=4)).cuda()
    x = torch.randn(2, 256, 256, device="cuda") * 0.5
    _compare(m, x, lambda mod, t: mod(t)[0], expect=("conv_silu_fwd", "m3_xw", "m3_state_pass", "gemm_bf16_batched"))


def test_feed_forward_block():
    from cppmega_mlx_b200.nn.basic import FeedForward
    torch.manual_seed(0)
    m = FeedForward(256, 512, "swiglu").cuda()
    _compare(m, torch.randn(4, 128, 256, device="cuda"), lambda mod, t: mod(t), expect=("gemm_bf16", "swiglu_fwd"))


def test_rmsnorm_block():
    from cppmega_mlx_b200.nn.basic import RMSNorm
    torch.manual_seed(0)
    m = RMSNorm(512).cuda()
    with torch.no_grad():
        m.weight.uniform_(0.5, 1.5)
    _compare(m, torch.randn(3, 100, 512, device="cuda"), lambda mod, t: mod(t), rel=2e-2, grad_rel=3e-2, expect=("rmsnorm_fwd",))


@pytest.mark.parametrize("S,H,Hk,Dq,Dv,topk", [(256, 4, 4, 64, 64, 0), (512, 4, 1, 192, 128, 96), (384, 2, 2, 192, 128, 200),
                                               (128, 2, 1, 64, 32, 40), (200, 2, 2, 128, 128, 50), (1000, 2, 1, 192, 128, 300),
                                               (72, 3, 3, 64, 64, 0)])
def test_masked_attention_matches_reference(S, H, Hk, Dq, Dv, topk):
    from cppmega_mlx_b200 import ops
    from cppmega_mlx_b200.ops import _backend as B
    from cppmega_mlx_b200.ops import attention as A
    torch.manual_seed(S + H)
    dev = "cuda"
    Bn = 2
    q = (torch.randn(Bn, S, H, Dq, device=dev) * 0.5).bfloat16().requires_grad_()
    k = (torch.randn(Bn, S, Hk, Dq, device=dev) * 0.5).bfloat16().requires_grad_()
    v = (torch.randn(Bn, S, Hk, Dv, device=dev) * 0.5).bfloat16().requires_grad_()
    bits = mask_bool = None
    if topk:
        sc = torch.randn(Bn, S, S, device=dev)
        ends = torch.arange(1, S + 1, device=dev, dtype=torch.int32).repeat(Bn)
        idx = ops.topk_select_reference(sc.view(Bn * S, S), topk, None, ends).view(Bn, S, topk)
        idx[0, 5, :] = -1  # a query with no key at all
        bits = A.build_mask_bits(idx, S)
        mask_bool = ops.indices_to_mask(idx[:, :, None, :], S)[:, 0]
    assert A.supported(q, k, v)
    n_flash = B.launch_count("flash_fwd")
    O, lse = ops.masked_attention(q, k, v, bits)
    assert B.launch_count("flash_fwd") == n_flash + (1 if (Dq, Dv) in A.FLASH_SHAPES else 0)     # the fused kernel ran for its head sizes
    gO = torch.randn_like(O)
    gq, gk, gv = torch.autograd.grad(O, [q, k, v], gO)
    torch.cuda.synchronize()
    B.check_status()
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    Or, lser = ops.masked_attention_reference(qr, kr, vr, mask_bool)
    rq, rk, rv = torch.autograd.grad(Or, [qr, kr, vr], gO.float())

    def close(a, b, name, rel):
        err = (a.float() - b.float()).abs().max().item()
        scale = b.float().abs().max().item() + 1e-4
        assert err <= rel * scale, f"{name}: err {err:.4g} scale {scale:.4g}"

    close(O, Or, "O", 4e-2)
    fin = torch.isfinite(lser)
    assert (lse[fin] - lser[fin]).abs().max() < 5e-2
    close(gq, rq, "dQ", 8e-2)
    close(gk, rk, "dK", 8e-2)
    close(gv, rv, "dV", 8e-2)


def test_sparse_mla_op_cuda_matches_reference():
    from cppmega_mlx_b200 import ops
    from cppmega_mlx_b200.ops import sparse_mla_cuda
    torch.manual_seed(3)
    dev = "cuda"
    Bn, S, H, D, dv, topk = 1, 256, 8, 192, 128, 64
    q = (torch.randn(Bn, S, H, D, device=dev) * 0.4).bfloat16().requires_grad_()
    kv = (torch.randn(Bn, S, 1, D, device=dev) * 0.4).bfloat16().requires_grad_()
    ends = torch.arange(1, S + 1, device=dev, dtype=torch.int32)
    idx = ops.topk_select_reference(torch.randn(S, S, device=dev), topk, None, ends).view(Bn, S, 1, topk)
    assert sparse_mla_cuda.supported(q, kv, idx, dv)
    o, lse = ops.sparse_mla_attention(q, kv, idx, d_v=dv)
    g = torch.randn_like(o)
    gq, gkv = torch.autograd.grad(o, [q, kv], g)
    qr, kvr = q.detach().float().requires_grad_(), kv.detach().float().requires_grad_()
    orf, lr = ops.sparse_mla_reference(qr, kvr, idx, d_v=dv)
    rq, rkv = torch.autograd.grad(orf, [qr, kvr], g.float())
    assert (o.float() - orf).abs().max() < 4e-2 * orf.abs().max() + 1e-3
    assert (lse - lr).abs().max() < 5e-2
    assert (gq.float() - rq).abs().max() < 8e-2 * rq.abs().max() + 1e-3
    assert (gkv.float() - rkv).abs().max() < 8e-2 * rkv.abs().max() + 1e-3


def test_mla_attention_block_sparse():
    from cppmega_mlx_b200.nn.mla import MLAAttention, MLABlockConfig
    torch.manual_seed(0)
    cfg = MLABlockConfig(hidden_size=256, num_heads=4, q_lora_rank=128, kv_lora_rank=128, qk_nope_head_dim=64,
                         qk_rope_head_dim=32, v_head_dim=64, index_topk=64, index_head_dim=64, zero_init_out=False)
    m = MLAAttention(cfg).cuda()
    x = torch.randn(2, 256, 256, device="cuda") * 0.5
    _compare(m, x, lambda mod, t: mod(t), rel=8e-2, grad_rel=1.5e-1)


@pytest.mark.parametrize("rows,cols", [(1, 2048), (32, 2048), (7, 1000), (300, 512)])
def test_add_rms_norm_matches_add_then_norm(rows, cols):
    from cppmega_mlx_b200 import ops
    from cppmega_mlx_b200.ops import _backend as B
    torch.manual_seed(rows + cols)
    h = torch.randn(rows, cols, device="cuda").bfloat16()
    d = (torch.randn(rows, cols, device="cuda") * 0.3).bfloat16()
    w = (1 + 0.1 * torch.randn(cols, device="cuda")).bfloat16()
    with torch.no_grad():
        before = B.launch_count()
        s, y = ops.add_rms_norm(h, d, w, 1e-5)
        assert B.launch_count() == before + 1
        ref_s = h + d
        ref_y = ops.rms_norm(ref_s, w, 1e-5)
    assert torch.equal(s, ref_s)
    assert torch.allclose(y.float(), ref_y.float(), rtol=1e-2, atol=1e-3)
    fp = ops.rms_norm_ref(ref_s, w, 1e-5)
    assert torch.allclose(y.float(), fp.float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("K,H,HV,per_dim,T,with_s0", [(64, 2, 4, False, 70, True), (64, 2, 2, True, 33, False), (16, 1, 2, True, 9, True),
                                                      (128, 1, 1, False, 40, False), (32, 2, 2, False, 1, True)])
def test_delta_rule_forward_kernel_matches_recurrence(K, H, HV, per_dim, T, with_s0):
    """GDN (scalar decay) and KDA (per-dimension decay) forward kernel against the token-by-token recurrence in fp32."""
    from cppmega_mlx_b200.ops import _backend as B
    from cppmega_mlx_b200.v4 import delta_rule as DR
    torch.manual_seed(0)
    dev, b = "cuda", 2
    q = torch.randn(b, T, H, K, device=dev) * 0.5
    k = torch.nn.functional.normalize(torch.randn(b, T, H, K, device=dev), dim=-1)
    v = torch.randn(b, T, HV, K, device=dev)
    beta = torch.rand(b, T, HV, device=dev)
    g = -torch.rand(b, T, HV, K, device=dev) * 0.2 if per_dim else -torch.rand(b, T, HV, device=dev) * 0.2
    s0 = torch.randn(b, HV, K, K, device=dev) * 0.1 if with_s0 else None
    n0 = B.launch_count("delta_rule_fwd")
    with torch.no_grad():
        o, S = DR.gated_delta_rule(q, k, v, beta, g, initial_state=s0)
    assert B.launch_count("delta_rule_fwd") == n0 + 1
    ro, rS = DR.recurrent_gated_delta_rule(q, k, v, beta, g, initial_state=s0)
    assert torch.allclose(o, ro, atol=2e-4, rtol=2e-4), float((o - ro).abs().max())
    assert torch.allclose(S, rS, atol=2e-4, rtol=2e-4)
    # with gradients enabled the differentiable chunked form is used instead
    with torch.enable_grad():
        DR.gated_delta_rule(q.requires_grad_(), k, v, beta, g, initial_state=s0)[0].sum().backward()
    assert B.launch_count("delta_rule_fwd") == n0 + 1 and q.grad is not None
    B.check_status()


@pytest.mark.parametrize("Bn,S,Skv,H,topk", [(1, 200, 256, 64, 64), (2, 96, 192, 16, 40), (1, 33, 48, 128, 48)])
def test_sparse_mla_gather_form_forward_matches_reference(Bn, S, Skv, H, topk):
    """Latent form (576-wide rows, 512-wide values, one shared KV head) without a gradient runs the gather kernel: arbitrary key
    lists (not causal, S != Skv), −1 slots, a row with no valid slot at all."""
    from cppmega_mlx_b200 import ops
    from cppmega_mlx_b200.ops import _backend as B
    from cppmega_mlx_b200.ops import sparse_mla as SM
    torch.manual_seed(5)
    dev, D, dv = "cuda", 576, 512
    q = (torch.randn(Bn, S, H, D, device=dev) * 0.2).bfloat16()
    kv = (torch.randn(Bn, Skv, 1, D, device=dev) * 0.3).bfloat16()
    idx = torch.stack([torch.stack([torch.randperm(Skv, device=dev)[:topk] for _ in range(S)]) for _ in range(Bn)]).int().view(Bn, S, 1, topk)
    idx[:, :, :, topk // 2:] = torch.where(torch.rand(Bn, S, 1, topk - topk // 2, device=dev) < 0.3, -1, idx[:, :, :, topk // 2:])
    idx[0, 3] = -1                                         # a query with no key at all
    assert SM.gather_forward_supported(q, kv, idx, dv)
    n0 = B.launch_count("paged_decode")
    with torch.no_grad():
        o, lse = SM.sparse_mla_gather_forward(q, kv, idx, d_v=dv)
        if S != Skv:                                       # a key list the masked (causal, S == Skv) form cannot take: the dispatcher gathers
            o2, _ = ops.sparse_mla_attention(q, kv, idx, d_v=dv)
            assert torch.equal(o, o2)
    assert B.launch_count("paged_decode") == n0 + (2 if S != Skv else 1)
    orf, lr = ops.sparse_mla_reference(q.float(), kv.float(), idx, d_v=dv)
    assert (o.float() - orf).abs().max() < 3e-2 * orf.abs().max() + 1e-3
    fin = torch.isfinite(lr)
    assert torch.equal(torch.isfinite(lse), fin) and (lse[fin] - lr[fin]).abs().max() < 3e-2
    assert float(o[0, 3].abs().max()) == 0.0
    # with a gradient requested the differentiable masked form is taken instead
    assert not SM.gather_forward_supported(q.requires_grad_(), kv, idx, dv)
    B.check_status()


@pytest.mark.parametrize("n,iters,batch", [(3, 5, 4), (4, 5, 37), (8, 16, 300), (2, 0, 5)])
def test_sinkhorn_kernel_matches_pytorch_ops(n, iters, batch):
    """Forward and backward of the one-launch Sinkhorn kernel against the element-wise PyTorch iteration in fp32."""
    from cppmega_mlx_b200.nn.mhc import sinkhorn_normalize
    from cppmega_mlx_b200.ops import _backend as B
    torch.manual_seed(n * 100 + iters)
    raw = (torch.randn(batch, n, n, device="cuda") * 2.0).requires_grad_()
    g = torch.randn(batch, n, n, device="cuda")
    out = sinkhorn_normalize(raw, iters=iters)
    out.backward(g)
    ref_in = raw.detach().clone().requires_grad_()
    with B.use_kernels(False):
        ref = sinkhorn_normalize(ref_in, iters=iters)
        ref.backward(g)
    B.check_status()
    assert (out - ref).abs().max().item() < 1e-5
    assert (raw.grad - ref_in.grad).abs().max().item() < 1e-4 * (1.0 + ref_in.grad.abs().max().item())


@pytest.mark.parametrize("rows,cols", [(64, 256), (1000, 2048), (7, 512)])
def test_add_rms_norm_training_form_matches_separate_ops(rows, cols):
    """The fused residual add + norm with gradients: outputs bit-identical to add-then-norm, gradients (input, delta, weight)
    equal to the separate ops' within bf16 rounding, with gradient arriving on both outputs."""
    from cppmega_mlx_b200 import ops
    torch.manual_seed(rows + cols)
    h0 = torch.randn(rows, cols, device="cuda").bfloat16()
    d0 = (torch.randn(rows, cols, device="cuda") * 0.3).bfloat16()
    w0 = (1.0 + 0.1 * torch.randn(cols, device="cuda")).bfloat16()
    gs = torch.randn(rows, cols, device="cuda").bfloat16()
    gy = torch.randn(rows, cols, device="cuda").bfloat16()

    def run(fused):
        h, d, w = (t.clone().requires_grad_() for t in (h0, d0, w0))
        if fused:
            s, y = ops.add_rms_norm(h, d, w, 1e-5)
        else:
            s = h + d
            y = ops.rms_norm(s, w, 1e-5)
        torch.autograd.backward([s, y], [gs, gy])
        return s.detach(), y.detach(), h.grad, d.grad, w.grad
    sf, yf, ghf, gdf, gwf = run(True)
    sr, yr, ghr, gdr, gwr = run(False)
    assert torch.equal(sf, sr) and torch.equal(yf, yr)
    assert torch.equal(ghf, gdf)
    assert (ghf.float() - ghr.float()).abs().max().item() <= 2e-2 * (ghr.float().abs().max().item() + 1e-6)
    assert (gwf.float() - gwr.float()).abs().max().item() <= 2e-2 * (gwr.float().abs().max().item() + 1e-6)
