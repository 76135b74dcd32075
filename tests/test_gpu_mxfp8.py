"""MXFP8 quantiser and block-scaled tcgen05 GEMM against the PyTorch oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_quantizer_matches_reference_and_layout():
    from cppmega_mlx_b200.ops import mxfp8 as MX
    torch.manual_seed(0)
    x = (torch.randn(300, 384, device="cuda") * torch.logspace(-3, 2, 384, device="cuda")).bfloat16()
    x[5, 64:96] = 0                                      # an all-zero block
    x[7, 0] = 3.0e4
    t, plain = MX.quantize_mxfp8(x, want_plain_scales=True)
    q_ref, e_ref = MX.quantize_mxfp8_reference(x)
    assert torch.equal(plain, e_ref)
    assert torch.equal(t.data.view(torch.float8_e4m3fn).float(), q_ref.float())
    idx = MX.tiled_scale_index(300, 384, device="cuda")
    assert torch.equal(t.scales[idx], e_ref)
    deq = MX.dequantize_mxfp8(t).float()
    assert torch.equal(deq, MX.dequantize_mxfp8_reference(q_ref, e_ref).bfloat16().float())
    rel = (deq - x.float()).abs() / x.float().abs().clamp_min(1e-30)
    blockmax = x.float().abs().view(300, 12, 32).amax(-1).repeat_interleave(32, 1)
    assert float(((deq - x.float()).abs() / blockmax.clamp_min(1e-30)).max()) < 0.07   # ≤ half an e4m3 ulp of the block max


@pytest.mark.parametrize("M,N,K,tile_n", [(128, 128, 128, 0), (256, 384, 512, 0), (300, 200, 1024, 0), (4096, 2048, 2048, 128),
                                          (4096, 2048, 2048, 256), (300, 512, 640, 256), (128, 256, 128, 0)])
def test_block_scaled_gemm(M, N, K, tile_n):
    from cppmega_mlx_b200.ops import _backend as B
    from cppmega_mlx_b200.ops import mxfp8 as MX
    torch.manual_seed(1)
    a = (torch.randn(M, K, device="cuda") * torch.logspace(-2, 1, K, device="cuda")).bfloat16()
    b = (torch.randn(N, K, device="cuda") * 0.1).bfloat16()
    b[:, K // 2:] *= 40.0                                 # make the per-block scales matter along K
    qa, qb = MX.quantize_mxfp8(a), MX.quantize_mxfp8(b)
    out = MX.gemm_mxfp8(qa, qb, tile_n=tile_n).float()
    ref = MX.dequantize_mxfp8(qa).float() @ MX.dequantize_mxfp8(qb).float().t()
    B.check_status()
    err = float((out - ref).abs().max()) / float(ref.abs().max())
    assert err < 1e-2, err
    full = a.float() @ b.float().t()
    assert float((out - full).abs().max()) / float(full.abs().max()) < 0.08            # quantisation error itself


def test_mxfp8_linear_forward_and_ste_backward():
    from cppmega_mlx_b200.ops import mxfp8 as MX
    torch.manual_seed(2)
    x = (torch.randn(4, 64, 256, device="cuda") * 0.5).bfloat16().requires_grad_()
    w = (torch.randn(384, 256, device="cuda") * 0.05).bfloat16().requires_grad_()
    y = MX.mxfp8_linear(x, w)
    ref = x.float() @ w.float().t()
    assert float((y.float() - ref).abs().max()) / float(ref.abs().max()) < 0.08
    gy = torch.randn_like(y)
    y.backward(gy)
    assert torch.allclose(x.grad.float(), gy.float() @ w.float(), atol=5e-2, rtol=5e-2)
    assert torch.allclose(w.grad.float(), gy.float().reshape(-1, 384).t() @ x.float().reshape(-1, 256), atol=0.5, rtol=5e-2)


def test_grouped_mxfp8_expert_ffn_matches_bf16_grouped():
    from cppmega_mlx_b200.nn.moe import MoE, MoEConfig
    from cppmega_mlx_b200.ops import _backend as B
    torch.manual_seed(3)
    kw = dict(d_model=256, num_experts=8, top_k=2, expert_hidden_size=128, shared_expert_hidden_size=None, activation="swiglu", scoring="sigmoid",
              aux_loss_free=True)
    a = MoE(MoEConfig(**kw)).cuda().bfloat16()
    b = MoE(MoEConfig(**kw, expert_gemm="mxfp8")).cuda().bfloat16()
    b.load_state_dict(a.state_dict())
    x = (torch.randn(2, 200, 256, device="cuda") * 0.5).bfloat16()
    xa, xb = x.clone().requires_grad_(), x.clone().requires_grad_()
    n0 = B.launch_count("gemm_mxfp8_grouped")
    ya, yb = a(xa).output, b(xb).output
    assert B.launch_count("gemm_mxfp8_grouped") >= n0 + 2      # up and down projections of the MXFP8 expert bank
    err = float((ya.float() - yb.float()).abs().max()) / float(ya.float().abs().max())
    assert 0 < err < 0.1                                   # fp8 forward: close to, but not identical with, the bf16 product
    g = torch.randn_like(ya)
    ya.backward(g)
    yb.backward(g)
    assert float((xa.grad.float() - xb.grad.float()).abs().max()) < 0.15 * float(xa.grad.float().abs().max())
    ga, gb = a.experts.w_down.grad.float(), b.experts.w_down.grad.float()
    assert float((ga - gb).abs().max()) < 0.15 * float(ga.abs().max())
    B.check_status()


def test_sparse_mla_blockscaled_gpu_matches_cpu_semantics():
    """GPU round trip (fused quantise + dequantise kernels) + tensor-core sparse MLA vs the CPU restatement of the same op."""
    from cppmega_mlx_b200 import ops
    torch.manual_seed(5)
    b, s, h, d, dv, topk = 1, 256, 16, 576, 512, 64
    q = torch.randn(b, s, h, d, device="cuda").bfloat16().requires_grad_()
    kv = torch.randn(b, s, 1, d, device="cuda").bfloat16().requires_grad_()
    ends = torch.arange(1, s + 1, device="cuda", dtype=torch.int32)
    idx = ops.topk_select(torch.randn(s, s, device="cuda"), topk, None, ends).view(b, s, 1, topk)
    out, _ = ops.sparse_mla_blockscaled(q, kv, idx, d_v=dv)
    ref, _ = ops.sparse_mla_blockscaled(q.detach().float().cpu(), kv.detach().float().cpu(), idx.cpu(), d_v=dv)
    assert (out.float().cpu() - ref).abs().max() < 3e-2
    rt = ops.mxfp8_roundtrip_ste(kv)
    rt_ref = ops.mxfp8_roundtrip_ste(kv.detach().float().cpu())
    assert torch.equal(rt.float().cpu(), rt_ref)           # the kernels reproduce the reference quantiser bit for bit
    out.float().sum().backward()
    assert q.grad is not None and kv.grad is not None and torch.isfinite(kv.grad.float()).all()


def test_fp8_block_dequant_kernel_matches_reference():
    from cppmega_mlx_b200.v4 import moe_fp8 as F8
    torch.manual_seed(0)
    w = torch.randn(3, 384, 1040, device="cuda") * 0.3
    q, s = F8.quantize_linear_to_fp8(w)
    got = F8.dequantize_fp8_blocks(q, s)
    ref = F8.dequantize_fp8_blocks_reference(q, s)
    assert got.dtype == torch.bfloat16 and torch.equal(got, ref)
    lin = F8.FP8Linear(1040, 384, device="cuda")
    lin.weight_fp8, lin.weight_scale_inv = q[0], s[0]
    x = torch.randn(64, 1040, device="cuda").bfloat16()
    y = lin(x)
    assert torch.allclose(y.float(), x.float() @ ref[0].float().t(), rtol=2e-2, atol=5e-2)


def test_fp8_amax_quantize_kernels_match_reference():
    from cppmega_mlx_b200.ops import _backend as B
    from cppmega_mlx_b200.ops import fp8_scale as F8
    torch.manual_seed(0)
    for dtype in (torch.bfloat16, torch.float16, torch.float32):
        x = (torch.randn(3, 1000, 257, device="cuda") * 5).to(dtype)
        x[1, 7, 3] = float("nan")
        n0 = B.launch_count("fp8_amax")
        a = F8.fp8_amax(x)
        assert B.launch_count("fp8_amax") == n0 + 1
        assert float(a) == float(F8.fp8_amax_reference(x))
        clean = torch.nan_to_num(x, nan=0.0)
        q, scale = F8.fp8_pack(clean)
        ref = F8.fp8_quantize_reference(clean, 448.0 / a.clamp_min(1e-12))
        same = (q.view(torch.uint8) == ref.view(torch.uint8)).float().mean()
        assert float(same) > 0.999, float(same)          # the two differ only where x·inv_scale sits on a rounding tie after fp32 rounding
        assert float((q.float() - ref.float()).abs().max()) <= 32.0
        assert abs(float(scale) - float(a) / 448) < 1e-6 * float(a)
    B.check_status()


def test_gemm_epilogue_amax_matches_a_pass_over_the_product():
    from cppmega_mlx_b200 import ops
    from cppmega_mlx_b200.ops import _backend as B
    torch.manual_seed(1)
    for (M, N, K) in ((300, 520, 256), (4096, 2048, 1024)):
        x = torch.randn(M, K, device="cuda").bfloat16()
        w = (torch.randn(N, K, device="cuda") * 0.1).bfloat16()
        y, am = ops.linear_with_amax(x, w)
        ref = ops.linear(x, w)
        assert torch.equal(y, ref)
        # the epilogue sees the fp32 accumulator, the reference the bf16-rounded output
        assert abs(float(am) - float(ref.float().abs().max())) <= 2 ** -7 * float(am)
        # folding: a second product into the same scalar keeps the larger value
        y2, am2 = ops.linear_with_amax(x * 0.01, w, am.clone())
        assert float(am2) == float(am)
    B.check_status()


def test_swiglu_quant_fused_equals_two_passes_and_moe_uses_it():
    from cppmega_mlx_b200 import ops
    from cppmega_mlx_b200.ops import _backend as B
    from cppmega_mlx_b200.ops import mxfp8 as MX
    torch.manual_seed(2)
    gu = (torch.randn(700, 2 * 1408, device="cuda") * 2).bfloat16().requires_grad_()
    h, hq = MX.swiglu_with_mxfp8(gu)
    ref = ops.swiglu(gu.detach())
    assert torch.equal(h, ref)
    two = MX.quantize_mxfp8(ref)
    assert torch.equal(hq.data, two.data) and torch.equal(hq.scales, two.scales)
    g = torch.randn_like(h)
    h.backward(g)
    gr = gu.detach().clone().requires_grad_()
    ops.swiglu(gr).backward(g)
    assert torch.equal(gu.grad, gr.grad)
    B.check_status()
