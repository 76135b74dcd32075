"""DSA indexer KL loss on the GPU: GEMM logits + the fused row kernel against the fp32 PyTorch statement of the same loss."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(b, s, h, d, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = (torch.randn(b, s, h, d, device="cuda", generator=g) * 0.3).bfloat16()
    k = (torch.randn(b, s, 1, d, device="cuda", generator=g) * 0.3).bfloat16()
    x = torch.randn(b, s, s, device="cuda", generator=g)
    return q, k, x


@pytest.mark.parametrize("b,s,h,d,topk", [(2, 256, 4, 64, None), (1, 512, 16, 576, None), (2, 384, 8, 128, 64)])
def test_kernel_loss_and_gradient_match_reference(b, s, h, d, topk):
    from cppmega_mlx_b200.ops import dsa_indexer_loss as D
    q, k, x = _inputs(b, s, h, d)
    assert D.kernel_supported(x, q, k)
    idx = None
    if topk is not None:
        causal = torch.ones(s, s, device="cuda").tril().bool()
        idx = x.masked_fill(~causal, float("-inf")).topk(topk, dim=-1).indices.int()
        rows = torch.arange(s, device="cuda")[None, :, None]
        idx = torch.where(idx <= rows, idx, torch.full_like(idx, -1))
    scale = d ** -0.5
    x1 = x.clone().requires_grad_(True)
    got = D.dsa_indexer_loss(x1, q, k, softmax_scale=scale, loss_coeff=0.7, topk_indices=idx)
    got.backward()
    x2 = x.clone().requires_grad_(True)
    ref = D.dsa_indexer_loss_reference(x2, q, k, softmax_scale=scale, loss_coeff=0.7, topk_indices=idx)
    ref.backward()
    assert torch.allclose(got, ref, rtol=2e-3, atol=1e-5), (float(got), float(ref))
    assert torch.allclose(x1.grad, x2.grad, rtol=1e-2, atol=2e-6), float((x1.grad - x2.grad).abs().max())


def test_kernel_path_blocks_of_rows_and_offset(monkeypatch):
    from cppmega_mlx_b200.ops import dsa_indexer_loss as D
    monkeypatch.setattr(D, "LOGIT_BLOCK_BYTES", 4 * 4 * 256 * 100)       # 100 query rows per block
    b, sq, sk, h, d = 1, 192, 256, 4, 64
    q, k, _ = _inputs(b, sk, h, d, seed=3)
    q = q[:, :sq].contiguous()
    x = torch.randn(b, sq, sk, device="cuda")
    x1 = x.clone().requires_grad_(True)
    got = D.dsa_indexer_loss(x1, q, k, softmax_scale=0.125, query_offset=sk - sq)
    got.backward()
    x2 = x.clone().requires_grad_(True)
    ref = D.dsa_indexer_loss_reference(x2, q, k, softmax_scale=0.125, query_offset=sk - sq)
    ref.backward()
    assert torch.allclose(got, ref, rtol=2e-3, atol=1e-5)
    assert torch.allclose(x1.grad, x2.grad, rtol=1e-2, atol=2e-6)


def test_index_scores_carry_gradient_to_the_indexer_projections():
    from cppmega_mlx_b200.ops.dsa_indexer_loss import index_score_matmul
    torch.manual_seed(0)
    b, s, d = 2, 256, 64
    qw = (torch.randn(b, s, d, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    k = (torch.randn(b, s, d, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    w = torch.randn(b, s, s, device="cuda").tril()
    out = index_score_matmul(qw, k, True)
    (out.tril() * w).sum().backward()
    qf, kf = qw.detach().float().requires_grad_(True), k.detach().float().requires_grad_(True)
    ((qf @ kf.transpose(1, 2)).tril() * w).sum().backward()
    assert torch.allclose(out.tril(), (qf @ kf.transpose(1, 2)).tril().detach(), rtol=1e-2, atol=1e-2)
    for got, ref in ((qw.grad, qf.grad), (k.grad, kf.grad)):
        assert got is not None
        err = (got.float() - ref).abs().max() / ref.abs().max()
        assert err < 2e-2, float(err)
