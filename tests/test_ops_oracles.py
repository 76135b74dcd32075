"""Pure-math oracles on CPU: each op's PyTorch restatement against an independent re-implementation."""
import math

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from cppmega_mlx_b200 import ops


def test_rmsnorm_and_rope_reference():
    x = torch.randn(3, 5, 16)
    w = torch.rand(16) + 0.5
    y = ops.rms_norm(x, w, 1e-5)
    assert torch.allclose(y, x * torch.rsqrt((x * x).mean(-1, keepdim=True) + 1e-5) * w, atol=1e-6)
    from cppmega_mlx_b200.ops.rope import apply_rope, rope_tables
    cos, sin = rope_tables(5, 8)
    q = torch.randn(2, 5, 4, 8)
    r = apply_rope(q, cos, sin)
    assert torch.allclose(r.norm(dim=-1), q.norm(dim=-1), atol=1e-5)       # a rotation
    assert torch.allclose(r[:, 0], q[:, 0], atol=1e-6)                      # position 0 is the identity
    # relative property: <R_m q, R_n k> depends on m - n only
    k = torch.randn(1, 1, 1, 8).expand(1, 5, 1, 8)
    qq = torch.randn(1, 1, 1, 8).expand(1, 5, 1, 8)
    rq, rk = apply_rope(qq.contiguous(), cos, sin), apply_rope(k.contiguous(), cos, sin)
    d1 = (rq[0, 3, 0] * rk[0, 1, 0]).sum()
    d2 = (rq[0, 4, 0] * rk[0, 2, 0]).sum()
    assert torch.allclose(d1, d2, atol=1e-5)


def test_swiglu_and_squared_relu():
    gu = torch.randn(4, 12, requires_grad=True)
    out = ops.swiglu(gu)
    assert torch.allclose(out, F.silu(gu[:, :6]) * gu[:, 6:])
    out.sum().backward()
    assert gu.grad is not None
    assert torch.allclose(ops.squared_relu(torch.tensor([-1.0, 2.0])), torch.tensor([0.0, 4.0]))


def _numpy_sparse_mla(q, kv, idx, scale, d_v):
    b, s, h, d = q.shape
    out = np.zeros((b, s, h, d_v), np.float64)
    for bi in range(b):
        for si in range(s):
            rows = [j for j in idx[bi, si] if j >= 0]
            if not rows:
                continue
            K = kv[bi, rows]                         # [n, d]
            for hi in range(h):
                sc = K @ q[bi, si, hi] * scale
                p = np.exp(sc - sc.max())
                p /= p.sum()
                out[bi, si, hi] = p @ K[:, :d_v]
    return out


def test_sparse_mla_reference_vs_numpy_and_sentinels():
    torch.manual_seed(0)
    b, s, h, d, dv, k = 2, 6, 3, 8, 4, 4
    q, kv = torch.randn(b, s, h, d), torch.randn(b, s, d)
    idx = torch.full((b, s, k), -1, dtype=torch.long)
    for si in range(s):
        c = torch.randperm(si + 1)[:k]
        idx[:, si, :len(c)] = c
    idx[0, 2] = -1                                    # a row with only sentinels → zeros
    out = ops.sparse_mla.sparse_mla_reference(q, kv[:, :, None], idx[:, :, None], d_v=dv)[0]
    ref = _numpy_sparse_mla(q.double().numpy(), kv.double().numpy(), idx.numpy(), d ** -0.5, dv)
    assert np.allclose(out.double().numpy(), ref, atol=1e-5)
    assert float(out[0, 2].abs().max()) == 0.0


def test_sparse_mla_masked_dense_equals_gather_form():
    torch.manual_seed(1)
    b, s, h, d, dv, k = 1, 12, 2, 8, 8, 5
    q, kv = torch.randn(b, s, h, d), torch.randn(b, s, d)
    idx = torch.stack([torch.cat([torch.randperm(i + 1)[:k], torch.full((max(0, k - i - 1),), -1)]) for i in range(s)])[None]
    a, la = ops.sparse_mla.sparse_mla_reference(q, kv[:, :, None], idx[:, :, None], d_v=dv)
    c, lc = ops.sparse_mla.sparse_mla_masked_dense(q, kv[:, :, None], idx[:, :, None], d_v=dv)
    assert torch.allclose(a, c, atol=1e-5) and torch.allclose(la, lc, atol=1e-5)


def test_sparse_mla_finite_difference_backward():
    torch.manual_seed(2)
    q = torch.randn(1, 4, 2, 6, requires_grad=True)
    kv = torch.randn(1, 4, 1, 6, requires_grad=True)
    idx = torch.tensor([[[0, -1], [0, 1], [2, 0], [3, 1]]])[:, :, None]
    wgt = torch.randn(1, 4, 2, 4)

    def f(q, kv):
        return (ops.sparse_mla.sparse_mla_reference(q, kv, idx, d_v=4)[0] * wgt).sum()
    gq, gkv = torch.autograd.grad(f(q, kv), (q, kv))
    eps = 1e-2
    for t, g in ((q, gq), (kv, gkv)):
        flat = t.detach().clone().reshape(-1)
        for j in range(0, flat.numel(), 5):
            d = torch.zeros_like(flat)
            d[j] = eps
            args_p = [(flat + d).reshape(t.shape) if u is t else u.detach() for u in (q, kv)]
            args_m = [(flat - d).reshape(t.shape) if u is t else u.detach() for u in (q, kv)]
            fd = (f(*args_p) - f(*args_m)) / (2 * eps)
            assert abs(float(fd) - float(g.reshape(-1)[j])) < 5e-3


def test_topk_reference_window_and_sentinel():
    sc = torch.tensor([[0.1, 0.9, 0.5, 0.7, 0.3], [5.0, 4.0, 3.0, 2.0, 1.0]])
    out = ops.topk_select_reference(sc, 3)
    assert sorted(out[0].tolist()) == [1, 2, 3] and sorted(out[1].tolist()) == [0, 1, 2]
    win = ops.topk_select_reference(sc, 3, starts=torch.tensor([0, 3]), ends=torch.tensor([2, 5]))
    assert sorted(win[0].tolist()) == [-1, 0, 1] and sorted(win[1].tolist()) == [-1, 3, 4]
    assert torch.equal(ops.topk_select(sc, 3).sort(-1).values, out.sort(-1).values)


def test_mamba3_chunked_equals_sequential_with_groups_and_h0():
    torch.manual_seed(3)
    b, s, h, p, n, g = 2, 37, 4, 6, 5, 2
    x, z = torch.randn(b, s, h, p), torch.randn(b, s, h, p)
    Bm, Cm = torch.randn(b, s, g, n), torch.randn(b, s, g, n)
    A, dt = -torch.rand(b, s, h) - 0.2, torch.rand(b, s, h) * 0.3
    D, h0 = torch.randn(h), torch.randn(b, h, p, n)
    y0, s0 = ops.mamba3_scan_sequential(x, Bm, Cm, z, A, dt, D, h0)
    for chunk in (8, 16, 64):
        y1, s1 = ops.mamba3_scan_chunked(x, Bm, Cm, z, A, dt, D, h0, chunk_size=chunk)
        assert torch.allclose(y0, y1, atol=2e-4, rtol=1e-4), chunk
        assert torch.allclose(s0, s1, atol=2e-4, rtol=1e-4)


def test_mamba3_chunked_gradients_match_sequential():
    torch.manual_seed(4)
    b, s, h, p, n = 1, 19, 2, 3, 4
    mk = lambda *sh: torch.randn(*sh, dtype=torch.double, requires_grad=True)
    x, z, Bm, Cm = mk(b, s, h, p), mk(b, s, h, p), mk(b, s, h, n), mk(b, s, h, n)
    A = (-torch.rand(b, s, h, dtype=torch.double) - 0.2).requires_grad_()
    dt = (torch.rand(b, s, h, dtype=torch.double) * 0.3).requires_grad_()
    D = mk(h)
    leaves = (x, Bm, Cm, z, A, dt, D)
    g0 = torch.autograd.grad(ops.mamba3_scan_sequential(*leaves)[0].square().sum(), leaves)
    g1 = torch.autograd.grad(ops.mamba3_scan_chunked(*leaves, chunk_size=8)[0].square().sum(), leaves)
    for a, c in zip(g0, g1):
        assert torch.allclose(a, c, atol=1e-3, rtol=1e-3)


def test_m2rnn_reference_recurrence():
    from cppmega_mlx_b200.ops.m2rnn_scan import m2rnn_scan_reference
    torch.manual_seed(5)
    b, s, h, kd, vd = 1, 5, 2, 3, 4
    q, k, v = torch.randn(b, s, h, kd), torch.randn(b, s, h, kd), torch.randn(b, s, h, vd)
    W, f = torch.randn(h, vd, vd) * 0.3, torch.rand(b, s, h)
    y, hl = m2rnn_scan_reference(q, k, v, W, f)
    st = torch.zeros(b, h, kd, vd)
    for t in range(s):
        zt = torch.einsum("bhkv,hvw->bhkw", st, W) + k[:, t, :, :, None] * v[:, t, :, None, :]
        ft = f[:, t, :, None, None]
        st = ft * st + (1 - ft) * torch.tanh(zt)
        assert torch.allclose(y[:, t], torch.einsum("bhk,bhkv->bhv", q[:, t], st), atol=1e-5)
    assert torch.allclose(hl, st, atol=1e-5)


def test_cut_cross_entropy_matches_materialised():
    torch.manual_seed(6)
    h = torch.randn(50, 16, requires_grad=True)
    w = torch.randn(40, 16, requires_grad=True)
    t = torch.randint(0, 40, (50,))
    t[::7] = -100
    loss = ops.linear_cross_entropy(h, w, t)
    ref = F.cross_entropy(h @ w.t(), t, ignore_index=-100)
    assert torch.allclose(loss, ref, atol=1e-5)
    g = torch.autograd.grad(loss, (h, w))
    gr = torch.autograd.grad(ref, (h, w))
    assert all(torch.allclose(a, c, atol=1e-5) for a, c in zip(g, gr))


@pytest.mark.parametrize("row_chunk", [7, 50, 4096])
def test_cut_cross_entropy_is_independent_of_the_row_chunk(row_chunk):
    """One chunk, several ragged chunks or one chunk per few rows: same loss and gradients (the weight gradient accumulates over
    chunks, or is written once when a single chunk covers the rows)."""
    torch.manual_seed(16)
    h = torch.randn(50, 16, requires_grad=True)
    w = torch.randn(40, 16, requires_grad=True)
    t = torch.randint(0, 40, (50,))
    t[3] = -100
    mask = torch.ones(50, dtype=torch.bool)
    mask[10:14] = False
    loss = ops.linear_cross_entropy(h, w, t, mask=mask, row_chunk=row_chunk)
    tt = t.clone()
    tt[~mask] = -100
    ref = F.cross_entropy(h @ w.t(), tt, ignore_index=-100)
    assert torch.allclose(loss, ref, atol=1e-5)
    g = torch.autograd.grad(loss * 3.0, (h, w))                # a scaled upstream gradient reaches both gradients
    gr = torch.autograd.grad(ref * 3.0, (h, w))
    assert all(torch.allclose(a, c, atol=2e-5) for a, c in zip(g, gr))


def test_cut_cross_entropy_chunk_size_follows_the_logits_budget():
    from cppmega_mlx_b200.ops import cce
    assert cce.auto_row_chunk(65536) == 32768                  # 4 GiB of bf16 logits: the flagship's 16384 rows are one chunk
    assert cce.auto_row_chunk(131072) == 16384
    assert cce.auto_row_chunk(1 << 22) == cce.DEFAULT_ROW_CHUNK    # never below the rows a GEMM needs to fill the GPU
    assert cce.auto_row_chunk(512) % cce.DEFAULT_ROW_CHUNK == 0


def test_grouped_linear_matches_per_expert_loop():
    from cppmega_mlx_b200.ops.grouped_gemm import grouped_linear
    torch.manual_seed(7)
    counts = [3, 0, 5, 2]
    xs = torch.randn(10, 6, requires_grad=True)
    w = torch.randn(4, 7, 6, requires_grad=True)
    out = grouped_linear(xs, w, counts)
    ref = torch.cat([xs[a:b] @ w[e].t() for e, (a, b) in enumerate([(0, 3), (3, 3), (3, 8), (8, 10)])])
    assert torch.allclose(out, ref, atol=1e-5)
    g = torch.autograd.grad(out.square().sum(), (xs, w))
    gr = torch.autograd.grad(ref.square().sum(), (xs, w))
    assert all(torch.allclose(a, c, atol=1e-4) for a, c in zip(g, gr))


def test_causal_conv_silu_reference():
    from cppmega_mlx_b200.ops.conv import causal_conv1d_silu
    torch.manual_seed(8)
    b, s, C, K = 2, 9, 5, 4
    proj = torch.randn(b, s, 12)
    w, bias = torch.randn(C, K, 1), torch.randn(C)
    out = causal_conv1d_silu(proj, 3, C, C, w, bias)
    x = proj[..., 3:3 + C].transpose(1, 2)
    ref = F.silu(F.conv1d(F.pad(x, (K - 1, 0)), w.permute(0, 2, 1), bias, groups=C)).transpose(1, 2)
    out = out[0] if isinstance(out, tuple) else out
    assert torch.allclose(out, ref, atol=1e-5)


def test_masked_attention_reference_is_causal_and_masked():
    torch.manual_seed(9)
    q, k, v = torch.randn(1, 6, 2, 8), torch.randn(1, 6, 1, 8), torch.randn(1, 6, 1, 4)
    out = ops.masked_attention_reference(q, k, v)
    out = out[0] if isinstance(out, tuple) else out
    ref = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2).expand(1, 2, 6, 8), v.transpose(1, 2).expand(1, 2, 6, 4),
                                         is_causal=True).transpose(1, 2)
    assert torch.allclose(out, ref, atol=1e-5)


def test_dsa_indexer_loss_properties_and_chunking():
    from cppmega_mlx_b200.ops.dsa_indexer_loss import dsa_indexer_loss, dsa_indexer_loss_reference
    torch.manual_seed(11)
    b, s, h, d = 2, 40, 4, 8
    q, k = torch.randn(b, s, h, d), torch.randn(b, s, 1, d)
    scale = d ** -0.5
    # an indexer that reproduces the mean attention distribution exactly has zero loss
    logits = torch.einsum("bqhd,bkd->bhqk", q, k[:, :, 0]) * scale
    causal = torch.tril(torch.ones(s, s, dtype=torch.bool))
    p = torch.softmax(logits.masked_fill(~causal, float("-inf")), -1).mean(1)
    perfect = torch.log(p.clamp_min(1e-30))
    assert float(dsa_indexer_loss_reference(perfect, q, k, softmax_scale=scale)) < 1e-5
    idx_scores = torch.randn(b, s, s, requires_grad=True)
    full = dsa_indexer_loss_reference(idx_scores, q, k, softmax_scale=scale, loss_coeff=0.5)
    assert float(full) > 0
    chunked = dsa_indexer_loss(idx_scores, q, k, softmax_scale=scale, loss_coeff=0.5, q_chunk=16)
    assert torch.allclose(full, chunked, atol=1e-5)
    g, = torch.autograd.grad(chunked, idx_scores)
    assert torch.isfinite(g).all() and float(g.abs().sum()) > 0 and float(g.triu(1).abs().max()) == 0.0     # nothing flows to masked keys
    topk = torch.stack([torch.cat([torch.randperm(i + 1)[:5], torch.full((max(0, 5 - i - 1),), -1)]) for i in range(s)])[None].expand(b, s, 5)
    sparse = dsa_indexer_loss(idx_scores, q, k, softmax_scale=scale, topk_indices=topk, q_chunk=16)
    assert torch.allclose(sparse, dsa_indexer_loss_reference(idx_scores, q, k, softmax_scale=scale, topk_indices=topk), atol=1e-5)
    assert float(dsa_indexer_loss(idx_scores[:, :0], q[:, :0], k, softmax_scale=scale)) == 0.0


def test_sparse_mla_blockscaled_roundtrip_semantics():
    """MXFP8 round trip (1x32 e8m0 scales) on q and kv, straight-through gradients, then the ordinary sparse attention."""
    from cppmega_mlx_b200.ops import mxfp8 as MX
    torch.manual_seed(11)
    b, s, h, d, dv, topk = 1, 12, 2, 64, 32, 5
    q = torch.randn(b, s, h, d, requires_grad=True)
    kv = (torch.randn(b, s, 1, d) * torch.logspace(-2, 1, d)).requires_grad_()
    idx = torch.stack([torch.randperm(s)[:topk] for _ in range(b * s)]).view(b, s, 1, topk).int()
    idx[0, 0, 0, 2:] = -1
    out, lse = ops.sparse_mla_blockscaled(q, kv, idx, d_v=dv)

    def rt(x):
        qv, e = MX.quantize_mxfp8_reference(x.detach().reshape(-1, d))
        return MX.dequantize_mxfp8_reference(qv, e).view(x.shape)
    ref, ref_lse = ops.sparse_mla_reference(rt(q), rt(kv), idx, d_v=dv)
    assert torch.allclose(out, ref, atol=1e-6) and torch.allclose(lse, ref_lse, atol=1e-6)
    assert not torch.allclose(out, ops.sparse_mla_reference(q, kv, idx, d_v=dv)[0], atol=1e-4)   # the quantisation is visible
    # e8m0 scales are powers of two and every recovered value is e4m3-representable after scaling
    r = rt(kv).view(-1, d // 32, 32)
    sc = torch.exp2(torch.ceil(torch.log2(kv.detach().reshape(-1, d // 32, 32).abs().amax(-1) / 448.0)))[..., None]
    assert torch.equal((r / sc).to(torch.float8_e4m3fn).float() * sc, r)
    out.sum().backward()
    q2, kv2 = rt(q).requires_grad_(), rt(kv).requires_grad_()
    ops.sparse_mla_reference(q2, kv2, idx, d_v=dv)[0].sum().backward()
    assert torch.allclose(q.grad, q2.grad, atol=1e-6) and torch.allclose(kv.grad, kv2.grad, atol=1e-6)   # straight-through
    # a head dimension that is not a multiple of 32 bypasses the quantisation
    q3, kv3 = torch.randn(1, 4, 2, 24), torch.randn(1, 4, 1, 24)
    i3 = torch.arange(4).view(1, 1, 1, 4).expand(1, 4, 1, 4).int().contiguous()
    assert torch.equal(ops.sparse_mla_blockscaled(q3, kv3, i3)[0], ops.sparse_mla_attention(q3, kv3, i3)[0])


def test_fp8_amax_quantize_pack_oracle():
    """Per-tensor FP8 scaling on the CPU path: NaNs are ignored by the abs-max, quantise clamps to ±448 and rounds to e4m3, and
    pack's scale reproduces the tensor to e4m3 precision."""
    import torch
    from cppmega_mlx_b200 import ops
    x = torch.randn(7, 33) * 3
    x[2, 5] = float("nan")
    x[0, 0] = -37.5
    a = ops.fp8_amax(x)
    assert a.shape == (1,) and float(a) == 37.5
    joint = ops.fp8_amax(torch.full((3,), 50.0), out=a.clone())
    assert float(joint) == 50.0
    clean = torch.nan_to_num(x, nan=0.0)
    q = ops.fp8_quantize(clean, 1000.0)
    assert q.dtype == torch.float8_e4m3fn and float(q.float().abs().max()) == 448.0
    q2, scale = ops.fp8_pack(clean)
    assert abs(float(scale) - 37.5 / 448) < 1e-7
    back = q2.float() * scale
    assert float((back - clean).abs().max()) <= 37.5 / 448 * 16 + 1e-6        # half an ulp at the top binade (ulp = 32 · scale)
    y, am = ops.linear_with_amax(torch.randn(5, 16), torch.randn(8, 16))
    assert abs(float(am) - float(y.abs().max())) < 1e-6
