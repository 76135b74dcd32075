"""tcgen05 GEMM vs fp32 torch.matmul, all operand layouts, odd sizes, both output types."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, a_mn, b_mn):
    A = a.float().t() if a_mn else a.float()
    Bm = b.float().t() if b_mn else b.float()
    return A @ Bm.t()


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (384, 320, 192), (1000, 136, 72), (4096, 2048, 2048),
                                   (130, 128, 64), (64, 64, 4096)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
def test_gemm_layouts(M, N, K, a_mn, b_mn):
    from cppmega_mlx_b200 import ops
    from cppmega_mlx_b200.ops import _backend as B
    torch.manual_seed(M + N + K)
    dev = "cuda"
    a = torch.randn((K, M) if a_mn else (M, K), device=dev).bfloat16()
    b = torch.randn((K, N) if b_mn else (N, K), device=dev).bfloat16()
    if (a.shape[1] % 8) or (b.shape[1] % 8):
        pytest.skip("pitch not a multiple of 8")
    c = ops.gemm_raw(a, b, a_mn=a_mn, b_mn=b_mn)
    torch.cuda.synchronize()
    B.check_status()
    ref = _ref(a, b, a_mn, b_mn)
    err = (c.float() - ref).abs().max().item()
    tol = 2e-2 * (K ** 0.5) + 1e-2 * ref.abs().max().item()
    assert err < tol, f"max err {err} (tol {tol})"
    c32 = ops.gemm_raw(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert (c32 - ref).abs().max().item() < 1e-3 * (K ** 0.5) + 1e-4 * ref.abs().max().item()


def test_gemm_accumulate_and_linear_grads():
    from cppmega_mlx_b200 import ops
    torch.manual_seed(0)
    x = torch.randn(512, 256, device="cuda").bfloat16().requires_grad_()
    w = torch.randn(384, 256, device="cuda").bfloat16().requires_grad_()
    y = ops.linear(x, w)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = xr @ wr.t()
    yr.backward(g.float())
    assert (y.float() - yr).abs().max() < 0.5
    assert (x.grad.float() - xr.grad).abs().max() < 0.6
    assert (w.grad.float() - wr.grad).abs().max() < 0.8
    acc = torch.ones(512, 384, device="cuda", dtype=torch.float32)
    ops.gemm_raw(x.detach(), w.detach(), out=acc, accumulate=True)
    assert (acc - 1 - yr.detach()).abs().max() < 1e-2


def test_gemm_batched_shared_operand_and_decay_epilogue():
    """[b, c, h] batch with the B operand shared per group of heads and the decay-mask epilogue."""
    from cppmega_mlx_b200 import ops
    from cppmega_mlx_b200.ops import _backend as Bk
    torch.manual_seed(1)
    nb_, nc, H, G, L, N = 2, 3, 4, 2, 256, 128
    C = torch.randn(nb_, nc, G, L, N, device="cuda").bfloat16()
    Bm = torch.randn(nb_, nc, G, L, N, device="cuda").bfloat16()
    cum = -torch.rand(nb_, nc, H, L, device="cuda").cumsum(-1) * 0.05
    out = torch.empty(nb_, nc, H, L, L, device="cuda", dtype=torch.bfloat16)
    ops.gemm_batched(C, Bm, out, M=L, N=L, K=N, a_mn=False, b_mn=False, lda=N, ldb=N, ldc=L, nb=(H, nc, nb_),
                     sA=(L * N, G * L * N, nc * G * L * N), sB=(L * N, G * L * N, nc * G * L * N),
                     sC=(L * L, H * L * L, nc * H * L * L), a_div2=H // G, b_div2=H // G, row_vec=cum, col_vec=cum,
                     sv=(L, H * L, nc * H * L))
    torch.cuda.synchronize()
    Bk.check_status()
    Gm = torch.einsum("bcgln,bcgsn->bcgls", C.float(), Bm.float()).repeat_interleave(H // G, dim=2)
    dec = torch.exp(cum[..., :, None] - cum[..., None, :])
    ref = Gm * dec * torch.ones(L, L, device="cuda").tril()
    err = (out.float() - ref).abs().max().item()
    assert err < 0.02 * ref.abs().max().item() + 0.05, err


def test_gemm_batched_mn_major_strided_views():
    """Y[b,c,h] = M[b,c,h] (L×L) · X[b, cL:(c+1)L, h, :] with X addressed in place (MN-major, strided)."""
    from cppmega_mlx_b200 import ops
    torch.manual_seed(2)
    nb_, nc, H, L, P = 2, 2, 3, 256, 64
    S = nc * L
    Mm = torch.randn(nb_, nc, H, L, L, device="cuda").bfloat16()
    X = torch.randn(nb_, S, H, P, device="cuda").bfloat16()
    Y = torch.empty(nb_, S, H, P, device="cuda", dtype=torch.float32)
    ops.gemm_batched(Mm, X, Y, M=L, N=P, K=L, a_mn=False, b_mn=True, lda=L, ldb=H * P, ldc=H * P, nb=(H, nc, nb_),
                     sA=(L * L, H * L * L, nc * H * L * L), sB=(P, L * H * P, S * H * P), sC=(P, L * H * P, S * H * P))
    torch.cuda.synchronize()
    ref = torch.einsum("bchls,bcshp->bclhp", Mm.float(), X.float().view(nb_, nc, L, H, P)).reshape(nb_, S, H, P)
    assert (Y - ref).abs().max().item() < 1e-2 * ref.abs().max().item() + 1e-2


@pytest.mark.parametrize("M,N,K,bias", [(1, 2048, 2048, False), (3, 1000, 5632, True), (8, 65536, 2048, False), (5, 24, 4104, False)])
def test_skinny_linear_matches_fp32(M, N, K, bias):
    """Decode-shape linears (≤ 8 rows, no autograd) take the weight-streaming kernel."""
    from cppmega_mlx_b200 import ops
    from cppmega_mlx_b200.ops import _backend as B
    torch.manual_seed(M + N)
    x = torch.randn(2, M, K, device="cuda").bfloat16()[0]          # a row-sliced view
    w = torch.randn(N, K, device="cuda").bfloat16()
    bvec = torch.randn(N, device="cuda").bfloat16() if bias else None
    before = B.launch_count()
    with torch.no_grad():
        y = ops.linear(x, w, bvec)
    assert B.launch_count() == before + 1
    ref = x.float() @ w.float().t() + (bvec.float() if bias else 0)
    assert y.shape == (M, N)
    assert (y.float() - ref).abs().max() <= 2e-2 * ref.abs().max()
    xr = x.clone().requires_grad_()                                # with autograd the tensor-core GEMM path is kept
    assert ops.linear(xr, w).requires_grad


@pytest.mark.parametrize("M,N,K,bias", [(2, 2048, 2048, False), (8, 1000, 5632, True), (16, 65536, 2048, False), (17, 2048, 5632, True),
                                        (32, 11264, 2048, False), (5, 24, 4104, False), (31, 9480, 40, True), (1, 4096, 2048, False)])
def test_skinny_mma_linear_matches_fp32(M, N, K, bias):
    """2–32 activation rows: warp-MMA weight streaming with the contraction split over the warps of a CTA."""
    from cppmega_mlx_b200.ops import gemm as G
    torch.manual_seed(M * 7 + N)
    x = torch.randn(2, M, K, device="cuda").bfloat16()[1]
    w = torch.randn(N + 3, K, device="cuda").bfloat16()[3:]         # a row-offset view (still 16-byte aligned rows)
    bvec = torch.randn(N, device="cuda").bfloat16() if bias else None
    with torch.no_grad():
        y = G.skinny_mma_linear(x, w, bvec)
    ref = x.float() @ w.float().t() + (bvec.float() if bias else 0)
    assert y.shape == (M, N) and y.dtype == torch.bfloat16
    assert (y.float() - ref).abs().max() <= 1e-2 * ref.abs().max()
    if G.MMA_MIN_ROWS <= M <= G.MMA_MAX_ROWS:                       # and ``linear`` routes these row counts here
        from cppmega_mlx_b200 import ops
        with torch.no_grad():
            assert torch.equal(ops.linear(x, w, bvec), y)


@pytest.mark.parametrize("M,N,K", [(9, 2048, 5632), (32, 11264, 2048), (64, 2048, 2048), (33, 4096, 320)])
def test_small_m_linear_split_k_matches_fp32(M, N, K):
    """Swapped operands + contraction split over the GPU (fp32 partial sums) for a few dozen activation rows."""
    from cppmega_mlx_b200.ops import _backend as B
    from cppmega_mlx_b200.ops import gemm as G
    torch.manual_seed(M)
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = torch.randn(N, K, device="cuda").bfloat16()
    with torch.no_grad():
        y = G.small_m_linear(x, w)
    B.check_status()
    ref = x.float() @ w.float().t()
    assert y.shape == (M, N) and y.dtype == torch.bfloat16 and y.is_contiguous()
    assert (y.float() - ref).abs().max() <= 2e-2 * ref.abs().max()


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 512, 256), (1000, 328, 192), (4096, 2048, 2048), (384, 5632, 512)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
def test_gemm_cta_pair_form_matches_fp32(M, N, K, a_mn, b_mn):
    """The cta_group::2 form (two SMs per 256-row tile, half of B staged per CTA) against fp32, every operand layout, ragged
    edges in M and N, bf16 / fp32 / accumulating outputs and the alpha·acc + beta·aux epilogue."""
    from cppmega_mlx_b200 import ops
    from cppmega_mlx_b200.ops import _backend as B
    from cppmega_mlx_b200.ops import gemm as G
    torch.manual_seed(M + N + K)
    dev = "cuda"
    a = torch.randn((K, M) if a_mn else (M, K), device=dev).bfloat16()
    b = torch.randn((K, N) if b_mn else (N, K), device=dev).bfloat16()
    ref = _ref(a, b, a_mn, b_mn)
    tol = 2e-2 * (K ** 0.5) + 1e-2 * ref.abs().max().item()
    prev = G.set_pair_mode(True)
    try:
        c = ops.gemm_raw(a, b, a_mn=a_mn, b_mn=b_mn)
        c32 = ops.gemm_raw(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
        acc = torch.ones(M, N, device=dev, dtype=torch.float32)
        ops.gemm_raw(a, b, a_mn=a_mn, b_mn=b_mn, out=acc, accumulate=True)
        aux = torch.randn(M, N, device=dev).bfloat16()
        ax = G.gemm_axpby(a, b, aux, a_mn=a_mn, b_mn=b_mn, alpha=0.5, beta=2.0)
        torch.cuda.synchronize()
        B.check_status()
    finally:
        G.set_pair_mode(prev)
    assert (c.float() - ref).abs().max().item() < tol
    assert (c32 - ref).abs().max().item() < 1e-3 * (K ** 0.5) + 1e-4 * ref.abs().max().item()
    assert (acc - 1.0 - ref).abs().max().item() < 1e-3 * (K ** 0.5) + 1e-4 * ref.abs().max().item()
    assert (ax.float() - (0.5 * ref + 2.0 * aux.float())).abs().max().item() < tol
    # the pair form is bit-identical to the single-CTA form: same products, same accumulation order
    c1 = ops.gemm_raw(a, b, a_mn=a_mn, b_mn=b_mn)
    assert torch.equal(c, c1)


@pytest.mark.parametrize("m,k,batch", [(512, 256, 1), (1024, 320, 3), (768, 2048, 2)])
def test_symmetric_product_with_mirror_in_cta_pair_form(m, k, batch):
    """X·Xᵀ with lower-triangle tile skipping and the in-epilogue mirror: the pair form (256-row tiles) fills the whole matrix,
    matches fp32 and equals the single-CTA form bit for bit."""
    from cppmega_mlx_b200.ops import _backend as B
    from cppmega_mlx_b200.ops import gemm as G
    torch.manual_seed(m + k)
    x = torch.randn(batch, m, k, device="cuda").bfloat16()
    ref = x.float() @ x.float().transpose(1, 2)
    outs = {}
    for mode in (True, False):
        prev = G.set_pair_mode(mode)
        try:
            out = torch.full((batch, m, m), float("nan"), device="cuda", dtype=torch.bfloat16)
            G.gemm_batched(x, x, out, M=m, N=m, K=k, a_mn=False, b_mn=False, lda=k, ldb=k, ldc=m, nb=(batch, 1, 1), sA=(m * k, 0, 0),
                           sB=(m * k, 0, 0), sC=(m * m, 0, 0), flags=G.CAUSAL_SKIP | G.EPI_SYM_MIRROR)
            torch.cuda.synchronize()
            B.check_status()
        finally:
            G.set_pair_mode(prev)
        outs[mode] = out
    assert not bool(torch.isnan(outs[True]).any())
    assert (outs[True].float() - ref).abs().max().item() < 2e-2 * (k ** 0.5) + 1e-2 * ref.abs().max().item()
    assert torch.equal(outs[True], outs[False])


@pytest.mark.parametrize("M,N,K", [(512, 384, 256), (130, 136, 64), (4096, 2048, 1024)])
def test_linear_relu2_epilogue_matches_fp32(M, N, K):
    """relu(x·Wᵀ)² from the GEMM epilogue, forward and both gradients, against fp32 PyTorch ops."""
    from cppmega_mlx_b200 import ops
    torch.manual_seed(M + N)
    x = (torch.randn(M, K, device="cuda") * 0.5).bfloat16().requires_grad_()
    w = (torch.randn(N, K, device="cuda") * 0.1).bfloat16().requires_grad_()
    y = ops.linear_relu2(x, w)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = torch.relu(xr @ wr.t()) ** 2
    yr.backward(g.float())
    close = lambda a, b, r: (a.float() - b).abs().max().item() <= r * (b.abs().max().item() + 1e-6)
    assert close(y, yr, 2e-2)
    assert close(x.grad, xr.grad, 3e-2)
    assert close(w.grad, wr.grad, 3e-2)


@pytest.mark.parametrize("act", ["relu2", "gelu"])
def test_moe_experts_with_non_gated_activations_use_the_grouped_kernels(act):
    """relu2 / gelu experts run the padded grouped GEMMs (relu2 fused into the up product's epilogue) and match the per-expert
    PyTorch loop of the same bf16 module, outputs and gradients."""
    from cppmega_mlx_b200.nn.moe import MoE, MoEConfig
    from cppmega_mlx_b200.ops import _backend as B
    torch.manual_seed(0)
    cfg = MoEConfig(d_model=128, num_experts=8, top_k=2, expert_hidden_size=256, activation=act, shared_expert_hidden_size=None)
    moe = MoE(cfg).cuda().bfloat16()
    x0 = (torch.randn(4, 96, 128, device="cuda") * 0.5).bfloat16()

    def run(kernels: bool):
        moe.zero_grad()
        x = x0.clone().requires_grad_()
        with B.use_kernels(kernels):
            before = B.launch_count()
            y = moe(x)
            y = y[0] if isinstance(y, tuple) else y
            launches = B.launch_count() - before
            y.float().square().mean().backward()
        return y.detach().float(), x.grad.float(), moe.experts.w_gate_up.grad.float().clone(), moe.experts.w_down.grad.float().clone(), launches
    yk, gxk, gu_k, gd_k, n_k = run(True)
    yr, gxr, gu_r, gd_r, _ = run(False)
    B.check_status()
    assert n_k > 0
    close = lambda a, b, r: (a - b).abs().max().item() <= r * (b.abs().max().item() + 1e-9)
    assert close(yk, yr, 3e-2)
    assert close(gxk, gxr, 6e-2)
    assert close(gu_k, gu_r, 6e-2)
    assert close(gd_k, gd_r, 6e-2)
