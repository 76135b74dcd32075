"""Fused optimizer kernels against the PyTorch restatements of the same updates."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(make, shapes, steps=3, dtype=torch.bfloat16, kernels=True, seed=0):
    from cppmega_mlx_b200.ops import _backend as B
    torch.manual_seed(seed)
    ps = [(f"layers.{i}.w", torch.nn.Parameter((torch.randn(*s, device="cuda") * 0.1).to(dtype))) for i, s in enumerate(shapes)]
    gs = [[(torch.randn(*s, device="cuda") * 0.01).to(dtype) for s in shapes] for _ in range(steps)]
    with B.use_kernels(kernels):
        opt = make(ps)
        for st in range(steps):
            for (_, p), g in zip(ps, gs[st]):
                p.grad = g.clone()
            opt.step()
    torch.cuda.synchronize()
    return [p.detach().float() for _, p in ps]


@pytest.mark.parametrize("name", ["adamw", "adam8bit", "adam8bit_dyn", "lion8bit", "lion8bit_dyn"])
def test_elementwise_optimizers_match(name):
    from cppmega_mlx_b200.training.optimizers import make_adamw
    from cppmega_mlx_b200.training.optimizers_quantized import make_adam8bit, make_lion8bit
    mk = {"adamw": lambda p: make_adamw(p, learning_rate=1e-2),
          "adam8bit": lambda p: make_adam8bit(p, learning_rate=1e-2),
          "adam8bit_dyn": lambda p: make_adam8bit(p, learning_rate=1e-2, quant_scheme="dynamic_int8_v1"),
          "lion8bit": lambda p: make_lion8bit(p, learning_rate=1e-3),
          "lion8bit_dyn": lambda p: make_lion8bit(p, learning_rate=1e-3, quant_scheme="dynamic_int8_v1")}[name]
    shapes = [(300, 70), (1000,), (64, 64)]
    a = _run(mk, shapes, kernels=True)
    b = _run(mk, shapes, kernels=False)
    for x, y in zip(a, b):
        assert (x - y).abs().max() < 2e-2 * y.abs().max() + 2e-3


def test_adamw_bias_correction_kernel_matches_torch_adamw():
    """With bias correction on, the kernel path, the PyTorch restatement and ``torch.optim.AdamW`` take the same steps."""
    from cppmega_mlx_b200.training.optimizers import make_adamw
    shapes = [(257, 33), (512,)]
    mk = lambda p: make_adamw(p, learning_rate=1e-2, weight_decay=0.1, bias_correction=True)
    a = _run(mk, shapes, steps=4, dtype=torch.float32, kernels=True)
    b = _run(mk, shapes, steps=4, dtype=torch.float32, kernels=False)
    torch.manual_seed(0)
    ps = [torch.nn.Parameter(torch.randn(*s, device="cuda") * 0.1) for s in shapes]
    gs = [[torch.randn(*s, device="cuda") * 0.01 for s in shapes] for _ in range(4)]
    ref = torch.optim.AdamW(ps, lr=1e-2, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.1)
    for st in range(4):
        for p, g in zip(ps, gs[st]):
            p.grad = g.clone()
        ref.step()
    for x, y, z in zip(a, b, ps):
        assert (x - y).abs().max() < 1e-5
        assert (x - z.detach()).abs().max() < 1e-4      # the first step alone moves every weight by ≈ lr = 1e-2


def test_muon_fused_matches_reference():
    from cppmega_mlx_b200.training.optimizers import MuonWithNSCarrier
    mk = lambda p: MuonWithNSCarrier(p, 2e-2, ns_carrier="bf16")
    shapes = [(256, 512), (768, 256), (128, 128)]
    a = _run(mk, shapes, kernels=True)
    b = _run(mk, shapes, kernels=False)
    for x, y in zip(a, b):
        assert (x - y).abs().max() < 3e-2, (x - y).abs().max()


def test_newton_schulz_orthogonalises():
    from cppmega_mlx_b200.ops.optim import newton_schulz5_bf16_
    torch.manual_seed(0)
    for shape in [(512, 1024), (1024, 256)]:
        u = torch.randn(*shape, device="cuda").bfloat16()
        ss = (u.float() ** 2).sum().reshape(1)
        o = newton_schulz5_bf16_(u.clone(), ss)
        sv = torch.linalg.svdvals(o.float())
        assert sv.max() < 1.35 and sv.min() > 0.4, (sv.min().item(), sv.max().item())


@pytest.mark.parametrize("n,pad", [(64, 0), (100, 4), (2048, 0), (511, 1), (130, 0)])
def test_mirror_lower_completes_symmetric_matrix(n, pad):
    """The Gram GEMM only computes tiles on or below the diagonal; the mirror kernel fills in the rest (vector and scalar forms)."""
    import ctypes

    from cppmega_mlx_b200.ops import _backend as B
    lib = B.load_library()
    torch.manual_seed(n)
    full = torch.randn(n, n + pad, device="cuda").bfloat16()
    g = full[:, :n]                                   # row pitch n + pad
    want = torch.tril(g.float()) + torch.tril(g.float(), -1).t()
    rc = lib.cmb_mirror_lower(ctypes.c_void_p(g.data_ptr()), n, ctypes.c_longlong(full.stride(0)),
                              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert rc == 0 and torch.equal(g.float(), want)
