"""Chunked Mamba3 scan kernels vs the token-by-token fp32 oracle (forward, final state, all gradients)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(Bn, S, H, G, P, N, seed=0, h0=True):
    torch.manual_seed(seed)
    dev = "cuda"
    mk = lambda *s: (torch.randn(*s, device=dev) * 0.5).bfloat16().requires_grad_()
    x, z = mk(Bn, S, H, P), mk(Bn, S, H, P)
    Bm, Cm = mk(Bn, S, G, N), mk(Bn, S, G, N)
    A = (-torch.rand(Bn, S, H, device=dev) - 0.1).requires_grad_()
    dt = (torch.rand(Bn, S, H, device=dev) * 0.2 + 0.01).requires_grad_()
    D = torch.randn(H, device=dev).requires_grad_()
    h = (torch.randn(Bn, H, P, N, device=dev) * 0.3).requires_grad_() if h0 else None
    return [x, Bm, Cm, z, A, dt, D, h]


@pytest.mark.parametrize("shape", [(2, 256, 4, 2, 64, 128, 128), (1, 512, 8, 8, 64, 64, 256), (2, 128, 4, 1, 32, 64, 64)])
@pytest.mark.parametrize("with_h0", [True, False])
def test_mamba3_scan_matches_sequential(shape, with_h0):
    from cppmega_mlx_b200 import ops
    from cppmega_mlx_b200.ops import _backend as B
    from cppmega_mlx_b200.ops import mamba3_scan_cuda
    Bn, S, H, G, P, N, L = shape
    ins = _inputs(Bn, S, H, G, P, N, h0=with_h0)
    assert mamba3_scan_cuda.supported(ins[0], ins[1], L)
    out, hl = ops.mamba3_scan(*ins[:7], ins[7], chunk_size=L)
    go = torch.randn_like(out)
    gh = torch.randn_like(hl) * 0.1
    wrt = [t for t in ins if t is not None]
    grads = torch.autograd.grad([out, hl], wrt, [go, gh])
    torch.cuda.synchronize()
    B.check_status()
    ref_in = [None if t is None else t.detach().float().requires_grad_() for t in ins]
    ro, rh = ops.mamba3_scan_sequential(*ref_in[:7], ref_in[7])
    rgrads = torch.autograd.grad([ro, rh], [t for t in ref_in if t is not None], [go.float(), gh.float()])

    def close(a, b, name, rel=3e-2):
        err = (a.float() - b.float()).abs().max().item()
        scale = b.float().abs().max().item() + 1e-3
        assert err <= rel * scale, f"{name}: err {err} scale {scale}"

    close(out, ro, "out")
    close(hl, rh, "h_last")
    names = [n for n, t in zip(["x", "B", "C", "z", "A", "dt", "D", "h0"], ins) if t is not None]
    for n, a, b in zip(names, grads, rgrads):
        close(a, b, "d" + n, rel=5e-2)


def test_fused_prep_matches_framework_ops(monkeypatch):
    """The fused B/C/dt/A preparation against the PyTorch statement of the same math (both feeding the kernel scan)."""
    import copy

    from cppmega_mlx_b200.nn.mamba3 import Mamba3Block, Mamba3Config
    from cppmega_mlx_b200.ops import _backend as B
    from cppmega_mlx_b200.ops import mamba3_prep as MP
    torch.manual_seed(0)
    blk = Mamba3Block(Mamba3Config(d_model=512, headdim=64, d_state=128, ngroups=8, chunk_size=64, d_conv=4)).cuda().bfloat16()
    with torch.no_grad():
        for n in ("B_norm_weight", "C_norm_weight", "B_bias", "C_bias"):
            getattr(blk, n).add_(torch.randn_like(getattr(blk, n)) * 0.2)
    ref = copy.deepcopy(blk)
    x = (torch.randn(2, 320, 512, device="cuda") * 0.5).bfloat16()
    g = torch.randn(2, 320, 512, device="cuda").bfloat16()

    def run(mod, fused):
        monkeypatch.setattr(MP, "supported", (lambda *a, **k: fused) if not fused else MP.__dict__["_orig_supported"])
        xi = x.clone().requires_grad_()
        y = mod(xi)[0]
        y.backward(g)
        return y.detach().float(), xi.grad.float(), {n: p.grad.float() for n, p in mod.named_parameters()}
    MP.__dict__.setdefault("_orig_supported", MP.supported)
    n0 = B.launch_count()
    yf, gxf, gpf = run(blk, True)
    fused_launches = B.launch_count() - n0
    yr, gxr, gpr = run(ref, False)
    B.check_status()
    assert fused_launches > 0

    def rel(a, b):
        return float((a - b).abs().max()) / (float(b.abs().max()) + 1e-6)
    assert rel(yf, yr) < 3e-2
    assert rel(gxf, gxr) < 5e-2
    for n in gpr:
        assert rel(gpf[n], gpr[n]) < 6e-2, (n, rel(gpf[n], gpr[n]))


@pytest.mark.parametrize("groups,state", [(8, 128), (2, 64), (1, 16)])
def test_single_step_kernel_matches_sequence_path(groups, state):
    """The one-launch decode step reproduces the sequence path run with S == 1 (outputs and every cache tensor)."""
    from cppmega_mlx_b200.nn.mamba3 import Mamba3Block, Mamba3Config
    from cppmega_mlx_b200.ops import _backend as B
    torch.manual_seed(3)
    blk = Mamba3Block(Mamba3Config(d_model=512, headdim=64, d_state=state, ngroups=groups, chunk_size=64)).cuda().bfloat16().eval()
    with torch.no_grad():
        for prm in (blk.B_bias, blk.C_bias, blk.conv_bias):
            prm.normal_(0, 0.3)
        blk.D.normal_(1, 0.2)
        x = torch.randn(3, 20, 512, device="cuda").bfloat16()
        _, cache = blk(x[:, :16], return_cache=True)
        got_c, ref_c = cache, cache
        for i in range(16, 20):
            before = B.launch_count()
            got, got_c = blk(x[:, i:i + 1], cache=got_c, return_cache=True)
            launches = B.launch_count() - before
            with B.use_kernels(False):
                ref, ref_c = blk(x[:, i:i + 1], cache=ref_c, return_cache=True)
            assert launches <= 4        # in_proj, step, out_proj
            assert (got.float() - ref.float()).abs().max() <= 3e-2 * max(1.0, float(ref.float().abs().max()))
            for name in ("angle_dt", "ssm", "k", "v", "conv"):
                a, r = getattr(got_c, name).float(), getattr(ref_c, name).float()
                assert a.shape == r.shape
                if name == "angle_dt":   # phases are compared on the circle
                    d = (a - r).abs()
                    d = torch.minimum(d, (2 * torch.pi - d).abs())
                    assert d.max() < 5e-2
                else:
                    assert (a - r).abs().max() <= 3e-2 * max(1.0, float(r.abs().max())), name


@pytest.mark.parametrize("groups,state,seq", [(8, 128, 200), (2, 64, 2)])
def test_prefill_cache_on_fused_path_matches_framework_path(groups, state, seq):
    """A from-scratch prefill on the fused kernels builds the same decode cache as the PyTorch-op path."""
    from cppmega_mlx_b200.nn.mamba3 import Mamba3Block, Mamba3Config
    from cppmega_mlx_b200.ops import _backend as B
    torch.manual_seed(4)
    blk = Mamba3Block(Mamba3Config(d_model=512, headdim=64, d_state=state, ngroups=groups, chunk_size=64)).cuda().bfloat16().eval()
    with torch.no_grad():
        for prm in (blk.B_bias, blk.C_bias, blk.conv_bias):
            prm.normal_(0, 0.3)
        x = torch.randn(2, seq, 512, device="cuda").bfloat16()
        before = B.launch_count()
        got_y, got = blk(x, return_cache=True)
        assert B.launch_count() - before >= 3            # the kernel path ran
        with B.use_kernels(False):
            ref_y, ref = blk(x, return_cache=True)
    assert (got_y.float() - ref_y.float()).abs().max() <= 3e-2 * max(1.0, float(ref_y.float().abs().max()))
    for name in ("angle_dt", "ssm", "k", "v", "conv"):
        a, r = getattr(got, name).float(), getattr(ref, name).float()
        assert a.shape == r.shape, name
        if name == "angle_dt":
            d = (a - r).abs()
            assert torch.minimum(d, (2 * torch.pi - d).abs()).max() < 6e-2
        else:
            assert (a - r).abs().max() <= 4e-2 * max(1.0, float(r.abs().max())), name


def test_fused_prep_with_supplied_phase_dt_equals_the_local_phase_heads():
    """Head-parallel layers hand the rotary phase's step sizes in from outside.  Supplying exactly the dt of the first ``ngroups``
    local heads (computed differentiably from the same tail and bias) must reproduce the plain op: outputs, and the gradients of
    tail and bias once both paths are added up."""
    from cppmega_mlx_b200.ops import _backend as B
    from cppmega_mlx_b200.ops import mamba3_prep as MP
    torch.manual_seed(0)
    dev, b, s, H, G, N, R = "cuda", 2, 200, 32, 8, 128, 32
    BC = (torch.randn(b, s, 2 * G * N, device=dev) * 0.5).bfloat16()
    tail = (torch.randn(b, s, 3 * H + R, device=dev) * 0.5).bfloat16()
    bias = (torch.randn(H, device=dev) * 0.1).bfloat16()
    w = [(1 + 0.1 * torch.randn(1, G, N, device=dev)).bfloat16() for _ in range(2)] + [(0.1 * torch.randn(1, G, N, device=dev)).bfloat16() for _ in range(2)]
    wB, wC, bB, bC = w
    assert MP.supported(BC, tail, (wB, bB, wC, bC, bias), H, G, N, R)
    gs = [torch.randn(b, s, G, N, device=dev).bfloat16(), torch.randn(b, s, G, N, device=dev).bfloat16(),
          torch.randn(b, s, H, device=dev), torch.randn(b, s, H, device=dev)]

    def run(with_phase):
        t, bi, bc = tail.clone().requires_grad_(), bias.clone().requires_grad_(), BC.clone().requires_grad_()
        ph = torch.nn.functional.softplus(t[..., :G].float() + bi[:G].float()) if with_phase else None
        outs = MP.mamba3_prep(bc, t, bi, wB, bB, wC, bC, nheads=H, ngroups=G, d_state=N, num_angles=R, a_floor=0.01, phase_dt=ph)
        torch.autograd.backward(outs, gs)
        return [o.detach().float() for o in outs], t.grad.float(), bi.grad.float(), bc.grad.float()
    o0, gt0, gb0, gbc0 = run(False)
    o1, gt1, gb1, gbc1 = run(True)
    B.check_status()
    for a, c in zip(o0, o1):
        assert torch.allclose(a, c, atol=2e-2, rtol=2e-2)
    rel = lambda x, y: float((x - y).abs().max()) / (float(y.abs().max()) + 1e-6)
    assert rel(gbc1, gbc0) < 2e-2
    assert rel(gt1, gt0) < 3e-2, rel(gt1, gt0)
    assert rel(gb1, gb0) < 3e-2, rel(gb1, gb0)
