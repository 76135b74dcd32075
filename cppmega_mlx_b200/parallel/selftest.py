"""Multi-GPU self-tests, launched with torchrun: ``python -m torch.distributed.run --nproc-per-node N -m
cppmega_mlx_b200.parallel.selftest <case>``.  Rank 0 prints one JSON line with the comparison result.

Cases: ``zero1`` — the fused symmetric-memory ZeRO-1 step against the NCCL reduce-scatter / all-gather step on the same
model, data and seeds (loss trajectory and final parameters must agree to bf16 tolerance); ``tp`` — a sequence-parallel
tensor-parallel SwiGLU FFN, forward and backward, with the fused GEMM↔collective pairs of ``fused_tp.py`` against the NCCL
pairs of ``tp.py`` (results and device time).
"""
from __future__ import annotations

import json
import os
import sys

import torch
import torch.distributed as dist


def _setup():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    return rank, world, dev


def _train(comm: str, steps: int, dev, rank: int, world: int):
    from cppmega_mlx_b200.data.batch import LMTokenBatch
    from cppmega_mlx_b200.models.hybrid_lm import HybridTinyConfig, HybridTinyLM
    from cppmega_mlx_b200.training.compiled import PretrainingStep
    from cppmega_mlx_b200.training.distributed_optimizer import DistributedZeRO1Optimizer
    from cppmega_mlx_b200.training.optimizers import make_muon
    torch.manual_seed(0)
    cfg = HybridTinyConfig(vocab_size=512, hidden_size=256, pattern="MA", depth=2, num_attention_heads=4, max_seq_length=256,
                           mamba_head_dim=64, mamba_state_dim=64, mamba_chunk_size=64, mamba_groups=2, mla_low_rank=True,
                           mla_q_lora_rank=128, mla_kv_lora_rank=128, mla_qk_nope_head_dim=64, mla_qk_rope_head_dim=32,
                           mla_v_head_dim=64, ffn_hidden_size=512, position_embedding=False)
    model = HybridTinyLM(cfg).to(dev, torch.bfloat16)
    opt = DistributedZeRO1Optimizer(model, lambda ps: make_muon(ps, lr_muon=2e-2, lr_adamw=1e-3, ns_carrier="bf16"), comm=comm)
    opt.zero_grad()
    step = PretrainingStep(model, opt, device=dev)
    gen = torch.Generator().manual_seed(100 + rank)
    losses = []
    for _ in range(steps):
        b = LMTokenBatch(tokens=torch.randint(0, 512, (2, 257), generator=gen))
        m = step(b)
        t = torch.tensor([m.loss], device=dev)
        dist.all_reduce(t)
        losses.append(float(t) / world)
    flat = torch.cat([p.detach().float().reshape(-1) for p in model.parameters()])
    fused = getattr(opt, "_fused", None)
    _train.multimem = bool(fused is not None and getattr(fused, "use_mc", 0))     # reported by the zero1 case
    return losses, flat


def case_zero1(rank, world, dev):
    from cppmega_mlx_b200.ops import _backend as B
    l_n, p_n = _train("nccl", 4, dev, rank, world)
    l_f, p_f = _train("fused", 4, dev, rank, world)
    torch.cuda.synchronize()
    B.check_status()
    diff = (p_n - p_f).abs().max()
    dist.all_reduce(diff, op=dist.ReduceOp.MAX)
    mean = (p_n - p_f).abs().mean()
    dist.all_reduce(mean, op=dist.ReduceOp.MAX)
    # every rank must hold identical parameters after the fused step
    ref = p_f.clone()
    dist.broadcast(ref, 0)
    spread = (ref - p_f).abs().max()
    dist.all_reduce(spread, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(json.dumps({"case": "zero1", "world": world, "loss_nccl": l_n, "loss_fused": l_f,
                          "max_param_diff": float(diff), "mean_param_diff": float(mean), "rank_spread": float(spread),
                          "multimem": _train.multimem}))


def _optimizer_only(steps: int, dev, rank: int, world: int):
    """`steps` fused optimizer steps on gradients filled from a seeded generator (no forward / backward, whose small reductions
    use floating-point atomics and are outside this check)."""
    from cppmega_mlx_b200.models.hybrid_lm import HybridTinyConfig, HybridTinyLM
    from cppmega_mlx_b200.training.distributed_optimizer import DistributedZeRO1Optimizer
    from cppmega_mlx_b200.training.optimizers import make_muon
    torch.manual_seed(0)
    cfg = HybridTinyConfig(vocab_size=512, hidden_size=256, pattern="MA", depth=2, num_attention_heads=4, max_seq_length=256,
                           mamba_head_dim=64, mamba_state_dim=64, mamba_chunk_size=64, mamba_groups=2, mla_low_rank=True,
                           mla_q_lora_rank=128, mla_kv_lora_rank=128, mla_qk_nope_head_dim=64, mla_qk_rope_head_dim=32,
                           mla_v_head_dim=64, ffn_hidden_size=512, position_embedding=False)
    model = HybridTinyLM(cfg).to(dev, torch.bfloat16)
    opt = DistributedZeRO1Optimizer(model, lambda ps: make_muon(ps, lr_muon=2e-2, lr_adamw=1e-3, ns_carrier="bf16"), comm="fused")
    opt.zero_grad()
    gen = torch.Generator(device=dev).manual_seed(1000 + rank)
    for _ in range(steps):
        for p in model.parameters():
            p.grad.copy_(torch.randn(p.shape, generator=gen, device=dev) * 0.01)
        opt.step()
        opt.zero_grad()
    return torch.cat([p.detach().float().reshape(-1) for p in model.parameters()])


def case_zero1det(rank, world, dev):
    """Determinism of the fused ZeRO-1 step: from the same parameters and the same per-rank gradients, two runs of three steps
    end with bit-identical parameters on every rank (each owner sums the peers' gradients in a fixed rank order, the squared norms
    are added per block in a fixed order, and nothing in the step uses atomics)."""
    from cppmega_mlx_b200.ops import _backend as B
    p_a = _optimizer_only(3, dev, rank, world)
    p_b = _optimizer_only(3, dev, rank, world)
    torch.cuda.synchronize()
    B.check_status()
    same = torch.tensor([int(torch.equal(p_a, p_b))], device=dev)
    dist.all_reduce(same, op=dist.ReduceOp.MIN)
    ref = p_a.clone()
    dist.broadcast(ref, 0)
    spread = (ref - p_a).abs().max()
    dist.all_reduce(spread, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(json.dumps({"case": "zero1det", "world": world, "bitwise_equal": bool(int(same)), "rank_spread": float(spread),
                          "finite": bool(torch.isfinite(p_a).all())}))


def case_zero1bw(rank, world, dev):
    """Rate of the three ZeRO-1 range kernels on one large owned range per rank, no flag wait (bucket −1): the fused
    reduce + AdamW + push kernel, the Muon reduce + momentum kernel (link reads only) and the Muon push kernel (link writes only).
    Each is compared with the slower of its link time (bytes crossing NVLink per direction ÷ 770 GB/s measured peer copy) and its
    local HBM time (bytes this GPU's memory serves, the peers' reads and writes included, ÷ the measured copy rate)."""
    import ctypes
    from cppmega_mlx_b200.ops import _backend as B
    from cppmega_mlx_b200.parallel.fused_zero1 import _table
    from cppmega_mlx_b200.parallel.symm import EpochBarrier, SymmetricBuffer
    n = int(os.environ.get("CMB_ZERO1BW_ELEMS", str(128 * 1024 * 1024)))          # owned elements per rank
    lib = B.load_library()
    grads, params = SymmetricBuffer(world * n, torch.bfloat16, dev), SymmetricBuffer(world * n, torch.bfloat16, dev)
    grads.tensor.normal_(0, 0.01)
    params.tensor.normal_(0, 0.02)
    m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    u = torch.zeros(n, dtype=torch.bfloat16, device=dev)
    parts = torch.zeros(148 * 4, device=dev)
    bar = EpochBarrier(dev)
    tab_a = _table([dict(off=rank * n, n=n, s0=m.data_ptr(), s1=v.data_ptr())], dev)
    tab_m = _table([dict(off=rank * n, n=n, s0=m.data_ptr(), u=u.data_ptr(), sumsq=parts.data_ptr())], dev)
    tab_p = _table([dict(off=rank * n, n=n, u=u.data_ptr(), coef=1.0)], dev)
    st = B.ptr(B.status_buffer(dev))
    I64, F32 = ctypes.c_longlong, ctypes.c_float
    f = (ctypes.c_float * 8)(1e-3, 0.9, 0.999, 1e-8, 0.01, 1.0, 1.0, 0.0)
    gp, pp = grads.peer_ptrs, params.peer_ptrs
    # CPPMEGA_ZERO1_MULTIMEM=1: the multimem forms (in-switch reduction, multicast store), if the buffers have a multicast binding
    mc = int(os.environ.get("CPPMEGA_ZERO1_MULTIMEM", "0") == "1" and grads.multicast_ptr != 0 and params.multicast_ptr != 0)

    def adamw():
        B.check(lib.cmb_zero1_adamw_ranges(gp, pp, gp, rank, world, B.ptr(tab_a), 1, I64(n), f, -1, 0, I64(0), st, 0, mc, B.stream_ptr()), "zero1_adamw_ranges")

    def muon():
        B.check(lib.cmb_zero1_muon_reduce_ranges(gp, pp, gp, rank, world, B.ptr(tab_m), 1, I64(n), F32(0.95), F32(0.0), 1, -1, 0, I64(0), st, 0, mc,
                                                 B.stream_ptr()), "zero1_muon_reduce_ranges")

    def push():
        B.check(lib.cmb_zero1_push_ranges(pp, rank, world, B.ptr(tab_p), 1, I64(n), F32(1e-3), mc, B.stream_ptr()), "zero1_push_ranges")

    def timed(fn):
        def step():
            bar()                 # ranks start together; the barrier kernel is inside the timed region on every rank alike
            fn()
        return _time(step, iters=8)
    t_bar = _time(bar, iters=8)
    hbm = float(os.environ.get("CMB_HBM_GBS", "6551")) * 1e9
    link = 770e9
    W = world
    rows = {}
    # bytes per element: (over the link per direction, served by this GPU's HBM)
    for name, fn, link_b, hbm_b in (("adamw_ranges", adamw, 2 * (W - 1), 2 + 2 + 16 + 2 + 4 * (W - 1)),
                                    ("muon_reduce_ranges", muon, 2 * (W - 1), 2 + 2 + 8 + 2 + 2 * (W - 1)),
                                    ("push_ranges", push, 2 * (W - 1), 2 + 2 + 2 + 2 * (W - 1))):
        t = timed(fn) - t_bar
        bound = max(n * link_b / link, n * hbm_b / hbm) * 1e3
        rows[name] = {"ms": t, "link_GBs_per_direction": n * link_b / t / 1e6, "hbm_GBs": n * hbm_b / t / 1e6, "roofline_ms": bound,
                      "achieved_over_roofline": bound / t, "bound": "link" if n * link_b / link > n * hbm_b / hbm else "hbm"}
    torch.cuda.synchronize()
    B.check_status()
    if rank == 0:
        print(json.dumps({"case": "zero1bw", "world": world, "owned_elems_per_rank": n, "multimem": bool(mc),
                          "multicast_binding": grads.multicast_ptr != 0, "barrier_ms": t_bar, **rows}))


def case_allreduce(rank, world, dev):
    """The stand-alone symmetric-memory all-reduce (peer form and, where the buffer has a multicast binding, multimem form)
    against NCCL: fp32 and bf16, a length that is not a multiple of the vector width, and its latency on a small message."""
    from cppmega_mlx_b200.ops import _backend as B
    from cppmega_mlx_b200.parallel.symm import SymmetricAllReduce
    out = {"case": "allreduce", "world": world}
    for dtype, name in ((torch.float32, "fp32"), (torch.bfloat16, "bf16")):
        for mm in (False, True):
            red = SymmetricAllReduce(1 << 20, dtype, dev, multimem=mm)
            if mm and not red.use_mc:
                out[f"{name}_multimem"] = "no multicast binding"
                continue
            worst = 0.0
            for n in (1 << 20, 99_991, 7):
                g = torch.Generator(device=dev).manual_seed(1000 * rank + n)
                x = torch.randn(n, generator=g, device=dev).to(dtype)
                ref = x.clone()
                dist.all_reduce(ref)
                got = red(x.clone())
                tol = 1e-5 if dtype == torch.float32 else 2e-2
                worst = max(worst, float((got.float() - ref.float()).abs().max() / (ref.float().abs().max() + 1e-6)))
                assert worst < tol, (name, mm, n, worst)
            small = torch.ones(8192, device=dev, dtype=dtype)
            t_ours = _time(lambda: red(small), iters=20)
            t_nccl = _time(lambda: dist.all_reduce(small), iters=20)
            out[f"{name}_{'multimem' if mm else 'peer'}"] = {"max_rel_err": worst, "ms_8192_elems": t_ours, "ms_nccl": t_nccl}
    torch.cuda.synchronize()
    B.check_status()
    if rank == 0:
        print(json.dumps(out))


def _time(fn, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def case_tp(rank, world, dev):
    """Sequence-parallel TP FFN (column-parallel up, SwiGLU, row-parallel down): fused symmetric-memory pairs vs the NCCL pairs."""
    from cppmega_mlx_b200 import ops
    from cppmega_mlx_b200.ops import _backend as B
    from cppmega_mlx_b200.parallel import tp as TP
    from cppmega_mlx_b200.parallel.fused_tp import FusedTPComm, column_parallel_fused, row_parallel_fused
    S, d, hid = (16384, 2048, 5632) if os.environ.get("CMB_TP_SMALL") != "1" else (1024, 256, 512)
    torch.manual_seed(0)
    x_full = (torch.randn(S, d, device=dev) * 0.5).bfloat16()
    w_up = (torch.randn(2 * hid, d, device=dev) * 0.02).bfloat16()
    w_dn = (torch.randn(d, hid, device=dev) * 0.02).bfloat16()
    g = dist.group.WORLD
    rows = S // world
    x_shard = x_full[rank * rows:(rank + 1) * rows].clone()
    wu = TP.shard_rows(w_up, g, blocks=2).clone()
    wd = TP.shard_cols(w_dn, g).clone()
    comm = FusedTPComm(g, dev, max_rows_per_rank=rows, max_cols=max(d, 2 * hid // world))

    def run(fused: bool):
        xs = x_shard.clone().requires_grad_()
        a, b = wu.clone().requires_grad_(), wd.clone().requires_grad_()
        if fused:
            h = ops.swiglu(column_parallel_fused(xs, a, comm))
            y = row_parallel_fused(h, b, comm)
        else:
            h = ops.swiglu(ops.linear(TP.gather_sequence(xs, g, 0), a))
            y = TP.reduce_scatter_sequence(ops.linear(h, b), g, 0)
        y.backward(torch.ones_like(y) * 0.01)
        return y.detach(), xs.grad, a.grad, b.grad
    ref, out = run(False), run(True)
    torch.cuda.synchronize()
    B.check_status()
    errs = []
    for r_, o_ in zip(ref, out):
        e = (r_.float() - o_.float()).abs().max() / r_.float().abs().max().clamp_min(1e-6)
        dist.all_reduce(e, op=dist.ReduceOp.MAX)
        errs.append(float(e))
    full_ref = ops.swiglu_reference((x_full.float() @ w_up.float().t())) @ w_dn.float().t()
    e_abs = (out[0].float() - full_ref[rank * rows:(rank + 1) * rows]).abs().max() / full_ref.abs().max()
    dist.all_reduce(e_abs, op=dist.ReduceOp.MAX)
    t_nccl, t_fused = _time(lambda: run(False)), _time(lambda: run(True))
    if rank == 0:
        print(json.dumps({"case": "tp", "world": world, "shape": [S, d, hid], "rel_err_vs_nccl[y,dx,dw_up,dw_down]": errs,
                          "rel_err_vs_fp32_single_gpu": float(e_abs), "ms_fwd_bwd_nccl": t_nccl, "ms_fwd_bwd_fused": t_fused}))


def case_tpar(rank, world, dev):
    """Tensor-parallel SwiGLU FFN with replicated activations, forward and backward: the fused GEMM → reduce-scatter + gather
    all-reduce of ``fused_tp.py`` against the NCCL all-reduce of ``tp.py`` (results and device time)."""
    from cppmega_mlx_b200.nn.basic import FeedForward
    from cppmega_mlx_b200.ops import _backend as B
    from cppmega_mlx_b200.parallel import tp as TP
    from cppmega_mlx_b200.parallel.fused_tp import FusedTPComm
    S, d, hid = (16384, 2048, 5632) if os.environ.get("CMB_TP_SMALL") != "1" else (1024, 256, 512)
    torch.manual_seed(0)
    ffn = FeedForward(d, hid, "swiglu").to(dev, torch.bfloat16)
    x = (torch.randn(S, d, device=dev) * 0.5).bfloat16()
    g = dist.group.WORLD
    comm = FusedTPComm(g, dev, max_rows_per_rank=S // world, max_cols=d)
    mods = {False: TP.TPFeedForward(ffn, g), True: TP.TPFeedForward(ffn, g, fused=comm)}

    def run(fused: bool):
        m = mods[fused]
        m.zero_grad()
        xs = x.clone().requires_grad_()
        y = m(xs)
        y.backward(torch.ones_like(y) * 0.01)
        return y.detach(), xs.grad, m.up.weight.grad.clone(), m.down.weight.grad.clone()
    ref, out = run(False), run(True)
    torch.cuda.synchronize()
    B.check_status()
    errs = []
    for r_, o_ in zip(ref, out):
        e = (r_.float() - o_.float()).abs().max() / r_.float().abs().max().clamp_min(1e-6)
        dist.all_reduce(e, op=dist.ReduceOp.MAX)
        errs.append(float(e))
    t_nccl, t_fused = _time(lambda: run(False)), _time(lambda: run(True))
    if rank == 0:
        print(json.dumps({"case": "tpar", "world": world, "shape": [S, d, hid], "rel_err_vs_nccl[y,dx,dw_up,dw_down]": errs,
                          "ms_fwd_bwd_nccl": t_nccl, "ms_fwd_bwd_fused": t_fused}))


def case_ep(rank, world, dev):
    """Expert-parallel MoE layer, forward and backward: fused dispatch/combine kernels vs the NCCL all-to-all path."""
    from cppmega_mlx_b200.nn.moe import MoE, MoEConfig
    from cppmega_mlx_b200.ops import _backend as B
    from cppmega_mlx_b200.parallel import ep as EP
    from cppmega_mlx_b200.parallel.fused_ep import FusedEPComm, fused_ep_moe_forward
    small = os.environ.get("CMB_EP_SMALL") == "1"
    T, d, E, k, hid = (512, 256, 8, 2, 128) if small else (16384, 2048, 64, 6, 1408)
    cfg = MoEConfig(d_model=d, num_experts=E, top_k=k, expert_hidden_size=hid, shared_expert_hidden_size=None, activation="swiglu",
                    scoring="sigmoid", aux_loss_free=True)
    torch.manual_seed(0)
    full = MoE(cfg).to(dev, torch.bfloat16)
    g = dist.group.WORLD
    local = MoE(cfg, ep_group=g).to(dev, torch.bfloat16)
    EP.shard_experts_(full, local)
    torch.manual_seed(100 + rank)
    x = (torch.randn(T, d, device=dev) * 0.5).bfloat16()
    comm = FusedEPComm(g, dev, max_tokens=T, top_k=k, d_model=d, num_experts=E, capacity_rows=None if small else 2 * T * k)

    def run(fused: bool):
        xs = x.clone().requires_grad_()
        local.zero_grad()
        r = local.router(xs[None])
        idx, w = r.top_indices.reshape(-1, k), r.top_weights.reshape(-1, k)
        y = fused_ep_moe_forward(local, comm, xs, idx, w) if fused else EP.ep_moe_forward(local, xs, idx, w)
        y.backward(torch.ones_like(y) * 0.01)
        return y.detach(), xs.grad.clone(), local.experts.w_gate_up.grad.clone(), local.experts.w_down.grad.clone(), local.router.gate.weight.grad.clone()
    ref, out = run(False), run(True)
    torch.cuda.synchronize()
    B.check_status()
    errs = []
    for r_, o_ in zip(ref, out):
        e = (r_.float() - o_.float()).abs().max() / r_.float().abs().max().clamp_min(1e-6)
        dist.all_reduce(e, op=dist.ReduceOp.MAX)
        errs.append(float(e))
    t_nccl, t_fused = _time(lambda: run(False), iters=5), _time(lambda: run(True), iters=5)
    if os.environ.get("CMB_EP_PROFILE") == "1":           # analysis aid: where the fused layer's time goes (rank 0, one forward + backward)
        from torch.profiler import ProfilerActivity, profile
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            run(True)
            torch.cuda.synchronize()
        if rank == 0:
            rows_ = sorted(prof.key_averages(), key=lambda e: -e.device_time_total)[:30]
            for e in rows_:
                print(json.dumps({"kernel": e.key[:110], "ms": e.device_time_total / 1e3, "launches": e.count}))
    if rank == 0:
        print(json.dumps({"case": "ep", "world": world, "shape": {"tokens_per_rank": T, "d": d, "experts": E, "top_k": k, "hidden": hid},
                          "rel_err_vs_nccl[y,dx,dw_gate_up,dw_down,dw_router]": errs, "ms_fwd_bwd_nccl": t_nccl, "ms_fwd_bwd_fused": t_fused}))


def case_epdrop(rank, world, dev):
    """A router that sends every token to expert 0 (plus one random expert) into a receive buffer that is far too small: the
    fused path drops the assignments that do not fit (slot −1, skipped by the kernels, counted), never writes outside a buffer
    (status words stay clean) and agrees with the all-to-all path under the same drop rule."""
    from cppmega_mlx_b200.nn.moe import MoE, MoEConfig
    from cppmega_mlx_b200.ops import _backend as B
    from cppmega_mlx_b200.parallel import ep as EP
    from cppmega_mlx_b200.parallel.fused_ep import FusedEPComm, fused_ep_moe_forward
    T, d, E, k, hid = 512, 256, 8, 2, 128
    cfg = MoEConfig(d_model=d, num_experts=E, top_k=k, expert_hidden_size=hid, shared_expert_hidden_size=None, activation="swiglu",
                    scoring="sigmoid", aux_loss_free=True)
    torch.manual_seed(0)
    full = MoE(cfg).to(dev, torch.bfloat16)
    g = dist.group.WORLD
    local = MoE(cfg, ep_group=g).to(dev, torch.bfloat16)
    EP.shard_experts_(full, local)
    torch.manual_seed(100 + rank)
    x = (torch.randn(T, d, device=dev) * 0.5).bfloat16()
    idx = torch.stack([torch.zeros(T, dtype=torch.long, device=dev), 1 + torch.randint(0, E - 1, (T,), device=dev)], 1)
    w = torch.rand(T, k, device=dev)
    comm = FusedEPComm(g, dev, max_tokens=T, top_k=k, d_model=d, num_experts=E, capacity_rows=512)
    outs = []
    for fused in (False, True):
        xs = x.clone().requires_grad_()
        local.zero_grad()
        y = fused_ep_moe_forward(local, comm, xs, idx, w) if fused else EP.ep_moe_forward(local, xs, idx, w, capacity_rows=comm.rows)
        y.backward(torch.ones_like(y) * 0.01)
        outs.append((y.detach(), xs.grad.clone(), local.experts.w_down.grad.clone()))
    torch.cuda.synchronize()
    B.check_status()                                       # no slot outside a buffer was ever presented to a kernel
    dropped = torch.tensor([comm.dropped_assignments()], device=dev)
    dist.all_reduce(dropped)
    errs = []
    for r_, o_ in zip(*outs):
        e = (r_.float() - o_.float()).abs().max() / r_.float().abs().max().clamp_min(1e-6)
        dist.all_reduce(e, op=dist.ReduceOp.MAX)
        errs.append(float(e))
    if rank == 0:
        print(json.dumps({"case": "epdrop", "world": world, "capacity_rows": comm.rows, "dropped_total": int(dropped),
                          "rel_err_vs_nccl[y,dx,dw_down]": errs}))


def _mixer_stack(dev, pattern: str, max_seq: int):
    from cppmega_mlx_b200.models.hybrid_lm import HybridTinyConfig, HybridTinyLM
    torch.manual_seed(0)
    cfg = HybridTinyConfig(vocab_size=512, hidden_size=256, pattern=pattern, depth=len(pattern), num_attention_heads=4, max_seq_length=max_seq,
                           mamba_head_dim=64, mamba_state_dim=64, mamba_chunk_size=64, mamba_groups=2, mla_low_rank=True,
                           mla_q_lora_rank=128, mla_kv_lora_rank=128, mla_qk_nope_head_dim=64, mla_qk_rope_head_dim=32,
                           mla_v_head_dim=64, m2rnn_k_head_dim=64, m2rnn_v_head_dim=16, m2rnn_num_v_heads=4, m2rnn_num_f_heads=4,
                           m2rnn_num_g_heads=4, ffn_hidden_size=512, position_embedding=False)
    model = HybridTinyLM(cfg)
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() == 2 and float(p.abs().sum()) == 0:
                p.normal_(std=0.02)                      # zero-initialised output projections would hide the mixers
    return model.to(dev, torch.bfloat16)


def _rel(a, b) -> float:
    a, b = a.detach().float(), b.detach().float()
    return float((a - b).norm() / (b.norm() + 1e-12))


def case_cp(rank, world, dev):
    """Context parallelism over all ranks (Mamba3 scanning on all ranks at once, M2RNN handing its state on, latent keys gathered)
    against the same model run over the whole sequence on one GPU: logits, loss and group-averaged parameter gradients."""
    from cppmega_mlx_b200.parallel import cp as CP
    n = 256
    S = n * world
    model = _mixer_stack(dev, "MAR", S)
    gen = torch.Generator().manual_seed(7)
    ids = torch.randint(0, 512, (2, S + 1), generator=gen).to(dev)
    inp, tgt = ids[:, :-1], ids[:, 1:]
    ce = torch.nn.functional.cross_entropy
    ref = model(inp)
    ref_loss = ce(ref.float().reshape(-1, 512), tgt.reshape(-1))
    ref_loss.backward()
    ref_g = {k: p.grad.float().clone() for k, p in model.named_parameters() if p.grad is not None}
    model.zero_grad()
    group = dist.group.WORLD
    CP.enable_context_parallel(model, group)
    mine = CP.shard_sequence(inp, group)
    out = model(mine)
    loss = ce(out.float().reshape(-1, 512), CP.shard_sequence(tgt, group).reshape(-1))
    loss.backward()
    CP.allreduce_context_parallel_grads(model, group)
    if dev.type == "cuda":
        torch.cuda.synchronize()
    rel_logits = torch.tensor([_rel(out, ref.detach()[:, rank * n:(rank + 1) * n])], device=dev)
    dist.all_reduce(rel_logits, op=dist.ReduceOp.MAX)
    total = loss.detach().clone()
    dist.all_reduce(total)
    worst, name = 0.0, None
    for k, want in ref_g.items():
        g = dict(model.named_parameters())[k].grad
        if g is None or float(want.norm()) < 1e-6:
            continue
        e = _rel(g, want)
        if e > worst:
            worst, name = e, k
    if rank == 0:
        print(json.dumps({"case": "cp", "world": world, "tokens_per_rank": n, "rel_err_logits": float(rel_logits),
                          "loss_whole": float(ref_loss), "loss_mean_over_ranks": float(total) / world,
                          "max_rel_err_grad": worst, "worst_parameter": name}))


def case_tpdecode(rank, world, dev):
    """Cached decode on the head-parallel stack (every rank keeps its share of each cache): prefill and one-token steps against the
    unsharded model's own session."""
    from cppmega_mlx_b200.inference import DecodeSession
    from cppmega_mlx_b200.parallel import tp as TP
    from cppmega_mlx_b200.parallel.state import init_parallel_state
    st = init_parallel_state(tp=world)
    full = _mixer_stack(dev, "MAR", 256).eval()
    shard = _mixer_stack(dev, "MAR", 256).eval()
    shard.load_state_dict(full.state_dict())
    done = TP.tensor_parallelize_mixers(shard, st.tp_group)
    TP.tensor_parallelize_ffn(shard, st.tp_group)
    gen = torch.Generator().manual_seed(11)
    ids = torch.randint(0, 512, (2, 72), generator=gen).to(dev)
    pieces = [slice(0, 64)] + [slice(t, t + 1) for t in range(64, 72)]
    with torch.no_grad():
        s0, s1 = DecodeSession(full), DecodeSession(shard)
        want = torch.cat([s0.forward(ids[:, p]) for p in pieces], 1)
        got = torch.cat([s1.forward(ids[:, p]) for p in pieces], 1)
    if dev.type == "cuda":
        torch.cuda.synchronize()
    err = torch.tensor([_rel(got[:, :64], want[:, :64]), _rel(got[:, 64:], want[:, 64:])], device=dev)
    dist.all_reduce(err, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(json.dumps({"case": "tpdecode", "world": world, "sharded_mixers": done, "rel_err_prefill": float(err[0]),
                          "rel_err_decode_steps": float(err[1]), "finite": bool(torch.isfinite(got).all())}))


def main():
    case = sys.argv[1] if len(sys.argv) > 1 else "zero1"
    rank, world, dev = _setup()
    cases = {"zero1": case_zero1, "zero1det": case_zero1det, "zero1bw": case_zero1bw, "allreduce": case_allreduce, "tp": case_tp, "tpar": case_tpar,
             "ep": case_ep, "epdrop": case_epdrop, "cp": case_cp, "tpdecode": case_tpdecode}
    try:
        cases[case](rank, world, dev)
    except BaseException:
        # the other ranks may be inside a collective that this rank will never join: report and leave without entering another
        # one (a barrier here would wait for them forever and hide the traceback); the launcher ends the remaining ranks
        import traceback
        traceback.print_exc()
        sys.stderr.flush()
        sys.stdout.flush()
        os._exit(1)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
