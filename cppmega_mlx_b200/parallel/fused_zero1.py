"""Fused ZeRO-1 step over symmetric memory.

With the flat gradient and parameter buffers living in symmetric memory, the optimizer step of the owner of
a tensor is a single pass that (1) sums that tensor's bf16 gradients straight out of all W ranks' gradient
buffers — the reduce-scatter —, (2) casts to fp32 and applies the update to its local state, and (3) stores
the new bf16 parameters into all W ranks' parameter buffers — the all-gather.  AdamW-owned tensors do all
three in one kernel; Muon-owned matrices do (1)+momentum in one kernel, run Newton–Schulz-5 locally on the
tensor cores, and do the update+(3) in a second kernel.  Two epoch barriers bracket the step: "all gradients
written" before, "all parameters delivered and all gradients consumed" after.  No NCCL call is on this path.

Per step and rank this moves (W−1)/W of the owned segment over NVLink in each direction.
"""
from __future__ import annotations

import ctypes

import torch

from ..ops import _backend as B
from .symm import EpochBarrier, SymmetricBuffer

I64 = ctypes.c_longlong
F32 = ctypes.c_float


class FusedZeRO1Comm:
    def __init__(self, group=None):
        self.group = group
        self.flat = None
        self.bufs: list[SymmetricBuffer] = []
        self.barrier: EpochBarrier | None = None
        self.enabled = True

    def alloc(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        buf = SymmetricBuffer(numel, dtype, torch.device("cuda", torch.cuda.current_device()), self.group)
        self.bufs.append(buf)
        return buf.tensor

    def bind(self, flat) -> None:
        self.flat = flat
        self.params_buf, self.grads_buf = self.bufs[0], self.bufs[1]
        if flat.dtype != torch.bfloat16 or flat.grad_dtype != torch.bfloat16:
            self.enabled = False
        self.barrier = EpochBarrier(flat.params.device, self.group)

    # ------------------------------------------------------------------------------------------
    def _supported(self, opt) -> bool:
        from ..training.optimizers import AdamWFP32Moments, MuonAdamWMulti, MuonWithNSCarrier
        inner = opt.inner
        if not (self.enabled and B.kernels_enabled()):
            return False
        if isinstance(inner, AdamWFP32Moments):
            return True
        return (isinstance(inner, MuonAdamWMulti) and type(inner.muon) is MuonWithNSCarrier
                and inner.muon.ns_carrier == "bf16" and isinstance(inner.other, AdamWFP32Moments))

    def try_fused_step(self, opt) -> bool:
        if not self._supported(opt):
            return False
        from ..training.optimizers import AdamWFP32Moments, newton_schulz5
        lib = B.load_library()
        flat, W, rank = self.flat, opt.world, opt.rank
        gp, pp = self.grads_buf.peer_ptrs, self.params_buf.peer_ptrs
        st = B.stream_ptr
        inner = opt.inner
        adamw = inner if isinstance(inner, AdamWFP32Moments) else inner.other
        muon = None if isinstance(inner, AdamWFP32Moments) else inner.muon
        self.barrier()  # every rank's backward has written its gradients
        adamw.step_count += 1
        b1, b2 = adamw.betas
        if adamw.bias_correction:
            t = adamw.step_count
            c1, c2 = 1.0 / (1 - b1 ** t), (1 - b2 ** t) ** -0.5      # c2 scales sqrt(v) (kernel convention)
        else:
            c1 = c2 = 1.0
        for name, p in adamw.params:
            owner, off, n = flat.slots[name]
            s = adamw.state_for(name, p)
            B.check(lib.cmb_zero1_adamw(gp, pp, rank, W, I64(owner * flat.segment + off), I64(n), B.ptr(s["m"]), B.ptr(s["v"]),
                                        F32(adamw.lr), F32(b1), F32(b2), F32(adamw.eps), F32(adamw.weight_decay), F32(c1),
                                        F32(c2), st()), "zero1_adamw")
        if muon is not None:
            from ..ops.optim import OP_SCALE_INV_NORM, MuonBatchPlan, newton_schulz5_batched_
            from ..training.optimizers import ns_streams
            muon.step_count += 1
            dev = flat.params.device
            work = [(name, p) for name, p in muon.params]
            for name, p in work:
                if flat.slots[name][2] % 8:
                    raise RuntimeError(f"fused Muon needs an element count that is a multiple of 8, got {tuple(p.shape)} for {name}")
            fast = [(n_, p) for n_, p in work if p.shape[0] % 8 == 0 and p.shape[1] % 8 == 0]
            slow = [(n_, p) for n_, p in work if p.shape[0] % 8 or p.shape[1] % 8]
            plan = getattr(self, "_plan", None)
            if plan is None:
                plan = self._plan = MuonBatchPlan(dev)
            nf = len(fast)
            if plan.sumsq is None or plan.sumsq.numel() != nf + len(slow):
                plan.sumsq = torch.zeros(nf + len(slow), dtype=torch.float32, device=dev)
            else:
                plan.sumsq.zero_()

            def reduce_into(name, p, u, sumsq_slot):
                owner, off, n = flat.slots[name]
                s = muon.state_for(name, p)
                B.check(lib.cmb_zero1_muon_reduce(gp, pp, rank, W, I64(owner * flat.segment + off), I64(n), B.ptr(s["v"]), B.ptr(u), B.ptr(sumsq_slot),
                                                  F32(muon.momentum), F32(muon.weight_decay), int(muon.nesterov), st()), "zero1_muon_reduce")

            def push(name, p, o):
                owner, off, n = flat.slots[name]
                coef = muon.lr * max(1.0, p.shape[0] / p.shape[1]) ** 0.5
                B.check(lib.cmb_zero1_push_update(pp, rank, W, I64(owner * flat.segment + off), I64(n), B.ptr(o), F32(coef), st()), "zero1_push_update")

            # (1) reduce the peers' gradients of every owned matrix into its slot of a same-shape stack (+ momentum, Σu²)
            stacks = plan.stacks([tuple(p.shape) for _, p in fast])
            rows, jobs = [None] * nf, []
            for sh, idx in stacks:
                x, nxt, gws, poly = plan.workspace((sh, idx[0]), sh, len(idx))
                jobs.append((x, nxt, gws, poly, idx))
                for j, i in enumerate(idx):
                    reduce_into(fast[i][0], fast[i][1], x[j], plan.sumsq[i:i + 1])
                    rows[i] = dict(u=x[j].data_ptr(), sumsq=plan.sumsq.data_ptr() + 4 * i, numel=fast[i][1].numel())
            # (2) Frobenius normalisation of all of them in one launch, (3) Newton–Schulz per stack as batched GEMMs on side streams
            plan.tab_in.update(rows)
            plan.tab_in.launch(OP_SCALE_INV_NORM, torch.bfloat16, (1e-7,), "scale_inv_norm_multi")
            main = torch.cuda.current_stream(dev)
            ready = main.record_event()
            streams = ns_streams(dev)
            for s_ in streams:
                s_.wait_event(ready)
            results = []
            for k_, (x, nxt, gws, poly, idx) in enumerate(jobs):
                with torch.cuda.stream(streams[k_ % len(streams)]):
                    res = newton_schulz5_batched_(x, nxt, gws, poly, muon.ns_steps)
                    for j, i in enumerate(idx):          # (4) owner pushes p − lr·U into every rank's parameter buffer
                        push(fast[i][0], fast[i][1], res[j])
            for s_ in streams:
                main.wait_stream(s_)
            for k_, (name, p) in enumerate(slow):         # too narrow for the tensor-core iteration (e.g. a 4-row gate): same maths in PyTorch ops
                u = torch.empty(p.shape, dtype=torch.bfloat16, device=dev)
                reduce_into(name, p, u, plan.sumsq[nf + k_:nf + k_ + 1])
                push(name, p, newton_schulz5(u, steps=muon.ns_steps, ns_carrier="bf16", output_dtype=torch.bfloat16).contiguous())
        self.barrier()  # all parameters delivered everywhere; all gradients consumed
        return True
