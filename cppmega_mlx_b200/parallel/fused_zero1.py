"""Fused ZeRO-1 step over symmetric memory, overlapped with the backward pass bucket by bucket.

The flat gradient and parameter buffers live in symmetric memory, so the owner of a tensor can (1) sum that tensor's bf16
gradients straight out of all W ranks' gradient buffers — the reduce-scatter —, (2) cast to fp32 and apply the update to its
local state, and (3) store the new bf16 parameters into all W ranks' parameter buffers — the all-gather — without any
collective call.  AdamW-owned tensors do all three in one kernel; Muon-owned matrices do (1) + momentum in one kernel, run
Newton–Schulz-5 locally as batched tensor-core GEMMs per stack of equal shapes, and do the update + (3) in a second kernel.

**Buckets.**  Parameters are grouped by layer (``layers.<i>.*`` → bucket i, everything else → one last bucket).  When a rank's
backward pass has accumulated every gradient of a bucket (autograd post-accumulate hooks), it raises its flag for that bucket
in every peer's flag block from a side stream; the owner's kernels for the bucket are queued right behind on that stream and
begin with a bounded wait for all W flags of the current step.  The reduction over NVLink, the AdamW updates and their
parameter pushes, and the Muon momentum stage therefore run while the main stream is still in the backward pass of the earlier
layers: once every rank has raised a bucket's flag no rank reads that bucket's weights again before the step ends, so pushing
new parameters early is safe.  After backward only the Newton–Schulz chains, the Muon pushes and whatever bucket was not
complete remain, closed by one epoch barrier ("all parameters delivered, all gradients consumed").  The hooks act only when the
training step has armed them for its last micro-batch (``arm_overlap``); otherwise every bucket is launched from ``step()``,
which is the same code path without the overlap.  ``CPPMEGA_ZERO1_OVERLAP`` = ``1`` / ``0`` / ``auto`` (default): on from four
ranks up.  Measured with the 1.76 B-parameter hybrid on B200s: on two ranks each owner's kernels are bound by local HBM, the whole
exchange costs 2.6 ms per step after backward (331.2 ms against 328.2 ms with no communication at all) and running it beside the
backward GEMMs slows those by as much as it hides (333.4 ms); on eight ranks the kernels are bound by the links ((W−1)/W of all
gradients in and of all parameters out per rank, 9 ms after backward) and the overlap takes the step from 308.6 to 301.5 ms,
2 ms above the run with no communication.

Per step and rank this moves (W−1)/W of the owned segment over NVLink in each direction.
"""
from __future__ import annotations

import ctypes
import os
import re

import torch

from ..ops import _backend as B
from .symm import SPIN_LIMIT, EpochBarrier, SymmetricBuffer

I64 = ctypes.c_longlong
F32 = ctypes.c_float
MAX_RANKS = 16
_RANGE = [("off", "<i8"), ("n", "<i8"), ("s0", "<u8"), ("s1", "<u8"), ("u", "<u8"), ("sumsq", "<u8"), ("coef", "<f4"), ("pad", "<i4")]
_LAYER = re.compile(r"(?:^|\.)layers\.(\d+)\.")
Z1_PARTS = 148 * 4         # per-block partial sums of u² per Muon tensor (the range kernels' grid cap)


def _reducer_blocks() -> int:
    """Grid cap of a bucket kernel launched during backward (0 = the full grid).  A small cap leaves the SMs to the backward GEMMs
    but lets the side stream fall behind: on two B200s 16 blocks cost 29 ms per step and 64 blocks 8 ms against the full grid."""
    return int(os.environ.get("CPPMEGA_ZERO1_REDUCER_BLOCKS", "0"))


def _table(rows: list[dict], device) -> torch.Tensor | None:
    import numpy as np
    if not rows:
        return None
    arr = np.zeros(len(rows), dtype=_RANGE)
    assert arr.dtype.itemsize == 56
    for i, r in enumerate(rows):
        for k, v in r.items():
            arr[i][k] = v
    return torch.from_numpy(arr.view(np.uint8).copy()).to(device)


class _Bucket:
    def __init__(self, idx: int):
        self.idx = idx
        self.params: list[str] = []          # every parameter of the bucket (owned or not): the hooks count these
        self.adamw: list[dict] = []          # owned AdamW ranges
        self.muon: list[dict] = []           # owned Muon ranges (fast path)
        self.adamw_tab = self.muon_tab = None
        self.adamw_elems = self.muon_elems = 0
        self.pending = 0
        self.launched = False


class FusedZeRO1Comm:
    def __init__(self, group=None):
        self.group = group
        self.flat = None
        self.bufs: list[SymmetricBuffer] = []
        self.barrier: EpochBarrier | None = None
        self.enabled = True
        self.overlap = None                  # decided in bind(): needs the group size
        self.armed = False
        self.epoch = 0
        self.buckets: list[_Bucket] | None = None
        self.comm_stream = None

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
        mode = os.environ.get("CPPMEGA_ZERO1_OVERLAP", "auto")
        self.overlap = mode == "1" or (mode == "auto" and self.params_buf.world >= 4)
        # CPPMEGA_ZERO1_MULTIMEM=1: reduce the gradients in the switch (multimem.ld_reduce) and push the parameters with one
        # multicast store (multimem.st) instead of W peer loads / stores; needs buffers with a multicast binding.  Off by default:
        # a rank that dies while bound to a multicast object can fault its peers' links, so failure tests keep to plain peer accesses.
        self.use_mc = int(os.environ.get("CPPMEGA_ZERO1_MULTIMEM", "0") == "1" and self.params_buf.multicast_ptr != 0
                          and self.grads_buf.multicast_ptr != 0)

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

    @staticmethod
    def _split(opt):
        from ..training.optimizers import AdamWFP32Moments
        inner = opt.inner
        adamw = inner if isinstance(inner, AdamWFP32Moments) else inner.other
        muon = None if isinstance(inner, AdamWFP32Moments) else inner.muon
        return adamw, muon

    def setup(self, opt) -> None:
        """Static plan, built once: buckets, the owner's range tables (device), stack workspaces of the owned Muon matrices, the flag
        blocks and the autograd hooks.  A collective over the group (symmetric allocation + barrier): every rank calls it."""
        if self.buckets is not None or not self._supported(opt):
            return
        import torch.distributed as dist
        from ..ops.optim import MuonBatchPlan, TensorTable
        flat, dev = self.flat, self.flat.params.device
        adamw, muon = self._split(opt)
        nlayers = 1 + max((int(m.group(1)) for n, _ in opt.named if (m := _LAYER.search(n))), default=-1)
        buckets = [_Bucket(i) for i in range(nlayers + 1)]               # the last bucket takes everything outside the layers
        bucket_of = {}
        for n, p in opt.named:
            m = _LAYER.search(n)
            b = buckets[int(m.group(1)) if m else nlayers]
            b.params.append(n)
            bucket_of[n] = b
        self.slow_muon, fast = [], []
        if muon is not None:
            for n, p in muon.params:
                if flat.slots[n][2] % 8:
                    raise RuntimeError(f"fused Muon needs an element count that is a multiple of 8, got {tuple(p.shape)} for {n}")
                (fast if p.shape[0] % 8 == 0 and p.shape[1] % 8 == 0 else self.slow_muon).append((n, p))
        self.plan = MuonBatchPlan(dev)
        self.fast = fast
        self.n_muon = len(fast) + len(self.slow_muon)
        self.sumsq = torch.zeros(max(1, self.n_muon), dtype=torch.float32, device=dev)
        self.parts = torch.zeros(max(1, self.n_muon) * Z1_PARTS, dtype=torch.float32, device=dev)   # written by block index, summed in fixed order
        self.stacks = []
        u_of, self.res_of = {}, {}
        steps = muon.ns_steps if muon is not None else 0
        for sh, idx in self.plan.stacks([tuple(p.shape) for _, p in fast]):
            x, nxt, gws, poly = self.plan.workspace((sh, idx[0]), sh, len(idx))
            res = nxt if steps % 2 else x
            self.stacks.append((x, nxt, gws, poly, idx))
            for j, i in enumerate(idx):
                u_of[i], self.res_of[i] = x[j], res[j]
        self.slow_u = [torch.zeros(p.shape, dtype=torch.bfloat16, device=dev) for _, p in self.slow_muon]
        for k_, (n, p) in enumerate(self.slow_muon):     # reduced with the bucket like the others; orthogonalised by PyTorch ops in step()
            owner, off, cnt = flat.slots[n]
            bucket_of[n].muon.append(dict(off=owner * flat.segment + off, n=cnt, s0=muon.state_for(n, p)["v"].data_ptr(),
                                          u=self.slow_u[k_].data_ptr(), sumsq=self.parts.data_ptr() + 4 * Z1_PARTS * (len(fast) + k_)))
        norm_rows = []
        for i, (n, p) in enumerate(fast):
            owner, off, cnt = flat.slots[n]
            st = muon.state_for(n, p)
            bucket_of[n].muon.append(dict(off=owner * flat.segment + off, n=cnt, s0=st["v"].data_ptr(), u=u_of[i].data_ptr(),
                                          sumsq=self.parts.data_ptr() + 4 * Z1_PARTS * i))
            norm_rows.append(dict(u=u_of[i].data_ptr(), sumsq=self.sumsq.data_ptr() + 4 * i, numel=cnt))
        self.norm_tab = TensorTable(dev).update(norm_rows) if norm_rows else None
        for n, p in adamw.params:
            owner, off, cnt = flat.slots[n]
            st = adamw.state_for(n, p)
            bucket_of[n].adamw.append(dict(off=owner * flat.segment + off, n=cnt, s0=st["m"].data_ptr(), s1=st["v"].data_ptr()))
        for b in buckets:
            b.adamw_elems, b.muon_elems = sum(r["n"] for r in b.adamw), sum(r["n"] for r in b.muon)
            b.adamw_tab, b.muon_tab = _table(b.adamw, dev), _table(b.muon, dev)
        # flag blocks: int32 [nbuckets][MAX_RANKS] per rank, written by peers, polled by the owner's kernels
        self.flags = SymmetricBuffer(len(buckets) * MAX_RANKS, torch.int32, dev, self.group)
        torch.cuda.synchronize(dev)
        dist.barrier(group=self.flags.group)                               # every rank's flags are zero before anyone signals
        # Two side streams: flags are raised from one that never waits on a peer, the owner's kernels (which do) run on the other.
        # A rank whose buckets complete in a different order therefore cannot hold back its own flags behind a waiting kernel.
        self.sig_stream = torch.cuda.Stream(dev, priority=-1)
        self.comm_stream = torch.cuda.Stream(dev, priority=-1)
        self.opt = opt
        self.push_tabs: dict = {}
        params = dict(opt.named)
        for b in buckets:
            for n in b.params:
                params[n].register_post_accumulate_grad_hook(self._make_hook(b))
        self.buckets = buckets
        self._reset_pending()

    def _reset_pending(self) -> None:
        for b in self.buckets:
            b.pending, b.launched = len(b.params), False

    def _make_hook(self, bucket: _Bucket):
        def hook(_param):
            if not self.armed:
                return
            bucket.pending -= 1
            if bucket.pending == 0 and not bucket.launched:
                self._launch_bucket(bucket, during_backward=True)
        return hook

    # ------------------------------------------------------------------------------------------
    def arm_overlap(self) -> None:
        """Called by the training step right before the backward pass of the step's last micro-batch: from here on a bucket's
        reduction starts as soon as its gradients are complete.  Without this call everything runs from ``step()``."""
        if self.overlap and self.buckets is not None and not self.armed:
            self._prepare_step_scalars(self._split(self.opt)[0])
            self.armed = True

    def _prepare_step_scalars(self, adamw) -> None:
        b1, b2 = adamw.betas
        if adamw.bias_correction:
            t = adamw.step_count + 1
            self._c1, self._c2 = 1.0 / (1 - b1 ** t), (1 - b2 ** t) ** -0.5      # c2 scales sqrt(v) (kernel convention)
        else:
            self._c1 = self._c2 = 1.0

    def _launch_bucket(self, b: _Bucket, during_backward: bool) -> None:
        """Raise this rank's flag for the bucket and queue the owner's kernels behind it (side stream; they wait for all W flags)."""
        lib = B.load_library()
        opt = self.opt
        adamw, muon = self._split(opt)
        flat, W, rank = self.flat, opt.world, opt.rank
        gp, pp, fp = self.grads_buf.peer_ptrs, self.params_buf.peer_ptrs, self.flags.peer_ptrs
        epoch = self.epoch + 1
        dev = flat.params.device
        main = torch.cuda.current_stream(dev)
        self.sig_stream.wait_event(main.record_event())                    # the bucket's gradients are final on the main stream
        status = B.ptr(B.status_buffer(dev))
        cap = _reducer_blocks() if during_backward else 0
        with torch.cuda.stream(self.sig_stream):
            B.check(lib.cmb_zero1_bucket_signal(fp, rank, W, b.idx, epoch, B.stream_ptr()), "zero1_bucket_signal")
            raised = self.sig_stream.record_event()
        if not (b.adamw or b.muon):
            b.launched = True
            return
        self.comm_stream.wait_event(raised)
        with torch.cuda.stream(self.comm_stream):
            st = B.stream_ptr()
            if b.adamw:
                f = (ctypes.c_float * 8)(adamw.lr, adamw.betas[0], adamw.betas[1], adamw.eps, adamw.weight_decay, self._c1, self._c2, 0.0)
                B.check(lib.cmb_zero1_adamw_ranges(gp, pp, fp, rank, W, B.ptr(b.adamw_tab), len(b.adamw), I64(b.adamw_elems), f, b.idx, epoch,
                                                   I64(SPIN_LIMIT), status, cap, self.use_mc, st), "zero1_adamw_ranges")
            if b.muon:
                B.check(lib.cmb_zero1_muon_reduce_ranges(gp, pp, fp, rank, W, B.ptr(b.muon_tab), len(b.muon), I64(b.muon_elems), F32(muon.momentum),
                                                         F32(muon.weight_decay), int(muon.nesterov), b.idx, epoch, I64(SPIN_LIMIT), status, cap, self.use_mc, st),
                        "zero1_muon_reduce_ranges")
        b.launched = True

    def try_fused_step(self, opt) -> bool:
        if not self._supported(opt):
            return False
        from ..ops.optim import OP_SCALE_INV_NORM, newton_schulz5_batched_
        from ..training.optimizers import newton_schulz5, ns_streams
        lib = B.load_library()
        adamw, muon = self._split(opt)
        self.setup(opt)
        if not self.armed:
            self._prepare_step_scalars(adamw)
        flat, W, rank = self.flat, opt.world, opt.rank
        dev = flat.params.device
        pp = self.params_buf.peer_ptrs
        for b in self.buckets:                       # whatever the backward pass did not start (all of it when the hooks were not armed)
            if not b.launched:
                self._launch_bucket(b, during_backward=False)
        main = torch.cuda.current_stream(dev)
        main.wait_stream(self.sig_stream)
        main.wait_stream(self.comm_stream)           # every owned range is reduced; AdamW ranges are updated and delivered
        self.epoch += 1
        self.armed = False
        adamw.step_count += 1
        if muon is not None:
            muon.step_count += 1
            B.check(lib.cmb_zero1_sumsq_finalize(B.ptr(self.parts), B.ptr(self.sumsq), self.n_muon, B.stream_ptr()), "zero1_sumsq_finalize")
            if self.norm_tab is not None:
                self.norm_tab.launch(OP_SCALE_INV_NORM, torch.bfloat16, (1e-7,), "scale_inv_norm_multi")
            ready = main.record_event()
            streams = ns_streams(dev)
            for s_ in streams:
                s_.wait_event(ready)
            lr = muon.lr
            for k_, (x, nxt, gws, poly, idx) in enumerate(self.stacks):
                with torch.cuda.stream(streams[k_ % len(streams)]):
                    newton_schulz5_batched_(x, nxt, gws, poly, muon.ns_steps)
                    ent = self.push_tabs.get(k_)
                    if ent is None:              # the owner pushes p − lr·U of the whole stack into every rank's parameter buffer
                        rows = []
                        for i in idx:
                            n, p = self.fast[i]
                            owner, off, cnt = flat.slots[n]
                            rows.append(dict(off=owner * flat.segment + off, n=cnt, u=self.res_of[i].data_ptr(),
                                             coef=max(1.0, p.shape[0] / p.shape[1]) ** 0.5))
                        ent = self.push_tabs[k_] = (_table(rows, dev), len(rows), sum(r["n"] for r in rows))
                    B.check(lib.cmb_zero1_push_ranges(pp, rank, W, B.ptr(ent[0]), ent[1], I64(ent[2]), F32(lr), self.use_mc, B.stream_ptr()), "zero1_push_ranges")
            for s_ in streams:
                main.wait_stream(s_)
            for k_, (n, p) in enumerate(self.slow_muon):   # too narrow for the tensor-core iteration (e.g. a 4-row gate): same maths in PyTorch ops
                owner, off, cnt = flat.slots[n]
                goff = owner * flat.segment + off
                o = newton_schulz5(self.slow_u[k_], steps=muon.ns_steps, ns_carrier="bf16", output_dtype=torch.bfloat16).contiguous()
                B.check(lib.cmb_zero1_push_update(pp, rank, W, I64(goff), I64(cnt), B.ptr(o), F32(lr * max(1.0, p.shape[0] / p.shape[1]) ** 0.5),
                                                  B.stream_ptr()), "zero1_push_update")
        self.barrier()  # all parameters delivered everywhere; all gradients consumed
        self._reset_pending()
        return True
