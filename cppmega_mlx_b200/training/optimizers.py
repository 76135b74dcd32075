"""Optimizers: AdamW / Lion with fp32 moments on bf16 parameters, Muon with Newton–Schulz-5
orthogonalisation (fp32 or bf16 carrier, optional 8-bit momentum), and the Muon+AdamW splitter.

Contracts kept from the reference (``cppmega_mlx/training/optimizers.py``):
  * parameters keep their dtype, moments are fp32, there is no fp32 master copy (``:92-113``);
  * AdamW = decoupled decay ``p·(1−lr·wd)`` then Adam without bias correction by default (``:116``);
  * Lion: ``c = β1 m + (1−β1) g``, ``p ← p(1−lr·wd) − lr·sign(c)``, ``m ← β2 m + (1−β2) g`` (``:135``);
  * Muon group = 2-D weights that are not embeddings / LM head / Mamba scalars (``:182-202``);
  * NS-5 coefficients (3.4445, −4.7750, 2.0315), Frobenius-normalised input (+1e-7), transposed when
    rows > cols (``:263-299``); weight decay folded into the gradient, ``v ← μv + (1−μ)g``, Nesterov
    update ``(1−μ)g + μv``, step ``lr·sqrt(max(1, rows/cols))`` (``:302-376``);
  * quantised momentum = uint8 codes + one fp32 absmax per 256 values (``:379-512``);
  * ``make_muon`` defaults lr_muon 2e-3 / lr_adamw 1e-4, scalar optimizer adamw|adam8bit|lion|lion8bit,
    ``cppmega_cuda_parity`` shares one lr (``:610-759``).

State is a flat ``{param_name: {slot: tensor}}`` dict so that ZeRO-1 can shard it by name and the
checkpoint writer can store it under world-size-independent names.  On CUDA the element-wise
updates run as fused multi-tensor kernels (``csrc/optim.cu``) and NS-5 runs on the tcgen05 GEMM.
"""
from __future__ import annotations

import math
import os
from typing import Callable, Iterable

import torch

from .. import ops
from ..ops import _backend as B
from ._quantize_8bit import BLOCK_SIZE, dequantize_blockwise, quantize_blockwise

MUON_NS_CARRIER_ENV = "CPPMEGA_MUON_NS_CARRIER"
MUON_NS_CARRIERS = ("fp32", "bf16")
MUON_QUANTIZED_MOMENTUM_SCHEME = "symmetric_int8_v1"
EMBEDDING_LIKE_NAME_HINTS = ("embed", "embedding", "lm_head", "wte", "wpe")
MAMBA_SCALAR_LEAVES = frozenset({"A_log", "dt_bias", "D", "B_bias", "C_bias", "B_norm_weight", "C_norm_weight",
                                 "mimo_x", "mimo_z", "mimo_o"})
NS_COEFFS = (3.4445, -4.7750, 2.0315)

NamedParams = list[tuple[str, torch.nn.Parameter]]


def named_trainable(model_or_params) -> NamedParams:
    if isinstance(model_or_params, torch.nn.Module):
        seen, out = set(), []
        for n, p in model_or_params.named_parameters():
            if p.requires_grad and id(p) not in seen:
                seen.add(id(p))
                out.append((n, p))
        return out
    return list(model_or_params)


def _lr_value(lr) -> float:
    return float(lr() if callable(lr) else lr)


class Optimizer:
    """Minimal optimizer base: ``step()`` consumes ``p.grad``; ``state`` is keyed by parameter name."""

    def __init__(self, params, learning_rate):
        self.params: NamedParams = named_trainable(params)
        self.learning_rate = learning_rate
        self.state: dict[str, dict[str, torch.Tensor]] = {}
        self.step_count = 0

    @property
    def lr(self) -> float:
        return _lr_value(self.learning_rate)

    def init_single(self, name: str, p: torch.Tensor) -> dict[str, torch.Tensor]:  # pragma: no cover
        raise NotImplementedError

    def apply_single(self, name: str, grad: torch.Tensor, p: torch.Tensor, st: dict) -> None:  # pragma: no cover
        raise NotImplementedError

    def state_for(self, name: str, p: torch.Tensor) -> dict:
        st = self.state.get(name)
        if st is None:
            st = self.state[name] = self.init_single(name, p)
        return st

    @torch.no_grad()
    def step(self, grads: dict[str, torch.Tensor] | None = None) -> None:
        self.step_count += 1
        for name, p in self.params:
            g = grads.get(name) if grads is not None else p.grad
            if g is None:
                continue
            self.apply_single(name, g, p, self.state_for(name, p))

    def zero_grad(self) -> None:
        for _, p in self.params:
            p.grad = None

    def state_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for st in self.state.values() for t in st.values())

    def state_dict(self) -> dict:
        return {"step": self.step_count, "state": {n: {k: v for k, v in st.items()} for n, st in self.state.items()}}

    def load_state_dict(self, sd: dict) -> None:
        self.step_count = int(sd.get("step", 0))
        pm = dict(self.params)
        self.state = {}
        for n, st in sd.get("state", {}).items():
            if n not in pm:
                raise KeyError(f"optimizer state for unknown parameter {n!r}")
            self.state[n] = {k: v.to(pm[n].device) for k, v in st.items()}


class AdamWFP32Moments(Optimizer):
    def __init__(self, params, learning_rate=1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01,
                 bias_correction: bool = False):
        super().__init__(params, learning_rate)
        self.betas, self.eps, self.weight_decay, self.bias_correction = tuple(betas), eps, weight_decay, bias_correction

    def init_single(self, name, p):
        return {"m": torch.zeros_like(p, dtype=torch.float32), "v": torch.zeros_like(p, dtype=torch.float32)}

    def apply_single(self, name, grad, p, st):
        b1, b2 = self.betas
        lr = self.lr
        if self.bias_correction:
            t = self.step_count
            # the update is m·c1 / (sqrt(v)·c2 + eps): c2 multiplies the root, so it is (1 − b2^t)^(−1/2)
            # (same convention as the kernels and as the 8-bit optimizers; cppmega_mlx/training/optimizers_quantized.py:211-218)
            c1, c2 = 1.0 / (1 - b1 ** t), (1 - b2 ** t) ** -0.5
        else:
            c1 = c2 = 1.0
        if p.is_cuda and B.kernels_enabled() and p.is_contiguous() and grad.is_contiguous():
            from ..ops.optim import fused_adamw_
            fused_adamw_(p, grad, st["m"], st["v"], lr, b1, b2, self.eps, self.weight_decay, c1, c2)
            return
        g = grad.float()
        st["m"].mul_(b1).add_(g, alpha=1 - b1)
        st["v"].mul_(b2).addcmul_(g, g, value=1 - b2)
        pf = p.float() * (1 - lr * self.weight_decay)
        denom = st["v"].sqrt().mul_(c2).add_(self.eps)
        pf.addcdiv_(st["m"] * c1, denom, value=-lr)
        p.copy_(pf)


def _adamw_step_multi(self, grads=None) -> None:
    """All tensors of one dtype on one GPU are updated by a single multi-tensor launch; the rest go one by one."""
    work = []
    for name, p in self.params:
        g = grads.get(name) if grads is not None else p.grad
        if g is not None:
            work.append((name, g, p, self.state_for(name, p)))
    if not work:
        self.step_count += 1
        return
    ok = lambda g, p: p.is_cuda and B.kernels_enabled() and p.is_contiguous() and g.is_contiguous() and p.dtype == g.dtype and \
        p.dtype in (torch.bfloat16, torch.float32, torch.float16)
    fast = [w for w in work if ok(w[1], w[2]) and w[2].dtype == work[0][2].dtype and w[2].device == work[0][2].device]
    if len(fast) < 2:
        return Optimizer.step(self, grads)
    self.step_count += 1
    fast_ids = {id(w[2]) for w in fast}
    for name, g, p, st in work:
        if id(p) not in fast_ids:
            self.apply_single(name, g, p, st)
    from ..ops.optim import OP_ADAMW, TensorTable
    dev = fast[0][2].device
    tab = getattr(self, "_table", None)
    if tab is None or tab.device != dev:
        tab = self._table = TensorTable(dev)
    b1, b2 = self.betas
    if self.bias_correction:
        t = self.step_count
        c1, c2 = 1.0 / (1 - b1 ** t), (1 - b2 ** t) ** -0.5
    else:
        c1 = c2 = 1.0
    tab.update([dict(p=p.data_ptr(), g=g.data_ptr(), s0=st["m"].data_ptr(), s1=st["v"].data_ptr(), numel=p.numel()) for _, g, p, st in fast])
    tab.launch(OP_ADAMW, fast[0][2].dtype, (self.lr, b1, b2, self.eps, self.weight_decay, c1, c2), "adamw_multi")


AdamWFP32Moments.step = torch.no_grad()(_adamw_step_multi)


def make_adamw(params, *, learning_rate=1e-3, weight_decay: float = 0.01, betas=None, eps: float = 1e-8,
               bias_correction: bool = False) -> AdamWFP32Moments:
    return AdamWFP32Moments(params, learning_rate, (0.9, 0.999) if betas is None else betas, eps, weight_decay,
                            bias_correction)


class LionFP32Moments(Optimizer):
    def __init__(self, params, learning_rate=1e-4, betas=(0.9, 0.99), weight_decay: float = 0.0):
        super().__init__(params, learning_rate)
        self.betas, self.weight_decay = tuple(betas), weight_decay

    def init_single(self, name, p):
        return {"m": torch.zeros_like(p, dtype=torch.float32)}

    def apply_single(self, name, grad, p, st):
        b1, b2 = self.betas
        lr = self.lr
        g = grad.float()
        c = st["m"] * b1 + g * (1 - b1)
        pf = p.float() * (1 - lr * self.weight_decay) - lr * torch.sign(c)
        st["m"].mul_(b2).add_(g, alpha=1 - b2)
        p.copy_(pf)


def make_lion(params, *, learning_rate=1e-4, weight_decay: float = 0.0, betas=None) -> LionFP32Moments:
    return LionFP32Moments(params, learning_rate, (0.9, 0.99) if betas is None else betas, weight_decay)


def is_muon_compatible(name: str, param: torch.Tensor) -> bool:
    if param.dim() != 2:
        return False
    if name.rsplit(".", 1)[-1] in MAMBA_SCALAR_LEAVES:
        return False
    low = name.lower()
    return not any(h in low for h in EMBEDDING_LIKE_NAME_HINTS)


def split_param_groups(params, *, predicate: Callable[[str, torch.Tensor], bool] = is_muon_compatible):
    muon, other = [], []
    for n, p in named_trainable(params):
        (muon if predicate(n, p) else other).append((n, p))
    return muon, other


def normalize_ns_carrier(ns_carrier: str) -> str:
    v = ns_carrier.strip().lower()
    if v not in MUON_NS_CARRIERS:
        raise ValueError(f"ns_carrier must be one of {', '.join(MUON_NS_CARRIERS)}; got {ns_carrier!r}")
    return v


def newton_schulz5(update: torch.Tensor, *, steps: int = 5, ns_carrier: str = "fp32", output_dtype=None) -> torch.Tensor:
    """Approximate the orthogonal polar factor of a 2-D matrix with the quintic Newton–Schulz iteration."""
    if update.dim() != 2:
        raise ValueError(f"Expected a 2D array for Newton-Schulz iteration, got shape {tuple(update.shape)} instead.")
    a, b, c = NS_COEFFS
    out_dtype = output_dtype or update.dtype
    transpose = update.shape[0] > update.shape[1]
    x = update.float()
    if transpose:
        x = x.t()
    x = x / (torch.linalg.norm(x) + 1e-7)
    carrier = torch.bfloat16 if normalize_ns_carrier(ns_carrier) == "bf16" else torch.float32
    x = x.to(carrier).contiguous()
    use_kernel = x.is_cuda and carrier == torch.bfloat16 and B.kernels_enabled() and x.shape[0] % 8 == 0 and x.shape[1] % 8 == 0
    for _ in range(steps):
        if use_kernel:
            gram = ops.gemm_raw(x, x)                                       # X Xᵀ
            basis = ops.gemm_raw(gram, gram, b_mn=True, out_dtype=torch.float32)  # G·G (G symmetric)
            basis = (b * gram.float() + c * basis).to(carrier)
            x = (a * x.float() + ops.gemm_raw(basis, x, b_mn=True, out_dtype=torch.float32)).to(carrier)
        else:
            gram = x @ x.t()
            basis = b * gram + c * (gram @ gram)
            x = (a * x + basis @ x).to(carrier)
    if transpose:
        x = x.t()
    return x.to(out_dtype)


class MuonWithNSCarrier(Optimizer):
    def __init__(self, params, learning_rate=2e-3, momentum: float = 0.95, weight_decay: float = 0.01,
                 nesterov: bool = True, ns_steps: int = 5, *, ns_carrier: str = "fp32"):
        super().__init__(params, learning_rate)
        self.momentum, self.weight_decay, self.nesterov, self.ns_steps = momentum, weight_decay, nesterov, ns_steps
        self.ns_carrier = normalize_ns_carrier(ns_carrier)

    def init_single(self, name, p):
        return {"v": torch.zeros_like(p, dtype=torch.float32)}

    def _momentum(self, g, p, st):
        if self.weight_decay != 0:
            g = g + self.weight_decay * p.float()
        st["v"].mul_(self.momentum).add_(g, alpha=1 - self.momentum)
        return g * (1 - self.momentum) + st["v"] * self.momentum if self.nesterov else st["v"]

    def _apply_update(self, update, p):
        lr = self.lr
        if update.dim() >= 2:
            shape = update.shape
            u2 = update.reshape(shape[0], -1)
            u2 = newton_schulz5(u2, steps=self.ns_steps, ns_carrier=self.ns_carrier, output_dtype=torch.float32)
            update = u2.reshape(shape)
            lr = lr * max(1.0, shape[-2] / shape[-1]) ** 0.5
        p.copy_(p.float() - lr * update)

    def apply_single(self, name, grad, p, st):
        if (p.is_cuda and B.kernels_enabled() and self.ns_carrier == "bf16" and p.dim() == 2 and p.is_contiguous()
                and grad.is_contiguous() and p.dtype == grad.dtype and p.shape[0] % 8 == 0 and p.shape[1] % 8 == 0
                and p.dtype in (torch.bfloat16, torch.float32) and type(self) is MuonWithNSCarrier):
            from ..ops.optim import muon_step_
            muon_step_(p, grad, st["v"], self.lr, self.momentum, self.weight_decay, self.nesterov, self.ns_steps)
            return
        self._apply_update(self._momentum(grad.float(), p, st), p)


NS_STREAMS = 4
_ns_stream_pool: dict = {}


def ns_streams(device) -> list:
    """Side streams on which independent Newton–Schulz chains run concurrently: one chain's Gram products only fill about half
    of the SMs (72–128 tiles of a 2048² matrix on 148 SMs), so several matrices are orthogonalised at the same time."""
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    if key not in _ns_stream_pool:
        _ns_stream_pool[key] = [torch.cuda.Stream(device=key) for _ in range(NS_STREAMS)]
    return _ns_stream_pool[key]


def _muon_fast_path(self, g, p) -> bool:
    return (p.is_cuda and B.kernels_enabled() and self.ns_carrier == "bf16" and p.dim() == 2 and p.is_contiguous() and g.is_contiguous()
            and p.dtype == g.dtype and p.shape[0] % 8 == 0 and p.shape[1] % 8 == 0 and p.dtype in (torch.bfloat16, torch.float32)
            and type(self) is MuonWithNSCarrier)


def _muon_step_multistream(self, grads=None) -> None:
    """One Muon step over all matrices.  On the GPU the element-wise stages are one multi-tensor launch each and Newton–Schulz runs
    per stack of equally shaped matrices as batched GEMMs (``ops.optim.MuonBatchPlan``); anything the kernels do not cover
    (fp32 carrier, odd shapes, CPU) takes the per-tensor path."""
    self.step_count += 1
    work = []
    for name, p in self.params:
        g = grads.get(name) if grads is not None else p.grad
        if g is not None:
            work.append((name, g, p, self.state_for(name, p)))
    if not work:
        return
    fast = [w for w in work if _muon_fast_path(self, w[1], w[2])]
    if fast:
        dt0 = fast[0][2].dtype
        fast = [w for w in fast if w[2].dtype == dt0 and w[2].device == fast[0][2].device]
    fast_ids = {id(w[2]) for w in fast}
    for name, g, p, st in work:
        if id(p) not in fast_ids:
            self.apply_single(name, g, p, st)
    if not fast:
        return
    from ..ops.optim import OP_AXPY_UPDATE, OP_MUON_MOMENTUM, OP_SCALE_INV_NORM, MuonBatchPlan, newton_schulz5_batched_
    dev = fast[0][2].device
    plan = getattr(self, "_batch_plan", None)
    if plan is None or plan.device != dev:
        plan = self._batch_plan = MuonBatchPlan(dev)
    n = len(fast)
    if plan.sumsq is None or plan.sumsq.numel() != n:
        plan.sumsq = torch.zeros(n, dtype=torch.float32, device=dev)
    else:
        plan.sumsq.zero_()
    lr = self.lr
    stacks = plan.stacks([tuple(w[2].shape) for w in fast])
    rows_in, rows_out, jobs = [None] * n, [None] * n, []
    for sh, idx in stacks:
        x, nxt, gws, poly = plan.workspace((sh, idx[0]), sh, len(idx))
        res = nxt if self.ns_steps % 2 else x
        jobs.append((x, nxt, gws, poly))
        coef = lr * max(1.0, sh[0] / sh[1]) ** 0.5
        for j, i in enumerate(idx):
            _, g, p, st = fast[i]
            rows_in[i] = dict(p=p.data_ptr(), g=g.data_ptr(), s0=st["v"].data_ptr(), u=x[j].data_ptr(),
                              sumsq=plan.sumsq.data_ptr() + 4 * i, numel=p.numel(), coef=coef)
            rows_out[i] = dict(p=p.data_ptr(), u=res[j].data_ptr(), numel=p.numel(), coef=coef)
    dt = fast[0][2].dtype
    plan.tab_in.update(rows_in)
    plan.tab_in.launch(OP_MUON_MOMENTUM, dt, (self.momentum, self.weight_decay, 1.0 if self.nesterov else 0.0), "muon_momentum_multi")
    plan.tab_in.launch(OP_SCALE_INV_NORM, dt, (1e-7,), "scale_inv_norm_multi")
    main = torch.cuda.current_stream(dev)
    ready = main.record_event()
    streams = ns_streams(dev)
    for s in streams:
        s.wait_event(ready)
    for k, (x, nxt, gws, poly) in enumerate(jobs):      # stacks are sorted largest first and dealt round-robin
        with torch.cuda.stream(streams[k % len(streams)]):
            newton_schulz5_batched_(x, nxt, gws, poly, self.ns_steps)
    for s in streams:
        main.wait_stream(s)
    plan.tab_out.update(rows_out)
    plan.tab_out.launch(OP_AXPY_UPDATE, dt, (), "axpy_update_multi")


MuonWithNSCarrier.step = torch.no_grad()(_muon_step_multistream)


class QuantizedMuonWithNSCarrier(MuonWithNSCarrier):
    """Muon whose momentum lives as uint8 codes + per-256 fp32 absmax (4× smaller state)."""

    def __init__(self, *a, quant_scheme: str = MUON_QUANTIZED_MOMENTUM_SCHEME, **kw):
        super().__init__(*a, **kw)
        if quant_scheme not in ("symmetric_int8_v1", "dynamic_int8_v1"):
            raise ValueError(f"unknown quant_scheme {quant_scheme!r}")
        self.quant_scheme = quant_scheme

    def init_single(self, name, p):
        q, am = quantize_blockwise(torch.zeros(p.numel(), dtype=torch.float32, device=p.device), scheme=self.quant_scheme)
        return {"v_quant": q, "v_absmax": am}

    def apply_single(self, name, grad, p, st):
        v = dequantize_blockwise(st["v_quant"], st["v_absmax"], p.numel(), scheme=self.quant_scheme).view(p.shape)
        tmp = {"v": v}
        update = self._momentum(grad.float(), p, tmp)
        st["v_quant"], st["v_absmax"] = quantize_blockwise(tmp["v"].reshape(-1), scheme=self.quant_scheme)
        self._apply_update(update, p)


class MuonAdamWMulti:
    """Routes 2-D hidden weights to Muon and everything else to a scalar optimizer; state = {muon, adamw}."""

    def __init__(self, muon: Optimizer, other: Optimizer):
        self.muon, self.other = muon, other

    @property
    def params(self) -> NamedParams:
        return self.muon.params + self.other.params

    @property
    def state(self):
        return {"muon": self.muon.state, "adamw": self.other.state}

    @property
    def step_count(self) -> int:
        return self.muon.step_count

    def step(self, grads=None) -> None:
        self.muon.step(grads)
        self.other.step(grads)

    def zero_grad(self) -> None:
        self.muon.zero_grad()
        self.other.zero_grad()

    def state_bytes(self) -> int:
        return self.muon.state_bytes() + self.other.state_bytes()

    def state_dict(self) -> dict:
        return {"muon": self.muon.state_dict(), "adamw": self.other.state_dict()}

    def load_state_dict(self, sd: dict) -> None:
        self.muon.load_state_dict(sd["muon"])
        self.other.load_state_dict(sd["adamw"])


def make_muon(params, *, lr_muon: float = 2e-3, lr_adamw: float = 1e-4, momentum: float = 0.95,
              weight_decay: float = 0.01, adamw_weight_decay: float | None = None, nesterov: bool = True,
              ns_steps: int = 5, ns_carrier: str | None = None, quantized_momentum: bool = False,
              quant_scheme: str = MUON_QUANTIZED_MOMENTUM_SCHEME, scalar_optimizer: str = "adamw",
              cppmega_cuda_parity: bool = False, betas=None, eps: float = 1e-8) -> MuonAdamWMulti:
    carrier = ns_carrier or os.environ.get(MUON_NS_CARRIER_ENV, "fp32")
    if cppmega_cuda_parity:
        lr_adamw = lr_muon
    muon_p, other_p = split_param_groups(params)
    cls = QuantizedMuonWithNSCarrier if quantized_momentum else MuonWithNSCarrier
    kw = dict(quant_scheme=quant_scheme) if quantized_momentum else {}
    muon = cls(muon_p, lr_muon, momentum, weight_decay, nesterov, ns_steps, ns_carrier=carrier, **kw)
    awd = weight_decay if adamw_weight_decay is None else adamw_weight_decay
    so = scalar_optimizer.lower()
    if so == "adamw":
        other = make_adamw(other_p, learning_rate=lr_adamw, weight_decay=awd, betas=betas, eps=eps)
    elif so == "lion":
        other = make_lion(other_p, learning_rate=lr_adamw, weight_decay=awd)
    elif so in ("adam8bit", "lion8bit"):
        from .optimizers_quantized import make_adam8bit, make_lion8bit
        other = (make_adam8bit if so == "adam8bit" else make_lion8bit)(other_p, learning_rate=lr_adamw, weight_decay=awd)
    else:
        raise ValueError(f"scalar_optimizer must be adamw|adam8bit|lion|lion8bit, got {scalar_optimizer!r}")
    return MuonAdamWMulti(muon, other)


def global_grad_norm(params: Iterable[torch.Tensor]) -> torch.Tensor:
    sq = [p.grad.float().pow(2).sum() for p in params if p.grad is not None]
    return torch.stack(sq).sum().sqrt() if sq else torch.zeros(())


def clip_grad_norm_(params, max_norm: float) -> torch.Tensor:
    ps = [p for p in params if p.grad is not None]
    norm = global_grad_norm(ps)
    scale = (max_norm / (norm + 1e-6)).clamp(max=1.0)
    for p in ps:
        p.grad.mul_(scale.to(p.grad.dtype))
    return norm
