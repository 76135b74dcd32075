"""ReDo: find dormant hidden units of the FFNs and re-initialise them.

``ReDoDiagnostics`` keeps an EMA of each hidden unit's mean |activation| (the FFN calls ``module._redo_probe(h)`` when a probe
is attached; ``cppmega_mlx/training/plasticity/redo.py:36-115``).  A unit is dormant when its EMA is below ``tau`` × the layer
mean.  ``recycle_dormant_neurons`` overwrites the unit's incoming rows and outgoing column with N(0, (0.1·std)²) noise, zeroes
its bias, and sets its statistic to the layer mean so it is not flagged again at once (``:118-184``).  A fused
``[gate | up]`` matrix is handled as two row blocks of the same unit.
"""
from __future__ import annotations

import torch

DEFAULT_EMA_ALPHA = 0.1
DEFAULT_REDO_TAU = 0.025


class ReDoDiagnostics:
    def __init__(self, ema_alpha: float = DEFAULT_EMA_ALPHA):
        self.stats: dict[str, torch.Tensor] = {}
        self.ema_alpha = float(ema_alpha)
        self._attached: dict[str, torch.nn.Module] = {}

    def attach(self, modules: dict[str, torch.nn.Module]) -> None:
        for name, mod in modules.items():
            mod._redo_probe = self._recorder(name)
            self._attached[name] = mod

    def detach(self) -> None:
        for mod in self._attached.values():
            mod._redo_probe = None
        self._attached.clear()

    def get_stats(self) -> dict[str, torch.Tensor]:
        return self.stats

    def get_dormant_ratio(self, *, tau: float = DEFAULT_REDO_TAU) -> dict[str, float]:
        out = {}
        for name, s in self.stats.items():
            out[name] = float(((s / s.mean().clamp_min(1e-8)) < tau).float().mean())
        return out

    def _recorder(self, name: str):
        def record(h: torch.Tensor) -> None:
            with torch.no_grad():
                m = h.detach().float().abs().reshape(-1, h.shape[-1]).mean(0)
                prev = self.stats.get(name)
                self.stats[name] = m if prev is None else (1 - self.ema_alpha) * prev + self.ema_alpha * m
        return record


def ffn_layer_map(model: torch.nn.Module) -> dict[str, torch.nn.Module]:
    """Every dense FFN in the model, keyed by module path."""
    from ...nn.basic import FeedForward
    return {n: m for n, m in model.named_modules() if isinstance(m, FeedForward)}


@torch.no_grad()
def recycle_dormant_neurons(layer_map: dict[str, torch.nn.Module], stats: dict[str, torch.Tensor], *, tau: float = DEFAULT_REDO_TAU,
                            generator: torch.Generator | None = None) -> int:
    total = 0
    for name, ffn in layer_map.items():
        s = stats.get(name)
        if s is None:
            continue
        mean = s.mean().clamp_min(1e-8)
        dormant = (s / mean) < tau
        n = int(dormant.sum())
        if n == 0:
            continue
        w_out = ffn.down_proj.weight                                   # [d, hidden]: column per unit
        noise = torch.randn(w_out.shape, generator=generator).to(w_out.device, w_out.dtype) * (w_out.float().std().clamp_min(1e-8) * 0.1)
        w_out.copy_(torch.where(dormant[None, :].to(w_out.device), noise, w_out))
        w_in = ffn.gate_up_proj.weight if hasattr(ffn, "gate_up_proj") else ffn.up_proj.weight
        rows = torch.cat([dormant, dormant]) if hasattr(ffn, "gate_up_proj") else dormant
        noise = torch.randn(w_in.shape, generator=generator).to(w_in.device, w_in.dtype) * (w_in.float().std().clamp_min(1e-8) * 0.1)
        w_in.copy_(torch.where(rows[:, None].to(w_in.device), noise, w_in))
        stats[name] = torch.where(dormant, mean, s)
        total += n
    return total
