"""Tensor-parity receipts: compare tensors produced here against tensors from an external artifact (another framework's dump,
a previous build, the eager arm) and record the verdict in a manifest.  An artifact that is missing yields a ``refused`` receipt
— never a silent pass (``cppmega_mlx/training/parity.py:443`` receipt, ``:499-560`` compare, ``:663-880`` manifests,
tolerances atol 1e-1 / rtol 1e-2 ``:43-44``)."""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, Mapping

import torch

DEFAULT_ATOL = 1e-1
DEFAULT_RTOL = 1e-2
STATUS_PASS, STATUS_FAIL, STATUS_REFUSED = "pass", "fail", "refused"


@dataclass(frozen=True)
class TensorParityReceipt:
    name: str
    status: str
    reason: str = ""
    shape: tuple[int, ...] = ()
    dtype: str = ""
    max_abs_diff: float | None = None
    max_rel_diff: float | None = None
    mismatched_fraction: float | None = None
    atol: float = DEFAULT_ATOL
    rtol: float = DEFAULT_RTOL

    def to_dict(self) -> dict:
        return asdict(self)


def compare_tensors(name: str, ours: torch.Tensor | None, theirs: torch.Tensor | None, *, atol: float = DEFAULT_ATOL,
                    rtol: float = DEFAULT_RTOL) -> TensorParityReceipt:
    if theirs is None:
        return TensorParityReceipt(name, STATUS_REFUSED, "external artifact has no tensor with this name", atol=atol, rtol=rtol)
    if ours is None:
        return TensorParityReceipt(name, STATUS_REFUSED, "no local tensor with this name", atol=atol, rtol=rtol)
    if tuple(ours.shape) != tuple(theirs.shape):
        return TensorParityReceipt(name, STATUS_FAIL, f"shape {tuple(ours.shape)} != {tuple(theirs.shape)}", tuple(ours.shape),
                                   str(ours.dtype), atol=atol, rtol=rtol)
    a, b = ours.detach().float().cpu(), theirs.detach().float().cpu()
    if not (torch.isfinite(a).all() and torch.isfinite(b).all()):
        return TensorParityReceipt(name, STATUS_FAIL, "non-finite values", tuple(a.shape), str(ours.dtype), atol=atol, rtol=rtol)
    diff = (a - b).abs()
    bad = diff > atol + rtol * b.abs()
    rel = (diff / b.abs().clamp_min(1e-12))
    ok = not bool(bad.any())
    return TensorParityReceipt(name, STATUS_PASS if ok else STATUS_FAIL, "" if ok else "values differ beyond tolerance", tuple(a.shape),
                               str(ours.dtype), float(diff.max()) if diff.numel() else 0.0, float(rel.max()) if rel.numel() else 0.0,
                               float(bad.float().mean()) if bad.numel() else 0.0, atol, rtol)


@dataclass
class ParityManifest:
    label: str
    artifact: str | None
    receipts: list[TensorParityReceipt] = field(default_factory=list)
    metadata: dict[str, Any] = field(default_factory=dict)

    @property
    def status(self) -> str:
        if not self.receipts or any(r.status == STATUS_REFUSED for r in self.receipts):
            return STATUS_REFUSED
        return STATUS_PASS if all(r.status == STATUS_PASS for r in self.receipts) else STATUS_FAIL

    def to_dict(self) -> dict:
        return {"label": self.label, "artifact": self.artifact, "status": self.status, "metadata": self.metadata,
                "receipts": [r.to_dict() for r in self.receipts]}

    def write(self, path) -> None:
        Path(path).write_text(json.dumps(self.to_dict(), indent=2, sort_keys=True) + "\n")


def parity_against_artifact(label: str, ours: Mapping[str, torch.Tensor], artifact_path, *, names=None, atol: float = DEFAULT_ATOL,
                            rtol: float = DEFAULT_RTOL) -> ParityManifest:
    """``artifact_path``: a safetensors file of reference tensors. Missing file → every receipt is ``refused``."""
    from . import safetensors_io as st
    p = Path(artifact_path) if artifact_path is not None else None
    names = list(names) if names is not None else sorted(ours)
    if p is None or not p.exists():
        why = "external artifact is absent" if p is None else f"external artifact {p} does not exist"
        return ParityManifest(label, str(p) if p else None, [TensorParityReceipt(n, STATUS_REFUSED, why, atol=atol, rtol=rtol) for n in names])
    theirs = st.load_file(p)
    return ParityManifest(label, str(p), [compare_tensors(n, ours.get(n), theirs.get(n), atol=atol, rtol=rtol) for n in names])


def forward_parity_manifest(model, input_ids: torch.Tensor, artifact_path, *, label: str = "forward") -> ParityManifest:
    """Logits and final hidden state of ``model`` on ``input_ids`` against an artifact holding ``logits`` / ``hidden``."""
    was = model.training
    model.eval()
    with torch.no_grad():
        h = model.decoder_hidden_states(input_ids)
        ours = {"hidden": h, "logits": model.lm_head(h)}
    model.train(was)
    return parity_against_artifact(label, ours, artifact_path)
