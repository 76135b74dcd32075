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


# ----------------------------------------------------------------------------------------------- MTP loss parity
MTP_ARTIFACT_FORMAT = "cppmega_mtp_reference_v1"
PREFLIGHT_STATUSES = ("not_supplied", "missing", "invalid", "valid")


def loss_values_sha256(loss_values: Mapping[str, Any]) -> str:
    """Checksum over the loss scalars of an artifact (keys sorted, values as repr of their float), so a manifest can show that
    the numbers it compared are the numbers the artifact was published with."""
    import hashlib
    blob = json.dumps({k: repr(float(v)) for k, v in sorted(loss_values.items())}, sort_keys=True).encode()
    return hashlib.sha256(blob).hexdigest()


def validate_mtp_artifact(payload: Any, *, profile: str | None, mtp_depth: int, mtp_beta: float, mtp_lambda: float) -> None:
    """Contract of an external MTP reference artifact (JSON): format tag, the profile and MTP hyper-parameters it was produced
    with (they must equal ours — comparing losses of different objectives proves nothing), finite ``loss_values`` with a main
    loss, one entry per depth and the total, and a matching checksum.  Raises ``ValueError`` naming the first violation."""
    if not isinstance(payload, Mapping):
        raise ValueError("artifact must be a JSON object")
    if payload.get("format") != MTP_ARTIFACT_FORMAT:
        raise ValueError(f"artifact format must be {MTP_ARTIFACT_FORMAT!r}")
    if profile is not None and payload.get("profile") != profile:
        raise ValueError(f"artifact profile {payload.get('profile')!r} is not {profile!r}")
    if payload.get("mtp_depth") != mtp_depth:
        raise ValueError(f"artifact mtp_depth {payload.get('mtp_depth')!r} is not {mtp_depth}")
    for key, want in (("mtp_beta", mtp_beta), ("mtp_lambda", mtp_lambda)):
        got = payload.get(key)
        if not isinstance(got, (int, float)) or isinstance(got, bool) or abs(float(got) - want) > 1e-12:
            raise ValueError(f"artifact {key} {got!r} is not {want}")
    lv = payload.get("loss_values")
    if not isinstance(lv, Mapping):
        raise ValueError("artifact loss_values must be an object")
    need = ["main_loss", "total_loss"] + [f"mtp_loss_depth_{d + 1}" for d in range(mtp_depth)]
    for k in need:
        v = lv.get(k)
        if not isinstance(v, (int, float)) or isinstance(v, bool) or v != v or v in (float("inf"), float("-inf")):
            raise ValueError(f"artifact loss_values.{k} must be a finite number")
    if payload.get("loss_values_sha256") != loss_values_sha256({k: lv[k] for k in need}):
        raise ValueError("artifact loss_values_sha256 does not match its loss_values")


def mtp_artifact_preflight(artifact_path, **contract) -> dict:
    """Status of the external artifact without comparing anything: ``not_supplied`` / ``missing`` / ``invalid`` / ``valid``."""
    out = {"artifact": None if artifact_path is None else str(artifact_path), "artifact_contract": {"format": MTP_ARTIFACT_FORMAT, **contract},
           "artifact_error": None, "payload": None}
    if artifact_path is None:
        return {**out, "artifact_preflight_status": "not_supplied", "artifact_error": "no reference artifact path was supplied"}
    p = Path(artifact_path)
    if not p.is_file():
        return {**out, "artifact_preflight_status": "missing", "artifact_error": f"reference artifact not found: {p}"}
    try:
        payload = json.loads(p.read_text())
        validate_mtp_artifact(payload, **contract)
    except (OSError, ValueError) as e:
        return {**out, "artifact_preflight_status": "invalid", "artifact_error": str(e)}
    return {**out, "artifact_preflight_status": "valid", "payload": payload}


def local_mtp_loss_values(model, batch) -> dict[str, float]:
    """Main next-token loss, the MTP loss of every depth, their weighted total and the global gradient norm of the total on
    ``model`` for ``batch`` (one forward + backward; gradients are cleared afterwards)."""
    from ..data.batch import ensure_lm_batch
    from .loss import _targets_and_mask, masked_cross_entropy
    from .mtp import compute_mtp_step_weights, next_token_and_mtp_loss
    cfg = model.config
    head = getattr(model, "mtp_head", None)
    depth = int(getattr(cfg, "mtp_depth", 0)) if (head is not None and getattr(cfg, "mtp_enabled", False)) else 0
    if depth <= 0:
        raise ValueError("the model has no MTP head (mtp_enabled is off)")
    model.zero_grad(set_to_none=True)
    b = ensure_lm_batch(batch)
    dev = next(model.parameters()).device
    t, valid = _targets_and_mask(b)
    t, valid = t.to(dev), valid.to(dev)
    side = {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in b.side_inputs().items()}
    h = model.decoder_hidden_states(b.inputs.to(dev), **side)
    main = masked_cross_entropy(model.lm_head(h), t, valid)
    tt = torch.where(valid, t, torch.full_like(t, head.config.ignore_index))
    mtp_loss, per, _ = head.loss(h, tt, document_ids=side.get("document_ids"))
    total = next_token_and_mtp_loss(main, mtp_loss, loss_weight=head.config.loss_weight)
    total.backward()
    gsq = sum(float(p.grad.float().pow(2).sum()) for p in model.parameters() if p.grad is not None)
    model.zero_grad(set_to_none=True)
    vals = {"main_loss": float(main.detach()), "total_loss": float(total.detach()), "mtp_loss": float(mtp_loss.detach()), "grad_norm": gsq ** 0.5}
    for d in range(depth):
        vals[f"mtp_loss_depth_{d + 1}"] = float(per[d].detach())
    vals["mtp_depth_weights"] = [float(w) for w in compute_mtp_step_weights(depth, float(cfg.mtp_decay))]
    return vals


def mtp_parity_manifest(model, batch, artifact_path, *, profile: str | None = None, atol: float = 1e-2, rtol: float = 1e-2) -> dict:
    """Fail-closed MTP parity manifest: local loss values are always recorded; the verdict is ``blocked`` without an artifact,
    ``refused`` for a missing or invalid one, and ``pass`` / ``fail`` only when a valid artifact's numbers were actually compared."""
    cfg = model.config
    contract = dict(profile=profile, mtp_depth=int(cfg.mtp_depth), mtp_beta=float(cfg.mtp_decay), mtp_lambda=float(cfg.mtp_loss_weight))
    pre = mtp_artifact_preflight(artifact_path, **contract)
    local = local_mtp_loss_values(model, batch)
    scalar_keys = [k for k in local if k.startswith(("main_loss", "total_loss", "mtp_loss_depth_"))]
    receipts, status = [], {"not_supplied": "blocked", "missing": STATUS_REFUSED, "invalid": STATUS_REFUSED}.get(pre["artifact_preflight_status"])
    if status is None:
        theirs = pre["payload"]["loss_values"]
        for k in scalar_keys:
            receipts.append(compare_tensors(k, torch.tensor([local[k]]), torch.tensor([float(theirs[k])]), atol=atol, rtol=rtol).to_dict())
        if "grad_norm" in theirs:
            receipts.append(compare_tensors("grad_norm", torch.tensor([local["grad_norm"]]), torch.tensor([float(theirs["grad_norm"])]),
                                            atol=atol, rtol=5 * rtol).to_dict())
        status = STATUS_PASS if all(r["status"] == STATUS_PASS for r in receipts) else STATUS_FAIL
    pre.pop("payload")
    return {"label": "mtp", "status": status, "profile": profile, "mtp_depth": contract["mtp_depth"], "mtp_beta": contract["mtp_beta"],
            "mtp_lambda": contract["mtp_lambda"], "reference": {**pre, "evaluated_by_this_manifest": bool(receipts)},
            "local": {"loss_values": local, "loss_values_sha256": loss_values_sha256({k: local[k] for k in scalar_keys})},
            "receipts": receipts, "tolerances": {"atol": atol, "rtol": rtol}}


def export_mtp_artifact(model, batch, path, *, profile: str | None = None) -> dict:
    """Write this build's own MTP loss values in the artifact format (what another implementation would compare against)."""
    cfg = model.config
    local = local_mtp_loss_values(model, batch)
    scalars = {k: v for k, v in local.items() if k.startswith(("main_loss", "total_loss", "mtp_loss_depth_"))}
    payload = {"format": MTP_ARTIFACT_FORMAT, "profile": profile, "mtp_depth": int(cfg.mtp_depth), "mtp_beta": float(cfg.mtp_decay),
               "mtp_lambda": float(cfg.mtp_loss_weight), "loss_values": {**scalars, "grad_norm": local["grad_norm"]},
               "loss_values_sha256": loss_values_sha256(scalars)}
    Path(path).write_text(json.dumps(payload, indent=2, sort_keys=True) + "\n")
    return payload
