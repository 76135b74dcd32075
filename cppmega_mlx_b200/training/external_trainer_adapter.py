"""Compatibility probes for an external trainer, kept at the edge of the training surface.

The reference keeps MLX-LM's tuner at arm's length: it reports which trainer APIs are installed, normalises its token batches
into the dense mapping that trainer's loss / batching code takes, and refuses the full integration with a stated reason
(``cppmega_mlx/training/mlx_lm_adapter.py:140`` API description, ``:222`` batch mapping, ``:261`` the refusal, ``:58-63`` the
reason).  On this platform the external trainer a user would reach for is Hugging Face ``transformers.Trainer``; the same three
pieces are provided for it.  ``transformers`` is imported lazily and only by ``describe_external_trainer_apis``.
"""
from __future__ import annotations

import importlib
import importlib.metadata
import inspect
from dataclasses import asdict, dataclass, field

import torch

from ..data.batch import LMTokenBatch, ensure_lm_batch

TRAINER_MODULE = "transformers"
TRAINER_API_NAMES = ("Trainer", "TrainingArguments", "DataCollatorForLanguageModeling")
REQUIRED_TRAINER_PARAMETERS: dict[str, tuple[str, ...]] = {
    "Trainer": ("model", "args", "train_dataset", "eval_dataset", "data_collator"),
    "TrainingArguments": ("per_device_train_batch_size", "gradient_accumulation_steps", "max_steps", "gradient_checkpointing"),
    "DataCollatorForLanguageModeling": ("tokenizer", "mlm"),
}
STRUCTURE_FIELD_NAMES = ("structure_ids", "dep_levels", "ast_depth_ids", "sibling_index_ids", "node_type_ids")
DENSE_BATCH_KEYS = ("input_ids", "labels", "attention_mask")
IGNORE_INDEX = -100
UNSUPPORTED_TRAINER_INTEGRATION_REASON = (
    "external trainer integration is unsupported for these models: the trainer takes dense input_ids / labels / attention_mask "
    "batches and drives its own optimizer and checkpoint format, while these batches carry structure side channels and document "
    "ids, the step owns Muon / ZeRO-1 state over flat buffers, and checkpoints hold full pre-training state")


@dataclass(frozen=True)
class ExternalTrainerAPIInfo:
    """Serialisable description of the installed trainer surface."""
    available: bool
    module: str = TRAINER_MODULE
    version: str | None = None
    api_signatures: dict[str, str] = field(default_factory=dict)
    missing_apis: tuple[str, ...] = ()
    incompatible_apis: tuple[str, ...] = ()
    integration_supported: bool = False
    unsupported_reason: str = UNSUPPORTED_TRAINER_INTEGRATION_REASON

    def to_dict(self) -> dict:
        return asdict(self)


@dataclass(frozen=True)
class BatchRouteMetadata:
    """What a batch carries beyond the dense mapping (everything listed in ``dropped`` is lost on the way to the trainer)."""
    batch_size: int
    seq_len: int
    has_attention_mask: bool
    structure_fields: tuple[str, ...]
    has_document_ids: bool
    dropped: tuple[str, ...]


class ExternalTrainerIntegrationUnsupported(NotImplementedError):
    pass


def _signature(obj) -> str:
    try:
        return str(inspect.signature(obj))
    except (TypeError, ValueError):
        return "<signature unavailable>"


def describe_external_trainer_apis(module_name: str = TRAINER_MODULE) -> ExternalTrainerAPIInfo:
    """Import the trainer lazily and report which of the expected entry points exist and take the expected parameters."""
    try:
        mod = importlib.import_module(module_name)
    except Exception:  # noqa: BLE001 - any import failure means "not available"
        return ExternalTrainerAPIInfo(available=False, module=module_name, missing_apis=TRAINER_API_NAMES)
    try:
        version = importlib.metadata.version(module_name)
    except importlib.metadata.PackageNotFoundError:
        version = getattr(mod, "__version__", None)
    sigs, missing, incompatible = {}, [], []
    for name in TRAINER_API_NAMES:
        obj = getattr(mod, name, None)
        if obj is None:
            missing.append(name)
            continue
        sigs[name] = _signature(obj)
        try:
            params = set(inspect.signature(obj).parameters)
        except (TypeError, ValueError):
            params = set()
        if any(p not in params for p in REQUIRED_TRAINER_PARAMETERS[name]):
            incompatible.append(name)
    return ExternalTrainerAPIInfo(available=True, module=module_name, version=version, api_signatures=sigs,
                                  missing_apis=tuple(missing), incompatible_apis=tuple(incompatible))


def as_dense_trainer_batch(batch) -> dict[str, torch.Tensor]:
    """``LMTokenBatch`` (or its mapping form) → ``{"input_ids", "labels", "attention_mask"}``.  ``labels`` are the tokens
    themselves (the external trainer shifts them), with masked positions set to ``-100``; structure channels and document
    ids have no place in this mapping and are dropped (see ``describe_batch_route_metadata``)."""
    b = ensure_lm_batch(batch)
    tokens = b.tokens.long()
    if tokens.numel() and int(tokens.min()) < 0:
        raise ValueError("token ids must be non-negative")
    mask = torch.ones_like(tokens) if b.attention_mask is None else b.attention_mask.to(tokens.dtype)
    labels = torch.where(mask.bool(), tokens, torch.full_like(tokens, IGNORE_INDEX))
    return {"input_ids": tokens, "labels": labels, "attention_mask": mask}


def describe_batch_route_metadata(batch) -> BatchRouteMetadata:
    b = ensure_lm_batch(batch)
    present = tuple(n for n in STRUCTURE_FIELD_NAMES if getattr(b, n) is not None)
    dropped = present + (("document_ids",) if b.document_ids is not None else ())
    return BatchRouteMetadata(batch_size=int(b.tokens.shape[0]), seq_len=int(b.tokens.shape[1]), has_attention_mask=b.attention_mask is not None,
                              structure_fields=present, has_document_ids=b.document_ids is not None, dropped=dropped)


def require_supported_external_trainer_integration(info: ExternalTrainerAPIInfo | None = None) -> None:
    """Always raises: the probe exists so that callers fail with the reason instead of training with silently dropped state."""
    info = info or ExternalTrainerAPIInfo(available=False)
    detail = "" if info.available else f" ({info.module} is not importable here)"
    raise ExternalTrainerIntegrationUnsupported(UNSUPPORTED_TRAINER_INTEGRATION_REASON + detail)
