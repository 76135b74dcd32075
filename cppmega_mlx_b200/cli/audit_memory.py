"""Parameter / optimizer-state memory audit of a model profile without allocating it (``scripts/audit_memory.py`` of the
reference): the model is built on the ``meta`` device, so even the 56-layer profile reports in a second.  Bytes by dtype, by
optimizer category (Muon matrices / AdamW tensors / embeddings) and by top-level module, the largest leaves, and what ZeRO-1
over ``--dp`` ranks leaves per GPU against the 180 GB of a B200."""
from __future__ import annotations

import argparse
import json
import sys

import torch


def run(profile: str, dp: int, seq_len: int | None) -> dict:
    from ..recipes.model_factory import get_model_profile
    from ..runtime.memory_audit import audit_memory
    p = get_model_profile(profile)
    kw = {} if seq_len is None else {"max_seq_length": seq_len}
    with torch.device("meta"):
        model = p.build_model(dtype=torch.bfloat16, device="meta", **kw)
    rep = audit_memory(model)
    params = sum(x.numel() for x in model.parameters())
    pbytes = 2 * params
    # ZeRO-1 budget per GPU: bf16 params + bf16 grads replicated, fp32 moments (Muon: 1 per matrix element, AdamW: 2) sharded
    cat = rep.get("by_category", {})
    muon_el, adam_el = cat.get("muon", 0) // 2, (cat.get("adamw", 0) + cat.get("embedding", 0)) // 2
    state = 4 * muon_el + 8 * adam_el
    per_gpu = 2 * pbytes + state / max(dp, 1)
    rep.update({"profile": profile, "parameters": params, "zero1": {"dp": dp, "replicated_param_and_grad_bytes": 2 * pbytes,
                "optimizer_state_bytes_total": state, "per_gpu_bytes_before_activations": int(per_gpu),
                "fraction_of_b200_hbm": per_gpu / (180 * 2**30)}})
    return rep


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--profile", default="hybrid_1b")
    ap.add_argument("--dp", type=int, default=8)
    ap.add_argument("--seq-len", type=int)
    args = ap.parse_args(argv)
    try:
        rep = run(args.profile, args.dp, args.seq_len)
    except Exception as e:  # noqa: BLE001
        print(json.dumps({"status": "error", "error": f"{type(e).__name__}: {e}"}))
        return 2
    print(json.dumps(rep, default=str))
    return 0


if __name__ == "__main__":
    sys.exit(main())
