"""Read-only environment report (``scripts/check_environment.py`` of the reference, ``:266-320`` for the distributed-backend
probe): interpreter, torch / CUDA / NCCL versions, GPUs, whether the kernel library is built and loads with the right ABI,
which ``torch.distributed`` backends exist, and the measured roofline file.  Changes nothing; always exits 0 unless ``--strict``
is given and the machine cannot run the kernel path."""
from __future__ import annotations

import argparse
import json
import sys


def collect() -> dict:
    import torch
    import torch.distributed as dist

    from ..ops import _backend as B
    from ..runtime.env import detect_runtime_environment
    from ..utils.measure import measured_peaks
    env = detect_runtime_environment().to_dict()
    lib = {"path": str(B.lib_path()), "built": B.has_library(), "loads": False, "abi": None, "error": None}
    if lib["built"]:
        try:
            handle = B.load_library()
            lib["loads"], lib["abi"] = True, int(handle.cmb_abi_version())
        except (OSError, RuntimeError) as e:   # a CPU-only machine cannot resolve libcudart: report, do not fail
            lib["error"] = str(e).splitlines()[0][:200]
    backends = {"nccl": dist.is_available() and dist.is_nccl_available(), "gloo": dist.is_available() and dist.is_gloo_available(),
                "mpi": dist.is_available() and dist.is_mpi_available()}
    peaks = measured_peaks()
    return {"environment": env, "kernel_library": lib, "distributed_backends": backends,
            "measured_peaks": {"fallback": bool(peaks.get("fallback", False)), "hbm_gbs": peaks.get("hbm_gbs"),
                               "bf16_tflops": peaks.get("bf16_tflops")},
            "kernel_path_ready": bool(env["cuda_available"] and lib["loads"] and env["hardware_tier"] == "b200")}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--strict", action="store_true", help="exit 1 when the sm_100a kernel path cannot run here")
    args = ap.parse_args(argv)
    rep = collect()
    if args.json:
        print(json.dumps(rep, indent=1))
    else:
        e = rep["environment"]
        print(f"python {e['python']}  torch {e['torch']}  cuda {e['cuda_runtime']}  nccl {e['nccl']}  tier {e['hardware_tier']}")
        for g in e["gpus"]:
            print(f"  gpu{g['index']}: {g['name']} sm_{g['capability'].replace('.', '')} {g['sm_count']} SMs "
                  f"{g['total_memory_bytes'] / 2**30:.0f} GiB")
        k = rep["kernel_library"]
        print(f"kernel library: built={k['built']} loads={k['loads']} abi={k['abi']}" + (f" ({k['error']})" if k["error"] else ""))
        print("distributed backends: " + ", ".join(n for n, ok in rep["distributed_backends"].items() if ok))
        print(f"kernel path ready: {rep['kernel_path_ready']}")
    return 1 if (args.strict and not rep["kernel_path_ready"]) else 0


if __name__ == "__main__":
    sys.exit(main())
