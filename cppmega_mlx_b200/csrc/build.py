"""Build the sm_100a kernel library in-tree: ``python -m cppmega_mlx_b200.csrc.build``.

Every ``*.cu`` beside this file is compiled with
``nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo`` to an object file and the objects are
linked into ``libcppmega_b200.so`` (plain C ABI, loaded with ctypes).  nvcc cross-compiles without
a GPU, so this also runs on CPU-only build machines.  Objects are rebuilt only when their source
(or a header) is newer.  Equivalent of the reference's CMake + metallib build
(``cppmega_mlx/training/native_optim/CMakeLists.txt:35-49``, ``setup.py:8-14``).
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB = HERE / "libcppmega_b200.so"
OBJ_DIR = HERE / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
    "--expt-relaxed-constexpr",
]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found")
    return exe


def sources() -> list[Path]:
    return sorted(HERE.glob("*.cu"))


def _newest_header() -> float:
    return max((p.stat().st_mtime for p in list(HERE.glob("*.cuh")) + list(HERE.glob("*.h"))), default=0.0)


def _compile(src: Path, verbose: bool, ptxas_v: bool) -> Path:
    obj = OBJ_DIR / (src.stem + ".o")
    stamp = max(src.stat().st_mtime, _newest_header())
    if obj.exists() and obj.stat().st_mtime >= stamp:
        return obj
    cmd = [nvcc(), *NVCC_FLAGS, "-c", str(src), "-o", str(obj), "-I", str(HERE)]
    if ptxas_v:
        cmd += ["-Xptxas", "-v"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    if verbose or ptxas_v:
        sys.stderr.write(res.stderr)
    return obj


def build(verbose: bool = False, ptxas_v: bool = False, force: bool = False) -> Path:
    OBJ_DIR.mkdir(exist_ok=True)
    if force:
        for o in OBJ_DIR.glob("*.o"):
            o.unlink()
    srcs = sources()
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(lambda s: _compile(s, verbose, ptxas_v), srcs))
    newest_obj = max(o.stat().st_mtime for o in objs)
    if LIB.exists() and LIB.stat().st_mtime >= newest_obj and not force:
        return LIB
    cmd = [nvcc(), "-shared", "-o", str(LIB), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a",
           "-Xcompiler", "-fPIC", "-lcudart"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB


if __name__ == "__main__":
    out = build(verbose="-v" in sys.argv, ptxas_v="--ptxas" in sys.argv, force="--force" in sys.argv)
    print(out)
