"""In-tree build of ``libstark_b200.so`` (nvcc, sm_100a only).

``python -m stark_b200.build`` compiles every ``csrc/*.cu`` into one shared library that sits next
to this file, so that it travels with the source tree.  No torch headers are involved: the library
is plain CUDA runtime code behind the C ABI in ``include/stark_b200.h``.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "csrc" / "build"
LIB = PKG / "libstark_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
]
if os.environ.get("STARK_B200_PTXAS_V"):
    NVCC_FLAGS += ["-Xptxas", "-v"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found: the CUDA toolkit is required to build libstark_b200.so")


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    nvcc = _nvcc()
    OBJ.mkdir(exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "stark_b200.h"]
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)

    def compile_one(src: Path) -> Path:
        obj = OBJ / (src.stem + ".o")
        if force or _stale(obj, [src] + headers):
            cmd = [nvcc, *NVCC_FLAGS, "-ccbin", "/usr/bin/g++", "-c", str(src), "-o", str(obj)]
            res = subprocess.run(cmd, capture_output=True, text=True, env=env)
            if verbose or res.returncode:
                sys.stderr.write(res.stdout + res.stderr)
            if res.returncode:
                raise RuntimeError(f"nvcc failed on {src.name}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        objs = list(pool.map(compile_one, sources))
    if force or _stale(LIB, objs):
        cmd = [nvcc, "-shared", "-ccbin", "/usr/bin/g++", "-o", str(LIB), *map(str, objs), "-lcudart"]
        res = subprocess.run(cmd, capture_output=True, text=True, env=env)
        if res.returncode:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("link of libstark_b200.so failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
