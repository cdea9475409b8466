"""Build libthvm_cuda.so (sm_100a) in-tree with nvcc.

`python -m tinyhvm_b200.build` compiles every `csrc/*.cu` to an object and
links `tinyhvm_b200/libthvm_cuda.so`.  Objects are rebuilt only when a source
or header is newer.  `--ptxas` prints register / shared-memory use per kernel.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "build"
LIB = PKG / "libthvm_cuda.so"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function",
         "--expt-relaxed-constexpr", "-Xcudafe", "--diag_suppress=177"]


def _deps(src: Path, seen=None) -> set:
    """The files a source includes with quotes, transitively (so that a change to one kernel's .inc rebuilds only it)."""
    import re
    seen = set() if seen is None else seen
    for name in re.findall(r'^\s*#include\s+"([^"]+)"', src.read_text(), flags=re.M):
        f = (src.parent / name).resolve()
        if f.exists() and f not in seen:
            seen.add(f)
            _deps(f, seen)
    return seen


def _compile(src: Path, verbose_ptxas: bool) -> Path:
    obj = OBJ / (src.stem + ".o")
    stamp = max([src.stat().st_mtime, Path(__file__).stat().st_mtime] + [d.stat().st_mtime for d in _deps(src)])
    if obj.exists() and obj.stat().st_mtime >= stamp and not verbose_ptxas:
        return obj
    cmd = [NVCC, *ARCH, *FLAGS, "-c", str(src), "-o", str(obj)]
    if verbose_ptxas:
        cmd[1:1] = ["-Xptxas", "-v"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    if verbose_ptxas or r.stderr.strip():
        sys.stderr.write(f"--- {src.name}\n{r.stderr}")
    return obj


def build(verbose_ptxas: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    srcs = sorted(CSRC.glob("*.cu"))
    if not srcs:
        raise RuntimeError("no CUDA sources found")
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: _compile(s, verbose_ptxas), srcs))
    if LIB.exists() and all(LIB.stat().st_mtime >= o.stat().st_mtime for o in objs):
        return LIB
    cmd = [NVCC, *ARCH, "-shared", "-o", str(LIB), *map(str, objs), "-lcudart_static", "-lrt", "-ldl", "-lpthread"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(verbose_ptxas="--ptxas" in sys.argv))
