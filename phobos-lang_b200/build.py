"""Builds libphobos_leaf.so (hand-written sm_100a CUDA + the C++ host side) in-tree with nvcc.

Usage: ``python phobos-lang_b200/build.py [--force] [--verbose]``.  nvcc cross-compiles
without a GPU; the resulting shared library sits next to this file.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OBJ = HERE / "build"
LIB = HERE / "libphobos_leaf.so"
SOURCES = ["api.cu", "gemm_tc.cu", "gemm_tc2.cu", "gemm_f32.cu", "flash.cu", "elementwise.cu", "kda.cu", "tmap.cu", "noalloc.cu", "selftest.cu",
           "host.cpp", "executor.cpp", "source.cpp", "planner.cpp", "plan_api.cpp", "wire.cpp"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall", "-Xptxas", "-v"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def _deps_mtime() -> float:
    files = [p for p in CSRC.iterdir() if p.suffix in (".cu", ".cuh", ".h", ".cpp")]
    files.append(HERE.parent / "include" / "phobos_leaf.h")
    files.append(Path(__file__))
    return max(p.stat().st_mtime for p in files)


def build(force: bool = False, verbose: bool = False) -> Path:
    sources = [s for s in SOURCES if (CSRC / s).exists()]
    if not force and LIB.exists() and LIB.stat().st_mtime >= _deps_mtime():
        return LIB
    OBJ.mkdir(exist_ok=True)
    nvcc = _nvcc()
    env = dict(os.environ)
    # the environment may export CC/CXX pointing at a wrapper; nvcc should use the system g++
    env.pop("CC", None)
    env.pop("CXX", None)

    def compile_one(src: str) -> tuple[str, str]:
        obj = OBJ / (src.rsplit(".", 1)[0] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-x", "cu", "-c", str(CSRC / src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True, env=env)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        return str(obj), r.stderr

    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        results = list(pool.map(compile_one, sources))
    if verbose:
        for _, log in results:
            for line in log.splitlines():
                if "registers" in line or "spill" in line:
                    print(line)
    link = [nvcc, "-shared", "-o", str(LIB), *[o for o, _ in results], "-gencode",
            "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"]
    r = subprocess.run(link, capture_output=True, text=True, env=env)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
