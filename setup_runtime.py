"""Build the C-ABI extension `llmrqt_sdv1_b200/libawq_b200.so` for sm_100a.

Same entry-point name as the reference's build script
(LLMQRT/setup_runtime.py:19-55), but it drives nvcc directly: the product is a
plain shared library with `extern "C"` symbols (see include/awq_b200.h), not a
torch/pybind extension, so nothing here needs a GPU or torch at build time.

    python setup_runtime.py            # build in-tree (also: `build_ext`, `install`)
    python setup_runtime.py --verbose  # add -Xptxas -v (registers / spills / smem)
    python setup_runtime.py --force    # rebuild even if up to date
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "llmrqt_sdv1_b200")
CSRC = os.path.join(PKG, "csrc")
INCLUDE = os.path.join(ROOT, "include")
BUILD = os.path.join(ROOT, "build", "awq_b200")
LIB = os.path.join(PKG, "libawq_b200.so")

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
          "-I", INCLUDE, "-I", CSRC]


def _nvcc() -> str:
    for cand in (os.environ.get("CUDA_NVCC_EXECUTABLE"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set CUDA_NVCC_EXECUTABLE)")


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _newest_input() -> float:
    files = sources() + [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    files += [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)]
    files.append(os.path.abspath(__file__))
    return max(os.path.getmtime(f) for f in files)


def up_to_date() -> bool:
    return os.path.exists(LIB) and os.path.getmtime(LIB) >= _newest_input()


def build(verbose: bool = False, force: bool = False) -> str:
    """Compile every .cu under csrc/ for sm_100a and link the shared library. Returns its path."""
    if not force and up_to_date():
        return LIB
    nvcc = _nvcc()
    os.makedirs(BUILD, exist_ok=True)
    extra = ["-Xptxas", "-v"] if verbose else []

    def compile_one(src: str) -> str:
        obj = os.path.join(BUILD, os.path.basename(src)[:-3] + ".o")
        cmd = [nvcc, *ARCH_FLAGS, *COMMON, *extra, "-c", src, "-o", obj]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or res.returncode != 0:
            sys.stderr.write(f"$ {' '.join(cmd)}\n{res.stdout}{res.stderr}")
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}")
        return obj

    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, sources()))
    tmp = LIB + ".tmp"
    cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", tmp, *objs, "-cudart", "static"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("link failed")
    os.replace(tmp, LIB)
    return LIB


if __name__ == "__main__":
    args = [a for a in sys.argv[1:] if a not in ("install", "build_ext", "--inplace", "develop")]
    path = build(verbose="--verbose" in args, force="--force" in args)
    print(path)
