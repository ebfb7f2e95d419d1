"""Builds the C-ABI shared library ``lib/librte_b200.so`` (CUDA kernels for sm_100a) in-tree.

    python -m speedup_thingy_b200.build          # rebuild if sources are newer than the library

nvcc cross-compiles without a GPU, so this also runs on a CPU-only build machine.
"""
from __future__ import annotations

import os
import shlex
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
LIB = PKG / "lib" / "librte_b200.so"
SOURCES = ["gemm_tcgen05.cu", "elementwise.cu", "attention.cu", "macro_phi.cu", "router.cu", "audit.cu", "shortlist.cu", "cluster_pool.cu", "svd_ffn.cu", "gemm_small.cu", "codebook.cu", "allreduce.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found: cannot build librte_b200.so")
    return exe


def needs_build() -> bool:
    if not LIB.exists():
        return True
    newest = max(p.stat().st_mtime for p in [*CSRC.glob("*.cu"), *CSRC.glob("*.cuh"), ROOT / "include" / "rte_b200.h",
                                             Path(__file__)])
    return newest > LIB.stat().st_mtime


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not needs_build():
        return LIB
    LIB.parent.mkdir(parents=True, exist_ok=True)
    objs = []
    procs = []
    for src in SOURCES:
        path = CSRC / src
        if not path.exists():
            continue
        obj = LIB.parent / (path.stem + ".o")
        # RTE_NVCC_EXTRA: extra compiler flags, e.g. -DRTE_GEMM_DIAG (the GEMM's timing diagnostics: with it the
        # environment variable RTE_GEMM_DIAG_FLAGS switches off stores / MMAs / loads inside the kernel)
        cmd = [_nvcc(), *NVCC_FLAGS, *shlex.split(os.environ.get("RTE_NVCC_EXTRA", "")), "-I", str(ROOT / "include"),
               "-I", str(CSRC), "-c", str(path), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(str(obj))
    for src, proc in procs:
        out, _ = proc.communicate()
        if verbose or proc.returncode != 0:
            sys.stderr.write(out)
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}")
    link = [_nvcc(), "-shared", "-o", str(LIB), *objs, "-cudart", "static", "-Xlinker", "--exclude-libs=ALL"]
    res = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout)
        raise RuntimeError("link of librte_b200.so failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
