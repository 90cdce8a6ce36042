"""Build libdecidra_b200.so in-tree with nvcc for sm_100a (no GPU needed to compile).

Usage: python -m decidra_b200.build [--force]
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB = HERE / "libdecidra_b200.so"
CUDA_SOURCES = ["gemm_tcgen05.cu", "gemm_nvfp4.cu", "gemm_w4a16.cu", "attn_tcgen05.cu", "attn_noalloc.cu", "gdn_chunked.cu", "gdn_tcgen05.cu", "gdn_wy.cu", "kernels.cu", "engine.cu", "kapi.cu"]
CXX_SOURCES = ["host_logic.cpp", "checkpoint.cpp", "scheduler.cpp", "prompt.cpp"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; the library cannot be built")


def _stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(CSRC.glob("*.cpp"))
    deps.append(HERE.parent / "include" / "decidra_b200.h")
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not _stale():
        return LIB
    nvcc = _nvcc()
    obj_dir = HERE / "_build"
    obj_dir.mkdir(exist_ok=True)
    common = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=hidden", *ARCH]
    objs = []
    procs = []
    for src in CUDA_SOURCES + CXX_SOURCES:
        obj = obj_dir / (src.rsplit(".", 1)[0] + ".o")
        cmd = [nvcc, *common, "-c", str(CSRC / src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(str(obj))
    for src, p in procs:
        out, _ = p.communicate()
        if verbose and out:
            print(out)
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{out}")
    link = [nvcc, "-shared", *ARCH, "-o", str(LIB), *objs, "-lcudart"]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}")
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
