"""In-tree build of the CUDA library: nvcc -> vibe_megakernel_b200/lib/libmoe_b200.so (sm_100a only)."""

from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "lib" / "libmoe_b200.so"
SOURCES = ("api.cu", "megamoe.cu", "gemm_mx.cu", "gemm_mx_wide.cu", "route.cu", "router_logits.cu", "route_static.cu","group.cu", "quant.cu", "combine.cu", "rmsnorm.cu", "gemm_tc.cu", "gemm_wide.cu", "gemm_simt.cu", "ep.cu", "experts.cu", "latent.cu", "dense_tc.cu", "selfcheck.cu")
FLAGS = ("-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
         "--expt-relaxed-constexpr")


def nvcc() -> str:
    return os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")


def stale() -> bool:
    if not LIB.exists():
        return True
    newest = max(p.stat().st_mtime for p in list(CSRC.iterdir()) + [PKG.parent / "include" / "moe_b200.h"])
    return newest > LIB.stat().st_mtime


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not stale():
        return LIB
    LIB.parent.mkdir(exist_ok=True)
    objs = []
    procs = []
    for src in SOURCES:
        obj = LIB.parent / (src + ".o")
        cmd = [nvcc(), *FLAGS, "-c", str(CSRC / src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(str(obj))
    failed = False
    for src, proc in procs:
        out, _ = proc.communicate()
        if proc.returncode or verbose:
            sys.stderr.write(f"--- {src}\n{out}\n")
        failed |= proc.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    subprocess.run([nvcc(), "-shared", "-o", str(LIB), *objs, "-lcudart"], check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
