"""In-tree build of the CUDA library: nvcc, sm_100a only, no fallback architecture.

    python -m dadgpt_b200.build            # build if sources are newer than the library
    python -m dadgpt_b200.build --force
    python -m dadgpt_b200.build --ptxas    # also print registers / spills / shared memory

Outputs (next to this file, git-ignored, they travel with the working tree):
    libdadattn.so          kernels + C ABI (include/dadattn.h)
    libdadattn_gpuops.so   the three C++ symbols DadGPT's model.cpp links against
                           (gpu_flash_attention_*, reference cuda/gpu_ops.cuh:115-122)
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "libdadattn.so")
SHIM = os.path.join(PKG, "libdadattn_gpuops.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA library cannot be built")
    return exe


def _newer(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build(force: bool = False, ptxas: bool = False) -> str:
    cu = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    deps = cu + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(ROOT, "include", "*.h"))
    inc = ["-I", os.path.join(ROOT, "include"), "-I", CSRC]
    if force or ptxas or _newer(LIB, deps):
        objs = []
        procs = []
        os.makedirs(os.path.join(PKG, "build"), exist_ok=True)
        for src in cu:
            obj = os.path.join(PKG, "build", os.path.basename(src)[:-3] + ".o")
            objs.append(obj)
            if not (force or ptxas) and not _newer(obj, [src] + deps[len(cu):]):
                continue
            cmd = [_nvcc(), *NVCC_FLAGS, *inc, "-c", src, "-o", obj]
            if ptxas:
                cmd += ["-Xptxas", "-v"]
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                                                text=True)))
        for src, p in procs:
            out, _ = p.communicate()
            if p.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src}:\n{out}")
            if ptxas or "warning" in out:
                sys.stderr.write(out)
        subprocess.run([_nvcc(), "-shared", "-o", LIB, *objs, "-ldl"], check=True)
    shim_src = os.path.join(CSRC, "gpu_ops_attention.cpp")
    if force or _newer(SHIM, [shim_src, LIB]):
        cxx = shutil.which("g++") or "g++"
        subprocess.run([cxx, "-std=c++20", "-O2", "-fPIC", "-shared", "-I", os.path.join(ROOT, "include"),
                        shim_src, "-o", SHIM, "-L", PKG, "-ldadattn", "-Wl,-rpath,$ORIGIN"], check=True)
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, ptxas="--ptxas" in sys.argv)
    print(LIB)
