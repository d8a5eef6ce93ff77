"""Build recipe of libsapphire_b200.so (nvcc, sm_100a only, in-tree).

    python -m sapphire_b200.build            # build if sources are newer
    python -m sapphire_b200.build --force

The library links the CUDA runtime statically and resolves the one driver
entry point it needs (cuTensorMapEncodeTiled) at run time, so it has no
link-time dependency on libcuda and cross-compiles on a machine without a GPU.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "libsapphire_b200.so")
SOURCES = ["abi.cu", "gemm_tcgen05.cu", "gemm_tcgen05_2cta.cu", "gemm_tcgen05_slices.cu", "gemm_simt.cu", "spgemm.cu", "csr_convert.cu", "elementwise.cu", "colsum_noalloc.cu", "im2col.cu", "dp_exchange.cu", "compat_c.cu"]
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC", "--use_fast_math=false"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise FileNotFoundError("nvcc not found")


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(PKG, "..", "include", "sapphire_b200.h"))
    for root, _, files in os.walk(os.path.join(PKG, "compat")):
        deps += [os.path.join(root, f) for f in files]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return LIB
    flags = [f for f in FLAGS if not f.startswith("--use_fast_math")]
    objs = []
    os.makedirs(os.path.join(PKG, "build"), exist_ok=True)
    procs = []
    for src in SOURCES:
        obj = os.path.join(PKG, "build", src.replace(".cu", ".o"))
        cmd = [_nvcc(), *flags, "-I", os.path.join(PKG, "compat"), "-c",
               os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
        objs.append(obj)
    for src, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode:
            sys.stderr.write(out.decode())
        if p.returncode:
            raise RuntimeError(f"nvcc failed on {src}")
    subprocess.run([_nvcc(), "-shared", "-o", LIB, *objs, "-cudart", "static",
                    "-gencode", "arch=compute_100a,code=sm_100a"], check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
