"""In-tree build of the CUDA library: nvcc -> mx230_b200/libmx230_attn.so (sm_100a only).

Replaces the reference's kernel-build crate (kernel-build/src/lib.rs:14-115), which
compiles every kernels/*.cu to sm_61 PTX from build.rs: same nvcc discovery order
(CUDA_HOME, /opt/cuda*, /usr/local/cuda, PATH), but the output is one shared library
holding sm_100a machine code behind the C ABI of include/mx230_attn.h.
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
LIB = os.path.join(PKG, "libmx230_attn.so")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def find_nvcc() -> str | None:
    cands = []
    if os.environ.get("CUDA_HOME"):
        cands.append(os.path.join(os.environ["CUDA_HOME"], "bin", "nvcc"))
    cands += sorted(glob.glob("/opt/cuda*/bin/nvcc")) + ["/usr/local/cuda/bin/nvcc"]
    for c in cands:
        if os.path.exists(c):
            return c
    return shutil.which("nvcc")


def sources() -> list[str]:
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + \
        glob.glob(os.path.join(ROOT, "include", "*.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every .cu under csrc/ for sm_100a and link the shared library."""
    if not force and not _stale():
        return LIB
    nvcc = find_nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found (set CUDA_HOME); cannot build libmx230_attn.so")
    objdir = os.path.join(PKG, "build")
    os.makedirs(objdir, exist_ok=True)
    common = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-I", os.path.join(ROOT, "include")]
    if verbose:
        common += ["-Xptxas", "-v"]
    objs, procs = [], []
    for src in sources():
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        cmd = [nvcc, *ARCH_FLAGS, *common, "-c", src, "-o", obj]
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
    for cmd, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stderr.write(out.decode())
        if p.returncode != 0:
            raise RuntimeError("nvcc failed: " + " ".join(cmd))
    link = [nvcc, *ARCH_FLAGS, "-shared", "-cudart", "static", "-o", LIB, *objs]
    subprocess.run(link, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
