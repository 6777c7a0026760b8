"""Build recipe for the test oracle (TEST INFRASTRUCTURE, never part of the product).

* ``build_oracle()``  compiles ``oracle/attn_oracle.c`` (this repository's own C
  restatement of the reference arithmetic) into ``oracle/liboracle.so``.
* ``build_ref()``     compiles the reference project's own, unmodified CUDA
  kernels from where they lie in the reference checkout into cubins under
  ``oracle/_ref/`` (outputs only; no reference source is copied).  Those cubins
  are launched by the GPU tests to pin the oracle against the real reference
  kernels.  Skipped silently when the reference checkout is absent.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_DIR = os.path.join(HERE, "_ref")

# kernels of the reference that lie on the attention path
REF_SOURCES = {
    "attention_flash": "02-flash-attention/kernels/attention_flash.cu",
    "attention_bwd": "02-flash-attention/kernels/attention_bwd.cu",
    "attention_naive": "02-flash-attention/kernels/attention_naive.cu",
    "llm": "03-llm-engine/kernels/llm.cu",
}


def _newer(dst: str, *srcs: str) -> bool:
    if not os.path.exists(dst):
        return False
    t = os.path.getmtime(dst)
    return all(os.path.getmtime(s) <= t for s in srcs)


def build_oracle(force: bool = False) -> str:
    src = os.path.join(HERE, "attn_oracle.c")
    if not force and _newer(ORACLE_SO, src):
        return ORACLE_SO
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        raise RuntimeError("no C compiler found to build the oracle")
    cmd = [cc, "-O2", "-ffp-contract=off", "-fno-fast-math", "-fopenmp", "-shared", "-fPIC",
           "-o", ORACLE_SO, src, "-lm"]
    subprocess.run(cmd, check=True)
    return ORACLE_SO


def build_ref(reference_root: str | None = None, force: bool = False) -> list[str]:
    """Compile the reference's attention-path kernels to sm_100a cubins in oracle/_ref."""
    # where the reference checkout lies: the argument, $MX230_REFERENCE, else a `reference` directory beside this repository
    root = reference_root or os.environ.get("MX230_REFERENCE") or os.path.join(
        os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")
    if not os.path.isdir(root):
        return []
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        return []
    os.makedirs(REF_DIR, exist_ok=True)
    outs = []
    for name, rel in REF_SOURCES.items():
        src = os.path.join(root, rel)
        dst = os.path.join(REF_DIR, name + ".cubin")
        if not os.path.exists(src):
            continue
        if force or not _newer(dst, src):
            # same flags as the reference's build (kernel-build/src/lib.rs:95:
            # -O3 -lineinfo, no fast-math), retargeted from sm_61 PTX to an sm_100a cubin
            cmd = [nvcc, "-cubin", "-O3", "-lineinfo", "-w",
                   "-gencode", "arch=compute_100a,code=sm_100a", "-o", dst, src]
            subprocess.run(cmd, check=True)
        outs.append(dst)
    return outs


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    for p in build_ref(force="--force" in sys.argv):
        print(p)
