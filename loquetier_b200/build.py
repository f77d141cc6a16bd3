"""Builds the CUDA library of the SMLM path in-tree with nvcc, for sm_100a only.

    python -m loquetier_b200.build [--force] [--verbose]

The product is ``loquetier_b200/libsmlm_b200.so``: a plain C-ABI shared library
(declared in ``include/smlm_b200.h``) with no dependency on torch or Python."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libsmlm_b200.so")
SOURCES = [os.path.join(CSRC, "smlm_capi.cu")]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "-shared", "-Xptxas", "-v",
]


def _deps():
    out = list(SOURCES)
    for d in (CSRC, os.path.join(HERE, "..", "include")):
        for f in sorted(os.listdir(d)):
            if f.endswith((".cuh", ".h")):
                out.append(os.path.join(d, f))
    return out


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(f) > t for f in _deps())


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile if any source is newer than the library.  Returns the library path."""
    if not force and not needs_build():
        return LIB
    nvcc = os.environ.get("NVCC", "nvcc")
    cmd = [nvcc] + NVCC_FLAGS + ["-o", LIB] + SOURCES
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building " + LIB)
    with open(os.path.join(HERE, "ptxas_report.txt"), "w") as f:
        f.write(res.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
