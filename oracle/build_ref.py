"""Builds the reference's own CUDA kernels of this path into ``oracle/_ref/libref.so`` (TEST
INFRASTRUCTURE: a GPU-side witness for the parity tests and a timing baseline; nothing in the
product loads it).

    python oracle/build_ref.py --reference /path/to/Loquetier [--force]

Sources are compiled from where they lie in the reference checkout - nothing is copied:
``kernel_src/csrc/smlm_forward/smlm_forward_cutlass.cu`` (a CUTLASS grouped GEMM) and
``kernel_src/csrc/rms_norm/rms_norm_cutlass.cu``, with the reference's vendored
``third_party/flashinfer/include`` for ``flashinfer/utils.cuh``.  The reference's CUTLASS submodule
is empty in a plain checkout (``.gitmodules:1-3``), so the CUTLASS headers come from this image (the
copy shipped inside the flashinfer Python package, or ``$CUTLASS_INCLUDE``).  ``oracle/ref_shim.cu``
adds ``extern "C"`` doorways with the dispatch logic of ``kernel_src/csrc/loquetier_ops.cc``;
``oracle/ref_shim_prefill.cu`` does the same for the prefill attention template and is compiled to
compute_80 PTX (its header explains why).
The output directory is git-ignored; the built library travels to the GPU box with the tree."""
from __future__ import annotations

import argparse
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
LIB = os.path.join(OUT_DIR, "libref.so")
REF_SOURCES = ["kernel_src/csrc/smlm_forward/smlm_forward_cutlass.cu", "kernel_src/csrc/rms_norm/rms_norm_cutlass.cu"]


def find_cutlass():
    env = os.environ.get("CUTLASS_INCLUDE")
    if env and os.path.exists(os.path.join(env, "cutlass", "cutlass.h")):
        return env
    for sp in sys.path:
        for cand in glob.glob(os.path.join(sp, "flashinfer", "data", "cutlass", "include")):
            if os.path.exists(os.path.join(cand, "cutlass", "cutlass.h")):
                return cand
    return None


def build(reference: str, force: bool = False, verbose: bool = False) -> str:
    srcs = [os.path.join(reference, s) for s in REF_SOURCES]
    for s in srcs:
        if not os.path.exists(s):
            raise FileNotFoundError(s)
    shim = os.path.join(HERE, "ref_shim.cu")
    shim_prefill = os.path.join(HERE, "ref_shim_prefill.cu")
    if not force and os.path.exists(LIB) and all(os.path.getmtime(LIB) >= os.path.getmtime(f)
                                                   for f in srcs + [shim, shim_prefill]):
        return LIB
    cutlass = find_cutlass()
    if cutlass is None:
        raise RuntimeError("no CUTLASS headers found (set CUTLASS_INCLUDE)")
    os.makedirs(OUT_DIR, exist_ok=True)
    nvcc = os.environ.get("NVCC", "nvcc")
    common = ["-O3", "-std=c++17", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-w",
              # the vendored flashinfer headers use uint32_t without including <cstdint>; newer compilers
              # no longer get it transitively, so it is pre-included instead of touching the sources
              "--pre-include", "cstdint",
              "-I", os.path.join(reference, "kernel_src", "csrc"),
              "-I", os.path.join(reference, "kernel_src", "third_party", "flashinfer", "include"),
              "-I", cutlass]
    # the prefill kernel only compiles for architectures below sm_90 (see ref_shim_prefill.cu): PTX for
    # compute_80, translated by the driver when the library is loaded on the GPU
    prefill_obj = os.path.join(OUT_DIR, "ref_shim_prefill.o")
    res = subprocess.run([nvcc, "-gencode", "arch=compute_80,code=compute_80", "-c", "-o", prefill_obj, shim_prefill]
                         + common, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building " + prefill_obj)
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", LIB] + common + srcs + [shim, prefill_obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building " + LIB)
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("LOQUETIER_REFERENCE"))
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    if not a.reference:
        sys.exit("give --reference or set LOQUETIER_REFERENCE")
    print(build(a.reference, force=a.force, verbose=True))
