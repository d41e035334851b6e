"""Builds liblokal_cuda.so in-tree with nvcc for sm_100a.

The library holds hand-written CUDA only (no Triton, no CUTLASS). Flags that
matter for parity with the reference's CPU arithmetic: -fmad=false keeps every
multiply and add separately rounded; no fast-math, so sqrt, division, expf and
sincosf are the accurate versions.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
SO = os.path.join(HERE, "liblokal_cuda.so")
SOURCES = ["api.cu", "norm.cu", "rope.cu", "swiglu.cu", "gather.cu", "pass.cu", "kvstage.cu", "deltanet_rows.cu", "deltanet_tokens.cu", "gguf_file.cu"]
HEADERS = [os.path.join(CSRC, "common.cuh"), os.path.join(HERE, "..", "include", "lokal_cuda.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-fmad=false",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--shared",
    "--threads", "0",  # the sources compile in parallel
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: liblokal_cuda.so cannot be built")


def needs_build() -> bool:
    if not os.path.exists(SO):
        return True
    t = os.path.getmtime(SO)
    deps = [os.path.join(CSRC, s) for s in SOURCES] + HEADERS + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return SO
    extra = os.environ.get("LOKAL_B200_NVCC_EXTRA", "").split()  # e.g. -DLOKAL_ROPE_MIN_CTAS=3 for experiments
    tmp = SO + ".partial"  # the library appears under its name only when it is complete
    cmd = [_nvcc()] + NVCC_FLAGS + extra + (["-Xptxas", "-v"] if verbose else []) + \
          [os.path.join(CSRC, s) for s in SOURCES] + ["-o", tmp]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose:
        sys.stderr.write(res.stderr)
    if res.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    os.replace(tmp, SO)
    return SO


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
