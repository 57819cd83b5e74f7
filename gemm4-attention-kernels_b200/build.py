"""Build libsplitd_attn.so in-tree with nvcc for sm_100a.

    python gemm4-attention-kernels_b200/build.py [--verbose] [--profile]

--profile compiles the in-kernel cycle counters in (-DSPLITD_PROFILE; they are written to splitd_params::debug).

nvcc cross-compiles without a GPU. The shared object lands next to the sources
(csrc/libsplitd_attn.so) and is what splitd_flash_attn/_capi.py loads.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(CSRC, "libsplitd_attn.so")
SOURCES = ["capi.cu", "fwd_kernel.cu", "bwd_preprocess.cu", "bwd_pds2_kernel.cu", "bwd_grad_kernel.cu",
           "no_alloc.cu", "wait_probe.cu"]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found")
    return exe


def _stale() -> bool:
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh"))]
    deps.append(os.path.join(HERE, "..", "include", "splitd_attn.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, profile: bool = False) -> str:
    srcs = [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    if not force and not _stale():
        return OUT
    cmd = [
        _nvcc(),
        "-gencode",
        "arch=compute_100a,code=sm_100a",
        "-lineinfo",
        "-O3",
        "-std=c++17",
        "-shared",
        "-Xcompiler",
        "-fPIC",
        "-o",
        OUT,
    ]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    if profile:
        cmd += ["-DSPLITD_PROFILE=1"]
    cmd += srcs
    res = subprocess.run(cmd, cwd=CSRC, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed")
    return OUT


if __name__ == "__main__":
    print(build(force=True, verbose="--verbose" in sys.argv, profile="--profile" in sys.argv))
