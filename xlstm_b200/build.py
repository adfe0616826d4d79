"""Ahead-of-time build of the C-ABI shared library (in-tree, sm_100a only).

    python -m xlstm_b200.build            # -> xlstm_b200/libxlstm_b200.so

nvcc cross-compiles for sm_100a without a GPU.  The library has no link-time
dependency on libcuda (the one driver entry point it needs, the tensor-map
encoder, is looked up at run time) and links the CUDA runtime statically, so
it loads on a machine without a driver; only launching needs a B200.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libxlstm_b200.so")
SOURCES = ["capi.cu", "mlstm_step.cu", "mlstm_recurrent.cu", "mlstm_chunkwise.cu", "slstm_fwd.cu", "slstm_bwd.cu", "layer_adjacent.cu", "greedy_head.cu", "peer_reduce.cu", "headwise_proj.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; set CUDA_HOME")
    return cand


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(HERE, "..", "include", "xlstm_b200.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return LIB
    cmd = [_nvcc(), *NVCC_FLAGS, "-o", LIB] + [os.path.join(CSRC, s) for s in SOURCES]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
