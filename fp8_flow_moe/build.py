"""Build this package's own sm_100a kernels into ``fp8_flow_moe/lib/libfp8flow.so`` (``python -m fp8_flow_moe.build``).

The sources under ``csrc/`` (block quantisers, scaling-aware transpose, SwiGLU + quantise, row permutation) need
nothing outside this directory. nvcc cross-compiles without a GPU. Inside the training framework's repository the
same sources are also linked into its one library, which ``_native.py`` prefers when it is there.
"""
from __future__ import annotations

import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC, LIB = PKG / "csrc", PKG / "lib" / "libfp8flow.so"
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
         "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr", "-shared"]


def build_extension(force: bool = False) -> Path:
    nvcc = shutil.which("nvcc") or ("/usr/local/cuda/bin/nvcc" if Path("/usr/local/cuda/bin/nvcc").exists() else None)
    if nvcc is None:
        raise RuntimeError("nvcc not found: cannot build the fp8_flow_moe kernels")
    srcs = sorted(CSRC.glob("*.cu"))
    newest = max(p.stat().st_mtime for p in [*srcs, *CSRC.glob("*.cuh")])
    if not force and LIB.exists() and LIB.stat().st_mtime >= newest:
        return LIB
    LIB.parent.mkdir(parents=True, exist_ok=True)
    proc = subprocess.run([nvcc, *FLAGS, "-I", str(CSRC), *map(str, srcs), "-o", str(LIB), "-lcudart_static", "-ldl",
                           "-lrt", "-lpthread"], capture_output=True, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError("nvcc failed on the fp8_flow_moe kernels")
    return LIB


if __name__ == "__main__":
    print(build_extension(force="--force" in sys.argv))
