"""Build the sm_100a CUDA library in-tree (``nanopysche_b200/lib/libnpb200.so``).

Every ``csrc/*.cu`` file is compiled with nvcc for ``compute_100a/sm_100a`` (relocatable device
code, one object per file, in parallel) and linked into one shared library that ``ops/_lib.py``
loads through ctypes. nvcc cross-compiles without a GPU, so this also works on a CPU-only box.

Run ``python -m nanopysche_b200.build`` (``--force`` to rebuild everything, ``-v`` for ptxas
resource usage).
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_DIR = PKG_DIR / "lib"
OBJ_DIR = LIB_DIR / "obj"
LIB_PATH = LIB_DIR / "libnpb200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "-rdc=true",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def find_nvcc() -> str | None:
    cand = shutil.which("nvcc")
    if cand:
        return cand
    for root in (os.environ.get("CUDA_HOME"), "/usr/local/cuda"):
        if root and os.path.exists(os.path.join(root, "bin", "nvcc")):
            return os.path.join(root, "bin", "nvcc")
    return None


FP8_CSRC = PKG_DIR.parent / "fp8_flow_moe" / "csrc"   # the stand-alone fp8_flow_moe package's kernels, linked in too


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu")) + (sorted(FP8_CSRC.glob("*.cu")) if FP8_CSRC.is_dir() else [])


def _newest_header_mtime() -> float:
    hs = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + (list(FP8_CSRC.glob("*.cuh")) if FP8_CSRC.is_dir() else [])
    return max((h.stat().st_mtime for h in hs), default=0.0)


def _compile_one(nvcc: str, src: Path, obj: Path, verbose: bool) -> tuple[str, int, str]:
    extra = os.environ.get("NPB200_NVCC_EXTRA", "").split()   # e.g. -DNP_ATTN_PROF for a development build
    cmd = [nvcc, *NVCC_FLAGS, *extra, "-I", str(src.parent), "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    return src.name, proc.returncode, proc.stdout + proc.stderr


def build_extension(force: bool = False, verbose: bool = False) -> Path:
    """Compile (if stale) and return the path of the shared library."""
    nvcc = find_nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found: cannot build the sm_100a kernels")
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    hdr_m = _newest_header_mtime()
    todo, objs = [], []
    for src in sources():
        obj = OBJ_DIR / (src.stem + ".o")
        objs.append(obj)
        stale = force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_m)
        if stale:
            todo.append((src, obj))
    if todo:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(todo))) as ex:
            futs = [ex.submit(_compile_one, nvcc, s, o, verbose) for s, o in todo]
            for f in futs:
                name, rc, out = f.result()
                if verbose or rc != 0:
                    sys.stderr.write(f"--- {name}\n{out}\n")
                if rc != 0:
                    raise RuntimeError(f"nvcc failed on {name}")
    need_link = force or bool(todo) or not LIB_PATH.exists() or any(
        o.stat().st_mtime > LIB_PATH.stat().st_mtime for o in objs
    )
    if need_link:
        tmp = LIB_PATH.with_suffix(".so.tmp")
        cmd = [nvcc, "-shared", "-rdc=true", "-gencode", "arch=compute_100a,code=sm_100a",
               "-Xcompiler", "-fPIC", "-o", str(tmp), *map(str, objs), "-lcudart_static", "-ldl", "-lrt",
               "-lpthread"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            sys.stderr.write(proc.stdout + proc.stderr)
            raise RuntimeError("link of libnpb200.so failed")
        os.replace(tmp, LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    p = build_extension(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(p)
