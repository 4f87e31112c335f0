"""In-tree build of the C-ABI shared library (``lmserve_b200/liblmserve_kv.so``).

nvcc compiles the ``csrc/*.cu`` files for sm_100a only; the result links the
static CUDA runtime and nothing else, so it can be loaded with ``ctypes`` (or
bound from cgo / JNI / FFI) without PyTorch.

Run ``python -m lmserve_b200.build`` to (re)build; ``build_library()`` is what
``__graft_entry__.build()`` calls.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_NAME = "liblmserve_kv.so"
LIB_PATH = PKG_DIR / LIB_NAME
SOURCES = ["capi.cu", "write_rows.cu", "chunk_copy.cu", "rope_cache.cu", "step_indices.cu"]
HEADERS = ["kv_common.cuh", "kernels.cuh"]
PUBLIC_HEADER = PKG_DIR.parent / "include" / "lmserve_kv.h"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall",
    "-Xptxas", "-v",
    "--cudart", "static",
]


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def is_stale() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    deps = [CSRC / s for s in SOURCES + HEADERS] + [PUBLIC_HEADER, Path(__file__)]
    return any(d.stat().st_mtime > built for d in deps)


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compiles the library if any source is newer than it; returns its path."""
    if not force and not is_stale():
        return LIB_PATH
    nvcc = find_nvcc()
    objs = []
    log = []
    for src in SOURCES:
        obj = CSRC / (Path(src).stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(CSRC / src), "-o", str(obj)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        log.append(res.stdout + res.stderr)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{res.stdout}\n{res.stderr}")
        objs.append(str(obj))
    tmp = LIB_PATH.with_suffix(".so.tmp")
    cmd = [nvcc, "-shared", "--cudart", "static", "-o", str(tmp), *objs,
           "-Xlinker", "--exclude-libs,ALL"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    os.replace(tmp, LIB_PATH)
    (PKG_DIR / "ptxas_info.txt").write_text("\n".join(log))
    if verbose:
        sys.stderr.write("\n".join(log))
    return LIB_PATH


if __name__ == "__main__":
    path = build_library(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
