"""In-tree build of the C-ABI shared library (``lmserve_b200/liblmserve_kv.so``).

nvcc compiles the ``csrc/*.cu`` files for sm_100a only; the result links the
static CUDA runtime and nothing else, so it can be loaded with ``ctypes`` (or
bound from cgo / JNI / FFI) without PyTorch.

``build_packer()`` compiles the small CPython extension ``_packer`` (``csrc/packer.c``, gcc)
that packs a step's request list for ``lms_build_step_indices``; it is host code only.

Run ``python -m lmserve_b200.build`` to (re)build both; ``build_library()`` and
``build_packer()`` are what ``__graft_entry__.build()`` calls.
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


PACKER_SRC = CSRC / "packer.c"
PACKER_PATH = PKG_DIR / "_packer.so"


def build_packer(force: bool = False) -> Path:
    """Compiles ``lmserve_b200/_packer.so`` (CPython C API, no CUDA) if it is missing or stale."""
    import sysconfig
    if (not force and PACKER_PATH.exists()
            and PACKER_PATH.stat().st_mtime >= max(PACKER_SRC.stat().st_mtime, Path(__file__).stat().st_mtime)):
        return PACKER_PATH
    cc = os.environ.get("CC") or shutil.which("gcc") or shutil.which("cc")
    if not cc:
        raise RuntimeError("no C compiler found for the request packer; set CC")
    tmp = PACKER_PATH.with_suffix(".so.tmp")
    cmd = [cc, "-O2", "-fPIC", "-shared", "-Wall", "-I", sysconfig.get_paths()["include"],
           str(PACKER_SRC), "-o", str(tmp)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"compiling the request packer failed:\n{res.stdout}\n{res.stderr}")
    os.replace(tmp, PACKER_PATH)
    return PACKER_PATH


if __name__ == "__main__":
    path = build_library(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
    print(build_packer(force="--force" in sys.argv))
