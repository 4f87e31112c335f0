"""The public header is plain C99 and the library is usable from C without Python or PyTorch."""
import shutil
import subprocess
from pathlib import Path

import pytest

from lmserve_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent
DEMO = ROOT / "tests" / "c_abi" / "demo.c"
CUDA_HOME = Path(shutil.which("nvcc")).resolve().parent.parent if shutil.which("nvcc") else Path("/usr/local/cuda")


def compile_args(out: Path, link: bool):
    args = ["gcc", "-std=c99", "-Wall", "-Wextra", "-Werror", "-pedantic", f"-I{ROOT / 'include'}",
            "-isystem", str(CUDA_HOME / "include"), str(DEMO)]
    if not link:
        return args + ["-c", "-o", str(out)]
    return args + ["-o", str(out), str(_lib.LIB_PATH), f"-L{CUDA_HOME / 'lib64'}", "-lcudart",
                   f"-Wl,-rpath,{_lib.LIB_PATH.parent}", f"-Wl,-rpath,{CUDA_HOME / 'lib64'}"]


@pytest.mark.skipif(shutil.which("gcc") is None, reason="gcc not available")
def test_header_and_demo_compile_as_c99(tmp_path):
    # the header alone, with nothing else in scope, as strict C99 and as C++
    (tmp_path / "only_header.c").write_text('#include "lmserve_kv.h"\nint main(void) { return LMS_OK; }\n')
    for compiler, std in (("gcc", "-std=c99"), ("g++", "-std=c++11")):
        res = subprocess.run([compiler, std, "-Wall", "-Wextra", "-Werror", "-pedantic", "-x",
                              "c" if compiler == "gcc" else "c++", f"-I{ROOT / 'include'}", "-c",
                              str(tmp_path / "only_header.c"), "-o", str(tmp_path / "h.o")],
                             capture_output=True, text=True)
        assert res.returncode == 0, res.stderr
    res = subprocess.run(compile_args(tmp_path / "demo.o", link=False), capture_output=True, text=True)
    assert res.returncode == 0, res.stderr


@pytest.mark.gpu
@pytest.mark.skipif(shutil.which("gcc") is None, reason="gcc not available")
def test_library_runs_from_plain_c(tmp_path):
    exe = tmp_path / "demo"
    res = subprocess.run(compile_args(exe, link=True), capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert run.returncode == 0, run.stdout + run.stderr
    assert "c abi demo: ok, 3 launches" in run.stdout
