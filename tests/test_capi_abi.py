"""CPU: the shared library loads, exports every symbol the public header declares, and
rejects bad arguments before touching CUDA (no compute calls are made here)."""
import ctypes
import re
from pathlib import Path

import pytest

from lmserve_b200 import _lib

INCLUDE = Path(__file__).resolve().parent.parent / "include"
HEADER = INCLUDE / "lmserve_kv.h"              # the drop-in boundary
BENCH_HEADER = INCLUDE / "lmserve_kv_bench.h"  # measurement / test instruments


def declared_functions(headers=(HEADER, BENCH_HEADER)):
    names = set()
    for h in headers:
        text = re.sub(r"/\*.*?\*/", "", h.read_text(), flags=re.S)
        names |= set(re.findall(r"\b(lms_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_the_product_header_carries_no_bench_hooks():
    product = declared_functions((HEADER,))
    for hook in ("lms_set_tuning", "lms_launch_count", "lms_memcpy_async", "lms_selftest_bounded_wait"):
        assert hook not in product
    assert "LMS_TUNE_" not in re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)


def test_header_declares_the_path():
    names = declared_functions()
    for required in ("lms_reshape_and_cache", "lms_reshape_and_cache_layers", "lms_copy_blocks",
                     "lms_swap_blocks", "lms_transfer_blocks", "lms_strerror", "lms_version"):
        assert required in names


def test_every_declared_symbol_is_exported_and_bound():
    handle = ctypes.CDLL(str(_lib.LIB_PATH))
    names = declared_functions()
    for name in names:
        assert hasattr(handle, name), f"{name} declared in the header but not exported"
    assert set(names) == set(_lib.SIGNATURES), "ctypes table and header disagree"


def test_version_and_strerror():
    L = _lib.lib()
    assert L.lms_version() == 200
    assert L.lms_strerror(0) == b"ok"
    for code in range(-7, 0):
        assert L.lms_strerror(code) not in (b"", b"unknown status")
    assert L.lms_strerror(-99) == b"unknown status"


def test_tuning_roundtrip_and_range():
    L = _lib.lib()
    assert L.lms_set_tuning(_lib.TUNE_WRITE_VARIANT, 2) == 0
    assert L.lms_get_tuning(_lib.TUNE_WRITE_VARIANT) == 2
    assert L.lms_set_tuning(_lib.TUNE_WRITE_VARIANT, -1) == 0
    assert L.lms_get_tuning(_lib.TUNE_WRITE_VARIANT) == -1
    assert L.lms_set_tuning(_lib.TUNE_WRITE_VARIANT, 8) == _lib.LMS_ERR_RANGE
    assert L.lms_set_tuning(_lib.TUNE_COPY_VARIANT, 5) == _lib.LMS_ERR_RANGE
    assert L.lms_set_tuning(0, 1) == _lib.LMS_ERR_RANGE
    assert L.lms_set_tuning(99, 1) == _lib.LMS_ERR_RANGE
    assert L.lms_set_tuning(_lib.TUNE_SWAP_OUT_CTAS, 64) == 0
    assert L.lms_get_tuning(_lib.TUNE_SWAP_OUT_CTAS) == 64
    assert L.lms_set_tuning(_lib.TUNE_SWAP_OUT_CTAS, 0) == 0


A = 0x10000  # a 16-byte aligned fake address; never dereferenced by the checks below


def write_args(**kw):
    d = dict(key=A, value=A, kt=1024, vt=1024, kc=A, vc=A, bs_stride=32768, slot_stride=1024,
             slots=A, T=4, row=1024, bs=16, ns=0, stream=None)
    d.update(kw)
    return (d["key"], d["value"], d["kt"], d["vt"], d["kc"], d["vc"], d["bs_stride"],
            d["slot_stride"], d["slots"], d["T"], d["row"], d["bs"], d["ns"], d["stream"])


def test_reshape_and_cache_argument_errors():
    f = _lib.lib().lms_reshape_and_cache
    assert f(*write_args(T=0)) == _lib.LMS_OK          # empty input: nothing to do
    assert f(*write_args(T=-1)) == _lib.LMS_ERR_RANGE
    assert f(*write_args(row=0)) == _lib.LMS_ERR_RANGE
    assert f(*write_args(bs=0)) == _lib.LMS_ERR_RANGE
    assert f(*write_args(key=None)) == _lib.LMS_ERR_NULL
    assert f(*write_args(slots=None)) == _lib.LMS_ERR_NULL
    assert f(*write_args(key=A + 8)) == _lib.LMS_ERR_ALIGN
    assert f(*write_args(row=1000)) == _lib.LMS_ERR_ALIGN
    assert f(*write_args(kt=1028)) == _lib.LMS_ERR_ALIGN
    assert f(*write_args(slots=A + 4)) == _lib.LMS_ERR_ALIGN


def test_copy_swap_transfer_argument_errors():
    L = _lib.lib()
    cb = L.lms_copy_blocks
    assert cb(A, 1 << 20, 4096, 4096, 2, A, 0, 0, None) == _lib.LMS_OK
    assert cb(A, 1 << 20, 4096, 4096, 2, A, -1, 0, None) == _lib.LMS_ERR_RANGE
    assert cb(None, 1 << 20, 4096, 4096, 2, A, 3, 0, None) == _lib.LMS_ERR_NULL
    assert cb(A, 1 << 20, 4096, 4100, 2, A, 3, 0, None) == _lib.LMS_ERR_ALIGN
    assert cb(A, 1 << 20, 4096, 4096, 2, A + 8, 3, 0, None) == _lib.LMS_ERR_ALIGN
    sw = L.lms_swap_blocks
    assert sw(7, A, 1 << 20, 4096, A, 8192, 4096, 4096, 0, 2, A, 1, 0, 0, None) == _lib.LMS_ERR_RANGE
    assert sw(0, A, 1 << 20, 4096, A, 8192, 4096, 4096, 2, 1, A, 1, 0, 0, None) == _lib.LMS_ERR_RANGE
    assert sw(0, A, 1 << 20, 4096, A, 8192, 4096, 4096, 1, 1, A, 1, 0, 0, None) == _lib.LMS_OK
    assert sw(1, A, 1 << 20, 4096, None, 8192, 4096, 4096, 0, 2, A, 1, 0, 0, None) == _lib.LMS_ERR_NULL
    tr = L.lms_transfer_blocks
    assert tr(A, 1 << 20, 4096, A, 1 << 20, 4096, 4096, 2, A, 0, 0, 0, None) == _lib.LMS_OK
    assert tr(A, 1 << 20, 4096, None, 1 << 20, 4096, 4096, 2, A, 1, 0, 0, None) == _lib.LMS_ERR_NULL
    assert tr(A, 1 << 20, 4096, A, 1 << 20, 4090, 4096, 2, A, 1, 0, 0, None) == _lib.LMS_ERR_ALIGN


def test_check_raises_with_message():
    with pytest.raises(_lib.LmsError) as e:
        _lib.check(_lib.LMS_ERR_ALIGN)
    assert e.value.status == _lib.LMS_ERR_ALIGN and "16" in str(e.value)


def test_launch_count_is_zero_without_launches():
    assert _lib.lib().lms_launch_count() >= 0


def test_write_plan_and_paged_argument_errors():
    L = _lib.lib()
    h = ctypes.c_void_p()
    mk = lambda **kw: L.lms_write_plan_create(
        kw.get("key", A), A, 1024, 1024, 0, 0, A, A, 0, 32768, kw.get("slot_stride", 1024),
        kw.get("slots", A), 0, kw.get("T", 4), 1, kw.get("row", 1024), 16, 0,
        ctypes.byref(h) if kw.get("out", True) else None)
    assert mk(out=False) == _lib.LMS_ERR_NULL
    assert mk(key=None) == _lib.LMS_ERR_NULL and not h.value
    assert mk(row=1000) == _lib.LMS_ERR_ALIGN
    assert mk(T=-1) == _lib.LMS_ERR_RANGE
    assert L.lms_write_plan_run(None, None) == _lib.LMS_ERR_NULL
    assert L.lms_write_plan_destroy(None) == _lib.LMS_OK
    f = L.lms_append_paged_kv_cache
    paged = lambda **kw: f(A, A, 1024, 1024, 0, 0, kw.get("bi", A), A, A, A, 0, 32768, 1024,
                           kw.get("ind", A), A, kw.get("T", 4), 1, 1024, 16, kw.get("nb", 8), None)
    assert paged(T=0) == _lib.LMS_OK
    assert paged(bi=None) == _lib.LMS_ERR_NULL
    assert paged(ind=A + 2) == _lib.LMS_ERR_ALIGN
    assert paged(nb=-1) == _lib.LMS_ERR_RANGE
    assert L.lms_copy_blocks_host_static(A, 1 << 20, 4096, 4096, 2, A,
                                         _lib.LMS_STATIC_MAX_PAIRS + 1, None) == _lib.LMS_ERR_TOO_LARGE
