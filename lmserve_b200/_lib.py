"""ctypes binding of ``liblmserve_kv.so`` (the C ABI in ``include/lmserve_kv.h``).

There is no fallback: if the shared library is missing or does not export a
symbol the header declares, importing this module's ``lib()`` raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_int, c_int32, c_int64, c_void_p, POINTER
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "liblmserve_kv.so"

LMS_OK = 0
LMS_ERR_NULL = -1
LMS_ERR_ALIGN = -2
LMS_ERR_RANGE = -3
LMS_ERR_CUDA = -4
LMS_ERR_INDEX = -5
LMS_ERR_PEER = -6
LMS_ERR_UNSUPPORTED = -7
LMS_ERR_TOO_LARGE = -8
LMS_STATIC_MAX_PAIRS = 16384
LMS_ROPE_CONTRACTED = 0
LMS_ROPE_ROUND_EACH = 1

LMS_SWAP_OUT = 0
LMS_SWAP_IN = 1

TUNE_WRITE_VARIANT = 1
TUNE_WRITE_TILE_BYTES = 2
TUNE_COPY_VARIANT = 3
TUNE_COPY_CTAS_PER_SM = 4
TUNE_SWAP_OUT_CTAS = 5
TUNE_SWAP_IN_CTAS = 6
TUNE_XFER_CTAS_PER_SM = 7
TUNE_XFER_VARIANT = 8
TUNE_WRITE_VPT = 9
TUNE_SWAP_VARIANT = 10
TUNE_WRITE_PDL = 11
TUNE_SWAP_ENGINE = 12
TUNE_WRITE_PREFETCH = 13
TUNE_STAGED_STREAMS = 14
TUNE_COUNT = 15

# name -> (restype, argtypes); one entry per declaration in include/lmserve_kv.h and
# include/lmserve_kv_bench.h
SIGNATURES = {
    "lms_version": (c_int, []),
    "lms_strerror": (c_char_p, [c_int]),
    "lms_last_cuda_error": (c_char_p, []),
    "lms_init_device": (c_int, []),
    "lms_set_tuning": (c_int, [c_int, c_int]),
    "lms_get_tuning": (c_int, [c_int]),
    "lms_set_debug_checks": (c_int, [c_int]),
    "lms_check_device_errors": (c_int, [c_void_p, POINTER(c_int64), POINTER(c_int64)]),
    "lms_error_record_async": (c_int, [c_void_p, c_void_p]),
    "lms_write_kernel_name": (c_char_p, [c_int64, c_int64]),
    "lms_reshape_and_cache": (c_int, [
        c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_int64, c_int64,
        c_void_p, c_int64, c_int64, c_int32, c_int64, c_void_p]),
    "lms_reshape_and_cache_layers": (c_int, [
        c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p, c_void_p,
        c_int64, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int32, c_int64,
        c_int32, c_int64, c_void_p]),
    "lms_write_plan_create": (c_int, [
        c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p, c_void_p,
        c_int64, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int32, c_int64,
        c_int32, c_int64, POINTER(c_void_p)]),
    "lms_write_plan_run": (c_int, [c_void_p, c_void_p]),
    "lms_write_plan_destroy": (c_int, [c_void_p]),
    "lms_append_paged_kv_cache": (c_int, [
        c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p, c_void_p,
        c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_int64,
        c_int32, c_int64, c_int32, c_int64, c_void_p]),
    "lms_paged_write_plan_create": (c_int, [
        c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p, c_void_p,
        c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_int64, c_int64,
        c_int32, c_int64, c_int32, c_int64, POINTER(c_void_p)]),
    "lms_rope_and_cache": (c_int, [
        c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int32, c_void_p,
        c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int64,
        c_void_p, c_int64, c_int32, c_int32, c_int32, c_int32, c_int32, c_int32, c_int64, c_int64,
        c_void_p]),
    "lms_build_step_indices": (c_int, [
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int64, c_int64,
        c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
        c_void_p, c_void_p, c_int32, c_int32, c_void_p, c_void_p]),
    "lms_copy_blocks": (c_int, [
        c_void_p, c_int64, c_int64, c_int64, c_int32, c_void_p, c_int64, c_int64, c_void_p]),
    "lms_swap_blocks": (c_int, [
        c_int, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64,
        c_int32, c_int32, c_void_p, c_int64, c_int64, c_int64, c_void_p]),
    "lms_transfer_blocks": (c_int, [
        c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64, c_int32,
        c_void_p, c_int64, c_int64, c_int64, c_void_p]),
    "lms_copy_blocks_host": (c_int, [
        c_void_p, c_int64, c_int64, c_int64, c_int32, c_void_p, c_int64, c_int64, c_void_p]),
    "lms_copy_blocks_host_static": (c_int, [
        c_void_p, c_int64, c_int64, c_int64, c_int32, c_void_p, c_int64, c_void_p]),
    "lms_swap_blocks_host": (c_int, [
        c_int, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64,
        c_int32, c_int32, c_void_p, c_int64, c_int64, c_int64, c_void_p]),
    "lms_swap_blocks_dma": (c_int, [
        c_int, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64,
        c_int32, c_int32, c_void_p, c_int64, c_int64, c_int64, c_void_p]),
    "lms_swap_blocks_staged": (c_int, [
        c_int, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64,
        c_int32, c_int32, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64, c_void_p]),
    "lms_transfer_blocks_host": (c_int, [
        c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64, c_int32,
        c_void_p, c_int64, c_int64, c_int64, c_void_p]),
    "lms_peer_enable": (c_int, [c_int]),
    "lms_host_alloc": (c_int, [c_int64, POINTER(c_void_p), POINTER(c_void_p)]),
    "lms_host_free": (c_int, [c_void_p]),
    "lms_host_register": (c_int, [c_void_p, c_int64, POINTER(c_void_p)]),
    "lms_host_unregister": (c_int, [c_void_p]),
    "lms_ipc_export": (c_int, [c_void_p, c_void_p, POINTER(c_int64)]),
    "lms_ipc_open": (c_int, [c_void_p, c_int64, POINTER(c_void_p)]),
    "lms_ipc_close": (c_int, [c_void_p, c_int64]),
    "lms_selftest_bounded_wait": (c_int, [c_int64, c_void_p]),
    "lms_memcpy_async": (c_int, [c_void_p, c_void_p, c_int64, c_void_p]),
    "lms_launch_count": (c_int64, []),
}

_lib = None


class LmsError(RuntimeError):
    """A C-ABI call returned a negative status."""

    def __init__(self, status: int, message: str):
        super().__init__(f"lmserve_kv status {status}: {message}")
        self.status = status


def lib() -> ctypes.CDLL:
    """Loads the shared library once and types every exported function."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m lmserve_b200.build` "
            "(nvcc, sm_100a). There is no CPU or PyTorch fallback for the cache ops.")
    handle = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(handle, name)  # AttributeError if the symbol is missing
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = handle
    return handle


def check(status: int) -> None:
    """Raises LmsError for a negative status."""
    if status == LMS_OK:
        return
    handle = lib()
    msg = handle.lms_strerror(status).decode()
    if status in (LMS_ERR_CUDA, LMS_ERR_UNSUPPORTED, LMS_ERR_INDEX):
        detail = handle.lms_last_cuda_error().decode()
        if detail:
            msg += ": " + detail
    raise LmsError(status, msg)
