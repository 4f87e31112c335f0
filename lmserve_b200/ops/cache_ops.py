"""Paged KV-cache operators with LMServe's Python signatures, backed by the
sm_100a kernels behind the C ABI (``include/lmserve_kv.h``).

``copy_blocks`` and ``fill_key_cache`` keep the names, argument order and
in-place semantics of ``runtime/worker/llm_worker/ops/cache_ops.py:8-59`` in
LMServe.  ``reshape_and_cache`` is the same write addressed into the
interleaved per-layer cache ``[num_blocks, 2, block_size, H, D]`` that
``models/layers/attention.py:76-85`` fills through flashinfer;
``reshape_and_cache_layers`` does all layers in one launch.  ``swap_blocks`` and
``transfer_blocks`` carry the device work of ``kv_worker.py:197-227`` and
``kv_worker.py:358-415``.

Every operator runs on the current CUDA stream of the cache tensor's device and
returns without synchronising.  There is no CPU path: tensors that are not on a
CUDA device are rejected, and a missing shared library is an ImportError.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Iterable, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from .. import _lib

try:  # C helpers for walking Python containers (csrc/packer.c)
    from .. import _packer
except ImportError as e:  # a build without it would silently run the 4x slower Python loops
    raise ImportError("lmserve_b200/_packer.so is missing: build it with "
                      "`python -m lmserve_b200.build` (gcc, no CUDA needed)") from e

PairList = Union[Sequence[Tuple[int, int]], np.ndarray, torch.Tensor]


try:  # the raw handle of the current stream without building a Stream object
    _raw_stream = torch._C._cuda_getCurrentRawStream
except AttributeError:  # pragma: no cover - older / newer torch
    _raw_stream = None


# Host address of a registered host pool -> the address the GPU uses for the same memory
# (filled by kv_worker.HostPool; read by the torch custom op of swap_blocks).
HOST_POOL_DEVICE_PTR: Dict[int, int] = {}


def _stream_ptr(device: torch.device) -> int:
    if _raw_stream is not None:
        return _raw_stream(device.index if device.index is not None else torch.cuda.current_device())
    return torch.cuda.current_stream(device).cuda_stream


class _OnDevice:
    """``with torch.cuda.device(dev)`` that costs nothing when `dev` is already current."""

    __slots__ = ("_guard",)

    def __init__(self, device: torch.device):
        idx = device.index
        self._guard = None if idx is None or idx == torch.cuda.current_device() else torch.cuda.device(idx)

    def __enter__(self):
        if self._guard is not None:
            self._guard.__enter__()

    def __exit__(self, *exc):
        if self._guard is not None:
            self._guard.__exit__(*exc)


def _require_cuda(name: str, t: torch.Tensor) -> None:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor, got {type(t).__name__}")
    if not t.is_cuda:
        raise RuntimeError(
            f"{name} must live on a CUDA device (got {t.device}); the cache ops have no CPU path")


def _row_layout(name: str, t: torch.Tensor) -> Tuple[int, int]:
    """(token stride in bytes, row bytes) of a [T, H, D] tensor whose rows are dense."""
    if t.dim() != 3:
        raise ValueError(f"{name} must be [num_tokens, num_kv_heads, head_dim], got {tuple(t.shape)}")
    T, H, D = t.shape
    es = t.element_size()
    if T > 0 and (t.stride(2) != 1 or (H > 1 and t.stride(1) != D)):
        raise ValueError(f"{name}: each token's [H, D] row must be contiguous (strides {t.stride()})")
    return t.stride(0) * es, H * D * es


def _slots_i64(slot_mapping: torch.Tensor, device: torch.device) -> torch.Tensor:
    if slot_mapping.dtype in (torch.float16, torch.bfloat16, torch.float32, torch.float64, torch.bool):
        raise TypeError(f"slot_mapping must be an integer tensor, got {slot_mapping.dtype}")
    if slot_mapping.device != device or slot_mapping.dtype != torch.int64:
        slot_mapping = slot_mapping.to(device=device, dtype=torch.int64, non_blocking=True)
    return slot_mapping.contiguous()


def flatten_block_map(src_to_dst: Union[Dict[int, Iterable[int]], PairList]) -> np.ndarray:
    """``{src: [dst, ...]}`` or a sequence of ``(src, dst)`` -> int64 array [n, 2].

    The dict form is what ``copy_blocks`` receives in LMServe
    (``cache_ops.py:12-15``); the pair form is the shape of
    ``BlockMapping.entries`` (``proto/worker.proto:78-86``).
    """
    if isinstance(src_to_dst, dict):
        if _packer is not None:
            try:
                arr = np.empty((sum(map(len, src_to_dst.values())), 2), dtype=np.int64)
            except TypeError:      # destinations given as iterators: no length to size the table by
                arr = None
            if arr is not None:
                n = _packer.flatten_dict(src_to_dst, arr)
                return arr[:n]
        flat = [x for src, dsts in src_to_dst.items() for dst in dsts for x in (src, dst)]
        return np.array(flat, dtype=np.int64).reshape(-1, 2)
    if isinstance(src_to_dst, torch.Tensor):
        arr = src_to_dst.detach().cpu().numpy()
    else:
        arr = np.asarray(src_to_dst)
    if arr.size == 0:
        return np.empty((0, 2), dtype=np.int64)
    if arr.ndim != 2 or arr.shape[1] != 2:
        raise ValueError(f"block pairs must have shape [n, 2], got {arr.shape}")
    if not np.issubdtype(arr.dtype, np.integer):
        raise TypeError(f"block ids must be integers, got {arr.dtype}")
    return np.ascontiguousarray(arr, dtype=np.int64)


def _pairs_on_device(pairs, device: torch.device) -> torch.Tensor:
    """int64 [n, 2] on `device`; host tables go through pinned memory, asynchronously."""
    if isinstance(pairs, torch.Tensor) and pairs.is_cuda:
        if pairs.dim() != 2 or pairs.shape[1] != 2:
            raise ValueError(f"block pairs must have shape [n, 2], got {tuple(pairs.shape)}")
        pairs = pairs.to(device=device, dtype=torch.int64).contiguous()
        # the kernels read one (src, dst) couple per 16-byte load
        return pairs if pairs.data_ptr() % 16 == 0 else pairs.clone()
    arr = flatten_block_map(pairs)
    if arr.shape[0] == 0:
        return torch.empty((0, 2), dtype=torch.int64, device=device)
    host = torch.from_numpy(arr).pin_memory()
    return host.to(device, non_blocking=True)


def _pair_table(pairs, device: torch.device):
    """(on_device, keepalive, pointer, n): a device tensor is used in place; anything else is
    flattened on the host and handed to the ``*_host`` entry points, which upload it."""
    if isinstance(pairs, torch.Tensor) and pairs.is_cuda:
        t = _pairs_on_device(pairs, device)
        return True, t, t.data_ptr(), t.shape[0]
    arr = flatten_block_map(pairs)
    return False, arr, arr.ctypes.data, arr.shape[0]


# --------------------------------------------------------------------- writes
def fill_key_cache(
    key: torch.Tensor,
    value: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    slot_mapping: torch.Tensor,
) -> None:
    """``key_cache[slot_mapping[t]] = key[t]`` and the same for value, in place.

    Same contract as LMServe's ``fill_key_cache`` (``ops/cache_ops.py:39-59``,
    kernel ``ops/triton/cache_kernels.py:39-58``): ``key``/``value`` are
    ``[T, H, D]``, the two caches are contiguous and addressed as
    ``[num_slots, H, D]``.  One difference, by specification: an entry
    ``slot_mapping[t] < 0`` is padding and is skipped (the Triton kernel would
    write out of bounds for it).
    """
    for n, t in (("key", key), ("value", value), ("key_cache", key_cache), ("value_cache", value_cache)):
        _require_cuda(n, t)
    dev = key_cache.device
    k_tok, row_bytes = _row_layout("key", key)
    v_tok, v_row = _row_layout("value", value)
    if v_row != row_bytes or value.shape[0] != key.shape[0]:
        raise ValueError("key and value must have the same shape")
    if not (key_cache.is_contiguous() and value_cache.is_contiguous()):
        raise ValueError("key_cache and value_cache must be contiguous")
    if key.dtype != key_cache.dtype or value.dtype != value_cache.dtype:
        raise TypeError("cache dtype must match key/value dtype (bytes are copied, not converted)")
    if slot_mapping.numel() != key.shape[0]:
        raise ValueError("slot_mapping must have one entry per token")
    slots = _slots_i64(slot_mapping, dev)
    num_slots = key_cache.numel() * key_cache.element_size() // row_bytes
    with _OnDevice(dev):
        _lib.check(_lib.lib().lms_reshape_and_cache(
            key.data_ptr(), value.data_ptr(), k_tok, v_tok,
            key_cache.data_ptr(), value_cache.data_ptr(),
            row_bytes, row_bytes,  # block_stride with block_size 1: flat slots
            slots.data_ptr(), key.shape[0], row_bytes, 1, num_slots,
            _stream_ptr(dev)))


def reshape_and_cache(
    key: torch.Tensor,
    value: torch.Tensor,
    kv_cache: torch.Tensor,
    slot_mapping: torch.Tensor,
) -> None:
    """Writes ``key``/``value`` ``[T, H, D]`` into one layer's interleaved paged cache.

    ``kv_cache`` is ``kv_caches[layer]`` = ``[num_blocks, 2, block_size, H, D]``
    (``model_worker.py:221-228``); token ``t`` goes to block
    ``slot // block_size``, entry ``slot % block_size``, K in plane 0 and V in
    plane 1 — the addressing ``flashinfer.append_paged_kv_cache`` performs at
    ``models/layers/attention.py:76-85`` with
    ``slot = block_table[pos // block_size] * block_size + pos % block_size``.
    Entries ``< 0`` are skipped.
    """
    _write_layers(key, value, kv_cache, slot_mapping)


def reshape_and_cache_layers(
    key: torch.Tensor,
    value: torch.Tensor,
    kv_caches: torch.Tensor,
    slot_mapping: torch.Tensor,
) -> None:
    """All layers of one step in a single launch.

    ``key``/``value``: ``[L, T, H, D]``; ``kv_caches``: the whole
    ``[L, num_blocks, 2, block_size, H, D]`` tensor; ``slot_mapping``: ``[T]``
    (shared by every layer, as the block tables are in LMServe) or ``[L, T]``.
    """
    _write_layers(key, value, kv_caches, slot_mapping)


_plan_run_address = None


def _PLAN_RUN_ADDRESS() -> int:
    """Address of ``lms_write_plan_run`` in the loaded library (looked up once)."""
    global _plan_run_address
    if _plan_run_address is None:
        _plan_run_address = ctypes.cast(_lib.lib().lms_write_plan_run, ctypes.c_void_p).value
    return _plan_run_address


def _prepare_paged(append_key, append_value, batch_indices, positions, paged_kv_cache,
                   kv_indices, kv_indptr, kv_layout):
    """Validates a paged append and returns (device, argument tuple of
    ``lms_paged_write_plan_create`` without the plan pointer).  Attribute reads only."""
    if kv_layout != "NHD":
        raise ValueError("only the NHD layout (LMServe's) is supported")
    if type(paged_kv_cache) is torch.Tensor:
        cache = paged_kv_cache
        cshape = cache.shape
        if len(cshape) != 5 or cshape[1] != 2:
            raise ValueError("paged_kv_cache must be [num_pages, 2, page_size, H, D]")
        NB, _, BS, H, D = cshape
        cstride = cache.stride()
        es = cache.element_size()
        if cstride[4] != 1 or cstride[3] != D or cstride[2] != H * D or cstride[1] != BS * H * D:
            raise ValueError("each cache page must be contiguous")
        block_stride = cstride[0] * es
        kptr = cache.data_ptr()
        vptr = kptr + BS * H * D * es
    else:
        k_cache, v_cache = paged_kv_cache
        cache = k_cache
        cshape = k_cache.shape
        if len(cshape) != 4 or cshape != v_cache.shape or k_cache.stride() != v_cache.stride():
            raise ValueError("k_cache and v_cache must both be [num_pages, page_size, H, D]")
        NB, BS, H, D = cshape
        cstride = k_cache.stride()
        es = k_cache.element_size()
        if cstride[3] != 1 or cstride[2] != D or cstride[1] != H * D or not v_cache.is_cuda:
            raise ValueError("each cache page must be contiguous and on the GPU")
        if v_cache.dtype != k_cache.dtype:
            raise TypeError("k_cache and v_cache must have the same dtype")
        block_stride = cstride[0] * es
        kptr, vptr = k_cache.data_ptr(), v_cache.data_ptr()
    if not cache.is_cuda:
        raise RuntimeError(
            f"paged_kv_cache must live on a CUDA device (got {cache.device}); the cache ops have no CPU path")
    dev = cache.device
    kshape = append_key.shape
    if len(kshape) != 3 or kshape[1] != H or kshape[2] != D or append_value.shape != kshape:
        raise ValueError("append_key / append_value must be [T, H, D] matching the cache")
    T = kshape[0]
    ks, vs = append_key.stride(), append_value.stride()
    if ks[2] != 1 or vs[2] != 1 or (H > 1 and (ks[1] != D or vs[1] != D)):
        raise ValueError("each token's [H, D] row must be contiguous")
    cdtype = cache.dtype
    if append_key.dtype != cdtype or append_value.dtype != cdtype:
        raise TypeError("cache dtype must match key/value dtype (bytes are copied, not converted)")
    if append_key.device != dev or append_value.device != dev:
        raise RuntimeError("append_key / append_value must be on the cache's device; the cache ops have no CPU path")
    i32 = torch.int32
    for name, t in (("batch_indices", batch_indices), ("positions", positions),
                    ("kv_indices", kv_indices), ("kv_indptr", kv_indptr)):
        if t.dtype != i32:
            raise TypeError(f"{name} must be int32 (got {t.dtype})")
        if t.device != dev or not t.is_contiguous():
            raise ValueError(f"{name} must be a contiguous tensor on the cache's device")
    if batch_indices.numel() != T or positions.numel() != T:
        raise ValueError("batch_indices and positions need one entry per appended token")
    row_bytes = H * D * es
    num_requests = max(0, kv_indptr.numel() - 1)
    return dev, (append_key.data_ptr(), append_value.data_ptr(), ks[0] * es, vs[0] * es, 0, 0,
                 batch_indices.data_ptr(), positions.data_ptr(), kptr, vptr, 0, block_stride,
                 row_bytes, kv_indices.data_ptr(), kv_indptr.data_ptr(), num_requests, T, 1,
                 row_bytes, BS, NB)


class PagedWritePlan:
    """A paged append (``flashinfer.append_paged_kv_cache``'s arguments) validated and resolved
    once; ``run()`` is one C call.  LMServe's attention layer passes the same buffers every
    step (``models/layers/attention.py:76-85`` with the step tensors of
    ``model_worker.py:399-433``), so one plan per layer serves the whole decode loop.  The plan
    records addresses and geometry, not tensors: it must be rebuilt when a tensor is
    reallocated (``append_paged_kv_cache`` does that by itself)."""

    __slots__ = ("device", "_handle", "_fn", "_plan", "_destroy", "_index")

    def __init__(self, append_key, append_value, batch_indices, positions, paged_kv_cache,
                 kv_indices, kv_indptr, kv_last_page_len=None, kv_layout: str = "NHD"):
        self.device, args = _prepare_paged(append_key, append_value, batch_indices, positions,
                                           paged_kv_cache, kv_indices, kv_indptr, kv_layout)
        self._index = self.device.index
        handle = ctypes.c_void_p()
        L_ = _lib.lib()
        with torch.cuda.device(self.device):
            _lib.check(L_.lms_paged_write_plan_create(*args, ctypes.byref(handle)))
        self._handle = handle
        self._destroy = L_.lms_write_plan_destroy
        self._fn = _PLAN_RUN_ADDRESS()
        self._plan = handle.value or 0

    def run(self, stream: Optional[int] = None) -> None:
        """Enqueues the append on `stream` (a raw ``cudaStream_t`` value; default: the current
        stream of the plan's device, which must be the current device)."""
        if stream is None:
            stream = _raw_stream(self._index) if _raw_stream is not None else \
                torch.cuda.current_stream(self.device).cuda_stream
        rc = _packer.call_plan(self._fn, self._plan, stream)
        if rc:
            _lib.check(rc)

    def __del__(self):
        h = getattr(self, "_handle", None)
        if h:
            self._destroy(h)
            self._handle = None


_PAGED_PLANS: Dict[tuple, PagedWritePlan] = {}
_PAGED_PLANS_MAX = 2048
# the index tensors of the previous call and their part of the plan key, as ONE object so that
# two threads can never pair one call's tensors with another call's key
_INDEX_CACHE: tuple = ((None, None, None, None), ())


def append_paged_kv_cache(
    append_key: torch.Tensor,
    append_value: torch.Tensor,
    batch_indices: torch.Tensor,
    positions: torch.Tensor,
    paged_kv_cache,
    kv_indices: torch.Tensor,
    kv_indptr: torch.Tensor,
    kv_last_page_len: Optional[torch.Tensor] = None,
    kv_layout: str = "NHD",
) -> None:
    """Drop-in for ``flashinfer.append_paged_kv_cache`` as LMServe calls it
    (``models/layers/attention.py:76-85``): same argument order and meaning, same in-place
    result, so the call site changes only its import.

    ``append_key``/``append_value``: ``[T, H, D]``; ``batch_indices``/``positions``: int32
    ``[T]`` (request index and position of every appended token, as produced by
    ``flashinfer.get_batch_indices_positions`` at ``model_worker.py:425-433``);
    ``paged_kv_cache``: one layer's ``[num_pages, 2, page_size, H, D]`` tensor, or a
    ``(k_cache, v_cache)`` pair of ``[num_pages, page_size, H, D]`` tensors; ``kv_indices`` /
    ``kv_indptr``: int32 page table in CSR form.  ``kv_last_page_len`` is accepted and ignored
    (the write does not need it).  Only the ``"NHD"`` layout, the one LMServe uses.

    This runs once per layer per step with the same buffers, so the validated call is kept as
    a :class:`PagedWritePlan` keyed on everything the validation looked at (addresses, shapes,
    strides, dtypes); a repeat call is a dictionary lookup and one C call.  The four index
    tensors are recognised by object identity from one call to the next (they are the same
    objects for every layer of a step), so re-pointing one of them at other storage in place
    (``Tensor.set_``) between two calls goes unnoticed; refilling them with ``copy_`` is fine.
    """
    # Two-part key.  The four index tensors are the same Python objects for every layer of a
    # step (``input_params.*`` in LMServe), so their part of the key is recomputed only when
    # one of the objects changes; the per-layer part reads what differs from layer to layer.
    global _INDEX_CACHE
    last = _INDEX_CACHE          # one read: (objects, key) is replaced as a whole, never in parts
    seen = last[0]
    if (seen[0] is batch_indices and seen[1] is positions
            and seen[2] is kv_indices and seen[3] is kv_indptr):
        index_key = last[1]
    else:
        index_key = (batch_indices.data_ptr(), positions.data_ptr(), kv_indices.data_ptr(),
                     kv_indptr.data_ptr(), batch_indices.dtype, positions.dtype, kv_indices.dtype,
                     kv_indptr.dtype, batch_indices.shape, positions.shape, kv_indptr.shape,
                     batch_indices.is_contiguous(), positions.is_contiguous(),
                     kv_indices.is_contiguous(), kv_indptr.is_contiguous(),
                     batch_indices.device, positions.device, kv_indices.device, kv_indptr.device)
        _INDEX_CACHE = ((batch_indices, positions, kv_indices, kv_indptr), index_key)
    if type(paged_kv_cache) is torch.Tensor:
        c0 = paged_kv_cache
        cache_key = (c0.data_ptr(), c0.shape, c0.stride(), c0.dtype)
    else:
        c0, c1 = paged_kv_cache
        cache_key = (c0.data_ptr(), c0.shape, c0.stride(), c0.dtype,
                     c1.data_ptr(), c1.shape, c1.stride(), c1.dtype, c1.device)
    key = (index_key, cache_key, c0.device, append_key.data_ptr(), append_value.data_ptr(),
           append_key.shape, append_key.stride(), append_value.shape, append_value.stride(),
           append_key.dtype, append_value.dtype, kv_layout)
    plan = _PAGED_PLANS.get(key)
    if plan is None:
        if append_key.dim() == 3 and append_key.shape[0] == 0:
            _prepare_paged(append_key, append_value, batch_indices, positions, paged_kv_cache,
                           kv_indices, kv_indptr, kv_layout)
            return
        plan = PagedWritePlan(append_key, append_value, batch_indices, positions, paged_kv_cache,
                              kv_indices, kv_indptr, kv_last_page_len, kv_layout)
        if len(_PAGED_PLANS) >= _PAGED_PLANS_MAX:
            _PAGED_PLANS.clear()
        _PAGED_PLANS[key] = plan
    idx = plan._index
    if idx == torch.cuda.current_device():
        plan.run()
    else:
        with torch.cuda.device(idx):
            plan.run()


def _prepare_write(key, value, kv_caches, slot_mapping):
    """Validates a write and returns (device, keepalive, argument tuple without the stream) for
    ``lms_reshape_and_cache_layers``.  ``key``/``value`` ``[L, T, H, D]`` with the 6-D cache, or
    ``[T, H, D]`` with one layer's 5-D cache.  Runs once per layer per step when the caller
    does not plan: only attribute reads, no tensor indexing."""
    kshape, cshape = key.shape, kv_caches.shape
    layered = len(kshape) == 4
    if layered:
        if len(cshape) != 6 or cshape[2] != 2:
            raise ValueError("kv cache must be [L, num_blocks, 2, block_size, H, D]")
        L, NB, _, BS, H, D = cshape
        cst = kv_caches.stride()
        c_layer, c_block, c_in = cst[0], cst[1], cst[2:]
        if kshape[0] != L:
            raise ValueError(f"key {tuple(kshape)} does not match cache {tuple(cshape)}")
        kst, vst = key.stride(), value.stride()
        k_layer, v_layer, kst, vst = kst[0], vst[0], kst[1:], vst[1:]
        T = kshape[1]
        row_shape = kshape[2:]
    elif len(kshape) == 3:
        if len(cshape) != 5 or cshape[1] != 2:
            raise ValueError("a layer's kv cache must be [num_blocks, 2, block_size, H, D]")
        NB, _, BS, H, D = cshape
        L = 1
        cst = kv_caches.stride()
        c_layer, c_block, c_in = 0, cst[0], cst[1:]
        kst, vst = key.stride(), value.stride()
        k_layer = v_layer = 0
        T = kshape[0]
        row_shape = kshape[1:]
    else:
        raise ValueError("key and value must both be [L, T, H, D] (or [T, H, D] for one layer)")
    if value.shape != kshape:
        raise ValueError("key and value must have the same shape")
    if tuple(row_shape) != (H, D):
        raise ValueError(f"key {tuple(kshape)} does not match cache {tuple(cshape)}")
    if not kv_caches.is_cuda or not key.is_cuda or not value.is_cuda:
        raise RuntimeError("key, value and the cache must live on a CUDA device; the cache ops have no CPU path")
    cdtype = kv_caches.dtype
    if key.dtype != cdtype or value.dtype != cdtype:
        raise TypeError("cache dtype must match key/value dtype (bytes are copied, not converted)")
    if NB > 0 and tuple(c_in) != (BS * H * D, H * D, D, 1):
        raise ValueError("each cache block [2, block_size, H, D] must be contiguous")
    if T > 0 and (kst[2] != 1 or vst[2] != 1 or (H > 1 and (kst[1] != D or vst[1] != D))):
        raise ValueError("each token's [H, D] row must be contiguous")
    es = kv_caches.element_size()
    dev = kv_caches.device
    row_bytes = H * D * es
    slots = slot_mapping
    if slots.dtype != torch.int64 or slots.device != dev or not slots.is_contiguous():
        slots = _slots_i64(slot_mapping, dev)
    sshape = slots.shape
    if len(sshape) == 1 and sshape[0] == T:
        slot_layer = 0
    elif len(sshape) == 2 and tuple(sshape) == (L, T):
        slot_layer = T
    else:
        raise ValueError(f"slot_mapping must be [T] or [L, T], got {tuple(sshape)}")
    kbase = kv_caches.data_ptr()
    args = (key.data_ptr(), value.data_ptr(), kst[0] * es, vst[0] * es,
            k_layer * es, v_layer * es,
            kbase, kbase + BS * row_bytes,
            c_layer * es, c_block * es, row_bytes,
            slots.data_ptr(), slot_layer, T, L, row_bytes, BS, NB * BS)
    return dev, (key, value, kv_caches, slots), args


def _write_layers(key, value, kv_caches, slot_mapping) -> None:
    dev, _keep, args = _prepare_write(key, value, kv_caches, slot_mapping)
    with _OnDevice(dev):
        rc = _lib.lib().lms_reshape_and_cache_layers(*args, _stream_ptr(dev))
    if rc:
        _lib.check(rc)


class WritePlan:
    """A cache write whose arguments were validated and resolved once.

    The decode loop writes the same ``key``/``value``/``slot_mapping`` buffers into the same
    cache every step (the buffers are refilled in place), once per layer.  ``WritePlan`` does
    the tensor checks and pointer arithmetic at construction; ``run()`` is one C call.  The
    plan keeps the tensors alive and must be rebuilt if any of them is reallocated.

    ``key``/``value`` may be ``[T, H, D]`` with ``kv_cache`` one layer ``[NB, 2, BS, H, D]``,
    or ``[L, T, H, D]`` with the whole ``[L, NB, 2, BS, H, D]`` cache.
    """

    def __init__(self, key: torch.Tensor, value: torch.Tensor, kv_cache: torch.Tensor,
                 slot_mapping: torch.Tensor):
        self.device, self._keep, args = _prepare_write(key, value, kv_cache, slot_mapping)
        handle = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            # validates once and does the per-device set-up, so that run() may be the first
            # call inside a graph capture
            _lib.check(_lib.lib().lms_write_plan_create(*args, ctypes.byref(handle)))
        self._handle = handle
        self._destroy = _lib.lib().lms_write_plan_destroy
        # run() goes through the C helper: address of lms_write_plan_run + the plan's address,
        # no ctypes argument conversion on the per-layer path
        self._fn = _PLAN_RUN_ADDRESS()
        self._plan = handle.value or 0

    def run(self, stream: Optional[int] = None) -> None:
        """Enqueues the write on `stream` (a raw ``cudaStream_t`` value such as
        ``torch.cuda.current_stream().cuda_stream``; default: the current stream).  The
        current CUDA device must be the plan's device."""
        if stream is None:
            stream = torch.cuda.current_stream(self.device).cuda_stream
        rc = _packer.call_plan(self._fn, self._plan, stream)
        if rc:
            _lib.check(rc)

    def __del__(self):
        h = getattr(self, "_handle", None)
        if h:
            self._destroy(h)
            self._handle = None


# --------------------------------------------------------------------- copies
def _cache_geometry(kv_caches: torch.Tensor) -> Tuple[int, int, int, int, int]:
    """(num_layers, num_blocks, layer stride, block stride, chunk bytes) of a layer-major cache
    ``[L, NB, ...]`` whose (layer, block) chunks are contiguous.  Attribute reads only."""
    shape = kv_caches.shape
    if len(shape) < 3:
        raise ValueError("kv_caches must be [num_layers, num_blocks, ...]")
    strides = kv_caches.stride()
    es = kv_caches.element_size()
    chunk_elems = 1
    for dim in range(len(shape) - 1, 1, -1):
        if shape[dim] != 1 and strides[dim] != chunk_elems:
            raise ValueError("each (layer, block) chunk of the cache must be contiguous")
        chunk_elems *= shape[dim]
    return shape[0], shape[1], strides[0] * es, strides[1] * es, chunk_elems * es


def copy_blocks(
    kv_caches: torch.Tensor,
    src_to_dst: Union[Dict[int, List[int]], PairList],
) -> None:
    """Copy-on-write: ``kv_caches[:, dst] = kv_caches[:, src]`` for every mapped pair, in place.

    Same contract as LMServe's ``copy_blocks`` (``ops/cache_ops.py:8-36``,
    kernel ``ops/triton/cache_kernels.py:5-36``): ``kv_caches`` is
    ``[L, num_blocks, 2, block_size, H, D]`` and ``src_to_dst`` maps a source
    block to the list of blocks that receive a copy, in every layer.  A sequence
    of ``(src, dst)`` pairs or an int64 ``[n, 2]`` tensor is accepted as well.
    Destinations must be distinct and must not also appear as sources.
    """
    _require_cuda("kv_caches", kv_caches)
    dev = kv_caches.device
    L, NB, layer_stride, block_stride, chunk = _cache_geometry(kv_caches)
    on_device, _keep, ptr, n = _pair_table(src_to_dst, dev)
    if n == 0:
        return
    L_ = _lib.lib()
    fn = L_.lms_copy_blocks if on_device else L_.lms_copy_blocks_host
    with _OnDevice(dev):
        _lib.check(fn(kv_caches.data_ptr(), layer_stride, block_stride, chunk, L,
                      ptr, n, NB, _stream_ptr(dev)))


def copy_blocks_no_alloc(
    kv_caches: torch.Tensor,
    src_to_dst: Union[Dict[int, List[int]], PairList],
) -> None:
    """``copy_blocks`` for a worker that must not allocate device memory while it serves.

    Same arguments and result as :func:`copy_blocks` with a host-side table (dict, list or
    ndarray), but the table is uploaded into a fixed 256 KiB array inside the library instead
    of a buffer the library allocates on demand — see ``lms_copy_blocks_host_static`` in
    ``include/lmserve_kv.h``.  At most ``LMS_STATIC_MAX_PAIRS`` (16 384) pairs per call;
    consecutive calls must be on one stream or ordered by the caller, because they share the
    array; debug index checks do not apply.
    """
    _require_cuda("kv_caches", kv_caches)
    dev = kv_caches.device
    L, NB, layer_stride, block_stride, chunk = _cache_geometry(kv_caches)
    arr = flatten_block_map(src_to_dst)
    if arr.shape[0] == 0:
        return
    with _OnDevice(dev):
        _lib.check(_lib.lib().lms_copy_blocks_host_static(
            kv_caches.data_ptr(), layer_stride, block_stride, chunk, L,
            arr.ctypes.data, arr.shape[0], _stream_ptr(dev)))


_STAGING: Dict[Tuple[int, str], torch.Tensor] = {}


def _default_staging(dev: torch.device, direction: str, min_bytes: int) -> torch.Tensor:
    """One staging buffer per device and direction for callers that pass none (128 MiB, or
    twice a block when that is more); allocated on first use, kept for the process."""
    key = (dev.index if dev.index is not None else torch.cuda.current_device(), direction)
    want = max(128 << 20, int(min_bytes))
    t = _STAGING.get(key)
    if t is None or t.numel() < want:
        t = torch.empty(want, dtype=torch.uint8, device=dev)
        _STAGING[key] = t
    return t


def swap_blocks(
    gpu_kv_caches: torch.Tensor,
    host_pool,
    block_pairs: PairList,
    direction: str,
    layers: Optional[Tuple[int, int]] = None,
    engine: str = "kernel",
    staging: Optional[torch.Tensor] = None,
) -> None:
    """Moves whole blocks between the GPU cache and a pinned host pool.

    ``gpu_kv_caches``: ``[L, num_gpu_blocks, ...]`` (layer-major);
    ``host_pool``: a :class:`lmserve_b200.kv_worker.HostPool`
    (``[num_host_blocks, L, chunk]``, block-major — ``kv_worker.py:123-130``);
    ``direction``: ``"out"`` copies ``gpu[l, src] -> host[dst, l]``
    (``kv_worker.py:213-227``), ``"in"`` copies ``host[src, l] -> gpu[l, dst]``
    (``kv_worker.py:197-211``); ``layers=(begin, end)`` restricts the call to a
    layer range so a caller can pipeline the swap against the forward pass.
    ``engine="kernel"`` runs the sm_100a gather/scatter kernel (fastest on an otherwise idle
    GPU); ``engine="dma"`` issues one strided copy-engine transfer per block instead
    (``lms_swap_blocks_dma``; needs a host-side pair table): it uses no SM, so GEMMs that run
    at the same time keep the whole GPU — measured against a stream of 8192^3 bf16 GEMMs: the
    built-in 3-CTA copy kernel costs them about 10 %, copy grids of 5 CTAs and more 85 % and
    upwards, the copy-engine form nothing.  ``engine="staged"`` gathers groups of blocks into
    ``staging`` (a device tensor of the caller, at least two blocks' worth of bytes; 128 MiB
    and more is sensible) and lets the copy engines move whole host blocks in one transfer each
    (``lms_swap_blocks_staged``): the form for swapping many whole blocks; it reaches the rate of
    a plain pinned ``cudaMemcpy`` when the host blocks of the call are adjacent, and the kernel's
    rate when they are scattered.
    """
    _require_cuda("gpu_kv_caches", gpu_kv_caches)
    if direction not in ("out", "in"):
        raise ValueError(f"Unsupported copy direction: {direction!r} (use 'out' or 'in')")
    dev = gpu_kv_caches.device
    L, NB, layer_stride, block_stride, chunk = _cache_geometry(gpu_kv_caches)
    if host_pool.num_layers != L or host_pool.chunk_bytes != chunk:
        raise ValueError("host pool geometry does not match the GPU cache")
    l0, l1 = (0, L) if layers is None else layers
    if not (0 <= l0 <= l1 <= L):
        raise ValueError(f"layer range {layers} outside [0, {L}]")
    if engine not in ("kernel", "dma", "staged"):
        raise ValueError(f"engine must be 'kernel', 'dma' or 'staged', got {engine!r}")
    if engine != "kernel" and isinstance(block_pairs, torch.Tensor) and block_pairs.is_cuda:
        block_pairs = block_pairs.cpu()          # the copy engines are driven from the host
    if engine == "staged":
        if staging is None:
            staging = _default_staging(dev, direction, 2 * (l1 - l0) * chunk)
        elif not (isinstance(staging, torch.Tensor) and staging.is_cuda and staging.device == dev
                  and staging.is_contiguous()):
            raise ValueError("staging must be a contiguous tensor on the cache's device")
    on_device, _keep, ptr, n = _pair_table(block_pairs, dev)
    if n == 0 or l0 == l1:
        return
    L_ = _lib.lib()
    if engine == "staged":
        with _OnDevice(dev):
            _lib.check(L_.lms_swap_blocks_staged(
                _lib.LMS_SWAP_OUT if direction == "out" else _lib.LMS_SWAP_IN,
                gpu_kv_caches.data_ptr(), layer_stride, block_stride,
                host_pool.device_ptr, host_pool.block_stride, host_pool.layer_stride,
                chunk, l0, l1, ptr, n, NB, host_pool.num_blocks,
                staging.data_ptr(), staging.numel() * staging.element_size(), _stream_ptr(dev)))
        return
    if engine == "dma":
        fn = L_.lms_swap_blocks_dma
    else:
        fn = L_.lms_swap_blocks if on_device else L_.lms_swap_blocks_host
    with _OnDevice(dev):
        _lib.check(fn(
            _lib.LMS_SWAP_OUT if direction == "out" else _lib.LMS_SWAP_IN,
            gpu_kv_caches.data_ptr(), layer_stride, block_stride,
            host_pool.device_ptr, host_pool.block_stride, host_pool.layer_stride,
            chunk, l0, l1, ptr, n, NB, host_pool.num_blocks,
            _stream_ptr(dev)))


def transfer_blocks(
    src_kv_caches,
    dst_kv_caches,
    block_pairs: PairList,
    layers: Optional[Tuple[int, int]] = None,
    pull: bool = False,
) -> None:
    """Moves blocks of one GPU's cache into another GPU's cache: ``dst[:, d] = src[:, s]``.

    Replaces the host-staged NIXL push of ``kv_worker.py:358-415`` with one kernel over NVLink.
    One side is a tensor of this process, the other a tensor on another device of this process
    (peer access is enabled on demand) or a :class:`lmserve_b200.kv_worker.PeerCache` opened
    from another process's IPC handle.  By default the kernel runs on the *source* GPU and
    stores into the peer (a push, ``src_kv_caches`` local); with ``pull=True`` it runs on the
    *destination* GPU and loads from the peer (``dst_kv_caches`` local) — over NVLink the loads
    are the faster direction (788 against 715 GB/s for the 2.5 GiB transfer of the 70B TP8
    shard).  Runs on the current stream of the GPU that executes the kernel.
    ``layers=(begin, end)`` moves only that layer range, so a prefill worker can ship each
    layer as soon as it is computed instead of waiting for the whole forward pass.
    """
    def geometry(c):
        if isinstance(c, torch.Tensor):
            _require_cuda("kv_caches", c)
            L_, NB_, layer, block, chunk_ = _cache_geometry(c)
            return L_, NB_, layer, block, chunk_, c.data_ptr(), c.device
        return (c.num_layers, c.num_blocks, c.layer_stride, c.block_stride, c.chunk_bytes,
                c.device_ptr, None)

    local = dst_kv_caches if pull else src_kv_caches
    if not isinstance(local, torch.Tensor):
        raise TypeError("the cache on the GPU that runs the kernel must be a tensor of this process "
                        f"({'dst' if pull else 'src'}_kv_caches)")
    L, NB, s_layer, s_block, chunk, src_ptr, src_dev = geometry(src_kv_caches)
    dL, dNB, d_layer, d_block, d_chunk, dst_ptr, dst_dev = geometry(dst_kv_caches)
    dev = local.device
    other = src_dev if pull else dst_dev
    if other is not None and other != dev:
        with _OnDevice(dev):
            _lib.check(_lib.lib().lms_peer_enable(other.index))
    if dL != L or d_chunk != chunk:
        raise ValueError("source and destination caches must have the same layers and chunk size")
    l0, l1 = (0, L) if layers is None else layers
    if not (0 <= l0 <= l1 <= L):
        raise ValueError(f"layer range {layers} outside [0, {L}]")
    on_device, _keep, ptr, n = _pair_table(block_pairs, dev)
    if n == 0 or l0 == l1:
        return
    L_ = _lib.lib()
    fn = L_.lms_transfer_blocks if on_device else L_.lms_transfer_blocks_host
    with _OnDevice(dev):
        _lib.check(fn(src_ptr + l0 * s_layer, s_layer, s_block,
                      dst_ptr + l0 * d_layer, d_layer, d_block,
                      chunk, l1 - l0, ptr, n, NB, dNB, _stream_ptr(dev)))
