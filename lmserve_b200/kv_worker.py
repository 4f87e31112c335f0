"""Host-side mirror of LMServe's ``KVWorker`` (``runtime/worker/llm_worker/kv_worker.py``)
for the parts that move KV blocks through the GPU: the pinned host pool, the
GPU<->host swap in both directions with the per-layer event + queue handshake, and the
prefill->decode push — here a direct GPU->GPU store over NVLink instead of the
reference's NIXL/UCX host-to-host write.

The disk tier (``kv_worker.py:229-247,297-322``) is kept as the reference's host-only numpy
copies so that its four ``copy_kv`` directions keep working; the NIXL agent bookkeeping is
not mirrored.
"""
from __future__ import annotations

import ctypes
import enum
import os
import queue as _queue
import struct
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from . import _lib
from .disagg import build_push_pairs
from .ops import cache_ops


class Device(enum.IntEnum):
    """``Device`` of ``proto/worker.proto:13-17``."""
    GPU = 0
    Host = 1
    Disk = 2


@dataclass
class BlockMappingEntry:
    """``BlockMappingEntry`` of ``proto/worker.proto:78-81``."""
    src_block_id: int
    dst_block_id: int


@dataclass
class BlockMapping:
    """``BlockMapping`` of ``proto/worker.proto:83-86``: a list of (src, dst) block ids."""
    entries: List[BlockMappingEntry] = field(default_factory=list)

    @classmethod
    def from_pairs(cls, pairs) -> "BlockMapping":
        return cls([BlockMappingEntry(int(s), int(d)) for s, d in pairs])


def mappings_to_pairs(block_mappings: Sequence) -> np.ndarray:
    """Concatenates the entries of several BlockMappings into one int64 [n, 2] table.

    Accepts the dataclasses above, protobuf messages with the same field names,
    or ready-made [n, 2] arrays.
    """
    chunks = []
    for m in block_mappings:
        if isinstance(m, (np.ndarray, torch.Tensor)):
            chunks.append(cache_ops.flatten_block_map(m))
            continue
        entries = m.entries
        arr = np.empty((len(entries), 2), dtype=np.int64)
        if cache_ops._packer is not None:
            cache_ops._packer.flatten_entries(entries, arr)
            chunks.append(arr)
            continue
        for i, e in enumerate(entries):
            arr[i, 0] = e.src_block_id
            arr[i, 1] = e.dst_block_id
        chunks.append(arr)
    if not chunks:
        return np.empty((0, 2), dtype=np.int64)
    return np.concatenate(chunks, axis=0)


class HostPool:
    """Page-locked, GPU-mapped host KV pool ``[num_blocks, num_layers, chunk_bytes]``.

    The block-major layout and the pinning follow ``kv_worker.py:123-130``
    (``pycuda.pagelocked_empty((num_host_blocks, num_layers, block_size), ...)``);
    the pool is additionally *mapped*, so the swap kernels address it directly.
    bf16 payloads are held as raw bytes, as the reference holds them as uint16.
    """

    def __init__(self, num_blocks: int, num_layers: int, chunk_bytes: int, _buffer=None):
        if num_blocks <= 0 or num_layers <= 0 or chunk_bytes <= 0 or chunk_bytes % 16:
            raise ValueError("host pool needs positive sizes and a chunk that is a multiple of 16 bytes")
        self.num_blocks = int(num_blocks)
        self.num_layers = int(num_layers)
        self.chunk_bytes = int(chunk_bytes)
        self.layer_stride = self.chunk_bytes
        self.block_stride = self.num_layers * self.chunk_bytes
        self.nbytes = self.num_blocks * self.block_stride
        hp, dp = ctypes.c_void_p(), ctypes.c_void_p()
        if _buffer is None:
            _lib.check(_lib.lib().lms_host_alloc(self.nbytes, ctypes.byref(hp), ctypes.byref(dp)))
            self._registered = None
            buf = (ctypes.c_uint8 * self.nbytes).from_address(hp.value)
            flat = np.frombuffer(buf, dtype=np.uint8)
        else:
            flat = _buffer
            hp = ctypes.c_void_p(flat.ctypes.data)
            _lib.check(_lib.lib().lms_host_register(hp, self.nbytes, ctypes.byref(dp)))
            self._registered = flat  # keeps the caller's memory alive while it is pinned
        self.host_ptr = hp.value
        self.device_ptr = dp.value
        self.array = flat.reshape(self.num_blocks, self.num_layers, self.chunk_bytes)
        self.tensor = torch.from_numpy(self.array)
        cache_ops.HOST_POOL_DEVICE_PTR[self.host_ptr] = self.device_ptr

    @classmethod
    def from_buffer(cls, array: np.ndarray, num_layers: int, chunk_bytes: int) -> "HostPool":
        """Pins and maps an existing host buffer in place (``lms_host_register``) instead of
        allocating one — for a pool that already exists, e.g. shared memory or the ``.npy``
        memmap of the reference's disk tier staging.  ``array``: C-contiguous, 16-byte aligned,
        a whole number of ``num_layers * chunk_bytes`` blocks; viewed as bytes."""
        flat = np.ascontiguousarray(array).reshape(-1).view(np.uint8)
        if flat.ctypes.data != np.asarray(array).ctypes.data:
            raise ValueError("the buffer must be C-contiguous (it is pinned in place, not copied)")
        per_block = int(num_layers) * int(chunk_bytes)
        if flat.nbytes == 0 or flat.nbytes % per_block or flat.ctypes.data % 16:
            raise ValueError("buffer size must be a whole number of blocks and 16-byte aligned")
        return cls(flat.nbytes // per_block, num_layers, chunk_bytes, _buffer=flat)

    @classmethod
    def with_huge_pages(cls, num_blocks: int, num_layers: int, chunk_bytes: int) -> "HostPool":
        """A pool on anonymous memory that asks the kernel for transparent 2 MiB pages
        (``madvise(MADV_HUGEPAGE)``), touched once and pinned in place.  The swap rates are the
        same as with the default allocation (measured); what changes is the time to set the
        pool up — 2.8 s against 6.4 s for 16 GiB on the B200 host measured — which a worker
        that pins hundreds of GiB at start-up feels.  Where the kernel does not grant huge
        pages the pool is simply made of small ones."""
        import mmap
        huge = 2 << 20
        nbytes = int(num_blocks) * int(num_layers) * int(chunk_bytes)
        if nbytes <= 0:
            raise ValueError("host pool needs positive sizes")
        region = mmap.mmap(-1, nbytes + huge, flags=mmap.MAP_PRIVATE | mmap.MAP_ANONYMOUS)
        base = ctypes.addressof(ctypes.c_char.from_buffer(region))
        offset = (-base) % huge
        libc = ctypes.CDLL(None, use_errno=True)
        libc.madvise.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
        libc.madvise(base + offset, nbytes, 14)          # MADV_HUGEPAGE; advice only
        flat = np.frombuffer(region, dtype=np.uint8, count=nbytes, offset=offset)
        flat[:] = 0                                      # fault the pages in before pinning
        pool = cls(num_blocks, num_layers, chunk_bytes, _buffer=flat)
        pool._region = region                            # unmapped when the last view goes
        return pool

    def close(self) -> None:
        if getattr(self, "host_ptr", None):
            cache_ops.HOST_POOL_DEVICE_PTR.pop(self.host_ptr, None)
            self.tensor = None
            self.array = None
            if self._registered is None:
                _lib.check(_lib.lib().lms_host_free(self.host_ptr))
            else:
                _lib.check(_lib.lib().lms_host_unregister(self.host_ptr))
                self._registered = None
            self.host_ptr = None
            self.device_ptr = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


IPC_HANDLE_BYTES = 64      # sizeof(cudaIpcMemHandle_t), LMS_IPC_HANDLE_BYTES of the C header
HANDSHAKE_TIMEOUT_S = 60.0  # how long either side waits for the other's per-layer token


@dataclass
class CacheDescriptor:
    """What a decode-side worker hands to a prefill-side worker so it can push blocks:
    the GPU-direct counterpart of the serialized NIXL descriptors of
    ``kv_worker.py:348-356`` (one descriptor per reserved block there; one IPC
    handle for the whole cache plus the reserved block ids here)."""
    handle: bytes
    offset: int
    device_index: int
    num_layers: int
    num_blocks: int
    layer_stride: int
    block_stride: int
    chunk_bytes: int
    block_ids: List[int]
    # An IPC handle cannot be opened by the process that exported it.  The exporter's pid and
    # the cache's address let a worker of the SAME process (two workers on threads, or on two
    # GPUs of one process) use the memory directly; they are honoured only for caches this
    # process has itself exported (``_LOCAL_EXPORTS``).
    pid: int = 0
    address: int = 0

    # Wire form: a fixed little-endian header (magic, ten integers, the 64-byte IPC handle)
    # followed by the reserved block ids as int64.  Nothing in it is executable or typed by the
    # sender: a malformed buffer raises ValueError.
    _HEADER = struct.Struct("<4s10q64s")
    _MAGIC = b"LMS2"

    def serialize(self) -> bytes:
        if len(self.handle) != IPC_HANDLE_BYTES:
            raise ValueError("the IPC handle must be 64 bytes")
        ids = np.asarray(self.block_ids, dtype="<i8").reshape(-1)
        head = self._HEADER.pack(self._MAGIC, self.offset, self.device_index, self.num_layers,
                                 self.num_blocks, self.layer_stride, self.block_stride,
                                 self.chunk_bytes, ids.size, self.pid, self.address,
                                 bytes(self.handle))
        return head + ids.tobytes()

    @classmethod
    def deserialize(cls, data: bytes) -> "CacheDescriptor":
        data = bytes(data)
        if len(data) < cls._HEADER.size:
            raise ValueError("cache descriptor is truncated")
        (magic, offset, device_index, num_layers, num_blocks, layer_stride, block_stride,
         chunk_bytes, n_ids, pid, address, handle) = cls._HEADER.unpack_from(data)
        if magic != cls._MAGIC:
            raise ValueError("not a cache descriptor")
        if n_ids < 0 or len(data) != cls._HEADER.size + 8 * n_ids:
            raise ValueError("cache descriptor length does not match its block count")
        if min(offset, device_index, num_layers, num_blocks, layer_stride, block_stride, chunk_bytes,
               pid, address) < 0:
            raise ValueError("cache descriptor holds a negative size")
        ids = np.frombuffer(data, dtype="<i8", count=n_ids, offset=cls._HEADER.size)
        return cls(handle, offset, device_index, num_layers, num_blocks, layer_stride,
                   block_stride, chunk_bytes, ids.tolist(), pid, address)


# address -> device index of every cache this process has described with get_descriptors
_LOCAL_EXPORTS: Dict[int, int] = {}


class PeerCache:
    """Another worker's GPU cache made addressable here: mapped through its CUDA IPC handle
    (``lms_ipc_open``) when it belongs to another process, used in place (with peer access
    enabled when it is on another GPU) when this process exported it."""

    def __init__(self, desc: CacheDescriptor):
        self.desc = desc
        self.num_layers = desc.num_layers
        self.num_blocks = desc.num_blocks
        self.layer_stride = desc.layer_stride
        self.block_stride = desc.block_stride
        self.chunk_bytes = desc.chunk_bytes
        self._mapped = False
        if desc.pid == os.getpid() and desc.pid != 0:
            if _LOCAL_EXPORTS.get(desc.address) != desc.device_index:
                raise ValueError("descriptor names this process but no cache it has exported")
            if desc.device_index != torch.cuda.current_device():
                _lib.check(_lib.lib().lms_peer_enable(desc.device_index))
            self.device_ptr = desc.address
            return
        buf = ctypes.create_string_buffer(desc.handle, IPC_HANDLE_BYTES)
        out = ctypes.c_void_p()
        _lib.check(_lib.lib().lms_ipc_open(buf, desc.offset, ctypes.byref(out)))
        self.device_ptr = out.value
        self._mapped = True

    def close(self) -> None:
        if getattr(self, "device_ptr", None):
            if self._mapped:
                _lib.check(_lib.lib().lms_ipc_close(self.device_ptr, self.desc.offset))
            self.device_ptr = None


@dataclass
class KVWorkerParams:
    """What the model process hands to the KV process so that it can map the model's cache and
    its per-layer events: the GPU-facing fields of ``KVWorkerParams`` (``kv_worker.py:34-45``).
    ``kv_cache_metadata`` is the tuple ``UntypedStorage._share_cuda_()`` returns
    (``model_worker.py:284``); the event handles come from ``Event.ipc_handle()`` of events
    created with ``interprocess=True`` (``model_worker.py:232-251,285-290``).

    ``model_queue`` / ``kv_queue`` are the reference's two token queues
    (``model_worker.py:239-240``) and are needed for the same reason: a stream wait binds to the
    most recent *record* of the event at the moment the wait is issued (and does nothing if the
    event was never recorded), so the waiting side must not issue its wait before the other
    side has issued this step's record.  The recorder puts one token per layer after its
    ``record``; the waiter takes one token before its ``wait_event``."""
    kv_cache_metadata: tuple
    cache_shape: tuple            # (num_layers, num_gpu_blocks, 2, block_size, H, D)
    dtype: torch.dtype
    num_host_blocks: int = 0
    device_index: int = 0
    pre_event_handles: Sequence[bytes] = ()
    post_event_handles: Sequence[bytes] = ()
    num_disk_blocks: int = 0
    disk_kv_cache_file: Optional[str] = None
    model_queue: object = None    # KV process -> model: "pre_events[l] of this step is recorded"
    kv_queue: object = None       # model -> KV process: "post_events[l] of this step is recorded"

    @classmethod
    def from_cache(cls, kv_caches: torch.Tensor, num_host_blocks: int = 0,
                   pre_events: Sequence[torch.cuda.Event] = (),
                   post_events: Sequence[torch.cuda.Event] = (),
                   model_queue=None, kv_queue=None) -> "KVWorkerParams":
        """Called in the model process (``ModelWorker.init_cache``, ``model_worker.py:278-306``)."""
        cache_ops._require_cuda("kv_caches", kv_caches)
        if not kv_caches.is_contiguous() or kv_caches.storage_offset() != 0:
            raise ValueError("the shared cache must be a whole contiguous allocation")
        return cls(kv_caches.untyped_storage()._share_cuda_(), tuple(kv_caches.shape), kv_caches.dtype,
                   num_host_blocks, kv_caches.device.index,
                   [e.ipc_handle() for e in pre_events], [e.ipc_handle() for e in post_events],
                   model_queue=model_queue, kv_queue=kv_queue)


def cache_block_counts(gpu_cache_size: int, host_cache_size: int, num_layers: int, num_kv_heads: int,
                       head_dim: int, block_size: int, dtype: torch.dtype):
    """``(num_gpu_blocks, num_host_blocks, kv_block_size)`` with the arithmetic of
    ``ModelWorker.init_cache`` (``model_worker.py:215-220,278-279``): ``kv_block_size`` is the
    bytes of the K (or V) half of one block of one layer, and a block costs
    ``num_layers * 2 * kv_block_size`` bytes in either pool."""
    dtype_byte = torch.finfo(dtype).bits // 8
    kv_block_size = block_size * num_kv_heads * head_dim * dtype_byte
    per_block = num_layers * 2 * kv_block_size
    return int(gpu_cache_size) // per_block, int(host_cache_size) // per_block, kv_block_size


def _take_token(q, what: str) -> None:
    """Blocks until the other side has put its token for `what` (or raises TimeoutError)."""
    try:
        q.get(timeout=HANDSHAKE_TIMEOUT_S)
    except _queue.Empty:
        raise TimeoutError(f"no token for {what} within {HANDSHAKE_TIMEOUT_S:.0f} s: the other "
                           "side of the layer handshake did not record its event") from None


@dataclass
class KVWorkerHandle:
    """The model process's end of the layer handshake: ``KVWorkerHandle`` of
    ``kv_worker.py:25-32``.  Layer ``i`` of the forward pass waits for ``pre_events[i]`` (its
    blocks have been swapped in) and records ``post_events[i]`` when it has written its KV
    (they may be swapped out or pushed).  With the queues set (always, when the KV worker runs
    in another process or thread) the pre-hook first takes a token from ``model_queue`` — the
    KV worker puts it after recording ``pre_events[i]`` — and the post-hook puts a token on
    ``kv_queue`` after its record, exactly as ``model_worker.py:259-270``; without that the
    stream wait could be issued before this step's record and bind to the previous step's."""
    pre_events: List[torch.cuda.Event]
    post_events: List[torch.cuda.Event]
    enable_wait_before_execute: bool = False
    enable_record_after_execute: bool = False
    model_queue: object = None
    kv_queue: object = None

    def wait_before_layer(self, i: int, stream=None) -> None:
        """What the pre-hook of layer `i` does (``model_worker.py:259-263``)."""
        if self.model_queue is not None:
            _take_token(self.model_queue, f"pre_events[{i}]")
        (stream or torch.cuda.current_stream()).wait_event(self.pre_events[i])

    def record_after_layer(self, i: int, stream=None) -> None:
        """What the post-hook of layer `i` does (``model_worker.py:265-270``)."""
        self.post_events[i].record(stream or torch.cuda.current_stream())
        if self.kv_queue is not None:
            self.kv_queue.put(b"")

    def register_hooks(self, attn_layers, stream: Optional[torch.cuda.Stream] = None) -> list:
        """Forward pre / post hooks on the attention modules, as ``model_worker.py:253-275``:
        the pre-hook makes `stream` (default: the current stream) wait for the layer's
        pre-event when ``enable_wait_before_execute`` is set, the post-hook records the layer's
        post-event when ``enable_record_after_execute`` is set.  Returns the hook handles."""
        handles = []
        for i, layer in enumerate(attn_layers):
            def pre_hook(mod, args, i=i):
                if self.enable_wait_before_execute:
                    self.wait_before_layer(i, stream)

            def post_hook(mod, args, output, i=i):
                if self.enable_record_after_execute:
                    self.record_after_layer(i, stream)

            handles.append(layer.register_forward_pre_hook(pre_hook))
            handles.append(layer.register_forward_hook(post_hook))
        return handles


def init_cache(gpu_cache_size: int, host_cache_size: int, *, num_layers: int, num_kv_heads: int,
               head_dim: int, block_size: int, dtype: torch.dtype, device="cuda", mp_context="spawn"):
    """``ModelWorker.init_cache`` (``model_worker.py:200-308``) for the GPU and host tiers:
    allocates the paged cache ``[L, num_gpu_blocks, 2, block_size, H, D]``, creates the per-layer
    interprocess events, and returns ``(kv_caches, handle, params)`` — the cache for the model,
    the :class:`KVWorkerHandle` for its hooks, and the :class:`KVWorkerParams` to send to the KV
    process (``KVWorker.from_params``).  The two token queues of the handshake are created in
    the multiprocessing context `mp_context` (a name or a context object; ``None`` = no queues,
    for a worker driven from the model's own thread) and travel inside ``params``."""
    num_gpu_blocks, num_host_blocks, _ = cache_block_counts(
        gpu_cache_size, host_cache_size, num_layers, num_kv_heads, head_dim, block_size, dtype)
    if num_gpu_blocks <= 0:
        raise ValueError("gpu_cache_size is smaller than one block")
    dev = torch.device(device)
    if dev.type != "cuda":
        raise RuntimeError("the KV cache lives on a CUDA device; there is no CPU path")
    with torch.cuda.device(dev):
        kv_caches = torch.empty(num_layers, num_gpu_blocks, 2, block_size, num_kv_heads, head_dim,
                                dtype=dtype, device=dev)
        pre = [torch.cuda.Event(interprocess=True) for _ in range(num_layers)]
        post = [torch.cuda.Event(interprocess=True) for _ in range(num_layers)]
    model_queue = kv_queue = None
    if mp_context is not None:
        import torch.multiprocessing as tmp
        ctx = tmp.get_context(mp_context) if isinstance(mp_context, str) else mp_context
        model_queue, kv_queue = ctx.Queue(), ctx.Queue()
    handle = KVWorkerHandle(pre, post, model_queue=model_queue, kv_queue=kv_queue)
    return kv_caches, handle, KVWorkerParams.from_cache(kv_caches, num_host_blocks, pre, post,
                                                        model_queue, kv_queue)


def open_disk_pool(path: str, shape) -> np.ndarray:
    """The disk tier's block pool ``[num_disk_blocks, L, chunk_bytes]`` as a writable ``.npy``
    memory map (role of ``memmap_disk_kv_cache``, ``kv_worker.py:48-84``): an existing file of the
    right shape is reused, anything else is replaced by a new file.  Payload is held as bytes."""
    shape = tuple(int(x) for x in shape)
    if os.path.exists(path):
        try:
            arr = np.load(path, mmap_mode="r+")
            if arr.shape == shape and arr.dtype == np.uint8:
                return arr
            del arr
        except Exception:  # noqa: BLE001 - an unreadable file is replaced, as in the reference
            pass
        os.remove(path)
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    return np.lib.format.open_memmap(path, mode="w+", dtype=np.uint8, shape=shape)


class KVWorker:
    """Per-GPU mover of KV blocks, API-compatible with the GPU-facing part of LMServe's
    ``KVWorker`` (``kv_worker.py:88-195,249-295,336-415``).

    ``gpu_kv_caches`` is the model's ``[L, num_gpu_blocks, 2, block_size, H, D]``
    tensor (or its ``[L, num_gpu_blocks, chunk]`` view); the worker does not own it.
    """

    def __init__(self, name: str, gpu_kv_caches: torch.Tensor, num_host_blocks: int = 0,
                 swap_engine: str = "kernel", num_disk_blocks: int = 0,
                 disk_kv_cache_file: Optional[str] = None, num_disk_copy_workers: int = 4,
                 staging_bytes: int = 256 << 20):
        cache_ops._require_cuda("gpu_kv_caches", gpu_kv_caches)
        if swap_engine not in ("kernel", "dma", "staged"):
            raise ValueError("swap_engine must be 'kernel', 'dma' or 'staged'")
        # "kernel": the sm_100a gather/scatter kernel on 3 CTAs - 0.92 of the PCIe memcpy rate
        # even when launched once per layer, at a cost of about 10 % to concurrent full-SM GEMMs.
        # "dma": copy engines only, no SM is touched; its rate (0.89 of memcpy) needs many layers per launch
        # (one 64 KiB copy per layer and block, the reference's pattern, reaches 13 GB/s).
        # "staged": whole-block swaps through a device staging ring and one DMA transfer per
        # host block; swaps that are pipelined layer by layer fall back to the kernel.
        self.swap_engine = swap_engine
        self.name = name
        self.gpu_kv_caches = gpu_kv_caches
        self.device = gpu_kv_caches.device
        (self.num_layers, self.num_gpu_blocks, self.layer_stride,
         self.block_stride, self.chunk_bytes) = cache_ops._cache_geometry(gpu_kv_caches)
        self.host_pool = (HostPool(num_host_blocks, self.num_layers, self.chunk_bytes)
                          if num_host_blocks > 0 else None)
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().lms_init_device())
            self.dtoh_stream = torch.cuda.Stream()
            self.htod_stream = torch.cuda.Stream()
            self.push_stream = torch.cuda.Stream()
        self._staging_bytes = int(staging_bytes)
        self._staging: Dict[str, torch.Tensor] = {}
        # the token queues of the layer handshake (None: the model runs in this thread and
        # issues its records before the worker's waits by construction)
        self.model_queue = None
        self.kv_queue = None
        self.pre_events: List[torch.cuda.Event] = []
        self.post_events: List[torch.cuda.Event] = []
        self._peers: Dict[str, PeerCache] = {}
        self.COPY_KV_OP_MAP = {
            (Device.GPU, Device.Host): self.save_kv_blocks_to_host,
            (Device.Host, Device.GPU): self.load_kv_blocks_from_host,
        }
        # Disk tier (kv_worker.py:131-139,229-247,296-322): a host-only path, no GPU involved -
        # blocks move between the pinned pool and a memory-mapped .npy file, one task per layer.
        self.disk_kv_caches = None
        self._disk_threads = None
        if num_disk_blocks > 0:
            if self.host_pool is None or not disk_kv_cache_file:
                raise ValueError("the disk tier needs a host pool and a disk_kv_cache_file")
            from concurrent.futures import ThreadPoolExecutor
            self.disk_kv_caches = open_disk_pool(
                disk_kv_cache_file, (num_disk_blocks, self.num_layers, self.chunk_bytes))
            self._disk_threads = ThreadPoolExecutor(max_workers=max(1, int(num_disk_copy_workers)))
            self.COPY_KV_OP_MAP[(Device.Host, Device.Disk)] = self.save_kv_blocks_to_disk
            self.COPY_KV_OP_MAP[(Device.Disk, Device.Host)] = self.load_kv_blocks_from_disk

    @classmethod
    def from_params(cls, name: str, params: KVWorkerParams, **kw) -> "KVWorker":
        """Built in the KV process: maps the model process's cache through CUDA IPC
        (``kv_worker.py:104-108``), opens its interprocess events (``kv_worker.py:140-147``) and
        keeps its two token queues (``kv_worker.py:149-154``).  The events are available as
        ``worker.pre_events`` / ``worker.post_events``; swaps that are given these events use the
        queues for the host side of the handshake."""
        dev = torch.device("cuda", params.device_index)
        with torch.cuda.device(dev):
            storage = torch.UntypedStorage._new_shared_cuda(*params.kv_cache_metadata)
            cache = torch.empty(0, dtype=params.dtype, device=dev)
            cache.set_(storage)
            cache = cache.view(*params.cache_shape)
            worker = cls(name, cache, params.num_host_blocks, num_disk_blocks=params.num_disk_blocks,
                         disk_kv_cache_file=params.disk_kv_cache_file, **kw)
            worker.pre_events = [torch.cuda.Event.from_ipc_handle(dev, h) for h in params.pre_event_handles]
            worker.post_events = [torch.cuda.Event.from_ipc_handle(dev, h) for h in params.post_event_handles]
        worker.model_queue = params.model_queue
        worker.kv_queue = params.kv_queue
        return worker

    # -- swap -----------------------------------------------------------------
    def load_kv_blocks_from_host(self, block_mappings, stream: Optional[torch.cuda.Stream] = None,
                                 pre_events: Optional[Sequence[torch.cuda.Event]] = None,
                                 layers_per_launch: Optional[int] = None) -> None:
        """Host -> GPU fetch (``kv_worker.py:249-270``).

        With ``pre_events`` the fetch runs ``layers_per_launch`` layers at a time
        (default 1, like the reference) and, once layer ``l`` has been enqueued, records
        ``pre_events[l]`` on the copy stream and puts one token on ``model_queue`` (when the
        worker has one), so the forward pass can wait per layer; without them it is one launch
        over all layers.  As in the reference nothing is recorded for an empty request.
        """
        self._swap(block_mappings, "in", stream or self.htod_stream, pre_events, None,
                   layers_per_launch)

    def save_kv_blocks_to_host(self, block_mappings, stream: Optional[torch.cuda.Stream] = None,
                               post_events: Optional[Sequence[torch.cuda.Event]] = None,
                               layers_per_launch: Optional[int] = None) -> None:
        """GPU -> host write-through (``kv_worker.py:272-295``).

        With ``post_events`` the worker takes the model's token for layer ``l`` from
        ``kv_queue`` (when it has one; the model puts it after recording, so the record has been
        issued), makes the copy stream wait for ``post_events[l]`` (recorded by the model after
        layer ``l``'s attention) and then copies layer ``l``.
        """
        self._swap(block_mappings, "out", stream or self.dtoh_stream, None, post_events,
                   layers_per_launch)

    def _disk_copy(self, block_mappings, dst, src, wait_for) -> None:
        pairs = mappings_to_pairs(block_mappings)
        if pairs.shape[0] == 0:
            return
        for name, ids, pool in (("source", pairs[:, 0], src), ("destination", pairs[:, 1], dst)):
            if ids.min() < 0 or ids.max() >= pool.shape[0]:
                raise IndexError(f"{name} block id outside the pool of {pool.shape[0]} blocks")
        for stream in wait_for:      # swaps in flight on the pinned pool must have landed / left
            stream.synchronize()
        s_ids, d_ids = pairs[:, 0], pairs[:, 1]

        def one_layer(l):
            dst[d_ids, l] = src[s_ids, l]

        list(self._disk_threads.map(one_layer, range(self.num_layers)))

    def save_kv_blocks_to_disk(self, block_mappings) -> None:
        """Host -> disk (``kv_worker.py:239-247,311-322``): ``disk[dst, l] = host[src, l]``."""
        self._disk_copy(block_mappings, self.disk_kv_caches, self.host_pool.array, (self.dtoh_stream,))

    def load_kv_blocks_from_disk(self, block_mappings) -> None:
        """Disk -> host (``kv_worker.py:229-237,296-309``): ``host[dst, l] = disk[src, l]``."""
        self._disk_copy(block_mappings, self.host_pool.array, self.disk_kv_caches,
                        (self.dtoh_stream, self.htod_stream))

    def _staging_for(self, direction: str) -> torch.Tensor:
        t = self._staging.get(direction)
        if t is None:
            want = max(self._staging_bytes, 2 * self.num_layers * self.chunk_bytes)
            t = torch.empty(want, dtype=torch.uint8, device=self.device)
            self._staging[direction] = t
        return t

    def _swap(self, block_mappings, direction, stream, pre_events, post_events, group) -> None:
        if self.host_pool is None:
            raise RuntimeError("this KVWorker was created without a host pool")
        pairs_np = mappings_to_pairs(block_mappings)
        if pairs_np.shape[0] == 0:
            return
        events = pre_events if pre_events is not None else post_events
        L = self.num_layers
        with torch.cuda.device(self.device), torch.cuda.stream(stream):
            engine = self.swap_engine
            if events is None:
                if engine == "staged":
                    cache_ops.swap_blocks(self.gpu_kv_caches, self.host_pool, pairs_np, direction,
                                          engine="staged", staging=self._staging_for(direction))
                    return
                pairs = pairs_np if engine == "dma" else cache_ops._pairs_on_device(pairs_np, self.device)
                cache_ops.swap_blocks(self.gpu_kv_caches, self.host_pool, pairs, direction, engine=engine)
                return
            if engine == "staged":
                engine = "kernel"     # layer by layer every transfer is one chunk: the kernel wins
            # the kernel reads the table on the device (uploaded once for all layer launches);
            # the copy engines are driven from the host table
            pairs = pairs_np if engine == "dma" else cache_ops._pairs_on_device(pairs_np, self.device)
            step = max(1, int(group or 1))
            for l0 in range(0, L, step):
                l1 = min(L, l0 + step)
                if post_events is not None:
                    for l in range(l0, l1):
                        if self.kv_queue is not None:
                            _take_token(self.kv_queue, f"post_events[{l}]")
                        stream.wait_event(post_events[l])
                cache_ops.swap_blocks(self.gpu_kv_caches, self.host_pool, pairs, direction,
                                      layers=(l0, l1), engine=engine)
                if pre_events is not None:
                    for l in range(l0, l1):
                        pre_events[l].record(stream)
                        if self.model_queue is not None:
                            self.model_queue.put(b"")

    def copy_kv(self, block_mappings, src: Device, dst: Device, **kw) -> None:
        """``KVWorker.copy_kv`` (``kv_worker.py:336-346``): dispatch on (src, dst)."""
        key = (src, dst)
        if key not in self.COPY_KV_OP_MAP:
            raise ValueError(f"Unsupported copy direction: {src} -> {dst}")
        self.COPY_KV_OP_MAP[key](block_mappings, **kw)

    # -- prefill -> decode ----------------------------------------------------
    def get_descriptors(self, block_ids: Sequence[int]) -> bytes:
        """Serialized descriptor of this worker's GPU cache and the reserved blocks
        (role of ``kv_worker.py:348-356``).  The ids are *GPU* block ids of this worker: the
        transfer goes cache to cache, so an engine that drives it reserves GPU blocks on the
        decode side where the reference's engine reserves host blocks."""
        ids = [int(b) for b in block_ids]
        if ids and (min(ids) < 0 or max(ids) >= self.num_gpu_blocks):
            raise IndexError(f"reserved block id outside the cache of {self.num_gpu_blocks} blocks")
        handle = ctypes.create_string_buffer(IPC_HANDLE_BYTES)
        offset = ctypes.c_int64()
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().lms_ipc_export(self.gpu_kv_caches.data_ptr(), handle,
                                                 ctypes.byref(offset)))
        address = self.gpu_kv_caches.data_ptr()
        _LOCAL_EXPORTS[address] = self.device.index
        return CacheDescriptor(handle.raw, offset.value, self.device.index, self.num_layers,
                               self.num_gpu_blocks, self.layer_stride, self.block_stride,
                               self.chunk_bytes, ids, os.getpid(), address).serialize()

    def _transfer_table(self, remote_descs: bytes, block_ids: Sequence[int]):
        """(descriptor, [n, 2] (local, remote) table) after every check the host can make: the
        descriptor parses, the geometries agree, and every id lies inside its cache — a bad id
        would otherwise overwrite another sequence's blocks on the peer without any error.
        Raises ValueError with the reason."""
        desc = CacheDescriptor.deserialize(remote_descs)
        if desc.num_layers != self.num_layers or desc.chunk_bytes != self.chunk_bytes:
            raise ValueError(f"cache geometries differ (peer {desc.num_layers} layers x {desc.chunk_bytes} B, "
                             f"local {self.num_layers} x {self.chunk_bytes} B)")
        if desc.block_stride < desc.chunk_bytes or desc.layer_stride < desc.chunk_bytes or \
                desc.block_stride % 16 or desc.layer_stride % 16:
            raise ValueError("peer descriptor has impossible strides")
        pairs = build_push_pairs(block_ids, desc.block_ids)
        if pairs.shape[0]:
            lo, hi = pairs.min(axis=0), pairs.max(axis=0)
            if lo[0] < 0 or hi[0] >= self.num_gpu_blocks:
                raise ValueError(f"local block id outside the cache of {self.num_gpu_blocks} blocks")
            if lo[1] < 0 or hi[1] >= desc.num_blocks:
                raise ValueError(f"remote block id outside the peer cache of {desc.num_blocks} blocks")
        return desc, pairs

    def _peer(self, peer_name: str, desc: CacheDescriptor) -> PeerCache:
        peer = self._peers.get(peer_name)
        if peer is not None and (peer.desc.handle != desc.handle or peer.desc.offset != desc.offset
                                 or peer.desc.address != desc.address):
            peer.close()          # the peer re-allocated its cache: map the new one
            peer = None
        if peer is None:
            peer = PeerCache(desc)
            self._peers[peer_name] = peer
        return peer

    def push_kv(self, peer_name: str, remote_descs: bytes, block_ids: Sequence[int],
                stream: Optional[torch.cuda.Stream] = None, post_events=None,
                layers_per_launch: int = 1) -> bool:
        """Pushes local GPU blocks ``block_ids`` into the peer's reserved blocks
        (role of ``kv_worker.py:358-415``).  As there, surplus remote blocks are
        dropped so that both lists have ``len(block_ids)`` entries.  Returns False
        (after printing the reason) instead of raising, like the reference.  With
        ``post_events`` (one event per layer, recorded by the model after it has written that
        layer's KV) the push is issued layer by layer behind the prefill instead of after it."""
        try:
            try:
                desc, pairs = self._transfer_table(remote_descs, block_ids)
            except (ValueError, struct.error) as e:
                print(f"Creating transfer failed. {e}")
                return False
            with torch.cuda.device(self.device):
                peer = self._peer(peer_name, desc)
                s = stream or self.push_stream
                with torch.cuda.stream(s):
                    if post_events is None:
                        cache_ops.transfer_blocks(self.gpu_kv_caches, peer, pairs)
                    else:
                        # layer by layer behind the forward pass: layer l leaves as soon as the
                        # model has recorded post_events[l] (the swap-out handshake, applied to
                        # the push); the pair table is uploaded once
                        table = cache_ops._pairs_on_device(pairs, self.device)
                        step = max(1, int(layers_per_launch or 1))
                        for l0 in range(0, self.num_layers, step):
                            l1 = min(self.num_layers, l0 + step)
                            for l in range(l0, l1):
                                if self.kv_queue is not None:
                                    _take_token(self.kv_queue, f"post_events[{l}]")
                                s.wait_event(post_events[l])
                            cache_ops.transfer_blocks(self.gpu_kv_caches, peer, table, layers=(l0, l1))
            return True
        except (_lib.LmsError, ValueError, TimeoutError) as e:
            print(f"Posting transfer failed. {e}")
            return False

    def pull_kv(self, peer_name: str, remote_descs: bytes, block_ids: Sequence[int],
                stream: Optional[torch.cuda.Stream] = None) -> bool:
        """The mirror image of :meth:`push_kv` (role of ``kv_worker.py:417-454``, NIXL "READ"):
        this GPU reads the blocks the peer's descriptor lists out of the peer's cache, over
        NVLink, into its own blocks ``block_ids``.  The kernel runs here, with plain loads from
        the mapped peer memory."""
        try:
            try:
                desc, pairs = self._transfer_table(remote_descs, block_ids)   # (local, remote)
            except (ValueError, struct.error) as e:
                print(f"Creating transfer failed. {e}")
                return False
            with torch.cuda.device(self.device):
                peer = self._peer(peer_name, desc)
                table = np.ascontiguousarray(pairs[:, ::-1])              # (remote src, local dst)
                with torch.cuda.stream(stream or self.push_stream):
                    cache_ops.transfer_blocks(peer, self.gpu_kv_caches, table, pull=True)
            return True
        except (_lib.LmsError, ValueError) as e:
            print(f"Posting transfer failed. {e}")
            return False

    def close(self) -> None:
        for p in self._peers.values():
            p.close()
        self._peers.clear()
        self._staging.clear()
        if self._disk_threads is not None:
            self._disk_threads.shutdown(wait=True)
            self._disk_threads = None
        if self.disk_kv_caches is not None:
            self.disk_kv_caches.flush()
            self.disk_kv_caches = None
        if self.host_pool is not None:
            self.host_pool.close()
            self.host_pool = None
