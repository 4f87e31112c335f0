"""Host-side mirror of LMServe's ``KVWorker`` (``runtime/worker/llm_worker/kv_worker.py``)
for the parts that move KV blocks through the GPU: the pinned host pool, the
GPU<->host swap in both directions with the per-layer event handshake, and the
prefill->decode push — here a direct GPU->GPU store over NVLink instead of the
reference's NIXL/UCX host-to-host write.

Not mirrored (no GPU data path): the disk tier (``kv_worker.py:229-247,297-322``)
and the NIXL agent bookkeeping.
"""
from __future__ import annotations

import ctypes
import enum
import pickle
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

    def serialize(self) -> bytes:
        return pickle.dumps(self.__dict__)

    @classmethod
    def deserialize(cls, data: bytes) -> "CacheDescriptor":
        return cls(**pickle.loads(data))


class PeerCache:
    """Another process's GPU cache mapped into this process (``lms_ipc_open``)."""

    def __init__(self, desc: CacheDescriptor):
        self.desc = desc
        self.num_layers = desc.num_layers
        self.num_blocks = desc.num_blocks
        self.layer_stride = desc.layer_stride
        self.block_stride = desc.block_stride
        self.chunk_bytes = desc.chunk_bytes
        buf = ctypes.create_string_buffer(desc.handle, _lib_handle_bytes())
        out = ctypes.c_void_p()
        _lib.check(_lib.lib().lms_ipc_open(buf, desc.offset, ctypes.byref(out)))
        self.device_ptr = out.value

    def close(self) -> None:
        if getattr(self, "device_ptr", None):
            _lib.check(_lib.lib().lms_ipc_close(self.device_ptr, self.desc.offset))
            self.device_ptr = None


def _lib_handle_bytes() -> int:
    return 64


@dataclass
class KVWorkerParams:
    """What the model process hands to the KV process so that it can map the model's cache and
    its per-layer events: the GPU-facing fields of ``KVWorkerParams`` (``kv_worker.py:34-45``).
    ``kv_cache_metadata`` is the tuple ``UntypedStorage._share_cuda_()`` returns
    (``model_worker.py:284``); the event handles come from ``Event.ipc_handle()`` of events
    created with ``interprocess=True`` (``model_worker.py:232-251,285-290``).  The queues of the
    reference carry only wake-up tokens for its polling loops; here ordering is by the events
    themselves, so no queue is needed."""
    kv_cache_metadata: tuple
    cache_shape: tuple            # (num_layers, num_gpu_blocks, 2, block_size, H, D)
    dtype: torch.dtype
    num_host_blocks: int = 0
    device_index: int = 0
    pre_event_handles: Sequence[bytes] = ()
    post_event_handles: Sequence[bytes] = ()
    num_disk_blocks: int = 0
    disk_kv_cache_file: Optional[str] = None

    @classmethod
    def from_cache(cls, kv_caches: torch.Tensor, num_host_blocks: int = 0,
                   pre_events: Sequence[torch.cuda.Event] = (),
                   post_events: Sequence[torch.cuda.Event] = ()) -> "KVWorkerParams":
        """Called in the model process (``ModelWorker.init_cache``, ``model_worker.py:278-306``)."""
        cache_ops._require_cuda("kv_caches", kv_caches)
        if not kv_caches.is_contiguous() or kv_caches.storage_offset() != 0:
            raise ValueError("the shared cache must be a whole contiguous allocation")
        return cls(kv_caches.untyped_storage()._share_cuda_(), tuple(kv_caches.shape), kv_caches.dtype,
                   num_host_blocks, kv_caches.device.index,
                   [e.ipc_handle() for e in pre_events], [e.ipc_handle() for e in post_events])


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


@dataclass
class KVWorkerHandle:
    """The model process's end of the layer handshake: ``KVWorkerHandle`` of ``kv_worker.py:25-32``
    without its two wake-up queues (the events order the streams by themselves).  Layer ``i`` of
    the forward pass waits for ``pre_events[i]`` (its blocks have been swapped in) and records
    ``post_events[i]`` when it has written its KV (they may be swapped out or pushed)."""
    pre_events: List[torch.cuda.Event]
    post_events: List[torch.cuda.Event]
    enable_wait_before_execute: bool = False
    enable_record_after_execute: bool = False

    def register_hooks(self, attn_layers, stream: Optional[torch.cuda.Stream] = None) -> list:
        """Forward pre / post hooks on the attention modules, as ``model_worker.py:253-275``:
        the pre-hook makes `stream` (default: the current stream) wait for the layer's
        pre-event when ``enable_wait_before_execute`` is set, the post-hook records the layer's
        post-event when ``enable_record_after_execute`` is set.  Returns the hook handles."""
        handles = []
        for i, layer in enumerate(attn_layers):
            def pre_hook(mod, args, i=i):
                if self.enable_wait_before_execute:
                    (stream or torch.cuda.current_stream()).wait_event(self.pre_events[i])

            def post_hook(mod, args, output, i=i):
                if self.enable_record_after_execute:
                    self.post_events[i].record(stream or torch.cuda.current_stream())

            handles.append(layer.register_forward_pre_hook(pre_hook))
            handles.append(layer.register_forward_hook(post_hook))
        return handles


def init_cache(gpu_cache_size: int, host_cache_size: int, *, num_layers: int, num_kv_heads: int,
               head_dim: int, block_size: int, dtype: torch.dtype, device="cuda"):
    """``ModelWorker.init_cache`` (``model_worker.py:200-308``) for the GPU and host tiers:
    allocates the paged cache ``[L, num_gpu_blocks, 2, block_size, H, D]``, creates the per-layer
    interprocess events, and returns ``(kv_caches, handle, params)`` — the cache for the model,
    the :class:`KVWorkerHandle` for its hooks, and the :class:`KVWorkerParams` to send to the KV
    process (``KVWorker.from_params``)."""
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
    handle = KVWorkerHandle(pre, post)
    return kv_caches, handle, KVWorkerParams.from_cache(kv_caches, num_host_blocks, pre, post)


def open_disk_pool(path: str, shape) -> np.ndarray:
    """The disk tier's block pool ``[num_disk_blocks, L, chunk_bytes]`` as a writable ``.npy``
    memory map (role of ``memmap_disk_kv_cache``, ``kv_worker.py:48-84``): an existing file of the
    right shape is reused, anything else is replaced by a new file.  Payload is held as bytes."""
    import os
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
                 disk_kv_cache_file: Optional[str] = None, num_disk_copy_workers: int = 4):
        cache_ops._require_cuda("gpu_kv_caches", gpu_kv_caches)
        if swap_engine not in ("kernel", "dma"):
            raise ValueError("swap_engine must be 'kernel' or 'dma'")
        # "kernel": the sm_100a gather/scatter kernel on 3 CTAs - full PCIe rate even when
        # launched once per layer, at a cost of about 10 % to concurrent full-SM GEMMs.
        # "dma": copy engines only, no SM is touched; full rate needs many layers per launch
        # (one 64 KiB copy per layer and block, the reference's pattern, reaches 13 GB/s).
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
    def from_params(cls, name: str, params: KVWorkerParams) -> "KVWorker":
        """Built in the KV process: maps the model process's cache through CUDA IPC
        (``kv_worker.py:104-108``) and opens its interprocess events (``kv_worker.py:140-147``).
        The events are available as ``worker.pre_events`` / ``worker.post_events``."""
        dev = torch.device("cuda", params.device_index)
        with torch.cuda.device(dev):
            storage = torch.UntypedStorage._new_shared_cuda(*params.kv_cache_metadata)
            cache = torch.empty(0, dtype=params.dtype, device=dev)
            cache.set_(storage)
            cache = cache.view(*params.cache_shape)
            worker = cls(name, cache, params.num_host_blocks, num_disk_blocks=params.num_disk_blocks,
                         disk_kv_cache_file=params.disk_kv_cache_file)
            worker.pre_events = [torch.cuda.Event.from_ipc_handle(dev, h) for h in params.pre_event_handles]
            worker.post_events = [torch.cuda.Event.from_ipc_handle(dev, h) for h in params.post_event_handles]
        return worker

    # -- swap -----------------------------------------------------------------
    def load_kv_blocks_from_host(self, block_mappings, stream: Optional[torch.cuda.Stream] = None,
                                 pre_events: Optional[Sequence[torch.cuda.Event]] = None,
                                 layers_per_launch: Optional[int] = None) -> None:
        """Host -> GPU fetch (``kv_worker.py:249-270``).

        With ``pre_events`` the fetch runs ``layers_per_launch`` layers at a time
        (default 1, like the reference) and records ``pre_events[l]`` on the copy
        stream once layer ``l`` has landed, so the forward pass can wait per layer;
        without them it is one launch over all layers.
        """
        self._swap(block_mappings, "in", stream or self.htod_stream, pre_events, None,
                   layers_per_launch)

    def save_kv_blocks_to_host(self, block_mappings, stream: Optional[torch.cuda.Stream] = None,
                               post_events: Optional[Sequence[torch.cuda.Event]] = None,
                               layers_per_launch: Optional[int] = None) -> None:
        """GPU -> host write-through (``kv_worker.py:272-295``).

        With ``post_events`` the copy stream waits for ``post_events[l]`` (recorded by
        the model after layer ``l``'s attention) before layer ``l`` is copied.
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
            # the kernel reads the table on the device (uploaded once for all layer launches);
            # the copy engines are driven from the host table
            pairs = pairs_np if engine == "dma" else cache_ops._pairs_on_device(pairs_np, self.device)
            if events is None:
                cache_ops.swap_blocks(self.gpu_kv_caches, self.host_pool, pairs, direction, engine=engine)
                return
            step = max(1, int(group or 1))
            for l0 in range(0, L, step):
                l1 = min(L, l0 + step)
                if post_events is not None:
                    for l in range(l0, l1):
                        stream.wait_event(post_events[l])
                cache_ops.swap_blocks(self.gpu_kv_caches, self.host_pool, pairs, direction,
                                      layers=(l0, l1), engine=engine)
                if pre_events is not None:
                    for l in range(l0, l1):
                        pre_events[l].record(stream)

    def copy_kv(self, block_mappings, src: Device, dst: Device, **kw) -> None:
        """``KVWorker.copy_kv`` (``kv_worker.py:336-346``): dispatch on (src, dst)."""
        key = (src, dst)
        if key not in self.COPY_KV_OP_MAP:
            raise ValueError(f"Unsupported copy direction: {src} -> {dst}")
        self.COPY_KV_OP_MAP[key](block_mappings, **kw)

    # -- prefill -> decode ----------------------------------------------------
    def get_descriptors(self, block_ids: Sequence[int]) -> bytes:
        """Serialized descriptor of this worker's GPU cache and the reserved blocks
        (role of ``kv_worker.py:348-356``)."""
        handle = ctypes.create_string_buffer(_lib_handle_bytes())
        offset = ctypes.c_int64()
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().lms_ipc_export(self.gpu_kv_caches.data_ptr(), handle,
                                                 ctypes.byref(offset)))
        return CacheDescriptor(handle.raw, offset.value, self.device.index, self.num_layers,
                               self.num_gpu_blocks, self.layer_stride, self.block_stride,
                               self.chunk_bytes, [int(b) for b in block_ids]).serialize()

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
            desc = CacheDescriptor.deserialize(remote_descs)
            try:
                pairs = build_push_pairs(block_ids, desc.block_ids)
            except ValueError as e:
                print(f"Creating transfer failed. {e}")
                return False
            with torch.cuda.device(self.device):
                peer = self._peers.get(peer_name)
                if peer is None:
                    peer = PeerCache(desc)
                    self._peers[peer_name] = peer
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
                                s.wait_event(post_events[l])
                            cache_ops.transfer_blocks(self.gpu_kv_caches, peer, table, layers=(l0, l1))
            return True
        except _lib.LmsError as e:
            print(f"Posting transfer failed. {e}")
            return False

    def pull_kv(self, peer_name: str, remote_descs: bytes, block_ids: Sequence[int],
                stream: Optional[torch.cuda.Stream] = None) -> bool:
        """The mirror image of :meth:`push_kv` (role of ``kv_worker.py:417-454``, NIXL "READ"):
        this GPU reads the blocks the peer's descriptor lists out of the peer's cache, over
        NVLink, into its own blocks ``block_ids``.  The kernel runs here, with plain loads from
        the mapped peer memory."""
        try:
            desc = CacheDescriptor.deserialize(remote_descs)
            try:
                pairs = build_push_pairs(block_ids, desc.block_ids)   # (local, remote)
            except ValueError as e:
                print(f"Creating transfer failed. {e}")
                return False
            with torch.cuda.device(self.device):
                peer = self._peers.get(peer_name)
                if peer is None:
                    peer = PeerCache(desc)
                    self._peers[peer_name] = peer
                if peer.num_layers != self.num_layers or peer.chunk_bytes != self.chunk_bytes:
                    print("Creating transfer failed. cache geometries differ")
                    return False
                table = np.ascontiguousarray(pairs[:, ::-1])              # (remote src, local dst)
                with torch.cuda.stream(stream or self.push_stream):
                    cache_ops.transfer_blocks(peer, self.gpu_kv_caches, table, pull=True)
            return True
        except _lib.LmsError as e:
            print(f"Posting transfer failed. {e}")
            return False

    def close(self) -> None:
        for p in self._peers.values():
            p.close()
        self._peers.clear()
        if self._disk_threads is not None:
            self._disk_threads.shutdown(wait=True)
            self._disk_threads = None
        if self.disk_kv_caches is not None:
            self.disk_kv_caches.flush()
            self.disk_kv_caches = None
        if self.host_pool is not None:
            self.host_pool.close()
            self.host_pool = None
