"""Runs LMServe's own ``KVWorker`` swap and transfer code on CPU buffers.

``runtime/worker/llm_worker/kv_worker.py`` is plain Python around three foreign libraries:
pycuda (two async memcpys, streams, events), NIXL (host-to-host block transfer) and the
generated protobuf module.  None of them is installable here, and none of them does
arithmetic: they move bytes between addresses the Python code computes.  This module loads
the file by path with stand-ins for those three in ``sys.modules`` and calls the reference's
own methods, so the address arithmetic, the layer loops, the descriptor truncation and the
block-major host layout that are exercised are the reference's, not a restatement:

* ``pycuda.driver.memcpy_dtoh_async(dst_ndarray, src_ptr, stream)`` and
  ``memcpy_htod_async(dst_ptr, src_ndarray, stream)`` become ``ctypes.memmove`` of
  ``ndarray.nbytes`` bytes — the "GPU" cache is a host array whose addresses play the device
  pointers of ``gpu_kv_cache_ptrs`` (``kv_worker.py:112-115``);
* the NIXL agent keeps (address, length) descriptors of the tensors it is given and its
  ``transfer`` copies local -> remote for ``"WRITE"`` and remote -> local for ``"READ"``,
  descriptor by descriptor (the documented meaning of ``initialize_xfer``);
* ``BlockMapping`` / ``Device`` are small Python classes with the fields of
  ``proto/worker.proto:13-17,78-91``.

Only usable where the LMServe tree is present (``LMSERVE_SRC`` or a ``reference`` directory
next to this repository).  ``tests/golden/make_swap_golden.py`` uses it to produce the
committed swap / transfer vectors.  TEST INFRASTRUCTURE ONLY.
"""
from __future__ import annotations

import asyncio
import ctypes
import enum
import importlib.util
import json
import queue
import sys
import types
from dataclasses import dataclass, field
from typing import List

import numpy as np

from .triton_ref import reference_root

KV_WORKER_FILE = "runtime/worker/llm_worker/kv_worker.py"


def available() -> bool:
    return (reference_root() / KV_WORKER_FILE).exists()


# ----------------------------------------------------------------------------- stand-ins

class _Stream:
    def synchronize(self):
        pass

    def wait_for_event(self, event):
        event.waited += 1


class _Event:
    def __init__(self):
        self.recorded = 0
        self.waited = 0

    def record(self, stream=None):
        self.recorded += 1


def _memcpy_dtoh_async(dst: np.ndarray, src_ptr: int, stream=None) -> None:
    assert dst.flags["C_CONTIGUOUS"]
    ctypes.memmove(dst.ctypes.data, int(src_ptr), dst.nbytes)


def _memcpy_htod_async(dst_ptr: int, src: np.ndarray, stream=None) -> None:
    assert src.flags["C_CONTIGUOUS"]
    ctypes.memmove(int(dst_ptr), src.ctypes.data, src.nbytes)


class Device(enum.IntEnum):
    """``enum Device`` of ``proto/worker.proto:13-17``."""
    GPU = 0
    Host = 1
    Disk = 2


@dataclass
class BlockMappingEntry:
    src_block_id: int
    dst_block_id: int


@dataclass
class BlockMapping:
    entries: List[BlockMappingEntry] = field(default_factory=list)


class _DescList:
    def __init__(self, descs):
        self.descs = list(descs)          # (address, nbytes)

    def descCount(self):
        return len(self.descs)

    def remDesc(self, i):
        del self.descs[i]


class _XferHandle:
    def __init__(self, op, local, remote):
        self.op, self.local, self.remote = op, local, remote


class FakeNixlAgent:
    """Same-process stand-in for ``nixl._api.nixl_agent``: "remote" memory is addressable."""

    def __init__(self, name="agent", config=None):
        self.name = name
        self.transfers = 0

    def create_backend(self, *a, **k):
        pass

    def register_memory(self, tensor, backends=None):
        return True

    def deregister_memory(self, desc):
        pass

    def get_agent_metadata(self):
        return self.name.encode()

    def get_xfer_descs(self, tensors):
        return _DescList((t.data_ptr(), t.numel() * t.element_size()) for t in tensors)

    def get_serialized_descs(self, descs) -> bytes:
        return json.dumps(descs.descs).encode()

    def deserialize_descs(self, blob: bytes):
        return _DescList(tuple(d) for d in json.loads(bytes(blob).decode()))

    def initialize_xfer(self, op, local, remote, peer_name, notif=b""):
        if op not in ("WRITE", "READ") or local.descCount() != remote.descCount():
            return None
        if any(a[1] != b[1] for a, b in zip(local.descs, remote.descs)):
            return None
        return _XferHandle(op, local, remote)

    def transfer(self, handle):
        for (la, ln), (ra, _) in zip(handle.local.descs, handle.remote.descs):
            if handle.op == "WRITE":
                ctypes.memmove(ra, la, ln)
            else:
                ctypes.memmove(la, ra, ln)
        self.transfers += 1
        return "DONE"

    def check_xfer_state(self, handle):
        return "DONE"


class _TorchWithoutCuda:
    cuda = types.SimpleNamespace(ipc_collect=lambda: None, empty_cache=lambda: None)

    def __getattr__(self, name):
        import torch
        return getattr(torch, name)


_module = None


def load_reference_module():
    """Import the reference's ``kv_worker.py`` by path with the stand-ins in place."""
    global _module
    if _module is not None:
        return _module
    saved = {k: sys.modules.get(k) for k in
             ("pycuda", "pycuda.driver", "nixl", "nixl._api", "llm_worker", "llm_worker.pb",
              "llm_worker.pb.worker_pb2")}
    drv = types.ModuleType("pycuda.driver")
    drv.Event, drv.Stream = _Event, _Stream
    drv.memcpy_dtoh_async, drv.memcpy_htod_async = _memcpy_dtoh_async, _memcpy_htod_async
    pycuda = types.ModuleType("pycuda")
    pycuda.driver = drv
    nixl_api = types.ModuleType("nixl._api")
    nixl_api.nixl_agent = FakeNixlAgent
    nixl_api.nixl_agent_config = lambda **k: None
    nixl = types.ModuleType("nixl")
    nixl._api = nixl_api
    pb2 = types.ModuleType("llm_worker.pb.worker_pb2")
    pb2.BlockMapping, pb2.Device = BlockMapping, Device
    pb = types.ModuleType("llm_worker.pb")
    pb.worker_pb2 = pb2
    pkg = types.ModuleType("llm_worker")
    pkg.pb = pb
    stubs = {"pycuda": pycuda, "pycuda.driver": drv, "nixl": nixl, "nixl._api": nixl_api,
             "llm_worker": pkg, "llm_worker.pb": pb, "llm_worker.pb.worker_pb2": pb2}
    sys.modules.update(stubs)
    try:
        spec = importlib.util.spec_from_file_location(
            "lmserve_ref_kv_worker", reference_root() / KV_WORKER_FILE)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    finally:
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v
    # the destructor (``kv_worker.py:456-464``) calls torch.cuda.ipc_collect / empty_cache, which
    # need a CUDA runtime; nothing else in the module touches torch.cuda after import
    mod.torch = _TorchWithoutCuda()
    _module = mod
    return mod


# ------------------------------------------------------------------ a worker on CPU buffers

class RefWorker:
    """An instance of the reference ``KVWorker`` whose attributes are set the way its
    ``__init__`` sets them (``kv_worker.py:108-195``), minus the CUDA-IPC mapping of the cache
    and the pinned allocation: ``gpu`` [L, NB, chunk_words] and ``host`` [NHB, L, chunk_words]
    are host arrays of 16-bit words owned by the caller.  Every method called afterwards is the
    reference's own."""

    def __init__(self, gpu: np.ndarray, host: np.ndarray, name: str = "kv"):
        import torch
        mod = load_reference_module()
        assert gpu.flags["C_CONTIGUOUS"] and host.flags["C_CONTIGUOUS"]
        L, NB, words = gpu.shape
        assert host.shape[1:] == (L, words)
        w = object.__new__(mod.KVWorker)
        w.gpu_kv_caches = gpu
        w.gpu_kv_cache_ptrs = [gpu[l].ctypes.data for l in range(L)]          # :112-115
        w.host_kv_caches = host                                              # :129
        w.host_kv_caches_tensor = torch.from_numpy(host.view(np.int16))     # :130
        w.disk_kv_caches = None
        self.kv_queue, self.model_queue = queue.Queue(), queue.Queue()
        w.kv_worker_handle = mod.KVWorkerHandle(
            [_Event() for _ in range(L)], [_Event() for _ in range(L)],
            self.model_queue, self.kv_queue)                                 # :149-154
        w.num_layers = L                                                     # :156
        w.block_stride = words * gpu.itemsize                                # :157
        w.dtoh_stream, w.htod_stream = _Stream(), _Stream()                  # :159-160
        w.kv_agent = FakeNixlAgent(name)
        w.kv_agent_name = name
        w.reg_desc = True
        w.ctx = types.SimpleNamespace(pop=lambda: None)                      # :117, for __del__
        w.COPY_KV_OP_MAP = {                                                 # :190-195
            (Device.GPU, Device.Host): w._copy_kv_gpu_to_host,
            (Device.Host, Device.GPU): w._copy_kv_host_to_gpu,
            (Device.Host, Device.Disk): w._copy_kv_host_to_disk,
            (Device.Disk, Device.Host): w._copy_kv_disk_to_host,
        }
        self.worker, self.mod = w, mod

    @staticmethod
    def mappings(pairs, split: int = 0) -> List[BlockMapping]:
        """[n, 2] (src, dst) -> the ``List[BlockMapping]`` the Rust side sends; ``split`` > 0
        spreads the entries over several mappings, as several sequences in one request do."""
        p = [BlockMappingEntry(int(s), int(d)) for s, d in np.asarray(pairs).reshape(-1, 2)]
        if not p:
            return []
        if split <= 0:
            return [BlockMapping(p)]
        return [BlockMapping(p[i:i + split]) for i in range(0, len(p), split)]

    def swap_out(self, pairs, split: int = 0) -> None:
        """``copy_kv(mappings, GPU, Host)`` (``kv_worker.py:336-346`` -> ``:272-295``).  The
        model's per-layer tokens are put on the queue first, as ``model_worker.py:272-276``
        does after each layer."""
        for _ in range(self.worker.num_layers):
            self.kv_queue.put(b"")
        asyncio.run(self.worker.copy_kv(self.mappings(pairs, split), Device.GPU, Device.Host))

    def swap_in(self, pairs, split: int = 0) -> None:
        """``copy_kv(mappings, Host, GPU)`` (``kv_worker.py:249-270``)."""
        asyncio.run(self.worker.copy_kv(self.mappings(pairs, split), Device.Host, Device.GPU))

    def save_layer(self, pairs, layer: int) -> None:
        for m in self.mappings(pairs):
            self.worker._save_layer_kv_blocks_to_host(m, layer, self.worker.dtoh_stream)

    def load_layer(self, pairs, layer: int) -> None:
        for m in self.mappings(pairs):
            self.worker._load_layer_kv_blocks_from_host(m, layer, self.worker.htod_stream)

    def get_descriptors(self, block_ids) -> bytes:
        return self.worker.get_descriptors([int(b) for b in block_ids])

    def push(self, remote_descs: bytes, block_ids) -> bool:
        return self.worker._push_kv("peer", remote_descs, [int(b) for b in block_ids])

    def pull(self, remote_descs: bytes, block_ids) -> bool:
        return asyncio.run(self.worker.pull_kv("peer", remote_descs, [int(b) for b in block_ids]))


def disaggregated_push(prefill: RefWorker, decode: RefWorker, src_gpu_blocks, dst_gpu_blocks,
                       prefill_host_blocks, decode_host_blocks, surplus_host_blocks=()) -> bool:
    """The whole prefill -> decode hand-over as the Rust engine drives it
    (``runtime/src/.../worker.rs:434-453,494-519``): write-through of the finished blocks to the
    prefill host pool, descriptors of the host blocks the decode side reserved (possibly more
    than needed), NIXL WRITE, fetch into the decode GPU's blocks."""
    prefill.swap_out(np.stack([src_gpu_blocks, prefill_host_blocks], axis=1))
    descs = decode.get_descriptors(list(decode_host_blocks) + list(surplus_host_blocks))
    ok = prefill.push(descs, prefill_host_blocks)
    decode.swap_in(np.stack([decode_host_blocks, dst_gpu_blocks], axis=1))
    return ok
