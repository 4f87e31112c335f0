"""The cache operators as PyTorch custom ops: ``torch.ops.lmserve_cache.*``.

Importing this module registers, with ``torch.library.custom_op``, in-place operators that
declare which argument they mutate, so code that goes through the dispatcher (tracing, CUDA
graph capture through ``torch.cuda.graph``, functionalisation) sees the cache write as a
mutation of the cache and nothing else:

    lmserve_cache::reshape_and_cache(key, value, kv_cache, slot_mapping)            kv_cache mutated
    lmserve_cache::reshape_and_cache_layers(key, value, kv_caches, slot_mapping)    kv_caches mutated
    lmserve_cache::copy_blocks(kv_caches, block_pairs)                              kv_caches mutated
    lmserve_cache::swap_blocks(gpu_kv_caches, host_pool, block_pairs, direction,
                               layer_begin, layer_end)                     both buffers declared mutated
    lmserve_cache::transfer_blocks(src_kv_caches, dst_kv_caches, block_pairs)       dst mutated

They are thin: each one calls the wrapper of the same name in ``lmserve_b200.ops.cache_ops``,
which calls the C ABI.  ``block_pairs`` is an int64 ``[n, 2]`` tensor of (source, destination)
block numbers, on the cache's device or on the host — the flattened form of LMServe's
``src_to_dst`` dict (``llm_worker/ops/cache_ops.py:12-24``) and of ``BlockMapping.entries``
(``proto/worker.proto:78-86``).  ``host_pool`` is the ``[num_host_blocks, L, chunk_bytes]`` uint8
tensor of a :class:`lmserve_b200.kv_worker.HostPool` (``pool.tensor``) or any pinned CPU tensor of
that shape.  There is no CPU implementation: CPU caches raise.
"""
from __future__ import annotations

from types import SimpleNamespace

from torch import Tensor
from torch.library import custom_op

from .ops import cache_ops


def _pool_view(host_pool: Tensor):
    if host_pool.is_cuda or host_pool.dim() != 3 or host_pool.element_size() != 1 or not host_pool.is_contiguous():
        raise ValueError("host_pool must be a contiguous CPU byte tensor [num_host_blocks, L, chunk_bytes]")
    ptr = host_pool.data_ptr()
    dev_ptr = cache_ops.HOST_POOL_DEVICE_PTR.get(ptr)
    if dev_ptr is None:
        if not host_pool.is_pinned():
            raise RuntimeError("host_pool must be page-locked: use HostPool(...).tensor or a pinned tensor")
        dev_ptr = ptr  # pinned by the CUDA allocator: one address on both sides
    nhb, layers, chunk = host_pool.shape
    return SimpleNamespace(num_blocks=nhb, num_layers=layers, chunk_bytes=chunk, device_ptr=dev_ptr,
                           layer_stride=chunk, block_stride=layers * chunk)


@custom_op("lmserve_cache::reshape_and_cache", mutates_args=("kv_cache",))
def reshape_and_cache(key: Tensor, value: Tensor, kv_cache: Tensor, slot_mapping: Tensor) -> None:
    cache_ops.reshape_and_cache(key, value, kv_cache, slot_mapping)


@custom_op("lmserve_cache::reshape_and_cache_layers", mutates_args=("kv_caches",))
def reshape_and_cache_layers(key: Tensor, value: Tensor, kv_caches: Tensor, slot_mapping: Tensor) -> None:
    cache_ops.reshape_and_cache_layers(key, value, kv_caches, slot_mapping)


@custom_op("lmserve_cache::copy_blocks", mutates_args=("kv_caches",))
def copy_blocks(kv_caches: Tensor, block_pairs: Tensor) -> None:
    cache_ops.copy_blocks(kv_caches, block_pairs)


@custom_op("lmserve_cache::swap_blocks", mutates_args=("gpu_kv_caches", "host_pool"))
def swap_blocks(gpu_kv_caches: Tensor, host_pool: Tensor, block_pairs: Tensor, direction: str,
                layer_begin: int, layer_end: int) -> None:
    cache_ops.swap_blocks(gpu_kv_caches, _pool_view(host_pool), block_pairs, direction,
                          layers=(layer_begin, layer_end))


@custom_op("lmserve_cache::transfer_blocks", mutates_args=("dst_kv_caches",))
def transfer_blocks(src_kv_caches: Tensor, dst_kv_caches: Tensor, block_pairs: Tensor) -> None:
    cache_ops.transfer_blocks(src_kv_caches, dst_kv_caches, block_pairs)


for _op in (reshape_and_cache, reshape_and_cache_layers, copy_blocks, swap_blocks, transfer_blocks):
    _op.register_fake(lambda *args, **kwargs: None)

OPS = ("reshape_and_cache", "reshape_and_cache_layers", "copy_blocks", "swap_blocks", "transfer_blocks")
