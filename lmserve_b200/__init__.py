"""B200-native KV-cache data movement for LMServe's paged cache.

``lmserve_b200.ops`` mirrors ``llm_worker.ops`` (``copy_blocks``,
``fill_key_cache`` and the paged/interleaved ``reshape_and_cache``);
``lmserve_b200.kv_worker`` mirrors ``llm_worker.kv_worker`` (swap, push / pull, cache
allocation and the per-layer event + queue handshake), ``lmserve_b200.host_topology`` the
CPU-affinity helper of ``llm_worker.utils``, ``lmserve_b200.step_inputs`` the per-step index
preparation of ``ModelWorker._make_inputs``, ``lmserve_b200.kv_service`` the ``worker.KVWorker``
gRPC service; ``lmserve_b200.torch_ops`` registers the operators as ``torch.ops.lmserve_cache.*``.
All device work is done by ``liblmserve_kv.so`` (C ABI: ``include/lmserve_kv.h``); there is no
CPU fallback.
"""
from . import _lib
from .ops import (copy_blocks, fill_key_cache, reshape_and_cache,
                  reshape_and_cache_layers, swap_blocks, transfer_blocks, PagedWritePlan, WritePlan)

__version__ = "0.2.0"

__all__ = ["copy_blocks", "fill_key_cache", "reshape_and_cache",
           "reshape_and_cache_layers", "swap_blocks", "transfer_blocks", "PagedWritePlan", "WritePlan",
           "_lib"]
