"""The cache side of one model step, in the order ``ModelWorker.execute`` runs it
(``runtime/worker/llm_worker/model_worker.py:507-528``): index preparation, copy-on-write of
diverging prefix blocks, the two handshake switches, and — from inside every attention layer —
the cache write of that layer's new K / V rows (``models/layers/attention.py:76-85``).

It owns nothing but a :class:`StepInputBuilder`; the cache belongs to the model, the events and
queues to the :class:`KVWorkerHandle`.  One difference from the reference, on purpose: the
copy-on-write is issued on the **model's stream**, ahead of the forward pass that reads the
copies (the reference issues it on the default stream and runs the model on another one, with
nothing ordering the two — ``model_worker.py:518-525``).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from .kv_worker import KVWorkerHandle
from .ops import cache_ops
from .step_inputs import StepIndices, StepInputBuilder


class ModelStepCache:
    """Drives the KV-cache operators of a model step.

    ``kv_caches``: the model's ``[L, num_blocks, 2, block_size, H, D]`` tensor;
    ``handle``: the model's end of the layer handshake (optional);
    ``stream``: the stream the forward pass runs on (default: the current stream at call time).
    """

    def __init__(self, kv_caches: torch.Tensor, handle: Optional[KVWorkerHandle] = None,
                 stream: Optional[torch.cuda.Stream] = None, max_batch: int = 256,
                 max_tokens: int = 8192, max_blocks: int = 65536):
        cache_ops._require_cuda("kv_caches", kv_caches)
        if kv_caches.dim() != 6 or kv_caches.shape[2] != 2:
            raise ValueError("kv_caches must be [L, num_blocks, 2, block_size, H, D]")
        self.kv_caches = kv_caches
        self.handle = handle
        self.stream = stream
        self.block_size = int(kv_caches.shape[3])
        self._layers = list(kv_caches.unbind(0))     # per-layer views, made once
        self.builder = StepInputBuilder(kv_caches.device, self.block_size, max_batch=max_batch,
                                        max_tokens=max_tokens, max_blocks=max_blocks)

    def _stream(self) -> torch.cuda.Stream:
        return self.stream or torch.cuda.current_stream(self.kv_caches.device)

    def begin_step(self, inputs: List, use_cache: bool = True, wait_before_execute: bool = False,
                   record_after_execute: bool = False,
                   blocks_to_copy: Optional[Dict[int, List[int]]] = None
                   ) -> Tuple[torch.Tensor, StepIndices]:
        """Everything ``execute`` does before it calls the model (``model_worker.py:515-522``):
        returns ``(input_ids, input_params)``; `inputs` is sorted in place as the reference
        sorts it.  ``wait_before_execute`` / ``record_after_execute`` switch the layer hooks of
        the handle for this step."""
        with torch.cuda.stream(self._stream()):
            input_ids, params = self.builder.make_inputs(inputs)
            if use_cache and blocks_to_copy:
                cache_ops.copy_blocks(self.kv_caches, blocks_to_copy)
        if self.handle is not None:
            self.handle.enable_wait_before_execute = bool(wait_before_execute)
            self.handle.enable_record_after_execute = bool(record_after_execute)
        return input_ids, params

    def write_layer(self, layer: int, key: torch.Tensor, value: torch.Tensor,
                    params: StepIndices) -> None:
        """The attention layer's cache write (``attention.py:76-85``): `key` / `value`
        ``[T, H, D]`` of this step's tokens go to the pages of ``kv_caches[layer]`` that the
        step's page table names.  Runs on the current stream."""
        cache_ops.append_paged_kv_cache(key, value, params.batch_indices, params.positions,
                                        self._layers[layer], params.kv_block_indices,
                                        params.kv_block_indptrs, params.kv_last_block_lens)
