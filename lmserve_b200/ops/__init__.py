"""Host-side mirror of LMServe's ``llm_worker.ops`` cache operators."""
from .cache_ops import (append_paged_kv_cache, copy_blocks, copy_blocks_no_alloc, fill_key_cache, reshape_and_cache,
                        reshape_and_cache_layers, swap_blocks, transfer_blocks,
                        flatten_block_map, PagedWritePlan, WritePlan)

from .rotary_embedding_ops import build_cos_sin_cache, rotary_pos_emb, rotary_pos_emb_and_cache

__all__ = ["build_cos_sin_cache", "rotary_pos_emb", "rotary_pos_emb_and_cache", "append_paged_kv_cache", "copy_blocks", "copy_blocks_no_alloc", "fill_key_cache", "reshape_and_cache",
           "reshape_and_cache_layers", "swap_blocks", "transfer_blocks",
           "flatten_block_map", "PagedWritePlan", "WritePlan"]
