"""Rotary position embedding with LMServe's signature, and its fusion with the cache write.

``rotary_pos_emb`` keeps the name, arguments and return value of
``runtime/worker/llm_worker/ops/rotary_embedding_ops.py:8-38``.  ``rotary_pos_emb_and_cache``
does the same rotation and, in the same launch, writes the rotated K and the V rows into one
layer's paged cache — the step that follows it in ``models/llama.py:156-167`` /
``models/layers/attention.py:76-85`` — so K is never materialised in between.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _lib
from .cache_ops import _OnDevice, _require_cuda, _slots_i64, _stream_ptr

_DTYPE_CODE = {torch.float16: 0, torch.bfloat16: 1}


def build_cos_sin_cache(max_position: int, head_dim: int, dtype: torch.dtype,
                        base: float = 10000.0, rope_scaling: Optional[dict] = None,
                        device=None) -> torch.Tensor:
    """The ``[max_position, 2 * head_dim]`` table (cos row, then sin row, of ``cat(freqs,
    freqs)``) that LMServe's ``RotaryEmbedding`` registers as ``cos_sin_cached``
    (``models/layers/rotary_embedding.py:27-71``), including the Llama-3 frequency rescaling
    when ``rope_scaling`` carries ``factor``, ``low_freq_factor``, ``high_freq_factor`` and
    ``original_max_position_embeddings``.  Computed in fp32 and cast once, as there."""
    import math
    inv_freq = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.int64).float() / head_dim))
    if rope_scaling is not None:
        factor = rope_scaling["factor"]
        low, high = rope_scaling["low_freq_factor"], rope_scaling["high_freq_factor"]
        old_len = rope_scaling["original_max_position_embeddings"]
        wavelen = 2 * math.pi / inv_freq
        scaled = torch.where(wavelen > old_len / low, inv_freq / factor, inv_freq)
        smooth = (old_len / wavelen - low) / (high - low)
        blended = (1 - smooth) * inv_freq / factor + smooth * inv_freq
        medium = ~(wavelen < old_len / high) & ~(wavelen > old_len / low)
        inv_freq = torch.where(medium, blended, scaled)
    t = torch.arange(max_position).float()
    freqs = torch.einsum("i,j->ij", t, inv_freq.float())
    emb = torch.cat((freqs, freqs), dim=-1)
    table = torch.cat((emb.cos().to(dtype), emb.sin().to(dtype)), dim=-1)
    return table if device is None else table.to(device)


def _check_inputs(query, key, positions, cos_sin_cache, head_dim):
    for n, t in (("query", query), ("key", key), ("positions", positions),
                 ("cos_sin_cache", cos_sin_cache)):
        _require_cuda(n, t)
    if query.dtype not in _DTYPE_CODE:
        raise TypeError(f"rotary embedding supports fp16 and bf16, got {query.dtype}")
    if key.dtype != query.dtype or cos_sin_cache.dtype != query.dtype:
        raise TypeError("query, key and cos_sin_cache must share one dtype")
    if query.dim() != 2 or key.dim() != 2 or query.shape[0] != key.shape[0]:
        raise ValueError("query and key must be [num_tokens, heads * head_dim]")
    if query.shape[1] % head_dim or key.shape[1] % head_dim:
        raise ValueError("hidden sizes must be multiples of head_dim")
    if cos_sin_cache.dim() != 2 or cos_sin_cache.shape[1] != 2 * head_dim:
        raise ValueError("only the full rotary dimension is supported: cos_sin_cache must be "
                         "[max_position, 2 * head_dim]")
    if query.stride(1) != 1 or key.stride(1) != 1 or cos_sin_cache.stride(1) != 1:
        raise ValueError("the last dimension of query, key and cos_sin_cache must be dense")
    if positions.dtype not in (torch.int32, torch.int64) or positions.numel() != query.shape[0]:
        raise TypeError("positions must be int32 or int64 with one entry per token")


_ARITHMETIC = {"compiled": _lib.LMS_ROPE_CONTRACTED, "round_each": _lib.LMS_ROPE_ROUND_EACH}


def _launch(query, key, value, positions, cos_sin_cache, head_dim, q_out, k_out, kv_cache, slots,
            arithmetic="compiled"):
    if arithmetic not in _ARITHMETIC:
        raise ValueError(f"arithmetic must be 'compiled' or 'round_each', got {arithmetic!r}")
    dev = query.device
    es = query.element_size()
    T = query.shape[0]
    nh, nkv = query.shape[1] // head_dim, key.shape[1] // head_dim
    positions = positions.contiguous()
    if kv_cache is not None:
        NB, _, BS, H, D = kv_cache.shape
        kptr = kv_cache.data_ptr()
        vptr = kptr + BS * H * D * es
        block_stride, slot_stride = kv_cache.stride(0) * es, H * D * es
        vp, vs, sp, ns = value.data_ptr(), value.stride(0) * es, slots.data_ptr(), NB * BS
    else:
        kptr = vptr = vp = sp = None
        block_stride = slot_stride = vs = ns = BS = 0
    with _OnDevice(dev):
        _lib.check(_lib.lib().lms_rope_and_cache(
            query.data_ptr(), key.data_ptr(), vp, query.stride(0) * es, key.stride(0) * es, vs,
            positions.data_ptr(), 1 if positions.dtype == torch.int64 else 0,
            cos_sin_cache.data_ptr(), cos_sin_cache.stride(0) * es,
            q_out.data_ptr(), q_out.stride(0) * es,
            k_out.data_ptr() if k_out is not None else None,
            k_out.stride(0) * es if k_out is not None else 0,
            kptr, vptr, block_stride, slot_stride, sp, T, nh, nkv, head_dim,
            _DTYPE_CODE[query.dtype], _ARITHMETIC[arithmetic], BS, ns, cos_sin_cache.shape[0],
            _stream_ptr(dev)))


def rotary_pos_emb(query: torch.Tensor, key: torch.Tensor, positions: torch.Tensor,
                   cos_sin_cache: torch.Tensor, head_dim: int,
                   arithmetic: str = "compiled") -> Tuple[torch.Tensor, torch.Tensor]:
    """``(q_out, k_out)``: query ``[T, num_heads*head_dim]`` and key ``[T, num_kv_heads*head_dim]``
    rotated by ``cos_sin_cache[positions]`` — LMServe's ``rotary_pos_emb``.

    ``arithmetic="compiled"`` (default) rounds as the Triton compiler's GPU code for the
    reference kernel does (the first product of ``x*cos - y*sin`` and of ``y*cos + x*sin`` fused
    into the sum), i.e. it returns what the reference returns when it runs on a GPU;
    ``"round_each"`` rounds every product and sum, the Triton language semantics (and the result
    of the Triton interpreter).  The two differ by one unit in the last place in about a quarter
    of the elements."""
    _check_inputs(query, key, positions, cos_sin_cache, head_dim)
    q_out = torch.empty_like(query, memory_format=torch.contiguous_format)
    k_out = torch.empty_like(key, memory_format=torch.contiguous_format)
    if query.shape[0]:
        _launch(query, key, None, positions, cos_sin_cache, head_dim, q_out, k_out, None, None,
                arithmetic)
    return q_out, k_out


def rotary_pos_emb_and_cache(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                             positions: torch.Tensor, cos_sin_cache: torch.Tensor, head_dim: int,
                             kv_cache: torch.Tensor, slot_mapping: torch.Tensor,
                             return_key: bool = False, arithmetic: str = "compiled"):
    """Rotates ``query`` (returned) and ``key``, and writes rotated K and ``value`` into
    ``kv_cache`` (one layer, ``[num_blocks, 2, block_size, H, D]``) at ``slot_mapping`` in the same
    launch.  ``slot_mapping[t] < 0`` skips the cache write of token ``t``.  With
    ``return_key=True`` the rotated key is returned as well (``(q_out, k_out)``), for callers
    that still need it outside the cache.  ``arithmetic`` as in :func:`rotary_pos_emb`."""
    _check_inputs(query, key, positions, cos_sin_cache, head_dim)
    _require_cuda("value", value)
    _require_cuda("kv_cache", kv_cache)
    if value.shape != key.shape or value.dtype != key.dtype or value.stride(1) != 1:
        raise ValueError("value must match key in shape, dtype and layout")
    if kv_cache.dim() != 5 or kv_cache.shape[1] != 2 or kv_cache.dtype != key.dtype:
        raise ValueError("kv_cache must be one layer [num_blocks, 2, block_size, H, D] of the key dtype")
    NB, _, BS, H, D = kv_cache.shape
    if D != head_dim or H * D != key.shape[1]:
        raise ValueError("kv_cache heads do not match key")
    if NB and not kv_cache[0].is_contiguous():
        raise ValueError("each cache block must be contiguous")
    slots = _slots_i64(slot_mapping, query.device)
    if slots.numel() != query.shape[0]:
        raise ValueError("slot_mapping must have one entry per token")
    q_out = torch.empty_like(query, memory_format=torch.contiguous_format)
    k_out = torch.empty_like(key, memory_format=torch.contiguous_format) if return_key else None
    if query.shape[0]:
        _launch(query, key, value, positions, cos_sin_cache, head_dim, q_out, k_out, kv_cache, slots,
                arithmetic)
    return (q_out, k_out) if return_key else q_out
