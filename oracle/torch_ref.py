"""The same semantics as ``cache_oracle`` written with PyTorch index ops on CPU tensors.

This is the form the CPU baseline is timed in (``index_copy_`` / ``index_select`` with
all host threads), and a second, independently written checker.  Tensors are viewed as
int16 so that the comparison and the copies are on bits.  TEST / BENCH INFRASTRUCTURE ONLY.
"""
from __future__ import annotations

import torch


def _bits(t: torch.Tensor) -> torch.Tensor:
    return t.view(torch.int16) if t.element_size() == 2 and t.dtype != torch.int16 else t


def fill_key_cache(key, value, key_cache, value_cache, slot_mapping) -> None:
    """``ops/cache_ops.py:39-59`` as ``index_copy_``; negative slots are dropped first."""
    T = key.shape[0]
    row = key[0].numel()
    mask = slot_mapping >= 0
    idx = slot_mapping[mask].to(torch.int64)
    _bits(key_cache).view(-1, row).index_copy_(0, idx, _bits(key).reshape(T, row)[mask])
    _bits(value_cache).view(-1, row).index_copy_(0, idx, _bits(value).reshape(T, row)[mask])


def reshape_and_cache(key, value, kv_cache, slot_mapping) -> None:
    """Interleaved layer cache [NB, 2, BS, H, D] (``models/layers/attention.py:76-85``)."""
    NB, _, BS = kv_cache.shape[:3]
    T = key.shape[0]
    row = key[0].numel()
    mask = slot_mapping >= 0
    s = slot_mapping[mask].to(torch.int64)
    blk, ent = s // BS, s % BS
    flat = _bits(kv_cache).view(NB * 2 * BS, row)
    flat.index_copy_(0, (blk * 2 + 0) * BS + ent, _bits(key).reshape(T, row)[mask])
    flat.index_copy_(0, (blk * 2 + 1) * BS + ent, _bits(value).reshape(T, row)[mask])


def reshape_and_cache_layers(key, value, kv_caches, slot_mapping) -> None:
    for l in range(kv_caches.shape[0]):
        s = slot_mapping if slot_mapping.dim() == 1 else slot_mapping[l]
        reshape_and_cache(key[l], value[l], kv_caches[l], s)


def copy_blocks(kv_caches, pairs) -> None:
    """``ops/cache_ops.py:8-36`` as ``index_select`` + ``index_copy_`` on the block axis."""
    pairs = torch.as_tensor(pairs, dtype=torch.int64).reshape(-1, 2)
    if pairs.numel() == 0:
        return
    L, NB = kv_caches.shape[:2]
    flat = _bits(kv_caches).view(L, NB, -1)
    flat.index_copy_(1, pairs[:, 1], flat.index_select(1, pairs[:, 0]))


def swap_out(gpu, host, pairs, layers=None) -> None:
    """``kv_worker.py:213-227``: gpu [L, NB, chunk] -> host [NHB, L, chunk]."""
    pairs = torch.as_tensor(pairs, dtype=torch.int64).reshape(-1, 2)
    L = gpu.shape[0]
    l0, l1 = (0, L) if layers is None else layers
    g = _bits(gpu).view(L, gpu.shape[1], -1)
    h = _bits(host).view(host.shape[0], L, -1)
    picked = g[l0:l1].index_select(1, pairs[:, 0]).transpose(0, 1)
    h[:, l0:l1].index_copy_(0, pairs[:, 1], picked.contiguous())


def swap_in(gpu, host, pairs, layers=None) -> None:
    """``kv_worker.py:197-211``: host [NHB, L, chunk] -> gpu [L, NB, chunk]."""
    pairs = torch.as_tensor(pairs, dtype=torch.int64).reshape(-1, 2)
    L = gpu.shape[0]
    l0, l1 = (0, L) if layers is None else layers
    g = _bits(gpu).view(L, gpu.shape[1], -1)
    h = _bits(host).view(host.shape[0], L, -1)
    picked = h[:, l0:l1].index_select(0, pairs[:, 0]).transpose(0, 1)
    g[l0:l1].index_copy_(1, pairs[:, 1], picked.contiguous())


def transfer(src, dst, pairs) -> None:
    """Folded effect of ``kv_worker.py:358-415`` between two layer-major caches."""
    pairs = torch.as_tensor(pairs, dtype=torch.int64).reshape(-1, 2)
    L = src.shape[0]
    s = _bits(src).view(L, src.shape[1], -1)
    d = _bits(dst).view(L, dst.shape[1], -1)
    d.index_copy_(1, pairs[:, 1], s.index_select(1, pairs[:, 0]))
