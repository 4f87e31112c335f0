"""NumPy restatement of LMServe's KV-cache data-movement semantics (the checker).

All payloads are raw 16-bit words (``np.uint16``): the operations are byte
movement, so fp16 / bf16 never need interpreting and NaN patterns compare
exactly.  Every function mutates its destination in place, like the reference.
"""
from __future__ import annotations

from typing import List, Tuple

import numpy as np


def flatten_block_map(src_to_dst) -> np.ndarray:
    """``{src: [dst, ...]}`` -> int64 [n, 2], in dict order.

    Follows the launcher loop of ``ops/cache_ops.py:12-15``
    (``for src, dsts in src_to_dst.items(): for dst in dsts: block_maps += [src, dst]``).
    """
    if isinstance(src_to_dst, dict):
        flat: List[int] = []
        for src, dsts in src_to_dst.items():
            for dst in dsts:
                flat += [src, dst]
        return np.asarray(flat, dtype=np.int64).reshape(-1, 2)
    return np.asarray(src_to_dst, dtype=np.int64).reshape(-1, 2)


def fill_key_cache(key: np.ndarray, value: np.ndarray, key_cache: np.ndarray,
                   value_cache: np.ndarray, slot_mapping: np.ndarray) -> None:
    """``key_cache[slot[t]] = key[t]``, ``value_cache[slot[t]] = value[t]``.

    Follows ``fill_key_cache_kernel`` (``ops/triton/cache_kernels.py:39-58``): program
    ``t`` reads row ``t`` of key/value (``num_kv_heads*head_size`` elements) and stores it
    at ``slot*num_kv_heads*head_size`` in the flat caches.  The ``slot < 0`` skip is not
    in that kernel; it is the padding contract this build was specified with.
    ``key``/``value``: [T, H, D]; caches: any shape with ``num_slots*H*D`` elements.
    """
    T = key.shape[0]
    row = int(np.prod(key.shape[1:]))
    kc = key_cache.reshape(-1, row)
    vc = value_cache.reshape(-1, row)
    k = key.reshape(T, row)
    v = value.reshape(T, row)
    for t in range(T):
        slot = int(slot_mapping[t])
        if slot < 0:
            continue
        kc[slot, :] = k[t]
        vc[slot, :] = v[t]


def reshape_and_cache(key: np.ndarray, value: np.ndarray, kv_cache: np.ndarray,
                      slot_mapping: np.ndarray) -> None:
    """The same write into one layer's interleaved cache ``[NB, 2, BS, H, D]``.

    Addressing of the live call site ``models/layers/attention.py:76-85`` with the paged
    metadata of ``model_worker.py:399-433``: block = ``slot // BS``, entry = ``slot % BS``,
    K in plane 0, V in plane 1.
    """
    NB, two, BS = kv_cache.shape[:3]
    assert two == 2
    T = key.shape[0]
    row = int(np.prod(key.shape[1:]))
    c = kv_cache.reshape(NB, 2, BS, row)
    k = key.reshape(T, row)
    v = value.reshape(T, row)
    for t in range(T):
        slot = int(slot_mapping[t])
        if slot < 0:
            continue
        c[slot // BS, 0, slot % BS, :] = k[t]
        c[slot // BS, 1, slot % BS, :] = v[t]


def append_paged_kv_cache(append_key: np.ndarray, append_value: np.ndarray,
                          batch_indices: np.ndarray, positions: np.ndarray,
                          kv_cache: np.ndarray, kv_indices: np.ndarray,
                          kv_indptr: np.ndarray) -> None:
    """The live cache write of the reference, ``flashinfer.append_paged_kv_cache`` as called at
    ``models/layers/attention.py:76-85``.  flashinfer is a third-party dependency that is not
    part of the LMServe tree (``flashinfer-python`` 0.3.1.post1 in ``runtime/worker/uv.lock``);
    this restates its published algorithm (``AppendPagedKVCacheKernel``,
    ``include/flashinfer/page.cuh``): for appended row ``i``,
    ``page = indices[indptr[batch_indices[i]] + positions[i] // page_size]``,
    ``entry = positions[i] % page_size``, K row to ``cache[page, 0, entry]``, V row to
    ``cache[page, 1, entry]`` (NHD layout).  kv_cache: [num_pages, 2, page_size, H, D]."""
    NB, two, BS = kv_cache.shape[:3]
    assert two == 2
    T = append_key.shape[0]
    row = int(np.prod(append_key.shape[1:]))
    c = kv_cache.reshape(NB, 2, BS, row)
    k = append_key.reshape(T, row)
    v = append_value.reshape(T, row)
    for i in range(T):
        b, pos = int(batch_indices[i]), int(positions[i])
        if b < 0 or pos < 0:
            continue
        page = int(kv_indices[int(kv_indptr[b]) + pos // BS])
        c[page, 0, pos % BS, :] = k[i]
        c[page, 1, pos % BS, :] = v[i]


def reshape_and_cache_layers(key: np.ndarray, value: np.ndarray, kv_caches: np.ndarray,
                             slot_mapping: np.ndarray) -> None:
    """Per-layer loop of ``models/llama.py:236-242``: layer ``l`` writes ``key[l]`` into
    ``kv_caches[l]``; ``slot_mapping`` is [T] (shared) or [L, T]."""
    for l in range(kv_caches.shape[0]):
        s = slot_mapping if slot_mapping.ndim == 1 else slot_mapping[l]
        reshape_and_cache(key[l], value[l], kv_caches[l], s)


def copy_blocks(kv_caches: np.ndarray, src_to_dst) -> None:
    """``kv_caches[l, dst] = kv_caches[l, src]`` for every pair and every layer.

    Follows ``copy_blocks`` / ``copy_blocks_kernel`` (``ops/cache_ops.py:8-36``,
    ``ops/triton/cache_kernels.py:5-36``): grid ``(num_layers, n_pairs)``, each program
    copies ``numel_per_block`` elements.  The programs are unordered, so the result is
    defined only when destinations are distinct and no destination is also a source;
    the sources are therefore snapshotted first.
    """
    pairs = flatten_block_map(src_to_dst)
    if len(pairs) == 0:
        return
    L, NB = kv_caches.shape[:2]
    flat = kv_caches.reshape(L, NB, -1)
    snap = flat[:, pairs[:, 0], :].copy()
    flat[:, pairs[:, 1], :] = snap


def swap_out(gpu: np.ndarray, host: np.ndarray, pairs: np.ndarray,
             layers: Tuple[int, int] = None) -> None:
    """``host[dst, l] = gpu[l, src]`` — ``kv_worker.py:213-227`` (one DtoH copy of
    ``block_stride`` bytes per entry per layer).  gpu: [L, NB, chunk]; host: [NHB, L, chunk]."""
    L = gpu.shape[0]
    l0, l1 = (0, L) if layers is None else layers
    g = gpu.reshape(L, gpu.shape[1], -1)
    h = host.reshape(host.shape[0], L, -1)
    for l in range(l0, l1):
        for s, d in np.asarray(pairs, dtype=np.int64).reshape(-1, 2):
            h[d, l, :] = g[l, s, :]


def swap_in(gpu: np.ndarray, host: np.ndarray, pairs: np.ndarray,
            layers: Tuple[int, int] = None) -> None:
    """``gpu[l, dst] = host[src, l]`` — ``kv_worker.py:197-211``."""
    L = gpu.shape[0]
    l0, l1 = (0, L) if layers is None else layers
    g = gpu.reshape(L, gpu.shape[1], -1)
    h = host.reshape(host.shape[0], L, -1)
    for l in range(l0, l1):
        for s, d in np.asarray(pairs, dtype=np.int64).reshape(-1, 2):
            g[l, d, :] = h[s, l, :]


def transfer(src: np.ndarray, dst: np.ndarray, pairs: np.ndarray) -> None:
    """``dst[l, d] = src[l, s]`` for all layers — the end-to-end effect of
    ``kv_worker.py:358-415`` (whole blocks = all layers of a block are shipped, local
    block ``block_ids[i]`` to the i-th remote descriptor) once the surrounding
    write-through and fetch (``kv_worker.py:197-227``) are folded in."""
    L = src.shape[0]
    s_ = src.reshape(L, src.shape[1], -1)
    d_ = dst.reshape(L, dst.shape[1], -1)
    for s, d in np.asarray(pairs, dtype=np.int64).reshape(-1, 2):
        d_[:, d, :] = s_[:, s, :]
