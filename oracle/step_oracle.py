"""CPU restatement of LMServe's per-step index preparation.  TEST INFRASTRUCTURE ONLY.

Follows ``ModelWorker._make_inputs`` (``runtime/worker/llm_worker/model_worker.py:310-433``) line
by line in NumPy, and restates the two flashinfer helpers it calls from their published
definitions (flashinfer-python, pinned at 0.3.1.post1 by the reference's lock file;
``flashinfer/page.py`` ``get_seq_lens`` and ``get_batch_indices_positions``):

    seq_lens      = clamp(indptr[1:] - indptr[:-1] - 1, min=0) * page_size + last_page_len
    batch_indices = request index of every appended token
    positions     = seq_lens[b] - (append_indptr[b+1] - append_indptr[b]) + offset in the request

Pins: the worked example in the ``get_batch_indices_positions`` documentation and vectors made
by flashinfer's own functions on a B200 (``tests/golden/step_indices_flashinfer.npz``), both
checked in the CPU tests; on a GPU box the installed flashinfer functions are called as well.  The slot
mapping is this build's addition: ``block_ids[pos // BS] * BS + pos % BS`` per request.
"""
from __future__ import annotations

from typing import Dict, List

import numpy as np


def get_seq_lens(kv_indptr: np.ndarray, kv_last_page_len: np.ndarray, page_size: int) -> np.ndarray:
    return np.maximum(kv_indptr[1:] - kv_indptr[:-1] - 1, 0) * page_size + kv_last_page_len


def get_batch_indices_positions(append_indptr: np.ndarray, seq_lens: np.ndarray, nnz: int):
    batch_indices = np.full(nnz, -1, dtype=np.int32)
    positions = np.zeros(nnz, dtype=np.int32)
    for b in range(len(append_indptr) - 1):
        lo, hi = int(append_indptr[b]), int(append_indptr[b + 1])
        batch_indices[lo:hi] = b
        positions[lo:hi] = np.arange(hi - lo) + int(seq_lens[b]) - (hi - lo)
    return batch_indices, positions


def make_inputs(inputs: List, page_size: int) -> Dict[str, np.ndarray]:
    """`_make_inputs` on the host: sorts `inputs` in place, returns every index array by name."""
    flatten_input_ids: List[int] = []
    position_ids: List[int] = []
    prefill_input_len = 0
    seqlens_q: List[int] = []
    inputs.sort(key=lambda x: -x.input_len)                       # model_worker.py:328
    for data in inputs:                                           # :330-350
        cache_seqlen = data.filled_token_len
        seqlen_q = data.input_len
        if seqlen_q > 1:
            prefill_input_len += seqlen_q
        seqlen_k = data.context_len
        flatten_input_ids += list(data.input_ids)
        position_ids += [i for i in range(cache_seqlen, seqlen_k)]
        seqlens_q.append(seqlen_q)
    cu_seqlens_q = np.cumsum([0] + seqlens_q).astype(np.int32)    # :362-365

    kv_block_indices: List[int] = []
    num_blocks_per_seqs: List[int] = []
    kv_last_block_lens: List[int] = []
    for data in inputs:                                           # :399-407
        seqlen_k = data.context_len
        kv_block_indices += list(data.block_ids)
        num_blocks_per_seqs.append(len(data.block_ids))
        kv_last_block_lens.append((seqlen_k - 1) % page_size + 1)
    kv_block_indptrs = np.cumsum([0] + num_blocks_per_seqs).astype(np.int32)
    kv_block_indices_a = np.asarray(kv_block_indices, dtype=np.int32)
    kv_last_block_lens_a = np.asarray(kv_last_block_lens, dtype=np.int32)

    nnz = int(sum(seqlens_q))
    batch_indices, positions = get_batch_indices_positions(       # :425-433
        cu_seqlens_q, get_seq_lens(kv_block_indptrs, kv_last_block_lens_a, page_size), nnz)

    slot_mapping = np.full(nnz, -1, dtype=np.int64)
    for i in range(nnz):
        b, pos = int(batch_indices[i]), int(positions[i])
        nb = int(kv_block_indptrs[b + 1] - kv_block_indptrs[b])
        if pos >= 0 and pos // page_size < nb:
            blk = int(kv_block_indices_a[kv_block_indptrs[b] + pos // page_size])
            slot_mapping[i] = blk * page_size + pos % page_size

    return {
        "input_ids": np.asarray(flatten_input_ids, dtype=np.int64),
        "position_ids": np.asarray(position_ids, dtype=np.int32),
        "cu_seqlens_q": cu_seqlens_q,
        "prefill_input_len": prefill_input_len,
        "kv_block_indices": kv_block_indices_a,
        "kv_block_indptrs": kv_block_indptrs,
        "kv_last_block_lens": kv_last_block_lens_a,
        "batch_indices": batch_indices,
        "positions": positions,
        "slot_mapping": slot_mapping,
    }
