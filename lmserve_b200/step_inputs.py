"""Per-step index preparation: the host mirror of ``ModelWorker._make_inputs``.

LMServe's model worker turns the scheduler's request list into about ten small CUDA tensors per
step, each built from a Python list and uploaded on its own
(``runtime/worker/llm_worker/model_worker.py:310-433``; fields of the result:
``llm_worker/models/input_params.py:10-22``).  `StepInputBuilder.make_inputs` takes the same
request objects (anything with the ``InferInput`` fields of ``proto/worker.proto:40-47``:
``input_ids, input_len, filled_token_len, context_len, block_ids``), packs four numbers per
request, the concatenated block tables and the token ids into ONE pinned int32 buffer, uploads it
with one asynchronous copy and lets one kernel (``lms_build_step_indices``) derive every index
tensor on the device, including the slot mapping the cache-write kernels take.  Field names of
the result are those of ``InputParams``; the attention wrappers (``prefill_wrapper`` /
``decode_wrapper``) are attention planning and are not built here.

Ordering follows the reference: requests are sorted in place by descending ``input_len``
(``model_worker.py:328``, a stable sort), so prefill requests come first.
"""
from __future__ import annotations

from dataclasses import dataclass
from itertools import chain
from operator import attrgetter
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import _lib
from .ops.cache_ops import _OnDevice, _stream_ptr

from .ops.cache_ops import _packer  # the C packer (csrc/packer.c); its absence is an ImportError

_INPUT_LEN = attrgetter("input_len")

MAX_BATCH = 4096  # LMS_STEP_MAX_BATCH


@dataclass
class InferInput:
    """The fields of ``worker.InferInput`` (``proto/worker.proto:40-47``) this path reads."""
    input_ids: Sequence[int]
    input_len: int
    filled_token_len: int
    context_len: int
    block_ids: Sequence[int]
    seq_id: int = 0


@dataclass
class PagedArrays:
    """The arrays one flashinfer attention plan takes (``prefill_wrapper.plan`` /
    ``decode_wrapper.plan``, ``model_worker.py:68-79,126-137``) for one phase of the batch."""
    qo_indptr: Optional[torch.Tensor]      # int32 [n + 1]; None for decode (one token per request)
    kv_indptr: torch.Tensor                # int32 [n + 1], starting at 0
    kv_indices: torch.Tensor               # int32
    kv_last_page_len: torch.Tensor         # int32 [n]


@dataclass
class StepIndices:
    """Index tensors of one step; names as in ``InputParams`` plus ``slot_mapping``."""
    position_ids: torch.Tensor        # int32 [T]
    cu_seqlens_q: torch.Tensor        # int32 [B + 1]
    prefill_input_len: int
    batch_indices: torch.Tensor       # int32 [T]
    positions: torch.Tensor           # int32 [T]
    kv_block_indices: torch.Tensor    # int32 [sum of table lengths]
    kv_block_indptrs: torch.Tensor    # int32 [B + 1]
    kv_last_block_lens: torch.Tensor  # int32 [B]
    slot_mapping: torch.Tensor        # int64 [T]
    num_prefill: int = 0
    num_decode: int = 0
    # the same page table split by phase, as the reference rebuilds it for its two attention
    # wrappers (build_prefill_wrapper / build_decode_wrapper, ``model_worker.py:20-140``); the
    # batch is sorted prefill first, so these are views (decode offsets rebased on the device)
    prefill: Optional[PagedArrays] = None
    decode: Optional[PagedArrays] = None


def pack_requests(inputs: List, out: Optional[np.ndarray] = None) -> tuple:
    """Sort `inputs` as the reference does and pack them into one int32 array (`out`, if it is
    given and large enough — a ValueError otherwise — else a new array).

    Layout: ``[input_len | filled_len | context_len | num_blocks]`` (each `batch` long), then the
    concatenated block ids, then the token ids.  Returns ``(packed, batch, total_tokens,
    total_blocks, prefill_input_len, num_prefill, num_decode, prefill_blocks, decode_blocks)``;
    the last two are the block-table entries of the prefill and of the decode requests.
    """
    # the reference's ``inputs.sort(key=lambda x: -x.input_len)``: a stable descending sort,
    # written so that the key is read in C
    inputs.sort(key=_INPUT_LEN, reverse=True)
    batch = len(inputs)
    if batch > MAX_BATCH:
        raise ValueError(f"at most {MAX_BATCH} requests per step, got {batch}")
    # block tables kept as NumPy arrays by the caller are concatenated by NumPy; judged by the
    # first request (either route takes any mix of lists and arrays, this only picks the faster)
    arrays = batch > 0 and isinstance(inputs[0].block_ids, np.ndarray)
    if _packer is not None and not arrays:
        # one pass in C over the request objects, written straight into `out`
        if out is None:
            out = np.empty(4 * batch + sum(len(d.block_ids) + len(d.input_ids) for d in inputs),
                           dtype=np.int32)
        batch, T, NB, prefill_input_len, num_prefill, num_decode, pb, db = _packer.pack(inputs, out)
        return out[:4 * batch + NB + T], batch, T, NB, prefill_input_len, num_prefill, num_decode, pb, db
    head = np.empty((4, batch), dtype=np.int32)
    prefill_input_len = num_prefill = num_decode = prefill_blocks = decode_blocks = 0
    for b, data in enumerate(inputs):
        q = int(data.input_len)
        if len(data.input_ids) != q:
            raise ValueError(f"request {b}: input_len {q} but {len(data.input_ids)} input ids")
        if int(data.context_len) - int(data.filled_token_len) != q:
            raise ValueError(
                f"request {b}: context_len - filled_token_len = "
                f"{int(data.context_len) - int(data.filled_token_len)} but input_len = {q}")
        if q > 1:
            prefill_input_len += q
            num_prefill += 1
            prefill_blocks += len(data.block_ids)
        elif q == 1:
            num_decode += 1
            decode_blocks += len(data.block_ids)
        head[0, b] = q
        head[1, b] = data.filled_token_len
        head[2, b] = data.context_len
        head[3, b] = len(data.block_ids)
    total_tokens = int(head[0].sum(dtype=np.int64))
    total_blocks = int(head[3].sum(dtype=np.int64))
    n = 4 * batch + total_blocks + total_tokens
    if out is None:
        packed = np.empty(n, dtype=np.int32)
    elif out.size < n:
        raise ValueError(f"step needs {n} int32 words of staging, the buffer has {out.size}")
    else:
        packed = out[:n]
    packed[:4 * batch] = head.reshape(-1)
    o = 4 * batch
    if arrays:
        # block tables kept as arrays by the caller: no per-element conversion
        np.concatenate([d.block_ids for d in inputs], out=packed[o:o + total_blocks], casting="unsafe")
    else:
        packed[o:o + total_blocks] = np.fromiter(
            chain.from_iterable(d.block_ids for d in inputs), dtype=np.int32, count=total_blocks)
    o += total_blocks
    packed[o:o + total_tokens] = np.fromiter(
        chain.from_iterable(d.input_ids for d in inputs), dtype=np.int32, count=total_tokens)
    return (packed, batch, total_tokens, total_blocks, prefill_input_len, num_prefill, num_decode,
            prefill_blocks, decode_blocks)


class StepInputBuilder:
    """Builds the index tensors of every step into buffers allocated once.

    `max_tokens` / `max_blocks` bound the new tokens and the block-table entries of one step
    (LMServe: ``max_num_batched_tokens`` and ``max_batch_size * max_seq_len / block_size``).
    The pinned staging buffer is double-buffered (`depth`); a staging buffer is reused only after
    the copy that read it has completed.  The returned tensors are views of the builder's device
    buffers: the next call on the same stream overwrites them, which is the lifetime the
    reference gives them too (one set per step).
    """

    def __init__(self, device, block_size: int, max_batch: int = 256, max_tokens: int = 8192,
                 max_blocks: int = 65536, depth: int = 2):
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("StepInputBuilder needs a CUDA device; there is no CPU path")
        if max_batch > MAX_BATCH:
            raise ValueError(f"max_batch is limited to {MAX_BATCH}")
        self.block_size = int(block_size)
        self.max_batch, self.max_tokens, self.max_blocks = int(max_batch), int(max_tokens), int(max_blocks)
        n_in = 4 * self.max_batch + self.max_blocks + self.max_tokens
        self._staging = [torch.empty(n_in, dtype=torch.int32, pin_memory=True) for _ in range(depth)]
        self._staging_np = [s.numpy() for s in self._staging]
        self._copied = [torch.cuda.Event() for _ in range(depth)]
        self._used = [False] * depth
        self._turn = 0
        with torch.cuda.device(self.device):
            self._in = torch.empty(n_in, dtype=torch.int32, device=self.device)
            # int32 outputs: position_ids, batch_indices, positions [T each]; cu_q, indptr [B+1];
            # last_lens [B]; decode indptr [B+1]; kv_block_indices [NB].  int64 outputs:
            # slot_mapping, input_ids [T].
            self._out32 = torch.empty(3 * self.max_tokens + 4 * self.max_batch + 3 + self.max_blocks,
                                      dtype=torch.int32, device=self.device)
            self._out64 = torch.empty(2 * self.max_tokens, dtype=torch.int64, device=self.device)
            _lib.check(_lib.lib().lms_init_device())

    def make_inputs(self, inputs: List) -> Tuple[torch.Tensor, StepIndices]:
        """``(flatten_input_ids_tensor, input_params)`` of ``_make_inputs``, on the current stream."""
        turn = self._turn
        self._turn = (turn + 1) % len(self._staging)
        if self._used[turn]:
            self._copied[turn].synchronize()
        packed, batch, T, NB, prefill_len, n_pre, n_dec, pb, db = pack_requests(inputs, self._staging_np[turn])
        if T > self.max_tokens or NB > self.max_blocks or batch > self.max_batch:
            raise ValueError(
                f"step of {batch} requests / {T} tokens / {NB} block-table entries exceeds the "
                f"builder's capacity ({self.max_batch} / {self.max_tokens} / {self.max_blocks})")
        n = packed.size
        with _OnDevice(self.device):
            self._in[:n].copy_(self._staging[turn][:n], non_blocking=True)
            self._copied[turn].record()
            self._used[turn] = True
            return self._launch(batch, T, NB, prefill_len, n_pre, n_dec, pb, db)

    def _launch(self, batch, T, NB, prefill_len, n_pre, n_dec, pb=0, db=0):
        i32, i64 = self._out32, self._out64
        mt, mb = self.max_tokens, self.max_batch
        position_ids = i32[0:T]
        batch_indices = i32[mt:mt + T]
        positions = i32[2 * mt:2 * mt + T]
        o = 3 * mt
        cu_q = i32[o:o + batch + 1]
        indptr = i32[o + mb + 1:o + mb + 1 + batch + 1]
        last = i32[o + 2 * mb + 2:o + 2 * mb + 2 + batch]
        dec_indptr = i32[o + 3 * mb + 2:o + 3 * mb + 2 + n_dec + 1]
        kv_idx = i32[o + 4 * mb + 3:o + 4 * mb + 3 + NB]
        slot_mapping = i64[0:T]
        input_ids = i64[mt:mt + T]
        base = self._in.data_ptr()
        _lib.check(_lib.lib().lms_build_step_indices(
            base, base + 4 * batch, base + 8 * batch, base + 12 * batch,
            base + 16 * batch, base + 16 * batch + 4 * NB, batch, T, NB, self.block_size,
            position_ids.data_ptr(), cu_q.data_ptr(), indptr.data_ptr(), kv_idx.data_ptr(),
            last.data_ptr(), batch_indices.data_ptr(), positions.data_ptr(),
            slot_mapping.data_ptr(), input_ids.data_ptr(), n_pre, n_dec, dec_indptr.data_ptr(),
            _stream_ptr(self.device)))
        return input_ids, StepIndices(
            position_ids=position_ids, cu_seqlens_q=cu_q, prefill_input_len=prefill_len,
            batch_indices=batch_indices, positions=positions, kv_block_indices=kv_idx,
            kv_block_indptrs=indptr, kv_last_block_lens=last, slot_mapping=slot_mapping,
            num_prefill=n_pre, num_decode=n_dec,
            prefill=PagedArrays(cu_q[:n_pre + 1], indptr[:n_pre + 1], kv_idx[:pb], last[:n_pre]) if n_pre else None,
            decode=PagedArrays(None, dec_indptr, kv_idx[pb:pb + db], last[n_pre:n_pre + n_dec]) if n_dec else None)


def make_inputs(inputs: List, block_size: int, device,
                builder: Optional[StepInputBuilder] = None) -> Tuple[torch.Tensor, StepIndices]:
    """One-shot form: builds a right-sized `StepInputBuilder` unless one is passed in."""
    if builder is None:
        batch = len(inputs)
        T = sum(int(d.input_len) for d in inputs)
        NB = sum(len(d.block_ids) for d in inputs)
        builder = StepInputBuilder(device, block_size, max_batch=max(batch, 1),
                                   max_tokens=max(T, 1), max_blocks=max(NB, 1), depth=1)
    return builder.make_inputs(inputs)
