"""Seeded synthetic inputs for the KV-cache data-movement workloads.

Five named presets follow the shapes of the models LMServe serves and its
default limits (``block_size 16``, ``max_batch_size 256`` —
``runtime/src/configs.rs:19-28``).  They produce *index* inputs (slot mappings,
block pairs) the way LMServe's block manager would: a shuffled free list dealt
out as per-sequence block tables (``runtime/src/llm_engine/block_manager.rs``),
``slot = table[pos // block_size] * block_size + pos % block_size``.
Payload bytes are drawn N(0,1) and held as raw 16-bit words.

Everything here is NumPy on the host and deterministic in (preset, seed, sizes);
tests use the same generators at reduced sizes.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np

BLOCK_SIZE = 16


@dataclass(frozen=True)
class KVShape:
    """Geometry of one GPU's paged cache."""
    name: str
    num_layers: int
    num_kv_heads: int
    head_dim: int
    dtype: str  # "fp16" | "bf16"
    num_blocks: int
    block_size: int = BLOCK_SIZE

    @property
    def elem_bytes(self) -> int:
        return 2

    @property
    def row_elems(self) -> int:
        return self.num_kv_heads * self.head_dim

    @property
    def row_bytes(self) -> int:
        return self.row_elems * self.elem_bytes

    @property
    def chunk_bytes(self) -> int:
        return 2 * self.block_size * self.row_bytes

    @property
    def cache_shape(self) -> Tuple[int, ...]:
        return (self.num_layers, self.num_blocks, 2, self.block_size, self.num_kv_heads, self.head_dim)

    @property
    def cache_bytes(self) -> int:
        return self.num_layers * self.num_blocks * self.chunk_bytes

    def scaled(self, **kw) -> "KVShape":
        d = dict(self.__dict__)
        d.update(kw)
        return KVShape(**d)


SHAPES: Dict[str, KVShape] = {
    # 1: Llama-3.2-1B plumbing case (CPU-runnable)
    "llama32_1b": KVShape("llama32_1b", 1, 8, 64, "fp16", 1024),
    # 2: Llama-3.1-8B decode step
    "llama31_8b": KVShape("llama31_8b", 32, 8, 128, "bf16", 65536),
    # 3: Qwen2.5-7B chunked prefill + copy-on-write
    "qwen25_7b": KVShape("qwen25_7b", 28, 4, 128, "bf16", 65536),
    # 4: Llama-3.1-8B swap (GPU side; the host pool is sized separately)
    "llama31_8b_swap": KVShape("llama31_8b_swap", 32, 8, 128, "bf16", 16384),
    # 5: Llama-3.1-70B under TP=8: one KV head per GPU
    "llama31_70b_tp8": KVShape("llama31_70b_tp8", 80, 1, 128, "bf16", 163840),
}


# ------------------------------------------------------------------ payloads
def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 bit patterns, round-to-nearest-even."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)
    return rounded.astype(np.uint16)


def normal_words(rng: np.random.Generator, shape, dtype: str) -> np.ndarray:
    """N(0,1) samples as raw uint16 words of `dtype` ("fp16" or "bf16")."""
    x = rng.standard_normal(size=shape, dtype=np.float32)
    if dtype == "fp16":
        return x.astype(np.float16).view(np.uint16)
    if dtype == "bf16":
        return f32_to_bf16_bits(x)
    raise ValueError(f"unsupported dtype {dtype}")


# ------------------------------------------------------------------ block tables
@dataclass
class BlockTables:
    """Per-sequence block tables dealt from one shuffled free list."""
    tables: List[np.ndarray]
    free: np.ndarray  # blocks that were not dealt out, in shuffled order

    @property
    def allocated(self) -> np.ndarray:
        return np.concatenate(self.tables) if self.tables else np.empty(0, np.int64)


def deal_block_tables(rng: np.random.Generator, num_blocks: int, blocks_per_seq) -> BlockTables:
    order = rng.permutation(num_blocks).astype(np.int64)
    need = int(np.sum(blocks_per_seq))
    if need > num_blocks:
        raise ValueError(f"workload needs {need} blocks, pool has {num_blocks}")
    tables, at = [], 0
    for n in blocks_per_seq:
        tables.append(order[at:at + int(n)])
        at += int(n)
    return BlockTables(tables, order[at:])


def slots_for_positions(table: np.ndarray, positions: np.ndarray, block_size: int) -> np.ndarray:
    return table[positions // block_size] * block_size + positions % block_size


# ------------------------------------------------------------------ workloads
@dataclass
class DecodeWrite:
    """One decode step: one new token per sequence (same slots for every layer)."""
    shape: KVShape
    context_lens: np.ndarray
    slot_mapping: np.ndarray  # int64 [batch]
    tables: BlockTables

    @property
    def num_tokens(self) -> int:
        return int(self.slot_mapping.shape[0])

    def algorithmic_bytes(self, layers: Optional[int] = None) -> int:
        live = int(np.sum(self.slot_mapping >= 0))
        L = self.shape.num_layers if layers is None else layers
        return L * live * 2 * self.shape.row_bytes * 2  # K and V, read + written


def make_decode_write(shape: KVShape, batch: int, ctx_lo: int, ctx_hi: int, seed: int) -> DecodeWrite:
    rng = np.random.default_rng(seed)
    ctx = rng.integers(ctx_lo, ctx_hi + 1, size=batch).astype(np.int64)
    nblk = (ctx + 1 + shape.block_size - 1) // shape.block_size
    bt = deal_block_tables(rng, shape.num_blocks, nblk)
    slots = np.array([slots_for_positions(t, np.array([c]), shape.block_size)[0]
                      for t, c in zip(bt.tables, ctx)], dtype=np.int64)
    return DecodeWrite(shape, ctx, slots, bt)


def paged_metadata(tables: List[np.ndarray]):
    """CSR page table (kv_indptr, kv_indices), int32, of a list of per-sequence block tables —
    the arrays ``model_worker.py:399-423`` builds from ``InferInput.block_ids``."""
    counts = np.array([len(t) for t in tables], dtype=np.int64)
    indptr = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    indices = (np.concatenate(tables) if tables else np.empty(0, np.int64)).astype(np.int32)
    return indptr, indices


@dataclass
class PrefillChunkCow:
    """Chunked prefill (runs of consecutive slots) plus copy-on-write pairs."""
    shape: KVShape
    slot_mapping: np.ndarray  # int64 [num_seqs * chunk_tokens]
    pairs: np.ndarray         # int64 [n, 2] (src, dst)
    tables: BlockTables

    def write_bytes(self, layers: Optional[int] = None) -> int:
        L = self.shape.num_layers if layers is None else layers
        return L * int(np.sum(self.slot_mapping >= 0)) * 2 * self.shape.row_bytes * 2

    def cow_bytes(self, layers: Optional[int] = None) -> int:
        """Compulsory traffic: every destination written once, every distinct source read once."""
        L = self.shape.num_layers if layers is None else layers
        n_src = len(np.unique(self.pairs[:, 0])) if len(self.pairs) else 0
        return L * (len(self.pairs) + n_src) * self.shape.chunk_bytes


def make_prefill_cow(shape: KVShape, num_seqs: int, chunk_tokens: int, max_offset: int,
                     n_src: int, fanout: int, seed: int) -> PrefillChunkCow:
    rng = np.random.default_rng(seed)
    bs = shape.block_size
    offs = rng.integers(0, max_offset, size=num_seqs).astype(np.int64)
    nblk = (offs + chunk_tokens + bs - 1) // bs
    bt = deal_block_tables(rng, shape.num_blocks, nblk)
    slots = np.concatenate([
        slots_for_positions(t, np.arange(o, o + chunk_tokens, dtype=np.int64), bs)
        for t, o in zip(bt.tables, offs)]) if num_seqs else np.empty(0, np.int64)
    n_pairs = n_src * fanout
    if n_pairs:
        srcs = rng.choice(bt.allocated, size=n_src, replace=False)
        if len(bt.free) < n_pairs:
            raise ValueError("not enough free blocks for the copy-on-write destinations")
        dsts = bt.free[:n_pairs]
        pairs = np.stack([np.repeat(srcs, fanout), dsts], axis=1)
        pairs = pairs[rng.permutation(n_pairs)]
    else:
        pairs = np.empty((0, 2), np.int64)
    return PrefillChunkCow(shape, slots.astype(np.int64), np.ascontiguousarray(pairs, np.int64), bt)


@dataclass
class PlumbingCase:
    """The CPU-runnable case: random distinct slots with padding, random block pairs."""
    shape: KVShape
    slot_mapping: np.ndarray
    pairs: np.ndarray


def make_plumbing(shape: KVShape, num_tokens: int, num_padding: int, n_pairs: int, seed: int) -> PlumbingCase:
    rng = np.random.default_rng(seed)
    num_slots = shape.num_blocks * shape.block_size
    slots = rng.permutation(num_slots)[:num_tokens].astype(np.int64)
    pad = rng.choice(num_tokens, size=num_padding, replace=False)
    slots[pad] = -1
    dsts = rng.choice(shape.num_blocks, size=n_pairs, replace=False).astype(np.int64)
    rest = np.setdiff1d(np.arange(shape.num_blocks, dtype=np.int64), dsts)
    srcs = rng.choice(rest, size=n_pairs, replace=True)
    return PlumbingCase(shape, slots, np.stack([srcs, dsts], axis=1).astype(np.int64))


def plumbing_payload(case: PlumbingCase, seed: int = 2001) -> Dict[str, np.ndarray]:
    """N(0,1) payloads for the plumbing case: token rows, the two flat caches of the
    contiguous layout, and the interleaved 6-D cache; all pre-filled (raw 16-bit words)."""
    s = case.shape
    rng = np.random.default_rng(seed)
    T = len(case.slot_mapping)
    num_slots = s.num_blocks * s.block_size
    return {
        "key": normal_words(rng, (T, s.num_kv_heads, s.head_dim), s.dtype),
        "value": normal_words(rng, (T, s.num_kv_heads, s.head_dim), s.dtype),
        "key_cache": normal_words(rng, (num_slots, s.num_kv_heads, s.head_dim), s.dtype),
        "value_cache": normal_words(rng, (num_slots, s.num_kv_heads, s.head_dim), s.dtype),
        "kv_caches": normal_words(rng, s.cache_shape, s.dtype),
    }


@dataclass
class SwapRoundTrip:
    """swap-out of random GPU blocks to random host blocks, then swap-in of those host
    blocks (in permuted order) into other free GPU blocks."""
    shape: KVShape
    num_host_blocks: int
    out_pairs: np.ndarray  # (gpu src, host dst)
    in_pairs: np.ndarray   # (host src, gpu dst)

    def bytes_per_direction(self) -> int:
        return len(self.out_pairs) * self.shape.num_layers * self.shape.chunk_bytes


def make_swap(shape: KVShape, num_host_blocks: int, n_blocks: int, seed: int) -> SwapRoundTrip:
    rng = np.random.default_rng(seed)
    if 2 * n_blocks > shape.num_blocks or n_blocks > num_host_blocks:
        raise ValueError("pools too small for the swap workload")
    gpu = rng.permutation(shape.num_blocks).astype(np.int64)
    src_gpu, dst_gpu = gpu[:n_blocks], gpu[n_blocks:2 * n_blocks]
    host = rng.choice(num_host_blocks, size=n_blocks, replace=False).astype(np.int64)
    perm = rng.permutation(n_blocks)
    out_pairs = np.stack([src_gpu, host], axis=1)
    in_pairs = np.stack([host[perm], dst_gpu], axis=1)
    return SwapRoundTrip(shape, num_host_blocks, np.ascontiguousarray(out_pairs),
                         np.ascontiguousarray(in_pairs))


@dataclass
class PrefillToDecode:
    """Finished-prefill sequences' blocks on the source GPU -> free blocks of the peer."""
    shape: KVShape
    pairs: np.ndarray  # (src block on prefill GPU, dst block on decode GPU)

    def bytes(self) -> int:
        return len(self.pairs) * self.shape.num_layers * self.shape.chunk_bytes


def make_transfer(shape: KVShape, num_seqs: int, tokens_per_seq: int, seed: int,
                  dst_num_blocks: Optional[int] = None) -> PrefillToDecode:
    rng = np.random.default_rng(seed)
    per = (tokens_per_seq + shape.block_size - 1) // shape.block_size
    bt = deal_block_tables(rng, shape.num_blocks, [per] * num_seqs)
    src = bt.allocated
    dst = rng.choice(dst_num_blocks or shape.num_blocks, size=len(src), replace=False).astype(np.int64)
    return PrefillToDecode(shape, np.ascontiguousarray(np.stack([src, dst], axis=1)))


def transfer_peer(rank: int, world: int) -> Tuple[str, Optional[int]]:
    """Role and partner of `rank` in the disaggregated pairing: prefill rank g sends to decode
    rank g + world / 2 (the pairing ``lmserve_b200.disagg.transfer_role`` gives the product;
    restated here so that the input generator does not import the product package)."""
    if world < 2 or world % 2 or not (0 <= rank < world):
        return "none", None
    half = world // 2
    return ("prefill", rank + half) if rank < half else ("decode", rank - half)


# ------------------------------------------------------------------ presets
def config1(seed: int = 1001) -> PlumbingCase:
    return make_plumbing(SHAPES["llama32_1b"], 256, 16, 64, seed)


def config2(seed: int = 1002, num_blocks: Optional[int] = None) -> DecodeWrite:
    s = SHAPES["llama31_8b"]
    return make_decode_write(s if num_blocks is None else s.scaled(num_blocks=num_blocks),
                             256, 128, 4096, seed)


def config3(seed: int = 1003, num_blocks: Optional[int] = None) -> PrefillChunkCow:
    s = SHAPES["qwen25_7b"]
    return make_prefill_cow(s if num_blocks is None else s.scaled(num_blocks=num_blocks),
                            64, 512, 8192, 32, 128, seed)


def config4(seed: int = 1004, num_host_blocks: int = 131072, n_blocks: int = 8192) -> SwapRoundTrip:
    return make_swap(SHAPES["llama31_8b_swap"], num_host_blocks, n_blocks, seed)


def config5_decode(rank: int = 0, seed: int = 1005, num_blocks: Optional[int] = None) -> DecodeWrite:
    s = SHAPES["llama31_70b_tp8"]
    return make_decode_write(s if num_blocks is None else s.scaled(num_blocks=num_blocks),
                             512, 512, 8192, seed + rank)


def config5_transfer(rank: int = 0, seed: int = 1005, num_blocks: Optional[int] = None) -> PrefillToDecode:
    s = SHAPES["llama31_70b_tp8"]
    return make_transfer(s if num_blocks is None else s.scaled(num_blocks=num_blocks),
                         32, 2048, seed + 100 + rank)


# ---------------------------------------------------------------- per-step request lists
@dataclass
class StepRequest:
    """One scheduled request with the ``InferInput`` fields of ``proto/worker.proto:40-47``."""
    input_ids: List[int]
    input_len: int
    filled_token_len: int
    context_len: int
    block_ids: List[int]
    seq_id: int = 0


def make_step_requests(num_blocks: int, block_size: int, num_decode: int, ctx_lo: int, ctx_hi: int,
                       num_prefill: int, chunk_tokens: int, max_offset: int, seed: int,
                       spare_blocks: int = 0, vocab: int = 128256) -> List[StepRequest]:
    """A mixed step in scheduler order (seeded shuffle): `num_decode` requests with one new token
    after ``ctx ~ U{ctx_lo..ctx_hi}`` cached tokens and `num_prefill` requests whose chunk of
    `chunk_tokens` tokens starts at ``off ~ U{0..max_offset-1}``.  Block tables are dealt from a
    seeded shuffle of the free list and hold exactly the blocks the context needs, plus
    `spare_blocks` reserved ahead when asked for."""
    rng = np.random.default_rng(seed)
    filled = np.concatenate([rng.integers(ctx_lo, ctx_hi + 1, size=num_decode),
                             rng.integers(0, max(max_offset, 1), size=num_prefill)]).astype(np.int64)
    new = np.concatenate([np.ones(num_decode, np.int64), np.full(num_prefill, chunk_tokens, np.int64)])
    ctx = filled + new
    nblk = (ctx + block_size - 1) // block_size + spare_blocks
    bt = deal_block_tables(rng, num_blocks, nblk)
    reqs = [StepRequest(input_ids=rng.integers(0, vocab, size=int(q)).tolist(), input_len=int(q),
                        filled_token_len=int(f), context_len=int(c),
                        block_ids=[int(x) for x in t], seq_id=i)
            for i, (q, f, c, t) in enumerate(zip(new, filled, ctx, bt.tables))]
    order = rng.permutation(len(reqs))
    return [reqs[i] for i in order]
