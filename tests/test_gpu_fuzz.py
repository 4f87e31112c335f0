"""GPU: seeded random geometries for every op and kernel variant, bit-exact against the oracle.
Each case draws its own row size, block size, layer count, strides, padding and index sets."""
import numpy as np
import pytest
import torch

from helpers import to_tensor, to_words
from lmserve_b200 import _lib
import workloads as W
from lmserve_b200.kv_worker import HostPool
from lmserve_b200.ops import cache_ops
from oracle import cache_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(autouse=True)
def _reset_tuning():
    yield
    for key in range(1, _lib.TUNE_COUNT):
        _lib.lib().lms_set_tuning(key, -1)


def draw_shape(rng):
    H = int(rng.choice([1, 2, 3, 4, 8]))
    D = int(rng.choice([8, 16, 24, 64, 128]))
    BS = int(rng.choice([1, 4, 7, 16, 32]))
    L = int(rng.integers(1, 5))
    NB = int(rng.integers(2, 40))
    return L, NB, BS, H, D


@pytest.mark.parametrize("seed", range(48))
def test_fuzz_cache_write(seed):
    rng = np.random.default_rng(9000 + seed)
    L, NB, BS, H, D = draw_shape(rng)
    dtype = "bf16" if seed % 2 else "fp16"
    variant = int(rng.choice([-1, 0, 1, 2, 3, 4, 5, 6, 7]))
    lib = _lib.lib()
    lib.lms_set_tuning(_lib.TUNE_WRITE_VARIANT, variant)
    lib.lms_set_tuning(_lib.TUNE_WRITE_TILE_BYTES, int(rng.choice([0, 1, 3, 512, 4096, 65536])))
    lib.lms_set_tuning(_lib.TUNE_WRITE_VPT, int(rng.choice([0, 1, 2, 4, 8])))
    lib.lms_set_tuning(_lib.TUNE_WRITE_PREFETCH, int(rng.choice([1, 2])))
    T = int(rng.integers(0, min(NB * BS, 300) + 1))
    pad = int(rng.integers(0, 4))                       # extra elements between token rows
    src = W.normal_words(rng, (2, L, T, H * D + pad * 8), dtype)
    cache = W.normal_words(rng, (L, NB, 2, BS, H, D), dtype)
    slots = rng.permutation(NB * BS)[:T].astype(np.int64)
    slots[rng.random(T) < 0.15] = -1
    per_layer = bool(rng.integers(0, 2)) and T > 0
    slot_arr = np.stack([np.roll(slots, l) for l in range(L)]) if per_layer else slots
    key_np = np.ascontiguousarray(src[0][..., :H * D]).reshape(L, T, H, D)
    val_np = np.ascontiguousarray(src[1][..., :H * D]).reshape(L, T, H, D)
    want = cache.copy()
    cache_oracle.reshape_and_cache_layers(key_np, val_np, want, slot_arr)
    dev_src = to_tensor(src, dtype, DEV)
    key = dev_src[0][..., :H * D].unflatten(-1, (H, D))     # strided view when pad > 0
    value = dev_src[1][..., :H * D].unflatten(-1, (H, D))
    got = to_tensor(cache, dtype, DEV)
    cache_ops.reshape_and_cache_layers(key, value, got, torch.from_numpy(slot_arr).to(DEV))
    torch.cuda.synchronize()
    assert np.array_equal(to_words(got), want), (seed, L, NB, BS, H, D, T, variant)


@pytest.mark.parametrize("seed", range(16))
def test_fuzz_copy_swap_transfer(seed):
    rng = np.random.default_rng(9500 + seed)
    L = int(rng.integers(1, 5))
    NB = int(rng.integers(4, 60))
    chunk_words = int(rng.choice([8, 24, 64, 1032, 4096, 16400]))
    variant = int(rng.choice([0, 1, 2, 3]))
    lib = _lib.lib()
    for key in (_lib.TUNE_COPY_VARIANT, _lib.TUNE_XFER_VARIANT, _lib.TUNE_SWAP_VARIANT):
        lib.lms_set_tuning(key, variant)
    words = rng.integers(0, 2**16, size=(L, NB, chunk_words), dtype=np.uint16)
    # copy-on-write: distinct destinations, sources outside the destinations
    n = int(rng.integers(0, NB // 2 + 1))
    perm = rng.permutation(NB)
    dsts, rest = perm[:n], perm[n:]
    pairs = np.stack([rng.choice(rest, size=n), dsts], axis=1).astype(np.int64) if n else np.empty((0, 2), np.int64)
    kv = to_tensor(words, "fp16", DEV)
    cache_ops.copy_blocks(kv, pairs)
    want = words.copy()
    cache_oracle.copy_blocks(want, pairs)
    torch.cuda.synchronize()
    assert np.array_equal(to_words(kv), want), ("cow", seed, variant)
    # swap out / in over a layer range
    NHB = int(rng.integers(2, 20))
    m = int(rng.integers(1, min(NB, NHB) + 1))
    out_pairs = np.stack([rng.permutation(NB)[:m], rng.permutation(NHB)[:m]], axis=1).astype(np.int64)
    l0 = int(rng.integers(0, L))
    l1 = int(rng.integers(l0, L + 1))
    pool = HostPool(NHB, L, chunk_words * 2)
    try:
        pool.array[...] = rng.integers(0, 256, size=pool.array.shape, dtype=np.uint8)
        host_want = pool.array.copy().view(np.uint16)
        cache_ops.swap_blocks(kv, pool, out_pairs, "out", layers=(l0, l1))
        torch.cuda.synchronize()
        cache_oracle.swap_out(want, host_want, out_pairs, layers=(l0, l1))
        assert np.array_equal(pool.array.view(np.uint16), host_want), ("swap out", seed, variant)
        in_pairs = np.stack([rng.permutation(NHB)[:m], rng.permutation(NB)[:m]], axis=1).astype(np.int64)
        cache_ops.swap_blocks(kv, pool, in_pairs, "in", layers=(l0, l1))
        torch.cuda.synchronize()
        cache_oracle.swap_in(want, host_want, in_pairs, layers=(l0, l1))
        assert np.array_equal(to_words(kv), want), ("swap in", seed, variant)
        # the same two swaps through the staging ring (a ring of 2 ... 5 blocks, so groups
        # alternate through its halves), with one or two copy streams
        if l1 > l0:
            lib.lms_set_tuning(_lib.TUNE_STAGED_STREAMS, int(rng.choice([1, 2])))
            per_block = (l1 - l0) * chunk_words * 2
            ring = torch.empty(int(rng.integers(2, 6)) * per_block + 512, dtype=torch.uint8, device=DEV)
            out2 = np.stack([rng.permutation(NB)[:m], rng.permutation(NHB)[:m]], axis=1).astype(np.int64)
            cache_ops.swap_blocks(kv, pool, out2, "out", layers=(l0, l1), engine="staged", staging=ring)
            torch.cuda.synchronize()
            cache_oracle.swap_out(want, host_want, out2, layers=(l0, l1))
            assert np.array_equal(pool.array.view(np.uint16), host_want), ("staged out", seed)
            in2 = np.stack([np.sort(rng.permutation(NHB)[:m]), rng.permutation(NB)[:m]], axis=1).astype(np.int64)
            cache_ops.swap_blocks(kv, pool, in2, "in", layers=(l0, l1), engine="staged", staging=ring)
            torch.cuda.synchronize()
            cache_oracle.swap_in(want, host_want, in2, layers=(l0, l1))
            assert np.array_equal(to_words(kv), want), ("staged in", seed)
    finally:
        pool.close()
    # transfer into a second cache, a layer range at a time
    NB2 = int(rng.integers(m, m + 10))
    dst_words = rng.integers(0, 2**16, size=(L, NB2, chunk_words), dtype=np.uint16)
    dst = to_tensor(dst_words, "fp16", DEV)
    tp = np.stack([rng.permutation(NB)[:m], rng.permutation(NB2)[:m]], axis=1).astype(np.int64)
    cache_ops.transfer_blocks(kv, dst, tp, layers=(l0, l1))
    torch.cuda.synchronize()
    d_want = dst_words.copy()
    if l1 > l0:
        cache_oracle.transfer(want[l0:l1], d_want[l0:l1], tp)
    assert np.array_equal(to_words(dst), d_want), ("transfer", seed, variant)



@pytest.mark.parametrize("seed", range(16))
def test_fuzz_paged_append(seed):
    """flashinfer's (batch index, position, page table) addressing with random request counts,
    chunk lengths, page sizes and request orders: decode-like steps (one token per request,
    where the kernel's early fetch of kv_indptr[t] is right), prefill-like steps (where it is
    wrong) and padded rows; through the cached drop-in and through an explicit plan."""
    rng = np.random.default_rng(9700 + seed)
    H, D = int(rng.choice([1, 2, 4])), int(rng.choice([16, 64, 128]))
    BS = int(rng.choice([1, 4, 16, 32]))
    nreq = int(rng.integers(1, 40))
    chunk = 1 if seed % 2 == 0 else int(rng.integers(1, 20))
    lib = _lib.lib()
    lib.lms_set_tuning(_lib.TUNE_WRITE_VARIANT, int(rng.choice([-1, 0, 3, 5, 7])))
    # every request gets its own pages; positions are distinct inside a request
    pages_per = rng.integers(1, 6, size=nreq)
    indptr = np.concatenate([[0], np.cumsum(pages_per)]).astype(np.int32)
    NB = int(indptr[-1]) + 3
    indices = rng.permutation(NB)[:indptr[-1]].astype(np.int32)
    batch, pos = [], []
    for b in range(nreq):
        room = int(pages_per[b]) * BS
        take = min(chunk, room)
        for p in rng.permutation(room)[:take]:
            batch.append(b)
            pos.append(int(p))
    order = rng.permutation(len(batch)) if seed % 3 == 0 else np.arange(len(batch))
    batch = np.asarray(batch, np.int32)[order]
    pos = np.asarray(pos, np.int32)[order]
    T = len(batch)
    if T > 2:
        batch[int(rng.integers(0, T))] = -1                 # a padded row
    key = W.normal_words(rng, (T, H, D), "bf16")
    value = W.normal_words(rng, (T, H, D), "bf16")
    cache = W.normal_words(rng, (NB, 2, BS, H, D), "bf16")
    want = cache.copy()
    cache_oracle.append_paged_kv_cache(key, value, batch, pos, want, indices, indptr)
    dev = lambda a: torch.from_numpy(a).to(DEV)
    k, v = to_tensor(key, "bf16", DEV), to_tensor(value, "bf16", DEV)
    got = to_tensor(cache, "bf16", DEV)
    args = (k, v, dev(batch), dev(pos), got, dev(indices), dev(indptr))
    cache_ops.append_paged_kv_cache(*args, None)
    torch.cuda.synchronize()
    assert np.array_equal(to_words(got), want), ("drop-in", seed, nreq, chunk, BS)
    got.copy_(to_tensor(cache, "bf16", DEV))
    cache_ops.PagedWritePlan(*args).run()
    torch.cuda.synchronize()
    assert np.array_equal(to_words(got), want), ("plan", seed)
