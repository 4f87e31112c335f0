"""The ``torch.ops.lmserve_cache.*`` custom ops: schemas (CPU) and, on a GPU, the same results as
the CPU oracle — bit-exact — eager and inside a CUDA graph."""
import numpy as np
import pytest
import torch

from helpers import to_tensor, to_words
import lmserve_b200.torch_ops as T
import workloads as W
from oracle import cache_oracle

DEV = "cuda:0"
ops = torch.ops.lmserve_cache


def test_ops_are_registered_with_their_mutations():
    want = {
        "reshape_and_cache": ["kv_cache"], "reshape_and_cache_layers": ["kv_caches"],
        "copy_blocks": ["kv_caches"], "swap_blocks": ["gpu_kv_caches", "host_pool"],
        "transfer_blocks": ["dst_kv_caches"],
    }
    assert set(T.OPS) == set(want)
    for name, mutated in want.items():
        schema = getattr(ops, name).default._schema
        written = [a.name for a in schema.arguments if a.alias_info is not None and a.alias_info.is_write]
        assert written == mutated, (name, written)
        assert len(schema.returns) == 0


def test_cpu_tensors_are_rejected_not_computed():
    kv = torch.zeros(1, 4, 2, 16, 1, 8, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.copy_blocks(kv, torch.zeros(1, 2, dtype=torch.int64))
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.reshape_and_cache(torch.zeros(1, 1, 8, dtype=torch.float16), torch.zeros(1, 1, 8, dtype=torch.float16),
                              kv[0], torch.zeros(1, dtype=torch.int64))


def small_case(seed=3):
    shape = W.SHAPES["llama31_8b"].scaled(num_layers=3, num_blocks=64)
    rng = np.random.default_rng(seed)
    cache = W.normal_words(rng, shape.cache_shape, "bf16")
    w = W.make_decode_write(shape, 12, 16, 60, seed=seed)
    key = W.normal_words(rng, (3, 12, 8, 128), "bf16")
    val = W.normal_words(rng, (3, 12, 8, 128), "bf16")
    return shape, cache, w.slot_mapping.copy(), key, val


@pytest.mark.gpu
def test_writes_and_copy_match_the_oracle_eager_and_in_a_cuda_graph():
    shape, cache, slots, key, val = small_case()
    slots[5] = -1
    want = cache.copy()
    cache_oracle.reshape_and_cache_layers(key, val, want, slots)
    pairs = np.array([[3, 60], [3, 61], [9, 62]], dtype=np.int64)
    cache_oracle.copy_blocks(want, {3: [60, 61], 9: [62]})
    k, v = to_tensor(key, "bf16", DEV), to_tensor(val, "bf16", DEV)
    s = torch.from_numpy(slots).to(DEV)
    p = torch.from_numpy(pairs).to(DEV)

    got = to_tensor(cache, "bf16", DEV)
    ops.reshape_and_cache_layers(k, v, got, s)
    ops.copy_blocks(got, p)
    torch.cuda.synchronize()
    assert np.array_equal(to_words(got), want)

    # layer by layer, pair table on the device, replayed from a graph
    got2 = to_tensor(cache, "bf16", DEV)
    ops.reshape_and_cache(k[0], v[0], got2[0], s)       # first call outside the capture
    got2.copy_(to_tensor(cache, "bf16", DEV))
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for l in range(3):
            ops.reshape_and_cache(k[l], v[l], got2[l], s)
        ops.copy_blocks(got2, p)
    g.replay()
    torch.cuda.synchronize()
    assert np.array_equal(to_words(got2), want)

    # a HOST-side pair table cannot be captured (a replay would re-read the caller's buffer):
    # the library says so instead of failing inside the runtime, and the capture stays usable
    from lmserve_b200 import _lib
    from lmserve_b200.ops import cache_ops
    g2 = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g2):
        with pytest.raises(_lib.LmsError) as e:
            cache_ops.copy_blocks(got2, pairs)
        assert e.value.status == _lib.LMS_ERR_UNSUPPORTED and "captured" in str(e.value)
        ops.reshape_and_cache(k[0], v[0], got2[0], s)
    g2.replay()
    torch.cuda.synchronize()


@pytest.mark.gpu
def test_swap_and_transfer_match_the_oracle():
    from lmserve_b200.kv_worker import HostPool
    shape, cache, *_ = small_case(seed=4)
    gw = cache.reshape(3, 64, -1).copy()
    out_pairs = np.array([[5, 1], [9, 6], [40, 0]], dtype=np.int64)
    in_pairs = np.array([[6, 50], [1, 51]], dtype=np.int64)
    host_want = np.zeros((8, 3, shape.chunk_bytes // 2), np.uint16)
    cache_oracle.swap_out(gw, host_want, out_pairs)
    cache_oracle.swap_in(gw, host_want, in_pairs)

    def run(pool_tensor):
        got = to_tensor(cache, "bf16", DEV)
        pool_tensor.zero_()
        ops.swap_blocks(got, pool_tensor, torch.from_numpy(out_pairs), "out", 0, 3)
        ops.swap_blocks(got, pool_tensor, torch.from_numpy(in_pairs).to(DEV), "in", 0, 3)
        torch.cuda.synchronize()
        assert np.array_equal(pool_tensor.numpy().view(np.uint16), host_want)
        assert np.array_equal(to_words(got).reshape(gw.shape), gw)
        return got

    pool = HostPool(8, 3, shape.chunk_bytes)
    try:
        got = run(pool.tensor)
    finally:
        pool.close()
    run(torch.empty(8, 3, shape.chunk_bytes, dtype=torch.uint8, pin_memory=True))
    with pytest.raises(RuntimeError, match="page-locked"):
        ops.swap_blocks(got, torch.empty(8, 3, shape.chunk_bytes, dtype=torch.uint8),
                        torch.from_numpy(out_pairs), "out", 0, 3)

    rng = np.random.default_rng(11)
    dst_words = W.normal_words(rng, shape.cache_shape, "bf16")
    dst = to_tensor(dst_words, "bf16", DEV)
    tp = np.array([[50, 3], [51, 4], [5, 63]], dtype=np.int64)
    want_src = gw.reshape(cache.shape)
    cache_oracle.transfer(want_src, dst_words, tp)
    ops.transfer_blocks(got, dst, torch.from_numpy(tp).to(DEV))
    torch.cuda.synchronize()
    assert np.array_equal(to_words(dst), dst_words)
