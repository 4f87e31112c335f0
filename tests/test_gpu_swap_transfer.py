"""GPU: GPU<->pinned-host swap and prefill->decode transfer against the oracle, through the
C ABI and through the KVWorker mirror (events per layer, descriptors, push from another
process)."""
import multiprocessing as mp

import numpy as np
import pytest
import torch

from helpers import to_tensor, to_words
from lmserve_b200 import _lib
import workloads as W
from lmserve_b200.kv_worker import BlockMapping, Device, HostPool, KVWorker
from lmserve_b200.ops import cache_ops
from oracle import cache_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(autouse=True)
def _reset_tuning():
    yield
    for key in range(1, _lib.TUNE_COUNT):
        _lib.lib().lms_set_tuning(key, -1)


def make_gpu_cache(shape, seed):
    words = W.normal_words(np.random.default_rng(seed), shape.cache_shape, shape.dtype)
    return words, to_tensor(words, shape.dtype, DEV)


@pytest.mark.parametrize("variant", [0, 1, 2, 3, 4])
@pytest.mark.parametrize("ctas", [0, 8, 300])
def test_swap_out_in_vs_oracle(ctas, variant):
    L = _lib.lib()
    L.lms_set_tuning(_lib.TUNE_SWAP_VARIANT, variant)
    L.lms_set_tuning(_lib.TUNE_SWAP_OUT_CTAS, ctas)
    L.lms_set_tuning(_lib.TUNE_SWAP_IN_CTAS, ctas)
    shape = W.SHAPES["llama31_8b_swap"].scaled(num_layers=3, num_blocks=64)
    sw = W.make_swap(shape, num_host_blocks=40, n_blocks=20, seed=61)
    words, gpu = make_gpu_cache(shape, 62)
    pool = HostPool(40, shape.num_layers, shape.chunk_bytes)
    try:
        rng = np.random.default_rng(63)
        pool.array[...] = rng.integers(0, 256, size=pool.array.shape, dtype=np.uint8)
        host_want = pool.array.copy().view(np.uint16)
        gpu_want = words.reshape(shape.num_layers, shape.num_blocks, -1).copy()
        cache_ops.swap_blocks(gpu, pool, sw.out_pairs, "out")
        torch.cuda.synchronize()
        cache_oracle.swap_out(gpu_want, host_want, sw.out_pairs)
        assert np.array_equal(pool.array.view(np.uint16), host_want)
        cache_ops.swap_blocks(gpu, pool, sw.in_pairs, "in")
        torch.cuda.synchronize()
        cache_oracle.swap_in(gpu_want, host_want, sw.in_pairs)
        got = to_words(gpu).reshape(gpu_want.shape)
        assert np.array_equal(got, gpu_want)
        # round trip: every swapped-in block equals the block that was swapped out
        back = {int(h): int(g) for g, h in sw.out_pairs}
        for h, d in sw.in_pairs:
            assert np.array_equal(got[:, d], got[:, back[int(h)]])
    finally:
        pool.close()


@pytest.mark.parametrize("big_stride", [False, True])
def test_swap_on_the_copy_engines(big_stride):
    """LMS_TUNE_SWAP_ENGINE = 2: the same swap issued as strided DMA copies (one per block), or
    as one copy per layer and block when the layer stride is beyond the 2D-copy pitch limit;
    host-side index check under debug checks."""
    lib = _lib.lib()
    lib.lms_set_tuning(_lib.TUNE_SWAP_ENGINE, 2)
    L_, NB, chunk_words = 3, 24, 4096
    rng = np.random.default_rng(90)
    words = rng.integers(0, 2**16, size=(L_, NB, chunk_words), dtype=np.uint16)
    if big_stride:   # layers 2.25 GiB apart inside one buffer: pitch > 2^31 - 1
        far = 9 * (1 << 27)                                   # elements
        buf = torch.zeros(2 * far + NB * chunk_words + 64, dtype=torch.float16, device=DEV)
        gpu = torch.as_strided(buf, (L_, NB, chunk_words), (far, chunk_words, 1))
        gpu.copy_(to_tensor(words, "fp16", DEV))
    else:
        gpu = to_tensor(words, "fp16", DEV)
    pool = HostPool(10, L_, chunk_words * 2)
    try:
        pool.array[...] = 0
        out_pairs = np.array([[3, 9], [23, 0], [7, 4]], dtype=np.int64)
        before = lib.lms_launch_count()
        cache_ops.swap_blocks(gpu, pool, out_pairs, "out", layers=(1, 3))
        torch.cuda.synchronize()
        assert lib.lms_launch_count() == before            # no kernel of ours was launched
        host_want = np.zeros((10, L_, chunk_words), np.uint16)
        gpu_want = words.copy()
        cache_oracle.swap_out(gpu_want, host_want, out_pairs, layers=(1, 3))
        assert np.array_equal(pool.array.view(np.uint16), host_want)
        in_pairs = np.array([[9, 10], [4, 11]], dtype=np.int64)
        cache_ops.swap_blocks(gpu, pool, in_pairs, "in")
        torch.cuda.synchronize()
        cache_oracle.swap_in(gpu_want, host_want, in_pairs)
        assert np.array_equal(to_words(gpu.contiguous()), gpu_want)
        lib.lms_set_debug_checks(1)
        try:
            with pytest.raises(_lib.LmsError) as e:
                cache_ops.swap_blocks(gpu, pool, np.array([[3, 1], [2, 77]], dtype=np.int64), "out")
            assert e.value.status == _lib.LMS_ERR_INDEX
        finally:
            lib.lms_set_debug_checks(0)
        torch.cuda.synchronize()
        assert np.array_equal(pool.array.view(np.uint16), host_want)   # nothing was copied
    finally:
        pool.close()


def test_swap_layer_range_and_empty():
    shape = W.SHAPES["llama31_8b_swap"].scaled(num_layers=4, num_blocks=16, num_kv_heads=2)
    words, gpu = make_gpu_cache(shape, 64)
    pool = HostPool(8, 4, shape.chunk_bytes)
    try:
        pool.array[...] = 0
        pairs = np.array([[3, 1], [15, 7], [0, 0]], dtype=np.int64)
        cache_ops.swap_blocks(gpu, pool, pairs, "out", layers=(1, 3))
        cache_ops.swap_blocks(gpu, pool, np.empty((0, 2), np.int64), "out")
        cache_ops.swap_blocks(gpu, pool, pairs, "out", layers=(2, 2))
        torch.cuda.synchronize()
        want = np.zeros((8, 4, shape.chunk_bytes // 2), np.uint16)
        cache_oracle.swap_out(words.reshape(4, 16, -1), want, pairs, layers=(1, 3))
        assert np.array_equal(pool.array.view(np.uint16), want)
        with pytest.raises(ValueError, match="Unsupported copy direction"):
            cache_ops.swap_blocks(gpu, pool, pairs, "sideways")
        with pytest.raises(ValueError):
            cache_ops.swap_blocks(gpu, pool, pairs, "out", layers=(3, 9))
    finally:
        pool.close()


def test_host_pool_from_existing_buffer():
    """A pool pinned in place over caller-owned memory (lms_host_register) behaves like an
    allocated one, and the caller sees the swapped-out bytes in its own array."""
    shape = W.SHAPES["llama31_8b_swap"].scaled(num_layers=2, num_blocks=16, num_kv_heads=1)
    words, gpu = make_gpu_cache(shape, 67)
    backing = np.zeros((6 * 2 * shape.chunk_bytes + 4096,), dtype=np.uint8)
    off = (-backing.ctypes.data) % 4096                      # page-align the pool inside it
    mine = backing[off:off + 6 * 2 * shape.chunk_bytes]
    pool = HostPool.from_buffer(mine, 2, shape.chunk_bytes)
    try:
        assert pool.num_blocks == 6 and pool.host_ptr == mine.ctypes.data
        pairs = np.array([[9, 4], [0, 1]], dtype=np.int64)
        cache_ops.swap_blocks(gpu, pool, pairs, "out")
        torch.cuda.synchronize()
        want = np.zeros((6, 2, shape.chunk_bytes // 2), np.uint16)
        cache_oracle.swap_out(words.reshape(2, 16, -1), want, pairs)
        assert np.array_equal(mine.view(np.uint16).reshape(want.shape), want)
        cache_ops.swap_blocks(gpu, pool, np.array([[4, 15]], dtype=np.int64), "in")
        torch.cuda.synchronize()
        assert np.array_equal(to_words(gpu).reshape(2, 16, -1)[:, 15], words.reshape(2, 16, -1)[:, 9])
    finally:
        pool.close()
    with pytest.raises(ValueError):
        HostPool.from_buffer(np.zeros(100, np.uint8), 2, shape.chunk_bytes)


def test_host_pool_on_huge_pages_round_trip():
    """The pool made of transparent huge pages (or of small ones where the kernel grants none)
    is 2 MiB aligned, starts zeroed and swaps like any other pool, with every engine."""
    shape = W.SHAPES["llama31_8b_swap"].scaled(num_layers=3, num_blocks=24, num_kv_heads=2)
    words, gpu = make_gpu_cache(shape, 71)
    pool = HostPool.with_huge_pages(40, 3, shape.chunk_bytes)
    try:
        assert pool.host_ptr % (2 << 20) == 0 and pool.num_blocks == 40
        assert not pool.array.any()
        rng = np.random.default_rng(72)
        out_pairs = np.stack([rng.permutation(24)[:10], rng.permutation(40)[:10]], 1).astype(np.int64)
        want = np.zeros((40, 3, shape.chunk_bytes // 2), np.uint16)
        cache_oracle.swap_out(words.reshape(3, 24, -1), want, out_pairs)
        for engine in ("kernel", "dma", "staged"):
            pool.array[:] = 0
            cache_ops.swap_blocks(gpu, pool, out_pairs, "out", engine=engine)
            torch.cuda.synchronize()
            assert np.array_equal(pool.array.view(np.uint16), want), engine
    finally:
        pool.close()


def test_kvworker_copy_kv_with_layer_events():
    """Write-through then fetch, one launch per layer, ordered by per-layer events the way the
    model's forward hooks and the KV worker hand layers to each other."""
    shape = W.SHAPES["llama31_8b_swap"].scaled(num_layers=4, num_blocks=32, num_kv_heads=2)
    words, gpu = make_gpu_cache(shape, 65)
    worker = KVWorker("kv0", gpu, num_host_blocks=16)
    try:
        sw = W.make_swap(shape, 16, 10, seed=66)
        maps_out = [BlockMapping.from_pairs(sw.out_pairs[:4]), BlockMapping.from_pairs(sw.out_pairs[4:])]
        post = [torch.cuda.Event() for _ in range(4)]
        for e in post:
            e.record(torch.cuda.current_stream())
        worker.copy_kv(maps_out, Device.GPU, Device.Host, post_events=post)
        worker.dtoh_stream.synchronize()
        pre = [torch.cuda.Event() for _ in range(4)]
        worker.copy_kv([sw.in_pairs], Device.Host, Device.GPU, pre_events=pre, layers_per_launch=2)
        for e in pre:
            torch.cuda.current_stream().wait_event(e)
        torch.cuda.synchronize()
        gpu_want = words.reshape(4, 32, -1).copy()
        host_want = np.zeros((16, 4, shape.chunk_bytes // 2), np.uint16)
        cache_oracle.swap_out(gpu_want, host_want, sw.out_pairs)
        cache_oracle.swap_in(gpu_want, host_want, sw.in_pairs)
        assert np.array_equal(to_words(gpu).reshape(gpu_want.shape), gpu_want)
        with pytest.raises(ValueError, match="Unsupported copy direction"):
            worker.copy_kv([], Device.Host, Device.Disk)
    finally:
        worker.close()


@pytest.mark.parametrize("variant", [0, 1, 2, 3, 4])
def test_transfer_blocks_same_device_vs_oracle(variant):
    _lib.lib().lms_set_tuning(_lib.TUNE_XFER_VARIANT, variant)
    shape = W.SHAPES["llama31_70b_tp8"].scaled(num_layers=6, num_blocks=300)
    tr = W.make_transfer(shape, 4, 300, seed=71, dst_num_blocks=200)
    src_words, src = make_gpu_cache(shape, 72)
    dshape = shape.scaled(num_blocks=200)
    dst_words, dst = make_gpu_cache(dshape, 73)
    cache_ops.transfer_blocks(src, dst, tr.pairs)
    torch.cuda.synchronize()
    want = dst_words.copy()
    cache_oracle.transfer(src_words, want, tr.pairs)
    assert np.array_equal(to_words(dst), want)
    assert np.array_equal(to_words(src), src_words)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_transfer_blocks_across_devices():
    shape = W.SHAPES["llama31_70b_tp8"].scaled(num_layers=4, num_blocks=128)
    tr = W.make_transfer(shape, 3, 400, seed=74)
    src_words, src = make_gpu_cache(shape, 75)
    dst_words = W.normal_words(np.random.default_rng(76), shape.cache_shape, shape.dtype)
    dst = to_tensor(dst_words, shape.dtype, "cuda:1")
    torch.cuda.synchronize("cuda:1")
    cache_ops.transfer_blocks(src, dst, tr.pairs)
    torch.cuda.synchronize("cuda:0")
    want = dst_words.copy()
    cache_oracle.transfer(src_words, want, tr.pairs)
    assert np.array_equal(to_words(dst), want)
    # the same transfer pulled: the kernel runs on cuda:1 and loads from cuda:0
    dst2 = to_tensor(dst_words, shape.dtype, "cuda:1")
    torch.cuda.synchronize("cuda:1")
    cache_ops.transfer_blocks(src, dst2, tr.pairs, pull=True)
    torch.cuda.synchronize("cuda:1")
    assert np.array_equal(to_words(dst2), want)
    assert np.array_equal(to_words(src), src_words)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_kv_workers_on_two_gpus_of_one_process_push_and_pull():
    """Two workers of ONE process on two GPUs: the descriptor names this process, so the peer
    cache is used in place over NVLink (peer access) instead of through an IPC mapping, which
    the exporting process could not open.  Push with surplus reservations, then pull back."""
    shape = W.SHAPES["llama31_70b_tp8"].scaled(num_layers=4, num_blocks=96)
    src_words, src = make_gpu_cache(shape, 175)
    dst_words = W.normal_words(np.random.default_rng(176), shape.cache_shape, shape.dtype)
    dst = to_tensor(dst_words, shape.dtype, "cuda:1")
    torch.cuda.synchronize("cuda:1")
    prefill, decode = KVWorker("p0", src), KVWorker("d0", dst)
    try:
        local, reserved = [3, 50, 51, 95], [9, 8, 70, 0, 33, 34]
        assert prefill.push_kv("d0", decode.get_descriptors(reserved), local) is True
        prefill.push_stream.synchronize()
        want = dst_words.copy()
        cache_oracle.transfer(src_words, want, np.stack([local, reserved[:4]], axis=1))
        assert np.array_equal(to_words(dst), want)
        # pull other blocks back into the first cache
        assert prefill.pull_kv("d0", decode.get_descriptors([9, 70]), [60, 61]) is True
        prefill.push_stream.synchronize()
        back = src_words.copy()
        cache_oracle.transfer(want, back, np.array([[9, 60], [70, 61]]))
        assert np.array_equal(to_words(src), back)
    finally:
        prefill.close()
        decode.close()


def test_transfer_blocks_pull_on_one_device_and_argument_errors():
    shape = W.SHAPES["llama31_70b_tp8"].scaled(num_layers=3, num_blocks=40)
    src_words, src = make_gpu_cache(shape, 77)
    dst_words, dst = make_gpu_cache(shape, 78)
    pairs = np.array([[1, 5], [2, 39], [30, 0]], dtype=np.int64)
    cache_ops.transfer_blocks(src, dst, pairs, pull=True, layers=(1, 3))
    torch.cuda.synchronize()
    want = dst_words.copy()
    cache_oracle.transfer(src_words[1:3], want[1:3], pairs)
    assert np.array_equal(to_words(dst), want)

    class NotATensor:
        num_layers, num_blocks, layer_stride, block_stride, chunk_bytes, device_ptr = 3, 40, 0, 0, 0, 0
    with pytest.raises(TypeError, match="dst_kv_caches"):
        cache_ops.transfer_blocks(src, NotATensor(), pairs, pull=True)
    with pytest.raises(TypeError, match="src_kv_caches"):
        cache_ops.transfer_blocks(NotATensor(), dst, pairs)


def _kv_process(params, out_pairs, in_pairs, q):
    """Child = the KV process: maps the parent's cache and events, writes blocks through to its
    host pool as the parent's post-events fire, then fetches them back into other blocks and
    records the pre-events."""
    try:
        import torch
        from lmserve_b200.kv_worker import Device, KVWorker
        w = KVWorker.from_params("kv0", params)
        w.copy_kv([out_pairs], Device.GPU, Device.Host, post_events=w.post_events)
        w.dtoh_stream.synchronize()
        w.copy_kv([in_pairs], Device.Host, Device.GPU, pre_events=w.pre_events)
        w.htod_stream.synchronize()
        host_sum = int(w.host_pool.array[out_pairs[:, 1]].astype("int64").sum())
        w.close()
        q.put(("ok", host_sum))
    except Exception as e:  # pragma: no cover - reported to the parent
        q.put(("error", repr(e)))


def test_kv_process_maps_the_model_process_cache_and_events():
    """The reference's two-process layout: the model process owns the cache and the per-layer
    events, the KV process maps both (CUDA IPC) and swaps blocks, ordered by the events."""
    from lmserve_b200.kv_worker import KVWorkerParams
    shape = W.SHAPES["llama31_8b_swap"].scaled(num_layers=3, num_blocks=32, num_kv_heads=2)
    words, gpu = make_gpu_cache(shape, 83)
    L_ = shape.num_layers
    pre = [torch.cuda.Event(interprocess=True) for _ in range(L_)]
    post = [torch.cuda.Event(interprocess=True) for _ in range(L_)]
    for e in post:                       # "attention of layer l is done"
        e.record(torch.cuda.current_stream())
    torch.cuda.synchronize()
    params = KVWorkerParams.from_cache(gpu, num_host_blocks=8, pre_events=pre, post_events=post)
    out_pairs = np.array([[3, 0], [17, 5], [30, 7]], dtype=np.int64)
    in_pairs = np.array([[5, 1], [0, 2], [7, 31]], dtype=np.int64)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_kv_process, args=(params, out_pairs, in_pairs, q))
    p.start()
    status, payload = q.get(timeout=300)
    p.join(timeout=60)
    assert status == "ok", payload
    for e in pre:                        # the model would wait on these before layer l
        torch.cuda.current_stream().wait_event(e)
    torch.cuda.synchronize()
    gw = words.reshape(L_, 32, -1).copy()
    hw = np.zeros((8, L_, shape.chunk_bytes // 2), np.uint16)
    cache_oracle.swap_out(gw, hw, out_pairs)
    assert payload == int(hw[out_pairs[:, 1]].view(np.uint8).astype(np.int64).sum())
    cache_oracle.swap_in(gw, hw, in_pairs)
    assert np.array_equal(to_words(gpu).reshape(gw.shape), gw)


def _kv_process_late(params, in_pairs, out_pairs, delay, q):
    """Child = the KV process of the waiter-first test: it fills host block 4 with a pattern,
    lets `delay` seconds pass (the model process has issued its pre-hooks long before), swaps
    the block in behind pre-events + tokens, and then at once asks for a swap-out that the
    model's post-events and tokens release only later."""
    try:
        import time
        import numpy as np
        from lmserve_b200.kv_worker import Device, KVWorker
        w = KVWorker.from_params("kv0", params)
        L_ = w.num_layers
        for l in range(L_):
            w.host_pool.array.view(np.float16).reshape(w.host_pool.num_blocks, L_, -1)[4, l] = 5.0 + l
        time.sleep(delay)
        w.copy_kv([in_pairs], Device.Host, Device.GPU, pre_events=w.pre_events)
        w.htod_stream.synchronize()
        w.copy_kv([out_pairs], Device.GPU, Device.Host, post_events=w.post_events)
        w.dtoh_stream.synchronize()
        got = w.host_pool.array.view(np.float16).reshape(w.host_pool.num_blocks, L_, -1)[2, :, 0].tolist()
        w.close()
        q.put(("ok", got))
    except Exception as e:  # pragma: no cover - reported to the parent
        q.put(("error", repr(e)))


def test_two_process_handshake_when_the_waiter_comes_first():
    """The model process issues its pre-hooks BEFORE the KV process has recorded this step's
    pre-events, and the KV process asks for its swap-out BEFORE the model has recorded the
    post-events.  A stream wait binds to the last record issued so far (none here), so without
    the token queues both sides would read stale blocks; with them the hook and the worker
    hold their waits back until the other side's record has been issued."""
    import time
    from lmserve_b200.kv_worker import init_cache
    L_, H, D, BS = 3, 2, 64, 16
    per_block = L_ * 2 * BS * H * D * 2
    kv, handle, params = init_cache(per_block * 12, per_block * 6, num_layers=L_, num_kv_heads=H,
                                    head_dim=D, block_size=BS, dtype=torch.float16, device=DEV)
    assert params.model_queue is not None and handle.kv_queue is params.kv_queue
    kv.zero_()
    torch.cuda.synchronize()

    class Attention(torch.nn.Module):
        def __init__(self, layer):
            super().__init__()
            self.layer = layer

        def forward(self, x):
            seen = kv[self.layer, 7].clone()
            kv[self.layer, 3] = x + self.layer
            return seen

    layers = torch.nn.ModuleList(Attention(i) for i in range(L_))
    handle.register_hooks(layers)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    in_pairs = np.array([[4, 7]], dtype=np.int64)
    out_pairs = np.array([[3, 2]], dtype=np.int64)
    p = ctx.Process(target=_kv_process_late, args=(params, in_pairs, out_pairs, 1.0, q))
    p.start()
    x = torch.full((2, BS, H, D), 2.0, dtype=torch.float16, device=DEV)
    handle.enable_wait_before_execute = True         # hooks run now; the child records in > 1 s
    seen = [layer(x) for layer in layers]
    torch.cuda.synchronize()
    for l in range(L_):
        assert (seen[l] == 5.0 + l).all(), "the layer read the block before it was swapped in"
    handle.enable_wait_before_execute = False
    time.sleep(0.5)                                  # the child is already waiting for post tokens
    kv[:, 3] = 0
    handle.enable_record_after_execute = True
    for layer in layers:
        layer(x)
    status, payload = q.get(timeout=300)
    p.join(timeout=60)
    assert status == "ok", payload
    assert payload == [2.0 + l for l in range(L_)]   # not the zeros that were there before


def test_two_thread_handshake_with_the_worker_in_this_process():
    """The same race with the KV worker on a second host thread of one process."""
    import queue
    import threading
    import time
    shape = W.SHAPES["llama31_8b_swap"].scaled(num_layers=4, num_blocks=16, num_kv_heads=2)
    words, gpu = make_gpu_cache(shape, 97)
    worker = KVWorker("kv0", gpu, num_host_blocks=4)
    from lmserve_b200.kv_worker import KVWorkerHandle
    try:
        worker.model_queue, worker.kv_queue = queue.Queue(), queue.Queue()
        pre = [torch.cuda.Event() for _ in range(4)]
        handle = KVWorkerHandle(pre, [], model_queue=worker.model_queue, kv_queue=worker.kv_queue)
        worker.host_pool.array[...] = 7
        before = to_words(gpu).reshape(4, 16, -1)[:, 9].copy()

        def kv_thread():
            torch.cuda.set_device(gpu.device)
            time.sleep(0.3)
            worker.load_kv_blocks_from_host([np.array([[1, 9]])], pre_events=pre)

        t = threading.Thread(target=kv_thread)
        t.start()
        got = []
        for l in range(4):
            handle.wait_before_layer(l)                  # blocks until the worker's token
            got.append(gpu[l, 9].clone())
        t.join()
        torch.cuda.synchronize()
        for l in range(4):
            assert (to_words(got[l]).view(np.uint8) == 7).all()
        assert not (before.view(np.uint8) == 7).all()
    finally:
        worker.close()


def test_init_cache_and_layer_hooks_drive_the_swap_handshake():
    """init_cache sizes and allocates the cache as the reference does; the forward hooks record
    post_events after each attention layer has written its KV and make a layer wait for its
    pre_event, and the KV worker's per-layer swaps are ordered by exactly those events."""
    from lmserve_b200.kv_worker import BlockMapping, init_cache
    L_, H, D, BS = 3, 2, 64, 16
    per_block = L_ * 2 * BS * H * D * 2
    kv, handle, params = init_cache(per_block * 12 + 100, per_block * 5, num_layers=L_, num_kv_heads=H,
                                    head_dim=D, block_size=BS, dtype=torch.float16, device=DEV,
                                    mp_context=None)   # worker and model share this thread
    assert kv.shape == (L_, 12, 2, BS, H, D) and params.num_host_blocks == 5
    assert params.cache_shape == tuple(kv.shape) and len(params.pre_event_handles) == L_
    kv.zero_()

    class Attention(torch.nn.Module):
        def __init__(self, layer):
            super().__init__()
            self.layer = layer

        def forward(self, x):
            seen = kv[self.layer, 7].clone()          # what the layer finds in block 7
            kv[self.layer, 3] = x + self.layer         # the KV this layer produces, in block 3
            return seen

    layers = torch.nn.ModuleList(Attention(i) for i in range(L_))
    handle.register_hooks(layers)
    worker = KVWorker("kv0", kv, num_host_blocks=5)
    side = torch.cuda.Stream()
    try:
        # forward pass that records post_events; the worker saves block 3 layer by layer behind it
        handle.enable_record_after_execute = True
        x = torch.full((2, BS, H, D), 2.0, dtype=torch.float16, device=DEV)
        for layer in layers:
            layer(x)
        worker.save_kv_blocks_to_host([BlockMapping.from_pairs([(3, 4)])], stream=side,
                                      post_events=handle.post_events)
        side.synchronize()
        got = worker.host_pool.array.view(np.float16).reshape(5, L_, -1)
        for l in range(L_):
            assert (got[4, l] == 2.0 + l).all()
        # the worker loads host block 4 into GPU block 7 and signals pre_events; the layers wait
        handle.enable_record_after_execute = False
        handle.enable_wait_before_execute = True
        worker.load_kv_blocks_from_host([BlockMapping.from_pairs([(4, 7)])], stream=side,
                                        pre_events=handle.pre_events)
        seen = [layer(x) for layer in layers]
        torch.cuda.synchronize()
        for l in range(L_):
            assert (seen[l] == 2.0 + l).all()
    finally:
        worker.close()
    with pytest.raises(ValueError, match="smaller than one block"):
        init_cache(10, 0, num_layers=L_, num_kv_heads=H, head_dim=D, block_size=BS, dtype=torch.float16, device=DEV)


def test_disk_tier_round_trip_through_copy_kv(tmp_path):
    """GPU -> host -> disk -> host -> GPU through KVWorker.copy_kv, the four directions of the
    reference's dispatch table; the disk file is a .npy memory map."""
    from lmserve_b200.kv_worker import BlockMapping, Device
    shape = W.SHAPES["llama31_8b_swap"].scaled(num_layers=3, num_blocks=32, num_kv_heads=2)
    words, gpu = make_gpu_cache(shape, 91)
    f = str(tmp_path / "disk-kv-cache-0.npy")
    worker = KVWorker("kv0", gpu, num_host_blocks=6, num_disk_blocks=10, disk_kv_cache_file=f)
    try:
        m = lambda pairs: [BlockMapping.from_pairs(pairs)]
        worker.copy_kv(m([(4, 0), (9, 5), (31, 2)]), Device.GPU, Device.Host)
        worker.copy_kv(m([(0, 7), (5, 1), (2, 9)]), Device.Host, Device.Disk)
        worker.host_pool.array[...] = 0
        worker.copy_kv(m([(7, 3), (9, 4)]), Device.Disk, Device.Host)
        worker.copy_kv(m([(3, 20), (4, 21)]), Device.Host, Device.GPU)
        torch.cuda.synchronize()
        gw = words.reshape(3, 32, -1)
        got = to_words(gpu).reshape(gw.shape)
        assert np.array_equal(got[:, 20], gw[:, 4]) and np.array_equal(got[:, 21], gw[:, 31])
        disk = np.load(f, mmap_mode="r")
        assert np.array_equal(disk[1].view(np.uint16), gw[:, 9])
        with pytest.raises(ValueError, match="Unsupported copy direction"):
            worker.copy_kv(m([(0, 0)]), Device.GPU, Device.Disk)
        with pytest.raises(IndexError):
            worker.copy_kv(m([(0, 10)]), Device.Host, Device.Disk)
    finally:
        worker.close()
    with pytest.raises(ValueError, match="disk tier needs"):
        KVWorker("kv1", gpu, num_host_blocks=0, num_disk_blocks=2, disk_kv_cache_file=f)


def _puller(desc_bytes, seed, local_blocks, q):
    """Child = the decode-side worker pulling blocks out of the parent's (prefill) cache."""
    try:
        import numpy as np
        from helpers import to_tensor, to_words
        import workloads as W
        from lmserve_b200.kv_worker import KVWorker
        shape = W.SHAPES["llama31_70b_tp8"].scaled(num_layers=4, num_blocks=64)
        words = W.normal_words(np.random.default_rng(seed), shape.cache_shape, shape.dtype)
        cache = to_tensor(words, shape.dtype, "cuda:0")
        w = KVWorker("decode0", cache)
        ok = w.pull_kv("prefill0", desc_bytes, local_blocks)
        w.push_stream.synchronize()
        got = to_words(cache)
        w.close()
        q.put(("ok", ok, got))
    except Exception as e:  # pragma: no cover - reported to the parent
        q.put(("error", repr(e), None))


def test_pull_kv_from_another_process():
    shape = W.SHAPES["llama31_70b_tp8"].scaled(num_layers=4, num_blocks=64)
    src_words, src = make_gpu_cache(shape, 85)
    prefill = KVWorker("prefill0", src)
    offered = [11, 12, 50, 3, 4]              # one more than the puller takes
    local = [20, 21, 22, 63]
    desc = prefill.get_descriptors(offered)
    torch.cuda.synchronize()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_puller, args=(desc, 86, local, q))
    p.start()
    status, ok, got = q.get(timeout=300)
    p.join(timeout=60)
    assert status == "ok" and ok is True, ok
    want = W.normal_words(np.random.default_rng(86), shape.cache_shape, shape.dtype)
    cache_oracle.transfer(src_words, want, np.stack([offered[:4], local], axis=1))
    assert np.array_equal(got, want)
    assert np.array_equal(to_words(src), src_words)
    prefill.close()


def _pusher(desc_bytes, seed, pairs_src, q, layered=False):
    """Child process = the prefill-side worker: builds its own cache and pushes blocks into the
    parent's cache through the IPC descriptor."""
    try:
        import numpy as np
        import torch
        from helpers import to_tensor
        import workloads as W
        from lmserve_b200.kv_worker import KVWorker
        shape = W.SHAPES["llama31_70b_tp8"].scaled(num_layers=4, num_blocks=64)
        words = W.normal_words(np.random.default_rng(seed), shape.cache_shape, shape.dtype)
        cache = to_tensor(words, shape.dtype, "cuda:0")
        w = KVWorker("prefill0", cache)
        if layered:
            # the model's side of the handshake: one event per layer, recorded in layer order
            events = [torch.cuda.Event() for _ in range(shape.num_layers)]
            for e in events:
                e.record()
            ok = w.push_kv("decode0", desc_bytes, pairs_src, post_events=events, layers_per_launch=3)
        else:
            ok = w.push_kv("decode0", desc_bytes, pairs_src)
        w.push_stream.synchronize()
        w.close()
        q.put(("ok", ok))
    except Exception as e:  # pragma: no cover - reported to the parent
        q.put(("error", repr(e)))


@pytest.mark.parametrize("layered", [False, True])
def test_push_kv_from_another_process(layered):
    """get_descriptors on the decode side, push_kv from a second process (CUDA IPC mapping of
    the destination cache), surplus remote blocks dropped as in the reference; in one launch, and
    layer by layer behind per-layer events."""
    shape = W.SHAPES["llama31_70b_tp8"].scaled(num_layers=4, num_blocks=64)
    dst_words, dst = make_gpu_cache(shape, 81)
    decode = KVWorker("decode0", dst)
    reserved = [5, 9, 33, 2, 60, 61]          # two more than will be pushed
    src_blocks = [7, 8, 40, 41]
    desc = decode.get_descriptors(reserved)
    torch.cuda.synchronize()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_pusher, args=(desc, 82, src_blocks, q, layered))
    p.start()
    status, payload = q.get(timeout=300)
    p.join(timeout=60)
    assert status == "ok" and payload is True, payload
    torch.cuda.synchronize()
    src_words = W.normal_words(np.random.default_rng(82), shape.cache_shape, shape.dtype)
    want = dst_words.copy()
    cache_oracle.transfer(src_words, want, np.stack([src_blocks, reserved[:4]], axis=1))
    assert np.array_equal(to_words(dst), want)
    decode.close()


def test_push_and_pull_refuse_ids_and_descriptors_that_do_not_fit(capsys):
    """Block ids outside either cache, a descriptor of another geometry and bytes that are no
    descriptor are refused on the host with ``False`` and a printed reason; nothing is written
    to the peer (the reference prints and returns False for a failed transfer,
    ``kv_worker.py:396-409``)."""
    from lmserve_b200.kv_worker import CacheDescriptor
    shape = W.SHAPES["llama31_70b_tp8"].scaled(num_layers=3, num_blocks=32)
    src_words, src = make_gpu_cache(shape, 87)
    dst_words, dst = make_gpu_cache(shape.scaled(num_blocks=20), 88)
    prefill, decode = KVWorker("p", src), KVWorker("d", dst)
    try:
        with pytest.raises(IndexError):
            decode.get_descriptors([3, 20])                      # 20 is outside the 20-block cache
        descs = decode.get_descriptors([3, 4, 5])
        assert prefill.push_kv("d", descs, [1, 32]) is False      # local id out of range
        assert prefill.push_kv("d", descs, [1, -1]) is False
        assert prefill.push_kv("d", descs, [1, 2, 3, 4]) is False  # more blocks than reserved
        forged = CacheDescriptor.deserialize(descs)
        forged.block_ids = [3, 25]                                # remote id outside the peer cache
        assert prefill.push_kv("d", forged.serialize(), [1, 2]) is False
        assert decode.pull_kv("p", prefill.get_descriptors([0, 1]), [2, 20]) is False
        other = CacheDescriptor.deserialize(descs)
        other.chunk_bytes *= 2                                    # another geometry
        assert prefill.push_kv("d", other.serialize(), [1]) is False
        assert prefill.push_kv("d", b"not a descriptor", [1]) is False
        out = capsys.readouterr().out
        assert out.count("Creating transfer failed.") == 7
        torch.cuda.synchronize()
        assert np.array_equal(to_words(dst), dst_words) and np.array_equal(to_words(src), src_words)
        assert prefill.push_kv("d", descs, [1, 2]) is True        # and a good one still works
        prefill.push_stream.synchronize()
        want = dst_words.copy()
        cache_oracle.transfer(src_words, want, np.array([[1, 3], [2, 4]]))
        assert np.array_equal(to_words(dst), want)
    finally:
        prefill.close()
        decode.close()


@pytest.mark.parametrize("variant", [0, 1, 2, 3, 4])
def test_chunk_ops_do_not_touch_memory_around_their_buffers(variant):
    """copy_blocks, swap-in and transfer run on caches that are slices of larger buffers; the
    guard blocks before and after (and the host pool's neighbours) must come out unchanged,
    including when the first and the last block of the cache are destinations."""
    lib = _lib.lib()
    for key in (_lib.TUNE_COPY_VARIANT, _lib.TUNE_XFER_VARIANT, _lib.TUNE_SWAP_VARIANT):
        lib.lms_set_tuning(key, variant)
    L_, NB, chunk_words, G = 3, 10, 2064, 2            # 4128-byte chunks
    rng = np.random.default_rng(88)

    def guarded():
        words = rng.integers(0, 2**16, size=(L_, NB + 2 * G, chunk_words), dtype=np.uint16)
        big = to_tensor(words, "fp16", DEV)
        return words, big, big[:, G:G + NB]

    words, big, kv = guarded()
    pairs = np.array([[4, 0], [4, NB - 1], [5, 3]], dtype=np.int64)
    cache_ops.copy_blocks(kv, pairs)
    want = words.copy()
    cache_oracle.copy_blocks(want[:, G:G + NB], pairs)
    torch.cuda.synchronize()
    assert np.array_equal(to_words(big), want)

    pool = HostPool(6, L_, chunk_words * 2)
    try:
        pool.array[...] = rng.integers(0, 256, size=pool.array.shape, dtype=np.uint8)
        host_before = pool.array.copy()
        in_pairs = np.array([[2, 0], [5, NB - 1]], dtype=np.int64)
        cache_ops.swap_blocks(kv, pool, in_pairs, "in")
        cache_oracle.swap_in(want[:, G:G + NB], host_before.view(np.uint16), in_pairs)
        torch.cuda.synchronize()
        assert np.array_equal(to_words(big), want)
        assert np.array_equal(pool.array, host_before)
        out_pairs = np.array([[0, 1], [NB - 1, 4]], dtype=np.int64)
        cache_ops.swap_blocks(kv, pool, out_pairs, "out")
        torch.cuda.synchronize()
        host_want = host_before.copy().view(np.uint16)
        cache_oracle.swap_out(want[:, G:G + NB], host_want, out_pairs)
        assert np.array_equal(pool.array.view(np.uint16), host_want)
        assert np.array_equal(to_words(big), want)
    finally:
        pool.close()

    dwords, dbig, dst = guarded()
    tp = np.array([[NB - 1, 0], [0, NB - 1], [3, 5]], dtype=np.int64)
    cache_ops.transfer_blocks(kv, dst, tp)
    dwant = dwords.copy()
    cache_oracle.transfer(want[:, G:G + NB], dwant[:, G:G + NB], tp)
    torch.cuda.synchronize()
    assert np.array_equal(to_words(dbig), dwant)
    assert np.array_equal(to_words(big), want)
