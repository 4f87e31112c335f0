"""CPU: host-side logic around the kernels — block-map flattening, workload generators,
the KVWorker mapping helpers, and the refusal to run on CPU tensors."""
import numpy as np
import pytest
import torch

import workloads as W
from lmserve_b200.kv_worker import (BlockMapping, BlockMappingEntry, CacheDescriptor, Device,
                                    mappings_to_pairs)
from lmserve_b200.ops import cache_ops
from oracle import cache_oracle


def test_flatten_block_map_matches_reference_order():
    d = {7: [1, 2, 3], 4: [], 9: [0]}
    got = cache_ops.flatten_block_map(d)
    assert got.dtype == np.int64
    assert got.tolist() == [[7, 1], [7, 2], [7, 3], [9, 0]]
    assert np.array_equal(got, cache_oracle.flatten_block_map(d))
    assert cache_ops.flatten_block_map({}).shape == (0, 2)
    assert cache_ops.flatten_block_map([]).shape == (0, 2)
    assert cache_ops.flatten_block_map([(1, 2), (3, 4)]).tolist() == [[1, 2], [3, 4]]
    with pytest.raises(ValueError):
        cache_ops.flatten_block_map([1, 2, 3])
    with pytest.raises(TypeError):
        cache_ops.flatten_block_map(np.zeros((2, 2), dtype=np.float32))


def test_c_and_python_flatteners_agree(monkeypatch):
    assert cache_ops._packer is not None, "lmserve_b200/_packer.so is not built (python -m lmserve_b200.build)"
    rng = np.random.default_rng(3)
    d = {int(s): [int(x) for x in rng.integers(0, 1 << 40, size=int(rng.integers(0, 9)))]
         for s in rng.permutation(100)[:40]}
    d[5] = (7, 8)                         # tuples and arrays as destination lists
    d[6] = np.array([9, 10], dtype=np.int32)
    ms = [BlockMapping([BlockMappingEntry(int(a), int(b)) for a, b in rng.integers(0, 1 << 31, size=(50, 2))]),
          BlockMapping(), BlockMapping.from_pairs([(5, 6)])]
    fast_d, fast_m = cache_ops.flatten_block_map(d), mappings_to_pairs(ms)
    it = cache_ops.flatten_block_map({3: iter([4, 5])})      # no len(): handled without the C helper
    monkeypatch.setattr(cache_ops, "_packer", None)
    assert np.array_equal(fast_d, cache_ops.flatten_block_map(d))
    assert np.array_equal(fast_m, mappings_to_pairs(ms))
    assert it.tolist() == [[3, 4], [3, 5]]
    monkeypatch.undo()
    with pytest.raises(TypeError):
        cache_ops.flatten_block_map({1: [2.5]})
    with pytest.raises(TypeError):
        cache_ops.flatten_block_map({"a": [2]})


def test_cache_block_counts_follow_the_reference_arithmetic():
    from lmserve_b200.kv_worker import cache_block_counts
    # Llama-3.1-8B: 32 layers, 8 KV heads of 128, block 16, bf16 -> 32 KiB per K (or V) half,
    # 2 MiB per block over all layers (model_worker.py:215-220)
    g, h, kvb = cache_block_counts(128 << 30, 256 << 30, 32, 8, 128, 16, torch.bfloat16)
    assert (g, h, kvb) == (65536, 131072, 32768)
    g, h, kvb = cache_block_counts((2 << 20) * 7 + 5, 0, 32, 8, 128, 16, torch.float16)
    assert (g, h) == (7, 0)
    assert cache_block_counts(100, 100, 1, 8, 64, 16, torch.float16)[:2] == (0, 0)


def test_disk_pool_file_is_reused_or_replaced(tmp_path):
    from lmserve_b200.kv_worker import open_disk_pool
    f = str(tmp_path / "sub" / "disk-kv-cache-0.npy")
    a = open_disk_pool(f, (4, 2, 64))
    assert a.shape == (4, 2, 64) and a.dtype == np.uint8
    a[1, 1, :] = 7
    a.flush()
    del a
    b = open_disk_pool(f, (4, 2, 64))            # same geometry: contents survive
    assert (b[1, 1] == 7).all()
    del b
    c = open_disk_pool(f, (5, 2, 64))            # geometry changed: a new, empty file
    assert c.shape == (5, 2, 64) and not c.any()
    del c
    (tmp_path / "junk.npy").write_bytes(b"not an npy file")
    d = open_disk_pool(str(tmp_path / "junk.npy"), (1, 1, 16))
    assert d.shape == (1, 1, 16)


def test_mappings_to_pairs():
    ms = [BlockMapping([BlockMappingEntry(1, 2), BlockMappingEntry(3, 4)]), BlockMapping(),
          BlockMapping.from_pairs([(5, 6)])]
    assert mappings_to_pairs(ms).tolist() == [[1, 2], [3, 4], [5, 6]]
    assert mappings_to_pairs([]).shape == (0, 2)
    assert Device.GPU == 0 and Device.Host == 1 and Device.Disk == 2


def test_ops_reject_cpu_tensors():
    k = torch.zeros(4, 2, 8, dtype=torch.float16)
    c = torch.zeros(16, 2, 8, dtype=torch.float16)
    s = torch.arange(4)
    with pytest.raises(RuntimeError, match="no CPU path"):
        cache_ops.fill_key_cache(k, k, c, c, s)
    with pytest.raises(RuntimeError, match="no CPU path"):
        cache_ops.copy_blocks(torch.zeros(1, 4, 2, 2, 2, 8), {0: [1]})
    with pytest.raises(RuntimeError, match="no CPU path"):
        cache_ops.reshape_and_cache(k, k, torch.zeros(4, 2, 4, 2, 8, dtype=torch.float16), s)


def test_descriptor_roundtrip():
    d = CacheDescriptor(b"\x01" * 64, 256, 3, 80, 1000, 1 << 23, 8192, 8192, [5, 9, 2])
    e = CacheDescriptor.deserialize(d.serialize())
    assert e == d
    assert CacheDescriptor.deserialize(CacheDescriptor(b"\x02" * 64, 0, 0, 1, 1, 16, 16, 16, []).serialize()).block_ids == []


def test_descriptor_rejects_anything_that_is_not_a_descriptor():
    """The descriptor arrives over RPC: it is a fixed binary layout, and bytes that do not
    fit it are refused (no object deserialization happens on the way)."""
    import pickle
    good = CacheDescriptor(b"\x01" * 64, 256, 3, 80, 1000, 1 << 23, 8192, 8192, [5, 9, 2]).serialize()
    for bad in (b"", good[:40], good[:-1], good + b"\x00", b"XXXX" + good[4:],
                pickle.dumps({"handle": b"x"}), good[:4] + b"\xff" * 8 + good[12:]):
        with pytest.raises(ValueError):
            CacheDescriptor.deserialize(bad)
    with pytest.raises(ValueError):
        CacheDescriptor(b"short", 0, 0, 1, 1, 16, 16, 16, []).serialize()


class _FakeEvent:
    def __init__(self, log, name):
        self.log, self.name = log, name

    def record(self, stream=None):
        self.log.append(("record", self.name))


class _FakeStream:
    def __init__(self, log):
        self.log = log

    def wait_event(self, e):
        self.log.append(("wait", e.name))


def test_layer_handshake_waiter_issued_before_the_record():
    """The model's pre-hook runs BEFORE the KV side has recorded this step's event (the order a
    two-process deployment produces at will): the hook must hold its stream wait back until
    the recorder's token arrives, because a stream wait binds to whatever record was issued
    last.  Fake events and streams, two host threads."""
    import queue
    import threading
    import time
    from lmserve_b200.kv_worker import KVWorkerHandle
    log = []
    pre = [_FakeEvent(log, f"pre{i}") for i in range(3)]
    post = [_FakeEvent(log, f"post{i}") for i in range(3)]
    h = KVWorkerHandle(pre, post, model_queue=queue.Queue(), kv_queue=queue.Queue())
    stream = _FakeStream(log)

    def kv_side():
        time.sleep(0.2)
        for i in range(3):
            pre[i].record()
            h.model_queue.put(b"")
            time.sleep(0.02)

    t = threading.Thread(target=kv_side)
    t.start()
    for i in range(3):
        h.wait_before_layer(i, stream)       # issued at once, long before the first record
    t.join()
    for i in range(3):
        assert log.index(("record", f"pre{i}")) < log.index(("wait", f"pre{i}"))
    # the other direction: the model records, then tells the KV side
    log.clear()
    for i in range(3):
        h.record_after_layer(i, stream)
    assert h.kv_queue.qsize() == 3 and [x for x in log] == [("record", f"post{i}") for i in range(3)]


def test_layer_handshake_times_out_instead_of_hanging(monkeypatch):
    import queue
    from lmserve_b200 import kv_worker
    monkeypatch.setattr(kv_worker, "HANDSHAKE_TIMEOUT_S", 0.05)
    log = []
    h = kv_worker.KVWorkerHandle([_FakeEvent(log, "pre0")], [], model_queue=queue.Queue())
    with pytest.raises(TimeoutError, match="pre_events"):
        h.wait_before_layer(0, _FakeStream(log))
    assert log == []                             # no wait was issued on a stale event


@pytest.mark.parametrize("cfg", ["config2", "config5_decode"])
def test_decode_write_workload_invariants(cfg):
    w = getattr(W, cfg)()
    s = w.shape
    assert w.slot_mapping.dtype == np.int64
    assert len(np.unique(w.slot_mapping)) == w.num_tokens           # distinct slots
    assert w.slot_mapping.min() >= 0 and w.slot_mapping.max() < s.num_blocks * s.block_size
    # slot = table[pos // BS] * BS + pos % BS with pos = context length
    for t, c, sl in zip(w.tables.tables, w.context_lens, w.slot_mapping):
        assert sl == t[c // s.block_size] * s.block_size + c % s.block_size
        assert len(t) == (c + 1 + s.block_size - 1) // s.block_size
    alloc = w.tables.allocated
    assert len(np.unique(alloc)) == len(alloc)                      # no block dealt twice
    assert not np.intersect1d(alloc, w.tables.free).size


def test_config_sizes_match_the_specification():
    assert W.config2().algorithmic_bytes() == 64 << 20
    assert W.config2().algorithmic_bytes(layers=1) == 2 << 20
    c3 = W.config3()
    assert len(c3.slot_mapping) == 32768 and len(c3.pairs) == 4096
    assert c3.write_bytes(layers=1) == 128 << 20
    assert c3.cow_bytes() == (4096 + 32) * 28 * 32768
    assert W.config4().bytes_per_direction() == 16 << 30
    assert W.config5_decode().algorithmic_bytes() == 40 << 20
    assert W.config5_transfer().bytes() == 2560 << 20
    assert W.SHAPES["llama31_8b"].cache_bytes == 128 << 30
    assert W.SHAPES["llama31_8b"].chunk_bytes == 65536


def test_prefill_cow_workload_invariants():
    w = W.config3()
    s = w.shape
    assert len(np.unique(w.slot_mapping)) == len(w.slot_mapping)
    src, dst = w.pairs[:, 0], w.pairs[:, 1]
    assert len(np.unique(dst)) == len(dst) == 4096
    assert len(np.unique(src)) == 32
    assert not np.intersect1d(src, dst).size
    assert np.all(np.bincount(np.unique(src, return_inverse=True)[1]) == 128)
    # destinations come from the free list, sources from allocated blocks
    assert np.isin(src, w.tables.allocated).all() and np.isin(dst, w.tables.free).all()
    # runs of consecutive slots inside a block
    runs = np.diff(w.slot_mapping.reshape(64, 512), axis=1)
    assert (runs == 1).mean() > 0.9


def test_swap_and_transfer_workload_invariants():
    w = W.config4(num_host_blocks=16384, n_blocks=1024)
    assert len(np.unique(w.out_pairs[:, 0])) == 1024 and len(np.unique(w.out_pairs[:, 1])) == 1024
    assert sorted(w.in_pairs[:, 0]) == sorted(w.out_pairs[:, 1])      # the same host blocks come back
    assert not np.intersect1d(w.in_pairs[:, 1], w.out_pairs[:, 0]).size
    t = W.config5_transfer()
    assert len(t.pairs) == 4096 and len(np.unique(t.pairs[:, 1])) == 4096
    assert [W.transfer_peer(r, 8) for r in (0, 3, 4, 7)] == [("prefill", 4), ("prefill", 7),
                                                             ("decode", 0), ("decode", 3)]
    assert W.transfer_peer(0, 2) == ("prefill", 1) and W.transfer_peer(1, 2) == ("decode", 0)
    assert W.transfer_peer(0, 1) == ("none", None)


def test_plumbing_case_matches_its_description():
    c = W.config1()
    assert len(c.slot_mapping) == 256 and int((c.slot_mapping < 0).sum()) == 16
    live = c.slot_mapping[c.slot_mapping >= 0]
    assert len(np.unique(live)) == 240
    assert len(c.pairs) == 64 and len(np.unique(c.pairs[:, 1])) == 64
    assert not np.intersect1d(c.pairs[:, 0], c.pairs[:, 1]).size


def test_bf16_rounding_matches_torch():
    x = np.random.default_rng(0).standard_normal(4096).astype(np.float32)
    ours = W.f32_to_bf16_bits(x)
    ref = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(ours, ref)


def test_host_topology_reads_link_and_local_cpus_from_sysfs(tmp_path, monkeypatch):
    """PCIe link and local CPU list come from the PCI device's sysfs directory (a fake one
    here); the affinity is the intersection with what the process may use, and nothing is
    touched when sysfs has no answer."""
    import os
    from lmserve_b200 import host_topology as H
    assert H.parse_cpu_list("0-3,8,10-11") == [0, 1, 2, 3, 8, 10, 11]
    monkeypatch.setattr(H, "pci_address", lambda i: "0000:1b:00.0")
    d = tmp_path / "0000:1b:00.0"
    d.mkdir()
    (d / "current_link_speed").write_text("32.0 GT/s PCIe\n")
    (d / "current_link_width").write_text("16\n")
    allowed = sorted(os.sched_getaffinity(0))
    (d / "local_cpulist").write_text(f"{allowed[0]},4000-4001\n")
    info = H.pcie_link(0, str(tmp_path))
    assert info["current_link_speed"] == "32.0 GT/s PCIe" and info["current_link_width"] == "16"
    assert info["max_link_speed"] is None
    assert H.local_cpus(0, str(tmp_path)) == [allowed[0], 4000, 4001]
    try:
        assert H.set_cpu_affinity_for_gpu(0, str(tmp_path)) == [allowed[0]]
        assert sorted(os.sched_getaffinity(0)) == [allowed[0]]
    finally:
        os.sched_setaffinity(0, allowed)
    (d / "local_cpulist").write_text("\n")
    assert H.set_cpu_affinity_for_gpu(0, str(tmp_path)) is None
    monkeypatch.setattr(H, "pci_address", lambda i: None)
    assert H.pcie_link(0, str(tmp_path)) == {"pci_address": None}


def _late_recorder(model_queue, kv_queue, layers, delay, log_queue):
    """Child = the KV process of the CPU handshake test: it 'records' each pre-event (reports it
    on log_queue) and only then puts the token; afterwards it takes the model's post tokens."""
    import time
    time.sleep(delay)
    for l in range(layers):
        log_queue.put(("record", f"pre{l}", time.monotonic()))
        model_queue.put(b"")
    got = 0
    for l in range(layers):
        kv_queue.get(timeout=30)
        got += 1
    log_queue.put(("post_tokens", got, time.monotonic()))


def test_layer_handshake_across_two_processes_with_queues_only():
    """The reference's two-process layout without a GPU: the token queues of ``init_cache``
    (spawn context) carry the 'recorded' signal across the process boundary; the model side's
    waits are issued only after the KV process has reported its records."""
    import multiprocessing as mp
    import time
    from lmserve_b200.kv_worker import KVWorkerHandle
    ctx = mp.get_context("spawn")
    model_queue, kv_queue, log_queue = ctx.Queue(), ctx.Queue(), ctx.Queue()
    log = []
    L_ = 3
    handle = KVWorkerHandle([_FakeEvent(log, f"pre{i}") for i in range(L_)],
                            [_FakeEvent(log, f"post{i}") for i in range(L_)],
                            model_queue=model_queue, kv_queue=kv_queue)
    p = ctx.Process(target=_late_recorder, args=(model_queue, kv_queue, L_, 0.5, log_queue))
    p.start()
    waited_at = []
    stream = _FakeStream(log)
    for l in range(L_):
        handle.wait_before_layer(l, stream)      # called at once; returns after the child's token
        waited_at.append(time.monotonic())
    for l in range(L_):
        handle.record_after_layer(l, stream)
    records = {}
    for _ in range(L_ + 1):
        kind, what, when = log_queue.get(timeout=60)
        records[what if kind == "record" else kind] = (what, when)
    p.join(timeout=30)
    assert p.exitcode == 0
    for l in range(L_):                           # CLOCK_MONOTONIC is shared by both processes
        assert records[f"pre{l}"][1] <= waited_at[l]
    assert records["post_tokens"][0] == L_
    assert [e for e in log if e[0] == "wait"] == [("wait", f"pre{l}") for l in range(L_)]


def test_plan_call_helper_goes_through_the_c_abi():
    """``_packer.call_plan`` calls ``lms_write_plan_run`` by address: a NULL plan is refused by
    the library itself (LMS_ERR_NULL), before any CUDA call, and a NULL address by the helper."""
    from lmserve_b200 import _lib, _packer
    fn = cache_ops._PLAN_RUN_ADDRESS()
    assert fn and _packer.call_plan(fn, 0, 0) == _lib.LMS_ERR_NULL
    with pytest.raises(ValueError):
        _packer.call_plan(0, 0, 0)
    with pytest.raises(TypeError):
        _packer.call_plan(fn, 0)
