"""The swap / transfer vectors that LMServe's own ``kv_worker.py`` produced on host buffers
(``tests/golden/make_swap_golden.py``): on CPU the oracle restatements must reproduce them, on
the GPU the CUDA path must — through ``swap_blocks`` / ``transfer_blocks`` and through the
``KVWorker`` mirror."""
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from helpers import load_npz
from oracle import cache_oracle, kv_worker_ref, torch_ref

SWAP_CASES = ["swap_bf16_l3", "swap_fp16_l5", "swap_empty"]
TRANSFER_CASES = ["transfer_push_surplus", "transfer_push_exact", "transfer_pull"]
DEV = "cuda:0"


def _t(words):
    return torch.from_numpy(words.view(np.int16).copy())


def _w(t):
    return t.cpu().numpy().view(np.uint16)


# ------------------------------------------------------------------------------------- CPU

@pytest.mark.parametrize("name", SWAP_CASES)
def test_oracle_swap_vs_reference_vectors(name):
    g = load_npz(name)
    gpu, host = g["gpu_in"].copy(), g["host_in"].copy()
    cache_oracle.swap_out(gpu, host, g["out_pairs"])
    assert np.array_equal(host, g["host_after_out"]) and np.array_equal(gpu, g["gpu_in"])
    cache_oracle.swap_in(gpu, host, g["in_pairs"])
    assert np.array_equal(gpu, g["gpu_after_in"]) and np.array_equal(host, g["host_after_in"])
    tg, th = _t(g["gpu_in"]), _t(g["host_in"])
    torch_ref.swap_out(tg, th, g["out_pairs"])
    assert np.array_equal(_w(th), g["host_after_out"])
    torch_ref.swap_in(tg, th, g["in_pairs"])
    assert np.array_equal(_w(tg), g["gpu_after_in"])
    # the reference waits for one post-event per layer going out and records one pre-event (and
    # queues one token) per layer coming in - none at all for an empty request
    L = g["gpu_in"].shape[0]
    n = 1 if len(g["out_pairs"]) else 0
    assert list(g["post_event_waits"]) == [n] * L and list(g["pre_event_records"]) == [n] * L
    assert int(g["model_queue_tokens"]) == n * L


def test_oracle_layer_range_vs_reference_vectors():
    g = load_npz("swap_layer2_of_4")
    l = int(g["layer"])
    gpu, host = g["gpu_in"].copy(), g["host_in"].copy()
    cache_oracle.swap_out(gpu, host, g["out_pairs"], layers=(l, l + 1))
    assert np.array_equal(host, g["host_after_out"])
    cache_oracle.swap_in(gpu, host, g["in_pairs"], layers=(l, l + 1))
    assert np.array_equal(gpu, g["gpu_after_in"])
    tg, th = _t(g["gpu_in"]), _t(g["host_in"])
    torch_ref.swap_out(tg, th, g["out_pairs"], layers=(l, l + 1))
    torch_ref.swap_in(tg, th, g["in_pairs"], layers=(l, l + 1))
    assert np.array_equal(_w(th), g["host_after_out"]) and np.array_equal(_w(tg), g["gpu_after_in"])


@pytest.mark.parametrize("name", TRANSFER_CASES)
def test_oracle_transfer_vs_reference_vectors(name):
    """The folded GPU -> GPU form of the oracle equals what the reference's write-through, NIXL
    transfer and fetch leave in the decode GPU's cache; block i of the local list lands in the
    i-th reserved remote block and surplus reservations stay untouched."""
    g = load_npz(name)
    dst = g["dst_gpu_in"].copy()
    cache_oracle.transfer(g["src_gpu"], dst, g["pairs"])
    assert np.array_equal(dst, g["dst_gpu_out"])
    td = _t(g["dst_gpu_in"])
    torch_ref.transfer(_t(g["src_gpu"]), td, g["pairs"])
    assert np.array_equal(_w(td), g["dst_gpu_out"])
    for b in g["surplus_host_blocks"]:
        assert np.array_equal(g["dst_host_out"][b], g["dst_host_in"][b])
    for i, b in enumerate(g["decode_host_blocks"]):
        assert np.array_equal(g["dst_host_out"][b], g["src_gpu"][:, g["pairs"][i, 0]])


@pytest.mark.skipif(not kv_worker_ref.available(), reason="LMServe source tree not present")
def test_swap_golden_regenerates_from_reference(tmp_path):
    """Where the reference tree is mounted, running its ``kv_worker.py`` again reproduces the
    committed vectors byte for byte."""
    root = Path(__file__).resolve().parent.parent
    code = (
        "import sys; sys.path.insert(0, %r); sys.path.insert(0, %r);"
        "import make_swap_golden as M; from pathlib import Path; M.HERE = Path(%r); M.main()"
    ) % (str(root), str(root / "tests" / "golden"), str(tmp_path))
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    for name in SWAP_CASES + TRANSFER_CASES + ["swap_layer2_of_4"]:
        a, b = load_npz(name), np.load(tmp_path / f"{name}.npz")
        assert sorted(a) == sorted(b.files)
        for k in a:
            assert np.array_equal(a[k], b[k]), (name, k)


# ------------------------------------------------------------------------------------- GPU

def _pool_from(words):
    from lmserve_b200.kv_worker import HostPool
    NHB, L, cw = words.shape
    pool = HostPool(NHB, L, cw * 2)
    pool.array.view(np.uint16)[...] = words
    return pool


@pytest.mark.gpu
@pytest.mark.parametrize("engine", ["kernel", "dma", "staged"])
@pytest.mark.parametrize("name", SWAP_CASES)
def test_gpu_swap_vs_reference_vectors(name, engine):
    from lmserve_b200.ops import cache_ops
    g = load_npz(name)
    gpu = _t(g["gpu_in"]).to(DEV)
    pool = _pool_from(g["host_in"])
    try:
        cache_ops.swap_blocks(gpu, pool, g["out_pairs"], "out", engine=engine)
        torch.cuda.synchronize()
        assert np.array_equal(pool.array.view(np.uint16), g["host_after_out"])
        cache_ops.swap_blocks(gpu, pool, g["in_pairs"], "in", engine=engine)
        torch.cuda.synchronize()
        assert np.array_equal(_w(gpu), g["gpu_after_in"])
        assert np.array_equal(pool.array.view(np.uint16), g["host_after_in"])
    finally:
        pool.close()


@pytest.mark.gpu
def test_gpu_swap_layer_range_vs_reference_vectors():
    from lmserve_b200.ops import cache_ops
    g = load_npz("swap_layer2_of_4")
    l = int(g["layer"])
    gpu = _t(g["gpu_in"]).to(DEV)
    pool = _pool_from(g["host_in"])
    try:
        cache_ops.swap_blocks(gpu, pool, g["out_pairs"], "out", layers=(l, l + 1))
        torch.cuda.synchronize()
        assert np.array_equal(pool.array.view(np.uint16), g["host_after_out"])
        cache_ops.swap_blocks(gpu, pool, g["in_pairs"], "in", layers=(l, l + 1))
        torch.cuda.synchronize()
        assert np.array_equal(_w(gpu), g["gpu_after_in"])
    finally:
        pool.close()


@pytest.mark.gpu
@pytest.mark.parametrize("engine", ["kernel", "dma", "staged"])
@pytest.mark.parametrize("name", SWAP_CASES)
def test_kv_worker_whole_block_copy_kv_vs_reference_vectors(name, engine):
    """``KVWorker.copy_kv`` without per-layer events (whole blocks in one call) in each of the
    worker's swap engines; the staged engine is given a staging ring of two blocks so that
    several groups alternate through its halves."""
    from lmserve_b200.kv_worker import BlockMapping, Device, KVWorker
    g = load_npz(name)
    L, NB, cw = g["gpu_in"].shape
    gpu = _t(g["gpu_in"]).to(DEV)
    w = KVWorker("golden", gpu, num_host_blocks=g["host_in"].shape[0], swap_engine=engine,
                 staging_bytes=2 * L * cw * 2)
    try:
        w.host_pool.array.view(np.uint16)[...] = g["host_in"]
        w.copy_kv([BlockMapping.from_pairs(g["out_pairs"])], Device.GPU, Device.Host)
        w.dtoh_stream.synchronize()
        assert np.array_equal(w.host_pool.array.view(np.uint16), g["host_after_out"])
        w.copy_kv([BlockMapping.from_pairs(g["in_pairs"])], Device.Host, Device.GPU)
        w.htod_stream.synchronize()
        assert np.array_equal(_w(gpu), g["gpu_after_in"])
        assert np.array_equal(w.host_pool.array.view(np.uint16), g["host_after_in"])
    finally:
        w.close()


@pytest.mark.gpu
@pytest.mark.parametrize("name", SWAP_CASES)
def test_kv_worker_copy_kv_vs_reference_vectors(name):
    """``KVWorker.copy_kv`` with the reference's request types and the per-layer handshake."""
    from lmserve_b200.kv_worker import BlockMapping, Device, KVWorker
    g = load_npz(name)
    L, NB, cw = g["gpu_in"].shape
    gpu = _t(g["gpu_in"]).to(DEV)
    w = KVWorker("golden", gpu, num_host_blocks=g["host_in"].shape[0])
    try:
        w.host_pool.array.view(np.uint16)[...] = g["host_in"]
        post = [torch.cuda.Event() for _ in range(L)]
        pre = [torch.cuda.Event() for _ in range(L)]
        for e in post:
            e.record()
        half = max(1, len(g["out_pairs"]) // 2)
        maps = [BlockMapping.from_pairs(g["out_pairs"][:half]), BlockMapping.from_pairs(g["out_pairs"][half:])]
        w.copy_kv(maps, Device.GPU, Device.Host, post_events=post)
        w.dtoh_stream.synchronize()
        assert np.array_equal(w.host_pool.array.view(np.uint16), g["host_after_out"])
        w.copy_kv([BlockMapping.from_pairs(g["in_pairs"])], Device.Host, Device.GPU, pre_events=pre)
        w.htod_stream.synchronize()
        assert np.array_equal(_w(gpu), g["gpu_after_in"])
    finally:
        w.close()


@pytest.mark.gpu
@pytest.mark.parametrize("name", TRANSFER_CASES)
def test_gpu_transfer_vs_reference_vectors(name):
    """Same-device form of the transfer (source and destination caches on one GPU); the
    cross-GPU form runs the same kernel on a peer mapping."""
    from lmserve_b200.ops import cache_ops
    g = load_npz(name)
    src, dst = _t(g["src_gpu"]).to(DEV), _t(g["dst_gpu_in"]).to(DEV)
    pull = name == "transfer_pull"
    cache_ops.transfer_blocks(src, dst, g["pairs"], pull=pull)
    torch.cuda.synchronize()
    assert np.array_equal(_w(dst), g["dst_gpu_out"])
    assert np.array_equal(_w(src), g["src_gpu"])


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["transfer_push_surplus", "transfer_pull"])
def test_kv_worker_push_pull_vs_reference_vectors(name):
    """``get_descriptors`` on the decode worker (with the surplus reservations of the vector),
    ``push_kv`` / ``pull_kv`` on the other: the descriptor truncation of ``kv_worker.py:386-387``
    and the block order come out as the reference's."""
    from lmserve_b200.kv_worker import KVWorker
    g = load_npz(name)
    src, dst = _t(g["src_gpu"]).to(DEV), _t(g["dst_gpu_in"]).to(DEV)
    prefill, decode = KVWorker("p", src), KVWorker("d", dst)
    try:
        if name == "transfer_pull":
            descs = prefill.get_descriptors(g["pairs"][:, 0])
            assert decode.pull_kv("p", descs, g["pairs"][:, 1]) is True
            decode.push_stream.synchronize()
        else:
            # reserve more remote blocks than are pushed; the extras must stay untouched
            used = set(int(b) for b in g["pairs"][:, 1])
            extra = [b for b in range(dst.shape[1]) if b not in used][:len(g["surplus_host_blocks"])]
            descs = decode.get_descriptors(list(g["pairs"][:, 1]) + extra)
            assert prefill.push_kv("d", descs, g["pairs"][:, 0]) is True
            prefill.push_stream.synchronize()
        torch.cuda.synchronize()
        assert np.array_equal(_w(dst), g["dst_gpu_out"])
    finally:
        prefill.close()
        decode.close()
