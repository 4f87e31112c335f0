"""GPU: the workloads at their full specified sizes, checked through properties that do not
need a host copy of a 128 GiB cache: every written row reads back equal to its source, every
other row of the touched blocks is untouched, every copy-on-write / swapped / transferred block
equals its source block."""
import numpy as np
import pytest
import torch

from lmserve_b200 import _lib
import workloads as W
from lmserve_b200.kv_worker import HostPool
from lmserve_b200.ops import cache_ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
GiB = 1 << 30


@pytest.fixture(scope="module")
def pool():
    """One 128 GiB device buffer that every full-size cache is a view of."""
    torch.cuda.empty_cache()
    free, _ = torch.cuda.mem_get_info(0)
    want = 128 * GiB
    if free < want + 8 * GiB:
        pytest.skip(f"needs {want >> 30} GiB of free device memory, {free >> 30} GiB available")
    buf = torch.empty(want // 2, dtype=torch.bfloat16, device=DEV)
    yield buf
    del buf
    torch.cuda.empty_cache()


def view(pool, shape):
    n = int(np.prod(shape.cache_shape))
    return pool[:n].view(*shape.cache_shape)


def check_written_rows(kv, key, value, slots_np, block_size):
    """kv: [L, NB, 2, BS, H, D]; rows at live slots equal key/value, the other rows of the
    touched blocks are still zero (the touched blocks were zeroed before the write)."""
    live = slots_np >= 0
    s = torch.from_numpy(slots_np[live]).to(kv.device)
    blk, ent = s // block_size, s % block_size
    live_t = torch.from_numpy(np.nonzero(live)[0]).to(kv.device)
    got_k = kv[:, blk, 0, ent].view(torch.int16)
    got_v = kv[:, blk, 1, ent].view(torch.int16)
    assert torch.equal(got_k, key[:, live_t].view(torch.int16))
    assert torch.equal(got_v, value[:, live_t].view(torch.int16))
    ublk = torch.unique(blk)
    L = kv.shape[0]
    for l0 in range(0, L, 8):
        touched = kv[l0:l0 + 8].index_select(1, ublk).view(torch.int16)  # [<=8, nb, 2, BS, H, D]
        nz_rows = (touched != 0).any(-1).any(-1)                          # [<=8, nb, 2, BS]
        # N(0,1) rows are never all-zero, so the non-zero rows are exactly the written ones
        assert int(nz_rows.sum()) == touched.shape[0] * 2 * int(live.sum())


def test_decode_write_llama31_8b_full(pool):
    s = W.SHAPES["llama31_8b"]
    assert s.cache_bytes == 128 * GiB
    kv = view(pool, s)
    w = W.config2()
    slots_np = w.slot_mapping.copy()
    slots_np[[7, 100]] = -1
    T = len(slots_np)
    blocks = torch.from_numpy(np.unique(w.slot_mapping // 16)).to(DEV)
    kv.index_fill_(1, blocks, 0)
    key = torch.randn(s.num_layers, T, 8, 128, device=DEV, dtype=torch.bfloat16)
    value = torch.randn_like(key)
    slots = torch.from_numpy(slots_np).to(DEV)
    cache_ops.reshape_and_cache_layers(key, value, kv, slots)
    torch.cuda.synchronize()
    check_written_rows(kv, key, value, slots_np, 16)
    # the last layer lives beyond 2^31 elements per layer x 31 layers: 64-bit offsets in use
    assert kv[31].data_ptr() - kv.data_ptr() == 31 * (1 << 32)
    # per-layer entry point gives the same cache
    kv.index_fill_(1, blocks, 0)
    for l in range(s.num_layers):
        cache_ops.reshape_and_cache(key[l], value[l], kv[l], slots)
    torch.cuda.synchronize()
    check_written_rows(kv, key, value, slots_np, 16)
    assert _lib.lib().lms_check_device_errors(None, None, None) == 0


def test_prefill_and_cow_qwen25_7b_full(pool):
    s = W.SHAPES["qwen25_7b"]
    kv = view(pool, s)
    w = W.config3()
    T = len(w.slot_mapping)
    blocks = torch.from_numpy(np.unique(w.slot_mapping // 16)).to(DEV)
    kv.index_fill_(1, blocks, 0)
    key = torch.randn(s.num_layers, T, 4, 128, device=DEV, dtype=torch.bfloat16)
    value = torch.randn_like(key)
    cache_ops.reshape_and_cache_layers(key, value, kv, torch.from_numpy(w.slot_mapping).to(DEV))
    torch.cuda.synchronize()
    check_written_rows(kv, key, value, w.slot_mapping, 16)
    del key, value
    # copy-on-write: 32 sources x 128 destinations, all 28 layers
    src = torch.from_numpy(w.pairs[:, 0].copy()).to(DEV)
    dst = torch.from_numpy(w.pairs[:, 1].copy()).to(DEV)
    flat = kv.view(s.num_layers, s.num_blocks, -1).view(torch.int16)
    before_src = [flat[l].index_select(0, torch.unique(src)).clone() for l in (0, 27)]
    d = {}
    for a, b in w.pairs:
        d.setdefault(int(a), []).append(int(b))
    cache_ops.copy_blocks(kv, d)
    torch.cuda.synchronize()
    for l in range(s.num_layers):
        assert torch.equal(flat[l].index_select(0, dst), flat[l].index_select(0, src)), l
    for l, b in zip((0, 27), before_src):
        assert torch.equal(flat[l].index_select(0, torch.unique(src)), b)   # sources unchanged
    assert bool((flat[0].index_select(0, src[:16]) != 0).any())            # and not trivially zero


@pytest.mark.parametrize("engine", ["kernel", "staged"])
def test_swap_round_trip_llama31_8b_full(pool, engine):
    s = W.SHAPES["llama31_8b_swap"]
    kv = view(pool, s)
    per_block = s.num_layers * s.chunk_bytes
    avail = None
    for line in open("/proc/meminfo"):
        if line.startswith("MemAvailable:"):
            avail = int(line.split()[1]) * 1024
    n_blocks = 8192
    while avail is not None and n_blocks * per_block > 0.3 * avail and n_blocks > 64:
        n_blocks //= 2
    w = W.make_swap(s, n_blocks, n_blocks, seed=1004)
    host = HostPool(n_blocks, s.num_layers, s.chunk_bytes)
    try:
        flat = kv.view(s.num_layers, s.num_blocks, -1)
        src = torch.from_numpy(w.out_pairs[:, 0].copy()).to(DEV)
        base = torch.randn(1, flat.shape[2], device=DEV, dtype=torch.float32)
        ramp = torch.arange(n_blocks, device=DEV, dtype=torch.float32)[:, None]
        for l in range(s.num_layers):
            flat[l].index_copy_(0, src, (base + ramp * (0.001 * (l + 1))).to(torch.bfloat16))
        staging = torch.empty(256 << 20, dtype=torch.uint8, device=DEV) if engine == "staged" else None
        cache_ops.swap_blocks(kv, host, w.out_pairs, "out", engine=engine, staging=staging)
        cache_ops.swap_blocks(kv, host, w.in_pairs, "in", engine=engine, staging=staging)
        torch.cuda.synchronize()
        back = {int(h): int(g) for g, h in w.out_pairs}
        src_of_dst = torch.tensor([back[int(h)] for h in w.in_pairs[:, 0]], device=DEV)
        dst = torch.from_numpy(w.in_pairs[:, 1].copy()).to(DEV)
        fi = flat.view(torch.int16)
        for l in range(s.num_layers):
            assert torch.equal(fi[l].index_select(0, dst), fi[l].index_select(0, src_of_dst)), l
        # the host pool holds the same bytes, block-major: spot-check 64 blocks on the host
        for g, h in w.out_pairs[:: max(1, n_blocks // 64)]:
            dev_block = fi[:, int(g)].cpu().numpy()
            assert np.array_equal(host.array[int(h)].view(np.int16), dev_block)
    finally:
        host.close()


def test_tp8_decode_and_transfer_llama31_70b_full(pool):
    s = W.SHAPES["llama31_70b_tp8"]
    kv = view(pool, s)                           # 100 GiB
    w = W.config5_decode(rank=3)
    T = len(w.slot_mapping)
    blocks = torch.from_numpy(np.unique(w.slot_mapping // 16)).to(DEV)
    kv.index_fill_(1, blocks, 0)
    key = torch.randn(s.num_layers, T, 1, 128, device=DEV, dtype=torch.bfloat16)
    value = torch.randn_like(key)
    cache_ops.reshape_and_cache_layers(key, value, kv, torch.from_numpy(w.slot_mapping).to(DEV))
    torch.cuda.synchronize()
    check_written_rows(kv, key, value, w.slot_mapping, 16)
    # transfer 4096 blocks x 80 layers into a second cache placed after the first
    tr = W.config5_transfer(rank=0)
    dshape = s.scaled(num_blocks=8192)
    off = int(np.prod(s.cache_shape))
    dst = pool[off: off + int(np.prod(dshape.cache_shape))].view(*dshape.cache_shape)
    pairs = tr.pairs.copy()
    pairs[:, 1] = np.random.default_rng(5).permutation(8192)[:len(pairs)]
    cache_ops.transfer_blocks(kv, dst, pairs)
    torch.cuda.synchronize()
    fs = kv.view(s.num_layers, s.num_blocks, -1).view(torch.int16)
    fd = dst.view(s.num_layers, 8192, -1).view(torch.int16)
    si, di = torch.from_numpy(pairs[:, 0].copy()).to(DEV), torch.from_numpy(pairs[:, 1].copy()).to(DEV)
    for l in range(0, s.num_layers, 7):
        assert torch.equal(fd[l].index_select(0, di), fs[l].index_select(0, si)), l
    assert _lib.lib().lms_check_device_errors(None, None, None) == 0
