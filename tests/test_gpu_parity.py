"""GPU: every cache op, called through the C ABI, against the CPU oracle — bit-exact.

Covers the golden vectors made by LMServe's own kernels, the full-size plumbing case, scaled
versions of the decode / chunked-prefill / TP-sharded workloads in every kernel variant, and
the edge cases: empty input, all-padding, single token, last slot of the pool, row and block
sizes that are not powers of two, strided inputs, guard regions around the cache, block
strides beyond 2^31 elements, and out-of-range indices under debug checks."""
import ctypes

import numpy as np
import pytest
import torch

from helpers import COPY_CASES, FILL_CASES, load_json, load_npz, sha, to_tensor, to_words
from lmserve_b200 import _lib
import workloads as W
from lmserve_b200.ops import cache_ops
from oracle import cache_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
# tiled 16/32-byte vectors, bulk (TMA) copies, untiled 32/16-byte, one-wave (K, V) pairs,
# one-wave independent vectors, persistent (K, V) pairs
VARIANTS = [0, 1, 2, 3, 4, 5, 6, 7]


@pytest.fixture(autouse=True)
def _reset_tuning():
    yield
    L = _lib.lib()
    for key in range(1, _lib.TUNE_COUNT):
        L.lms_set_tuning(key, -1)
    L.lms_set_debug_checks(0)


def set_variant(v):
    """Write-kernel variant v; the copy kernels have variants 0..2 only."""
    L = _lib.lib()
    assert L.lms_set_tuning(_lib.TUNE_WRITE_VARIANT, v) == 0
    for key in (_lib.TUNE_COPY_VARIANT, _lib.TUNE_XFER_VARIANT):
        assert L.lms_set_tuning(key, min(v, 3)) == 0


@pytest.mark.parametrize("per_thread", [1, 2, 4])
@pytest.mark.parametrize("variant", [5, 6, 7])
def test_one_wave_write_kernels_units_per_thread(variant, per_thread):
    """The one-wave write kernels with 1, 2 and 4 units per thread: 2 KiB rows, 256-byte rows,
    rows that are not a power of two, a per-layer slot table and a persistent grid of one CTA."""
    L = _lib.lib()
    set_variant(variant)
    L.lms_set_tuning(_lib.TUNE_WRITE_VPT, per_thread)
    shape = W.SHAPES["llama31_8b"].scaled(num_layers=3, num_blocks=512)
    w = W.make_decode_write(shape, 53, 16, 160, seed=131)
    slots = w.slot_mapping.copy()
    slots[5] = -1
    run_layers_case(shape, slots, 141)
    run_layers_case(shape, slots, 142, slot_per_layer=True)
    shape = W.SHAPES["llama31_70b_tp8"].scaled(num_layers=7, num_blocks=8192)
    w = W.make_decode_write(shape, 301, 64, 300, seed=135)
    run_layers_case(shape, w.slot_mapping, 145)
    odd = W.KVShape("odd", num_layers=2, num_blocks=9, num_kv_heads=5, head_dim=24, block_size=7,
                    dtype="bf16")
    rng = np.random.default_rng(146)
    slots = rng.permutation(9 * 7)[:41].astype(np.int64)
    run_layers_case(odd, slots, 147)


# ----------------------------------------------------------------- golden vectors
@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("name", FILL_CASES)
def test_fill_key_cache_golden(name, variant):
    set_variant(variant)
    g = load_npz(name)
    dt = g["dtype"]
    kc, vc = to_tensor(g["key_cache_in"], dt, DEV), to_tensor(g["value_cache_in"], dt, DEV)
    before = _lib.lib().lms_launch_count()
    cache_ops.fill_key_cache(to_tensor(g["key"], dt, DEV), to_tensor(g["value"], dt, DEV), kc, vc,
                             torch.from_numpy(g["slot_mapping"]).to(DEV))
    torch.cuda.synchronize()
    assert _lib.lib().lms_launch_count() == before + 1
    assert np.array_equal(to_words(kc), g["key_cache_out"])
    assert np.array_equal(to_words(vc), g["value_cache_out"])


@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("name", COPY_CASES)
def test_copy_blocks_golden(name, variant):
    set_variant(variant)
    g = load_npz(name)
    kv = to_tensor(g["kv_in"], g["dtype"], DEV)
    d = {}
    for s, dst in g["pairs"]:
        d.setdefault(int(s), []).append(int(dst))
    cache_ops.copy_blocks(kv, d)
    torch.cuda.synchronize()
    assert np.array_equal(to_words(kv), g["kv_out"])


@pytest.mark.parametrize("variant", VARIANTS)
def test_plumbing_case_full_size(variant):
    """Llama-3.2-1B shape, 256 tokens with 16 padded slots, 64 block pairs: digests of the
    outputs equal those of the reference kernels; padding is skipped."""
    set_variant(variant)
    g = load_json("plumbing_llama32_1b")
    case = W.config1()
    pay = W.plumbing_payload(case)
    dt = case.shape.dtype
    slots = torch.from_numpy(case.slot_mapping).to(DEV)
    kc, vc = to_tensor(pay["key_cache"], dt, DEV), to_tensor(pay["value_cache"], dt, DEV)
    key, value = to_tensor(pay["key"], dt, DEV), to_tensor(pay["value"], dt, DEV)
    cache_ops.fill_key_cache(key, value, kc, vc, slots)
    kv = to_tensor(pay["kv_caches"], dt, DEV)
    cache_ops.copy_blocks(kv, case.pairs)
    torch.cuda.synchronize()
    assert sha(to_words(kc)) == g["outputs"]["key_cache"]
    assert sha(to_words(vc)) == g["outputs"]["value_cache"]
    assert sha(to_words(kv)) == g["outputs"]["kv_caches"]
    # the interleaved layout of the same case, against the oracle
    kv2 = to_tensor(pay["kv_caches"], dt, DEV)
    cache_ops.reshape_and_cache(key, value, kv2[0], slots)
    want = pay["kv_caches"].copy()
    cache_oracle.reshape_and_cache(pay["key"], pay["value"], want[0], case.slot_mapping)
    torch.cuda.synchronize()
    assert np.array_equal(to_words(kv2), want)


# ----------------------------------------------------------------- multi-layer writes
def run_layers_case(shape, slots_np, seed, slot_per_layer=False):
    rng = np.random.default_rng(seed)
    L, T = shape.num_layers, len(slots_np)
    key = W.normal_words(rng, (L, T, shape.num_kv_heads, shape.head_dim), shape.dtype)
    value = W.normal_words(rng, (L, T, shape.num_kv_heads, shape.head_dim), shape.dtype)
    cache = W.normal_words(rng, shape.cache_shape, shape.dtype)
    if slot_per_layer:
        slots_np = np.stack([np.roll(slots_np, l) for l in range(L)])
    want = cache.copy()
    cache_oracle.reshape_and_cache_layers(key, value, want, slots_np)
    got = to_tensor(cache, shape.dtype, DEV)
    cache_ops.reshape_and_cache_layers(to_tensor(key, shape.dtype, DEV),
                                       to_tensor(value, shape.dtype, DEV), got,
                                       torch.from_numpy(slots_np).to(DEV))
    torch.cuda.synchronize()
    assert np.array_equal(to_words(got), want)


@pytest.mark.parametrize("variant", VARIANTS)
def test_decode_write_scaled(variant):
    set_variant(variant)
    shape = W.SHAPES["llama31_8b"].scaled(num_layers=4, num_blocks=512)
    w = W.make_decode_write(shape, 48, 16, 160, seed=31)
    run_layers_case(shape, w.slot_mapping, 41)
    run_layers_case(shape, w.slot_mapping, 42, slot_per_layer=True)


@pytest.mark.parametrize("variant", VARIANTS)
def test_chunked_prefill_scaled(variant):
    set_variant(variant)
    shape = W.SHAPES["qwen25_7b"].scaled(num_layers=3, num_blocks=1024)
    w = W.make_prefill_cow(shape, 6, 200, 1500, 4, 8, seed=33)
    slots = w.slot_mapping.copy()
    slots[::37] = -1
    run_layers_case(shape, slots, 43)


@pytest.mark.parametrize("variant", VARIANTS)
def test_tp_sharded_decode_write_scaled(variant):
    """One KV head per GPU (256-byte rows), the TP=8 shape."""
    set_variant(variant)
    shape = W.SHAPES["llama31_70b_tp8"].scaled(num_layers=5, num_blocks=2048)
    w = W.make_decode_write(shape, 100, 64, 300, seed=35)
    run_layers_case(shape, w.slot_mapping, 45)


@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("tile", [0, 2048, 1 << 20])
def test_write_tile_sizes(variant, tile):
    set_variant(variant)
    _lib.lib().lms_set_tuning(_lib.TUNE_WRITE_TILE_BYTES, tile)
    shape = W.SHAPES["llama31_8b"].scaled(num_layers=2, num_blocks=640)
    w = W.make_decode_write(shape, 37, 8, 200, seed=36)
    run_layers_case(shape, w.slot_mapping, 46)


# ----------------------------------------------------------------- edge cases
@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("H,D,BS", [(3, 8, 12), (1, 8, 16), (5, 24, 7), (3, 256, 16)])
def test_odd_geometries(variant, H, D, BS):
    """Rows of 48 / 16 / 240 / 1536 bytes, block sizes that are not powers of two."""
    set_variant(variant)
    shape = W.KVShape("odd", 2, H, D, "fp16", 9, BS)
    rng = np.random.default_rng(7)
    slots = rng.permutation(9 * BS)[:20].astype(np.int64)
    slots[[2, 11]] = -1
    slots[0] = 9 * BS - 1  # the last slot of the pool
    run_layers_case(shape, slots, 47)


@pytest.mark.parametrize("variant", VARIANTS)
def test_empty_all_padding_and_single_token(variant):
    set_variant(variant)
    shape = W.KVShape("tiny", 2, 2, 64, "bf16", 8)
    for slots in (np.empty(0, np.int64), np.full(5, -1, np.int64), np.array([77], np.int64)):
        run_layers_case(shape, slots, 48)
    kv = torch.randn(2, 8, 2, 16, 2, 64, device=DEV).to(torch.bfloat16)
    ref = kv.clone()
    cache_ops.copy_blocks(kv, {})
    cache_ops.copy_blocks(kv, np.empty((0, 2), np.int64))
    torch.cuda.synchronize()
    assert torch.equal(kv.view(torch.int16), ref.view(torch.int16))


@pytest.mark.parametrize("variant", VARIANTS)
def test_strided_key_value_and_guard_regions(variant):
    """key/value are slices of a fused qkv projection (token stride > row); the cache is a
    slice of a larger buffer whose guard blocks on both sides must stay untouched."""
    set_variant(variant)
    T, H, D, BS, NB = 33, 4, 64, 16, 10
    rng = np.random.default_rng(8)
    qkv = to_tensor(W.normal_words(rng, (T, 3 * H * D), "bf16"), "bf16", DEV)
    key = qkv[:, H * D:2 * H * D].view(T, H, D)
    value = qkv[:, 2 * H * D:].view(T, H, D)
    big_words = W.normal_words(rng, (NB + 4, 2, BS, H, D), "bf16")
    big = to_tensor(big_words, "bf16", DEV)
    cache = big[2:NB + 2]
    slots = rng.permutation(NB * BS)[:T].astype(np.int64)
    slots[5] = -1
    slots[0], slots[1] = 0, NB * BS - 1  # first and last slot, next to the guards
    cache_ops.reshape_and_cache(key, value, cache, torch.from_numpy(slots).to(DEV))
    want = big_words.copy()
    cache_oracle.reshape_and_cache(to_words(key), to_words(value), want[2:NB + 2], slots)
    torch.cuda.synchronize()
    got = to_words(big)
    assert np.array_equal(got[:2], big_words[:2]) and np.array_equal(got[NB + 2:], big_words[NB + 2:])
    assert np.array_equal(got, want)


def test_int32_slot_mapping_is_accepted():
    g = load_npz("fill_fp16_t8")
    kc, vc = to_tensor(g["key_cache_in"], "fp16", DEV), to_tensor(g["value_cache_in"], "fp16", DEV)
    cache_ops.fill_key_cache(to_tensor(g["key"], "fp16", DEV), to_tensor(g["value"], "fp16", DEV),
                             kc, vc, torch.from_numpy(g["slot_mapping"].astype(np.int32)).to(DEV))
    torch.cuda.synchronize()
    assert np.array_equal(to_words(kc), g["key_cache_out"])


@pytest.mark.parametrize("variant", VARIANTS)
def test_block_stride_beyond_2_31_elements(variant):
    """Two cache blocks 2.5 Gi elements apart inside one 5.1 GiB buffer: offsets need 64 bits."""
    set_variant(variant)
    H, D, BS, T = 8, 128, 16, 24
    far = 5 * (1 << 29)  # elements between the two blocks (2.5 Gi)
    buf = torch.zeros(far + 2 * BS * H * D + 64, dtype=torch.bfloat16, device=DEV)
    cache = torch.as_strided(buf, (1, 2, 2, BS, H, D),
                             (far * 2, far, BS * H * D, H * D, D, 1))
    rng = np.random.default_rng(10)
    key_w, val_w = W.normal_words(rng, (T, H, D), "bf16"), W.normal_words(rng, (T, H, D), "bf16")
    slots = np.concatenate([np.arange(0, 12), BS + np.arange(4, 16)]).astype(np.int64)
    cache_ops.reshape_and_cache_layers(to_tensor(key_w, "bf16", DEV)[None],
                                       to_tensor(val_w, "bf16", DEV)[None], cache,
                                       torch.from_numpy(slots).to(DEV))
    torch.cuda.synchronize()
    want = np.zeros((2, 2, BS, H, D), np.uint16)
    cache_oracle.reshape_and_cache(key_w, val_w, want, slots)
    got = to_words(cache[0].contiguous())
    assert np.array_equal(got, want)
    # nothing landed where a 32-bit wrap of the far block's offset would point
    wrapped = (far * 2) % (1 << 32) // 2
    assert not buf[wrapped:wrapped + 2 * BS * H * D].view(torch.int16).any()
    # copy_blocks across the same distance
    kv3 = torch.as_strided(buf, (1, 2, 2 * BS * H * D), (far * 2, far, 1))
    cache_ops.copy_blocks(kv3, [(1, 0)])
    torch.cuda.synchronize()
    assert np.array_equal(to_words(kv3[0, 0]), want[1].reshape(-1))


# ----------------------------------------------------------------- copy-on-write
@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("per_sm", [0, 1, 16])
def test_copy_blocks_fanout_scaled(variant, per_sm):
    set_variant(variant)
    _lib.lib().lms_set_tuning(_lib.TUNE_COPY_CTAS_PER_SM, per_sm)
    shape = W.SHAPES["qwen25_7b"].scaled(num_layers=3, num_blocks=700)
    w = W.make_prefill_cow(shape, 4, 100, 900, 5, 40, seed=51)
    words = W.normal_words(np.random.default_rng(52), shape.cache_shape, shape.dtype)
    kv = to_tensor(words, shape.dtype, DEV)
    cache_ops.copy_blocks(kv, w.pairs)
    want = words.copy()
    cache_oracle.copy_blocks(want, w.pairs)
    torch.cuda.synchronize()
    assert np.array_equal(to_words(kv), want)


@pytest.mark.parametrize("variant", VARIANTS)
def test_copy_blocks_odd_chunk_and_many_pairs(variant):
    """Chunk of 48 KiB + 16 bytes (not a multiple of the slice), more pairs than one staging round."""
    set_variant(variant)
    L, NB, chunk_words = 2, 900, (48 * 1024 + 16) // 2
    rng = np.random.default_rng(53)
    words = rng.integers(0, 2**16, size=(L, NB, chunk_words), dtype=np.uint16)
    kv = to_tensor(words, "fp16", DEV)
    perm = rng.permutation(NB)
    pairs = np.stack([perm[:10].repeat(40), perm[10:410]], axis=1).astype(np.int64)
    cache_ops.copy_blocks(kv, pairs)
    want = words.copy()
    cache_oracle.copy_blocks(want, pairs)
    torch.cuda.synchronize()
    assert np.array_equal(to_words(kv), want)


# ----------------------------------------------------------------- debug checks
def test_debug_checks_report_bad_slot_and_skip_it():
    L = _lib.lib()
    assert L.lms_set_debug_checks(1) == 0
    T, H, D, NS = 6, 2, 32, 40
    key = torch.randn(T, H, D, device=DEV).half()
    kc = torch.zeros(NS, H, D, device=DEV).half()
    vc = torch.zeros_like(kc)
    guard = torch.zeros(64, H, D, device=DEV).half()  # likely neighbours in the allocator
    slots = torch.tensor([0, 1, NS + 3, 5, -1, 7], device=DEV)
    cache_ops.fill_key_cache(key, key, kc, vc, slots)
    idx, val = ctypes.c_int64(-1), ctypes.c_int64(-1)
    rc = L.lms_check_device_errors(None, ctypes.byref(idx), ctypes.byref(val))
    assert rc == _lib.LMS_ERR_INDEX and idx.value == 2 and val.value == NS + 3
    assert L.lms_check_device_errors(None, None, None) == 0  # cleared
    assert torch.equal(kc[[0, 1, 5, 7]], key[[0, 1, 3, 5]])
    assert not guard.any()
    with pytest.raises(_lib.LmsError):
        _lib.check(rc)


def test_debug_checks_report_bad_block_pair():
    L = _lib.lib()
    L.lms_set_debug_checks(1)
    kv = torch.randn(2, 6, 2, 4, 2, 16, device=DEV).half()
    ref = kv.clone()
    cache_ops.copy_blocks(kv, [(0, 1), (9, 2), (3, 4)])
    idx, val = ctypes.c_int64(), ctypes.c_int64()
    assert L.lms_check_device_errors(None, ctypes.byref(idx), ctypes.byref(val)) == _lib.LMS_ERR_INDEX
    assert (idx.value, val.value) == (1, 9)
    assert torch.equal(kv[:, 1], ref[:, 0]) and torch.equal(kv[:, 4], ref[:, 3])
    assert torch.equal(kv[:, 2], ref[:, 2])
    cache_ops.copy_blocks(kv, [(0, 7)])
    assert L.lms_check_device_errors(None, ctypes.byref(idx), ctypes.byref(val)) == _lib.LMS_ERR_INDEX
    assert (idx.value, val.value) == (0, 7)


def test_runs_on_the_callers_stream():
    s = torch.cuda.Stream()
    g = load_npz("fill_bf16_t24")
    kc, vc = to_tensor(g["key_cache_in"], "bf16", DEV), to_tensor(g["value_cache_in"], "bf16", DEV)
    key, value = to_tensor(g["key"], "bf16", DEV), to_tensor(g["value"], "bf16", DEV)
    slots = torch.from_numpy(g["slot_mapping"]).to(DEV)
    torch.cuda.synchronize()
    with torch.cuda.stream(s):
        cache_ops.fill_key_cache(key, value, kc, vc, slots)
    s.synchronize()
    assert np.array_equal(to_words(kc), g["key_cache_out"])


# ----------------------------------------------------------------- plans and pair tables
def test_write_plan_matches_wrapper_and_tracks_buffer_refills():
    shape = W.SHAPES["llama31_8b"].scaled(num_layers=3, num_blocks=256)
    w = W.make_decode_write(shape, 24, 16, 150, seed=91)
    rng = np.random.default_rng(92)
    cache_words = W.normal_words(rng, shape.cache_shape, "bf16")
    key = to_tensor(W.normal_words(rng, (3, 24, 8, 128), "bf16"), "bf16", DEV)
    value = to_tensor(W.normal_words(rng, (3, 24, 8, 128), "bf16"), "bf16", DEV)
    slots = torch.from_numpy(w.slot_mapping).to(DEV)
    kv = to_tensor(cache_words, "bf16", DEV)
    plan = cache_ops.WritePlan(key, value, kv, slots)
    layer_plans = [cache_ops.WritePlan(key[l], value[l], kv[l], slots) for l in range(3)]
    want = cache_words.copy()
    for step in range(2):  # the second step refills the same buffers in place
        if step:
            key.copy_(to_tensor(W.normal_words(rng, (3, 24, 8, 128), "bf16"), "bf16", DEV))
            slots.copy_(torch.from_numpy(np.roll(w.slot_mapping, 5)).to(DEV))
        cache_oracle.reshape_and_cache_layers(to_words(key), to_words(value), want, slots.cpu().numpy())
        plan.run()
        torch.cuda.synchronize()
        assert np.array_equal(to_words(kv), want)
        kv.copy_(to_tensor(cache_words, "bf16", DEV))
        for p in layer_plans:
            p.run(torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert np.array_equal(to_words(kv), want)
        cache_words = want.copy()


def test_pair_table_on_device_and_on_host_agree():
    """Device tensors are read in place; host tables (dict, list, ndarray) are uploaded by the
    library, including a table larger than its initial buffer and back-to-back calls on two
    streams that share that buffer."""
    L, NB, chunk_words = 2, 12000, 64
    rng = np.random.default_rng(93)
    words = rng.integers(0, 2**16, size=(L, NB, chunk_words), dtype=np.uint16)
    perm = rng.permutation(NB)
    pairs = np.stack([perm[:200].repeat(25), perm[200:5200]], axis=1).astype(np.int64)  # 5000 pairs
    want = words.copy()
    cache_oracle.copy_blocks(want, pairs)
    for table in (pairs, torch.from_numpy(pairs).to(DEV), [tuple(p) for p in pairs.tolist()]):
        kv = to_tensor(words, "fp16", DEV)
        cache_ops.copy_blocks(kv, table)
        torch.cuda.synchronize()
        assert np.array_equal(to_words(kv), want)
    # an unaligned slice of a device table is realigned by the wrapper
    padded = torch.zeros(5001, 2, dtype=torch.int64, device=DEV)
    padded[1:] = torch.from_numpy(pairs).to(DEV)
    view = padded.view(-1)[1:-1].view(5000, 2)  # starts 8 bytes into the allocation
    view.copy_(torch.from_numpy(pairs).to(DEV))
    kv = to_tensor(words, "fp16", DEV)
    cache_ops.copy_blocks(kv, view)
    torch.cuda.synchronize()
    assert np.array_equal(to_words(kv), want)
    # two streams, different host tables, same library buffer
    a, b = to_tensor(words, "fp16", DEV), to_tensor(words, "fp16", DEV)
    torch.cuda.synchronize()
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    p1, p2 = pairs[:2500], pairs[2500:]
    for _ in range(3):
        with torch.cuda.stream(s1):
            cache_ops.copy_blocks(a, p1)
        with torch.cuda.stream(s2):
            cache_ops.copy_blocks(b, p2)
    torch.cuda.synchronize()
    wa, wb = words.copy(), words.copy()
    cache_oracle.copy_blocks(wa, p1)
    cache_oracle.copy_blocks(wb, p2)
    assert np.array_equal(to_words(a), wa) and np.array_equal(to_words(b), wb)


# ----------------------------------------------------------------- flashinfer-style call
def paged_case(seed, num_seqs, chunk, num_blocks=400, H=4, D=64):
    shape = W.KVShape("paged", 1, H, D, "bf16", num_blocks)
    w = W.make_prefill_cow(shape, num_seqs, chunk, 300, 0, 0, seed=seed)
    indptr, indices = W.paged_metadata(w.tables.tables)
    T = len(w.slot_mapping)
    batch = np.repeat(np.arange(num_seqs, dtype=np.int32), chunk)
    pos = np.empty(T, np.int32)
    for i, s in enumerate(w.slot_mapping):
        t = w.tables.tables[batch[i]]
        pos[i] = int(np.nonzero(t == s // 16)[0][0]) * 16 + s % 16
    rng = np.random.default_rng(seed + 1)
    key, value = W.normal_words(rng, (T, H, D), "bf16"), W.normal_words(rng, (T, H, D), "bf16")
    cache = W.normal_words(rng, shape.cache_shape[1:], "bf16")
    return shape, key, value, cache, batch, pos, indices, indptr


@pytest.mark.parametrize("variant", VARIANTS)
def test_append_paged_kv_cache_vs_oracle(variant):
    set_variant(variant)
    shape, key, value, cache, batch, pos, indices, indptr = paged_case(101, 7, 33)
    batch[[4, 90]] = -1                       # padded rows are skipped
    want = cache.copy()
    cache_oracle.append_paged_kv_cache(key, value, batch, pos, want, indices, indptr)
    got = to_tensor(cache, "bf16", DEV)
    dev = lambda a: torch.from_numpy(a).to(DEV)
    cache_ops.append_paged_kv_cache(to_tensor(key, "bf16", DEV), to_tensor(value, "bf16", DEV),
                                    dev(batch), dev(pos), got, dev(indices), dev(indptr),
                                    torch.ones(7, dtype=torch.int32, device=DEV))
    torch.cuda.synchronize()
    assert np.array_equal(to_words(got), want)
    # separate K and V caches, as flashinfer also accepts
    kc = to_tensor(np.ascontiguousarray(cache[:, 0]), "bf16", DEV)
    vc = to_tensor(np.ascontiguousarray(cache[:, 1]), "bf16", DEV)
    cache_ops.append_paged_kv_cache(to_tensor(key, "bf16", DEV), to_tensor(value, "bf16", DEV),
                                    dev(batch), dev(pos), (kc, vc), dev(indices), dev(indptr), None)
    torch.cuda.synchronize()
    assert np.array_equal(to_words(kc), want[:, 0]) and np.array_equal(to_words(vc), want[:, 1])
    with pytest.raises(TypeError, match="int32"):
        cache_ops.append_paged_kv_cache(to_tensor(key, "bf16", DEV), to_tensor(value, "bf16", DEV),
                                        dev(batch).long(), dev(pos), got, dev(indices), dev(indptr))


@pytest.mark.parametrize("variant", [3, 5, 7])
def test_append_paged_decode_step_plan_is_reused_and_guess_may_be_wrong(variant):
    """A decode step (one token per request): token t belongs to request t, the case the
    kernel's early fetch of kv_indptr[t] is made for.  The same call is repeated after the
    index tensors were refilled in place (the cached plan must read the new contents), and
    with the requests in shuffled order, where the guess is wrong for most tokens."""
    set_variant(variant)
    n = 57
    shape, key, value, cache, batch, pos, indices, indptr = paged_case(111, n, 1, num_blocks=900)
    dev = lambda a: torch.from_numpy(a).to(DEV)
    k, v = to_tensor(key, "bf16", DEV), to_tensor(value, "bf16", DEV)
    d_batch, d_pos, d_ind, d_ptr = dev(batch), dev(pos), dev(indices), dev(indptr)
    got = to_tensor(cache, "bf16", DEV)
    want = cache.copy()
    cache_ops._PAGED_PLANS.clear()      # the allocator may hand this test an earlier test's addresses
    before = 0
    cache_ops.append_paged_kv_cache(k, v, d_batch, d_pos, got, d_ind, d_ptr, None)
    cache_oracle.append_paged_kv_cache(key, value, batch, pos, want, indices, indptr)
    torch.cuda.synchronize()
    assert np.array_equal(to_words(got), want)
    assert len(cache_ops._PAGED_PLANS) == before + 1
    # next step: same buffers, new contents - requests in shuffled order, one padded row
    perm = np.random.default_rng(5).permutation(n).astype(np.int32)
    batch2, pos2 = batch[perm].copy(), (pos[perm] + 1).astype(np.int32)
    # a position one further may need a page the request does not own: keep it inside
    room = (indptr[1:] - indptr[:-1])[batch2] * 16
    pos2 = np.minimum(pos2, room - 1).astype(np.int32)
    batch2[7] = -1
    d_batch.copy_(dev(batch2))
    d_pos.copy_(dev(pos2))
    cache_ops.append_paged_kv_cache(k, v, d_batch, d_pos, got, d_ind, d_ptr, None)
    cache_oracle.append_paged_kv_cache(key, value, batch2, pos2, want, indices, indptr)
    torch.cuda.synchronize()
    assert np.array_equal(to_words(got), want)
    assert len(cache_ops._PAGED_PLANS) == before + 1          # the plan was reused
    # an explicit plan, run on a side stream
    plan = cache_ops.PagedWritePlan(k, v, d_batch, d_pos, got, d_ind, d_ptr)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    got.copy_(to_tensor(cache, "bf16", DEV))
    side.wait_stream(torch.cuda.current_stream())
    plan.run(side.cuda_stream)
    side.synchronize()
    want2 = cache.copy()
    cache_oracle.append_paged_kv_cache(key, value, batch2, pos2, want2, indices, indptr)
    assert np.array_equal(to_words(got), want2)


def test_write_then_copy_on_write_chains_land_in_stream_order():
    """Cache write and copy-on-write launched back to back on one stream, each with
    programmatic stream serialization: every copy must see the rows written just before it and
    every write the blocks copied just before it, over many rounds without a synchronize."""
    shape = W.SHAPES["llama31_8b"].scaled(num_layers=2, num_blocks=64, num_kv_heads=2)
    rng = np.random.default_rng(321)
    cache = W.normal_words(rng, shape.cache_shape, shape.dtype)
    got = to_tensor(cache, shape.dtype, DEV)
    want = cache.copy()
    rounds = 12
    keys = W.normal_words(rng, (rounds, 2, 16, 2, 128), shape.dtype)
    vals = W.normal_words(rng, (rounds, 2, 16, 2, 128), shape.dtype)
    d_keys, d_vals = to_tensor(keys, shape.dtype, DEV), to_tensor(vals, shape.dtype, DEV)
    plan = []
    for r in range(rounds):
        blk = int(rng.integers(0, 32))                       # written block
        dst = int(rng.integers(32, 64))                      # its copy
        slots = (blk * 16 + rng.permutation(16)).astype(np.int64)
        plan.append((slots, np.array([[blk, dst]], dtype=np.int64)))
    d_slots = [torch.from_numpy(s).to(DEV) for s, _ in plan]
    d_pairs = [torch.from_numpy(p).to(DEV) for _, p in plan]
    torch.cuda.synchronize()
    for r in range(rounds):
        cache_ops.reshape_and_cache_layers(d_keys[r], d_vals[r], got, d_slots[r])
        cache_ops.copy_blocks(got, d_pairs[r])
    torch.cuda.synchronize()
    for r, (slots, pairs) in enumerate(plan):
        cache_oracle.reshape_and_cache_layers(keys[r], vals[r], want, slots)
        cache_oracle.copy_blocks(want, pairs)
    assert np.array_equal(to_words(got), want)


def test_append_paged_kv_cache_matches_flashinfer():
    """The reference's live cache write is flashinfer's kernel; where flashinfer is importable on
    the GPU box, its result on the same inputs is the golden output."""
    flashinfer = pytest.importorskip("flashinfer")
    shape, key, value, cache, batch, pos, indices, indptr = paged_case(103, 9, 50, H=8, D=128)
    dev = lambda a: torch.from_numpy(a).to(DEV)
    k, v = to_tensor(key, "bf16", DEV), to_tensor(value, "bf16", DEV)
    last = torch.ones(9, dtype=torch.int32, device=DEV)
    theirs = to_tensor(cache, "bf16", DEV)
    try:
        flashinfer.append_paged_kv_cache(k, v, dev(batch), dev(pos), theirs, dev(indices),
                                         dev(indptr), last)
        torch.cuda.synchronize()
    except Exception as e:  # JIT toolchain missing on the box, etc.
        pytest.skip(f"flashinfer could not run here: {e!r}"[:200])
    ours = to_tensor(cache, "bf16", DEV)
    cache_ops.append_paged_kv_cache(k, v, dev(batch), dev(pos), ours, dev(indices), dev(indptr), last)
    torch.cuda.synchronize()
    assert torch.equal(ours.view(torch.int16), theirs.view(torch.int16))
    assert not np.array_equal(to_words(ours), cache)


# ----------------------------------------------------------------- failure handling
def test_bounded_wait_times_out_and_the_context_survives():
    """A device-side wait that nothing satisfies gives up after its limit, reports through the
    error record, and the next kernels run normally."""
    import time
    L = _lib.lib()
    assert L.lms_check_device_errors(None, None, None) == 0
    t0 = time.perf_counter()
    assert L.lms_selftest_bounded_wait(20000, None) == 0        # 20 ms limit
    rc = L.lms_check_device_errors(None, None, None)
    waited = time.perf_counter() - t0
    assert rc == _lib.LMS_ERR_CUDA
    assert b"gave up waiting" in L.lms_last_cuda_error()
    assert 0.015 < waited < 2.0
    assert L.lms_check_device_errors(None, None, None) == 0     # record cleared
    g = load_npz("fill_fp16_t8")
    kc, vc = to_tensor(g["key_cache_in"], "fp16", DEV), to_tensor(g["value_cache_in"], "fp16", DEV)
    cache_ops.fill_key_cache(to_tensor(g["key"], "fp16", DEV), to_tensor(g["value"], "fp16", DEV),
                             kc, vc, torch.from_numpy(g["slot_mapping"]).to(DEV))
    torch.cuda.synchronize()
    assert np.array_equal(to_words(kc), g["key_cache_out"])


def test_peer_enable_errors_are_statuses():
    L = _lib.lib()
    assert L.lms_peer_enable(torch.cuda.current_device()) == 0   # self: nothing to enable
    rc = L.lms_peer_enable(4096)                                 # no such device
    assert rc in (_lib.LMS_ERR_CUDA, _lib.LMS_ERR_PEER)
    x = torch.ones(8, device=DEV)                                # context still fine
    assert float(x.sum()) == 8.0


def test_other_element_sizes_float32_and_int8():
    """The kernels move bytes: a float32 cache (the reference's dtype map also lists it,
    kv_worker.py:17-22) and a 1-byte cache go through the same path."""
    g = torch.Generator(device="cpu").manual_seed(3)
    for dtype, D in ((torch.float32, 32), (torch.int8, 64), (torch.float64, 16)):
        L_, NB, BS, H, T = 2, 12, 4, 2, 17
        make = (lambda *s: torch.randn(*s, generator=g).to(dtype)) if dtype.is_floating_point else \
            (lambda *s: torch.randint(-100, 100, s, generator=g).to(dtype))
        cache, key, value = make(L_, NB, 2, BS, H, D), make(L_, T, H, D), make(L_, T, H, D)
        slots = torch.randperm(NB * BS, generator=g)[:T]
        slots[4] = -1
        want = cache.clone()
        for l in range(L_):
            for t in range(T):
                s = int(slots[t])
                if s >= 0:
                    want[l, s // BS, 0, s % BS] = key[l, t]
                    want[l, s // BS, 1, s % BS] = value[l, t]
        got = cache.to(DEV)
        cache_ops.reshape_and_cache_layers(key.to(DEV), value.to(DEV), got, slots.to(DEV))
        cache_ops.copy_blocks(got, {3: [10, 11]})
        want[:, 10] = want[:, 3]
        want[:, 11] = want[:, 3]
        torch.cuda.synchronize()
        assert torch.equal(got.cpu().view(torch.uint8), want.view(torch.uint8)), dtype


@pytest.mark.parametrize("pdl", [1, 2])
def test_back_to_back_writes_to_the_same_slots_land_in_stream_order(pdl):
    """With programmatic dependent launch (1) the next kernel's grid is resident before the
    previous one has finished; it must still not overtake it.  Eight writes of different data
    to the same slots, repeated: the last one wins, every time."""
    _lib.lib().lms_set_tuning(_lib.TUNE_WRITE_PDL, pdl)
    shape = W.SHAPES["llama31_8b"].scaled(num_layers=8, num_blocks=4096)
    w = W.make_decode_write(shape, 128, 16, 400, seed=95)
    slots = torch.from_numpy(w.slot_mapping).to(DEV)
    kv = torch.zeros(shape.cache_shape, dtype=torch.bfloat16, device=DEV)
    keys = [torch.randn(8, 128, 8, 128, device=DEV).to(torch.bfloat16) for _ in range(8)]
    vals = [torch.randn(8, 128, 8, 128, device=DEV).to(torch.bfloat16) for _ in range(8)]
    plans = [cache_ops.WritePlan(keys[j], vals[j], kv, slots) for j in range(8)]
    sp = torch.cuda.current_stream().cuda_stream
    blk, ent = slots // 16, slots % 16
    for trial in range(10):
        order = np.random.default_rng(trial).permutation(8)
        for j in order:
            plans[j].run(sp)
        last = int(order[-1])
        torch.cuda.synchronize()
        assert torch.equal(kv[:, blk, 0, ent].view(torch.int16), keys[last].view(torch.int16)), trial
        assert torch.equal(kv[:, blk, 1, ent].view(torch.int16), vals[last].view(torch.int16)), trial


def test_attention_backend_reads_the_cache_we_wrote():
    """The consumer of the cache in LMServe is flashinfer's paged attention
    (models/layers/attention.py:87-106).  Fill a paged cache through this library, run
    flashinfer's batch decode over it, and compare with attention computed from the dense K/V:
    the layout and the addressing are what the reference's attention backend expects."""
    flashinfer = pytest.importorskip("flashinfer")
    torch.manual_seed(0)
    NH, NKV, HD, BS, NB, B = 32, 8, 128, 16, 256, 5
    ctx = np.array([17, 33, 1, 64, 100])          # cached tokens per sequence (the last one is new)
    bt = W.deal_block_tables(np.random.default_rng(0), NB, (ctx + BS) // BS)
    indptr, indices = W.paged_metadata(bt.tables)
    dev = lambda a: torch.from_numpy(a).to(DEV)
    kv = torch.zeros(NB, 2, BS, NKV, HD, dtype=torch.bfloat16, device=DEV)
    dense_k = [torch.randn(c + 1, NKV, HD, device=DEV).to(torch.bfloat16) for c in ctx]
    dense_v = [torch.randn(c + 1, NKV, HD, device=DEV).to(torch.bfloat16) for c in ctx]
    batch = dev(np.repeat(np.arange(B), ctx + 1).astype(np.int32))
    pos = dev(np.concatenate([np.arange(c + 1) for c in ctx]).astype(np.int32))
    last = dev((ctx % BS + 1).astype(np.int32))
    cache_ops.append_paged_kv_cache(torch.cat(dense_k), torch.cat(dense_v), batch, pos, kv,
                                    dev(indices), dev(indptr), last)
    q = torch.randn(B, NH, HD, device=DEV).to(torch.bfloat16)
    try:
        ws = torch.empty(128 << 20, dtype=torch.uint8, device=DEV)
        wrapper = flashinfer.BatchDecodeWithPagedKVCacheWrapper(ws, "NHD")
        wrapper.plan(dev(indptr), dev(indices), last, NH, NKV, HD, BS,
                     q_data_type=torch.bfloat16, kv_data_type=torch.bfloat16)
        out = wrapper.run(q, kv)
        torch.cuda.synchronize()
    except Exception as e:  # JIT toolchain missing on the box, API drift, ...
        pytest.skip(f"flashinfer attention could not run here: {e!r}"[:200])
    ref = []
    for b in range(B):
        k = dense_k[b].float().repeat_interleave(NH // NKV, dim=1)
        v = dense_v[b].float().repeat_interleave(NH // NKV, dim=1)
        p = torch.softmax(torch.einsum("hd,shd->hs", q[b].float(), k) / HD ** 0.5, dim=-1)
        ref.append(torch.einsum("hs,shd->hd", p, v))
    # attention itself is flashinfer's arithmetic in bf16: 2e-2 absolute on O(1) values
    assert torch.allclose(out.float(), torch.stack(ref), atol=2e-2, rtol=2e-2)
