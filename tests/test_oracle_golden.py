"""CPU: the oracle (NumPy restatement and the torch index-op form) against the golden
vectors produced by LMServe's own Triton kernels, and against each other."""
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
from hypothesis import given, settings, strategies as st

from helpers import (COPY_CASES, FILL_CASES, GOLDEN, load_json, load_npz, sha, to_tensor,
                     to_words)
import workloads as W
from oracle import cache_oracle, torch_ref, triton_ref


@pytest.mark.parametrize("name", FILL_CASES)
def test_fill_numpy_vs_golden(name):
    g = load_npz(name)
    kc, vc = g["key_cache_in"].copy(), g["value_cache_in"].copy()
    cache_oracle.fill_key_cache(g["key"], g["value"], kc, vc, g["slot_mapping"])
    assert np.array_equal(kc, g["key_cache_out"])
    assert np.array_equal(vc, g["value_cache_out"])


@pytest.mark.parametrize("name", FILL_CASES)
def test_fill_torch_vs_golden(name):
    g = load_npz(name)
    dt = g["dtype"]
    kc, vc = to_tensor(g["key_cache_in"], dt), to_tensor(g["value_cache_in"], dt)
    torch_ref.fill_key_cache(to_tensor(g["key"], dt), to_tensor(g["value"], dt), kc, vc,
                             torch.from_numpy(g["slot_mapping"]))
    assert np.array_equal(to_words(kc), g["key_cache_out"])
    assert np.array_equal(to_words(vc), g["value_cache_out"])


@pytest.mark.parametrize("name", COPY_CASES)
def test_copy_numpy_and_torch_vs_golden(name):
    g = load_npz(name)
    kv = g["kv_in"].copy()
    cache_oracle.copy_blocks(kv, g["pairs"])
    assert np.array_equal(kv, g["kv_out"])
    t = to_tensor(g["kv_in"], g["dtype"])
    torch_ref.copy_blocks(t, g["pairs"])
    assert np.array_equal(to_words(t), g["kv_out"])
    # the dict form of the reference launcher gives the same table
    d = {}
    for s, dst in g["pairs"]:
        d.setdefault(int(s), []).append(int(dst))
    kv2 = g["kv_in"].copy()
    cache_oracle.copy_blocks(kv2, d)
    assert np.array_equal(kv2, g["kv_out"])


def test_plumbing_case_digests():
    """Full-size Llama-3.2-1B plumbing case: seeded inputs reproduce, and the oracle's
    outputs hash to what the reference kernels produced."""
    g = load_json("plumbing_llama32_1b")
    case = W.config1(seed=g["generator"]["workload_seed"])
    pay = W.plumbing_payload(case, seed=g["generator"]["payload_seed"])
    assert sha(case.slot_mapping) == g["inputs"]["slot_mapping"]
    assert sha(case.pairs) == g["inputs"]["pairs"]
    for k in ("key", "value", "key_cache", "value_cache", "kv_caches"):
        assert sha(pay[k]) == g["inputs"][k], k
    assert int((case.slot_mapping >= 0).sum()) == g["live_tokens"] == 240
    # padded (-1) entries are skipped by the oracle; the reference only saw the live tokens
    kc, vc = pay["key_cache"].copy(), pay["value_cache"].copy()
    cache_oracle.fill_key_cache(pay["key"], pay["value"], kc, vc, case.slot_mapping)
    assert sha(kc) == g["outputs"]["key_cache"]
    assert sha(vc) == g["outputs"]["value_cache"]
    kv = pay["kv_caches"].copy()
    cache_oracle.copy_blocks(kv, case.pairs)
    assert sha(kv) == g["outputs"]["kv_caches"]
    # torch index-op form, same digests
    dt = case.shape.dtype
    tkc, tvc = to_tensor(pay["key_cache"], dt), to_tensor(pay["value_cache"], dt)
    torch_ref.fill_key_cache(to_tensor(pay["key"], dt), to_tensor(pay["value"], dt), tkc, tvc,
                             torch.from_numpy(case.slot_mapping))
    assert sha(to_words(tkc)) == g["outputs"]["key_cache"]
    assert sha(to_words(tvc)) == g["outputs"]["value_cache"]
    tkv = to_tensor(pay["kv_caches"], dt)
    torch_ref.copy_blocks(tkv, case.pairs)
    assert sha(to_words(tkv)) == g["outputs"]["kv_caches"]


def test_interleaved_equals_contiguous_planes():
    """The interleaved write is the flat write applied to the K plane and the V plane."""
    rng = np.random.default_rng(5)
    NB, BS, H, D, T = 6, 4, 2, 8, 9
    kv = W.normal_words(rng, (NB, 2, BS, H, D), "bf16")
    key, value = W.normal_words(rng, (T, H, D), "bf16"), W.normal_words(rng, (T, H, D), "bf16")
    slots = rng.permutation(NB * BS)[:T].astype(np.int64)
    slots[3] = -1
    a = kv.copy()
    cache_oracle.reshape_and_cache(key, value, a, slots)
    kplane, vplane = kv[:, 0].copy(), kv[:, 1].copy()
    cache_oracle.fill_key_cache(key, value, kplane, vplane, slots)
    assert np.array_equal(a[:, 0], kplane) and np.array_equal(a[:, 1], vplane)
    t = to_tensor(kv, "bf16")
    torch_ref.reshape_and_cache(to_tensor(key, "bf16"), to_tensor(value, "bf16"), t,
                                torch.from_numpy(slots))
    assert np.array_equal(to_words(t), a)


@settings(max_examples=40, deadline=None)
@given(L=st.integers(1, 3), NB=st.integers(2, 12), NHB=st.integers(1, 10),
       chunk=st.sampled_from([8, 24, 64]), seed=st.integers(0, 2**31 - 1))
def test_swap_and_transfer_numpy_vs_torch(L, NB, NHB, chunk, seed):
    rng = np.random.default_rng(seed)
    gpu = rng.integers(0, 2**16, size=(L, NB, chunk), dtype=np.uint16)
    host = rng.integers(0, 2**16, size=(NHB, L, chunk), dtype=np.uint16)
    n = int(rng.integers(0, min(NB, NHB) + 1))
    out_pairs = np.stack([rng.permutation(NB)[:n], rng.permutation(NHB)[:n]], axis=1).astype(np.int64)
    g1, h1 = gpu.copy(), host.copy()
    cache_oracle.swap_out(g1, h1, out_pairs)
    tg, th = torch.from_numpy(gpu.view(np.int16).copy()), torch.from_numpy(host.view(np.int16).copy())
    torch_ref.swap_out(tg, th, out_pairs)
    assert np.array_equal(th.numpy().view(np.uint16), h1)
    in_pairs = np.stack([rng.permutation(NHB)[:n], rng.permutation(NB)[:n]], axis=1).astype(np.int64)
    cache_oracle.swap_in(g1, h1, in_pairs, layers=(0, L))
    torch_ref.swap_in(tg, th, in_pairs)
    assert np.array_equal(tg.numpy().view(np.uint16), g1)
    dst = rng.integers(0, 2**16, size=(L, NHB + 1, chunk), dtype=np.uint16)
    d1 = dst.copy()
    cache_oracle.transfer(gpu, d1, out_pairs)
    td = torch.from_numpy(dst.view(np.int16).copy())
    torch_ref.transfer(torch.from_numpy(gpu.view(np.int16).copy()), td, out_pairs)
    assert np.array_equal(td.numpy().view(np.uint16), d1)


def test_swap_layer_range_only_touches_range():
    rng = np.random.default_rng(9)
    gpu = rng.integers(0, 2**16, size=(4, 5, 16), dtype=np.uint16)
    host = np.zeros((3, 4, 16), dtype=np.uint16)
    pairs = np.array([[4, 0], [1, 2]], dtype=np.int64)
    cache_oracle.swap_out(gpu, host, pairs, layers=(1, 3))
    assert not host[:, 0].any() and not host[:, 3].any() and not host[1].any()
    assert np.array_equal(host[0, 1], gpu[1, 4]) and np.array_equal(host[2, 2], gpu[2, 1])


@pytest.mark.skipif(not triton_ref.available(), reason="LMServe source tree not present")
def test_golden_regenerates_from_reference(tmp_path):
    """Where the reference tree is mounted, re-running its kernels reproduces the committed
    digests (run in a child process: the interpreter flag must precede the triton import)."""
    code = (
        "import os, sys, json; os.environ['TRITON_INTERPRET']='1'; sys.path.insert(0, %r);"
        "import numpy as np, torch;"
        "import workloads as W; from oracle import triton_ref;"
        "import hashlib;"
        "c=W.config1(); p=W.plumbing_payload(c);"
        "t=torch.from_numpy(p['kv_caches'].view(np.int16).copy()).view(torch.float16);"
        "triton_ref.copy_blocks(t, torch.from_numpy(c.pairs));"
        "print(hashlib.sha256(t.view(torch.int16).numpy().tobytes()).hexdigest())"
    ) % str(Path(__file__).resolve().parent.parent)
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    assert out.stdout.strip().splitlines()[-1] == load_json("plumbing_llama32_1b")["outputs"]["kv_caches"]


def test_paged_append_equals_slot_write():
    """flashinfer's (batch index, position, page table) addressing and the slot mapping
    ``table[pos // BS] * BS + pos % BS`` describe the same write."""
    shape = W.SHAPES["llama31_8b"].scaled(num_layers=1, num_blocks=96, num_kv_heads=2, head_dim=16)
    w = W.make_prefill_cow(shape, 5, 40, 200, 0, 0, seed=77)
    rng = np.random.default_rng(78)
    T = len(w.slot_mapping)
    key, value = W.normal_words(rng, (T, 2, 16), "bf16"), W.normal_words(rng, (T, 2, 16), "bf16")
    cache = W.normal_words(rng, shape.cache_shape[1:], "bf16")
    indptr, indices = W.paged_metadata(w.tables.tables)
    batch = np.repeat(np.arange(5, dtype=np.int32), 40)
    # recover each token's position from its slot and table
    pos = np.empty(T, np.int32)
    for i, s in enumerate(w.slot_mapping):
        t = w.tables.tables[batch[i]]
        pos[i] = int(np.nonzero(t == s // 16)[0][0]) * 16 + s % 16
    a, b = cache.copy(), cache.copy()
    cache_oracle.append_paged_kv_cache(key, value, batch, pos, a, indices, indptr)
    cache_oracle.reshape_and_cache(key, value, b, w.slot_mapping)
    assert np.array_equal(a, b) and not np.array_equal(a, cache)
    batch[3] = -1
    c = cache.copy()
    cache_oracle.append_paged_kv_cache(key, value, batch, pos, c, indices, indptr)
    slots = w.slot_mapping.copy()
    slots[3] = -1
    d = cache.copy()
    cache_oracle.reshape_and_cache(key, value, d, slots)
    assert np.array_equal(c, d)
