"""GPU: the copy-on-write entry point that allocates nothing.

Collected last on purpose (the file name sorts after every other test file): if it fails, a
run that stops at the first failure has already run everything else.

An LMServe worker gives all remaining device memory to the KV cache at start-up, so a later
cudaMalloc may fail and always stalls the device; ``lms_copy_blocks_host_static`` therefore
keeps its uploaded (src, dst) table in a fixed array inside the library.  Its result must be
identical to ``lms_copy_blocks_host`` (bit-exact, the tolerance of every test here), including
on a second call that reuses the array while it still holds the first call's longer table.
"""
import ctypes

import numpy as np
import pytest
import torch

from lmserve_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _run(entry, kv, pairs, with_num_blocks):
    L_, NB, chunk_elems = kv.shape
    es = kv.element_size()
    args = [kv.data_ptr(), NB * chunk_elems * es, chunk_elems * es, chunk_elems * es, L_,
            pairs.ctypes.data, pairs.shape[0]]
    if with_num_blocks:
        args.append(NB)
    args.append(torch.cuda.current_stream().cuda_stream)
    return entry(*args)


def test_static_table_entry_point_matches_allocating_one_twice_in_a_row():
    lib = _lib.lib()
    torch.cuda.set_device(0)
    rng = np.random.default_rng(2024)
    L_, NB, chunk_elems = 3, 6000, 1024 + 8          # 2064-byte chunks, three layers
    base = torch.from_numpy(rng.integers(-2**15, 2**15, size=(L_, NB, chunk_elems),
                                         dtype=np.int16)).to(DEV)
    perm = rng.permutation(NB)
    # first call: 4000 pairs with fan-out; second call: 37 different pairs (shorter table)
    first = np.stack([perm[:400].repeat(10), perm[400:4400]], axis=1).astype(np.int64)
    second = np.stack([perm[4400:4437], perm[5000:5037]], axis=1).astype(np.int64)
    want, got = base.clone(), base.clone()
    for pairs in (first, second):
        pairs = np.ascontiguousarray(pairs)
        assert _run(lib.lms_copy_blocks_host, want, pairs, True) == _lib.LMS_OK
        assert _run(lib.lms_copy_blocks_host_static, got, pairs, False) == _lib.LMS_OK
        torch.cuda.synchronize()
        assert torch.equal(got, want)
    assert not torch.equal(got, base)                # the copies really happened
    # plain restatement of both calls on the device, as a second opinion
    ref = base.clone()
    for pairs in (first, second):
        src = torch.from_numpy(pairs[:, 0].copy()).to(DEV)
        dst = torch.from_numpy(pairs[:, 1].copy()).to(DEV)
        ref.index_copy_(1, dst, ref.index_select(1, src))
    assert torch.equal(got, ref)


def test_static_table_entry_point_limits_and_argument_errors():
    lib = _lib.lib()
    f = lib.lms_copy_blocks_host_static
    kv = torch.zeros(1, 8, 64, dtype=torch.int16, device=DEV)
    too_many = np.zeros((_lib.LMS_STATIC_MAX_PAIRS + 1, 2), dtype=np.int64)
    rc = _run(f, kv, too_many, False)
    assert rc == _lib.LMS_ERR_TOO_LARGE
    assert b"fixed-size table" in lib.lms_strerror(rc)
    with pytest.raises(_lib.LmsError, match="fixed-size table"):
        _lib.check(rc)
    empty = np.zeros((0, 2), dtype=np.int64)
    assert _run(f, kv, empty, False) == _lib.LMS_OK
    one = np.array([[1, 2]], dtype=np.int64)
    s = torch.cuda.current_stream().cuda_stream
    assert f(None, 1024, 128, 128, 1, one.ctypes.data, 1, s) == _lib.LMS_ERR_NULL
    assert f(kv.data_ptr(), 1024, 128, 120, 1, one.ctypes.data, 1, s) == _lib.LMS_ERR_ALIGN
    assert f(kv.data_ptr(), 1024, 128, 128, 1, one.ctypes.data, -1, s) == _lib.LMS_ERR_RANGE
    # exactly the maximum is accepted
    kv2 = torch.arange(2 * 40000 * 8, dtype=torch.int16, device=DEV).view(2, 40000, 8)
    n = _lib.LMS_STATIC_MAX_PAIRS
    pairs = np.stack([np.arange(n), 20000 + np.arange(n)], axis=1).astype(np.int64)
    assert _run(f, kv2, pairs, False) == _lib.LMS_OK
    torch.cuda.synchronize()
    assert torch.equal(kv2[:, 20000:20000 + n], kv2[:, :n])


_FRESH_PROCESS = r"""
import sys, json
sys.path.insert(0, {root!r})
import numpy as np, torch
from lmserve_b200 import _lib
torch.cuda.set_device(0)
lib = _lib.lib()
kv = torch.arange(2 * 40000 * 8, dtype=torch.int16, device="cuda:0").view(2, 40000, 8)
stream = torch.cuda.current_stream().cuda_stream
torch.cuda.synchronize()

def call(n):
    pairs = np.stack([np.arange(n), 20000 + np.arange(n)], axis=1).astype(np.int64)
    before = lib.lms_launch_count()
    rc = lib.lms_copy_blocks_host_static(kv.data_ptr(), 40000 * 16, 16, 16, 2, pairs.ctypes.data, n, stream)
    torch.cuda.synchronize()
    return rc, lib.lms_launch_count() - before, torch.cuda.mem_get_info(0)[0]

free0 = torch.cuda.mem_get_info(0)[0]
out = dict(free0=free0, calls=[call(64), call(5), call(16384), call(64)])
out["ok"] = bool(torch.equal(kv[:, 20000:20000 + 16384], kv[:, :16384]))
print(json.dumps(out))
"""


def test_static_table_entry_point_allocates_nothing_in_a_fresh_process():
    """The property the entry point exists for, checked where nothing else has run: a child
    process makes its very first call into the library through ``lms_copy_blocks_host_static``
    (no ``lms_init_device``, no other ``*_host`` call before it, so no error record and no
    upload table exist), then calls it again with a short, the longest possible and a short
    table.  Free device memory (``cudaMemGetInfo``) must not move from the first call's level —
    the largest table included, where a growing buffer would have to be allocated — and every
    call must launch exactly one kernel.  The first call itself may lower the level once: the
    driver loads the library's code image, which contains the 256 KiB table, on first use."""
    import json
    import subprocess
    import sys
    from pathlib import Path
    root = str(Path(__file__).resolve().parent.parent)
    out = subprocess.run([sys.executable, "-c", _FRESH_PROCESS.format(root=root)], capture_output=True,
                         text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    d = json.loads(out.stdout.strip().splitlines()[-1])
    assert d["ok"]
    (rc1, n1, f1), rest = d["calls"][0], d["calls"][1:]
    assert rc1 == _lib.LMS_OK and n1 == 1
    assert 0 <= d["free0"] - f1 <= 64 << 20, "the first call took more than a code image from the device"
    for rc, launches, free in rest:
        assert rc == _lib.LMS_OK and launches == 1
        assert free == f1, "a later call changed the amount of free device memory"
