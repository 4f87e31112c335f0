"""Per-step index preparation: the oracle against flashinfer's documented example and a case
worked by hand (CPU), the packed upload format (CPU), and the kernel against the oracle and
against flashinfer's own helpers (GPU, exact)."""
import copy

import numpy as np
import pytest
import torch

from lmserve_b200 import _lib
import workloads as W
from lmserve_b200.step_inputs import InferInput, pack_requests
from oracle import step_oracle

DEV = "cuda:0"
FIELDS = ["position_ids", "cu_seqlens_q", "kv_block_indices", "kv_block_indptrs",
          "kv_last_block_lens", "batch_indices", "positions", "slot_mapping"]


# ------------------------------------------------------------------ CPU: oracle and packing
def test_oracle_matches_the_documented_flashinfer_example():
    # flashinfer.get_batch_indices_positions, documentation example
    indptr = np.array([0, 1, 3, 6, 10], dtype=np.int32)
    b, p = step_oracle.get_batch_indices_positions(indptr, np.array([5, 5, 5, 5]), 10)
    assert b.tolist() == [0, 1, 1, 2, 2, 2, 3, 3, 3, 3]
    assert p.tolist() == [4, 3, 4, 2, 3, 4, 1, 2, 3, 4]
    # get_seq_lens: (pages - 1) * page_size + last_page_len, clamped for an empty table
    assert step_oracle.get_seq_lens(np.array([0, 3, 3, 4]), np.array([5, 16, 1]), 16).tolist() == [37, 16, 1]


def test_oracle_matches_vectors_made_by_flashinfer_on_a_gpu():
    """tests/golden/step_indices_flashinfer.npz: flashinfer.get_seq_lens and
    get_batch_indices_positions run on a B200 on a seeded request list
    (tests/golden/make_step_golden.py); the oracle reproduces them from the same list."""
    import importlib.util
    from helpers import GOLDEN
    spec = importlib.util.spec_from_file_location("make_step_golden", GOLDEN / "make_step_golden.py")
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    z = np.load(GOLDEN / "step_indices_flashinfer.npz")
    reqs = W.make_step_requests(**gen.GENERATOR)
    o = step_oracle.make_inputs(reqs, gen.GENERATOR["block_size"])
    assert np.array_equal(o["batch_indices"], z["batch_indices"])
    assert np.array_equal(o["positions"], z["positions"])
    assert np.array_equal(step_oracle.get_seq_lens(o["kv_block_indptrs"], o["kv_last_block_lens"], 16),
                          z["seq_lens"])
    assert (o["positions"] != o["position_ids"]).any()     # spare blocks: the two differ, as in flashinfer


def hand_case():
    return [
        InferInput(input_ids=[7], input_len=1, filled_token_len=16, context_len=17, block_ids=[5, 9]),
        InferInput(input_ids=[1, 2, 3, 4], input_len=4, filled_token_len=14, context_len=18, block_ids=[3, 8]),
        InferInput(input_ids=[11], input_len=1, filled_token_len=2, context_len=3, block_ids=[6]),
    ]


def test_oracle_on_a_case_worked_by_hand():
    inputs = hand_case()
    o = step_oracle.make_inputs(inputs, 16)
    # sorted by descending input_len, stable: the 4-token prefill first, then the two decodes
    assert [d.input_len for d in inputs] == [4, 1, 1]
    assert o["input_ids"].tolist() == [1, 2, 3, 4, 7, 11]
    assert o["position_ids"].tolist() == [14, 15, 16, 17, 16, 2]
    assert o["cu_seqlens_q"].tolist() == [0, 4, 5, 6]
    assert o["prefill_input_len"] == 4
    assert o["kv_block_indptrs"].tolist() == [0, 2, 4, 5]
    assert o["kv_block_indices"].tolist() == [3, 8, 5, 9, 6]
    assert o["kv_last_block_lens"].tolist() == [2, 1, 3]
    assert o["batch_indices"].tolist() == [0, 0, 0, 0, 1, 2]
    assert o["positions"].tolist() == [14, 15, 16, 17, 16, 2]
    assert o["slot_mapping"].tolist() == [3 * 16 + 14, 3 * 16 + 15, 8 * 16, 8 * 16 + 1, 9 * 16, 6 * 16 + 2]


def test_pack_requests_layout_sort_and_validation():
    inputs = hand_case()
    packed, batch, T, NB, prefill_len, n_pre, n_dec, pb, db = pack_requests(inputs)
    assert (batch, T, NB, prefill_len, n_pre, n_dec, pb, db) == (3, 6, 5, 4, 1, 2, 2, 3)
    assert packed.dtype == np.int32
    assert packed.tolist() == [4, 1, 1, 14, 16, 2, 18, 17, 3, 2, 2, 1,
                               3, 8, 5, 9, 6, 1, 2, 3, 4, 7, 11]
    out = np.zeros(64, dtype=np.int32)
    again = pack_requests(hand_case(), out)[0]
    assert again.base is out and again.tolist() == packed.tolist()
    with pytest.raises(ValueError, match="staging"):
        pack_requests(hand_case(), np.zeros(8, dtype=np.int32))
    arrays = hand_case()
    for d, dt in zip(arrays, (np.int64, np.uint32, np.int32)):
        d.block_ids = np.asarray(d.block_ids, dtype=dt)   # tables kept as arrays by the caller
    assert pack_requests(arrays)[0].tolist() == packed.tolist()
    bad = hand_case()
    bad[0].input_ids = [1, 2]
    with pytest.raises(ValueError, match="input ids"):
        pack_requests(bad)
    bad = hand_case()
    bad[1].filled_token_len = 10
    with pytest.raises(ValueError, match="context_len - filled_token_len"):
        pack_requests(bad)


def test_c_packer_and_python_packer_agree(monkeypatch):
    import lmserve_b200.step_inputs as S
    assert S._packer is not None, "lmserve_b200/_packer.so is not built (python -m lmserve_b200.build)"
    reqs = W.make_step_requests(65536, 16, 70, 1, 900, 6, 129, 400, seed=44, spare_blocks=1)
    reqs += [InferInput([], 0, 9, 9, [1, 2])]
    fast = S.pack_requests(copy.deepcopy(reqs))
    out = np.zeros(fast[0].size + 5, dtype=np.int32)
    fast_into = S.pack_requests(copy.deepcopy(reqs), out)
    monkeypatch.setattr(S, "_packer", None)
    slow = S.pack_requests(copy.deepcopy(reqs))
    for a in (fast, fast_into):
        assert a[1:] == slow[1:]
        assert np.array_equal(a[0], slow[0])
    assert fast_into[0].base is out
    # the C packer raises the same errors
    monkeypatch.undo()
    bad = hand_case()
    bad[2].input_ids = []
    with pytest.raises(ValueError, match="input ids"):
        S.pack_requests(bad)
    bad = hand_case()
    bad[0].context_len = 99
    with pytest.raises(ValueError, match="context_len - filled_token_len"):
        S.pack_requests(bad)
    bad = hand_case()
    bad[0].block_ids = [1 << 40]
    with pytest.raises(OverflowError):
        S.pack_requests(bad)
    # both conversions of the C packer: one-digit ints are read in place, everything else
    # (two-digit ints, negative values, NumPy integers) takes the general route
    for value in (0, 1, (1 << 30) - 1, 1 << 30, (1 << 31) - 1, -1, -(1 << 31)):
        edge = hand_case()
        edge[1].block_ids = [value, np.int64(value)]      # the prefill request: first after the sort
        packed, batch = S.pack_requests(edge)[:2]
        assert packed[4 * batch:4 * batch + 2].tolist() == [value, value]
    for value in (1 << 31, -(1 << 31) - 1):
        edge = hand_case()
        edge[0].block_ids = [value]
        with pytest.raises(OverflowError):
            S.pack_requests(edge)
    with pytest.raises(ValueError, match="staging"):
        S.pack_requests(hand_case(), np.zeros(13, dtype=np.int32))
    with pytest.raises(AttributeError):
        S.pack_requests([object()])


def test_step_request_generator_is_consistent():
    reqs = W.make_step_requests(4096, 16, 12, 20, 300, 3, 64, 100, seed=5, spare_blocks=1)
    assert len(reqs) == 15
    seen = set()
    for r in reqs:
        assert r.context_len - r.filled_token_len == r.input_len == len(r.input_ids)
        assert len(r.block_ids) == -(-r.context_len // 16) + 1
        assert not seen & set(r.block_ids)
        seen |= set(r.block_ids)
    o = step_oracle.make_inputs(copy.deepcopy(reqs), 16)
    # spare blocks make flashinfer's seq_len (counted from the table) exceed context_len: the
    # reference's positions then differ from its position_ids, and so do the oracle's
    assert (o["positions"] != o["position_ids"]).any()


def test_argument_errors_need_no_gpu():
    lib = _lib.lib()
    z = [None] * 6
    outs = [None] * 9 + [0, 0, None]
    assert lib.lms_build_step_indices(*z, -1, 0, 0, 16, *outs, None) == _lib.LMS_ERR_RANGE
    assert lib.lms_build_step_indices(*z, 0, 0, 0, 0, *outs, None) == _lib.LMS_ERR_RANGE
    assert lib.lms_build_step_indices(*z, 4097, 1, 1, 16, *outs, None) == _lib.LMS_ERR_TOO_LARGE
    assert lib.lms_build_step_indices(*z, 0, 0, 0, 16, *outs, None) == _lib.LMS_OK
    assert lib.lms_build_step_indices(*z, 2, 2, 2, 16, *outs, None) == _lib.LMS_ERR_NULL
    assert lib.lms_build_step_indices(16, 16, 16, 16, 18, 16, 2, 2, 2, 16, *outs, None) == _lib.LMS_ERR_ALIGN
    assert lib.lms_build_step_indices(*z, 2, 2, 2, 16, *([None] * 9), 2, 1, None, None) == _lib.LMS_ERR_RANGE


# ------------------------------------------------------------------ GPU: kernel vs oracle
def run_builder(reqs, block_size=16, **kw):
    from lmserve_b200.step_inputs import make_inputs
    ids, s = make_inputs(reqs, block_size, DEV, **kw)
    torch.cuda.synchronize()
    got = {f: getattr(s, f).cpu().numpy() for f in FIELDS}
    got["input_ids"] = ids.cpu().numpy()
    got["prefill_input_len"] = s.prefill_input_len
    return got, s


def phase_arrays(reqs, page_size):
    """The page table of the prefill and of the decode requests alone, built the way
    build_prefill_wrapper / build_decode_wrapper do (model_worker.py:30-63, 94-124)."""
    reqs = sorted(reqs, key=lambda x: -x.input_len)
    out = {}
    for name, sel in (("prefill", [d for d in reqs if d.input_len > 1]),
                      ("decode", [d for d in reqs if d.input_len == 1])):
        if not sel:
            out[name] = None
            continue
        out[name] = dict(
            qo_indptr=np.cumsum([0] + [d.input_len for d in sel]).astype(np.int32),
            kv_indptr=np.cumsum([0] + [len(d.block_ids) for d in sel]).astype(np.int32),
            kv_indices=np.asarray([b for d in sel for b in d.block_ids], dtype=np.int32),
            kv_last_page_len=np.asarray([(d.context_len - 1) % page_size + 1 for d in sel], dtype=np.int32))
    return out


def assert_phases(s, reqs, page_size=16):
    want = phase_arrays(reqs, page_size)
    for name in ("prefill", "decode"):
        got = getattr(s, name)
        if want[name] is None:
            assert got is None
            continue
        for f in ("kv_indptr", "kv_indices", "kv_last_page_len"):
            assert np.array_equal(getattr(got, f).cpu().numpy(), want[name][f]), (name, f)
        if name == "prefill":
            assert np.array_equal(got.qo_indptr.cpu().numpy(), want[name]["qo_indptr"])
        else:
            assert got.qo_indptr is None


def assert_same(got, want):
    for f in FIELDS + ["input_ids"]:
        assert got[f].dtype == want[f].dtype, f
        assert np.array_equal(got[f], want[f]), f
    assert got["prefill_input_len"] == want["prefill_input_len"]


STEP_CASES = {
    "decode256": dict(num_decode=256, ctx_lo=128, ctx_hi=4096, num_prefill=0, chunk_tokens=0, max_offset=0),
    "mixed": dict(num_decode=100, ctx_lo=1, ctx_hi=700, num_prefill=9, chunk_tokens=512, max_offset=3000),
    "prefill64": dict(num_decode=0, ctx_lo=0, ctx_hi=0, num_prefill=64, chunk_tokens=512, max_offset=8192),
    "many_requests": dict(num_decode=3000, ctx_lo=1, ctx_hi=90, num_prefill=57, chunk_tokens=33, max_offset=50),
    "max_batch": dict(num_decode=4090, ctx_lo=1, ctx_hi=40, num_prefill=6, chunk_tokens=17, max_offset=30),
    "spare_blocks": dict(num_decode=40, ctx_lo=5, ctx_hi=400, num_prefill=4, chunk_tokens=100, max_offset=64,
                         spare_blocks=2),
}


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(STEP_CASES))
def test_kernel_matches_oracle(name):
    reqs = W.make_step_requests(65536, 16, seed=31 + len(name), **STEP_CASES[name])
    want = step_oracle.make_inputs(copy.deepcopy(reqs), 16)
    got, s = run_builder(copy.deepcopy(reqs))
    assert_same(got, want)
    assert_phases(s, reqs)


@pytest.mark.gpu
def test_hand_case_requests_without_tokens_and_other_block_sizes():
    got, _ = run_builder(hand_case())
    assert_same(got, step_oracle.make_inputs(hand_case(), 16))
    # requests with no new token keep their table entries and are stepped over by the tokens
    reqs = hand_case() + [InferInput([], 0, 40, 40, [21, 22, 23]), InferInput([], 0, 5, 5, [30])]
    reqs = [reqs[3], reqs[0], reqs[4], reqs[1], reqs[2]]
    got, s = run_builder(copy.deepcopy(reqs))
    assert_same(got, step_oracle.make_inputs(copy.deepcopy(reqs), 16))
    assert_phases(s, reqs)       # requests without new tokens belong to neither phase
    for bs in (1, 8, 24, 32):
        reqs = W.make_step_requests(4096, bs, 17, 1, 200, 3, 50, 70, seed=bs)
        got, _ = run_builder(copy.deepcopy(reqs), block_size=bs)
        assert_same(got, step_oracle.make_inputs(copy.deepcopy(reqs), bs))


@pytest.mark.gpu
def test_empty_step_and_reused_builder():
    from lmserve_b200.step_inputs import StepInputBuilder
    b = StepInputBuilder(DEV, 16, max_batch=300, max_tokens=6000, max_blocks=70000)
    ids, s = b.make_inputs([])
    assert ids.numel() == 0 and s.cu_seqlens_q.cpu().tolist() == [0] and s.slot_mapping.numel() == 0
    # steps of different sizes through the same buffers, more calls than staging buffers
    for i in range(5):
        reqs = W.make_step_requests(65536, 16, 10 + 40 * i, 10, 2000, i, 256, 500, seed=70 + i)
        want = step_oracle.make_inputs(copy.deepcopy(reqs), 16)
        ids, s = b.make_inputs(reqs)
        torch.cuda.synchronize()
        got = {f: getattr(s, f).cpu().numpy() for f in FIELDS}
        got["input_ids"], got["prefill_input_len"] = ids.cpu().numpy(), s.prefill_input_len
        assert_same(got, want)
    with pytest.raises(ValueError, match="capacity"):
        b.make_inputs(W.make_step_requests(65536, 16, 301, 1, 5, 0, 0, 0, seed=1))


@pytest.mark.gpu
def test_against_flashinfer_helpers():
    flashinfer = pytest.importorskip("flashinfer")
    reqs = W.make_step_requests(65536, 16, 60, 1, 900, 5, 128, 400, seed=9, spare_blocks=1)
    got, s = run_builder(reqs)
    seq_lens = flashinfer.get_seq_lens(s.kv_block_indptrs, s.kv_last_block_lens, 16)
    b, p = flashinfer.get_batch_indices_positions(s.cu_seqlens_q, seq_lens, int(s.slot_mapping.numel()))
    torch.cuda.synchronize()
    assert torch.equal(b, s.batch_indices) and torch.equal(p, s.positions)


@pytest.mark.gpu
def test_slot_mapping_drives_the_cache_write_like_the_paged_arguments():
    from lmserve_b200.ops import append_paged_kv_cache, reshape_and_cache
    reqs = W.make_step_requests(512, 16, 20, 1, 300, 2, 40, 64, seed=12)
    _, s = run_builder(reqs)
    T = int(s.slot_mapping.numel())
    g = torch.Generator(device="cpu").manual_seed(3)
    key = torch.randn(T, 2, 64, generator=g).to(torch.bfloat16).to(DEV)
    value = torch.randn(T, 2, 64, generator=g).to(torch.bfloat16).to(DEV)
    a = torch.zeros(512, 2, 16, 2, 64, dtype=torch.bfloat16, device=DEV)
    b = torch.zeros_like(a)
    reshape_and_cache(key, value, a, s.slot_mapping)
    append_paged_kv_cache(key, value, s.batch_indices, s.positions, b, s.kv_block_indices,
                          s.kv_block_indptrs, s.kv_last_block_lens)
    torch.cuda.synchronize()
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    assert int((a.view(torch.int16) != 0).any(-1).any(-1).sum()) == 2 * T


@pytest.mark.gpu
def test_page_missing_from_the_table_gives_slot_minus_one_and_is_reported():
    import ctypes
    lib = _lib.lib()
    req = [InferInput([1, 2], 2, 38, 40, [4, 5, 6])]
    got, _ = run_builder(copy.deepcopy(req))
    assert got["slot_mapping"].tolist() == [6 * 16 + 6, 6 * 16 + 7]
    # a table shorter than the context: flashinfer's seq_len, counted from the table, is 4, so
    # the first 16 of the 20 new tokens get negative positions
    short = [InferInput(list(range(20)), 20, 0, 20, [4])]
    lib.lms_set_debug_checks(1)
    try:
        got, _ = run_builder(copy.deepcopy(short))
        assert got["positions"].tolist() == list(range(-16, 4))
        assert got["slot_mapping"].tolist() == [-1] * 16 + [4 * 16 + i for i in range(4)]
        idx, val = ctypes.c_int64(-1), ctypes.c_int64(0)
        assert lib.lms_check_device_errors(None, ctypes.byref(idx), ctypes.byref(val)) == _lib.LMS_ERR_INDEX
        assert 0 <= idx.value < 16 and val.value == idx.value - 16
        assert b"block table" in lib.lms_last_cuda_error()
        assert lib.lms_check_device_errors(None, None, None) == _lib.LMS_OK
    finally:
        lib.lms_set_debug_checks(0)
