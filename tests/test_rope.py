"""Rotary position embedding: the oracle against the golden vectors made by LMServe's Triton
kernel (CPU), and the fused rotary + cache-write kernel against the oracle (GPU, bit-exact)."""
import ctypes

import numpy as np
import pytest
import torch

from helpers import load_npz, to_tensor, to_words
from lmserve_b200 import _lib
import workloads as W
from oracle import cache_oracle, rope_oracle

ROPE_CASES = ["rope_fp16_llama", "rope_fp16_d64"]
DEV = "cuda:0"


def golden(name):
    z = np.load(str(__import__("helpers").GOLDEN / f"{name}.npz"))
    f = lambda k: to_tensor(z[k], "fp16")
    return (int(z["head_dim"]), f("query"), f("key"), torch.from_numpy(z["positions"]),
            f("cos_sin_cache"), z["q_out"], z["k_out"])


@pytest.mark.parametrize("name", ROPE_CASES)
def test_oracle_matches_reference_kernel_fp16(name):
    hd, q, k, pos, cs, q_out, k_out = golden(name)
    qo, ko = rope_oracle.rotary_pos_emb(q, k, pos, cs, hd)
    assert np.array_equal(to_words(qo), q_out)
    assert np.array_equal(to_words(ko), k_out)
    # rounding every operation matters: a single-rounding fp32 evaluation differs in places
    E = hd // 2
    h = q.float().view(q.shape[0], -1, hd)
    row = cs[pos.long()].float()
    once = torch.cat((h[..., :E] * row[:, None, :E] - h[..., E:] * row[:, None, hd:hd + E],
                      h[..., E:] * row[:, None, E:hd] + h[..., :E] * row[:, None, hd + E:]), -1)
    assert not np.array_equal(to_words(once.to(torch.float16).view_as(q)), q_out)
    assert torch.allclose(once.view_as(q), qo.float(), atol=4e-3, rtol=4e-3)


COMPILED_CASES = [("rope_compiled_fp16", "fp16"), ("rope_compiled_bf16", "bf16")]


def compiled_golden(name, dt):
    z = np.load(str(__import__("helpers").GOLDEN / f"{name}.npz"))
    f = lambda k: to_tensor(z[k], dt)
    return (int(z["head_dim"]), f("query"), f("key"), torch.from_numpy(z["positions"]),
            f("cos_sin_cache"), z["q_out"], z["k_out"])


@pytest.mark.parametrize("name,dt", COMPILED_CASES)
def test_contracted_oracle_matches_compiled_triton_kernel(name, dt):
    """The golden vectors come from a compiled Triton kernel on a B200: the first product of
    each line is fused into the sum.  fp16 and bf16."""
    hd, q, k, pos, cs, q_out, k_out = compiled_golden(name, dt)
    qo, ko = rope_oracle.rotary_pos_emb(q, k, pos, cs, hd, contracted=True)
    assert np.array_equal(to_words(qo), q_out)
    assert np.array_equal(to_words(ko), k_out)
    # and the distinction matters: rounding every operation gives other last bits
    qe, _ = rope_oracle.rotary_pos_emb(q, k, pos, cs, hd, contracted=False)
    differ = (to_words(qe) != q_out).mean()
    assert 0.05 < differ < 0.5
    assert torch.allclose(qe.float(), qo.float(), atol=2e-2, rtol=2e-2)


def test_package_cos_sin_cache_matches_oracle_and_llama3_scaling():
    from lmserve_b200.ops import build_cos_sin_cache
    a = build_cos_sin_cache(128, 64, torch.bfloat16, base=500000.0)
    b = rope_oracle.build_cos_sin_cache(128, 64, torch.bfloat16, base=500000.0)
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    scaling = {"factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
               "original_max_position_embeddings": 8192}
    c = build_cos_sin_cache(64, 128, torch.float32, base=500000.0, rope_scaling=scaling)
    plain = build_cos_sin_cache(64, 128, torch.float32, base=500000.0)
    # high frequencies (short wavelengths) are untouched, the lowest frequency is divided by 8
    assert torch.equal(c[:, 0], plain[:, 0])
    inv_last = 1.0 / (500000.0 ** (126 / 128))
    assert torch.allclose(c[5, 63], torch.cos(torch.tensor(5 * inv_last / 8.0)))
    assert torch.allclose(c[5, 128 + 63], torch.sin(torch.tensor(5 * inv_last / 8.0)), atol=1e-7)


def test_cos_sin_cache_layout():
    cs = rope_oracle.build_cos_sin_cache(16, 8, torch.float32)
    assert cs.shape == (16, 16)
    inv = 1.0 / (10000.0 ** (torch.arange(0, 8, 2).float() / 8))
    assert torch.allclose(cs[3, :4], torch.cos(3 * inv)) and torch.allclose(cs[3, 4:8], torch.cos(3 * inv))
    assert torch.allclose(cs[3, 8:12], torch.sin(3 * inv))


# ------------------------------------------------------------------------------- GPU
gpu = pytest.mark.gpu


@gpu
@pytest.mark.parametrize("name", ROPE_CASES)
def test_rotary_pos_emb_golden_gpu(name):
    from lmserve_b200.ops import rotary_pos_emb
    hd, q, k, pos, cs, q_out, k_out = golden(name)
    before = _lib.lib().lms_launch_count()
    qo, ko = rotary_pos_emb(q.to(DEV), k.to(DEV), pos.to(DEV), cs.to(DEV), hd, arithmetic="round_each")
    torch.cuda.synchronize()
    assert _lib.lib().lms_launch_count() == before + 1
    assert np.array_equal(to_words(qo), q_out)
    assert np.array_equal(to_words(ko), k_out)


@gpu
@pytest.mark.parametrize("name,dt", COMPILED_CASES)
def test_rotary_pos_emb_compiled_golden_gpu(name, dt):
    """Default arithmetic = what the compiled reference kernel returns on a GPU."""
    from lmserve_b200.ops import rotary_pos_emb
    hd, q, k, pos, cs, q_out, k_out = compiled_golden(name, dt)
    qo, ko = rotary_pos_emb(q.to(DEV), k.to(DEV), pos.to(DEV), cs.to(DEV), hd)
    torch.cuda.synchronize()
    assert np.array_equal(to_words(qo), q_out)
    assert np.array_equal(to_words(ko), k_out)
    with pytest.raises(ValueError, match="arithmetic"):
        rotary_pos_emb(q.to(DEV), k.to(DEV), pos.to(DEV), cs.to(DEV), hd, arithmetic="fp32")


def fused_case(dtype, seed, T=37, NH=8, NKV=2, HD=128, NB=24, BS=16, max_pos=300, pos_dtype=torch.int32):
    g = torch.Generator().manual_seed(seed)
    qkv = torch.randn(T, (NH + 2 * NKV) * HD, generator=g).to(dtype)
    q, k, v = qkv[:, :NH * HD], qkv[:, NH * HD:(NH + NKV) * HD], qkv[:, (NH + NKV) * HD:]
    pos = torch.randint(0, max_pos, (T,), generator=g).to(pos_dtype)
    cs = rope_oracle.build_cos_sin_cache(max_pos, HD, dtype)
    cache = torch.randn(NB, 2, BS, NKV, HD, generator=g).to(dtype)
    slots = torch.randperm(NB * BS, generator=g)[:T]
    slots[[5, 20]] = -1
    return q, k, v, pos, cs, cache, slots, HD


@gpu
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("pos_dtype", [torch.int32, torch.int64])
@pytest.mark.parametrize("arithmetic", ["compiled", "round_each"])
def test_rotary_and_cache_fused_vs_oracle(dtype, pos_dtype, arithmetic):
    from lmserve_b200.ops import rotary_pos_emb, rotary_pos_emb_and_cache
    q, k, v, pos, cs, cache, slots, hd = fused_case(dtype, 7, pos_dtype=pos_dtype)
    want_q, want_k = rope_oracle.rotary_pos_emb(q, k, pos, cs, hd, contracted=arithmetic == "compiled")
    want_cache = to_words(cache).copy()
    T = q.shape[0]
    cache_oracle.reshape_and_cache(to_words(want_k).reshape(T, -1, hd), to_words(v).reshape(T, -1, hd),
                                   want_cache, slots.numpy())
    d = lambda t: t.to(DEV)
    got_cache = d(cache)
    qo, ko = rotary_pos_emb_and_cache(d(q), d(k), d(v), d(pos), d(cs), hd, got_cache, d(slots),
                                      return_key=True, arithmetic=arithmetic)
    torch.cuda.synchronize()
    assert np.array_equal(to_words(qo), to_words(want_q))
    assert np.array_equal(to_words(ko), to_words(want_k))
    assert np.array_equal(to_words(got_cache), want_cache)
    # without the key output, and the unfused op, give the same tensors
    cache2 = d(cache)
    qo2 = rotary_pos_emb_and_cache(d(q), d(k), d(v), d(pos), d(cs), hd, cache2, d(slots), arithmetic=arithmetic)
    qo3, ko3 = rotary_pos_emb(d(q), d(k), d(pos), d(cs), hd, arithmetic=arithmetic)
    torch.cuda.synchronize()
    assert torch.equal(qo2.view(torch.int16), qo.view(torch.int16))
    assert torch.equal(cache2.view(torch.int16), got_cache.view(torch.int16))
    assert torch.equal(qo3.view(torch.int16), qo.view(torch.int16))
    assert torch.equal(ko3.view(torch.int16), ko.view(torch.int16))
    if arithmetic != "round_each":
        return
    # the same values on the device one torch operation at a time (the Triton language semantics)
    E = hd // 2
    h = d(q).view(T, -1, hd)
    row = d(cs)[d(pos).long()]
    ox = h[..., :E] * row[:, None, :E] - h[..., E:] * row[:, None, hd:hd + E]
    oy = h[..., E:] * row[:, None, E:hd] + h[..., :E] * row[:, None, hd + E:]
    assert torch.equal(torch.cat((ox, oy), -1).view(T, -1).view(torch.int16), qo.view(torch.int16))


@gpu
def test_rotary_edge_cases_and_errors():
    from lmserve_b200.ops import rotary_pos_emb, rotary_pos_emb_and_cache
    cs = rope_oracle.build_cos_sin_cache(32, 64, torch.float16).to(DEV)
    q = torch.zeros(0, 4 * 64, dtype=torch.float16, device=DEV)
    k = torch.zeros(0, 64, dtype=torch.float16, device=DEV)
    qo, ko = rotary_pos_emb(q, k, torch.zeros(0, dtype=torch.int32, device=DEV), cs, 64)
    assert qo.shape == q.shape and ko.shape == k.shape
    q1 = torch.randn(3, 2 * 64, device=DEV).half()
    k1 = torch.randn(3, 64, device=DEV).half()
    pos = torch.tensor([0, 31, 7], dtype=torch.int32, device=DEV)
    qo, _ = rotary_pos_emb(q1, k1, pos, cs, 64)
    torch.cuda.synchronize()
    assert torch.equal(qo[0], q1[0])                      # position 0: cos = 1, sin = 0
    with pytest.raises(ValueError, match="full rotary"):
        rotary_pos_emb(q1, k1, pos, cs[:, :64], 64)
    with pytest.raises(TypeError):
        rotary_pos_emb(q1.float(), k1.float(), pos, cs.float(), 64)
    with pytest.raises(RuntimeError, match="no CPU path"):
        rotary_pos_emb(q1.cpu(), k1.cpu(), pos.cpu(), cs.cpu(), 64)
    # debug checks: a position outside the table is reported and the token is left unwritten
    L = _lib.lib()
    L.lms_set_debug_checks(1)
    try:
        bad = torch.tensor([0, 99, 7], dtype=torch.int32, device=DEV)
        qo, _ = rotary_pos_emb(q1, k1, bad, cs, 64)
        idx, val = ctypes.c_int64(), ctypes.c_int64()
        assert L.lms_check_device_errors(None, ctypes.byref(idx), ctypes.byref(val)) == _lib.LMS_ERR_INDEX
        assert (idx.value, val.value) == (1, 99)
    finally:
        L.lms_set_debug_checks(0)


@gpu
def test_rotary_and_cache_llama_decode_shape_bf16():
    """Llama-3.1-8B decode layer: 256 tokens, 32 query heads, 8 KV heads of 128."""
    from lmserve_b200.ops import rotary_pos_emb_and_cache
    q, k, v, pos, cs, cache, slots, hd = fused_case(torch.bfloat16, 11, T=256, NH=32, NKV=8, HD=128,
                                                     NB=64, max_pos=4096)
    want_q, want_k = rope_oracle.rotary_pos_emb(q, k, pos, cs, hd, contracted=True)
    want_cache = to_words(cache).copy()
    cache_oracle.reshape_and_cache(to_words(want_k).reshape(256, -1, hd), to_words(v).reshape(256, -1, hd),
                                   want_cache, slots.numpy())
    d = lambda t: t.to(DEV)
    got = d(cache)
    qo = rotary_pos_emb_and_cache(d(q), d(k), d(v), d(pos), d(cs), hd, got, d(slots))
    torch.cuda.synchronize()
    assert np.array_equal(to_words(qo), to_words(want_q))
    assert np.array_equal(to_words(got), want_cache)
