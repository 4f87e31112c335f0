"""Generates the golden vectors in this directory from LMServe's own Triton kernels.

Run where the LMServe source tree is available (``LMSERVE_SRC``, or a ``reference`` directory
next to this repository) and triton is installed:

    TRITON_INTERPRET=1 python tests/golden/make_golden.py

The two kernels of ``runtime/worker/llm_worker/ops/triton/cache_kernels.py`` are executed
on CPU tensors by the Triton interpreter (see ``oracle/triton_ref.py``).  Small cases are
stored whole (inputs and outputs, raw 16-bit words); the full-size plumbing case (Llama-3.2-1B
shape, 256 tokens / 64 block pairs) is stored as SHA-256 digests of its seeded inputs and of
the reference outputs, because the caches are 32 MiB each.
"""
from __future__ import annotations

import hashlib
import json
import os
import sys
from pathlib import Path

os.environ.setdefault("TRITON_INTERPRET", "1")
HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

import numpy as np
import torch

import workloads as W
from oracle import triton_ref

TORCH_DT = {"fp16": torch.float16, "bf16": torch.bfloat16}


def words_to_tensor(words: np.ndarray, dtype: str) -> torch.Tensor:
    return torch.from_numpy(words.view(np.int16).copy()).view(TORCH_DT[dtype])


def tensor_to_words(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def small_fill(name, seed, dtype, T, H, D, num_slots):
    rng = np.random.default_rng(seed)
    key = W.normal_words(rng, (T, H, D), dtype)
    value = W.normal_words(rng, (T, H, D), dtype)
    kc = W.normal_words(rng, (num_slots, H, D), dtype)
    vc = W.normal_words(rng, (num_slots, H, D), dtype)
    slots = rng.permutation(num_slots)[:T].astype(np.int64)
    tk, tv = words_to_tensor(key, dtype), words_to_tensor(value, dtype)
    tkc, tvc = words_to_tensor(kc, dtype), words_to_tensor(vc, dtype)
    triton_ref.fill_key_cache(tk, tv, tkc, tvc, torch.from_numpy(slots))
    np.savez_compressed(HERE / f"{name}.npz", dtype=dtype, key=key, value=value,
                        key_cache_in=kc, value_cache_in=vc, slot_mapping=slots,
                        key_cache_out=tensor_to_words(tkc), value_cache_out=tensor_to_words(tvc))


def small_copy(name, seed, dtype, L, NB, BS, H, D, pairs):
    rng = np.random.default_rng(seed)
    kv = W.normal_words(rng, (L, NB, 2, BS, H, D), dtype)
    t = words_to_tensor(kv, dtype)
    p = np.asarray(pairs, dtype=np.int64)
    triton_ref.copy_blocks(t, torch.from_numpy(p))
    np.savez_compressed(HERE / f"{name}.npz", dtype=dtype, kv_in=kv, pairs=p,
                        kv_out=tensor_to_words(t))


def plumbing_digests():
    case = W.config1()
    s = case.shape
    pay = W.plumbing_payload(case, seed=2001)
    key, value, kc, vc, kv = (pay[k] for k in ("key", "value", "key_cache", "value_cache", "kv_caches"))
    live = case.slot_mapping >= 0
    tkc, tvc = words_to_tensor(kc, s.dtype), words_to_tensor(vc, s.dtype)
    # the reference kernel has no padding guard: it only ever sees the live tokens
    triton_ref.fill_key_cache(words_to_tensor(key[live], s.dtype), words_to_tensor(value[live], s.dtype),
                              tkc, tvc, torch.from_numpy(case.slot_mapping[live]))
    tkv = words_to_tensor(kv, s.dtype)
    triton_ref.copy_blocks(tkv, torch.from_numpy(case.pairs))
    out = {
        "generator": {"workload_seed": 1001, "payload_seed": 2001},
        "inputs": {"key": sha(key), "value": sha(value), "key_cache": sha(kc), "value_cache": sha(vc),
                   "kv_caches": sha(kv), "slot_mapping": sha(case.slot_mapping), "pairs": sha(case.pairs)},
        "outputs": {"key_cache": sha(tensor_to_words(tkc)), "value_cache": sha(tensor_to_words(tvc)),
                    "kv_caches": sha(tensor_to_words(tkv))},
        "live_tokens": int(live.sum()),
    }
    (HERE / "plumbing_llama32_1b.json").write_text(json.dumps(out, indent=1) + "\n")


def rope_case(name, seed, T, NH, NKV, HD, max_pos=512):
    """fp16 only: the interpreter evaluates bf16 arithmetic to NaN."""
    from oracle import rope_oracle
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(T, NH * HD, generator=g).to(torch.float16)
    k = torch.randn(T, NKV * HD, generator=g).to(torch.float16)
    pos = torch.randint(0, max_pos, (T,), generator=g, dtype=torch.int32)
    cs = rope_oracle.build_cos_sin_cache(max_pos, HD, torch.float16)
    qo, ko = triton_ref.rotary_pos_emb(q, k, pos, cs, HD)
    np.savez_compressed(HERE / f"{name}.npz", head_dim=HD, query=tensor_to_words(q),
                        key=tensor_to_words(k), positions=pos.numpy(),
                        cos_sin_cache=tensor_to_words(cs), q_out=tensor_to_words(qo),
                        k_out=tensor_to_words(ko))


def main():
    if not triton_ref.available():
        raise SystemExit("LMServe source tree not found; set LMSERVE_SRC")
    small_fill("fill_fp16_t8", 11, "fp16", 8, 2, 8, 64)
    small_fill("fill_bf16_t24", 12, "bf16", 24, 4, 16, 128)
    small_fill("fill_bf16_row1536", 13, "bf16", 5, 3, 256, 16)   # row not a power of two
    small_copy("copy_fp16_fanout", 21, "fp16", 2, 16, 4, 2, 8,
               [(1, 9), (1, 10), (1, 15), (3, 0), (7, 12)])
    small_copy("copy_bf16_l3", 22, "bf16", 3, 12, 16, 1, 16, [(0, 11), (5, 6), (5, 7), (2, 1)])
    rope_case("rope_fp16_llama", 31, 6, 4, 2, 128)
    rope_case("rope_fp16_d64", 32, 9, 3, 1, 64, max_pos=64)
    plumbing_digests()
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    main()
