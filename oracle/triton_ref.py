"""Runs LMServe's own Triton cache kernels on CPU through the Triton interpreter.

Only usable where the LMServe source tree is present (the directory named by ``LMSERVE_SRC``,
or a ``reference`` directory next to this repository); it is what ``tests/golden/make_golden.py`` uses to produce the
committed golden vectors, and what the optional cross-check test uses when the tree is
there.  ``cache_kernels.py`` is loaded by file path because importing the ``llm_worker``
package pulls in pycuda and nixl; the launch arguments are those of the reference
launchers (``ops/cache_ops.py:26-36`` and ``:49-59``), which themselves hard-code
``device='cuda'`` and cannot run here.  TEST INFRASTRUCTURE ONLY.
"""
from __future__ import annotations

import importlib.util
import os
from pathlib import Path

KERNEL_FILE = "runtime/worker/llm_worker/ops/triton/cache_kernels.py"


def reference_root() -> Path:
    env = os.environ.get("LMSERVE_SRC")
    if env:
        return Path(env)
    return Path(__file__).resolve().parents[2] / "reference"


def available() -> bool:
    return (reference_root() / KERNEL_FILE).exists()


ROPE_KERNEL_FILE = "runtime/worker/llm_worker/ops/triton/rotary_embedding.py"
_modules = {}


def _load(rel_path: str):
    if rel_path not in _modules:
        if os.environ.get("TRITON_INTERPRET") != "1":
            raise RuntimeError("set TRITON_INTERPRET=1 before triton is first imported")
        spec = importlib.util.spec_from_file_location(
            "lmserve_ref_" + Path(rel_path).stem, reference_root() / rel_path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _modules[rel_path] = mod
    return _modules[rel_path]


def _kernels():
    return _load(KERNEL_FILE)


def rotary_pos_emb(query, key, positions, cos_sin_cache, head_dim):
    """``rotary_pos_emb`` of ``ops/rotary_embedding_ops.py:8-38`` (same launch arguments)."""
    import torch
    num_tokens = positions.shape[0]
    num_heads = query.shape[1] // head_dim
    num_kv_heads = key.shape[1] // head_dim
    rotary_dim = cos_sin_cache.shape[-1] // 2
    q_out, k_out = torch.empty_like(query), torch.empty_like(key)
    _load(ROPE_KERNEL_FILE).apply_rotary_pos_emb_kernel[(num_tokens,)](
        query, key, positions, cos_sin_cache, q_out, k_out, num_tokens, num_heads,
        num_kv_heads, head_dim, rotary_dim, BLOCK_SIZE=rotary_dim // 2)
    return q_out, k_out


def copy_blocks(kv_caches, pairs) -> None:
    """``copy_blocks`` of ``ops/cache_ops.py:8-36`` minus the device='cuda' table upload.
    kv_caches: CPU torch tensor [L, NB, ...]; pairs: int64 torch tensor [n, 2]."""
    import torch
    block_maps = pairs.reshape(-1).to(torch.long).contiguous()
    n = block_maps.numel() // 2
    if n == 0:
        return
    grid = (kv_caches.shape[0], n)
    _kernels().copy_blocks_kernel[grid](
        kv_caches,
        block_maps_ptr=block_maps,
        numel_per_layer=kv_caches[0].numel(),
        numel_per_block=kv_caches[0][0].numel(),
        BLOCK_SIZE=1024,
    )


def fill_key_cache(key, value, key_cache, value_cache, slot_mapping) -> None:
    """``fill_key_cache`` of ``ops/cache_ops.py:39-59``.  The kernel has no guard for
    negative slots (it would write before the cache), so they are refused here."""
    if bool((slot_mapping < 0).any()):
        raise ValueError("the reference kernel must not be given negative slots")
    grid = (len(slot_mapping),)
    _kernels().fill_key_cache_kernel[grid](
        key, value, key_cache, value_cache, slot_mapping,
        key.shape[1], key.shape[2], BLOCK_SIZE=1024,
    )
