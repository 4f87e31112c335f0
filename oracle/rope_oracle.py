"""CPU restatement of LMServe's rotary position embedding (the checker for the fused
rotary + cache-write kernel).  TEST INFRASTRUCTURE ONLY.

Follows ``apply_rotary_pos_emb_kernel`` (``runtime/worker/llm_worker/ops/triton/
rotary_embedding.py:5-66``) and its launcher ``rotary_pos_emb`` (``ops/rotary_embedding_ops.py:
8-38``): per token, per head, ``x`` = first half of the head, ``y`` = second half,

    out_x = x * cos[i] - y * sin[i]          out_y = y * cos[E + i] + x * sin[E + i]

with ``cos = cos_sin_cache[pos, :D]``, ``sin = cos_sin_cache[pos, D:]`` and ``E = D / 2``.
The kernel computes in the tensors' element type, so every product and every sum is rounded
to fp16 / bf16; this restatement does the same by evaluating one torch CPU operation at a
time on fp16 / bf16 tensors.

Parity pin: for fp16 the restatement is bit-identical to the reference kernel executed by the
Triton interpreter (golden vectors ``tests/golden/rope_fp16_*.npz``).  For bf16 the interpreter
does not produce usable output (it returns NaN for bf16 arithmetic), so bf16 is the same
operation sequence, unpinned by the reference.  A compiled Triton kernel may contract a product
and a sum into one fused operation, which changes some last bits; neither form is "the"
reference result, the per-operation form is the one the kernel's source states.
"""
from __future__ import annotations

import torch


def build_cos_sin_cache(max_position: int, head_dim: int, dtype: torch.dtype,
                        base: float = 10000.0) -> torch.Tensor:
    """``[max_position, 2 * head_dim]``: cos then sin of ``cat(freqs, freqs)`` — the table
    ``RotaryEmbedding.__init__`` registers (``models/layers/rotary_embedding.py:27-71``,
    without the Llama-3 frequency rescaling, which only changes ``inv_freq``)."""
    inv_freq = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.int64).float() / head_dim))
    t = torch.arange(max_position).float()
    freqs = torch.einsum("i,j->ij", t, inv_freq)
    emb = torch.cat((freqs, freqs), dim=-1)
    return torch.cat((emb.cos().to(dtype), emb.sin().to(dtype)), dim=-1)


def rotate(x: torch.Tensor, positions: torch.Tensor, cos_sin_cache: torch.Tensor,
           head_dim: int) -> torch.Tensor:
    """x: [T, heads * head_dim] (fp16 / bf16, CPU) -> rotated tensor of the same shape."""
    T = x.shape[0]
    E = head_dim // 2
    h = x.reshape(T, -1, head_dim)
    row = cos_sin_cache[positions.long()]            # [T, 2D]
    cos, sin = row[:, None, :head_dim], row[:, None, head_dim:]
    xx, xy = h[..., :E], h[..., E:]
    out_x = xx * cos[..., :E] - xy * sin[..., :E]    # each op rounds to the element type
    out_y = xy * cos[..., E:] + xx * sin[..., E:]
    return torch.cat((out_x, out_y), dim=-1).reshape(T, -1)


def rotary_pos_emb(query, key, positions, cos_sin_cache, head_dim):
    """(q_out, k_out) of ``ops/rotary_embedding_ops.py:8-38``."""
    return (rotate(query, positions, cos_sin_cache, head_dim),
            rotate(key, positions, cos_sin_cache, head_dim))
