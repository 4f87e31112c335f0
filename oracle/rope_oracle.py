"""CPU restatement of LMServe's rotary position embedding (the checker for the fused
rotary + cache-write kernel).  TEST INFRASTRUCTURE ONLY.

Follows ``apply_rotary_pos_emb_kernel`` (``runtime/worker/llm_worker/ops/triton/
rotary_embedding.py:5-66``) and its launcher ``rotary_pos_emb`` (``ops/rotary_embedding_ops.py:
8-38``): per token, per head, ``x`` = first half of the head, ``y`` = second half,

    out_x = x * cos[i] - y * sin[i]          out_y = y * cos[E + i] + x * sin[E + i]

with ``cos = cos_sin_cache[pos, :D]``, ``sin = cos_sin_cache[pos, D:]`` and ``E = D / 2``.
The kernel computes in the tensors' element type, and the two lines have two evaluations:

* ``contracted=False`` — every product and every sum rounded to fp16 / bf16, the Triton language
  semantics; restated by evaluating one torch CPU operation at a time on fp16 / bf16 tensors.
  Pin: for fp16, bit-identical to the reference kernel executed by the Triton interpreter
  (golden vectors ``tests/golden/rope_fp16_*.npz``); the interpreter returns NaN for bf16
  arithmetic, so bf16 in this form is the same operation sequence, unpinned.
* ``contracted=True`` — what the Triton compiler emits for a GPU, i.e. what the reference
  returns when it runs: the first product of each line is fused into the sum,
  ``out_x = fma(x, cos, -rn(y * sin))``, ``out_y = fma(y, cos, rn(x * sin))``.  Restated here
  with exact arithmetic (error-free sums in float64, one explicit rounding to the element
  type).  Pin: ``tests/golden/rope_compiled_{fp16,bf16}.npz``, made on a B200 by a compiled
  Triton kernel of the same two lines (``tests/golden/make_rope_compiled_golden.py``).
"""
from __future__ import annotations

import numpy as np
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


_FORMAT = {torch.float16: (11, -14), torch.bfloat16: (8, -126)}  # significand bits, min normal exponent


def _round_sum_to(s: np.ndarray, e: np.ndarray, dtype: torch.dtype) -> torch.Tensor:
    """Rounds the exact value s + e (float64 arrays, |e| <= ulp(s)/2) to `dtype`, nearest-even."""
    p, emin = _FORMAT[dtype]
    neg = np.signbit(s)
    a = np.abs(s)
    ee = np.where(neg, -e, e)
    _, ex = np.frexp(a)                      # a = m * 2**ex with m in [0.5, 1)
    q = np.ldexp(1.0, np.maximum(ex - 1, emin) - (p - 1))   # spacing of `dtype` at |s|
    k = np.floor(a / q)
    lo = k * q
    r = a - lo
    half = q / 2
    up = (r > half) | ((r == half) & ((ee > 0) | ((ee == 0) & (np.mod(k, 2) == 1))))
    res = np.where(up, lo + q, lo)
    return torch.from_numpy(np.where(neg, -res, res)).to(dtype)


def _fma(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor) -> torch.Tensor:
    """rn(a * b + c) in the element type of `a` with a single rounding (fp16 / bf16, CPU)."""
    p = a.double().numpy() * b.double().numpy()       # exact: at most 22 significant bits
    cc = np.broadcast_to(c.double().numpy(), p.shape)
    s = p + cc
    bb = s - p
    err = (p - (s - bb)) + (cc - bb)                  # two-sum: p + c == s + err exactly
    return _round_sum_to(s, err, a.dtype)


def rotate(x: torch.Tensor, positions: torch.Tensor, cos_sin_cache: torch.Tensor,
           head_dim: int, contracted: bool = False) -> torch.Tensor:
    """x: [T, heads * head_dim] (fp16 / bf16, CPU) -> rotated tensor of the same shape."""
    T = x.shape[0]
    E = head_dim // 2
    h = x.reshape(T, -1, head_dim)
    row = cos_sin_cache[positions.long()]            # [T, 2D]
    cos, sin = row[:, None, :head_dim], row[:, None, head_dim:]
    xx, xy = h[..., :E], h[..., E:]
    if contracted:
        cx, cy, sx, sy = (t.expand_as(xx) for t in (cos[..., :E], cos[..., E:], sin[..., :E], sin[..., E:]))
        out_x = _fma(xx, cx, -(xy * sx))             # the second product is rounded on its own
        out_y = _fma(xy, cy, xx * sy)
    else:
        out_x = xx * cos[..., :E] - xy * sin[..., :E]    # each op rounds to the element type
        out_y = xy * cos[..., E:] + xx * sin[..., E:]
    return torch.cat((out_x, out_y), dim=-1).reshape(T, -1)


def rotary_pos_emb(query, key, positions, cos_sin_cache, head_dim, contracted: bool = False):
    """(q_out, k_out) of ``ops/rotary_embedding_ops.py:8-38``."""
    return (rotate(query, positions, cos_sin_cache, head_dim, contracted),
            rotate(key, positions, cos_sin_cache, head_dim, contracted))
