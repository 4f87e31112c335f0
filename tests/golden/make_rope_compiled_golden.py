"""Golden vectors for the rotary embedding as a COMPILED Triton kernel evaluates it on a GPU.

Needs a CUDA GPU with Triton; writes ``rope_compiled_{fp16,bf16}.npz`` beside this file (or into
the directory given as the first argument).  The LMServe source tree is not needed and not
read: the kernel below restates the two arithmetic lines of LMServe's
``apply_rotary_pos_emb_kernel`` (``ops/triton/rotary_embedding.py:48-49`` and ``:60-61``)

    out_x = x * cos_x - y * sin_x          out_y = y * cos_y + x * sin_y

on operands gathered on the host exactly as that kernel indexes them, so that the Triton
compiler decides — as it does for the reference — which products are fused into the sums.
(The Triton interpreter, which produced ``rope_fp16_*.npz``, rounds every operation instead and
cannot evaluate bf16 at all.)  Inputs are seeded; the same seeds regenerate them anywhere.
"""
import sys
from pathlib import Path

import numpy as np
import torch
import triton
import triton.language as tl

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
from lmserve_b200.ops import build_cos_sin_cache  # noqa: E402


@triton.jit
def rotate_lines(x_ptr, y_ptr, cx_ptr, cy_ptr, sx_ptr, sy_ptr, ox_ptr, oy_ptr, n, BLOCK: tl.constexpr):
    i = tl.program_id(0) * BLOCK + tl.arange(0, BLOCK)
    m = i < n
    x = tl.load(x_ptr + i, mask=m)
    y = tl.load(y_ptr + i, mask=m)
    cos_x = tl.load(cx_ptr + i, mask=m)
    cos_y = tl.load(cy_ptr + i, mask=m)
    sin_x = tl.load(sx_ptr + i, mask=m)
    sin_y = tl.load(sy_ptr + i, mask=m)
    tl.store(ox_ptr + i, x * cos_x - y * sin_x, mask=m)
    tl.store(oy_ptr + i, y * cos_y + x * sin_y, mask=m)


def rotate(x, positions, cos_sin_cache, head_dim):
    T, E = x.shape[0], head_dim // 2
    h = x.reshape(T, -1, head_dim)
    heads = h.shape[1]
    row = cos_sin_cache[positions.long()]
    ex = lambda t: t[:, None, :].expand(T, heads, E).contiguous().reshape(-1)
    xx, xy = h[..., :E].contiguous().reshape(-1), h[..., E:].contiguous().reshape(-1)
    ox, oy = torch.empty_like(xx), torch.empty_like(xy)
    n = xx.numel()
    rotate_lines[(triton.cdiv(n, 256),)](
        xx, xy, ex(row[:, :E]), ex(row[:, E:head_dim]), ex(row[:, head_dim:head_dim + E]),
        ex(row[:, head_dim + E:]), ox, oy, n, BLOCK=256)
    return torch.cat((ox.reshape(T, heads, E), oy.reshape(T, heads, E)), dim=-1).reshape(T, -1)


def words(t):
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def case(out_dir, name, dtype, seed, T, NH, NKV, HD, max_pos):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(T, NH * HD, generator=g).to(dtype)
    k = torch.randn(T, NKV * HD, generator=g).to(dtype)
    pos = torch.randint(0, max_pos, (T,), generator=g, dtype=torch.int32)
    cs = build_cos_sin_cache(max_pos, HD, dtype, base=500000.0)
    qo = rotate(q.cuda(), pos.cuda(), cs.cuda(), HD)
    ko = rotate(k.cuda(), pos.cuda(), cs.cuda(), HD)
    torch.cuda.synchronize()
    np.savez_compressed(out_dir / f"{name}.npz", head_dim=HD, query=words(q), key=words(k),
                        positions=pos.numpy(), cos_sin_cache=words(cs), q_out=words(qo), k_out=words(ko),
                        triton_version=triton.__version__, gpu=torch.cuda.get_device_name(0))


def main():
    out_dir = Path(sys.argv[1]) if len(sys.argv) > 1 else HERE
    out_dir.mkdir(parents=True, exist_ok=True)
    case(out_dir, "rope_compiled_fp16", torch.float16, 41, 16, 4, 2, 128, 4096)
    case(out_dir, "rope_compiled_bf16", torch.bfloat16, 42, 16, 4, 2, 128, 4096)
    print("written to", out_dir)


if __name__ == "__main__":
    main()
