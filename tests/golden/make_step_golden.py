"""Golden vectors for the per-step index preparation, made with flashinfer's own helpers.

Needs a CUDA GPU with flashinfer; writes ``step_indices_flashinfer.npz`` beside this file (or
into the directory given as the first argument).  The request list is seeded
(``workloads.make_step_requests``); the page-table arrays are built from it the way
``ModelWorker._make_inputs`` does (``model_worker.py:399-423``) and handed to
``flashinfer.get_seq_lens`` / ``flashinfer.get_batch_indices_positions`` (``:425-433``), whose
outputs are what the CPU oracle has to reproduce.  The LMServe tree is not read.
"""
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
import workloads as W  # noqa: E402

GENERATOR = dict(num_blocks=65536, block_size=16, num_decode=60, ctx_lo=1, ctx_hi=900, num_prefill=5,
                 chunk_tokens=128, max_offset=400, seed=9, spare_blocks=1)


def main():
    import flashinfer
    out_dir = Path(sys.argv[1]) if len(sys.argv) > 1 else HERE
    out_dir.mkdir(parents=True, exist_ok=True)
    reqs = W.make_step_requests(**GENERATOR)
    reqs.sort(key=lambda x: -x.input_len)
    page = GENERATOR["block_size"]
    dev = "cuda:0"
    t = lambda a: torch.tensor(a, dtype=torch.int).to(dev)
    cu_q = t(np.cumsum([0] + [r.input_len for r in reqs]))
    indptr = t(np.cumsum([0] + [len(r.block_ids) for r in reqs]))
    last = t([(r.context_len - 1) % page + 1 for r in reqs])
    nnz = int(sum(r.input_len for r in reqs))
    seq_lens = flashinfer.get_seq_lens(indptr, last, page)
    b, p = flashinfer.get_batch_indices_positions(cu_q, seq_lens, nnz)
    torch.cuda.synchronize()
    np.savez_compressed(out_dir / "step_indices_flashinfer.npz", seq_lens=seq_lens.cpu().numpy(),
                        batch_indices=b.cpu().numpy(), positions=p.cpu().numpy(),
                        flashinfer_version=getattr(flashinfer, "__version__", "?"))
    print("written to", out_dir)


if __name__ == "__main__":
    main()
