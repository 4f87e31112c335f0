"""CPU oracle of the KV-cache data-movement path.  TEST INFRASTRUCTURE ONLY.

Nothing in ``lmserve_b200`` imports this package.  It may be imported by
``tests/``, by ``__graft_entry__.smoke()`` and by ``bench.py``'s CPU-baseline /
reference arm, always as the checker or the timed baseline and never as a data
path of the product.

Parity pin: LMServe ships no tests, golden vectors or fixtures for this path, so
the oracle is pinned against LMServe's own Triton cache kernels
(``runtime/worker/llm_worker/ops/triton/cache_kernels.py``) executed on CPU with
the Triton interpreter; the outputs are committed under ``tests/golden/`` together
with ``tests/golden/make_golden.py`` that produced them.  The swap and transfer
restatements are pinned the same way: LMServe's own ``kv_worker.py`` is loaded by path
with stand-ins for pycuda / NIXL / the protobuf module (``oracle/kv_worker_ref.py``)
and its methods are run on host buffers; ``tests/golden/make_swap_golden.py`` committed
the vectors (``swap_*.npz``, ``transfer_*.npz``).
``rope_oracle`` has two arithmetic forms: rounded per operation (pinned for fp16 by the
reference kernel under the Triton interpreter) and contracted as compiled Triton evaluates it
(pinned for fp16 and bf16 by vectors made on a B200, ``tests/golden/rope_compiled_*.npz``).
``step_oracle`` (per-step index preparation) restates ``model_worker.py:310-433`` and the two
flashinfer helpers it calls; it is pinned by the worked example in flashinfer's documentation
and, on a GPU box, by the installed flashinfer functions themselves.
"""
