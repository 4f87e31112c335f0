"""Generates the swap / transfer golden vectors from LMServe's own ``kv_worker.py``.

Run where the LMServe source tree is available (``LMSERVE_SRC``, or a ``reference`` directory
next to this repository):

    python tests/golden/make_swap_golden.py

``oracle/kv_worker_ref.py`` loads ``runtime/worker/llm_worker/kv_worker.py`` by path with
stand-ins for pycuda / NIXL / the protobuf module and calls the reference's own methods on host
arrays (``copy_kv`` -> ``save_kv_blocks_to_host`` / ``load_kv_blocks_from_host``, the per-layer
``_save_layer_…`` / ``_load_layer_…``, ``get_descriptors``, ``_push_kv``, ``pull_kv``).  Inputs
and outputs are stored whole as raw 16-bit words.
"""
from __future__ import annotations

import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

import numpy as np

from oracle import kv_worker_ref as R


def words(rng, shape):
    return rng.integers(0, 2 ** 16, size=shape, dtype=np.uint16)


def distinct(rng, n, k):
    return rng.permutation(n)[:k].astype(np.int64)


def swap_case(name, seed, L, NB, NHB, chunk_words, n_out, n_in, split):
    """copy_kv(GPU -> Host) of n_out blocks, then copy_kv(Host -> GPU) of n_in blocks."""
    rng = np.random.default_rng(seed)
    gpu, host = words(rng, (L, NB, chunk_words)), words(rng, (NHB, L, chunk_words))
    out_pairs = np.stack([distinct(rng, NB, n_out), distinct(rng, NHB, n_out)], axis=1)
    in_pairs = np.stack([distinct(rng, NHB, n_in), distinct(rng, NB, n_in)], axis=1)
    g, h = gpu.copy(), host.copy()
    w = R.RefWorker(g, h)
    w.swap_out(out_pairs, split=split)
    host_after_out = h.copy()
    assert np.array_equal(g, gpu)
    posted = [e.waited for e in w.worker.kv_worker_handle.post_events]
    w.swap_in(in_pairs, split=split)
    recorded = [e.recorded for e in w.worker.kv_worker_handle.pre_events]
    np.savez_compressed(HERE / f"{name}.npz", gpu_in=gpu, host_in=host, out_pairs=out_pairs,
                        in_pairs=in_pairs, host_after_out=host_after_out, gpu_after_in=g.copy(),
                        host_after_in=h.copy(), post_event_waits=np.asarray(posted),
                        pre_event_records=np.asarray(recorded),
                        model_queue_tokens=w.model_queue.qsize())


def layer_case(name, seed, L, NB, NHB, chunk_words, n, layer):
    """One layer only, through ``_save_layer_kv_blocks_to_host`` / ``_load_layer_…``."""
    rng = np.random.default_rng(seed)
    gpu, host = words(rng, (L, NB, chunk_words)), words(rng, (NHB, L, chunk_words))
    out_pairs = np.stack([distinct(rng, NB, n), distinct(rng, NHB, n)], axis=1)
    in_pairs = np.stack([distinct(rng, NHB, n), distinct(rng, NB, n)], axis=1)
    g, h = gpu.copy(), host.copy()
    w = R.RefWorker(g, h)
    w.save_layer(out_pairs, layer)
    host_after_out = h.copy()
    w.load_layer(in_pairs, layer)
    np.savez_compressed(HERE / f"{name}.npz", gpu_in=gpu, host_in=host, out_pairs=out_pairs,
                        in_pairs=in_pairs, layer=layer, host_after_out=host_after_out,
                        gpu_after_in=g.copy())


def transfer_case(name, seed, L, NB_src, NB_dst, NHB, chunk_words, n, surplus, pull=False):
    """Prefill GPU blocks -> decode GPU blocks through both host pools, the way the engine
    drives it: write-through, descriptors of the reserved (and ``surplus`` extra) decode host
    blocks, NIXL WRITE (``_push_kv``) or READ (``pull_kv``), fetch."""
    rng = np.random.default_rng(seed)
    src_gpu, dst_gpu = words(rng, (L, NB_src, chunk_words)), words(rng, (L, NB_dst, chunk_words))
    src_host, dst_host = words(rng, (NHB, L, chunk_words)), words(rng, (NHB, L, chunk_words))
    src_blocks, dst_blocks = distinct(rng, NB_src, n), distinct(rng, NB_dst, n)
    hp = distinct(rng, NHB, n)                       # prefill-side host blocks
    hd_all = distinct(rng, NHB, n + surplus)         # decode-side host blocks (reserved ahead)
    hd, extra = hd_all[:n], hd_all[n:]
    sg, dg, sh, dh = src_gpu.copy(), dst_gpu.copy(), src_host.copy(), dst_host.copy()
    prefill, decode = R.RefWorker(sg, sh, "prefill"), R.RefWorker(dg, dh, "decode")
    if not pull:
        ok = R.disaggregated_push(prefill, decode, src_blocks, dst_blocks, hp, hd, extra)
    else:
        # READ has no truncation (``kv_worker.py:417-434``): the lists must be equally long
        prefill.swap_out(np.stack([src_blocks, hp], axis=1))
        ok = decode.pull(prefill.get_descriptors(hp), hd)
        decode.swap_in(np.stack([hd, dst_blocks], axis=1))
    assert ok is True
    np.savez_compressed(HERE / f"{name}.npz", src_gpu=src_gpu, dst_gpu_in=dst_gpu,
                        dst_host_in=dst_host, pairs=np.stack([src_blocks, dst_blocks], axis=1),
                        prefill_host_blocks=hp, decode_host_blocks=hd, surplus_host_blocks=extra,
                        dst_host_out=dh.copy(), dst_gpu_out=dg.copy())


def main():
    if not R.available():
        raise SystemExit("LMServe source tree not found; set LMSERVE_SRC")
    # chunk = 2 * BS * H * D words
    swap_case("swap_bf16_l3", 41, L=3, NB=12, NHB=9, chunk_words=2 * 4 * 2 * 8, n_out=6, n_in=5,
              split=4)
    swap_case("swap_fp16_l5", 42, L=5, NB=7, NHB=16, chunk_words=2 * 16 * 1 * 8, n_out=7, n_in=7,
              split=0)
    swap_case("swap_empty", 43, L=2, NB=4, NHB=4, chunk_words=64, n_out=0, n_in=0, split=0)
    layer_case("swap_layer2_of_4", 44, L=4, NB=9, NHB=6, chunk_words=96, n=4, layer=2)
    transfer_case("transfer_push_surplus", 45, L=4, NB_src=10, NB_dst=14, NHB=12,
                  chunk_words=2 * 4 * 1 * 16, n=6, surplus=3)
    transfer_case("transfer_push_exact", 46, L=2, NB_src=6, NB_dst=6, NHB=8, chunk_words=64,
                  n=5, surplus=0)
    transfer_case("transfer_pull", 47, L=3, NB_src=8, NB_dst=9, NHB=8, chunk_words=128, n=4,
                  surplus=0, pull=True)
    print("swap / transfer golden vectors written to", HERE)


if __name__ == "__main__":
    main()
