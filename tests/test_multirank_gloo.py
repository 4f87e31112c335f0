"""CPU, world_size 2 over gloo: the host logic of the multi-GPU cases — rank roles, descriptor
exchange, push-pair construction with surplus reservations dropped, per-rank sharded workloads
and the max-over-ranks timing reduction.  The byte movement itself is stood in for by a
point-to-point send plus the oracle (there is no GPU here)."""
import multiprocessing as mp
import os
import socket

import numpy as np
import pytest
import torch

import workloads as W
from lmserve_b200.disagg import (Comm, build_push_pairs, kv_heads_per_rank, transfer_role)
from lmserve_b200.kv_worker import CacheDescriptor


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, q):
    try:
        from oracle import cache_oracle
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        comm = Comm(world, torch.device("cpu"), rank=rank, backend="gloo")
        dist = comm.dist
        shape = W.SHAPES["llama31_70b_tp8"].scaled(num_layers=3, num_blocks=96)
        role, peer = transfer_role(rank, world)

        # rank-local sharded work: each rank has its own seeded decode step, no exchange
        dec = W.make_decode_write(shape, 8, 16, 100, seed=1005 + rank)
        all_slots = comm.gather_objects(dec.slot_mapping.tolist())
        assert all_slots[0] != all_slots[1]

        # decode side reserves blocks (two more than needed) and publishes a descriptor
        reserved = list(range(40, 40 + 14)) if role == "decode" else []
        desc = CacheDescriptor(bytes([rank]) * 64, 0, rank, shape.num_layers, shape.num_blocks,
                               shape.num_blocks * shape.chunk_bytes, shape.chunk_bytes,
                               shape.chunk_bytes, reserved)
        descs = [CacheDescriptor.deserialize(d) for d in comm.gather_objects(desc.serialize())]
        assert [d.device_index for d in descs] == [0, 1]

        words = W.normal_words(np.random.default_rng(500 + rank), shape.cache_shape, shape.dtype)
        src_blocks = [3, 4, 5, 20, 21, 22, 60, 61, 62, 63, 7, 8]
        if role == "prefill":
            pairs = build_push_pairs(src_blocks, descs[peer].block_ids)
            assert pairs.shape == (12, 2) and pairs[:, 1].tolist() == list(range(40, 52))
            dist.send(torch.from_numpy(pairs.copy()), dst=peer)
            dist.send(torch.from_numpy(words.view(np.int16).copy()), dst=peer)
            ok = True
        else:
            pairs = torch.empty((12, 2), dtype=torch.int64)
            dist.recv(pairs, src=peer)
            src = torch.empty(shape.cache_shape, dtype=torch.int16)
            dist.recv(src, src=peer)
            got = words.copy()
            cache_oracle.transfer(src.numpy().view(np.uint16), got, pairs.numpy())
            want = words.copy()
            src_words = W.normal_words(np.random.default_rng(500 + peer), shape.cache_shape, shape.dtype)
            for s, d in zip(src_blocks, range(40, 52)):
                want[:, d] = src_words[:, s]
            ok = bool(np.array_equal(got, want)) and bool(np.array_equal(got[:, 52:54], words[:, 52:54]))
        comm.barrier()
        slowest = comm.max(10.0 + rank)
        comm.close()
        q.put((rank, ok, slowest))
    except Exception as e:  # pragma: no cover - reported to the parent
        q.put((rank, False, repr(e)))


def test_two_rank_prefill_to_decode_host_logic():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=180) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    assert [r[0] for r in results] == [0, 1]
    assert all(r[1] is True for r in results), results
    assert all(r[2] == 11.0 for r in results), results   # max over ranks seen by both


def test_roles_and_head_sharding():
    assert [transfer_role(r, 4) for r in range(4)] == [("prefill", 2), ("prefill", 3),
                                                       ("decode", 0), ("decode", 1)]
    assert transfer_role(0, 3) == ("none", None)
    assert transfer_role(5, 4) == ("none", None)
    assert kv_heads_per_rank(8, 8) == 1 and kv_heads_per_rank(8, 2) == 4
    with pytest.raises(ValueError):
        kv_heads_per_rank(8, 3)


def test_build_push_pairs_errors():
    assert build_push_pairs([], [1, 2]).shape == (0, 2)
    with pytest.raises(ValueError, match="reserved"):
        build_push_pairs([1, 2, 3], [9, 8])
    with pytest.raises(ValueError, match="distinct"):
        build_push_pairs([1, 2], [9, 9])


def test_single_process_comm_degenerates():
    c = Comm(1, torch.device("cpu"))
    c.barrier()
    assert c.max(3.5) == 3.5 and c.gather_objects("x") == ["x"]
    c.close()
