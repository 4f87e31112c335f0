"""GPU: whole model steps through the cache path — index preparation, copy-on-write, the
per-layer paged cache write from inside attention layers with the handshake hooks, and a KV
worker on another thread writing finished blocks through to the host — against the composition
of the oracles."""
import copy
import queue
import threading

import numpy as np
import pytest
import torch

from helpers import to_tensor, to_words
import workloads as W
from lmserve_b200.kv_worker import BlockMapping, Device, KVWorker, KVWorkerHandle
from lmserve_b200.model_step import ModelStepCache
from oracle import cache_oracle, step_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


class Attention(torch.nn.Module):
    """A stand-in attention layer: derives this step's K / V rows from the token ids and its
    layer number, and writes them into the paged cache the way LMServe's layer does."""

    def __init__(self, layer, step_cache, H, D):
        super().__init__()
        self.layer, self.step_cache, self.H, self.D = layer, step_cache, H, D
        self.params = None

    def kv(self, input_ids):
        T = input_ids.shape[0]
        base = (input_ids.to(torch.float32) % 997)[:, None, None] / 64.0
        ramp = torch.arange(self.H * self.D, device=input_ids.device, dtype=torch.float32).view(1, self.H, self.D)
        k = (base + ramp / 512.0 + self.layer).to(torch.bfloat16).expand(T, self.H, self.D).contiguous()
        return k, (k.float() * -1.5).to(torch.bfloat16)

    def forward(self, input_ids):
        k, v = self.kv(input_ids)
        self.step_cache.write_layer(self.layer, k, v, self.params)
        return input_ids


def test_three_model_steps_with_copy_on_write_and_write_through():
    L_, NB, BS, H, D = 3, 96, 16, 2, 64
    shape = W.KVShape("toy", L_, H, D, "bf16", NB, BS)
    rng = np.random.default_rng(2025)
    words = W.normal_words(rng, shape.cache_shape, "bf16")
    kv = to_tensor(words, "bf16", DEV)
    want = words.copy()
    events = ([torch.cuda.Event() for _ in range(L_)], [torch.cuda.Event() for _ in range(L_)])
    handle = KVWorkerHandle(*events, model_queue=queue.Queue(), kv_queue=queue.Queue())
    model_stream = torch.cuda.Stream()
    step_cache = ModelStepCache(kv, handle, stream=model_stream, max_batch=32, max_tokens=512, max_blocks=512)
    layers = torch.nn.ModuleList(Attention(l, step_cache, H, D) for l in range(L_))
    handle.register_hooks(layers, stream=model_stream)
    worker = KVWorker("kv0", kv, num_host_blocks=8)
    worker.model_queue, worker.kv_queue = handle.model_queue, handle.kv_queue
    host_want = np.zeros((8, L_, shape.chunk_bytes // 2), np.uint16)
    worker.host_pool.array[...] = 0
    try:
        for step in range(3):
            # a mixed step: 5 decode requests and 2 prefill chunks, in blocks 0 .. 63
            reqs = W.make_step_requests(64, BS, 5, 3, 60, 2, 40, 100, seed=700 + step)
            ref = step_oracle.make_inputs(copy.deepcopy(reqs), BS)
            # copy-on-write of two blocks into the free range 64 .. 95 before the forward pass
            cow = {int(ref["kv_block_indices"][0]): [64 + 2 * step, 65 + 2 * step]}
            save = np.array([[int(ref["kv_block_indices"][1]), step]], dtype=np.int64)  # -> host block
            record = True
            t = threading.Thread(target=lambda: (torch.cuda.set_device(0), worker.copy_kv(
                [BlockMapping.from_pairs(save)], Device.GPU, Device.Host, post_events=handle.post_events)))
            t.start()                                    # asks for its post tokens at once
            input_ids, params = step_cache.begin_step(reqs, True, False, record, blocks_to_copy=cow)
            with torch.cuda.stream(model_stream):
                x = input_ids
                for layer in layers:
                    layer.params = params
                    x = layer(x)
            t.join()
            worker.dtoh_stream.synchronize()
            model_stream.synchronize()
            # the same step on the oracles
            assert np.array_equal(input_ids.cpu().numpy(), ref["input_ids"])
            cache_oracle.copy_blocks(want, cow)
            ids = torch.from_numpy(ref["input_ids"]).to(DEV)
            for l, layer in enumerate(layers):
                k, v = layer.kv(ids)
                cache_oracle.append_paged_kv_cache(to_words(k), to_words(v), ref["batch_indices"],
                                                   ref["positions"], want[l], ref["kv_block_indices"],
                                                   ref["kv_block_indptrs"])
            cache_oracle.swap_out(want.reshape(L_, NB, -1), host_want, save)
            assert np.array_equal(to_words(kv), want), f"cache differs after step {step}"
            assert np.array_equal(worker.host_pool.array.view(np.uint16), host_want), f"host pool, step {step}"
        assert handle.kv_queue.empty()                   # every token was taken
    finally:
        worker.close()


@pytest.mark.parametrize("seed", [11, 12, 13, 14, 15, 16])
def test_random_step_sequences_match_the_oracles(seed):
    """Five steps in a row on one cache with a random mix per step (decode only, prefill only,
    both; with and without copy-on-write): the cached per-layer plans are reused whenever a
    step has the shape of an earlier one, and the cache must match the oracles after each."""
    L_, NB, BS, H, D = 4, 160, 16, 2, 32
    shape = W.KVShape("toy", L_, H, D, "bf16", NB, BS)
    rng = np.random.default_rng(seed)
    words = W.normal_words(rng, shape.cache_shape, "bf16")
    kv = to_tensor(words, "bf16", DEV)
    want = words.copy()
    step_cache = ModelStepCache(kv, max_batch=64, max_tokens=1024, max_blocks=2048)
    layers = [Attention(l, step_cache, H, D) for l in range(L_)]
    for step in range(5):
        kind = int(rng.integers(0, 3))
        n_dec = 0 if kind == 1 else int(rng.integers(1, 20))
        n_pre = 0 if kind == 0 else int(rng.integers(1, 4))
        reqs = W.make_step_requests(128, BS, n_dec, 1, 90, n_pre, int(rng.integers(2, 70)), 60,
                                    seed=seed * 100 + step)
        ref = step_oracle.make_inputs(copy.deepcopy(reqs), BS)
        cow = None
        if rng.integers(0, 2):
            src = rng.choice(ref["kv_block_indices"], size=2, replace=False)
            dst = 128 + rng.permutation(32)[:5]
            cow = {int(src[0]): [int(d) for d in dst[:3]], int(src[1]): [int(d) for d in dst[3:]]}
        input_ids, params = step_cache.begin_step(reqs, blocks_to_copy=cow)
        for layer in layers:
            layer.params = params
            layer(input_ids)
        torch.cuda.synchronize()
        assert np.array_equal(input_ids.cpu().numpy(), ref["input_ids"])
        if cow:
            cache_oracle.copy_blocks(want, cow)
        ids = torch.from_numpy(ref["input_ids"]).to(DEV)
        for l, layer in enumerate(layers):
            k, v = layer.kv(ids)
            cache_oracle.append_paged_kv_cache(to_words(k), to_words(v), ref["batch_indices"],
                                               ref["positions"], want[l], ref["kv_block_indices"],
                                               ref["kv_block_indptrs"])
        assert np.array_equal(to_words(kv), want), f"seed {seed}: cache differs after step {step}"


def test_model_step_cache_argument_errors():
    with pytest.raises(ValueError, match="kv_caches must be"):
        ModelStepCache(torch.zeros(2, 4, 16, 2, 8, device=DEV))
    with pytest.raises(RuntimeError, match="no CPU path"):
        ModelStepCache(torch.zeros(1, 4, 2, 16, 2, 8))
