"""The gRPC face of the KV worker: wire format against hand-encoded protobuf bytes (CPU), the
service over a Unix socket with a recording stand-in worker (CPU), and end to end with the real
worker on a GPU."""
import os
import tempfile

import grpc
import numpy as np
import pytest
import torch

from lmserve_b200 import kv_service as S
from lmserve_b200.kv_worker import Device, mappings_to_pairs


def test_wire_format_matches_worker_proto():
    # CopyKVRequest{block_mappings=[{entries=[{src=3,dst=300},{src=0,dst=7}]}], src=GPU, dst=Host}
    # BlockMapping.entries is field 2; BlockMappingEntry fields 1, 2 (varints); enum fields 2, 3.
    entry1 = bytes([0x08, 3, 0x10, 0xAC, 0x02])          # src=3, dst=300
    entry2 = bytes([0x10, 7])                            # src=0 omitted (proto3 default), dst=7
    mapping = bytes([0x12, len(entry1)]) + entry1 + bytes([0x12, len(entry2)]) + entry2
    wire = bytes([0x0A, len(mapping)]) + mapping + bytes([0x18, 1])   # dst_device=Host, src=GPU omitted
    req = S.CopyKVRequest.FromString(wire)
    assert [(e.src_block_id, e.dst_block_id) for e in req.block_mappings[0].entries] == [(3, 300), (0, 7)]
    assert req.src_device == Device.GPU and req.dst_device == Device.Host
    assert req.SerializeToString() == wire
    assert mappings_to_pairs(req.block_mappings).tolist() == [[3, 300], [0, 7]]
    # PushKVRequest: peer_name=1 (string), kv_descs=2 (bytes), block_ids=3 (packed uint32)
    p = S.PushKVRequest(peer_name="kv1", kv_descs=b"\x01\x02", block_ids=[5, 130])
    assert p.SerializeToString() == b"\x0a\x03kv1\x12\x02\x01\x02\x1a\x03\x05\x82\x01"
    assert S.GetDescriptorsRequest.FromString(b"\x0a\x02\x09\x0a").block_ids == [9, 10]
    assert S.PullKVRequest.DESCRIPTOR.fields_by_name["descs"].number == 2
    assert set(S.METHODS) == {"CopyKV", "GetLocalAgentMetadata", "AddRemoteAgentMetadata",
                              "GetDescriptors", "PushKV", "PullKV"}


class RecordingWorker:
    """Stands in for KVWorker: records calls, no GPU."""
    name = "kv-test"

    class _Stream:
        def synchronize(self):
            pass
    dtoh_stream = htod_stream = push_stream = _Stream()

    def __init__(self):
        self.calls = []

    def copy_kv(self, block_mappings, src, dst):
        if (src, dst) not in ((Device.GPU, Device.Host), (Device.Host, Device.GPU)):
            raise ValueError(f"Unsupported copy direction: {src} -> {dst}")
        self.calls.append(("copy_kv", mappings_to_pairs(block_mappings).tolist(), src, dst))

    def get_descriptors(self, block_ids):
        self.calls.append(("get_descriptors", list(block_ids)))
        return b"desc:" + bytes(block_ids)

    def push_kv(self, peer_name, descs, block_ids):
        self.calls.append(("push_kv", peer_name, bytes(descs), list(block_ids)))
        return len(block_ids) <= 3

    def pull_kv(self, peer_name, descs, block_ids):
        self.calls.append(("pull_kv", peer_name, bytes(descs), list(block_ids)))
        return bytes(descs) == b"good"


def test_service_over_unix_socket_with_recording_worker():
    worker = RecordingWorker()
    with tempfile.TemporaryDirectory() as d:
        addr = "unix://" + os.path.join(d, "kv.sock")
        server = S.serve(worker, addr)
        try:
            with grpc.insecure_channel(addr) as ch:
                stub = S.KVWorkerStub(ch)
                req = S.CopyKVRequest(src_device=Device.Host, dst_device=Device.GPU)
                m = req.block_mappings.add()
                m.entries.add(src_block_id=4, dst_block_id=9)
                m.entries.add(src_block_id=5, dst_block_id=1)
                req.block_mappings.add().entries.add(src_block_id=7, dst_block_id=2)
                assert stub.CopyKV(req).success is True
                bad = S.CopyKVRequest(src_device=Device.Host, dst_device=Device.Disk)
                with pytest.raises(grpc.RpcError) as e:
                    stub.CopyKV(bad)
                assert e.value.code() == grpc.StatusCode.INVALID_ARGUMENT
                assert "Unsupported copy direction" in e.value.details()
                assert stub.GetDescriptors(S.GetDescriptorsRequest(block_ids=[1, 2, 3])).descs == b"desc:\x01\x02\x03"
                assert stub.PushKV(S.PushKVRequest(peer_name="p", kv_descs=b"x", block_ids=[1, 2])).success is True
                assert stub.PushKV(S.PushKVRequest(peer_name="p", kv_descs=b"x", block_ids=[1, 2, 3, 4])).success is False
                assert stub.PullKV(S.PullKVRequest(peer_name="p")).success is False
                assert stub.PullKV(S.PullKVRequest(peer_name="p", descs=b"good", block_ids=[8])).success is True
                assert stub.GetLocalAgentMetadata(S.Empty()).agent_name == "kv-test"
                assert stub.AddRemoteAgentMetadata(S.AgentMetadata(agent_name="peer7")).peer_name == "peer7"
        finally:
            server.stop(0)
    assert worker.calls[0] == ("copy_kv", [[4, 9], [5, 1], [7, 2]], Device.Host, Device.GPU)
    assert worker.calls[1] == ("get_descriptors", [1, 2, 3])
    assert worker.calls[2] == ("push_kv", "p", b"x", [1, 2])


@pytest.mark.gpu
def test_service_end_to_end_on_gpu():
    """CopyKV GPU->Host then Host->GPU through the socket, with the real kernels."""
    from helpers import to_tensor, to_words
    import workloads as W
    from lmserve_b200.kv_worker import KVWorker
    from oracle import cache_oracle
    shape = W.SHAPES["llama31_8b_swap"].scaled(num_layers=3, num_blocks=32, num_kv_heads=2)
    words = W.normal_words(np.random.default_rng(5), shape.cache_shape, shape.dtype)
    gpu = to_tensor(words, shape.dtype, "cuda:0")
    worker = KVWorker("kv0", gpu, num_host_blocks=8)
    with tempfile.TemporaryDirectory() as d:
        addr = "unix://" + os.path.join(d, "kv.sock")
        server = S.serve(worker, addr)
        try:
            with grpc.insecure_channel(addr) as ch:
                stub = S.KVWorkerStub(ch)
                out = S.CopyKVRequest(src_device=Device.GPU, dst_device=Device.Host)
                m = out.block_mappings.add()
                for s_, d_ in ((3, 0), (17, 5), (30, 7)):
                    m.entries.add(src_block_id=s_, dst_block_id=d_)
                assert stub.CopyKV(out).success
                back = S.CopyKVRequest(src_device=Device.Host, dst_device=Device.GPU)
                m = back.block_mappings.add()
                for s_, d_ in ((5, 1), (0, 2), (7, 31)):
                    m.entries.add(src_block_id=s_, dst_block_id=d_)
                assert stub.CopyKV(back).success
                descs = stub.GetDescriptors(S.GetDescriptorsRequest(block_ids=[4, 6])).descs
                assert len(descs) > 64
        finally:
            server.stop(0)
    torch.cuda.synchronize()
    gw = words.reshape(3, 32, -1).copy()
    hw = np.zeros((8, 3, shape.chunk_bytes // 2), np.uint16)
    cache_oracle.swap_out(gw, hw, np.array([[3, 0], [17, 5], [30, 7]]))
    cache_oracle.swap_in(gw, hw, np.array([[5, 1], [0, 2], [7, 31]]))
    assert np.array_equal(to_words(gpu).reshape(gw.shape), gw)
    worker.close()
