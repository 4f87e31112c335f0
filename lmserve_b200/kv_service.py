"""gRPC face of the KV worker: a servicer that is wire-compatible with LMServe's ``KVWorker``
service (``proto/worker.proto:19-27,78-117``) and backed by :class:`lmserve_b200.kv_worker.KVWorker`,
so the Rust ``KVWorkerGroup`` (``runtime/src/llm_engine/worker.rs:420-548``) can drive the B200
kernels over the same Unix socket and messages it uses today.  One thing changes on the engine
side: ``GetDescriptors`` / ``PushKV`` / ``PullKV`` carry **GPU** block ids, because blocks move
cache to cache; the reference's engine reserves and pins *host* blocks for a transfer
(``engine.rs:272-280,425-430``) and has to reserve GPU blocks instead.  The worker range-checks
every id against the two caches and answers ``success=False`` for ids that do not fit.

The reference generates its message classes with ``protoc`` (``llm_worker/pb/``, git-ignored).
``protoc`` is not required here: the handful of messages the KV service uses are declared below
as a ``FileDescriptorProto`` built in code, with the field names, numbers and types of
``worker.proto``, and the method handlers are registered through gRPC's generic-handler API.

Mirrors ``KVWorkerService`` of ``runtime/worker/llm_worker/cli.py:145-229``:
``CopyKV`` always answers ``success=True`` after the copy was enqueued and the copy stream
synchronised; ``GetDescriptors`` returns the serialized GPU-direct descriptor; ``PushKV`` returns
the boolean of ``KVWorker.push_kv``.  ``GetLocalAgentMetadata`` / ``AddRemoteAgentMetadata``
exist for the NIXL handshake of the reference; with CUDA-IPC descriptors there is no agent to
register, so they echo the worker's name.  ``PullKV`` reads the message's ``descs`` field (the
reference's handler reads a field the message does not have, ``cli.py:219-221``, and the Rust
side never calls it, ``worker.rs:521``) and runs ``KVWorker.pull_kv``.
"""
from __future__ import annotations

from concurrent import futures
import grpc
from google.protobuf import descriptor_pb2, descriptor_pool, empty_pb2, message_factory

from .kv_worker import Device, KVWorker

_T = descriptor_pb2.FieldDescriptorProto
SERVICE_NAME = "worker.KVWorker"


def _build_messages():
    fd = descriptor_pb2.FileDescriptorProto()
    fd.name = "lmserve_b200/kv_worker_service.proto"
    fd.package = "worker"
    fd.syntax = "proto3"

    enum = fd.enum_type.add()
    enum.name = "Device"
    for name, number in (("GPU", 0), ("Host", 1), ("Disk", 2)):
        v = enum.value.add()
        v.name, v.number = name, number

    def message(name, *fields):
        m = fd.message_type.add()
        m.name = name
        for fname, number, ftype, label, type_name in fields:
            f = m.field.add()
            f.name, f.number, f.type, f.label = fname, number, ftype, label
            if type_name:
                f.type_name = type_name

    opt, rep = _T.LABEL_OPTIONAL, _T.LABEL_REPEATED
    message("BlockMappingEntry",
            ("src_block_id", 1, _T.TYPE_UINT32, opt, None),
            ("dst_block_id", 2, _T.TYPE_UINT32, opt, None))
    message("BlockMapping",
            ("entries", 2, _T.TYPE_MESSAGE, rep, ".worker.BlockMappingEntry"))
    message("CopyKVRequest",
            ("block_mappings", 1, _T.TYPE_MESSAGE, rep, ".worker.BlockMapping"),
            ("src_device", 2, _T.TYPE_ENUM, opt, ".worker.Device"),
            ("dst_device", 3, _T.TYPE_ENUM, opt, ".worker.Device"))
    message("CopyKVResponse", ("success", 1, _T.TYPE_BOOL, opt, None))
    message("AgentMetadata",
            ("agent_name", 1, _T.TYPE_STRING, opt, None),
            ("data", 2, _T.TYPE_BYTES, opt, None))
    message("AddRemoteAgentMetadataResponse", ("peer_name", 1, _T.TYPE_STRING, opt, None))
    message("GetDescriptorsRequest", ("block_ids", 1, _T.TYPE_UINT32, rep, None))
    message("GetDescriptorsResponse", ("descs", 1, _T.TYPE_BYTES, opt, None))
    message("PushKVRequest",
            ("peer_name", 1, _T.TYPE_STRING, opt, None),
            ("kv_descs", 2, _T.TYPE_BYTES, opt, None),
            ("block_ids", 3, _T.TYPE_UINT32, rep, None))
    message("PushKVResponse", ("success", 1, _T.TYPE_BOOL, opt, None))
    message("PullKVRequest",
            ("peer_name", 1, _T.TYPE_STRING, opt, None),
            ("descs", 2, _T.TYPE_BYTES, opt, None),
            ("block_ids", 3, _T.TYPE_UINT32, rep, None))
    message("PullKVResponse", ("success", 1, _T.TYPE_BOOL, opt, None))

    pool = descriptor_pool.DescriptorPool()
    pool.Add(fd)
    return {m.name: message_factory.GetMessageClass(pool.FindMessageTypeByName("worker." + m.name))
            for m in fd.message_type}


_MSG = _build_messages()
BlockMappingEntry = _MSG["BlockMappingEntry"]
BlockMapping = _MSG["BlockMapping"]
CopyKVRequest = _MSG["CopyKVRequest"]
CopyKVResponse = _MSG["CopyKVResponse"]
AgentMetadata = _MSG["AgentMetadata"]
AddRemoteAgentMetadataResponse = _MSG["AddRemoteAgentMetadataResponse"]
GetDescriptorsRequest = _MSG["GetDescriptorsRequest"]
GetDescriptorsResponse = _MSG["GetDescriptorsResponse"]
PushKVRequest = _MSG["PushKVRequest"]
PushKVResponse = _MSG["PushKVResponse"]
PullKVRequest = _MSG["PullKVRequest"]
PullKVResponse = _MSG["PullKVResponse"]
Empty = empty_pb2.Empty

# method -> (request class, response class), as in proto/worker.proto:19-27
METHODS = {
    "CopyKV": (CopyKVRequest, CopyKVResponse),
    "GetLocalAgentMetadata": (Empty, AgentMetadata),
    "AddRemoteAgentMetadata": (AgentMetadata, AddRemoteAgentMetadataResponse),
    "GetDescriptors": (GetDescriptorsRequest, GetDescriptorsResponse),
    "PushKV": (PushKVRequest, PushKVResponse),
    "PullKV": (PullKVRequest, PullKVResponse),
}


class KVWorkerService:
    """Servicer methods with the names and message types of ``KVWorkerService``
    (``cli.py:145-229``), synchronous: every call returns once its device work is complete, which
    is what the reference's ``await ... stream.synchronize`` amounts to for the caller."""

    def __init__(self, worker: KVWorker):
        self.worker = worker

    def CopyKV(self, request, context):
        src, dst = Device(request.src_device), Device(request.dst_device)
        try:
            self.worker.copy_kv(request.block_mappings, src, dst)
        except ValueError as e:
            context.abort(grpc.StatusCode.INVALID_ARGUMENT, str(e))
        stream = self.worker.dtoh_stream if src == Device.GPU else self.worker.htod_stream
        stream.synchronize()
        return CopyKVResponse(success=True)

    def GetLocalAgentMetadata(self, request, context):
        return AgentMetadata(agent_name=self.worker.name, data=b"")

    def AddRemoteAgentMetadata(self, request, context):
        return AddRemoteAgentMetadataResponse(peer_name=request.agent_name)

    def GetDescriptors(self, request, context):
        try:
            return GetDescriptorsResponse(descs=self.worker.get_descriptors(list(request.block_ids)))
        except IndexError as e:
            context.abort(grpc.StatusCode.INVALID_ARGUMENT, str(e))

    def PushKV(self, request, context):
        ok = self.worker.push_kv(request.peer_name, request.kv_descs, list(request.block_ids))
        if ok:
            self.worker.push_stream.synchronize()
        return PushKVResponse(success=bool(ok))

    def PullKV(self, request, context):
        ok = self.worker.pull_kv(request.peer_name, request.descs, list(request.block_ids))
        if ok:
            self.worker.push_stream.synchronize()
        return PullKVResponse(success=bool(ok))


def add_kv_worker_servicer(servicer, server: grpc.Server) -> None:
    """Registers `servicer` under the service name ``worker.KVWorker`` (the generic-handler
    equivalent of the generated ``add_KVWorkerServicer_to_server``)."""
    handlers = {
        name: grpc.unary_unary_rpc_method_handler(
            getattr(servicer, name),
            request_deserializer=req.FromString,
            response_serializer=resp.SerializeToString)
        for name, (req, resp) in METHODS.items()
    }
    server.add_generic_rpc_handlers((grpc.method_handlers_generic_handler(SERVICE_NAME, handlers),))


def serve(worker: KVWorker, address: str, max_workers: int = 4) -> grpc.Server:
    """Starts a server for `worker` on `address` and returns it; stop it with
    ``server.stop(grace)``.  Use a Unix socket (``unix:///path``), as LMServe does between its
    Rust runtime and its workers: the port is unauthenticated and a caller can move KV blocks of
    any sequence.  ``host:port`` is accepted for tests and for deployments that fence the port
    themselves; every id and descriptor that arrives is still range-checked by the worker."""
    server = grpc.server(futures.ThreadPoolExecutor(max_workers=max_workers))
    add_kv_worker_servicer(KVWorkerService(worker), server)
    if server.add_insecure_port(address) == 0 and not address.startswith("unix:"):
        raise RuntimeError(f"could not bind {address}")
    server.start()
    return server


class KVWorkerStub:
    """Client side of the same six methods (what the Rust ``WorkerImpl`` does over tonic);
    used by the tests and handy for driving a worker from Python."""

    def __init__(self, channel: grpc.Channel):
        for name, (req, resp) in METHODS.items():
            setattr(self, name, channel.unary_unary(
                f"/{SERVICE_NAME}/{name}",
                request_serializer=req.SerializeToString,
                response_deserializer=resp.FromString))
