"""The reference's gRPC contract for the engine sidecar, built at import time without ``protoc``.

The messages and the ``pegaflow.Engine`` service below are the wire contract of
``pegaflow-proto/proto/engine.proto`` (field numbers, types and names as published there, lines
22-279): a client or server generated from that file and one built on this module interoperate.
The schema is declared as plain tables and turned into protobuf descriptors with
``google.protobuf.descriptor_pb2``; message classes come from ``message_factory``.

Only the calls on the save/load path are served by :mod:`pegaflow_b200.server`; the cross-node
transfer calls (``QueryBlocksForTransfer``, ``ReleaseTransferLock``, ``RdmaHandshake``) are part
of the contract and are declared so that they can be answered with UNIMPLEMENTED.
"""
from __future__ import annotations

from google.protobuf import descriptor_pb2, descriptor_pool, message_factory

PACKAGE = "pegaflow"
SERVICE = "pegaflow.Engine"
# service.rs:119-130: a client must announce the version the server was built as
PROTOCOL_VERSION = "0.23.12"

_F = descriptor_pb2.FieldDescriptorProto
_SCALARS = {"bool": _F.TYPE_BOOL, "string": _F.TYPE_STRING, "bytes": _F.TYPE_BYTES, "uint32": _F.TYPE_UINT32,
            "uint64": _F.TYPE_UINT64, "int32": _F.TYPE_INT32}

ENUMS = {"TransferMode": [("TRANSFER_MODE_DIRECT", 0), ("TRANSFER_MODE_KERNEL", 1)]}

# message -> [(field name, number, type[, "repeated" | "oneof:<name>"])]
MESSAGES = {
    "ResponseStatus": [("ok", 1, "bool"), ("message", 2, "string")],
    "RegisterContextRequest": [
        ("instance_id", 1, "string"), ("namespace", 2, "string"), ("tp_rank", 3, "uint32"), ("tp_size", 4, "uint32"),
        ("world_size", 5, "uint32"), ("device_id", 6, "int32"), ("layer_names", 8, "string", "repeated"),
        ("wrapper_bytes", 9, "bytes", "repeated"), ("num_blocks", 10, "uint64", "repeated"),
        ("bytes_per_block", 11, "uint64", "repeated"), ("kv_stride_bytes", 12, "uint64", "repeated"),
        ("segments", 13, "uint32", "repeated"), ("pp_rank", 14, "uint32"), ("client_version", 15, "string"),
        ("transfer_mode", 17, "TransferMode"), ("page_first", 18, "bool"), ("layer_group_ids", 19, "uint32", "repeated")],
    "RegisterContextResponse": [("status", 1, "ResponseStatus")],
    "SaveLayer": [("layer_name", 1, "string"), ("block_ids", 2, "uint32", "repeated"), ("block_hashes", 3, "bytes", "repeated")],
    "SaveRequest": [("instance_id", 1, "string"), ("tp_rank", 2, "uint32"), ("device_id", 3, "int32"),
                    ("saves", 4, "SaveLayer", "repeated"), ("pp_rank", 5, "uint32")],
    "SaveResponse": [("status", 1, "ResponseStatus")],
    "LoadRequest": [("instance_id", 1, "string"), ("tp_rank", 2, "uint32"), ("device_id", 3, "int32"),
                    ("load_state_shm", 4, "string"), ("groups", 5, "LoadGroup", "repeated"), ("loads", 6, "LeaseLoad", "repeated")],
    "LoadGroup": [("layer_names", 1, "string", "repeated")],
    "LoadBlockIds": [("targets", 1, "LoadBlockTarget", "repeated")],
    "LoadBlockTarget": [("block_id", 1, "uint32", "oneof:target")],
    "LeaseLoad": [("lease", 1, "bytes"), ("block_ids_by_group", 2, "LoadBlockIds", "repeated")],
    "LoadResponse": [("status", 1, "ResponseStatus")],
    "QueryRequest": [("instance_id", 1, "string"), ("block_hashes", 2, "bytes", "repeated"), ("req_id", 3, "string"),
                     ("wait_for_full_prefix", 4, "bool"), ("group_id", 5, "uint32")],
    "QueryResponse": [("loading", 1, "QueryLoading", "oneof:outcome"), ("ready", 2, "QueryReady", "oneof:outcome")],
    "QueryLoading": [],
    "QueryReady": [("num_hit_blocks", 1, "uint64"), ("lease", 2, "bytes"), ("hit_positions", 3, "uint32", "repeated")],
    "ReleaseRequest": [("lease", 1, "bytes")],
    "ReleaseResponse": [],
    "UnregisterRequest": [("instance_id", 1, "string")],
    "UnregisterResponse": [("status", 1, "ResponseStatus")],
    "ShutdownRequest": [],
    "ShutdownResponse": [("status", 1, "ResponseStatus")],
    "HealthRequest": [],
    "HealthResponse": [("status", 1, "ResponseStatus")],
    "SessionRequest": [("instance_id", 1, "string"), ("namespace", 2, "string"), ("tp_size", 3, "uint32"),
                       ("world_size", 4, "uint32")],
    "SessionEvent": [],
    "TransferSlotInfo": [("k_ptr", 1, "uint64"), ("k_size", 2, "uint64"), ("v_ptr", 3, "uint64"), ("v_size", 4, "uint64"),
                         ("numa_node", 5, "uint32")],
    "TransferBlockInfo": [("block_hash", 1, "bytes"), ("slots", 2, "TransferSlotInfo", "repeated")],
    "QueryBlocksForTransferRequest": [("namespace", 1, "string"), ("block_hashes", 2, "bytes", "repeated"),
                                      ("requester_id", 3, "string")],
    "QueryBlocksForTransferResponse": [("status", 1, "ResponseStatus"), ("blocks", 2, "TransferBlockInfo", "repeated"),
                                       ("transfer_session_id", 3, "string"), ("lock_timeout_secs", 4, "uint32")],
    "RdmaHandshakeRequest": [("requester_id", 1, "string"), ("handshake_metadata", 2, "bytes")],
    "RdmaHandshakeResponse": [("status", 1, "ResponseStatus"), ("handshake_metadata", 2, "bytes")],
    "ReleaseTransferLockRequest": [("transfer_session_id", 1, "string")],
    "ReleaseTransferLockResponse": [("status", 1, "ResponseStatus"), ("released_blocks", 2, "uint64")],
}

# method -> (request, response, server streaming)
METHODS = {
    "RegisterContextBatch": ("RegisterContextRequest", "RegisterContextResponse", False),
    "Save": ("SaveRequest", "SaveResponse", False),
    "Load": ("LoadRequest", "LoadResponse", False),
    "QueryPrefetch": ("QueryRequest", "QueryResponse", False),
    "Release": ("ReleaseRequest", "ReleaseResponse", False),
    "UnregisterContext": ("UnregisterRequest", "UnregisterResponse", False),
    "QueryBlocksForTransfer": ("QueryBlocksForTransferRequest", "QueryBlocksForTransferResponse", False),
    "ReleaseTransferLock": ("ReleaseTransferLockRequest", "ReleaseTransferLockResponse", False),
    "RdmaHandshake": ("RdmaHandshakeRequest", "RdmaHandshakeResponse", False),
    "Shutdown": ("ShutdownRequest", "ShutdownResponse", False),
    "Health": ("HealthRequest", "HealthResponse", False),
    "Session": ("SessionRequest", "SessionEvent", True),
}


def _file_descriptor() -> descriptor_pb2.FileDescriptorProto:
    fd = descriptor_pb2.FileDescriptorProto(name="pegaflow_b200/engine.proto", package=PACKAGE, syntax="proto3")
    for name, values in ENUMS.items():
        e = fd.enum_type.add(name=name)
        for vname, number in values:
            e.value.add(name=vname, number=number)
    for name, fields in MESSAGES.items():
        m = fd.message_type.add(name=name)
        oneofs = {}
        for spec in fields:
            fname, number, ftype = spec[:3]
            extra = spec[3] if len(spec) > 3 else ""
            f = m.field.add(name=fname, number=number, json_name=fname)
            f.label = _F.LABEL_REPEATED if extra == "repeated" else _F.LABEL_OPTIONAL
            if ftype in _SCALARS:
                f.type = _SCALARS[ftype]
            elif ftype in ENUMS:
                f.type, f.type_name = _F.TYPE_ENUM, f".{PACKAGE}.{ftype}"
            else:
                f.type, f.type_name = _F.TYPE_MESSAGE, f".{PACKAGE}.{ftype}"
            if extra.startswith("oneof:"):
                group = extra[6:]
                if group not in oneofs:
                    oneofs[group] = len(m.oneof_decl)
                    m.oneof_decl.add(name=group)
                f.oneof_index = oneofs[group]
    svc = fd.service.add(name="Engine")
    for mname, (req, resp, streaming) in METHODS.items():
        svc.method.add(name=mname, input_type=f".{PACKAGE}.{req}", output_type=f".{PACKAGE}.{resp}",
                       server_streaming=streaming)
    return fd


_POOL = descriptor_pool.DescriptorPool()
_POOL.Add(_file_descriptor())


def message_class(name: str):
    return message_factory.GetMessageClass(_POOL.FindMessageTypeByName(f"{PACKAGE}.{name}"))


class _Messages:
    def __getattr__(self, name):
        if name not in MESSAGES:
            raise AttributeError(name)
        cls = message_class(name)
        setattr(self, name, cls)
        return cls


pb = _Messages()
TRANSFER_MODE = {"direct": 0, "kernel": 1}
TRANSFER_MODE_NAME = {0: "direct", 1: "kernel"}


def method_path(method: str) -> str:
    return f"/{SERVICE}/{method}"
