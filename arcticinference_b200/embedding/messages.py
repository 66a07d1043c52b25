"""Protobuf message classes of the embedding service, built at import time.

The reference generates these with protoc while the package is built
(arctic_inference/embedding/generate_proto.py:1-79). Here a table of (name, number, type,
repeated) rows is turned into a ``FileDescriptorProto`` and handed to the protobuf runtime,
so there is no generated code to keep in sync and no compiler to install. The schema is the
one in ``proto/inference.proto``.
"""

from __future__ import annotations

from google.protobuf import descriptor_pb2, descriptor_pool, message_factory

PACKAGE = "arctic_inference"
SERVICE = "InferenceService"

_T = descriptor_pb2.FieldDescriptorProto
_SCALARS = {"string": _T.TYPE_STRING, "int32": _T.TYPE_INT32, "bytes": _T.TYPE_BYTES,
            "bool": _T.TYPE_BOOL}

# message -> [(field, number, type, repeated)]
SCHEMA = {
    "EncodeRequest": [("request_id", 1, "string", False), ("n_prompts", 2, "int32", False),
                      ("prompts", 3, "string", True), ("token_id_bytes_i32", 4, "bytes", True),
                      ("model_name", 5, "string", False), ("priority", 6, "int32", False)],
    "EncodeResponse": [("request_id", 1, "string", False), ("n_prompts", 2, "int32", False),
                       ("embedding_dim", 3, "int32", False),
                       ("embedding_bytes_fp32", 4, "bytes", True), ("error", 5, "string", False)],
    "AbortRequest": [("request_id", 1, "string", False)],
    "AbortResponse": [("success", 1, "bool", False), ("message", 2, "string", False)],
    "ReplicaInfoRequest": [],
    "SingleReplicaInfoResponse": [("model_name", 1, "string", False), ("task", 2, "string", False),
                                  ("dtype", 3, "string", False), ("ready", 4, "bool", False),
                                  ("parallel_config", 5, "string", False),
                                  ("decoding_config", 6, "string", False),
                                  ("scheduler_config", 7, "string", False),
                                  ("lora_config", 8, "string", False)],
    "ReplicaInfoResponse": [("replica_infos", 1, "SingleReplicaInfoResponse", True),
                            ("n_replicas", 2, "int32", False),
                            ("n_healthy_replicas", 3, "int32", False),
                            ("message", 4, "string", False)],
    "HealthCheckRequest": [],
    "HealthCheckResponse": [("healthy", 1, "bool", False), ("message", 2, "string", False)],
}

# rpc -> (request message, response message)
METHODS = {
    "Encode": ("EncodeRequest", "EncodeResponse"),
    "Abort": ("AbortRequest", "AbortResponse"),
    "GetReplicaInfo": ("ReplicaInfoRequest", "ReplicaInfoResponse"),
    "HealthCheck": ("HealthCheckRequest", "HealthCheckResponse"),
}


def _build():
    fd = descriptor_pb2.FileDescriptorProto()
    fd.name = "arcticinference_b200/embedding/inference.proto"
    fd.package = PACKAGE
    fd.syntax = "proto3"
    for msg, fields in SCHEMA.items():
        m = fd.message_type.add()
        m.name = msg
        for name, number, typ, repeated in fields:
            f = m.field.add()
            f.name, f.number = name, number
            f.label = _T.LABEL_REPEATED if repeated else _T.LABEL_OPTIONAL
            if typ in _SCALARS:
                f.type = _SCALARS[typ]
            else:
                f.type = _T.TYPE_MESSAGE
                f.type_name = ".%s.%s" % (PACKAGE, typ)
    svc = fd.service.add()
    svc.name = SERVICE
    for rpc, (req, resp) in METHODS.items():
        m = svc.method.add()
        m.name = rpc
        m.input_type = ".%s.%s" % (PACKAGE, req)
        m.output_type = ".%s.%s" % (PACKAGE, resp)
    pool = descriptor_pool.DescriptorPool()
    pool.Add(fd)
    return {name: message_factory.GetMessageClass(pool.FindMessageTypeByName(
        "%s.%s" % (PACKAGE, name))) for name in SCHEMA}


_CLASSES = _build()
globals().update(_CLASSES)
__all__ = list(_CLASSES) + ["METHODS", "SERVICE", "PACKAGE", "method_path"]


def method_path(rpc: str) -> str:
    return "/%s.%s/%s" % (PACKAGE, SERVICE, rpc)


def request_class(rpc: str):
    return _CLASSES[METHODS[rpc][0]]


def response_class(rpc: str):
    return _CLASSES[METHODS[rpc][1]]
