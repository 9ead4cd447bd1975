"""GraphDef / NodeDef / AttrValue message classes for the graph-optimizer
tests, declared at run time with the protobuf library (field numbers and types
as published in TensorFlow's graph.proto, node_def.proto, attr_value.proto,
versions.proto, tensor_shape.proto).  They let the tests build and read real
protobuf wire bytes, which is what the C++ optimizer consumes, and check its
hand-written wire codec against the protobuf implementation."""
from google.protobuf import descriptor_pb2, descriptor_pool, message_factory

_F = descriptor_pb2.FieldDescriptorProto

DT_FLOAT, DT_DOUBLE, DT_INT32, DT_INT64, DT_BFLOAT16, DT_HALF = 1, 2, 3, 9, 14, 19


def _field(msg, name, number, ftype, label=_F.LABEL_OPTIONAL, type_name=None, oneof=None):
    f = msg.field.add()
    f.name, f.number, f.type, f.label = name, number, ftype, label
    if type_name:
        f.type_name = type_name
    if oneof is not None:
        f.oneof_index = oneof
    return f


def _build():
    fd = descriptor_pb2.FileDescriptorProto()
    fd.name = "musa_test_graph.proto"
    fd.package = "musatest"
    fd.syntax = "proto3"

    dim = fd.message_type.add()
    dim.name = "Dim"
    _field(dim, "size", 1, _F.TYPE_INT64)
    _field(dim, "name", 2, _F.TYPE_STRING)

    shape = fd.message_type.add()
    shape.name = "TensorShapeProto"
    _field(shape, "dim", 2, _F.TYPE_MESSAGE, _F.LABEL_REPEATED, ".musatest.Dim")
    _field(shape, "unknown_rank", 3, _F.TYPE_BOOL)

    lst = fd.message_type.add()
    lst.name = "ListValue"
    _field(lst, "s", 2, _F.TYPE_BYTES, _F.LABEL_REPEATED)
    _field(lst, "i", 3, _F.TYPE_INT64, _F.LABEL_REPEATED)
    _field(lst, "type", 6, _F.TYPE_INT32, _F.LABEL_REPEATED)

    attr = fd.message_type.add()
    attr.name = "AttrValue"
    attr.oneof_decl.add().name = "value"
    _field(attr, "list", 1, _F.TYPE_MESSAGE, type_name=".musatest.ListValue", oneof=0)
    _field(attr, "s", 2, _F.TYPE_BYTES, oneof=0)
    _field(attr, "i", 3, _F.TYPE_INT64, oneof=0)
    _field(attr, "f", 4, _F.TYPE_FLOAT, oneof=0)
    _field(attr, "b", 5, _F.TYPE_BOOL, oneof=0)
    _field(attr, "type", 6, _F.TYPE_INT32, oneof=0)
    _field(attr, "shape", 7, _F.TYPE_MESSAGE, type_name=".musatest.TensorShapeProto", oneof=0)
    _field(attr, "placeholder", 9, _F.TYPE_STRING, oneof=0)

    node = fd.message_type.add()
    node.name = "NodeDef"
    entry = node.nested_type.add()
    entry.name = "AttrEntry"
    entry.options.map_entry = True
    _field(entry, "key", 1, _F.TYPE_STRING)
    _field(entry, "value", 2, _F.TYPE_MESSAGE, type_name=".musatest.AttrValue")
    _field(node, "name", 1, _F.TYPE_STRING)
    _field(node, "op", 2, _F.TYPE_STRING)
    _field(node, "input", 3, _F.TYPE_STRING, _F.LABEL_REPEATED)
    _field(node, "device", 4, _F.TYPE_STRING)
    _field(node, "attr", 5, _F.TYPE_MESSAGE, _F.LABEL_REPEATED, ".musatest.NodeDef.AttrEntry")

    ver = fd.message_type.add()
    ver.name = "VersionDef"
    _field(ver, "producer", 1, _F.TYPE_INT32)
    _field(ver, "min_consumer", 2, _F.TYPE_INT32)
    _field(ver, "bad_consumers", 3, _F.TYPE_INT32, _F.LABEL_REPEATED)

    graph = fd.message_type.add()
    graph.name = "GraphDef"
    _field(graph, "node", 1, _F.TYPE_MESSAGE, _F.LABEL_REPEATED, ".musatest.NodeDef")
    _field(graph, "version", 3, _F.TYPE_INT32)
    _field(graph, "versions", 4, _F.TYPE_MESSAGE, type_name=".musatest.VersionDef")

    pool = descriptor_pool.DescriptorPool()
    pool.Add(fd)
    get = getattr(message_factory, "GetMessageClass", None)
    if get is None:  # older protobuf
        factory = message_factory.MessageFactory(pool)
        return {n: factory.GetPrototype(pool.FindMessageTypeByName("musatest." + n))
                for n in ("GraphDef", "NodeDef", "AttrValue")}
    return {n: get(pool.FindMessageTypeByName("musatest." + n))
            for n in ("GraphDef", "NodeDef", "AttrValue")}


_CLS = _build()
GraphDef, NodeDef, AttrValue = _CLS["GraphDef"], _CLS["NodeDef"], _CLS["AttrValue"]

MUSA = "/job:localhost/replica:0/task:0/device:MUSA:0"
CPU = "/job:localhost/replica:0/task:0/device:CPU:0"


class Builder:
    """Small GraphDef builder: g.node(name, op, inputs, device, T=..., ...)."""

    def __init__(self):
        self.graph = GraphDef()
        self.graph.versions.producer = 808
        self.graph.versions.min_consumer = 12

    def node(self, name, op, inputs=(), device=MUSA, **attrs):
        n = self.graph.node.add()
        n.name, n.op, n.device = name, op, device
        n.input.extend(inputs)
        for key, val in attrs.items():
            a = n.attr[key]
            if key in ("T", "SrcT", "DstT", "dtype"):
                a.type = val
            elif isinstance(val, bool):
                a.b = val
            elif isinstance(val, int):
                a.i = val
            elif isinstance(val, float):
                a.f = val
            elif isinstance(val, (bytes, str)):
                a.s = val.encode() if isinstance(val, str) else val
            elif isinstance(val, (list, tuple)):
                for d in val:
                    a.shape.dim.add().size = d
            else:
                raise TypeError(key)
        return n

    def bytes(self):
        return self.graph.SerializeToString()


def parse(data):
    g = GraphDef()
    g.ParseFromString(data)
    return g


def by_name(graph):
    return {n.name: n for n in graph.node}
