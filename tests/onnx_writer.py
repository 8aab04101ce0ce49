"""A minimal ONNX file writer for the tests: encodes a denox_b200.nets.Net as ModelProto bytes (protobuf wire
format by hand, field numbers of onnx.proto), the way torch.onnx.export lays such a model out: Conv with
kernel_shape / pads / strides / dilations / group attributes and initializer weights, Relu, LeakyRelu(alpha),
MaxPool(kernel_shape, strides), Resize(mode nearest, asymmetric, scales from a Constant node), Concat(axis 1).
Neither the onnx package nor an exporter exists on the test machines."""
import struct

import numpy as np

from denox_b200 import nets


def _varint(v):
    v &= (1 << 64) - 1
    out = bytearray()
    while True:
        b = v & 0x7F
        v >>= 7
        if v:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def _tag(field, wire):
    return _varint((field << 3) | wire)


def f_varint(field, v):
    return _tag(field, 0) + _varint(v)


def f_bytes(field, b):
    return _tag(field, 2) + _varint(len(b)) + b


def f_str(field, s):
    return f_bytes(field, s.encode())


def f_float(field, v):
    return _tag(field, 5) + struct.pack("<f", v)


def tensor(name, arr, as_raw=True):
    """TensorProto: dims = 1, data_type = 2, raw_data = 9, float_data = 4 (packed), int32_data = 5, name = 8."""
    arr = np.asarray(arr)
    out = b"".join(f_varint(1, d) for d in arr.shape)
    if arr.dtype == np.float32:
        out += f_varint(2, 1)
        out += f_bytes(9, arr.tobytes()) if as_raw else f_bytes(4, arr.astype("<f4").tobytes())
    elif arr.dtype == np.float16:
        out += f_varint(2, 10)
        if as_raw:
            out += f_bytes(9, arr.tobytes())
        else:
            out += f_bytes(5, b"".join(_varint(int(x)) for x in arr.view(np.uint16).reshape(-1)))
    elif arr.dtype == np.int64:
        out += f_varint(2, 7) + f_bytes(9, arr.tobytes())
    else:
        raise ValueError(arr.dtype)
    return out + f_str(8, name)


def attr_int(name, v):
    return f_str(1, name) + f_varint(3, v) + f_varint(20, 2)


def attr_float(name, v):
    return f_str(1, name) + f_float(2, v) + f_varint(20, 1)


def attr_str(name, v):
    return f_str(1, name) + f_bytes(4, v.encode()) + f_varint(20, 3)


def attr_ints(name, vs):
    return f_str(1, name) + b"".join(f_varint(8, v) for v in vs) + f_varint(20, 7)


def attr_tensor(name, t):
    return f_str(1, name) + f_bytes(5, t) + f_varint(20, 4)


def node(op, inputs, outputs, attrs=(), name=""):
    out = b"".join(f_str(1, i) for i in inputs) + b"".join(f_str(2, o) for o in outputs)
    if name:
        out += f_str(3, name)
    out += f_str(4, op)
    return out + b"".join(f_bytes(5, a) for a in attrs)


def value_info(name, channels, elem_type=10):
    dims = [f_bytes(1, f_varint(1, 1)), f_bytes(1, f_varint(1, channels)), f_bytes(1, f_str(2, "H")), f_bytes(1, f_str(2, "W"))]
    shape = b"".join(dims)
    ttype = f_varint(1, elem_type) + f_bytes(2, shape)
    return f_str(1, name) + f_bytes(2, f_bytes(1, ttype))


def from_net(net, weights_dtype=np.float16, raw=True, opset=17, auto_pad=None):
    """ModelProto bytes of a nets.Net."""
    names = {net.input_tensor: "input"}
    nm = lambda t: names.setdefault(t, f"t{t}")
    nodes, inits = [], []
    for i, nd in enumerate(net.nodes):
        if nd.kind == nets.CONV:
            w = f"w{i}"
            inits.append(tensor(w, nd.weights.astype(weights_dtype), raw))
            ins = [nm(nd.in0), w]
            if nd.bias is not None:
                inits.append(tensor(f"b{i}", nd.bias.astype(weights_dtype), raw))
                ins.append(f"b{i}")
            attrs = [attr_ints("dilations", [1, 1]), attr_int("group", 1), attr_ints("kernel_shape", [3, 3]),
                     attr_ints("strides", [1, 1])]
            attrs.append(attr_str("auto_pad", auto_pad) if auto_pad else attr_ints("pads", [1, 1, 1, 1]))
            nodes.append(node("Conv", ins, [nm(nd.out)], attrs, nd.name))
        elif nd.kind == nets.RELU:
            nodes.append(node("Relu", [nm(nd.in0)], [nm(nd.out)], name=nd.name))
        elif nd.kind == nets.LEAKY_RELU:
            nodes.append(node("LeakyRelu", [nm(nd.in0)], [nm(nd.out)], [attr_float("alpha", nd.alpha)], nd.name))
        elif nd.kind == nets.MAXPOOL:
            nodes.append(node("MaxPool", [nm(nd.in0)], [nm(nd.out)],
                              [attr_int("ceil_mode", 0), attr_ints("kernel_shape", [2, 2]), attr_ints("pads", [0, 0, 0, 0]),
                               attr_ints("strides", [2, 2])], nd.name))
        elif nd.kind == nets.UPSAMPLE:
            sc = f"scales{i}"
            nodes.append(node("Constant", [], [sc], [attr_tensor("value", tensor("", np.array([1, 1, 2, 2], np.float32)))]))
            nodes.append(node("Resize", [nm(nd.in0), "", sc], [nm(nd.out)],
                              [attr_str("coordinate_transformation_mode", "asymmetric"), attr_str("mode", "nearest"),
                               attr_str("nearest_mode", "floor")], nd.name))
        elif nd.kind == nets.CONCAT:
            nodes.append(node("Concat", [nm(nd.in0), nm(nd.in1)], [nm(nd.out)], [attr_int("axis", 1)], nd.name))
    names[net.output_tensor] = names.get(net.output_tensor, "output")
    graph = b"".join(f_bytes(1, n) for n in nodes) + f_str(2, "main_graph") + b"".join(f_bytes(5, t) for t in inits)
    graph += f_bytes(11, value_info("input", net.in_channels))
    graph += f_bytes(12, value_info(nm(net.output_tensor), net.channels[net.output_tensor]))
    model = f_varint(1, 8) + f_str(2, "pytorch") + f_str(3, "2.11") + f_bytes(7, graph)
    model += f_bytes(8, f_str(1, "") + f_varint(2, opset))
    return model
