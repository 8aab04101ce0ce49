"""The ONNX subset import without a GPU: a model imported from ONNX bytes compiles to the same dnx file, byte for
byte, as the same network handed over as a node list; what the reference's importer refuses is refused here with
a reason."""
import ctypes as C

import numpy as np
import pytest

import onnx_writer as ow
from denox_b200 import lib, nets


def import_onnx(blob, options=0):
    h = C.c_void_p()
    st = lib.L.dnxcu_model_create_from_onnx(blob, len(blob), None, -1, options, C.byref(h))
    return st, h, lib.L.dnxcu_last_error_message().decode()


def dnx_of(handle):
    return lib._write_blob(lib.L.dnxcu_model_write_dnx, handle, "write")


@pytest.mark.parametrize("which", ["tiny", "tiny_bias", "tiny_leaky", "oidn", "oidn_reference"])
@pytest.mark.parametrize("raw", [True, False])
def test_import_equals_node_list(which, raw):
    net = {"tiny": nets.tiny_unet, "tiny_bias": lambda: nets.tiny_unet(bias=True), "tiny_leaky": lambda: nets.tiny_unet(leaky=0.1),
           "oidn": nets.oidn_unet, "oidn_reference": nets.oidn_unet_reference}[which]()
    st, h, msg = import_onnx(ow.from_net(net, raw=raw))
    assert st == 0, msg
    want = lib.Model(net, device=-1)
    assert dnx_of(h) == want.write_dnx()
    lib.L.dnxcu_model_destroy(h)
    want.close()


def test_fp32_weights_are_truncated_like_the_reference():
    net = nets.tiny_unet()
    # fp32 weights with bits below binary16 precision: the import must truncate (f16.cpp:6-20), not round
    for nd in net.nodes:
        if nd.kind == nets.CONV:
            w32 = nd.weights.astype(np.float32) * np.float32(1.0003)
            nd.weights32 = w32
    blob = ow.from_net(_With32(net), weights_dtype=np.float32)
    st, h, msg = import_onnx(blob)
    assert st == 0, msg
    for nd in net.nodes:
        if nd.kind == nets.CONV:
            bits = np.array([lib.L.dnxcu_f16_from_float(float(v)) for v in nd.weights32.reshape(-1)], dtype=np.uint16)
            nd.weights = bits.view(np.float16).reshape(nd.weights.shape)
    want = lib.Model(net, device=-1)
    assert dnx_of(h) == want.write_dnx()
    lib.L.dnxcu_model_destroy(h)
    want.close()


class _With32:
    """A view of a net whose conv nodes hand out their fp32 weights."""

    def __init__(self, net):
        self._net = net

    def __getattr__(self, k):
        if k == "nodes":
            out = []
            for nd in self._net.nodes:
                if nd.kind == nets.CONV:
                    c = nets.Node(nd.kind, nd.in0, nd.out, nd.in1, nd.c_out, nd.weights32, nd.bias, nd.name, nd.alpha)
                    out.append(c)
                else:
                    out.append(nd)
            return out
        return getattr(self._net, k)


def _single(op_node, extra_inits=(), channels=8, out_channels=8):
    graph = ow.f_bytes(1, op_node) + b"".join(ow.f_bytes(5, t) for t in extra_inits)
    graph += ow.f_bytes(11, ow.value_info("input", channels)) + ow.f_bytes(12, ow.value_info("output", out_channels))
    return ow.f_varint(1, 8) + ow.f_bytes(7, graph) + ow.f_bytes(8, ow.f_str(1, "") + ow.f_varint(2, 17))


W8 = np.zeros((8, 8, 3, 3), np.float16)


@pytest.mark.parametrize("name,blob,reason", [
    ("group", _single(ow.node("Conv", ["input", "w"], ["output"], [ow.attr_int("group", 2), ow.attr_ints("pads", [1, 1, 1, 1])]),
                      [ow.tensor("w", W8)]), "group"),
    ("dilation", _single(ow.node("Conv", ["input", "w"], ["output"], [ow.attr_ints("dilations", [2, 2]), ow.attr_ints("pads", [1, 1, 1, 1])]),
                         [ow.tensor("w", W8)]), "dilation"),
    ("valid_padding", _single(ow.node("Conv", ["input", "w"], ["output"], [ow.attr_ints("pads", [0, 0, 0, 0])]),
                              [ow.tensor("w", W8)]), "padding"),
    ("5x5", _single(ow.node("Conv", ["input", "w"], ["output"], [ow.attr_ints("pads", [2, 2, 2, 2])]),
                    [ow.tensor("w", np.zeros((8, 8, 5, 5), np.float16))]), "3x3"),
    ("pool_ceil", _single(ow.node("MaxPool", ["input"], ["output"], [ow.attr_int("ceil_mode", 1), ow.attr_ints("kernel_shape", [2, 2]),
                                                                       ow.attr_ints("strides", [2, 2])])), "ceil_mode"),
    ("pool_indices", _single(ow.node("MaxPool", ["input"], ["output", "idx"], [ow.attr_ints("kernel_shape", [2, 2]),
                                                                               ow.attr_ints("strides", [2, 2])])), "indices"),
    ("resize_linear", _single(ow.node("Resize", ["input", "", "s"], ["output"], [ow.attr_str("mode", "linear")]),
                              [ow.tensor("s", np.array([1, 1, 2, 2], np.float32))]), "nearest"),
    ("resize_x3", _single(ow.node("Resize", ["input", "", "s"], ["output"], [ow.attr_str("mode", "nearest"),
                                                                             ow.attr_str("coordinate_transformation_mode", "asymmetric")]),
                          [ow.tensor("s", np.array([1, 1, 3, 3], np.float32))]), "2x"),
    ("resize_half_pixel", _single(ow.node("Resize", ["input", "", "s"], ["output"], [ow.attr_str("mode", "nearest"),
                                                                                     ow.attr_str("coordinate_transformation_mode", "half_pixel")]),
                                  [ow.tensor("s", np.array([1, 1, 2, 2], np.float32))]), "asymmetric"),
    ("concat_axis", _single(ow.node("Concat", ["input", "input"], ["output"], [ow.attr_int("axis", 2)])), "channel axis"),
    ("concat_three", _single(ow.node("Concat", ["input", "input", "input"], ["output"], [ow.attr_int("axis", 1)])), "exactly 2"),
    ("unknown_op", _single(ow.node("Softmax", ["input"], ["output"])), "not supported"),
])
def test_importer_refuses_what_the_reference_refuses(name, blob, reason):
    st, h, msg = import_onnx(blob)
    assert st == lib.E_UNSUPPORTED, (name, st, msg)
    assert reason in msg, msg


def test_same_upper_padding_and_garbage():
    net = nets.tiny_unet()
    st, h, msg = import_onnx(ow.from_net(net, auto_pad="SAME_UPPER"))
    assert st == 0, msg
    lib.L.dnxcu_model_destroy(h)
    for junk in (b"", b"\xff" * 40, b"\x0a\x05abc"):
        st, h, msg = import_onnx(junk)
        assert st < 0
