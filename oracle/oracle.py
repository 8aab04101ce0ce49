"""ctypes front end of the CPU oracle (oracle.c) and a whole-network runner.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
CPU-baseline leg of the benchmark — never by the product path.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liboracle.so")

ACC_F32, ACC_F16, ACC_F16_FMA = 0, 1, 2


def build(force=False):
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "-B", "liboracle.so"])
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = C.CDLL(_SO)
        vp, i = C.c_void_p, C.c_int
        _lib.orc_conv3x3.restype = i
        _lib.orc_conv3x3.argtypes = [vp, i, i, vp, i, i, i, vp, vp, i, i, i, vp, vp, vp, vp, vp]
        _lib.orc_conv3x3_act.restype = i
        _lib.orc_conv3x3_act.argtypes = [vp, i, i, vp, i, i, i, vp, vp, i, i, C.c_float, i, vp, vp, vp, vp, vp]
        _lib.orc_leaky_relu.argtypes = [vp, C.c_int64, C.c_float, vp]
        _lib.orc_set_num_threads.argtypes = [i]
        _lib.orc_maxpool2x2.argtypes = [vp, i, i, i, vp]
        _lib.orc_upsample2x.argtypes = [vp, i, i, i, vp]
        _lib.orc_concat.argtypes = [vp, i, vp, i, i, i, vp]
        _lib.orc_relu.argtypes = [vp, C.c_int64, vp]
        _lib.orc_pad_edge.restype = i
        _lib.orc_pad_edge.argtypes = [vp, i, i, i, i, i, i, i, vp]
        _lib.orc_slice.restype = i
        _lib.orc_slice.argtypes = [vp, i, i, i, i, i, i, i, vp]
        _lib.orc_f32_to_f16_trunc.argtypes = [vp, vp, C.c_int64]
        _lib.orc_num_threads.restype = i
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data


def _f16(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float16)


def conv3x3(a, w_kcrs, bias=None, relu=False, mode=ACC_F32, b=None, up_a=False, halo=(None, None, None, None),
            leaky=None):
    """a: [H(/2)][W(/2)][Ca], b: [H][W][Cb] or None, w: [K][Ca+Cb][3][3]; returns [H][W][K] binary16.
    relu: max(0, x) on the finished sum; leaky=alpha: max(alpha * x, x) in binary16 instead."""
    a, b, w, bias = _f16(a), _f16(b), _f16(w_kcrs), _f16(bias)
    halo = [_f16(h) for h in halo]
    ca = a.shape[2]
    cb = 0 if b is None else b.shape[2]
    h, wd = (a.shape[0] * 2, a.shape[1] * 2) if up_a else a.shape[:2]
    if b is not None:
        assert b.shape[:2] == (h, wd)
    k = w.shape[0]
    assert w.shape == (k, ca + cb, 3, 3), (w.shape, ca, cb)
    out = np.empty((h, wd, k), dtype=np.float16)
    act = 2 if leaky is not None else (1 if relu else 0)
    st = lib().orc_conv3x3_act(_p(a), ca, int(up_a), _p(b), cb, h, wd, _p(w), _p(bias), k, act,
                               float(leaky or 0.0), mode, _p(out), *[_p(x) for x in halo])
    assert st == 0, st
    return out


def maxpool2x2(x):
    x = _f16(x)
    h, w, c = x.shape
    out = np.empty((h // 2, w // 2, c), dtype=np.float16)
    lib().orc_maxpool2x2(_p(x), h, w, c, _p(out))
    return out


def upsample2x(x):
    x = _f16(x)
    h, w, c = x.shape
    out = np.empty((h * 2, w * 2, c), dtype=np.float16)
    lib().orc_upsample2x(_p(x), h, w, c, _p(out))
    return out


def concat(a, b):
    a, b = _f16(a), _f16(b)
    h, w, ca = a.shape
    out = np.empty((h, w, ca + b.shape[2]), dtype=np.float16)
    lib().orc_concat(_p(a), ca, _p(b), b.shape[2], h, w, _p(out))
    return out


def relu(x):
    x = _f16(x)
    out = np.empty_like(x)
    lib().orc_relu(_p(x), x.size, _p(out))
    return out


def leaky_relu(x, alpha):
    x = _f16(x)
    out = np.empty_like(x)
    lib().orc_leaky_relu(_p(x), x.size, float(alpha), _p(out))
    return out


def pad_edge(x, left=0, right=0, top=0, bottom=0):
    """Edge replicating spatial pad (memory_pad.comp)."""
    x = _f16(x)
    h, w, c = x.shape
    out = np.empty((h + top + bottom, w + left + right, c), dtype=np.float16)
    assert lib().orc_pad_edge(_p(x), h, w, c, left, right, top, bottom, _p(out)) == 0
    return out


def slice_hw(x, left, top, oh, ow):
    """Spatial slice (memory_slice.comp)."""
    x = _f16(x)
    h, w, c = x.shape
    out = np.empty((oh, ow, c), dtype=np.float16)
    assert lib().orc_slice(_p(x), h, w, c, left, top, oh, ow, _p(out)) == 0
    return out


def run_network_aligned(net, x, alignment=16, mode=ACC_F32):
    """The network behind the reference's alignment wrapper (oidn_model.py:334-347): pad right and bottom
    to a multiple of `alignment` by edge replication, run, slice the output back.  Returns the output."""
    h, w = x.shape[:2]
    ph, pw = (-h) % alignment, (-w) % alignment
    y = run_network(net, pad_edge(x, 0, pw, 0, ph), mode)[net.output_tensor]
    return slice_hw(y, 0, 0, h, w)


def f32_to_f16_trunc(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().orc_f32_to_f16_trunc(_p(x), _p(out), x.size)
    return out


def num_threads():
    return lib().orc_num_threads()


def set_num_threads(n):
    """Threads of the oracle's parallel loops from now on (OMP_NUM_THREADS=1, which process launchers like to
    export, would otherwise make a timing of the oracle a one core figure)."""
    lib().orc_set_num_threads(int(n))


def run_network(net, x, mode=ACC_F32):
    """Runs a denox_b200.nets.Net node by node (un-fused, the reference's own
    dispatch granularity).  Returns {tensor id: array} for every tensor."""
    CONV, RELU, MAXPOOL, UPSAMPLE, CONCAT, LEAKY_RELU = 1, 2, 3, 4, 5, 6
    t = {net.input_tensor: _f16(x)}
    # the activation works on the rounded sum in binary16, so a conv followed by its activation gives the same
    # bits fused (ReLU on the accumulator, direct_conv.comp:559-590) or as two steps
    for nd in net.nodes:
        if nd.kind == CONV:
            t[nd.out] = conv3x3(t[nd.in0], nd.weights, nd.bias, relu=False, mode=mode)
        elif nd.kind == RELU:
            t[nd.out] = relu(t[nd.in0])
        elif nd.kind == LEAKY_RELU:
            t[nd.out] = leaky_relu(t[nd.in0], nd.alpha)
        elif nd.kind == MAXPOOL:
            t[nd.out] = maxpool2x2(t[nd.in0])
        elif nd.kind == UPSAMPLE:
            t[nd.out] = upsample2x(t[nd.in0])
        elif nd.kind == CONCAT:
            t[nd.out] = concat(t[nd.in0], t[nd.in1])
    return t
