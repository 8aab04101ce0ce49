"""ctypes bindings of libdnxcu.so and a small object layer over them.

Names mirror the reference's runtime objects: `Model` / `Instance`
(runtime/src/denox/runtime/model.hpp:107-168, instance.hpp:44-81), `Db`
(database/src/denox/db/Db.hpp:15-76).  There is no fallback: a missing library
is an ImportError, a failing call raises DnxcuError.
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libdnxcu.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python -m denox_b200.build` "
        "(there is no CPU or PyTorch fallback for this backend)")

L = C.CDLL(LIB_PATH)

OK = 0
E_BAD_ARG, E_UNSUPPORTED, E_MISALIGNED, E_CUDA, E_DEVICE, E_NO_MEMORY, E_STATE, E_IO, E_LIMIT = range(-1, -10, -1)

OP_CONV3X3, OP_MAXPOOL2X2, OP_UPSAMPLE2X, OP_CONCAT, OP_RELU, OP_PAD_CHANNELS, OP_PAD_EDGE, OP_SLICE = 1, 2, 3, 4, 5, 6, 7, 8
F_RELU, F_BIAS, F_UP2X_A, F_POOL_OUT, F_NO_FULL_OUT, F_LEAKY = 0x01, 0x02, 0x04, 0x08, 0x10, 0x20
OPT_NO_FUSE_ACTIVATION, OPT_NO_FUSE_POOL, OPT_NO_FUSE_UPSAMPLE, OPT_NO_FUSE_CONCAT, OPT_NO_TCGEN05 = 1, 2, 4, 8, 16
OPT_NO_PAD_INPUT = 32
OPT_SELECT_BY_COST_ONLY = 64


class DnxcuError(RuntimeError):
    def __init__(self, status, what=""):
        self.status = status
        msg = L.dnxcu_status_string(status).decode()
        if status == E_CUDA:
            msg += f" (cudaError {L.dnxcu_last_cuda_error()})"
        super().__init__(f"{what}: {msg} [{status}]" if what else f"{msg} [{status}]")


def check(status, what=""):
    if status < 0:
        raise DnxcuError(status, what)
    return status


class Caps(C.Structure):
    _fields_ = [("device", C.c_int32), ("cc_major", C.c_int32), ("cc_minor", C.c_int32), ("sm_count", C.c_int32),
                ("max_threads_per_block", C.c_int32), ("tmem_columns", C.c_int32), ("tcgen05", C.c_int32),
                ("reserved", C.c_int32), ("smem_per_block_optin", C.c_uint64), ("l2_bytes", C.c_uint64),
                ("global_bytes", C.c_uint64), ("name", C.c_char * 64)]


class VariantDesc(C.Structure):
    _fields_ = [("id", C.c_int32), ("op", C.c_int32), ("family", C.c_char_p), ("config", C.c_char_p),
                ("allowed_flags", C.c_uint32), ("needs_tcgen05", C.c_int32), ("c_align", C.c_int32),
                ("k_align", C.c_int32), ("max_c_out", C.c_int32), ("reserved", C.c_int32)]


class Dispatch(C.Structure):
    _fields_ = [("variant", C.c_int32), ("flags", C.c_uint32), ("pc", C.c_uint32 * 2), ("c_a", C.c_int32),
                ("c_b", C.c_int32), ("c_out", C.c_int32), ("leaky_alpha", C.c_float), ("in_a", C.c_void_p),
                ("in_b", C.c_void_p), ("out", C.c_void_p), ("out_pool", C.c_void_p), ("weights", C.c_void_p),
                ("bias", C.c_void_p), ("halo", C.c_void_p * 4), ("device_status", C.c_void_p),
                ("pc_ext", C.c_uint32 * 4)]


class NodeC(C.Structure):
    _fields_ = [("kind", C.c_int32), ("in0", C.c_int32), ("in1", C.c_int32), ("out", C.c_int32),
                ("c_out", C.c_int32), ("alpha", C.c_float), ("weights_kcrs", C.c_void_p), ("bias", C.c_void_p)]


class ModelDesc(C.Structure):
    _fields_ = [("n_nodes", C.c_int32), ("n_tensors", C.c_int32), ("nodes", C.POINTER(NodeC)),
                ("input_tensor", C.c_int32), ("input_channels", C.c_int32), ("output_tensor", C.c_int32),
                ("options", C.c_uint32)]


class Band(C.Structure):
    _fields_ = [("image_h", C.c_int32), ("row0", C.c_int32), ("rows", C.c_int32)]


class DispatchInfo(C.Structure):
    _fields_ = [("name", C.c_char * 48), ("variant", C.c_int32), ("src_node", C.c_int32), ("grid", C.c_uint32 * 3),
                ("flags", C.c_uint32), ("bytes_read", C.c_uint64), ("bytes_written", C.c_uint64),
                ("flops", C.c_uint64), ("ms", C.c_float), ("h", C.c_int32), ("w", C.c_int32), ("c_a", C.c_int32),
                ("c_b", C.c_int32), ("c_out", C.c_int32), ("out_tensor", C.c_int32)]


class PeerHandle(C.Structure):
    _fields_ = [("ipc", C.c_ubyte * 64), ("arena_bytes", C.c_uint64), ("layout", C.c_uint64),
                ("local_ptr", C.c_uint64), ("pid", C.c_int64), ("device", C.c_int32), ("row0", C.c_int32),
                ("rows", C.c_int32), ("reserved", C.c_int32)]


class HaloPoint(C.Structure):
    _fields_ = [("before_dispatch", C.c_int32), ("tensor", C.c_int32), ("send_top", C.c_void_p),
                ("send_bottom", C.c_void_p), ("recv_top", C.c_void_p), ("recv_bottom", C.c_void_p),
                ("row_bytes", C.c_uint64)]


# every symbol include/dnxcu.h declares, with its C signature
SIGNATURES = {
    "dnxcu_status_string": (C.c_char_p, [C.c_int]),
    "dnxcu_last_cuda_error": (C.c_int, []),
    "dnxcu_get_device_caps": (C.c_int, [C.c_int, C.POINTER(Caps)]),
    "dnxcu_variant_count": (C.c_int, []),
    "dnxcu_variant": (C.POINTER(VariantDesc), [C.c_int]),
    "dnxcu_find_variant": (C.c_int, [C.c_char_p, C.c_char_p]),
    "dnxcu_variant_sha256": (C.c_int, [C.c_int, C.c_char_p]),
    "dnxcu_validate": (C.c_int, [C.POINTER(Dispatch)]),
    "dnxcu_launch": (C.c_int, [C.POINTER(Dispatch), C.c_void_p]),
    "dnxcu_plan_create": (C.c_int, [C.POINTER(Dispatch), C.POINTER(C.c_void_p)]),
    "dnxcu_plan_launch": (C.c_int, [C.c_void_p, C.c_void_p]),
    "dnxcu_plan_destroy": (None, [C.c_void_p]),
    "dnxcu_set_wait_limit_us": (C.c_int, [C.c_uint32]),
    "dnxcu_grid": (C.c_int, [C.POINTER(Dispatch), C.POINTER(C.c_uint32 * 3)]),
    "dnxcu_cost": (C.c_int, [C.POINTER(Dispatch), C.POINTER(C.c_uint64), C.POINTER(C.c_uint64),
                             C.POINTER(C.c_uint64)]),
    "dnxcu_prepare_weights": (C.c_int, [C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                        C.POINTER(C.c_size_t)]),
    "dnxcu_conv3x3_pool_static": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_int,
                                            C.c_uint32, C.c_void_p, C.c_void_p]),
    "dnxcu_f16_from_float": (C.c_uint16, [C.c_float]),
    "dnxcu_f16_to_float": (C.c_float, [C.c_uint16]),
    "dnxcu_model_create": (C.c_int, [C.POINTER(ModelDesc), C.c_void_p, C.c_int, C.POINTER(C.c_void_p)]),
    "dnxcu_model_destroy": (None, [C.c_void_p]),
    "dnxcu_model_write_dnx": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_size_t)]),
    "dnxcu_instance_write_dnx": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_size_t)]),
    "dnxcu_model_create_from_dnx": (C.c_int, [C.c_void_p, C.c_size_t, C.c_int, C.POINTER(C.c_void_p)]),
    "dnxcu_model_create_from_onnx": (C.c_int, [C.c_void_p, C.c_size_t, C.c_void_p, C.c_int, C.c_uint32, C.POINTER(C.c_void_p)]),
    "dnxcu_last_error_message": (C.c_char_p, []),
    "dnxcu_model_io": (C.c_int, [C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "dnxcu_model_dispatch_count": (C.c_int, [C.c_void_p]),
    "dnxcu_instance_dispatch_count": (C.c_int, [C.c_void_p]),
    "dnxcu_select_min_cost": (C.c_int, [C.c_int, C.c_int, C.POINTER(C.c_int32), C.POINTER(C.c_int32),
                                        C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_double),
                                        C.POINTER(C.c_int32), C.c_int, C.POINTER(C.c_int32), C.c_int, C.c_int,
                                        C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_double)]),
    "dnxcu_instance_create": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.POINTER(Band), C.POINTER(C.c_void_p)]),
    "dnxcu_instance_destroy": (None, [C.c_void_p]),
    "dnxcu_instance_infer": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p]),
    "dnxcu_instance_infer_async": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p]),
    "dnxcu_instance_wait": (C.c_int, [C.c_void_p]),
    "dnxcu_instance_enqueue": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "dnxcu_instance_graph_cache": (C.c_int, [C.c_void_p, C.c_int]),
    "dnxcu_instance_tensor": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_int),
                                        C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "dnxcu_instance_dispatch_info": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(DispatchInfo)]),
    "dnxcu_instance_bench": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.POINTER(DispatchInfo), C.c_int,
                                       C.POINTER(C.c_float)]),
    "dnxcu_instance_halo_count": (C.c_int, [C.c_void_p]),
    "dnxcu_instance_halo": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(HaloPoint)]),
    "dnxcu_instance_halo_export": (C.c_int, [C.c_void_p, C.POINTER(PeerHandle)]),
    "dnxcu_instance_halo_connect": (C.c_int, [C.c_void_p, C.POINTER(PeerHandle), C.POINTER(PeerHandle), C.c_int]),
    "dnxcu_instance_halo_step": (C.c_int, [C.c_void_p, C.c_int, C.c_uint32, C.c_void_p]),
    "dnxcu_instance_halo_auto": (C.c_int, [C.c_void_p, C.c_int]),
    "dnxcu_instance_halo_reset": (C.c_int, [C.c_void_p]),
    "dnxcu_instance_enqueue_range": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "dnxcu_instance_io": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p)]),
    "dnxcu_instance_extent": (C.c_int, [C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int),
                                        C.POINTER(C.c_int)]),
    "dnxcu_db_open": (C.c_int, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "dnxcu_db_close": (None, [C.c_void_p]),
    "dnxcu_db_size": (C.c_int, [C.c_void_p]),
    "dnxcu_db_populate": (C.c_int, [C.c_void_p, C.POINTER(ModelDesc), C.c_int, C.c_int, C.c_int]),
    "dnxcu_db_populate_model": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]),
    "dnxcu_db_bench": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_double, C.c_int]),
    "dnxcu_db_atomic_writeback": (C.c_int, [C.c_void_p]),
    "dnxcu_db_query": (C.c_int, [C.c_void_p, C.POINTER(Dispatch), C.POINTER(C.c_double), C.POINTER(C.c_double),
                                 C.POINTER(C.c_int)]),
    "dnxcu_db_add_result": (C.c_int, [C.c_void_p, C.POINTER(Dispatch), C.POINTER(C.c_double), C.c_int]),
}
for _name, (_res, _args) in SIGNATURES.items():
    _f = getattr(L, _name)
    _f.restype = _res
    _f.argtypes = _args


def device_caps(device=0) -> Caps:
    caps = Caps()
    check(L.dnxcu_get_device_caps(device, C.byref(caps)), "dnxcu_get_device_caps")
    return caps


def variants():
    out = []
    for i in range(L.dnxcu_variant_count()):
        v = L.dnxcu_variant(i).contents
        out.append(dict(id=v.id, op=v.op, family=v.family.decode(), config=v.config.decode(),
                        allowed_flags=v.allowed_flags, needs_tcgen05=v.needs_tcgen05))
    return out


def find_variant(family: str, config: str) -> int:
    return check(L.dnxcu_find_variant(family.encode(), config.encode()), f"find_variant {family} {config}")


def variant_sha256(vid: int) -> str:
    buf = C.create_string_buffer(65)
    check(L.dnxcu_variant_sha256(vid, buf))
    return buf.value.decode()


def prepare_weights(variant: int, w_kcrs: np.ndarray, c_a: int, c_b: int = 0) -> np.ndarray:
    """Host re-layout of [K][C][3][3] binary16 weights for `variant`; returns a uint8 blob."""
    w = np.ascontiguousarray(w_kcrs, dtype=np.float16)
    k = w.shape[0]
    assert w.shape == (k, c_a + c_b, 3, 3)
    n = C.c_size_t(0)
    check(L.dnxcu_prepare_weights(variant, None, k, c_a, c_b, None, C.byref(n)), "prepare_weights(size)")
    blob = np.zeros(n.value, dtype=np.uint8)
    check(L.dnxcu_prepare_weights(variant, w.ctypes.data, k, c_a, c_b, blob.ctypes.data, C.byref(n)),
          "prepare_weights")
    return blob


def select_min_cost(n_nodes, edges, inputs, outputs, min_dispatches=False):
    """The schedule search on a hand built hypergraph.  edges: list of (sources, destinations, weight).
    Returns (chosen edge indices in firing order, total cost) or None when the outputs cannot be derived."""
    i32 = C.c_int32
    src_off, srcs, dst_off, dsts, w = [0], [], [0], [], []
    for (s, d, wt) in edges:
        srcs += list(s)
        dsts += list(d)
        src_off.append(len(srcs))
        dst_off.append(len(dsts))
        w.append(float(wt))
    arr = lambda t, v: (t * max(1, len(v)))(*v)
    chosen = (i32 * max(1, len(edges)))()
    n, cost = i32(0), C.c_double(0)
    st = L.dnxcu_select_min_cost(n_nodes, len(edges), arr(i32, src_off), arr(i32, srcs), arr(i32, dst_off), arr(i32, dsts),
                                 arr(C.c_double, w), arr(i32, list(inputs)), len(inputs), arr(i32, list(outputs)),
                                 len(outputs), int(min_dispatches), chosen, C.byref(n), C.byref(cost))
    if st == E_UNSUPPORTED:
        return None
    check(st, "dnxcu_select_min_cost")
    return list(chosen[:n.value]), cost.value


def _model_desc(net, options=0):
    """ModelDesc for a nets.Net; returns (desc, keepalive)."""
    arr = (NodeC * len(net.nodes))()
    keep = [arr]
    for i, nd in enumerate(net.nodes):
        arr[i].kind, arr[i].in0, arr[i].in1, arr[i].out, arr[i].c_out = nd.kind, nd.in0, nd.in1, nd.out, nd.c_out
        arr[i].alpha = float(getattr(nd, "alpha", 0.0))
        if nd.weights is not None:
            w = np.ascontiguousarray(nd.weights, dtype=np.float16)
            keep.append(w)
            arr[i].weights_kcrs = w.ctypes.data
        if nd.bias is not None:
            b = np.ascontiguousarray(nd.bias, dtype=np.float16)
            keep.append(b)
            arr[i].bias = b.ctypes.data
    desc = ModelDesc(len(net.nodes), net.n_tensors, arr, net.input_tensor, net.in_channels, net.output_tensor,
                     options)
    return desc, keep


class Db:
    """Benchmark database handle (denox::Db)."""

    def __init__(self, path):
        self._h = C.c_void_p()
        check(L.dnxcu_db_open(str(path).encode(), C.byref(self._h)), "dnxcu_db_open")

    def close(self):
        if self._h:
            L.dnxcu_db_close(self._h)
            self._h = C.c_void_p()

    def __len__(self):
        return check(L.dnxcu_db_size(self._h))

    def populate(self, net, h, w, device=0, options=0):
        """device < 0: enumerate for a device with every capability, without touching one."""
        desc, keep = _model_desc(net, options)
        return check(L.dnxcu_db_populate(self._h, C.byref(desc), h, w, device), "dnxcu_db_populate")

    def bench(self, device=0, min_samples=10, max_relative_error=0.05, max_rounds=8):
        return check(L.dnxcu_db_bench(self._h, device, min_samples, max_relative_error, max_rounds), "dnxcu_db_bench")

    def writeback(self):
        return check(L.dnxcu_db_atomic_writeback(self._h), "dnxcu_db_atomic_writeback")

    def query(self, d: Dispatch):
        mean, std, n = C.c_double(), C.c_double(), C.c_int()
        st = L.dnxcu_db_query(self._h, C.byref(d), C.byref(mean), C.byref(std), C.byref(n))
        return None if st < 0 else (mean.value, std.value, n.value)

    def add_result(self, d: Dispatch, samples_ms):
        arr = (C.c_double * len(samples_ms))(*samples_ms)
        return check(L.dnxcu_db_add_result(self._h, C.byref(d), arr, len(samples_ms)), "dnxcu_db_add_result")


def _write_blob(fn, handle, what):
    n = C.c_size_t(0)
    check(fn(handle, None, C.byref(n)), what + "(size)")
    buf = (C.c_ubyte * n.value)()
    check(fn(handle, buf, C.byref(n)), what)
    return bytes(buf[:n.value])


class Model:
    """Fused dispatch list of a network (runtime::Model)."""

    def __init__(self, net, device=0, options=0, db: Db = None):
        self.net = net
        desc, self._keep = _model_desc(net, options)
        self._db = db
        self._h = C.c_void_p()
        check(L.dnxcu_model_create(C.byref(desc), db._h if db else None, device, C.byref(self._h)),
              "dnxcu_model_create")
        self.device = device

    @classmethod
    def from_dnx(cls, blob: bytes, net=None, device=0):
        """A model that runs the dispatches of a dnx file (runtime::Model::make).  `net` only supplies the
        channel counts the host-side convenience calls need; device < 0 parses without touching a device."""
        self = cls.__new__(cls)
        self.net, self._keep, self._db, self.device = net, None, None, device
        self._h = C.c_void_p()
        check(L.dnxcu_model_create_from_dnx(blob, len(blob), device, C.byref(self._h)), "dnxcu_model_create_from_dnx")
        return self

    @classmethod
    def from_onnx(cls, blob: bytes, device=0, options=0, db: Db = None):
        """A model imported from the bytes of an ONNX file (the reference's frontend subset)."""
        self = cls.__new__(cls)
        self.net, self._keep, self._db, self.device = None, None, db, device
        self._h = C.c_void_p()
        st = L.dnxcu_model_create_from_onnx(blob, len(blob), db._h if db else None, device, options, C.byref(self._h))
        if st < 0:
            raise DnxcuError(st, "dnxcu_model_create_from_onnx: " + L.dnxcu_last_error_message().decode())
        return self

    def io(self):
        """(input tensor id, input channels, output tensor id)."""
        a, c, b = C.c_int(), C.c_int(), C.c_int()
        check(L.dnxcu_model_io(self._h, C.byref(a), C.byref(c), C.byref(b)))
        return a.value, c.value, b.value

    def write_dnx(self) -> bytes:
        """The default schedule with the preferred variant per dispatch as a dnx file (no device needed)."""
        return _write_blob(L.dnxcu_model_write_dnx, self._h, "dnxcu_model_write_dnx")

    def dispatch_count(self):
        return check(L.dnxcu_model_dispatch_count(self._h))

    def close(self):
        if self._h:
            L.dnxcu_model_destroy(self._h)
            self._h = C.c_void_p()


class Instance:
    """A model bound to one image extent (runtime::Instance)."""

    def __init__(self, model: Model, h: int, w: int, band=None):
        self.model = model
        self.h, self.w = h, w
        self._h = C.c_void_p()
        b = Band(*band) if band else None
        check(L.dnxcu_instance_create(model._h, h, w, C.byref(b) if b else None, C.byref(self._h)),
              "dnxcu_instance_create")
        self.rows = band[2] if band else h

    def infer(self, x: np.ndarray) -> np.ndarray:
        """Host in, host out, synchronous (Instance::infer)."""
        _, in_channels, out_tensor = self.model.io()
        x = np.ascontiguousarray(x, dtype=np.float16)
        assert x.shape == (self.rows, self.w, in_channels), x.shape
        _, h, w, c = self.tensor(out_tensor)
        fh, fw, rh, rw = self.extent()
        if (fh, fw) != (rh, rw):  # the instance pads the frame and slices the output back
            h, w = fh, fw
        y = np.empty((h, w, c), dtype=np.float16)
        check(L.dnxcu_instance_infer(self._h, x.ctypes.data, y.ctypes.data), "dnxcu_instance_infer")
        return y

    def infer_async(self, x: np.ndarray, y: np.ndarray):
        """Stream ordered infer: x and y must stay alive (pinned for overlap) until wait()."""
        check(L.dnxcu_instance_infer_async(self._h, x.ctypes.data, y.ctypes.data), "dnxcu_instance_infer_async")

    def wait(self):
        check(L.dnxcu_instance_wait(self._h), "dnxcu_instance_wait")

    def enqueue(self, dev_in: int, dev_out: int, stream: int = 0):
        check(L.dnxcu_instance_enqueue(self._h, dev_in, dev_out, stream), "dnxcu_instance_enqueue")

    def write_dnx(self) -> bytes:
        """This instance's schedule and variants (what a benchmark database chose) as a dnx file."""
        return _write_blob(L.dnxcu_instance_write_dnx, self._h, "dnxcu_instance_write_dnx")

    def graph_cache(self, pairs: int):
        """Keep the captured graphs of this many (input, output) pointer pairs."""
        check(L.dnxcu_instance_graph_cache(self._h, pairs), "dnxcu_instance_graph_cache")

    def enqueue_range(self, first, last, stream=0):
        check(L.dnxcu_instance_enqueue_range(self._h, first, last, stream), "dnxcu_instance_enqueue_range")

    def io(self):
        a, b = C.c_void_p(), C.c_void_p()
        check(L.dnxcu_instance_io(self._h, C.byref(a), C.byref(b)))
        return a.value, b.value

    def extent(self):
        """(h, w) of the caller's frames and (h_run, w_run) the schedule runs at."""
        v = [C.c_int() for _ in range(4)]
        check(L.dnxcu_instance_extent(self._h, *[C.byref(x) for x in v]))
        return tuple(x.value for x in v)

    def tensor(self, tid):
        p, h, w, c = C.c_void_p(), C.c_int(), C.c_int(), C.c_int()
        check(L.dnxcu_instance_tensor(self._h, tid, C.byref(p), C.byref(h), C.byref(w), C.byref(c)),
              f"dnxcu_instance_tensor({tid})")
        return p.value, h.value, w.value, c.value

    def dispatch_count(self):
        """Dispatches of this instance's schedule (a database may have chosen another than the model's default)."""
        return check(L.dnxcu_instance_dispatch_count(self._h))

    def dispatch_info(self):
        n = self.dispatch_count()
        out = []
        for i in range(n):
            info = DispatchInfo()
            check(L.dnxcu_instance_dispatch_info(self._h, i, C.byref(info)))
            out.append(info)
        return out

    def bench(self, warmup=3, iters=10):
        n = self.dispatch_count()
        infos = (DispatchInfo * n)()
        total = C.c_float()
        check(L.dnxcu_instance_bench(self._h, warmup, iters, infos, n, C.byref(total)), "dnxcu_instance_bench")
        return list(infos), total.value

    def halo_points(self):
        n = check(L.dnxcu_instance_halo_count(self._h))
        pts = []
        for e in range(n):
            p = HaloPoint()
            check(L.dnxcu_instance_halo(self._h, e, C.byref(p)))
            pts.append(p)
        return pts

    def halo_export(self) -> "PeerHandle":
        h = PeerHandle()
        check(L.dnxcu_instance_halo_export(self._h, C.byref(h)), "dnxcu_instance_halo_export")
        return h

    def halo_connect(self, up, down, auto_exchange=True):
        check(L.dnxcu_instance_halo_connect(self._h, C.byref(up) if up is not None else None,
                                            C.byref(down) if down is not None else None, int(auto_exchange)),
              "dnxcu_instance_halo_connect")

    def halo_reset(self):
        check(L.dnxcu_instance_halo_reset(self._h), "dnxcu_instance_halo_reset")

    def halo_auto(self, on: bool):
        check(L.dnxcu_instance_halo_auto(self._h, int(on)), "dnxcu_instance_halo_auto")

    def halo_step(self, dispatch, mode, stream=0):
        check(L.dnxcu_instance_halo_step(self._h, dispatch, mode, stream), "dnxcu_instance_halo_step")

    def close(self):
        if self._h:
            L.dnxcu_instance_destroy(self._h)
            self._h = C.c_void_p()
