"""Helpers for the GPU parity tests: device buffers through torch, dispatches through the C ABI."""
import ctypes as C

import numpy as np
import torch

from denox_b200 import lib


def dev(x: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def host(t: torch.Tensor) -> np.ndarray:
    return t.cpu().numpy()


class _Raw:
    def __init__(self, ptr, shape):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": "<f2", "data": (int(ptr), False),
                                         "version": 2}


def wrap(ptr, shape) -> torch.Tensor:
    """A torch view of device memory the library owns (binary16)."""
    torch.cuda.synchronize()
    return torch.as_tensor(_Raw(ptr, shape), device="cuda")


CANARY = 12345.0


class Guarded:
    """Output buffer with a canary region on both sides (no sanitizer on the box:
    out-of-bounds writes show up as damaged canaries)."""

    def __init__(self, shape, pad=4096):
        n = int(np.prod(shape))
        self.pad = pad
        self.buf = torch.full((n + 2 * pad,), CANARY, dtype=torch.float16, device="cuda")
        self.view = self.buf[pad:pad + n].view(*shape)
        self.view.fill_(float("nan"))  # unwritten elements are caught by the finiteness check

    def ptr(self):
        return self.view.data_ptr()

    def check(self):
        b = self.buf
        assert bool((b[:self.pad] == CANARY).all()) and bool((b[-self.pad:] == CANARY).all()), "canary damaged"
        return host(self.view)


def run_conv(variant, a, w_kcrs, bias=None, relu=False, b=None, up_a=False, pool=False, full=True, halo=None,
             leaky=None, planned=False):
    """Launches one conv dispatch through dnxcu_launch; returns (out, out_pool) as numpy (None when not written)."""
    ca = a.shape[2]
    cb = 0 if b is None else b.shape[2]
    h, w = (a.shape[0] * 2, a.shape[1] * 2) if up_a else a.shape[:2]
    k = w_kcrs.shape[0]
    d = lib.Dispatch()
    d.variant = variant
    d.flags = (lib.F_RELU if relu else 0) | (lib.F_BIAS if bias is not None else 0) | (lib.F_UP2X_A if up_a else 0) \
        | (lib.F_POOL_OUT if pool else 0) | (0 if full else lib.F_NO_FULL_OUT) | (lib.F_LEAKY if leaky is not None else 0)
    d.leaky_alpha = float(leaky or 0.0)
    d.pc[0], d.pc[1] = w, h
    d.c_a, d.c_b, d.c_out = ca, cb, k
    keep = []
    ta = dev(a); keep.append(ta); d.in_a = ta.data_ptr()
    if b is not None:
        tb = dev(b); keep.append(tb); d.in_b = tb.data_ptr()
    tw = dev(lib.prepare_weights(variant, w_kcrs, ca, cb)); keep.append(tw); d.weights = tw.data_ptr()
    if bias is not None:
        tbias = dev(np.asarray(bias, dtype=np.float16)); keep.append(tbias); d.bias = tbias.data_ptr()
    if halo is not None:
        for i, hrow in enumerate(halo):
            if hrow is not None:
                th = dev(np.asarray(hrow, dtype=np.float16)); keep.append(th); d.halo[i] = th.data_ptr()
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    d.device_status = status.data_ptr()
    out = Guarded((h, w, k)) if full else None
    outp = Guarded((h // 2, w // 2, k)) if pool else None
    if out is not None:
        d.out = out.ptr()
    if outp is not None:
        d.out_pool = outp.ptr()
    torch.cuda.synchronize()
    if planned:  # plan once, launch twice: the second launch must give the same bits as the first
        plan = C.c_void_p()
        lib.check(lib.L.dnxcu_plan_create(C.byref(d), C.byref(plan)), f"dnxcu_plan_create variant {variant}")
        lib.check(lib.L.dnxcu_plan_launch(plan, None), "dnxcu_plan_launch")
        lib.check(lib.L.dnxcu_plan_launch(plan, None), "dnxcu_plan_launch (second)")
        torch.cuda.synchronize()
        lib.L.dnxcu_plan_destroy(plan)
    else:
        lib.check(lib.L.dnxcu_launch(C.byref(d), None), f"dnxcu_launch variant {variant}")
    torch.cuda.synchronize()
    assert int(status[0].item()) == 0, f"kernel reported a bounded wait that ran out: code {int(status[0].item())}"
    return (out.check() if out else None), (outp.check() if outp else None)


def run_mem(variant, a, b=None, leaky=None):
    d = lib.Dispatch()
    d.variant = variant
    if leaky is not None:
        d.flags = lib.F_LEAKY
        d.leaky_alpha = float(leaky)
    h, w, ca = a.shape
    d.pc[0], d.pc[1] = w, h
    d.c_a = ca
    ta = dev(a); d.in_a = ta.data_ptr()
    op = lib.L.dnxcu_variant(variant).contents.op
    if op == lib.OP_MAXPOOL2X2:
        shape = (h // 2, w // 2, ca)
    elif op == lib.OP_UPSAMPLE2X:
        shape = (2 * h, 2 * w, ca)
    elif op == lib.OP_CONCAT:
        tb = dev(b); d.in_b = tb.data_ptr(); d.c_b = b.shape[2]
        shape = (h, w, ca + b.shape[2])
    else:
        shape = (h, w, ca)
    out = Guarded(shape)
    d.out = out.ptr()
    lib.check(lib.L.dnxcu_launch(C.byref(d), None), f"dnxcu_launch variant {variant}")
    torch.cuda.synchronize()
    return out.check()
