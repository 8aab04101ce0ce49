"""Per kernel parity on the GPU, through the C ABI, against the CPU oracle and the
PyTorch generated golden fixtures.  Tolerance: |d| <= 2e-2 + 1e-2 |ref| per element
against the binary16-accumulating oracle (the stand-in for the reference's own
arithmetic); against the fp32-accumulating oracle the kernels (fp32 accumulation,
one rounding) must agree to one binary16 ulp."""
import importlib.util
import os

import numpy as np
import pytest

from conftest import assert_close
from denox_b200 import lib, nets, rng
from oracle import oracle

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_golden.py"))
mg = importlib.util.module_from_spec(spec)
spec.loader.exec_module(mg)
GOLD = np.load(os.path.join(HERE, "golden", "golden.npz"))

CONV_VARIANTS = [v["id"] for v in lib.variants() if v["op"] == lib.OP_CONV3X3]


def one_ulp(got, ref):
    g, r = got.astype(np.float32), ref.astype(np.float32)
    return np.abs(g - r) <= np.maximum(np.abs(r) * 2.0 ** -10, 2.0 ** -14) * 1.01


def supports(variant, flags, ca, cb, k, h, w):
    import ctypes as C
    d = lib.Dispatch()
    d.variant, d.flags, d.c_a, d.c_b, d.c_out = variant, flags, ca, cb, k
    d.pc[0], d.pc[1] = w, h
    d.in_a = d.out = d.weights = d.bias = 0x1000
    d.in_b = 0x1000 if cb else None
    d.out_pool = 0x1000
    return lib.L.dnxcu_validate(C.byref(d)) == 0


@pytest.mark.parametrize("variant", CONV_VARIANTS)
@pytest.mark.parametrize("case", mg.CONV_CASES, ids=[c[0] for c in mg.CONV_CASES])
def test_conv_against_oracle_and_golden(variant, case):
    from gpu_util import run_conv
    name, h, w, ca, cb, k, relu, bias, up = case
    flags = (lib.F_RELU if relu else 0) | (lib.F_BIAS if bias else 0) | (lib.F_UP2X_A if up else 0)
    if not supports(variant, flags, ca, cb, k, h, w):
        pytest.skip("variant does not take this dispatch")
    a, b, wt, bs = mg.conv_case_tensors(case)
    y, _ = run_conv(variant, a, wt, bs, relu=relu, b=b, up_a=up)
    ref32 = oracle.conv3x3(a, wt, bs, relu=relu, mode=oracle.ACC_F32, b=b, up_a=up)
    ref16 = oracle.conv3x3(a, wt, bs, relu=relu, mode=oracle.ACC_F16, b=b, up_a=up)
    assert one_ulp(y, ref32).all(), (name, np.abs(y.astype(np.float32) - ref32.astype(np.float32)).max())
    assert_close(y, ref16, f"{name} vs acc=f16 oracle", max_violation_fraction=1e-3)
    assert_close(y, GOLD["conv/" + name], f"{name} vs PyTorch golden")


@pytest.mark.parametrize("variant", CONV_VARIANTS)
@pytest.mark.parametrize("case", mg.CONV_CASES2, ids=[c[0] for c in mg.CONV_CASES2])
def test_conv_more_shapes_and_leaky_relu(variant, case):
    """The remaining channel pairs of the reference's conv test list (test/system/test_conv.py, up to 256 -> 256,
    bias on) and LeakyReLU epilogues, launched through a plan that is used twice."""
    from gpu_util import run_conv
    name, h, w, ca, cb, k, relu, bias, up, leaky = case
    flags = (lib.F_RELU if relu else 0) | (lib.F_BIAS if bias else 0) | (lib.F_UP2X_A if up else 0) | \
        (lib.F_LEAKY if leaky is not None else 0)
    if not supports(variant, flags, ca, cb, k, h, w):
        pytest.skip("variant does not take this dispatch")
    a, b, wt, bs = mg.conv_case_tensors(case)
    y, _ = run_conv(variant, a, wt, bs, relu=relu, b=b, up_a=up, leaky=leaky, planned=True)
    ref32 = oracle.conv3x3(a, wt, bs, relu=relu, mode=oracle.ACC_F32, b=b, up_a=up, leaky=leaky)
    # one ulp of the sum (another summation order) becomes up to three of a negative output once it is scaled by alpha
    ulps = 3.0 if leaky is not None else 1.0
    d32 = np.abs(y.astype(np.float32) - ref32.astype(np.float32))
    assert (d32 <= ulps * np.maximum(np.abs(ref32.astype(np.float32)) * 2.0 ** -10, 2.0 ** -14) * 1.01).all(), (name, d32.max())
    ref16 = oracle.conv3x3(a, wt, bs, relu=relu, mode=oracle.ACC_F16, b=b, up_a=up, leaky=leaky)
    if ca + cb >= 256:  # the reference's own tests relax to atol = 1e-1 here (test_conv.py:113-123)
        assert (np.abs(y.astype(np.float32) - ref16.astype(np.float32)) <= 1e-1).all()
    else:
        assert_close(y, ref16, f"{name} vs acc=f16 oracle", max_violation_fraction=5e-3)
    assert_close(y, GOLD["conv/" + name], f"{name} vs PyTorch golden")


@pytest.mark.parametrize("c", [8, 24, 9])
def test_leaky_relu_standalone_bit_exact(c):
    from gpu_util import run_mem
    h, w = 12, 20
    x = rng.to_f16(rng.uniform(9100 if c == 24 else 9200 + c, h * w * c, -8.0, 8.0)).reshape(h, w, c)
    x[0, 0, :3] = [0.0, -0.0, -6e-8]
    for v in lib.variants():
        if v["op"] != lib.OP_RELU or (v["config"] == "VEC=8" and (h * w * c) % 8):
            continue
        for alpha in (0.3, 0.01):
            got = run_mem(v["id"], x, leaky=alpha)
            assert (got.view(np.uint16) == oracle.leaky_relu(x, alpha).view(np.uint16)).all(), (v["config"], alpha)
    if c == 24:
        assert_close(oracle.leaky_relu(x, 0.3)[1:], GOLD["leaky/standalone_c24"][1:], "leaky vs PyTorch golden")


@pytest.mark.parametrize("variant", CONV_VARIANTS)
@pytest.mark.parametrize("shape", [(16, 128, 32, 32), (18, 130, 16, 48), (34, 300, 48, 64), (16, 16, 64, 80),
                                   (2, 2, 16, 16), (6, 1922 // 2 * 2, 32, 32)])
def test_conv_pool_epilogue(variant, shape):
    """conv + relu + 2x2 max pool in one dispatch: single (pooled only) and dual output."""
    from gpu_util import run_conv
    h, w, c, k = shape
    flags = lib.F_RELU | lib.F_POOL_OUT
    if not supports(variant, flags, c, 0, k, h, w):
        pytest.skip("variant does not take this dispatch")
    a = rng.to_f16(rng.uniform(77 + h + w, h * w * c, -1, 1)).reshape(h, w, c)
    wt = rng.he_normal_weights(78, k, c)
    ref = oracle.conv3x3(a, wt, relu=True)
    refp = oracle.maxpool2x2(ref)
    y, yp = run_conv(variant, a, wt, relu=True, pool=True, full=True)
    assert one_ulp(y, ref).all() and one_ulp(yp, refp).all()
    # pooling commutes with rounding: the pooled tensor must be exactly the pool of the kernel's own full output
    assert (yp == oracle.maxpool2x2(y)).all()
    _, yp2 = run_conv(variant, a, wt, relu=True, pool=True, full=False)
    assert (yp2 == yp).all()


@pytest.mark.parametrize("variant", CONV_VARIANTS)
def test_conv_row_band_with_halo_rows(variant):
    """A band of a taller image plus halo rows gives bit-identical rows (row band multi-GPU path)."""
    from gpu_util import run_conv
    h, w, ca, cb, k = 32, 200, 32, 16, 32
    flags = lib.F_RELU | lib.F_UP2X_A
    if not supports(variant, flags, ca, cb, k, h, w):
        pytest.skip("variant does not take this dispatch")
    a = rng.to_f16(rng.uniform(91, (h // 2) * (w // 2) * ca, -1, 1)).reshape(h // 2, w // 2, ca)
    b = rng.to_f16(rng.uniform(92, h * w * cb, -1, 1)).reshape(h, w, cb)
    wt = rng.he_normal_weights(93, k, ca + cb)
    full, _ = run_conv(variant, a, wt, relu=True, b=b, up_a=True)
    ref = oracle.conv3x3(a, wt, relu=True, b=b, up_a=True)
    assert one_ulp(full, ref).all()
    # rows [16, 32): top halo = row 15 of the virtual upsampled a = source row 7, of b = row 15; bottom = image border
    band, _ = run_conv(variant, a[8:16], wt, relu=True, b=b[16:32], up_a=True, halo=(a[7], None, b[15], None))
    assert (band == full[16:32]).all()
    band0, _ = run_conv(variant, a[0:8], wt, relu=True, b=b[0:16], up_a=True, halo=(None, a[8], None, b[16]))
    assert (band0 == full[0:16]).all()


@pytest.mark.parametrize("c", [8, 32, 48, 80, 3, 9, 67])
def test_pool_upsample_concat_relu(c):
    from gpu_util import run_mem
    h, w = 34, 46
    x = rng.to_f16(rng.normal(5 + c, h * w * c)).reshape(h, w, c)
    y = rng.to_f16(rng.normal(6 + c, h * w * c)).reshape(h, w, c)
    for v in lib.variants():
        vec = v["config"] == "VEC=8"
        if v["op"] == lib.OP_CONV3X3 or (vec and c % 8):
            continue
        if v["op"] == lib.OP_MAXPOOL2X2:
            assert (run_mem(v["id"], x) == oracle.maxpool2x2(x)).all()
        elif v["op"] == lib.OP_UPSAMPLE2X:
            assert (run_mem(v["id"], x) == oracle.upsample2x(x)).all()
        elif v["op"] == lib.OP_CONCAT:
            assert (run_mem(v["id"], x, y) == oracle.concat(x, y)).all()
        elif v["op"] == lib.OP_RELU:
            assert (run_mem(v["id"], x) == oracle.relu(x)).all()


def test_pool_odd_extent_floor():
    from gpu_util import run_mem
    x = rng.to_f16(rng.normal(3, 7 * 9 * 8)).reshape(7, 9, 8)
    for vid in (lib.find_variant("basic-pool", "VEC=8"), lib.find_variant("basic-pool", "VEC=1")):
        assert (run_mem(vid, x) == oracle.maxpool2x2(x)).all()


def test_launch_rejects_bad_dispatches_without_touching_the_device():
    import ctypes as C
    d = lib.Dispatch()
    d.variant = 2
    assert lib.L.dnxcu_launch(C.byref(d), None) == lib.E_BAD_ARG
    d.variant = 999
    assert lib.L.dnxcu_launch(C.byref(d), None) == lib.E_BAD_ARG
    assert lib.L.dnxcu_launch(None, None) == lib.E_BAD_ARG


def test_device_caps():
    caps = lib.device_caps(0)
    assert caps.sm_count > 0 and caps.cc_major == 10 and caps.tcgen05 == 1 and caps.tmem_columns == 512


@pytest.mark.parametrize("case", mg.PAD_CASES + [("c16_big", 270, 481, 16, 0, 15, 0, 2)], ids=lambda c: c[0])
def test_pad_edge_and_slice_bit_exact(case):
    """memory-pad / memory-slice against the oracle, both vector widths where the channel count allows."""
    import ctypes as C
    import torch
    from gpu_util import Guarded, dev
    name, h, w, c, l, r, t, b = case
    x = mg.pad_case_input(case)
    ref = oracle.pad_edge(x, l, r, t, b)
    if "pad/" + name in GOLD.files:
        assert (ref.view(np.uint16) == GOLD["pad/" + name].view(np.uint16)).all()
    oh, ow = h + t + b, w + l + r
    tx = dev(x)
    for vec in (["VEC=8", "VEC=1"] if c % 8 == 0 else ["VEC=1"]):
        d = lib.Dispatch()
        d.variant = lib.L.dnxcu_find_variant(b"memory-pad", vec.encode())
        d.pc[0], d.pc[1], d.c_a = ow, oh, c
        d.pc_ext[0], d.pc_ext[1], d.pc_ext[2], d.pc_ext[3] = l, r, t, b
        out = Guarded((oh, ow, c))
        d.in_a, d.out = tx.data_ptr(), out.ptr()
        lib.check(lib.L.dnxcu_launch(C.byref(d), None))
        y = out.check()
        assert (y.view(np.uint16) == ref.view(np.uint16)).all(), (name, vec, "pad")
        q = lib.Dispatch()
        q.variant = lib.L.dnxcu_find_variant(b"memory-slice", vec.encode())
        q.pc[0], q.pc[1], q.c_a = w, h, c
        q.pc_ext[0], q.pc_ext[1], q.pc_ext[2], q.pc_ext[3] = l, t, ow, oh
        back = Guarded((h, w, c))
        ty = dev(y)
        q.in_a, q.out = ty.data_ptr(), back.ptr()
        lib.check(lib.L.dnxcu_launch(C.byref(q), None))
        assert (back.check().view(np.uint16) == x.view(np.uint16)).all(), (name, vec, "slice")
    # a slice that would read outside its input is refused before any launch
    bad = lib.Dispatch()
    bad.variant = lib.L.dnxcu_find_variant(b"memory-slice", b"VEC=1")
    bad.pc[0], bad.pc[1], bad.c_a = w, h, c
    bad.pc_ext[0], bad.pc_ext[1], bad.pc_ext[2], bad.pc_ext[3] = 1, 0, w, h
    bad.in_a, bad.out = tx.data_ptr(), tx.data_ptr()
    assert lib.L.dnxcu_launch(C.byref(bad), None) == lib.E_BAD_ARG


@pytest.mark.parametrize("shape", [(7, 37, 9, 16), (16, 16, 3, 8), (33, 129, 9, 16), (5, 11, 67, 72), (3, 700, 12, 16)])
def test_pad_channels_bit_exact(shape):
    """copy-transform PAD=8: HWC with C channels -> HWC with c_out channels, the new ones zero."""
    import ctypes as C
    from gpu_util import Guarded, dev
    h, w, c, co = shape
    x = rng.to_f16(rng.uniform(9100 + c, h * w * c, -3.0, 3.0)).reshape(h, w, c)
    ref = np.zeros((h, w, co), dtype=np.float16)
    ref[:, :, :c] = x
    d = lib.Dispatch()
    d.variant = lib.L.dnxcu_find_variant(b"copy-transform", b"PAD=8")
    d.pc[0], d.pc[1], d.c_a, d.c_out = w, h, c, co
    tx = dev(x)
    out = Guarded((h, w, co))
    d.in_a, d.out = tx.data_ptr(), out.ptr()
    lib.check(lib.L.dnxcu_launch(C.byref(d), None))
    y = out.check()
    assert (y.view(np.uint16) == ref.view(np.uint16)).all()

def test_conv_kernel_gives_up_cleanly_when_its_wait_limit_is_tiny():
    """The bounded waits of the tensor core conv kernel itself: with a limit of one microsecond the wait for the
    layer's weights (some hundred KB from DRAM) runs out; the kernel reports a code through device_status, all its
    roles leave, it frees its tensor memory and ends.  The launch after that, with the normal limit, is right."""
    import ctypes as C
    import torch
    from gpu_util import dev
    h, w, c, k = 64, 256, 96, 96
    a = rng.to_f16(rng.uniform(801, h * w * c, -1, 1)).reshape(h, w, c)
    wt = rng.he_normal_weights(802, k, c)
    variant = lib.find_variant("direct-conv-tc", "DY=stack#KG=2#W=resident")
    ta, tw = dev(a), dev(lib.prepare_weights(variant, wt, c))
    out = torch.zeros((h, w, k), dtype=torch.float16, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    d = lib.Dispatch()
    d.variant, d.flags, d.c_a, d.c_out = variant, lib.F_RELU, c, k
    d.pc[0], d.pc[1] = w, h
    d.in_a, d.out, d.weights, d.device_status = ta.data_ptr(), out.data_ptr(), tw.data_ptr(), status.data_ptr()
    lib.check(lib.L.dnxcu_set_wait_limit_us(1))
    try:
        codes = []
        for _ in range(3):  # cold caches make the first launch the slowest; any of them may run out
            lib.check(lib.L.dnxcu_launch(C.byref(d), None))
            torch.cuda.synchronize()
            codes.append(int(status[0].item()))
            status.zero_()
    finally:
        lib.check(lib.L.dnxcu_set_wait_limit_us(0))
    assert all(0 <= cd <= 10 for cd in codes), codes
    print("wait codes with a 1 us limit:", codes)
    # whatever happened above, the device and the library are in order
    lib.check(lib.L.dnxcu_launch(C.byref(d), None))
    torch.cuda.synchronize()
    assert int(status[0].item()) == 0
    ref = oracle.conv3x3(a, wt, relu=True, mode=oracle.ACC_F32)
    assert one_ulp(out.cpu().numpy(), ref).all()
    assert any(codes), "a one microsecond limit was expected to run out at least once"


def test_split_dispatches_from_two_threads_on_two_streams():
    """Output channel split dispatches (several launches between a fork and a join on side streams) issued by two
    host threads at the same time, each on its own stream: every thread has its own side streams, so neither can
    pick up the other's fork."""
    import ctypes as C
    import threading
    import torch
    from gpu_util import dev
    variant = lib.find_variant("direct-conv-tc", "DY=stack#KG=2#W=resident#NSPLIT=2")
    h, w, c, k = 48, 200, 64, 96
    jobs = []
    for t in range(2):
        a = rng.to_f16(rng.uniform(900 + t, h * w * c, -1, 1)).reshape(h, w, c)
        wt = rng.he_normal_weights(910 + t, k, c)
        jobs.append(dict(a=a, wt=wt, ta=dev(a), tw=dev(lib.prepare_weights(variant, wt, c)),
                         mid=torch.zeros((h, w, k), dtype=torch.float16, device="cuda"),
                         stream=torch.cuda.Stream(), errors=[]))
    torch.cuda.synchronize()

    def work(j):
        try:
            d = lib.Dispatch()
            d.variant, d.flags, d.c_a, d.c_out = variant, lib.F_RELU, c, k
            d.pc[0], d.pc[1] = w, h
            d.in_a, d.out, d.weights = j["ta"].data_ptr(), j["mid"].data_ptr(), j["tw"].data_ptr()
            for _ in range(200):
                st = lib.L.dnxcu_launch(C.byref(d), j["stream"].cuda_stream)
                if st:
                    j["errors"].append((st, lib.L.dnxcu_last_cuda_error()))  # the CUDA code is kept per host thread
                    return
            j["stream"].synchronize()
        except Exception as e:  # noqa: BLE001
            j["errors"].append(repr(e))

    threads = [threading.Thread(target=work, args=(j,)) for j in jobs]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    torch.cuda.synchronize()
    for j in jobs:
        assert not j["errors"], j["errors"]
        ref = oracle.conv3x3(j["a"], j["wt"], relu=True, mode=oracle.ACC_F32)
        assert one_ulp(j["mid"].cpu().numpy(), ref).all()
