"""Parity at the benchmark's full frame sizes (1088 x 1920 and its pooled levels).

The small cases of test_kernels_gpu.py never give a persistent CTA more than one work
unit; these do (15 strips x 1088 rows over 148 SMs), so they cover the state a CTA
carries from unit to unit: slot ring, TMEM block ring, barrier phases.  Checks, per
tensor core variant that takes the dispatch:
  * every element against the CUDA core kernel (a separate implementation, fp32
    accumulation, other summation order): two binary16 ulps;
  * three bands of rows (top, middle, bottom) against the CPU oracle with fp32
    accumulation: one binary16 ulp, the same bound as the small cases;
  * the pooled output against the 2x2 max of the full output: bit exact.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from denox_b200 import lib, nets, rng
from gpu_util import Guarded
from oracle import oracle

pytestmark = pytest.mark.gpu

H, W = 1088, 1920
# name, h, w, c_a, c_b, k, relu, bias, up_a, pool
CASES = [
    ("c32_k32_pool", H, W, 32, 0, 32, True, False, False, True),
    ("c16_k32", H, W, 16, 0, 32, True, False, False, False),
    ("c64_k64", H, W, 64, 0, 64, True, False, False, False),
    ("c64_k32_bias", H, W, 64, 0, 32, True, True, False, False),
    ("c32_k3", H, W, 32, 0, 3, False, False, False, False),
    ("up64_cat16_k64", H, W, 64, 16, 64, True, False, True, False),
    ("up96_cat32_k64", H // 2, W // 2, 96, 32, 64, True, False, True, False),
    ("c96_k96", H // 4, W // 4, 96, 0, 96, True, False, False, False),
    ("up112_cat48_k96", H // 4, W // 4, 112, 48, 96, True, False, True, False),
    # the remaining layer shapes of the benchmark net
    ("c32_k48_pool", H // 2, W // 2, 32, 0, 48, True, False, False, True),
    ("c48_k64_pool", H // 4, W // 4, 48, 0, 64, True, False, False, True),
    ("c64_k80_pool_dual", H // 8, W // 8, 64, 0, 80, True, False, False, True),
    ("c80_k96", H // 16, W // 16, 80, 0, 96, True, False, False, False),
    ("c96_k96_small", H // 16, W // 16, 96, 0, 96, True, False, False, False),
    ("up96_cat80_k112", H // 8, W // 8, 96, 80, 112, True, False, True, False),
    ("c112_k112", H // 8, W // 8, 112, 0, 112, True, False, False, False),
    ("c64_k64_half", H // 2, W // 2, 64, 0, 64, True, False, False, False),
    ("c96_k96_leaky", H // 4, W // 4, 96, 0, 96, False, True, False, False),
    # the 9 channel network input read as it is (raw row bytes re-laid in shared memory)
    ("c9_k32_raw", H, W, 9, 0, 32, True, False, False, False),
    ("up64_cat9_k64_raw", H, W, 64, 9, 64, True, False, True, False),
]
LEAKY = {"c96_k96_leaky": 0.1}
# variants that must be among those that run a case (the ones the benchmark database picks there)
MUST_RUN = {"up96_cat80_k112": ["R=2#KG=2#W=stream3"], "c112_k112": ["DY=stack#KG=2#W=resident#NSPLIT=2"]}


def _tensor(seed, shape):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    return (torch.rand(shape, generator=g, device="cuda", dtype=torch.float32) * 2 - 1).to(torch.float16)


def _launch(variant, case, ta, tb, wt, tbias, full=True):
    name, h, w, ca, cb, k, relu, bias, up, pool = case
    d = lib.Dispatch()
    d.variant = variant
    d.flags = (lib.F_RELU if relu else 0) | (lib.F_BIAS if bias else 0) | (lib.F_UP2X_A if up else 0) | \
        (lib.F_POOL_OUT if pool else 0) | (0 if full else lib.F_NO_FULL_OUT) | (lib.F_LEAKY if name in LEAKY else 0)
    d.leaky_alpha = LEAKY.get(name, 0.0)
    d.pc[0], d.pc[1] = w, h
    d.c_a, d.c_b, d.c_out = ca, cb, k
    d.in_a = ta.data_ptr()
    d.in_b = tb.data_ptr() if tb is not None else None
    d.bias = tbias.data_ptr() if tbias is not None else None
    d.weights = 0x1000
    d.out = 0x1000 if full else None
    d.out_pool = 0x1000 if pool else None
    if lib.L.dnxcu_validate(C.byref(d)) != 0:
        return None
    tw = torch.from_numpy(lib.prepare_weights(variant, wt, ca, cb)).cuda()
    d.weights = tw.data_ptr()
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    d.device_status = status.data_ptr()
    out = Guarded((h, w, k)) if full else None
    outp = Guarded((h // 2, w // 2, k)) if pool else None
    d.out = out.ptr() if full else None
    d.out_pool = outp.ptr() if pool else None
    lib.check(lib.L.dnxcu_launch(C.byref(d), None))
    torch.cuda.synchronize()
    assert int(status[0].item()) == 0, f"bounded wait ran out, code {int(status[0].item())}"
    for gbuf in (out, outp):
        if gbuf is not None:
            b = gbuf.buf
            assert bool((b[:gbuf.pad] == 12345.0).all()) and bool((b[-gbuf.pad:] == 12345.0).all()), "canary damaged"
    return (out.view if full else None), (outp.view if pool else None)


def _within_ulps(got, ref, n):
    g, r = got.float(), ref.float()
    tol = torch.maximum(r.abs() * 2.0 ** -10, torch.full_like(r, 2.0 ** -14)) * (n + 0.01)
    return (g - r).abs() <= tol


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_fullsize_conv(case):
    name, h, w, ca, cb, k, relu, bias, up, pool = case
    seed = 7000 + sum(name.encode())
    ha, wa = (h // 2, w // 2) if up else (h, w)
    ta = _tensor(seed, (ha, wa, ca))
    tb = _tensor(seed + 1, (h, w, cb)) if cb else None
    wt = rng.he_normal_weights(seed + 2, k, ca + cb)
    bs = rng.to_f16(rng.uniform(seed + 3, k, -0.5, 0.5)) if bias else None
    tbias = torch.from_numpy(bs).cuda() if bias else None

    variants = lib.variants()
    direct = next(v["id"] for v in variants if v["op"] == lib.OP_CONV3X3 and not v["needs_tcgen05"])
    ref, _ = _launch(direct, case[:9] + (False,), ta, tb, wt, tbias)  # the pooled output is checked against the full one
    assert bool(torch.isfinite(ref).all())

    # the CUDA core kernel itself against the oracle on three bands of rows
    bands = [(0, 8), ((h // 2) & ~1, ((h // 2) & ~1) + 8), (h - 8, h)]
    for (r0, r1) in bands:
        c0, c1 = max(0, r0 - 2), min(h, r1 + 2)  # even: r0, r1 are
        a_np = (ta[c0 // 2:c1 // 2] if up else ta[c0:c1]).cpu().numpy()
        b_np = tb[c0:c1].cpu().numpy() if cb else None
        o = oracle.conv3x3(a_np, wt, bs, relu=relu, mode=oracle.ACC_F32, b=b_np, up_a=up, leaky=LEAKY.get(name))
        # rows whose window the crop cut are not comparable
        lo = 0 if c0 == 0 else 1
        hi = (c1 - c0) if c1 == h else (c1 - c0 - 1)
        got = ref[c0 + lo:c0 + hi]
        ok = _within_ulps(got, torch.from_numpy(o[lo:hi]).cuda(), 3 if name in LEAKY else 1)
        assert bool(ok.all()), (name, "direct kernel vs oracle rows", c0 + lo, c0 + hi, int((~ok).sum()))

    ran = []
    for v in variants:
        if v["op"] != lib.OP_CONV3X3 or not v["needs_tcgen05"]:
            continue
        res = _launch(v["id"], case, ta, tb, wt, tbias)
        if res is None:
            continue
        ran.append(v["config"])
        y, yp = res
        ok = _within_ulps(y, ref, 4 if name in LEAKY else 2)
        nbad = int((~ok).sum())
        assert nbad == 0, (name, v["config"], "elements off by more than two ulps", nbad,
                           float((y.float() - ref.float()).abs().max()))
        if pool:
            want = torch.maximum(torch.maximum(y[0::2, 0::2], y[0::2, 1::2]), torch.maximum(y[1::2, 0::2], y[1::2, 1::2]))
            assert bool((yp == want).all()), (name, v["config"], "pooled output is not the 2x2 max of the full output")
            # pooled output alone (the form the encoder layers run in): the same bits without the full tensor
            _, yp_only = _launch(v["id"], case, ta, tb, wt, tbias, full=False)
            assert bool((yp_only == yp).all()), (name, v["config"], "pooled-only output differs from the dual output form")
    assert ran, "no tensor core variant took this dispatch"
    for cfg in MUST_RUN.get(name, []):
        assert cfg in ran, (name, "variant did not take the dispatch", cfg, ran)


def test_fullsize_network_tensor_core_against_cuda_core():
    """The whole OIDN-style net at 1088 x 1920: tcgen05 schedule against the CUDA core schedule
    (|d| <= 2e-2 + 1e-2 |ref| per element, the benchmark's acceptance rule), and frame to frame
    determinism of the tcgen05 schedule."""
    net = nets.oidn_unet()
    x = nets.oidn_input(1005, H, W)
    m_tc = lib.Model(net)
    m_cc = lib.Model(net, options=lib.OPT_NO_TCGEN05)
    i_tc = lib.Instance(m_tc, H, W)
    i_cc = lib.Instance(m_cc, H, W)
    y = i_tc.infer(x)
    y2 = i_tc.infer(x)
    ref = i_cc.infer(x)
    assert np.isfinite(y.astype(np.float32)).all()
    assert (y.view(np.uint16) == y2.view(np.uint16)).all(), "two runs of the same frame differ"
    d = np.abs(y.astype(np.float32) - ref.astype(np.float32))
    bad = d > 2e-2 + 1e-2 * np.abs(ref.astype(np.float32))
    assert bad.mean() <= 1e-3, (float(bad.mean()), float(d.max()))
    for o in (i_tc, i_cc, m_tc, m_cc):
        o.close()


def test_fullsize_network_against_oracle_with_report():
    """The whole OIDN-style net at 1088 x 1920 against the CPU oracle itself: end to end (free running) with
    binary16 accumulation (the reference's arithmetic: at most 0.5 % of the elements outside the acceptance rule)
    and with fp32 accumulation (none outside), and every layer teacher forced (the oracle recomputes the layer
    from the GPU's own input tensors).  The table is written out as a report."""
    import parity_util
    net = nets.oidn_unet()
    x = nets.oidn_input(1006, H, W)
    model = lib.Model(net)
    inst = lib.Instance(model, H, W)
    y = inst.infer(x)
    rep = parity_util.report(net, x, inst, y)
    parity_util.save(rep, "parity_oidn_1088x1920")
    print(parity_util.to_markdown(rep, "OIDN-style U-Net 1088 x 1920"))
    e = rep["end_to_end"]
    assert e["acc=f32"]["violation_fraction"] == 0.0, e
    assert e["acc=f16"]["violation_fraction"] <= 5e-3, e
    for r in rep["layers"]:
        assert r["acc=f32"]["violation_fraction"] == 0.0, r
        assert r["acc=f16"]["violation_fraction"] <= 1e-3, r
        # one rounding apart from the fp32 oracle on identical inputs: a binary16 ulp of the largest activations
        assert r["acc=f32"]["max"] <= 0.05, r
    inst.close()
    model.close()


def test_small_network_report():
    """The same report for the CPU-runnable configuration (tiny U-Net, 128 x 128)."""
    import parity_util
    net = nets.tiny_unet()
    x = nets.tiny_input(1000, 128, 128)
    model = lib.Model(net)
    inst = lib.Instance(model, 128, 128)
    y = inst.infer(x)
    rep = parity_util.report(net, x, inst, y)
    parity_util.save(rep, "parity_tiny_128x128")
    assert rep["end_to_end"]["acc=f32"]["violation_fraction"] == 0.0
    assert rep["end_to_end"]["acc=f16"]["violation_fraction"] <= 1e-3
    assert len(rep["layers"]) >= 4
    inst.close()
    model.close()
