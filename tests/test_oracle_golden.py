"""The CPU oracle against the PyTorch generated golden fixtures (tolerance of the
reference's own tests: allclose(rtol=1e-3, atol=1e-2), test/__init__.py:48-49)."""
import importlib.util
import os

import numpy as np
import pytest

from denox_b200 import nets
from oracle import oracle

HERE = os.path.dirname(os.path.abspath(__file__))
spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_golden.py"))
mg = importlib.util.module_from_spec(spec)
spec.loader.exec_module(mg)
GOLD = np.load(os.path.join(HERE, "golden", "golden.npz"))


def ref_allclose(got, ref, rtol=1e-3, atol=1e-2):
    g, r = got.astype(np.float32), ref.astype(np.float32)
    return np.abs(g - r) <= atol + rtol * np.abs(r)


@pytest.mark.parametrize("case", mg.CONV_CASES, ids=[c[0] for c in mg.CONV_CASES])
def test_conv_f32_matches_torch(case):
    name, h, w, ca, cb, k, relu, bias, up = case
    a, b, wt, bs = mg.conv_case_tensors(case)
    y = oracle.conv3x3(a, wt, bs, relu=relu, mode=oracle.ACC_F32, b=b, up_a=up)
    ref = GOLD["conv/" + name]
    assert y.shape == ref.shape == (h, w, k)
    # fp32 accumulation in a different order than PyTorch: at most one binary16 ulp apart
    d = np.abs(y.astype(np.float32) - ref.astype(np.float32))
    assert ref_allclose(y, ref).all()
    assert (d <= np.maximum(np.abs(ref.astype(np.float32)) * 2.0 ** -10, 2.0 ** -14)).all()


@pytest.mark.parametrize("case", mg.CONV_CASES, ids=[c[0] for c in mg.CONV_CASES])
@pytest.mark.parametrize("mode", [oracle.ACC_F16, oracle.ACC_F16_FMA])
def test_conv_f16_accumulation_within_reference_tolerance(case, mode):
    """The reference's own arithmetic (binary16 accumulation, direct_conv.comp:481-543)
    stays inside the benchmark's acceptance band |d| <= 2e-2 + 1e-2 |ref| around the
    PyTorch result on these shapes (its error grows with the reduction length)."""
    name, h, w, ca, cb, k, relu, bias, up = case
    a, b, wt, bs = mg.conv_case_tensors(case)
    y = oracle.conv3x3(a, wt, bs, relu=relu, mode=mode, b=b, up_a=up)
    ref = GOLD["conv/" + name]
    ok = ref_allclose(y, ref, rtol=1e-2, atol=2e-2)
    assert ok.mean() > 0.999, (name, float(1 - ok.mean()))


@pytest.mark.parametrize("case", mg.CONV_CASES2, ids=[c[0] for c in mg.CONV_CASES2])
def test_more_shapes_and_leaky_relu_match_torch(case):
    """The remaining channel pairs of the reference's conv test list (up to 256 -> 256) and LeakyReLU epilogues."""
    name, h, w, ca, cb, k, relu, bias, up, leaky = case
    a, b, wt, bs = mg.conv_case_tensors(case)
    ref = GOLD["conv/" + name]
    y = oracle.conv3x3(a, wt, bs, relu=relu, mode=oracle.ACC_F32, b=b, up_a=up, leaky=leaky)
    assert y.shape == ref.shape == (h, w, k)
    assert ref_allclose(y, ref).all()
    d = np.abs(y.astype(np.float32) - ref.astype(np.float32))
    # PyTorch applies the slope to the fp32 sum, the oracle (like the reference) to the rounded sum: two ulps
    ulps = 2.0 if leaky is not None else 1.0
    assert (d <= ulps * np.maximum(np.abs(ref.astype(np.float32)) * 2.0 ** -10, 2.0 ** -14)).all()
    # binary16 accumulation: the reference's own tests relax to atol = 1e-1 at 256 channels (test_conv.py:113-123)
    y16 = oracle.conv3x3(a, wt, bs, relu=relu, mode=oracle.ACC_F16, b=b, up_a=up, leaky=leaky)
    if ca + cb >= 256:
        assert ref_allclose(y16, ref, rtol=0.0, atol=1e-1).all()
    else:
        assert ref_allclose(y16, ref, rtol=1e-2, atol=2e-2).mean() > 0.995, name


def test_leaky_relu_standalone_and_zero_signs():
    xs = mg.rng.to_f16(mg.rng.uniform(9100, 12 * 20 * 24, -8.0, 8.0)).reshape(12, 20, 24)
    y = oracle.leaky_relu(xs, 0.3)
    assert ref_allclose(y, GOLD["leaky/standalone_c24"], rtol=1e-3, atol=1e-4).all()
    z = np.array([0.0, -0.0, -6e-8, 1.0, -1.0], dtype=np.float16)
    got = oracle.leaky_relu(z, 0.1).view(np.uint16)
    # +0 stays +0, -0 stays -0, a product that underflows becomes -0, negative values scale
    assert list(got[:3]) == [0x0000, 0x8000, 0x8000] and got[3] == np.float16(1.0).view(np.uint16)
    assert oracle.leaky_relu(z, 0.1)[4] == np.float16(-0.1)


def test_tiny_net_with_leaky_relu_matches_torch():
    net = nets.tiny_unet(leaky=0.1)
    x = nets.tiny_input(1003, 32, 48)
    y = oracle.run_network(net, x, oracle.ACC_F32)[net.output_tensor]
    assert ref_allclose(y, GOLD["tiny_leaky/out"]).all()


@pytest.mark.parametrize("key,seed,shape", [("ref_unet_32x48/out", 1010, (32, 48)), ("ref_unet_40x52/out", 1011, (40, 52))])
def test_reference_model_file_output(key, seed, shape):
    """The oracle against the output of the reference's own PyTorch module (oidn_model.py UNet + UNetAlignment,
    run in binary16 when the fixture was made), its channel list (first decoder conv 160 = 96 + 64), biases on,
    an aligned and an unaligned extent."""
    net = nets.oidn_unet_reference()
    x = nets.oidn_input(seed, *shape)
    ref = GOLD[key]
    y32 = oracle.run_network_aligned(net, x, 16, oracle.ACC_F32)
    assert y32.shape == ref.shape == shape + (3,)
    assert ref_allclose(y32, ref).all()           # the reference's own test tolerance (test/__init__.py:48-49)
    y16 = oracle.run_network_aligned(net, x, 16, oracle.ACC_F16)
    assert ref_allclose(y16, ref, rtol=1e-2, atol=2e-2).mean() > 0.9  # 16 layers of binary16 accumulation drift


def test_concat_phase_order_equals_explicit_concat_in_f32():
    case = next(c for c in mg.CONV_CASES if c[0] == "cat32_16_k16")
    a, b, wt, bs = mg.conv_case_tensors(case)
    fused = oracle.conv3x3(a, wt, bs, relu=True, b=b, up_a=True)
    explicit = oracle.conv3x3(oracle.concat(oracle.upsample2x(a), b), wt, bs, relu=True)
    d = np.abs(fused.astype(np.float32) - explicit.astype(np.float32))
    assert (d <= np.abs(explicit.astype(np.float32)) * 2.0 ** -10 + 2.0 ** -14).all()


def test_pool_upsample_concat_relu_small():
    rs = np.random.RandomState(1)
    x = rs.randn(6, 10, 5).astype(np.float16)
    p = oracle.maxpool2x2(x)
    ref = x.reshape(3, 2, 5, 2, 5).max(axis=(1, 3))
    assert (p == ref).all()
    assert (oracle.maxpool2x2(rs.randn(7, 9, 3).astype(np.float16)).shape == (3, 4, 3))  # floor size
    u = oracle.upsample2x(x)
    assert (u == np.repeat(np.repeat(x, 2, 0), 2, 1)).all()
    y = rs.randn(6, 10, 3).astype(np.float16)
    assert (oracle.concat(x, y) == np.concatenate([x, y], 2)).all()
    assert (oracle.relu(x) == np.maximum(x, np.float16(0))).all()


def test_halo_rows_equal_taller_image():
    """A row band with halo rows computes exactly the rows of the whole image."""
    case = next(c for c in mg.CONV_CASES if c[0] == "c32_k32")
    a, _, wt, bs = mg.conv_case_tensors(case)
    full = oracle.conv3x3(a, wt, bs, relu=True)
    band = oracle.conv3x3(a[8:16], wt, bs, relu=True, halo=(a[7], a[16], None, None))
    assert (band == full[8:16]).all()
    top = oracle.conv3x3(a[:8], wt, bs, relu=True, halo=(None, a[8], None, None))
    assert (top == full[:8]).all()


def test_f32_to_f16_truncation_matches_reference_rule():
    x = np.array([1.0, 1.0009765625 + 2 ** -12, -2.5, 6.0e-8, 1e6, 65504.0, 3.0e-5], dtype=np.float32)
    h = oracle.f32_to_f16_trunc(x).view(np.float16)
    assert h[0] == 1.0 and h[1] == np.float16(1.0009765625) and h[2] == -2.5
    assert h[3] == 0.0 and np.isinf(h[4]) and h[5] == 65504.0 and h[6] == 0.0  # sub-normals flush to zero


@pytest.mark.parametrize("key,net,shape,seed", [
    ("tiny/out", "tiny", (128, 128), 1000),
    ("tiny_bias/out", "tiny_bias", (48, 80), 1001),
    ("oidn_32x48/out", "oidn", (32, 48), 1000),
])
def test_networks_match_torch(key, net, shape, seed):
    if net == "oidn":
        n, x = nets.oidn_unet(), nets.oidn_input(seed, *shape)
    else:
        n, x = nets.tiny_unet(bias=(net == "tiny_bias")), nets.tiny_input(seed, *shape)
    t = oracle.run_network(n, x, oracle.ACC_F32)
    assert ref_allclose(t[n.output_tensor], GOLD[key]).all()
    t16 = oracle.run_network(n, x, oracle.ACC_F16)
    assert ref_allclose(t16[n.output_tensor], GOLD[key], rtol=1e-2, atol=2e-2).mean() > 0.999


def test_oidn_intermediates_match_torch():
    n, x = nets.oidn_unet(), nets.oidn_input(1000, 32, 48)
    t = oracle.run_network(n, x, oracle.ACC_F32)
    for name in ("enc_conv1", "enc_conv4", "dec_conv4a", "dec_conv1a"):
        nd = next(q for q in n.nodes if q.name == name + ".relu")
        assert ref_allclose(t[nd.out], GOLD[f"oidn_32x48/{name}"]).all(), name


@pytest.mark.parametrize("case", mg.PAD_CASES, ids=[c[0] for c in mg.PAD_CASES])
def test_pad_edge_and_slice_match_torch_bit_exact(case):
    name, h, w, c, l, r, t, b = case
    x = mg.pad_case_input(case)
    y = oracle.pad_edge(x, l, r, t, b)
    ref = GOLD["pad/" + name]
    assert y.shape == ref.shape == (h + t + b, w + l + r, c)
    assert (y.view(np.uint16) == ref.view(np.uint16)).all()
    back = oracle.slice_hw(y, l, t, h, w)
    assert (back.view(np.uint16) == x.view(np.uint16)).all()


def test_aligned_network_matches_torch():
    """OIDN-style net on a 40 x 52 frame behind the alignment wrapper (pad to 48 x 64, run, slice)."""
    net = nets.oidn_unet()
    x = nets.oidn_input(1002, 40, 52)
    y = oracle.run_network_aligned(net, x)
    ref = GOLD["oidn_40x52_aligned/out"]
    assert y.shape == ref.shape == (40, 52, 3)
    assert ref_allclose(y, ref).all()
