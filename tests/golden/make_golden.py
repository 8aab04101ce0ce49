"""Generates the golden fixtures of tests/golden/ with PyTorch on CPU.

The reference's own tests define correctness as agreement with PyTorch's
forward pass (test/__init__.py:84-97 of the reference: conv / relu / max_pool2d
/ interpolate(nearest) / cat), so PyTorch is the generator here.  Convolutions
are evaluated in float32 on binary16 inputs and rounded to binary16 after every
layer.  Inputs and weights come from denox_b200.rng (seeded), so only outputs
are stored.

    DENOX_REFERENCE=<checkout of kistenklaus/denox> python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from denox_b200 import nets, rng  # noqa: E402

CONV, RELU, MAXPOOL, UPSAMPLE, CONCAT, LEAKY_RELU = 1, 2, 3, 4, 5, 6
# checkout of the reference project (its oidn_model.py is executed for the ref_unet_* fixtures); without it those
# fixtures are carried over from the existing golden.npz
REFERENCE_ROOT = os.environ.get("DENOX_REFERENCE", "")


def t_in(x):  # HWC binary16 -> 1CHW float32
    return torch.from_numpy(np.asarray(x, dtype=np.float32)).permute(2, 0, 1)[None]


def t_out(y):  # 1CHW float32 -> HWC binary16
    return y[0].permute(1, 2, 0).contiguous().numpy().astype(np.float16)


def run_torch(net, x):
    t = {net.input_tensor: t_in(x)}
    half = lambda v: v.half().float()  # one rounding to binary16 per layer
    for nd in net.nodes:
        if nd.kind == CONV:
            w = torch.from_numpy(nd.weights.astype(np.float32))
            b = None if nd.bias is None else torch.from_numpy(nd.bias.astype(np.float32))
            t[nd.out] = half(F.conv2d(t[nd.in0], w, b, padding=1))
        elif nd.kind == RELU:
            t[nd.out] = F.relu(t[nd.in0])
        elif nd.kind == LEAKY_RELU:
            t[nd.out] = half(F.leaky_relu(t[nd.in0], nd.alpha))
        elif nd.kind == MAXPOOL:
            t[nd.out] = F.max_pool2d(t[nd.in0], 2, 2)
        elif nd.kind == UPSAMPLE:
            t[nd.out] = F.interpolate(t[nd.in0], scale_factor=2, mode="nearest")
        elif nd.kind == CONCAT:
            t[nd.out] = torch.cat((t[nd.in0], t[nd.in1]), 1)
    return {k: t_out(v) for k, v in t.items()}


# (name, H, W, Ca, Cb, K, relu, bias, up_a): single layer cases; channel counts follow
# the reference's test list (test/system/test_conv.py) and the benchmark networks
CONV_CASES = [
    ("c3_k16", 20, 36, 3, 0, 16, True, False, False),
    ("c9_k32", 16, 40, 9, 0, 32, True, False, False),
    ("c32_k32", 24, 150, 32, 0, 32, True, True, False),
    ("c16_k3", 18, 34, 16, 0, 3, False, False, False),
    ("c67_k24", 10, 22, 67, 0, 24, True, True, False),
    ("c48_k64", 12, 20, 48, 0, 64, True, False, False),
    ("cat32_16_k16", 16, 32, 32, 16, 16, True, False, True),
    ("cat96_80_k112", 8, 16, 96, 80, 112, True, False, True),
    ("cat64_9_k64", 12, 140, 64, 9, 64, True, False, True),
    ("cat16_8_k8", 10, 12, 16, 8, 8, False, True, False),
]


# More single layer cases, same tuple plus the LeakyReLU slope (None: the `relu` field decides).  The channel
# pairs not covered above from the reference's list (test/system/test_conv.py:9-502: 3->3, 8->16, 16->8, 24->24,
# 128->128, 160->112, 112->112, 160->96, 256->256, all with nn.Conv2d's default bias) at small extents, and
# LeakyReLU epilogues (onnx LeakyRelu, frontend/onnx/details/ops/leaky_relu.cpp).
CONV_CASES2 = [
    ("r3_k3", 14, 20, 3, 0, 3, False, True, False, None),
    ("r8_k16", 12, 24, 8, 0, 16, False, True, False, None),
    ("r16_k8", 12, 24, 16, 0, 8, False, True, False, None),
    ("r24_k24", 10, 18, 24, 0, 24, False, True, False, None),
    ("r128_k128", 8, 20, 128, 0, 128, False, True, False, None),
    ("r160_k112", 8, 16, 160, 0, 112, False, True, False, None),
    ("r112_k112", 8, 16, 112, 0, 112, False, True, False, None),
    ("r160_k96", 8, 16, 160, 0, 96, False, True, False, None),
    ("r256_k256", 6, 20, 256, 0, 256, False, True, False, None),
    ("leaky_c32_k32", 16, 40, 32, 0, 32, False, True, False, 0.1),
    ("leaky_cat32_16_k16", 16, 32, 32, 16, 16, False, False, True, 0.2),
    ("leaky_c9_k24", 10, 22, 9, 0, 24, False, False, False, 0.01),
]


def conv_case_tensors(case):
    name, h, w, ca, cb, k, relu, bias, up = case[:9]
    seed = 5000 + sum(name.encode())
    ha, wa = (h // 2, w // 2) if up else (h, w)
    a = rng.to_f16(rng.uniform(seed, ha * wa * ca, -1.0, 1.0)).reshape(ha, wa, ca)
    b = rng.to_f16(rng.uniform(seed + 1, h * w * cb, -1.0, 1.0)).reshape(h, w, cb) if cb else None
    wt = rng.he_normal_weights(seed + 2, k, ca + cb)
    bs = rng.to_f16(rng.uniform(seed + 3, k, -0.5, 0.5)) if bias else None
    return a, b, wt, bs


def conv_case_torch(case):
    name, h, w, ca, cb, k, relu, bias, up = case[:9]
    leaky = case[9] if len(case) > 9 else None
    a, b, wt, bs = conv_case_tensors(case)
    x = t_in(a)
    if up:
        x = F.interpolate(x, scale_factor=2, mode="nearest")
    if b is not None:
        x = torch.cat((x, t_in(b)), 1)
    y = F.conv2d(x, torch.from_numpy(wt.astype(np.float32)),
                 None if bs is None else torch.from_numpy(bs.astype(np.float32)), padding=1)
    if relu:
        y = F.relu(y)
    if leaky is not None:
        y = F.leaky_relu(y, leaky)
    return t_out(y)


def load_reference_unet():
    """UNet and UNetAlignment as the reference's own model file defines them (oidn_model.py:206-347).  That file
    is a script: below its definitions it loads a weight archive and an image and runs on CUDA.  Only its import,
    def and class statements are executed here (imports of packages that are absent here are dropped)."""
    import ast
    src = open(os.path.join(REFERENCE_ROOT, "oidn_model.py")).read()
    absent = ("torchvision", "PIL")

    def wanted(node):
        if isinstance(node, ast.ImportFrom):
            return (node.module or "").split(".")[0] not in absent
        if isinstance(node, ast.Import):
            return not any(a.name.split(".")[0] in absent for a in node.names)
        return isinstance(node, (ast.FunctionDef, ast.ClassDef))

    tree = ast.parse(src)
    mod = ast.Module(body=[nd for nd in tree.body if wanted(nd)], type_ignores=[])
    ns = {}
    exec(compile(mod, "oidn_model.py", "exec"), ns)
    return ns["UNet"], ns["UNetAlignment"]


def run_reference_unet(net, x):
    """Runs the reference's own PyTorch module (binary16, as the reference runs it) with the weights and biases of
    `net` (denox_b200.nets.oidn_unet_reference) on the HWC frame x; the UNetAlignment wrapper pads and slices."""
    UNet, UNetAlignment = load_reference_unet()
    model = UNetAlignment(UNet(net.in_channels, net.channels[net.output_tensor], False)).to(torch.float16).eval()
    with torch.no_grad():
        for nd in net.nodes:
            if nd.kind != CONV:
                continue
            conv = getattr(model.net, nd.name)
            assert tuple(conv.weight.shape) == nd.weights.shape, (nd.name, conv.weight.shape, nd.weights.shape)
            conv.weight.copy_(torch.from_numpy(nd.weights))
            conv.bias.copy_(torch.from_numpy(nd.bias) if nd.bias is not None else torch.zeros_like(conv.bias))
        xin = torch.from_numpy(np.ascontiguousarray(x)).permute(2, 0, 1)[None]
        y = model(xin)
    return y[0].permute(1, 2, 0).contiguous().numpy()


# (name, H, W, C, left, right, top, bottom): spatial pads (torch: F.pad(mode="replicate")) and the slices that undo them
PAD_CASES = [
    ("c3", 5, 7, 3, 0, 9, 0, 11),
    ("c9", 13, 10, 9, 0, 6, 0, 3),
    ("c8", 6, 20, 8, 2, 1, 3, 0),
    ("c32", 17, 33, 32, 0, 15, 0, 15),
]


def pad_case_input(case):
    name, h, w, c = case[:4]
    return rng.to_f16(rng.uniform(8000 + sum(name.encode()), h * w * c, -4.0, 4.0)).reshape(h, w, c)


def run_torch_aligned(net, x, alignment=16):
    """The reference's alignment wrapper (oidn_model.py:334-347): replicate pad right / bottom, net, slice."""
    h, w = x.shape[:2]
    ph, pw = (-h) % alignment, (-w) % alignment
    xp = t_out(F.pad(t_in(x), (0, pw, 0, ph), mode="replicate"))
    return run_torch(net, xp)[net.output_tensor][:h, :w].copy()


def main():
    torch.set_num_threads(4)
    out = {}
    for case in CONV_CASES:
        out["conv/" + case[0]] = conv_case_torch(case)
    tiny = nets.tiny_unet()
    res = run_torch(tiny, nets.tiny_input(1000, 128, 128))
    out["tiny/out"] = res[tiny.output_tensor]
    tinyb = nets.tiny_unet(bias=True)
    res = run_torch(tinyb, nets.tiny_input(1001, 48, 80))
    out["tiny_bias/out"] = res[tinyb.output_tensor]
    oidn = nets.oidn_unet()
    res = run_torch(oidn, nets.oidn_input(1000, 32, 48))
    out["oidn_32x48/out"] = res[oidn.output_tensor]
    for name in ("enc_conv1", "enc_conv4", "dec_conv4a", "dec_conv1a"):
        nd = next(n for n in oidn.nodes if n.name == name + ".relu")
        out[f"oidn_32x48/{name}"] = res[nd.out]
    for case in PAD_CASES:
        name, h, w, c, l, r, t, b = case
        out["pad/" + name] = t_out(F.pad(t_in(pad_case_input(case)), (l, r, t, b), mode="replicate"))
    out["oidn_40x52_aligned/out"] = run_torch_aligned(oidn, nets.oidn_input(1002, 40, 52))
    for case in CONV_CASES2:
        out["conv/" + case[0]] = conv_case_torch(case)
    tinyl = nets.tiny_unet(leaky=0.1)
    res = run_torch(tinyl, nets.tiny_input(1003, 32, 48))
    out["tiny_leaky/out"] = res[tinyl.output_tensor]
    xs = rng.to_f16(rng.uniform(9100, 12 * 20 * 24, -8.0, 8.0)).reshape(12, 20, 24)
    out["leaky/standalone_c24"] = t_out(F.leaky_relu(t_in(xs), 0.3))
    # the reference's own PyTorch module, run here, with seeded weights: an aligned and an unaligned extent
    if REFERENCE_ROOT and os.path.exists(os.path.join(REFERENCE_ROOT, "oidn_model.py")):
        ref_net = nets.oidn_unet_reference()
        out["ref_unet_32x48/out"] = run_reference_unet(ref_net, nets.oidn_input(1010, 32, 48))
        out["ref_unet_40x52/out"] = run_reference_unet(ref_net, nets.oidn_input(1011, 40, 52))
    else:  # keep what an earlier run generated from the reference
        old = np.load(os.path.join(HERE, "golden.npz"))
        for k in ("ref_unet_32x48/out", "ref_unet_40x52/out"):
            out[k] = old[k]
    path = os.path.join(HERE, "golden.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes", len(out), "arrays")


if __name__ == "__main__":
    main()
