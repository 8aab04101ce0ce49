"""The benchmark networks as un-fused node lists (what an ONNX import yields:
Conv, Relu, MaxPool, Resize-nearest-2x, Concat), with seeded weights.

tiny_unet: the CPU-runnable configuration (128x128x3 input).
oidn_unet: the OIDN-style U-Net (oidn_model.py:231-331 of the reference for
the op order; channel counts as the benchmark configuration lists them: the
level-4 skip is the un-pooled 80 channel tensor, the others are pooled tensors
and the network input).
"""
from dataclasses import dataclass, field
from typing import List, Optional

import numpy as np

from . import rng

CONV, RELU, MAXPOOL, UPSAMPLE, CONCAT, LEAKY_RELU = 1, 2, 3, 4, 5, 6


@dataclass
class Node:
    kind: int
    in0: int
    out: int
    in1: int = -1
    c_out: int = 0
    weights: Optional[np.ndarray] = None  # [c_out][c_in][3][3] binary16
    bias: Optional[np.ndarray] = None     # [c_out] binary16
    name: str = ""
    alpha: float = 0.0                    # slope of a LEAKY_RELU node


@dataclass
class Net:
    name: str
    in_channels: int
    nodes: List[Node] = field(default_factory=list)
    n_tensors: int = 1
    input_tensor: int = 0
    output_tensor: int = 0
    channels: List[int] = field(default_factory=list)
    _wseed: int = 2000

    def _new(self, c):
        self.channels.append(c)
        self.n_tensors = len(self.channels)
        return self.n_tensors - 1

    def conv(self, x, c_out, relu=True, bias_seed=None, name="", leaky=None):
        """conv3x3 followed by ReLU (relu=True), by LeakyReLU with slope `leaky`, or by nothing."""
        c_in = self.channels[x]
        w = rng.he_normal_weights(self._wseed, c_out, c_in)
        b = None
        if bias_seed is not None:
            b = rng.to_f16(rng.uniform(bias_seed, c_out, -0.1, 0.1))
        self._wseed += 1
        y = self._new(c_out)
        self.nodes.append(Node(CONV, x, y, c_out=c_out, weights=w, bias=b, name=name))
        if leaky is not None:
            z = self._new(c_out)
            self.nodes.append(Node(LEAKY_RELU, y, z, name=name + ".leaky", alpha=float(leaky)))
            return z
        if relu:
            z = self._new(c_out)
            self.nodes.append(Node(RELU, y, z, name=name + ".relu"))
            return z
        return y

    def pool(self, x, name=""):
        y = self._new(self.channels[x])
        self.nodes.append(Node(MAXPOOL, x, y, name=name))
        return y

    def upsample(self, x, name=""):
        y = self._new(self.channels[x])
        self.nodes.append(Node(UPSAMPLE, x, y, name=name))
        return y

    def concat(self, a, b, name=""):
        y = self._new(self.channels[a] + self.channels[b])
        self.nodes.append(Node(CONCAT, a, y, in1=b, name=name))
        return y


def _start(name, c_in):
    net = Net(name, c_in)
    net.channels = [c_in]
    net.n_tensors = 1
    return net


def tiny_unet(bias=False, leaky=None) -> Net:
    """leaky: slope of a LeakyReLU that takes the place of every ReLU."""
    n = _start("tiny-unet", 3)
    bs = (lambda i: 3000 + i) if bias else (lambda i: None)
    x = n.conv(0, 16, name="conv0", bias_seed=bs(0), leaky=leaky)
    p = n.pool(x, "pool0")
    y = n.conv(p, 32, name="conv1", bias_seed=bs(1), leaky=leaky)
    u = n.upsample(y, "up0")
    c = n.concat(u, x, "cat0")
    z = n.conv(c, 16, name="conv2", bias_seed=bs(2), leaky=leaky)
    o = n.conv(z, 3, relu=False, name="conv3", bias_seed=bs(3))
    n.output_tensor = o
    return n


def oidn_unet() -> Net:
    n = _start("oidn-unet", 9)
    x = n.conv(0, 32, name="enc_conv0")
    x = n.conv(x, 32, name="enc_conv1")
    pool1 = n.pool(x, "pool1")
    x = n.conv(pool1, 48, name="enc_conv2")
    pool2 = n.pool(x, "pool2")
    x = n.conv(pool2, 64, name="enc_conv3")
    pool3 = n.pool(x, "pool3")
    enc4 = n.conv(pool3, 80, name="enc_conv4")
    x = n.pool(enc4, "pool4")
    x = n.conv(x, 96, name="enc_conv5a")
    x = n.conv(x, 96, name="enc_conv5b")
    x = n.concat(n.upsample(x, "upsample4"), enc4, "concat4")     # 96 + 80 = 176
    x = n.conv(x, 112, name="dec_conv4a")
    x = n.conv(x, 112, name="dec_conv4b")
    x = n.concat(n.upsample(x, "upsample3"), pool2, "concat3")    # 112 + 48 = 160
    x = n.conv(x, 96, name="dec_conv3a")
    x = n.conv(x, 96, name="dec_conv3b")
    x = n.concat(n.upsample(x, "upsample2"), pool1, "concat2")    # 96 + 32 = 128
    x = n.conv(x, 64, name="dec_conv2a")
    x = n.conv(x, 64, name="dec_conv2b")
    x = n.concat(n.upsample(x, "upsample1"), 0, "concat1")        # 64 + 9 = 73
    x = n.conv(x, 64, name="dec_conv1a")
    x = n.conv(x, 32, name="dec_conv1b")
    x = n.conv(x, 3, relu=False, name="dec_conv0")
    n.output_tensor = x
    return n


def oidn_unet_reference(in_channels: int = 9, out_channels: int = 3, wseed: int = 2100, bias: bool = True) -> Net:
    """The U-Net exactly as the reference's own model file builds it (oidn_model.py:206-331, the large
    configuration): every skip is a pooled tensor or the input, so the first decoder conv takes
    96 + 64 = 160 channels (pool3 is the level-4 skip), where the benchmark configuration's list says
    96 + 80 = 176.  Conv names are the module names of that file; its convs carry a bias (nn.Conv2d default)."""
    n = _start("oidn-unet-reference", in_channels)
    n._wseed = wseed
    nb = [0]

    def conv(x, c, name, relu=True):
        nb[0] += 1
        return n.conv(x, c, relu=relu, name=name, bias_seed=(4000 + nb[0]) if bias else None)

    x = conv(0, 32, "enc_conv0")
    x = conv(x, 32, "enc_conv1")
    pool1 = n.pool(x, "pool1")
    x = conv(pool1, 48, "enc_conv2")
    pool2 = n.pool(x, "pool2")
    x = conv(pool2, 64, "enc_conv3")
    pool3 = n.pool(x, "pool3")
    x = conv(pool3, 80, "enc_conv4")
    x = n.pool(x, "pool4")
    x = conv(x, 96, "enc_conv5a")
    x = conv(x, 96, "enc_conv5b")
    x = n.concat(n.upsample(x, "upsample4"), pool3, "concat4")    # 96 + 64 = 160
    x = conv(x, 112, "dec_conv4a")
    x = conv(x, 112, "dec_conv4b")
    x = n.concat(n.upsample(x, "upsample3"), pool2, "concat3")    # 112 + 48 = 160
    x = conv(x, 96, "dec_conv3a")
    x = conv(x, 96, "dec_conv3b")
    x = n.concat(n.upsample(x, "upsample2"), pool1, "concat2")    # 96 + 32 = 128
    x = conv(x, 64, "dec_conv2a")
    x = conv(x, 64, "dec_conv2b")
    x = n.concat(n.upsample(x, "upsample1"), 0, "concat1")        # 64 + in_channels
    x = conv(x, 64, "dec_conv1a")
    x = conv(x, 32, "dec_conv1b")
    x = conv(x, out_channels, "dec_conv0", relu=False)
    n.output_tensor = x
    return n


def tiny_input(seed: int = 1000, h: int = 128, w: int = 128) -> np.ndarray:
    """H x W x 3 binary16, uniform [0, 1)."""
    return rng.to_f16(rng.uniform(seed, h * w * 3)).reshape(h, w, 3)


def oidn_input(seed: int = 1000, h: int = 1088, w: int = 1920) -> np.ndarray:
    """H x W x 9 binary16: colour and albedo uniform [0, 1), normal uniform [-1, 1)."""
    u = rng.uniform(seed, h * w * 9).reshape(h, w, 9)
    u[:, :, 6:9] = u[:, :, 6:9] * 2.0 - 1.0
    return rng.to_f16(u)


def oidn_input_torch(seed: int = 1000, h: int = 1088, w: int = 1920, device="cuda"):
    """oidn_input generated on `device` with torch: the same bits (see rng.uniform_torch), in a fraction of the time."""
    import torch
    u = rng.uniform_torch(seed, h * w * 9, device=device).reshape(h, w, 9)
    u[:, :, 6:9] = u[:, :, 6:9] * 2.0 - 1.0
    return u.to(torch.float32).to(torch.float16)


def total_flops(net: Net, h: int, w: int) -> int:
    """2 H W 9 C K summed over the convs, at each conv's own resolution."""
    level = {0: 0}
    flops = 0
    for nd in net.nodes:
        lv = level[nd.in0]
        if nd.kind == MAXPOOL:
            lv += 1
        elif nd.kind == UPSAMPLE:
            lv -= 1
        level[nd.out] = lv
        if nd.kind == CONV:
            flops += 2 * (h >> lv) * (w >> lv) * 9 * net.channels[nd.in0] * nd.c_out
    return flops
