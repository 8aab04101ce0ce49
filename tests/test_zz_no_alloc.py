"""The allocation-free conv + pool entry point (collected last on purpose: a failure
here must not hide the result of any other test).

dnxcu_conv3x3_pool_static keeps its full resolution intermediate in a fixed
array inside the library, for hosts that may not call cudaMalloc while frames
are in flight.  It must give what the ordinary path gives: the fused
conv+relu+pool dispatch of the tensor core variant through dnxcu_launch."""
import ctypes as C

import numpy as np
import pytest

from denox_b200 import lib, rng
from oracle import oracle

pytestmark = pytest.mark.gpu


def _case(seed, h, w, c, k, bias):
    a = rng.to_f16(rng.uniform(seed, h * w * c, -1, 1)).reshape(h, w, c)
    wt = rng.he_normal_weights(seed + 1, k, c)
    bs = rng.to_f16(rng.uniform(seed + 2, k, -0.5, 0.5)) if bias else None
    return a, wt, bs


def _static(a, wt, bs):
    import torch
    from gpu_util import Guarded, dev
    h, w, c = a.shape
    k = wt.shape[0]
    ta, tw = dev(a), dev(lib.prepare_weights(0, wt, c))
    tb = dev(bs) if bs is not None else None
    out = Guarded((h // 2, w // 2, k))
    flags = lib.F_RELU | (lib.F_BIAS if bs is not None else 0)
    st = lib.L.dnxcu_conv3x3_pool_static(ta.data_ptr(), h, w, c, tw.data_ptr(), tb.data_ptr() if tb is not None else None,
                                         k, flags, out.ptr(), None)
    lib.check(st, "dnxcu_conv3x3_pool_static")
    torch.cuda.synchronize()
    return out.check()


def test_static_scratch_matches_fused_dispatch_twice_in_a_row():
    from gpu_util import run_conv
    fused_variant = lib.find_variant("direct-conv-tc", "R=2#KG=1#W=resident")
    # two calls in a row, different shapes: the second must not see the first one's leftovers
    for seed, (h, w, c, k, bias) in enumerate([(64, 96, 32, 32, True), (34, 50, 16, 24, False)]):
        a, wt, bs = _case(300 + 10 * seed, h, w, c, k, bias)
        got = _static(a, wt, bs)
        _, want = run_conv(fused_variant, a, wt, bs, relu=True, pool=True, full=False)
        g, r = got.astype(np.float32), want.astype(np.float32)
        # both accumulate in fp32 and round once; the summation order differs: one binary16 ulp
        assert (np.abs(g - r) <= np.maximum(np.abs(r) * 2.0 ** -10, 2.0 ** -14) * 1.01).all()
        assert np.isfinite(g).all()
        # and against the CPU oracle (conv + ReLU, then 2x2 max pool), the same bound
        o = oracle.maxpool2x2(oracle.conv3x3(a, wt, bs, relu=True, mode=oracle.ACC_F32)).astype(np.float32)
        assert (np.abs(g - o) <= np.maximum(np.abs(o) * 2.0 ** -10, 2.0 ** -14) * 1.01).all()


def test_static_scratch_rejects_oversized_and_bad_arguments():
    import torch
    x = torch.zeros(16, dtype=torch.float16, device="cuda")
    p = x.data_ptr()
    f = lib.L.dnxcu_conv3x3_pool_static
    # 2048 x 2048 x 64 halves is far beyond the fixed array
    assert f(p, 2048, 2048, 8, p, None, 64, 0, p, None) == lib.E_LIMIT
    assert f(p, 15, 16, 8, p, None, 8, 0, p, None) == lib.E_BAD_ARG          # odd height
    assert f(p, 16, 16, 8, p, None, 8, lib.F_BIAS, p, None) == lib.E_BAD_ARG  # bias flag without bias
    assert f(p, 16, 16, 8, p, None, 8, lib.F_POOL_OUT, p, None) == lib.E_BAD_ARG
    assert f(None, 16, 16, 8, p, None, 8, 0, p, None) == lib.E_BAD_ARG
