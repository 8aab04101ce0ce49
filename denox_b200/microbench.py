"""Layer microbenchmark at 1920 x 1088 (binary16 HWC, seeded He-normal weights).

    python -m denox_b200.microbench [--variants all|best] [--iters N] [--json FILE]

Cases: conv3x3+ReLU for (C_in, C_out) in {(9,32), (32,32), (64,64), (96,96),
(176,112)}, conv+ReLU+2x2 max pool in the epilogue at (32,32), and the 2x
upsample + concat prologue conv (96 at half resolution + 64 -> 96).  Each case
is timed with CUDA events (median of `iters` launches after warm-up; the
tensors of one launch exceed the L2, so consecutive launches do not hit in
cache) and reported against the tensor and HBM roofs: algorithmic flops
2 H W 9 C K and bytes 2 H W (C + K) + 18 C K, counting only tensors that cross
HBM for the fused forms.
"""
import argparse
import ctypes as C
import json
import os
import sys

import numpy as np
import torch

from . import lib, rng

H, W = 1088, 1920
CASES = [
    # name, c_a, c_b, k, flags
    ("conv 9->32 +relu", 9, 0, 32, lib.F_RELU),
    ("conv 16->32 +relu", 16, 0, 32, lib.F_RELU),
    ("conv 32->32 +relu", 32, 0, 32, lib.F_RELU),
    ("conv 64->64 +relu", 64, 0, 64, lib.F_RELU),
    ("conv 96->96 +relu", 96, 0, 96, lib.F_RELU),
    ("conv 176->112 +relu", 176, 0, 112, lib.F_RELU),
    ("conv 32->32 +relu +pool (pooled only)", 32, 0, 32, lib.F_RELU | lib.F_POOL_OUT | lib.F_NO_FULL_OUT),
    ("conv 32->32 +relu +pool (dual)", 32, 0, 32, lib.F_RELU | lib.F_POOL_OUT),
    ("up2x(96)+concat(64) -> 96 +relu", 96, 64, 96, lib.F_RELU | lib.F_UP2X_A),
    ("concat(64, 9) up2x -> 64 +relu", 64, 9, 64, lib.F_RELU | lib.F_UP2X_A),
    ("up2x(64)+concat(16) -> 64 +relu", 64, 16, 64, lib.F_RELU | lib.F_UP2X_A),
    ("conv 64->32 +relu", 64, 0, 32, lib.F_RELU),
    ("conv 32->3", 32, 0, 3, 0),
]


def peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        j = json.load(open(p))
        return j["hbm_gbs"], j["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def time_dispatch(d, iters, warmup=3):
    """Median launch time in ms; the dispatch is planned once (dnxcu_plan), so the host only enqueues."""
    plan = C.c_void_p()
    lib.check(lib.L.dnxcu_plan_create(C.byref(d), C.byref(plan)), "dnxcu_plan_create")
    e = [torch.cuda.Event(enable_timing=True) for _ in range(iters + 1)]
    for _ in range(warmup):
        lib.check(lib.L.dnxcu_plan_launch(plan, None))
    torch.cuda.synchronize()
    e[0].record()
    for i in range(iters):
        lib.check(lib.L.dnxcu_plan_launch(plan, None))
        e[i + 1].record()
    torch.cuda.synchronize()
    lib.L.dnxcu_plan_destroy(plan)
    return float(np.median([e[i].elapsed_time(e[i + 1]) for i in range(iters)]))


def run(variants="best", iters=20, h=H, w=W, only=None, config=None):
    hbm, tc, src = peaks()
    rows = []
    conv_variants = [v for v in lib.variants() if v["op"] == lib.OP_CONV3X3 and v["needs_tcgen05"]]
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    for name, ca, cb, k, flags in CASES:
        if only and only not in name:
            continue
        up = bool(flags & lib.F_UP2X_A)
        ha, wa = (h // 2, w // 2) if up else (h, w)
        gen = lambda seed, hh, ww, cc: rng.uniform_torch(seed, hh * ww * cc, -1, 1).to(torch.float32).to(torch.float16).reshape(hh, ww, cc)
        a = gen(11, ha, wa, ca)
        b = gen(12, h, w, cb) if cb else None
        wt = rng.he_normal_weights(13, k, ca + cb)
        out = torch.empty((h, w, k), dtype=torch.float16, device="cuda")
        outp = torch.empty((h // 2, w // 2, k), dtype=torch.float16, device="cuda")
        best = None
        for v in conv_variants:
            if config and v["config"] != config:
                continue
            d = lib.Dispatch()
            d.variant, d.flags, d.c_a, d.c_b, d.c_out = v["id"], flags, ca, cb, k
            d.pc[0], d.pc[1] = w, h
            d.in_a = a.data_ptr()
            d.in_b = b.data_ptr() if cb else None
            d.out = None if flags & lib.F_NO_FULL_OUT else out.data_ptr()
            d.out_pool = outp.data_ptr() if flags & lib.F_POOL_OUT else None
            d.device_status = status.data_ptr()
            d.weights = 0x1000
            if lib.L.dnxcu_validate(C.byref(d)) != 0:
                continue
            wd = torch.from_numpy(lib.prepare_weights(v["id"], wt, ca, cb)).cuda()
            d.weights = wd.data_ptr()
            ms = time_dispatch(d, iters)
            r_, w_, f_ = C.c_uint64(), C.c_uint64(), C.c_uint64()
            lib.L.dnxcu_cost(C.byref(d), C.byref(r_), C.byref(w_), C.byref(f_))
            byts, flops = r_.value + w_.value, f_.value
            t_tc, t_hbm = flops / (tc * 1e12) * 1e3, byts / (hbm * 1e9) * 1e3
            row = dict(case=name, variant=v["config"], ms=round(ms, 4), tflops=round(flops / ms / 1e9, 1),
                       gbs=round(byts / ms / 1e6, 1), bound="tensor" if t_tc >= t_hbm else "hbm",
                       roof_ms=round(max(t_tc, t_hbm), 4), frac=round(max(t_tc, t_hbm) / ms, 4),
                       frac_tensor=round(t_tc / ms, 4), frac_hbm=round(t_hbm / ms, 4))
            if variants == "all":
                rows.append(row)
            if best is None or ms < best["ms"]:
                best = row
        if variants != "all" and best:
            rows.append(best)
    assert int(status[0].item()) == 0, "a kernel reported a bounded wait that ran out"
    return dict(h=h, w=w, peaks=dict(hbm_gbs=hbm, tensor_tflops=tc, source=src), rows=rows)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--variants", default="best", choices=["best", "all"])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--json", default=None)
    ap.add_argument("--only", default=None, help="run only the cases whose name contains this text")
    ap.add_argument("--config", default=None, help="run only the variant with exactly this config string")
    args = ap.parse_args()
    res = run(args.variants, args.iters, only=args.only, config=args.config)
    for r in res["rows"]:
        print(f"{r['case']:40s} {r['variant']:22s} {r['ms']:8.4f} ms  {r['tflops']:7.1f} TF/s  {r['gbs']:7.1f} GB/s  "
              f"{r['bound']:6s} roof {r['roof_ms']:.4f} ms  frac {r['frac']:.3f}")
    if args.json:
        json.dump(res, open(args.json, "w"), indent=1)


if __name__ == "__main__":
    main()
