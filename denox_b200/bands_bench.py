"""4K frame split into row bands over the GPUs of one node (benchmark configuration 3).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \\
        -m denox_b200.bands_bench [--steps K] [--warmup W] [--height 2176] [--width 3840]

Every rank owns H/N rows; before each conv the boundary rows of its operands are swapped with the neighbouring
ranks over NCCL.  Prints one JSON line on rank 0: frames/s of the whole frame (device timed, max over ranks)."""
import argparse
import json
import os

import numpy as np
import torch
import torch.distributed as dist

from . import lib, nets, parallel


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--height", type=int, default=2176)
    ap.add_argument("--width", type=int, default=3840)
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    net = nets.oidn_unet()
    model = lib.Model(net, device=local)
    runner = parallel.BandRunner(model, args.height, args.width, rank, world, dist)
    _, row0, rows = runner.band
    din, dout = runner.io()
    x = nets.oidn_input(1000 + rank, rows, args.width)  # band content does not matter for timing
    from .parallel import _Raw
    torch.as_tensor(_Raw(din, x.nbytes), device="cuda").copy_(torch.from_numpy(x.reshape(-1)).cuda())
    for _ in range(args.warmup):
        runner.run()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        runner.run()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    if rank == 0:
        t = float(ms.item()) / args.steps
        print(json.dumps({"metric": "OIDN-UNet 4K fp16 frames/s, row bands", "value": 1e3 / t, "unit": "frames/s",
                          "n_gpus": world, "ms_per_frame": t, "height": args.height, "width": args.width,
                          "gflop_per_frame": nets.total_flops(net, args.height, args.width) / 1e9,
                          "exchanges_per_frame": sum(len(v) for v in runner.points.values()),
                          "scaling": "strong"}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
