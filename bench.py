#!/usr/bin/env python
"""Benchmark of the hot path: OIDN-style U-Net, 1 x 1088 x 1920 x 9 binary16 HWC, frames/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one frame through the whole dispatch schedule.  With N > 1 (launched
by torch.distributed.run, one rank per GPU) every rank runs its own frames
(frame parallel, no data-path collective): weak scaling.  Prints ONE JSON line
on rank 0.

  value : frames/s with inputs already resident in HBM (CUDA events around K
          graph replays; input frames rotate through a set larger than L2)
  e2e   : frames/s through Instance.infer with pinned HOST buffers
          (H2D of the frame and D2H of the result inside the timed region)
  roofline : the dispatch with the largest share of the frame time, algorithmic
          flops (2 H W 9 C K) or bytes per launch over its mean event-timed
          duration, against the measured peak of MEASURED_PEAKS.json
  cpu_baseline : the CPU oracle (the restatement of the reference's shader
          arithmetic, binary16 accumulation) on a crop of the same frame

--impl reference times that CPU restatement alone (the reference's own
implementation needs Vulkan, which does not exist on these machines).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "OIDN-UNet 1080p fp16 frames/s"
H, W, C_IN = 1088, 1920, 9
WORKLOAD = "OIDN-style U-Net fp16 HWC, batch 1, 1920x1088, 9 input channels (configs[1])"
CROP = (544, 960)  # CPU sample: 1/4 of the frame's pixels, every layer of the net


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        j = json.load(open(p))
        return dict(hbm=j["hbm_gbs"], tc=j["bf16_tflops"], tc_sustained=j.get("bf16_tflops_sustained"), src="measured")
    return dict(hbm=6650.0, tc=1590.0, tc_sustained=1400.0, src="fallback")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons during the timed region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.lines = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if not self.proc:
            return None
        time.sleep(0.15)
        self.proc.terminate()
        sm, smax, reasons = [], [], set()
        rows = [l for (t, l) in self.lines if t0 - 0.05 <= t <= t1 + 0.15] or [l for (_, l) in self.lines]
        for l in rows:
            f = [x.strip() for x in l.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); smax.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return None
        return dict(sm_mhz=float(np.median(sm)), sm_max_mhz=float(max(smax)), reasons=sorted(reasons),
                    samples=len(sm))


def cpu_oracle_sample(mode_name="f16"):
    """Times the CPU oracle on the crop; returns (frames/s scaled to the full frame, seconds, threads)."""
    from denox_b200 import nets
    from oracle import oracle
    net = nets.oidn_unet()
    full = nets.oidn_input(1000, H, W)
    y0, x0 = (H - CROP[0]) // 2, (W - CROP[1]) // 2
    x = np.ascontiguousarray(full[y0:y0 + CROP[0], x0:x0 + CROP[1]])
    mode = oracle.ACC_F16 if mode_name == "f16" else oracle.ACC_F32
    t0 = time.perf_counter()
    oracle.run_network(net, x, mode)
    dt = time.perf_counter() - t0
    frac = (CROP[0] * CROP[1]) / (H * W)
    return frac / dt, dt, oracle.num_threads()


def run_reference(args, rank, result_out):
    """The reference arm: the CPU restatement of the reference's arithmetic on the host cores."""
    if rank != 0:
        return
    vals = []
    for i in range(args.warmup + args.steps):
        fps, dt, threads = cpu_oracle_sample("f16")
        if i >= args.warmup:
            vals.append((fps, dt))
    fps = float(np.mean([v[0] for v in vals]))
    ms = float(np.mean([v[1] for v in vals])) * 1e3
    sample = (f"whole net on a {CROP[0]}x{CROP[1]} crop of the 1088x1920 frame (1/4 of the pixels), binary16 "
              f"accumulation (reference arithmetic), scaled by pixel count")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": fps, "unit": "frames/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "note": "reference's Vulkan runtime unavailable on this box; CPU "
                   "restatement of its shader arithmetic (oracle/oracle.c), OpenMP over rows"},
        "cpu_baseline": {"value": fps, "unit": "frames/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": fps, "unit": "frames/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }), file=result_out, flush=True)


def _private_stdout():
    """The one JSON line must be alone on stdout: libraries (NCCL's version banner) write there too.  Keep a private
    copy of stdout for the result and point file descriptor 1 at stderr for everything else."""
    out = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    return out


def bind_to_gpu_numa_node(torch, device):
    """Several ranks share the host: run this rank on the CPUs of the NUMA node its GPU hangs off, so that the
    pinned frame buffers it allocates next are local to that GPU's PCIe root (first touch).  Returns the node
    or None when the topology cannot be read."""
    try:
        bdf = torch.cuda.get_device_properties(device)
        bus = f"{bdf.pci_domain_id:04x}:{bdf.pci_bus_id:02x}:{bdf.pci_device_id:02x}.0"
        node = int(open(f"/sys/bus/pci/devices/{bus}/numa_node").read())
        if node < 0:
            return None
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)
        if not cpus:
            return None
        os.sched_setaffinity(0, cpus)
        return node
    except Exception:
        return None


def main():
    result_out = _private_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-db", action="store_true", help="fixed variant preference instead of a benchmark database")
    ap.add_argument("--db", default=None, help="benchmark database file (default: a temporary file)")
    ap.add_argument("--streams", type=int, default=2, help="CUDA streams the resident frames are spread over")
    ap.add_argument("--e2e-steps", type=int, default=0, help="default: same as --steps")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        if args.steps > 3:
            args.steps = 3  # each step is several seconds of CPU work
        args.warmup = min(args.warmup, 1)
        run_reference(args, rank, result_out)
        return

    import torch
    from denox_b200 import lib, nets

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this backend has no CPU path")
    torch.cuda.set_device(local_rank)
    numa = bind_to_gpu_numa_node(torch, local_rank) if world > 1 else None
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    net = nets.oidn_unet()
    # the reference's flow: populate the benchmark database with every (dispatch, variant) candidate of the
    # model, time them on this device, then let the schedule selection pick the fastest per dispatch
    db = None
    if not args.no_db:
        import tempfile
        path = args.db or os.path.join(tempfile.gettempdir(), f"dnxcu_bench_{os.getpid()}.db")
        db = lib.Db(path)
        db.populate(net, H, W, device=local_rank)
        db.bench(device=local_rank, min_samples=5, max_relative_error=0.05, max_rounds=2)
    model = lib.Model(net, device=local_rank, db=db)
    inst = lib.Instance(model, H, W)
    n_disp = model.dispatch_count()
    # kernels per frame: a dispatch whose output channels are split is several launches (grid[2] counts them)
    tc_ids = {v["id"] for v in lib.variants() if v["needs_tcgen05"]}
    launches_per_frame = sum(max(1, int(i.grid[2])) if i.variant in tc_ids else 1 for i in inst.dispatch_info())

    # resident inputs: 4 distinct frames = 150 MB > L2 (126 MB); one frame's activations are 1.7 GB anyway
    NF = 4
    frames = [nets.oidn_input(1000 + rank * 64 + i, H, W) for i in range(NF)]
    dev_in = [torch.from_numpy(f).cuda() for f in frames]
    # frames are independent: they go round robin to NS streams, so that the tail of one frame's small layers
    # overlaps the next frame's large ones (the sustained "stream of frames" rate); every stream has its own
    # output buffer, every resident frame slot its own instance (an instance caches the CUDA graph of its
    # schedule for one (input, output) pointer pair)
    NS = max(1, min(args.streams, NF))
    dev_outs = [torch.empty((H, W, 3), dtype=torch.float16, device="cuda") for _ in range(NS)]
    dev_out = dev_outs[0]
    streams = [torch.cuda.Stream() for _ in range(NS)]
    stream = streams[0]
    insts = [inst] + [lib.Instance(model, H, W) for _ in range(NF - 1)]

    def step(i):
        k = i % NF
        insts[k].enqueue(dev_in[k].data_ptr(), dev_outs[k % NS].data_ptr(), streams[k % NS].cuda_stream)

    for i in range(NF):
        step(i)
    for st in streams:
        st.synchronize()
    for i in range(args.warmup):
        step(i)
    for st in streams:
        st.synchronize()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ends = [torch.cuda.Event() for _ in range(NS)]
    t_wall0 = time.time()
    e0.record(streams[0])
    for st in streams[1:]:
        st.wait_event(e0)
    for i in range(args.steps):
        step(i)
    for st, ev in zip(streams, ends):
        ev.record(st)
    for ev in ends[1:]:
        streams[0].wait_event(ev)
    e1.record(streams[0])
    for st in streams:
        st.synchronize()
    t_wall1 = time.time()
    barrier()
    ms_total = e0.elapsed_time(e1)
    clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None
    if dist is not None:
        t = torch.tensor([ms_total], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_per_step = ms_total / args.steps
    value = world * args.steps / (ms_total * 1e-3)

    # ---- end to end: host buffers through Instance.infer ----
    e2e_steps = args.e2e_steps or args.steps
    pin_in = [torch.from_numpy(f).pin_memory() for f in frames]
    host_in = [p.numpy() for p in pin_in]
    in_bytes = frames[0].nbytes
    out_bytes = H * W * 3 * 2
    # three instances round robin: frame i's copies overlap frame i-1's kernels (each instance has its own
    # stream, buffers and graph); every frame still goes host -> device -> host through the public call
    NI = 3
    pin_out = [torch.empty((H, W, 3), dtype=torch.float16).pin_memory() for _ in range(NI)]
    host_out = [p.numpy() for p in pin_out]
    for i in range(NI):
        insts[i].infer_async(host_in[i % NF], host_out[i])
    for i in range(NI):
        insts[i].wait()
    barrier()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        k = i % NI
        if i >= NI:
            insts[k].wait()
        insts[k].infer_async(host_in[i % NF], host_out[k])
    for k in range(NI):
        insts[k].wait()
    e2e_s = time.perf_counter() - t0
    y = host_out[(e2e_steps - 1) % NI]
    if dist is not None:
        t = torch.tensor([e2e_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e = world * e2e_steps / e2e_s
    assert np.isfinite(y.astype(np.float32)).all()

    if rank != 0:
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        return

    # ---- per dispatch timing and roofline (rank 0) ----
    pk = peaks()
    infos, total_ms = insts[0].bench(warmup=3, iters=10)
    table = []
    for d in infos:
        byts, flops = d.bytes_read + d.bytes_written, d.flops
        nd = net.nodes[d.src_node]
        if nd.kind == nets.CONV and d.flops > 0:
            # algorithmic work from the model's own channel counts (no credit for zero padded channels)
            c_real = net.channels[nd.in0]
            c_run = d.c_a + d.c_b
            flops = flops // c_run * c_real
            byts -= 2 * d.h * d.w * (c_run - c_real) + 18 * (c_run - c_real) * d.c_out
        t_s = d.ms * 1e-3
        tf = flops / t_s / 1e12 if t_s > 0 else 0.0
        gb = byts / t_s / 1e9 if t_s > 0 else 0.0
        t_tc, t_hbm = flops / (pk["tc"] * 1e12), byts / (pk["hbm"] * 1e9)
        bound = "tensor" if t_tc >= t_hbm else "hbm"
        v = lib.L.dnxcu_variant(d.variant).contents
        table.append(dict(name=net.nodes[d.src_node].name, dispatch=d.name.decode(), variant=v.config.decode(),
                          hw=[d.h, d.w], c=[d.c_a, d.c_b, d.c_out], ms=round(d.ms, 5), tflops=round(tf, 2),
                          gbs=round(gb, 1), bound=bound, frac=round(max(t_tc, t_hbm) / t_s, 4) if t_s > 0 else 0,
                          share=round(d.ms / total_ms, 4), roof_ms=round(max(t_tc, t_hbm) * 1e3, 5)))
    top = max(range(len(infos)), key=lambda i: infos[i].ms)
    dt, tt = infos[top], table[top]
    if tt["bound"] == "tensor":
        roof = dict(bound="tensor", achieved=tt["tflops"], peak=pk["tc"], unit="TFLOP/s",
                    frac=round(tt["tflops"] / pk["tc"], 4))
    else:
        roof = dict(bound="hbm", achieved=tt["gbs"], peak=pk["hbm"], unit="GB/s", frac=round(tt["gbs"] / pk["hbm"], 4))
    # DRAM bytes per launch of that kernel from the ncu capture summarised in
    # profiles/conv3x3_tc_stack_upconcat_64_16_to_64_1080p.md (dram__bytes_read.sum + dram__bytes_write.sum); only
    # valid while the dominant dispatch is that shape
    traffic = 352.7e6 if (dt.c_a, dt.c_b, dt.c_out, dt.h, dt.w) == (64, 16, 64, 1088, 1920) else None
    roof.update(traffic=traffic, kernel=f"conv3x3_tc {tt['name']} {dt.c_a}+{dt.c_b}->{dt.c_out} @{dt.h}x{dt.w}",
                peak_source=pk["src"], duration_ms=round(dt.ms, 5), share_of_frame=tt["share"])
    sum_bound_ms = sum(r["roof_ms"] for r in table)

    cpu = None
    if not args.no_cpu_baseline:
        fps, dt_s, threads = cpu_oracle_sample("f16")
        cpu = {"value": fps, "unit": "frames/s", "cores": threads, "kind": "port",
               "sample": f"whole net on a {CROP[0]}x{CROP[1]} crop (1/4 of the frame), binary16 accumulation, "
                         f"{dt_s:.1f} s, scaled by pixel count"}

    out = {
        "metric": METRIC, "value": value, "unit": "frames/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "parallelism": f"frame-parallel x{world}" if world > 1 else "single GPU",
                   "l2": f"inputs rotate over {NF} resident frames (150 MB > L2); activations per frame 1.7 GB",
                   "dispatches_per_frame": n_disp, "launches_per_frame": launches_per_frame, "streams": NS, "gflop_per_frame": nets.total_flops(net, H, W) / 1e9,
                   "roofline_bound_ms_per_frame": round(sum_bound_ms, 4)},
        "e2e": {"value": e2e, "unit": "frames/s", "h2d_bytes_per_step": in_bytes, "d2h_bytes_per_step": out_bytes,
                "api": "dnxcu_instance_infer_async + dnxcu_instance_wait, 3 instances round robin, pinned host buffers",
                "numa_node": numa},
        "gpu_launches": args.steps * launches_per_frame,
        "clocks": clocks,
        "roofline": roof,
        "cpu_baseline": cpu,
        "tensor_tflops_whole_frame": round(nets.total_flops(net, H, W) / (ms_per_step * 1e-3) / 1e12, 2),
        "per_dispatch": table,
    }
    print(json.dumps(out), file=result_out, flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
