"""Parity report of a whole network on the GPU against the CPU oracle: end to end (free running) and per
layer with the layer's inputs taken from the GPU run ("teacher forced": the oracle recomputes every node from
the tensors the GPU produced, so accumulation drift of earlier layers does not leak into a layer's figures).

Test infrastructure: imports the oracle, never imported by the product."""
import json
import os

import numpy as np

from denox_b200 import lib, nets
from oracle import oracle

ATOL, RTOL = 2e-2, 1e-2  # the benchmark's acceptance rule: |d| <= 2e-2 + 1e-2 |ref| per element


def stats(got, ref):
    g, r = np.asarray(got, dtype=np.float32), np.asarray(ref, dtype=np.float32)
    d = np.abs(g - r)
    return dict(max=float(d.max()), mean=float(d.mean()), violation_fraction=float((d > ATOL + RTOL * np.abs(r)).mean()),
                n=int(d.size))


def _fetch(inst, tid):
    import torch
    try:
        p, h, w, c = inst.tensor(tid)
    except lib.DnxcuError:
        return None
    torch.cuda.synchronize()
    iface = {"shape": (h, w, c), "typestr": "<f2", "data": (int(p), False), "version": 2}
    holder = type("Raw", (), {"__cuda_array_interface__": iface})()
    return torch.as_tensor(holder, device="cuda").cpu().numpy()


def _apply(nd, t, mode):
    if nd.kind == nets.CONV:
        return oracle.conv3x3(t[nd.in0], nd.weights, nd.bias, mode=mode)
    if nd.kind == nets.RELU:
        return oracle.relu(t[nd.in0])
    if nd.kind == nets.LEAKY_RELU:
        return oracle.leaky_relu(t[nd.in0], nd.alpha)
    if nd.kind == nets.MAXPOOL:
        return oracle.maxpool2x2(t[nd.in0])
    if nd.kind == nets.UPSAMPLE:
        return oracle.upsample2x(t[nd.in0])
    if nd.kind == nets.CONCAT:
        return oracle.concat(t[nd.in0], t[nd.in1])
    raise ValueError(nd.kind)


def report(net, x, inst, y, modes=(("acc=f16", oracle.ACC_F16), ("acc=f32", oracle.ACC_F32))):
    """inst has just produced y from x.  Returns {"layers": [...], "end_to_end": {...}}."""
    out = {"layers": [], "end_to_end": {}}
    for mname, mode in modes:
        ref = oracle.run_network(net, x, mode)[net.output_tensor]
        out["end_to_end"][mname] = stats(y, ref)
        del ref
    # teacher forced, node by node; a tensor the schedule fused away is rebuilt from GPU tensors by the oracle
    rows = {}
    for mname, mode in modes:
        t = {net.input_tensor: np.ascontiguousarray(x)}
        last_conv = None
        for nd in net.nodes:
            if nd.kind == nets.CONV:
                last_conv = nd.name
            want = _apply(nd, t, mode)
            got = _fetch(inst, nd.out)
            if nd.out == net.output_tensor and got is None:
                got = y
            if got is not None and got.shape == want.shape and nd.kind in (nets.CONV, nets.RELU, nets.LEAKY_RELU, nets.MAXPOOL):
                key = (last_conv or nd.name) + ("+pool" if nd.kind == nets.MAXPOOL else "")
                r = rows.setdefault(key, dict(layer=key, shape=list(want.shape)))
                r[mname] = stats(got, want)
            t[nd.out] = got if got is not None and got.shape == want.shape else want
            # inputs nobody reads any more can go (full resolution tensors are hundreds of MB)
            for tid in (nd.in0, nd.in1):
                if tid >= 0 and tid != net.input_tensor and not any(
                        n2.in0 == tid or n2.in1 == tid for n2 in net.nodes[net.nodes.index(nd) + 1:]):
                    t.pop(tid, None)
    out["layers"] = list(rows.values())
    return out


def to_markdown(rep, title):
    lines = [f"## {title}", "",
             "| layer | output H x W x C | max abs d vs acc=f16 | mean | violations | max abs d vs acc=f32 | mean | violations |",
             "|---|---|---|---|---|---|---|---|"]
    for r in rep["layers"]:
        a, b = r.get("acc=f16", {}), r.get("acc=f32", {})
        lines.append(f"| {r['layer']} | {'x'.join(map(str, r['shape']))} | {a.get('max', 0):.4g} | {a.get('mean', 0):.3g} | "
                     f"{a.get('violation_fraction', 0):.2e} | {b.get('max', 0):.4g} | {b.get('mean', 0):.3g} | "
                     f"{b.get('violation_fraction', 0):.2e} |")
    e = rep["end_to_end"]
    a, b = e.get("acc=f16", {}), e.get("acc=f32", {})
    lines.append(f"| **end to end (free running)** | | {a.get('max', 0):.4g} | {a.get('mean', 0):.3g} | "
                 f"{a.get('violation_fraction', 0):.2e} | {b.get('max', 0):.4g} | {b.get('mean', 0):.3g} | "
                 f"{b.get('violation_fraction', 0):.2e} |")
    return "\n".join(lines) + "\n"


def save(rep, name):
    """Writes the report as JSON and as a markdown table into the folder DNXCU_REPORT_DIR names, if it is set."""
    d = os.environ.get("DNXCU_REPORT_DIR")
    if not d:
        return None
    os.makedirs(d, exist_ok=True)
    path = os.path.join(d, name + ".json")
    with open(path, "w") as f:
        json.dump(rep, f)
    with open(os.path.join(d, name + ".md"), "w") as f:
        f.write(to_markdown(rep, name))
    return path
