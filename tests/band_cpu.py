"""CPU model of the row band protocol: the oracle as the per-band compute, torch CPU tensors over gloo as the
halo exchange (denox_b200.parallel.exchange_rows, the function the GPU path uses).  Test infrastructure."""
import numpy as np

from denox_b200.parallel import exchange_rows

def run_network_banded_cpu(net, x_band, rank, world, dist, oracle, mode=0):
    """The same band protocol with the CPU oracle as the per-band compute and torch CPU tensors over gloo as the
    exchange: every conv first swaps its operands' boundary rows.  Returns this band's tensors."""
    import torch
    CONV, RELU, MAXPOOL, UPSAMPLE, CONCAT = 1, 2, 3, 4, 5
    t = {net.input_tensor: np.ascontiguousarray(x_band, dtype=np.float16)}
    producer = {nd.out: nd for nd in net.nodes}

    def halo(arr):
        top = torch.from_numpy(arr[0].copy().view(np.int16))
        bot = torch.from_numpy(arr[-1].copy().view(np.int16))
        rt = torch.empty_like(top) if rank > 0 else None
        rb = torch.empty_like(bot) if rank < world - 1 else None
        exchange_rows(dist, rank, world, top, bot, rt, rb)
        f = lambda v: None if v is None else v.numpy().view(np.float16)
        return f(rt), f(rb)

    for nd in net.nodes:
        if nd.kind == CONV:
            src = t[nd.in0]
            p = producer.get(nd.in0)
            if p is not None and p.kind == CONCAT:
                a, b = t[p.in0], t[p.in1]
                pa = producer.get(p.in0)
                up = pa is not None and pa.kind == UPSAMPLE
                if up:
                    a = t[pa.in0]
                ha, hb = halo(a), halo(b)
                t[nd.out] = oracle.conv3x3(a, nd.weights, nd.bias, mode=mode, b=b, up_a=up,
                                           halo=(ha[0], ha[1], hb[0], hb[1]))
            else:
                h = halo(src)
                t[nd.out] = oracle.conv3x3(src, nd.weights, nd.bias, mode=mode, halo=(h[0], h[1], None, None))
        elif nd.kind == RELU:
            t[nd.out] = oracle.relu(t[nd.in0])
        elif nd.kind == MAXPOOL:
            t[nd.out] = oracle.maxpool2x2(t[nd.in0])
        elif nd.kind == UPSAMPLE:
            t[nd.out] = oracle.upsample2x(t[nd.in0])
        elif nd.kind == CONCAT:
            t[nd.out] = oracle.concat(t[nd.in0], t[nd.in1])
    return t
