"""Row band execution on GPUs: a band instance with halo slabs gives bit-identical rows.

One device: two band instances on the same GPU, the halo rows moved between them by device copies in the
order `denox_b200.parallel.BandRunner` uses.  Two or more devices: one process per GPU, rows swapped with NCCL."""
import os
import sys

import numpy as np
import pytest

from denox_b200 import lib, nets, parallel

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _whole(net, x, h, w):
    model = lib.Model(net)
    inst = lib.Instance(model, h, w)
    y = inst.infer(x)
    inst.close(); model.close()
    return y


@pytest.mark.parametrize("which,h,w,world", [("tiny", 64, 160, 2), ("oidn", 64, 144, 2), ("oidn", 128, 48, 4)])
def test_bands_on_one_device_equal_whole_image(which, h, w, world):
    import torch
    from gpu_util import wrap
    net = nets.oidn_unet() if which == "oidn" else nets.tiny_unet()
    x = nets.oidn_input(1000, h, w) if which == "oidn" else nets.tiny_input(1000, h, w)
    want = _whole(net, x, h, w)
    model = lib.Model(net)
    insts = [lib.Instance(model, parallel.band_of(r, world, h)[2], w, band=parallel.band_of(r, world, h))
             for r in range(world)]
    pts = [i.halo_points() for i in insts]
    assert len(pts[0]) == len(pts[1]) > 0
    n = model.dispatch_count()
    rows = h // world
    for r, inst in enumerate(insts):
        din, _ = inst.io()
        wrap(din, (rows, w, x.shape[2])).copy_(torch.from_numpy(x[r * rows:(r + 1) * rows]).cuda())
    cuts = sorted({p.before_dispatch for p in pts[0]})
    first = 0
    for cut in cuts + [n]:
        for inst in insts:
            inst.enqueue_range(first, cut, 0)
        first = cut
        torch.cuda.synchronize()
        for e, p0 in enumerate(pts[0]):
            if p0.before_dispatch != cut:
                continue
            nel = int(p0.row_bytes) // 2
            for r in range(world - 1):
                up, down = pts[r][e], pts[r + 1][e]
                wrap(down.recv_top, (nel,)).copy_(wrap(up.send_bottom, (nel,)))
                wrap(up.recv_bottom, (nel,)).copy_(wrap(down.send_top, (nel,)))
            assert pts[0][e].recv_top is None and pts[-1][e].recv_bottom is None  # image borders: zero padding
        torch.cuda.synchronize()
    got = []
    for inst in insts:
        _, dout = inst.io()
        got.append(wrap(dout, (rows, w, want.shape[2])).cpu().numpy())
    got = np.concatenate(got, 0)
    assert (got == want).all(), float(np.abs(got.astype(np.float32) - want.astype(np.float32)).max())
    for inst in insts:
        inst.close()
    model.close()


def _nccl_worker(rank, world, port, h, w, out_dir):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        sys.path.insert(0, HERE)
        from gpu_util import wrap
        net = nets.oidn_unet()
        x = nets.oidn_input(1000, h, w)
        model = lib.Model(net, device=rank)
        runner = parallel.BandRunner(model, h, w, rank, world, dist)
        _, row0, rows = runner.band
        din, dout = runner.io()
        wrap(din, (rows, w, 9)).copy_(torch.from_numpy(x[row0:row0 + rows]).cuda())
        runner.run()
        torch.cuda.synchronize()
        np.save(os.path.join(out_dir, f"band{rank}.npy"), wrap(dout, (rows, w, 3)).cpu().numpy())
    finally:
        dist.destroy_process_group()


def test_bands_over_nccl_equal_whole_image(tmp_path):
    import torch
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs two GPUs")
    h, w = 64 * world, 176
    mp.spawn(_nccl_worker, args=(world, 29700 + os.getpid() % 1000, h, w, str(tmp_path)), nprocs=world, join=True)
    net = nets.oidn_unet()
    want = _whole(net, nets.oidn_input(1000, h, w), h, w)
    got = np.concatenate([np.load(tmp_path / f"band{r}.npy") for r in range(world)], 0)
    assert (got == want).all()
