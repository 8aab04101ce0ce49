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


# (the last case is large enough for the conv kernel to cut its work units as contiguous row ranges, with other
# boundaries in a band than in the whole image)
@pytest.mark.parametrize("which,h,w,world", [("tiny", 64, 160, 2), ("oidn", 64, 144, 2), ("oidn", 128, 48, 4), ("oidn", 384, 160, 8),
                                             ("oidn", 1280, 1920, 2)])
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


@pytest.mark.parametrize("which,h,w,world", [("tiny", 64, 160, 2), ("oidn", 64, 144, 2), ("oidn", 128, 48, 4), ("oidn", 384, 160, 8)])
def test_bands_with_peer_exchange_on_one_device(which, h, w, world):
    """The exchange kernel itself, with all bands on one device: every band pushes its boundary rows into its
    neighbours' slabs (the same stores that cross NVLink between GPUs), then every band waits for its flags,
    which are set by then (bands that share a device never wait on one another inside one launch).  Two frames
    in a row: slabs, flags and counters are reused."""
    import torch
    from gpu_util import wrap
    net = nets.oidn_unet() if which == "oidn" else nets.tiny_unet()
    model = lib.Model(net)
    bands = [parallel.band_of(r, world, h) for r in range(world)]
    insts = [lib.Instance(model, b[2], w, band=b) for b in bands]
    handles = [i.halo_export() for i in insts]
    for r, inst in enumerate(insts):
        inst.halo_connect(handles[r - 1] if r > 0 else None, handles[r + 1] if r < world - 1 else None,
                          auto_exchange=False)
    n = model.dispatch_count()
    rows = h // world
    for frame in range(2):
        x = nets.oidn_input(1000 + frame, h, w) if which == "oidn" else nets.tiny_input(1000 + frame, h, w)
        want = _whole(net, x, h, w)
        for r, inst in enumerate(insts):
            din, _ = inst.io()
            wrap(din, (rows, w, x.shape[2])).copy_(torch.from_numpy(x[r * rows:(r + 1) * rows]).cuda())
        for i in range(n):
            for inst in insts:
                inst.halo_step(i, 1)  # push
            for inst in insts:
                inst.halo_step(i, 2)  # wait: already satisfied
            for inst in insts:
                inst.enqueue_range(i, i + 1, 0)
        torch.cuda.synchronize()
        got = []
        for inst in insts:
            _, dout = inst.io()
            got.append(wrap(dout, (rows, w, want.shape[2])).cpu().numpy())
            inst.wait()  # no wait ran out
        got = np.concatenate(got, 0)
        assert (got == want).all(), (frame, float(np.abs(got.astype(np.float32) - want.astype(np.float32)).max()))
    for inst in insts:
        inst.close()
    model.close()


def test_peer_connect_rejects_wrong_neighbours():
    net = nets.tiny_unet()
    model = lib.Model(net)
    a = lib.Instance(model, 32, 64, band=(96, 0, 32))
    b = lib.Instance(model, 32, 64, band=(96, 32, 32))
    c = lib.Instance(model, 32, 64, band=(96, 64, 32))
    wide = lib.Instance(model, 32, 80, band=(96, 32, 32))
    tall = lib.Instance(model, 48, 64, band=(96, 48, 48))
    ha, hb, hc = a.halo_export(), b.halo_export(), c.halo_export()
    with pytest.raises(lib.DnxcuError):
        a.halo_connect(None, hc)                      # not the adjacent band
    with pytest.raises(lib.DnxcuError):
        a.halo_connect(None, wide.halo_export())      # another width
    with pytest.raises(lib.DnxcuError):
        a.halo_connect(None, tall.halo_export())      # another band height
    with pytest.raises(lib.DnxcuError):
        b.halo_connect(ha, None)                      # a middle band needs both neighbours
    b.halo_connect(ha, hc, auto_exchange=False)
    with pytest.raises(lib.DnxcuError):
        b.halo_connect(ha, hc)                        # already connected
    for i in (a, b, c, wide, tall):
        i.close()
    model.close()


def test_wait_for_a_row_that_never_comes_is_bounded():
    """A band waits for its neighbour's row and nobody pushes it: with a limit of 2 ms the exchange kernel gives
    up, the instance reports DNXCU_E_DEVICE once, and the same instance then runs a whole frame correctly."""
    import time
    import torch
    from gpu_util import wrap
    net = nets.tiny_unet()
    model = lib.Model(net)
    h, w = 64, 96
    insts = [lib.Instance(model, 32, w, band=(h, r * 32, 32)) for r in range(2)]
    hs = [i.halo_export() for i in insts]
    insts[0].halo_connect(None, hs[1], auto_exchange=False)
    insts[1].halo_connect(hs[0], None, auto_exchange=False)
    first = min(p.before_dispatch for p in insts[0].halo_points())
    lib.check(lib.L.dnxcu_set_wait_limit_us(2000))
    try:
        t0 = time.time()
        insts[0].halo_step(first, 1)  # band 0 pushes its row (its count becomes 1) ...
        insts[0].halo_step(first, 2)  # ... and waits for band 1's first row, which nobody pushes
        torch.cuda.synchronize()
        assert time.time() - t0 < 1.0
        with pytest.raises(lib.DnxcuError) as err:
            insts[0].wait()
        assert err.value.status == lib.E_DEVICE
        insts[0].wait()  # reported once, then cleared
    finally:
        lib.check(lib.L.dnxcu_set_wait_limit_us(0))
    # the bands disagree on their counts now; once both are idle they start over and work again
    for inst in insts:
        inst.halo_reset()
    x = nets.tiny_input(1000, h, w)
    want = _whole(net, x, h, w)
    for r, inst in enumerate(insts):
        din, _ = inst.io()
        wrap(din, (32, w, 3)).copy_(torch.from_numpy(x[r * 32:(r + 1) * 32]).cuda())
    for i in range(model.dispatch_count()):
        for inst in insts:
            inst.halo_step(i, 1)
        for inst in insts:
            inst.halo_step(i, 2)
        for inst in insts:
            inst.enqueue_range(i, i + 1, 0)
    torch.cuda.synchronize()
    got = np.concatenate([wrap(inst.io()[1], (32, w, 3)).cpu().numpy() for inst in insts], 0)
    assert (got == want).all()
    for inst in insts:
        inst.wait()
        inst.close()
    model.close()


def _nccl_worker(rank, world, port, h, w, out_dir, exchange="auto"):
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
        runner = parallel.BandRunner(model, h, w, rank, world, dist, exchange=exchange)
        assert runner.transport == exchange
        _, row0, rows = runner.band
        din, dout = runner.io()
        for frame in range(2):  # the second frame replays the graph and reuses slabs, flags and counters
            wrap(din, (rows, w, 9)).copy_(torch.from_numpy(x[row0:row0 + rows]).cuda())
            runner.run()
            torch.cuda.synchronize()
        runner.inst.wait()
        np.save(os.path.join(out_dir, f"band{rank}.npy"), wrap(dout, (rows, w, 3)).cpu().numpy())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("exchange", ["peer", "nccl"])
def test_bands_on_several_gpus_equal_whole_image(tmp_path, exchange):
    import torch
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs two GPUs")
    h, w = 64 * world, 176
    port = 29700 + os.getpid() % 1000 + (7 if exchange == "peer" else 0)
    mp.spawn(_nccl_worker, args=(world, port, h, w, str(tmp_path), exchange), nprocs=world, join=True)
    net = nets.oidn_unet()
    want = _whole(net, nets.oidn_input(1000, h, w), h, w)
    got = np.concatenate([np.load(tmp_path / f"band{r}.npy") for r in range(world)], 0)
    assert (got == want).all()
