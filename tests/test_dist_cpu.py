"""Multi-process host logic on CPU (gloo, world size 2): frame sharding, band partition, and the halo exchange
protocol of the row band path, with the oracle standing in for the kernels."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from denox_b200 import nets, parallel
from oracle import oracle

HERE = os.path.dirname(os.path.abspath(__file__))


def test_frame_shard_covers_every_frame_once():
    for world in (1, 2, 4, 8):
        got = sorted(i for r in range(world) for i in parallel.frame_shard(64, world, r))
        assert got == list(range(64))
        assert max(len(parallel.frame_shard(64, world, r)) for r in range(world)) == 64 // world


def test_band_partition():
    assert parallel.band_of(0, 1, 1088) == (1088, 0, 1088)
    for world in (2, 4, 8):
        bands = [parallel.band_of(r, world, 2176) for r in range(world)]
        assert bands[0][1] == 0 and bands[-1][1] + bands[-1][2] == 2176
        assert all(b[2] % 16 == 0 for b in bands)
        assert all(bands[i][1] + bands[i][2] == bands[i + 1][1] for i in range(world - 1))
    with pytest.raises(ValueError):
        parallel.band_of(0, 8, 1088 + 16)


def _worker(rank, world, port, which, h, w, out_dir):
    sys.path.insert(0, HERE)
    from band_cpu import run_network_banded_cpu
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        net = nets.oidn_unet() if which == "oidn" else nets.tiny_unet()
        x = nets.oidn_input(1000, h, w) if which == "oidn" else nets.tiny_input(1000, h, w)
        _, row0, rows = parallel.band_of(rank, world, h)
        t = run_network_banded_cpu(net, x[row0:row0 + rows], rank, world, dist, oracle)
        np.save(os.path.join(out_dir, f"band{rank}.npy"), t[net.output_tensor])
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("which,h,w", [("tiny", 64, 40), ("oidn", 64, 48)])
def test_row_bands_equal_whole_image(tmp_path, which, h, w):
    """Two bands with per-conv halo exchange reproduce the one-process result bit for bit."""
    world = 2
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, which, h, w, str(tmp_path)), nprocs=world, join=True)
    net = nets.oidn_unet() if which == "oidn" else nets.tiny_unet()
    x = nets.oidn_input(1000, h, w) if which == "oidn" else nets.tiny_input(1000, h, w)
    # the one-process result of the same fused evaluation order (two K phases for a concat)
    sys.path.insert(0, HERE)
    from band_cpu import run_network_banded_cpu
    whole = run_network_banded_cpu(net, x, 0, 1, dist, oracle)[net.output_tensor]
    ref = oracle.run_network(net, x)[net.output_tensor]
    assert np.abs(whole.astype(np.float32) - ref.astype(np.float32)).max() < 2e-2
    got = np.concatenate([np.load(tmp_path / f"band{r}.npy") for r in range(world)], axis=0)
    assert got.shape == whole.shape
    assert (got == whole).all()
