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


# ---- failure paths of the exchange protocol (host side, gloo) ---------------------------------------------

def _failure_worker(rank, world, port, scenario, out_dir):
    import datetime
    import time
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    result = "ok"
    try:
        if scenario == "mismatched_band_height":
            # rank 1 believes the image is split 48 / 16 instead of 32 / 32
            band = (64, 0, 32) if rank == 0 else (64, 48, 16)
            try:
                parallel.check_bands(dist, rank, world, band, 40)
            except ValueError as e:
                result = "refused: " + str(e)[:40]
        elif scenario == "missing_peer":
            row = torch.arange(8, dtype=torch.int16)
            if rank == 0:
                got = torch.empty_like(row)
                t0 = time.time()
                try:
                    parallel.exchange_rows(dist, rank, world, row, row, None, got)
                    result = "returned"
                except Exception as e:  # the process group's timeout ends the wait
                    result = f"timeout after {time.time() - t0:.0f}s: {type(e).__name__}"
            else:
                time.sleep(6)  # never takes part in the exchange
                result = "absent"
        elif scenario == "late_row":
            row = torch.full((8,), 10 + rank, dtype=torch.int16)
            got = torch.empty_like(row)
            if rank == 1:
                time.sleep(1.0)  # the neighbour is late, but inside the limit
            if rank == 0:
                parallel.exchange_rows(dist, rank, world, row, row, None, got)
            else:
                parallel.exchange_rows(dist, rank, world, row, row, got, None)
            result = f"got {int(got[0])}"
    finally:
        with open(os.path.join(out_dir, f"r{rank}.txt"), "w") as f:
            f.write(result)
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def _run_failure(tmp_path, scenario):
    port = 29100 + (os.getpid() % 800) + {"mismatched_band_height": 1, "missing_peer": 2, "late_row": 3}[scenario]
    try:
        mp.spawn(_failure_worker, args=(2, port, scenario, str(tmp_path)), nprocs=2, join=True)
    except Exception:
        pass  # a rank may exit with an error after it wrote its result
    return [open(tmp_path / f"r{r}.txt").read() for r in range(2)]


def test_mismatched_band_heights_are_refused_on_every_rank(tmp_path):
    r = _run_failure(tmp_path, "mismatched_band_height")
    assert all(x.startswith("refused") for x in r), r


def test_missing_peer_ends_in_a_timeout_not_a_hang(tmp_path):
    r = _run_failure(tmp_path, "missing_peer")
    assert r[0].startswith("timeout"), r
    assert r[1] == "absent"


def test_late_row_is_waited_for(tmp_path):
    r = _run_failure(tmp_path, "late_row")
    assert r == ["got 11", "got 10"], r
