"""Multi-GPU execution of the dispatch schedule: one process per GPU.

Two ways to shard, both without touching the kernels:

* frame parallel — independent frames, round robin over ranks, no exchange;
* row bands — rank r owns rows [r*H/G, (r+1)*H/G) of every tensor (at every
  resolution level).  A 3x3 conv needs one row of each operand from the band
  above and below, so before every conv dispatch the ranks swap their boundary
  rows (`torch.distributed` send/recv: NCCL on GPUs, gloo in the CPU tests).
  The rows land in halo slabs of the consumer's own memory
  (`dnxcu_dispatch.halo`); image borders keep NULL slabs (zero padding).  Pool
  and nearest upsample need no halo because band heights are multiples of 16.

The reference has no multi-device code at all; this module is new.
"""
import numpy as np


def frame_shard(n_frames: int, world: int, rank: int):
    """Frame indices of `rank` (round robin)."""
    return list(range(rank, n_frames, world))


def band_of(rank: int, world: int, image_h: int, align: int = 16):
    """(image_h, row0, rows) of rank's band: equal bands, heights multiple of `align`."""
    if image_h % (world * align):
        raise ValueError(f"image height {image_h} is not a multiple of {world} bands x {align} rows")
    rows = image_h // world
    return image_h, rank * rows, rows


def exchange_rows(dist, rank, world, send_top, send_bottom, recv_top, recv_bottom):
    """Swaps boundary rows with the neighbouring bands.

    send_top / send_bottom: this band's first / last row (tensors);
    recv_top / recv_bottom: where the row above / below must land (None at an image border).
    All ranks must call this for the same exchange point in the same order."""
    ops = []
    if rank > 0:
        ops.append(dist.P2POp(dist.isend, send_top, rank - 1))
        ops.append(dist.P2POp(dist.irecv, recv_top, rank - 1))
    if rank < world - 1:
        ops.append(dist.P2POp(dist.isend, send_bottom, rank + 1))
        ops.append(dist.P2POp(dist.irecv, recv_bottom, rank + 1))
    if ops:
        for req in dist.batch_isend_irecv(ops):
            req.wait()


class _Raw:
    """Device memory owned by the library, exposed through the CUDA array interface."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes // 2,), "typestr": "<f2", "data": (int(ptr), False),
                                         "version": 2}


class BandRunner:
    """Runs one row band of a model on this rank's GPU, swapping halo rows before every conv."""

    def __init__(self, model, image_h, width, rank, world, dist):
        import torch
        from . import lib
        self.torch, self.dist, self.rank, self.world = torch, dist, rank, world
        self.band = band_of(rank, world, image_h)
        self.inst = lib.Instance(model, self.band[2], width, band=self.band if world > 1 else None)
        self.n = model.dispatch_count()
        # exchange points grouped by the dispatch they precede, rows wrapped as torch views once
        self.points = {}
        for p in (self.inst.halo_points() if world > 1 else []):
            nb = int(p.row_bytes)
            wrap = lambda ptr: torch.as_tensor(_Raw(ptr, nb), device="cuda") if ptr else None
            self.points.setdefault(p.before_dispatch, []).append(
                (wrap(p.send_top), wrap(p.send_bottom), wrap(p.recv_top), wrap(p.recv_bottom)))
        self.cuts = sorted(self.points)

    def run(self, dev_in_ptr=None):
        """Enqueues the whole schedule on torch's current stream (input already in the instance's input tensor
        unless `dev_in_ptr` is given: then it is copied there first)."""
        torch = self.torch
        stream = torch.cuda.current_stream().cuda_stream
        first = 0
        for cut in self.cuts + [self.n]:
            if cut > first:
                self.inst.enqueue_range(first, cut, stream)
                first = cut
            for (st, sb, rt, rb) in self.points.get(cut, []):
                exchange_rows(self.dist, self.rank, self.world, st, sb, rt, rb)

    def io(self):
        return self.inst.io()
