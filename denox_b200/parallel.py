"""Multi-GPU execution of the dispatch schedule: one process per GPU.

Two ways to shard, both without touching the conv kernels:

* frame parallel — independent frames, round robin over ranks, no exchange;
* row bands — rank r owns rows [r*H/G, (r+1)*H/G) of every tensor (at every
  resolution level).  A 3x3 conv needs one row of each operand from the band
  above and below.  The rows land in halo slabs of the consumer's own memory
  (`dnxcu_dispatch.halo`); image borders keep NULL slabs (zero padding).  Pool
  and nearest upsample need no halo because band heights are multiples of 16.
  Two transports:
    - "peer": the library's own exchange kernel in front of every conv writes
      the boundary rows straight into the neighbours' slabs over NVLink (peer
      mappings of the slab allocations, exchanged once through
      `torch.distributed` as IPC handles) and waits, bounded, for theirs; the
      whole frame, exchange included, replays from one CUDA graph;
    - "nccl": `torch.distributed` send/recv in front of every conv (NCCL on
      GPUs, gloo in the CPU tests): bootstrap and fallback.

The reference has no multi-device code at all; this module is new.
"""
import ctypes as C

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


def check_bands(dist, rank: int, world: int, band, width: int):
    """Every rank tells the others which band it holds; raises ValueError on all ranks when the bands do not
    tile one image (unequal heights or widths, a gap, an overlap, different image heights)."""
    mine = [int(band[0]), int(band[1]), int(band[2]), int(width)]
    allb = [None] * world
    dist.all_gather_object(allb, mine)
    problem = None
    if any(b[0] != allb[0][0] or b[3] != allb[0][3] for b in allb):
        problem = f"ranks disagree on the image extent: {allb}"
    elif any(b[2] != allb[0][2] for b in allb):
        problem = f"band heights differ: {[b[2] for b in allb]}"
    elif any(allb[r][1] != r * allb[0][2] for r in range(world)) or allb[-1][1] + allb[-1][2] != allb[0][0]:
        problem = f"bands do not tile the image: {allb}"
    if problem:
        raise ValueError(problem)


def exchange_rows(dist, rank, world, send_top, send_bottom, recv_top, recv_bottom):
    """Swaps boundary rows with the neighbouring bands.

    send_top / send_bottom: this band's first / last row (tensors);
    recv_top / recv_bottom: where the row above / below must land (None at an image border).
    All ranks must call this for the same exchange point in the same order.  A neighbour that never
    shows up makes the wait end with the process group's timeout (an exception), not hang."""
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
    """Runs one row band of a model on this rank's GPU.

    exchange: "peer" (direct stores into the neighbours' slabs), "nccl" (send/recv before every conv) or
    "auto" (peer when every rank could connect, else nccl)."""

    def __init__(self, model, image_h, width, rank, world, dist, exchange="auto"):
        import torch
        from . import lib
        self.torch, self.dist, self.rank, self.world = torch, dist, rank, world
        self.band = band_of(rank, world, image_h)
        if world > 1:
            check_bands(dist, rank, world, self.band, width)
        self.inst = lib.Instance(model, self.band[2], width, band=self.band if world > 1 else None)
        self.n = model.dispatch_count()
        self.transport = "none" if world == 1 else "nccl"
        if world > 1 and exchange in ("auto", "peer"):
            ok = 1
            try:
                mine = bytes(self.inst.halo_export())
            except lib.DnxcuError:
                mine, ok = b"", 0
            handles = [None] * world
            dist.all_gather_object(handles, mine)
            if ok and all(len(h) == C.sizeof(lib.PeerHandle) for h in handles):
                up = lib.PeerHandle.from_buffer_copy(handles[rank - 1]) if rank > 0 else None
                down = lib.PeerHandle.from_buffer_copy(handles[rank + 1]) if rank < world - 1 else None
                try:
                    self.inst.halo_connect(up, down, auto_exchange=False)
                except lib.DnxcuError:
                    ok = 0
            else:
                ok = 0
            t = torch.tensor([ok], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MIN)
            if int(t.item()) == 1:
                self.inst.halo_auto(True)
                self.transport = "peer"
            elif exchange == "peer":
                raise RuntimeError("peer halo exchange could not be set up on every rank")
        # exchange points grouped by the dispatch they precede, rows wrapped as torch views once (nccl transport)
        self.points = {}
        for p in (self.inst.halo_points() if world > 1 else []):
            nb = int(p.row_bytes)
            wrap = lambda ptr: torch.as_tensor(_Raw(ptr, nb), device="cuda") if ptr else None
            self.points.setdefault(p.before_dispatch, []).append(
                (wrap(p.send_top), wrap(p.send_bottom), wrap(p.recv_top), wrap(p.recv_bottom)))
        self.cuts = sorted(self.points)

    def run(self):
        """Enqueues the whole schedule on torch's current stream; the band's input is in the instance's input
        tensor (see io())."""
        torch = self.torch
        stream = torch.cuda.current_stream().cuda_stream
        if self.transport in ("peer", "none"):
            din, dout = self.inst.io()
            self.inst.enqueue(din, dout, stream)  # one graph replay; with "peer" the exchange kernels are in it
            return
        first = 0
        for cut in self.cuts + [self.n]:
            if cut > first:
                self.inst.enqueue_range(first, cut, stream)
                first = cut
            for (st, sb, rt, rb) in self.points.get(cut, []):
                exchange_rows(self.dist, self.rank, self.world, st, sb, rt, rb)

    def exchanges_per_frame(self):
        """Exchange steps between dispatches: one kernel per conv with "peer", one send/recv group per conv
        operand with "nccl"."""
        if self.transport == "peer":
            return len(self.cuts)
        return sum(len(v) for v in self.points.values())

    def io(self):
        return self.inst.io()
