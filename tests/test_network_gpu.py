"""Whole network parity on the GPU through the model / instance runtime (host in,
host out, like Instance::infer), free running and per tensor, against the CPU
oracle and the golden fixtures."""
import os

import numpy as np
import pytest

from conftest import assert_close, error_report
from denox_b200 import lib, nets
from oracle import oracle

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
GOLD = np.load(os.path.join(HERE, "golden", "golden.npz"))


def fetch(inst, tid):
    from gpu_util import wrap
    p, h, w, c = inst.tensor(tid)
    return wrap(p, (h, w, c)).cpu().numpy()


@pytest.mark.parametrize("options", [0, lib.OPT_NO_TCGEN05, lib.OPT_NO_PAD_INPUT,
                                     lib.OPT_NO_FUSE_POOL | lib.OPT_NO_FUSE_UPSAMPLE | lib.OPT_NO_FUSE_CONCAT
                                     | lib.OPT_NO_FUSE_ACTIVATION])
@pytest.mark.parametrize("which,shape,seed,key", [
    ("tiny", (128, 128), 1000, "tiny/out"),
    ("tiny_bias", (48, 80), 1001, "tiny_bias/out"),
    ("oidn", (32, 48), 1000, "oidn_32x48/out"),
])
def test_network_matches_oracle_and_golden(which, shape, seed, key, options):
    if which == "oidn":
        net, x = nets.oidn_unet(), nets.oidn_input(seed, *shape)
    else:
        net, x = nets.tiny_unet(bias=(which == "tiny_bias")), nets.tiny_input(seed, *shape)
    model = lib.Model(net, options=options)
    inst = lib.Instance(model, *shape)
    y = inst.infer(x)
    y2 = inst.infer(x)  # second call replays the captured graph
    assert (y == y2).all()
    ref32 = oracle.run_network(net, x, oracle.ACC_F32)
    ref16 = oracle.run_network(net, x, oracle.ACC_F16)
    assert_close(y, ref32[net.output_tensor], f"{which} end to end vs acc=f32 oracle")
    assert_close(y, ref16[net.output_tensor], f"{which} end to end vs acc=f16 oracle", max_violation_fraction=1e-3)
    assert_close(y, GOLD[key], f"{which} end to end vs PyTorch golden")
    # every materialised tensor, free running
    for info in inst.dispatch_info():
        tid = info.out_tensor
        if tid not in ref32:
            # the zero padded copy of a ragged input (not a tensor of the model)
            got = fetch(inst, tid)
            c = x.shape[2]
            assert (got[:, :, :c] == x).all() and (got[:, :, c:] == 0).all()
            continue
        got = fetch(inst, tid)
        rep = assert_close(got, ref32[tid], f"{which} tensor {tid} ({info.name.decode()})")
        assert rep["max"] < 0.05
    if options == 0:
        n_conv = sum(1 for nd in net.nodes if nd.kind == nets.CONV)
        # pool / upsample / concat / relu all fused away; one extra copy pads the ragged input to 16 channels
        assert model.dispatch_count() == n_conv + 1
    inst.close()
    model.close()


@pytest.mark.parametrize("key,seed,shape", [("ref_unet_32x48/out", 1010, (32, 48)), ("ref_unet_40x52/out", 1011, (40, 52))])
def test_reference_model_file_output(key, seed, shape):
    """The GPU schedule against the output of the reference's own PyTorch module (oidn_model.py UNet behind
    UNetAlignment, run when the fixture was made): its channel list (160 = 96 + 64 into the first decoder conv),
    biases on every conv, an aligned extent and one that runs behind pad and slice."""
    net = nets.oidn_unet_reference()
    x = nets.oidn_input(seed, *shape)
    model = lib.Model(net)
    inst = lib.Instance(model, *shape)
    y = inst.infer(x)
    assert_close(y, GOLD[key], f"{key}: GPU vs the reference's PyTorch module")
    ref32 = oracle.run_network_aligned(net, x, 16, oracle.ACC_F32)
    assert_close(y, ref32, f"{key}: GPU vs acc=f32 oracle")
    inst.close()
    model.close()


def test_tiny_net_with_leaky_relu():
    net = nets.tiny_unet(leaky=0.1)
    x = nets.tiny_input(1003, 32, 48)
    ref = oracle.run_network(net, x, oracle.ACC_F32)
    for options in (0, lib.OPT_NO_TCGEN05, lib.OPT_NO_FUSE_ACTIVATION):
        model = lib.Model(net, options=options)
        inst = lib.Instance(model, 32, 48)
        y = inst.infer(x)
        names = [i.name.decode() for i in inst.dispatch_info()]
        assert_close(y, ref[net.output_tensor], f"tiny leaky, options {options}")
        assert_close(y, GOLD["tiny_leaky/out"], f"tiny leaky vs PyTorch golden, options {options}")
        if options == lib.OPT_NO_FUSE_ACTIVATION:
            assert any("basic-activation(leaky)" in n for n in names), names
        else:
            assert any("+leaky" in n for n in names), names
        inst.close()
        model.close()


def test_wide_conv_before_pool_runs_unfused():
    """conv(-> 1024) + relu + maxpool: no variant with a pooling epilogue takes 1024 output channels, so the
    schedule keeps conv (CUDA core variant) and basic-pool apart instead of refusing the model."""
    n = nets._start("wide", 8)
    x = n.conv(0, 1024, name="wide_conv")
    p = n.pool(x, "pool")
    o = n.conv(p, 8, relu=False, name="out_conv")
    n.output_tensor = o
    frame = nets.rng.to_f16(nets.rng.uniform(31, 16 * 24 * 8, -1, 1)).reshape(16, 24, 8)
    model = lib.Model(n)
    inst = lib.Instance(model, 16, 24)
    names = [i.name.decode() for i in inst.dispatch_info()]
    assert any(nm.startswith("basic-pool") for nm in names), names
    y = inst.infer(frame)
    ref = oracle.run_network(n, frame, oracle.ACC_F32)[n.output_tensor]
    assert_close(y, ref, "conv(->1024)+pool, un-fused")
    inst.close()
    model.close()


def test_enqueue_caches_graphs_per_pointer_pair_and_clears_nothing():
    """Device resident enqueue with two alternating (input, output) pairs: both replay from their own graph,
    results equal the host path's."""
    import torch
    net = nets.tiny_unet()
    model = lib.Model(net)
    inst = lib.Instance(model, 64, 128)
    xs = [nets.tiny_input(40 + i, 64, 128) for i in range(2)]
    want = [inst.infer(x) for x in xs]
    din = [torch.from_numpy(x).cuda() for x in xs]
    dout = [torch.empty((64, 128, 3), dtype=torch.float16, device="cuda") for _ in xs]
    s = torch.cuda.Stream()
    for rep in range(3):
        for i in range(2):
            inst.enqueue(din[i].data_ptr(), dout[i].data_ptr(), s.cuda_stream)
    s.synchronize()
    for i in range(2):
        assert (dout[i].cpu().numpy() == want[i]).all()
    inst.close()
    model.close()


def test_oidn_larger_frame_properties():
    """At a size the oracle still finishes in seconds: 96 x 256."""
    net = nets.oidn_unet()
    x = nets.oidn_input(1003, 96, 256)
    model = lib.Model(net)
    inst = lib.Instance(model, 96, 256)
    y = inst.infer(x)
    ref = oracle.run_network(net, x, oracle.ACC_F32)[net.output_tensor]
    rep = assert_close(y, ref, "oidn 96x256")
    print("oidn 96x256 end-to-end", rep)
    infos, total = inst.bench(warmup=1, iters=2)
    assert total > 0 and all(i.ms > 0 for i in infos)
    inst.close()
    model.close()


def test_unaligned_extent_runs_behind_pad_and_slice():
    """A frame whose extent is not a multiple of 16 (the reference pads such frames by edge replication and
    slices the output, oidn_model.py:334-347): the instance does both, results as the oracle's wrapper and
    PyTorch's."""
    net = nets.oidn_unet()
    model = lib.Model(net)
    inst = lib.Instance(model, 40, 52)
    assert inst.extent() == (40, 52, 48, 64)
    x = nets.oidn_input(1002, 40, 52)
    y = inst.infer(x)
    assert y.shape == (40, 52, 3)
    ref = oracle.run_network_aligned(net, x)
    assert_close(y, ref, "oidn 40x52 behind pad/slice vs oracle")
    assert_close(y, GOLD["oidn_40x52_aligned/out"], "oidn 40x52 behind pad/slice vs PyTorch golden")
    # stream ordered form with the same buffers
    import torch
    xs = torch.from_numpy(x).pin_memory()
    ys = torch.empty((40, 52, 3), dtype=torch.float16).pin_memory()
    inst.infer_async(xs.numpy(), ys.numpy())
    inst.wait()
    assert (ys.numpy().view(np.uint16) == y.view(np.uint16)).all()
    inst.close()
    # a row band must still be aligned: bands of an unaligned frame are not offered
    with pytest.raises(lib.DnxcuError):
        lib.Instance(model, 24, 52, band=(40, 0, 24))
    model.close()


def test_database_populate_bench_select(tmp_path):
    """populate -> bench -> selection, the reference's `denox populate / bench / compile` flow, on a small frame."""
    net = nets.tiny_unet()
    db = lib.Db(tmp_path / "gpu.db")
    added = db.populate(net, 64, 128)
    assert added >= 5
    db.bench(min_samples=3, max_relative_error=0.5, max_rounds=2)
    db.close()
    db = lib.Db(tmp_path / "gpu.db")          # resumes from the file (checkpoint semantics of the reference)
    assert len(db) == added
    assert db.populate(net, 64, 128) == 0
    model = lib.Model(net, db=db)
    inst = lib.Instance(model, 64, 128)
    x = nets.tiny_input(7, 64, 128)
    y = inst.infer(x)
    ref = oracle.run_network(net, x, oracle.ACC_F32)[net.output_tensor]
    assert_close(y, ref, "tiny with database selected variants")
    # every chosen variant must be one the database has timed
    import ctypes as C
    for info in inst.dispatch_info():
        d = lib.Dispatch()
        d.variant, d.flags, d.c_a, d.c_b, d.c_out = info.variant, info.flags, info.c_a, info.c_b, info.c_out
        d.pc[0], d.pc[1] = info.w, info.h
        assert db.query(d) is not None, info.name
    inst.close(); model.close(); db.close()


def test_selection_prefers_the_unfused_schedule_when_the_database_says_so(tmp_path):
    """Schedule selection by cost: with every candidate timed, the default choice is the fused schedule; after the
    database is told that every conv with a pooling epilogue takes 100 ms, the search picks conv + basic-pool
    instead, and the result still matches the oracle."""
    net = nets.tiny_unet()
    x = nets.tiny_input(9, 64, 128)
    ref = oracle.run_network(net, x, oracle.ACC_F32)[net.output_tensor]
    opts = lib.OPT_SELECT_BY_COST_ONLY
    db = lib.Db(tmp_path / "sel.db")
    assert db.populate(net, 64, 128, options=opts) > 20
    db.bench(min_samples=3, max_relative_error=0.5, max_rounds=1)
    model = lib.Model(net, db=db, options=opts)
    inst = lib.Instance(model, 64, 128)
    names = [i.name.decode() for i in inst.dispatch_info()]
    assert_close(inst.infer(x), ref, "selected schedule")
    inst.close()
    # poison every fused conv + pool candidate of conv0 (16 output channels, full output kept for the skip
    # connection), whichever way it reads the 3 channel input
    for v in lib.variants():
        if v["op"] != lib.OP_CONV3X3 or not (v["allowed_flags"] & lib.F_POOL_OUT):
            continue
        for c_in in (3, 16):
            d = lib.Dispatch()
            d.variant, d.flags, d.c_a, d.c_out = v["id"], lib.F_RELU | lib.F_POOL_OUT, c_in, 16
            d.pc[0], d.pc[1] = 128, 64
            db.add_result(d, [100.0] * 50)
    inst2 = lib.Instance(model, 64, 128)
    names2 = [i.name.decode() for i in inst2.dispatch_info()]
    assert any(n.startswith("basic-pool") for n in names2), (names, names2)
    assert not any("+pool" in n for n in names2), names2
    assert inst2.dispatch_count() == len(names2)
    assert_close(inst2.infer(x), ref, "un-fused schedule chosen by cost")
    inst2.close()
    model.close()
    db.close()


@pytest.mark.parametrize("which,shape,other", [("tiny", (128, 128), (64, 160)), ("oidn", (64, 96), (32, 48)),
                                               ("oidn", (40, 52), (64, 96))])
def test_dnx_round_trip_runs_bit_identical(which, shape, other):
    """model -> dnx file -> model: the file's dispatches give the same bits as the node list path, at the extent
    the instance was made for and (the file's extents are symbolic) at another one."""
    net = nets.oidn_unet() if which == "oidn" else nets.tiny_unet(bias=True)
    mk = (lambda seed, hw: nets.oidn_input(seed, *hw)) if which == "oidn" else (lambda seed, hw: nets.tiny_input(seed, *hw))
    model = lib.Model(net)
    inst = lib.Instance(model, *shape)
    x = mk(77, shape)
    y = inst.infer(x)
    blob = inst.write_dnx()
    assert blob[4:8] == b"dnxx" and len(blob) > 1000
    m2 = lib.Model.from_dnx(blob)
    i2 = lib.Instance(m2, *shape)
    assert i2.dispatch_count() == inst.dispatch_count()
    assert [a.variant for a in i2.dispatch_info()] == [a.variant for a in inst.dispatch_info()]
    y2 = i2.infer(x)
    assert (y2.view(np.uint16) == y.view(np.uint16)).all()
    # the same file at another extent against the node list path at that extent
    x3 = mk(78, other)
    i3a, i3b = lib.Instance(model, *other), lib.Instance(m2, *other)
    assert (i3a.infer(x3).view(np.uint16) == i3b.infer(x3).view(np.uint16)).all()
    # the extent independent file written from the model alone
    m4 = lib.Model.from_dnx(model.write_dnx())
    i4 = lib.Instance(m4, *shape)
    ref = oracle.run_network_aligned(net, x, 16 if which == "oidn" else 2, oracle.ACC_F32)
    assert_close(i4.infer(x), ref, "dnx written from the model")
    for o in (inst, i2, i3a, i3b, i4, m2, m4, model):
        o.close()


def test_onnx_import_runs_like_the_node_list():
    """ONNX bytes -> model -> instance: the same bits as the same network handed over as a node list."""
    import sys
    sys.path.insert(0, HERE)
    import onnx_writer
    net = nets.oidn_unet_reference()
    x = nets.oidn_input(55, 48, 80)
    a = lib.Model(net)
    b = lib.Model.from_onnx(onnx_writer.from_net(net))
    ia, ib = lib.Instance(a, 48, 80), lib.Instance(b, 48, 80)
    assert (ia.infer(x).view(np.uint16) == ib.infer(x).view(np.uint16)).all()
    with pytest.raises(lib.DnxcuError) as err:
        lib.Model.from_onnx(b"\x08\x08")
    assert "ONNX import" in str(err.value)
    for o in (ia, ib, a, b):
        o.close()


def test_cli_populate_bench_compile_infer(tmp_path):
    """The reference's three stage flow through the command line: populate a database for an assumed extent, bench
    it, compile the ONNX file to a dnx file with it, run a frame (an .npy file in, an .npy file out)."""
    import subprocess
    import sys
    sys.path.insert(0, HERE)
    import onnx_writer
    cli = os.path.join(os.path.dirname(lib.LIB_PATH), "dnxcu-cli")
    net = nets.tiny_unet(bias=True)
    onnx, db, dnx = tmp_path / "net.onnx", tmp_path / "gpu.db", tmp_path / "net.dnx"
    onnx.write_bytes(onnx_writer.from_net(net))

    def run(*args):
        p = subprocess.run([cli, *map(str, args)], capture_output=True, text=True, timeout=600)
        assert p.returncode == 0, (args, p.stdout, p.stderr)
        return p.stdout

    run("populate", db, onnx, "--assume", "H=64", "W=96")
    run("bench", db, "--samples=3", "--relative-error=0.5", "--rounds=1")
    out = run("compile", onnx, "-o", dnx, "--db", db, "--assume", "H=64", "W=96")
    assert "dispatches" in out and dnx.exists()
    x = nets.tiny_input(5, 64, 96)
    np.save(tmp_path / "x.npy", x)
    run("infer", dnx, "--input", tmp_path / "x.npy", "--output", tmp_path / "y.npy")
    y = np.load(tmp_path / "y.npy")
    assert y.dtype == np.float16 and y.shape == (64, 96, 3)
    ref = oracle.run_network(net, x, oracle.ACC_F32)[net.output_tensor]
    assert_close(y, ref, "frame through the command line")
    table = run("bench", dnx, "--spec", "H=64", "W=96", "--samples=3")
    assert "frames/s" in table and "direct-conv" in table


def test_infer_async_round_robin_matches_infer():
    import torch
    net = nets.tiny_unet()
    model = lib.Model(net)
    insts = [lib.Instance(model, 64, 128) for _ in range(2)]
    xs = [nets.tiny_input(20 + i, 64, 128) for i in range(4)]
    want = [insts[0].infer(x) for x in xs]
    pin_in = [torch.from_numpy(x).pin_memory() for x in xs]
    pin_out = [torch.empty((64, 128, 3), dtype=torch.float16).pin_memory() for _ in xs]
    for i in range(4):
        k = i % 2
        if i >= 2:
            insts[k].wait()
        insts[k].infer_async(pin_in[i].numpy(), pin_out[i].numpy())
    for inst in insts:
        inst.wait()
    for i in range(4):
        assert (pin_out[i].numpy() == want[i]).all()
    for inst in insts:
        inst.close()
    model.close()
