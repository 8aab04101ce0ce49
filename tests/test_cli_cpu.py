"""The command line front door without a GPU: version / help, compiling an ONNX file to a dnx file (no device
needed without a database), populating a database for an assumed extent, and its error behaviour."""
import os
import subprocess

import numpy as np
import pytest

import onnx_writer
from denox_b200 import lib, nets

CLI = os.path.join(os.path.dirname(lib.LIB_PATH), "dnxcu-cli")


def run(*args, ok=True):
    p = subprocess.run([CLI, *args], capture_output=True, text=True, timeout=120)
    if ok:
        assert p.returncode == 0, (args, p.stdout, p.stderr)
    return p


def test_version_and_help():
    assert os.path.exists(CLI), "the build step makes dnxcu-cli next to the library"
    assert "kernel variants" in run("version").stdout
    h = run("help").stdout
    for verb in ("populate", "bench", "compile", "infer"):
        assert verb in h
    assert run("frobnicate", ok=False).returncode != 0


def test_compile_onnx_to_dnx_without_a_device(tmp_path):
    net = nets.tiny_unet(bias=True)
    onnx = tmp_path / "net.onnx"
    onnx.write_bytes(onnx_writer.from_net(net))
    out = tmp_path / "net.dnx"
    # the reference's flag set is accepted where this backend has the same answer
    run("compile", str(onnx), "-o", str(out), "--type", "input=f16", "output=f16", "--shape", "input=H:W:C",
        "--storage", "input=ssbo", "output=ssbo", "--format", "input=hwc", "output=hwc", "--use-descriptor-sets", "1", "1", "1", "1", "1")
    want = lib.Model(net, device=-1)
    assert out.read_bytes() == want.write_dnx()
    want.close()
    # ... and refused where it has not
    p = run("compile", str(onnx), "-o", str(out), "--format", "input=chwc8", ok=False)
    assert p.returncode != 0 and "hwc" in p.stderr
    p = run("compile", str(tmp_path / "missing.onnx"), "-o", str(out), ok=False)
    assert p.returncode != 0 and "cannot open" in p.stderr
    bad = tmp_path / "bad.onnx"
    bad.write_bytes(b"\\xff" * 30)
    p = run("compile", str(bad), "-o", str(out), ok=False)
    assert p.returncode != 0 and "ONNX import" in p.stderr


def test_populate_for_an_assumed_extent(tmp_path):
    net = nets.tiny_unet()
    onnx = tmp_path / "net.onnx"
    onnx.write_bytes(onnx_writer.from_net(net))
    db = tmp_path / "gpu.db"
    out = run("populate", str(db), str(onnx), "--assume", "H=64", "W=128", "--device", "-1").stdout
    n = int(out.split()[0])
    assert n > 4 and db.exists()
    d = lib.Db(db)
    assert len(d) == n
    d.close()
    out = run("populate", str(db), str(onnx), "--assume", "H=64", "W=128", "--device", "-1").stdout
    assert out.startswith("0 dispatches added")  # populate extends, never duplicates
    assert run("populate", str(db), str(onnx), ok=False).returncode != 0  # no extent
