"""The benchmark database file without a GPU: a FlatBuffer of the reference's schema (db.fbs: root table Db,
identifier "dbdb"), checked with an independent mini parser of the published binary format, through an
open -> writeback -> open round trip, and against damaged files."""
import ctypes as C
import struct

import pytest

from denox_b200 import lib, nets
from test_dnx_cpu import FB


class DbFB(FB):
    def root(self):
        assert self.b[4:8] == b"dbdb"
        return self.u("I", 0)


def conv_dispatch(variant_config="DY=stack#KG=1#W=resident", c=32, k=32, h=64, w=128, flags=lib.F_RELU):
    d = lib.Dispatch()
    d.variant = lib.find_variant("direct-conv-tc", variant_config)
    d.flags, d.c_a, d.c_out = flags, c, k
    d.pc[0], d.pc[1] = w, h
    return d


def filled_db(path):
    db = lib.Db(path)
    added = db.populate(nets.tiny_unet(), 64, 128, device=-1)
    assert added > 0
    d = conv_dispatch()
    db.add_result(d, [0.5, 0.25, 0.75, 0.5])
    db.writeback()
    return db, d, added


def test_file_is_a_db_fbs_flatbuffer(tmp_path):
    path = tmp_path / "gpu.db"
    db, d, added = filled_db(path)
    total = len(db)
    db.close()
    data = path.read_bytes()
    fb = DbFB(data)
    root = fb.root()
    assert fb.u("I", fb.field(root, 0)) == 0 if fb.field(root, 0) else True   # version 0, as the reference writes
    # env: the one session that added samples
    n_env, _ = fb.vector(root, 1)
    assert n_env == 1
    env = fb.table_at(root, 1, 0)
    assert fb.string(env, 0) and fb.string(env, 4).startswith("dnxcu")
    assert len(fb.string(env, 3)) == 64                                        # source digest in the commit hash field
    assert fb.u("H", fb.field(env, 6)) == 1                                    # ClockMode None: clocks are not touched
    # binaries: eight identity words and the DNXC descriptor
    n_bin, _ = fb.vector(root, 2)
    assert n_bin >= 1
    sha_of = []
    for i in range(n_bin):
        b = fb.table_at(root, 2, i)
        n, p = fb.vector(b, 0)
        assert n == 8
        sha_of.append("".join(f"{fb.u('I', p + 4 * k):08x}" for k in range(8)))
        n, p = fb.vector(b, 1)
        assert n >= 2 and data[p:p + 4] == b"DNXC"
    assert len(set(sha_of)) == n_bin
    # dispatches
    n_disp, _ = fb.vector(root, 3)
    assert n_disp == total
    want_sha = lib.variant_sha256(d.variant)
    found = 0
    for i in range(n_disp):
        t = fb.table_at(root, 3, i)
        bid = fb.u("I", fb.field(t, 0)) if fb.field(t, 0) else 0
        n, p = fb.vector(t, 4)
        assert n == 24
        pc = struct.unpack_from("<6I", data, p)
        info = fb.table_at(t, 8)
        assert fb.string(info, 0) and fb.string(info, 1) and fb.string(info, 2)
        tm = fb.table_at(t, 7)
        ns, _ = fb.vector(tm, 0)
        if sha_of[bid] == want_sha and pc == (128, 64, 32, 0, 32, lib.F_RELU):
            found += 1
            assert ns == 4
            lat = [fb.u("Q", fb.field(fb.table_at(tm, 0, k), 1)) for k in range(4)]
            assert lat == [500000, 250000, 750000, 500000]
            assert fb.u("Q", fb.field(tm, 1)) == 500000                       # mean in ns
            assert abs(fb.u("Q", fb.field(tm, 2)) - 204124) <= 1               # standard deviation in ns
            assert fb.string(info, 1) == "direct-conv-tc" and fb.string(info, 2) == "DY=stack#KG=1#W=resident"
            assert fb.u("Q", fb.field(info, 5)) == 2 * 64 * 128 * 9 * 32 * 32   # flops
            assert fb.u("B", fb.field(info, 6)) == 1                            # coopmat: a tensor core variant
            assert fb.u("I", fb.field(t, 1)) >= 1                               # workgroup count x
        else:
            assert ns == 0
    assert found == 1


def test_round_trip_keeps_samples_sessions_and_unknown_identities(tmp_path):
    path = tmp_path / "gpu.db"
    db, d, _ = filled_db(path)
    total = len(db)
    db.close()
    first = path.read_bytes()
    db = lib.Db(path)
    assert len(db) == total
    mean, std, n = db.query(d)
    assert n == 4 and abs(mean - 0.5) < 1e-12 and abs(std - 0.2041241452) < 1e-6
    db.writeback()
    assert path.read_bytes() == first          # nothing added: the file is reproduced byte for byte
    db.add_result(d, [1.0])                    # a second session appends its own environment record
    db.writeback()
    db.close()
    fb = DbFB(path.read_bytes())
    assert fb.vector(fb.root(), 1)[0] == 2
    # an entry whose identity this build does not know (another build's kernels) survives open + writeback
    data = bytearray(path.read_bytes())
    root = fb.root()
    b0 = fb.table_at(root, 2, 0)
    _, p = fb.vector(b0, 0)
    data[p] ^= 0xFF
    path.write_bytes(bytes(data))
    db = lib.Db(path)
    assert len(db) == total
    db.writeback()
    db.close()
    fb2 = DbFB(path.read_bytes())
    _, p2 = fb2.vector(fb2.table_at(fb2.root(), 2, 0), 0)
    assert fb2.b[p2] == data[p]
    assert fb2.vector(fb2.root(), 3)[0] == total


def test_damaged_and_foreign_files_are_refused(tmp_path):
    path = tmp_path / "gpu.db"
    db, _, _ = filled_db(path)
    db.close()
    data = path.read_bytes()
    h = C.c_void_p()
    for name, blob in [("short", data[:6]), ("ident", data[:4] + b"dnxx" + data[8:]), ("text", b"dnxcu-db 1\n")]:
        p = tmp_path / f"{name}.db"
        p.write_bytes(blob)
        assert lib.L.dnxcu_db_open(str(p).encode(), C.byref(h)) == lib.E_IO
    # truncations and bit flips: an error or an opened database, never a crash
    for cut in (16, len(data) // 3, len(data) // 2, len(data) - 5):
        p = tmp_path / f"cut{cut}.db"
        p.write_bytes(data[:cut])
        st = lib.L.dnxcu_db_open(str(p).encode(), C.byref(h))
        assert st in (0, lib.E_IO)
        if st == 0:
            lib.L.dnxcu_db_close(h)
    for pos in range(8, min(len(data), 4000), 37):
        b = bytearray(data)
        b[pos] ^= 0x5A
        p = tmp_path / "flip.db"
        p.write_bytes(bytes(b))
        st = lib.L.dnxcu_db_open(str(p).encode(), C.byref(h))
        assert st in (0, lib.E_IO)
        if st == 0:
            lib.L.dnxcu_db_close(h)
    # a database whose binaries are SPIR-V (the reference's own) holds timings of other kernels: refused
    fb = DbFB(data)
    _, p = fb.vector(fb.table_at(fb.root(), 2, 0), 1)
    b = bytearray(data)
    b[p:p + 4] = struct.pack("<I", 0x07230203)
    q = tmp_path / "spirv.db"
    q.write_bytes(bytes(b))
    assert lib.L.dnxcu_db_open(str(q).encode(), C.byref(h)) == lib.E_IO
