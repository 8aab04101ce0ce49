"""dnx files without a GPU: the hand written FlatBuffers codec and the writer / reader of the compiled-model
container (dnx.fbs of the reference), checked structurally with an independent mini parser of the published
binary format, and through a write -> read -> write round trip."""
import struct

import numpy as np
import pytest

from denox_b200 import lib, nets


class FB:
    """Independent reader of the FlatBuffers wire format (only what the checks below need)."""

    def __init__(self, buf):
        self.b = buf

    def u(self, fmt, pos):
        return struct.unpack_from("<" + fmt, self.b, pos)[0]

    def root(self):
        assert self.b[4:8] == b"dnxx"
        return self.u("I", 0)

    def field(self, table, slot):
        vt = table - self.u("i", table)
        vsize = self.u("H", vt)
        if 4 + 2 * slot + 2 > vsize:
            return 0
        off = self.u("H", vt + 4 + 2 * slot)
        return table + off if off else 0

    def indirect(self, pos):
        return pos + self.u("I", pos)

    def string(self, table, slot):
        f = self.field(table, slot)
        p = self.indirect(f)
        n = self.u("I", p)
        assert self.b[p + 4 + n] == 0
        return self.b[p + 4:p + 4 + n].decode()

    def vector(self, table, slot):
        f = self.field(table, slot)
        if not f:
            return 0, 0
        p = self.indirect(f)
        return self.u("I", p), p + 4

    def table_at(self, table, slot, i=None):
        if i is None:
            return self.indirect(self.field(table, slot))
        n, p = self.vector(table, slot)
        assert i < n
        return self.indirect(p + 4 * i)


@pytest.mark.parametrize("which", ["tiny_bias", "oidn", "tiny_leaky_unfused"])
def test_model_dnx_structure_and_round_trip(which):
    if which == "oidn":
        net, options = nets.oidn_unet(), 0
    elif which == "tiny_bias":
        net, options = nets.tiny_unet(bias=True), 0
    else:
        net, options = nets.tiny_unet(leaky=0.1), lib.OPT_NO_FUSE_ACTIVATION | lib.OPT_NO_FUSE_POOL
    m = lib.Model(net, device=-1, options=options)
    data = m.write_dnx()
    check_structure(data, net)
    # read it back (parse only) and write it again: the same bytes
    m2 = lib.Model.from_dnx(data, device=-1)
    assert m2.dispatch_count() == m.dispatch_count()
    assert m2.io()[1] == net.in_channels
    assert m2.write_dnx() == data
    m.close(); m2.close()


def check_structure(data, net):
    fb = FB(data)
    root = fb.root()
    assert root % 4 == 0
    n_disp, _ = fb.vector(root, 8)
    n_conv = sum(1 for nd in net.nodes if nd.kind == nets.CONV)
    assert n_disp >= n_conv
    n_tensors, _ = fb.vector(root, 3)
    n_buffers, _ = fb.vector(root, 7)
    assert n_tensors == n_buffers  # one buffer per tensor, like the reference's memory plan
    n_inits, _ = fb.vector(root, 4)
    assert n_inits >= n_conv
    n_in, p_in = fb.vector(root, 5)
    n_out, p_out = fb.vector(root, 6)
    assert n_in == n_out == 1
    # symbolic expression list over two variables (H, W); struct SymIROp is 24 bytes, 8 byte aligned
    sym = fb.table_at(root, 10)
    assert fb.u("H", fb.field(sym, 0)) == 2
    n_ops, p_ops = fb.vector(sym, 1)
    assert n_ops > 0 and p_ops % 8 == 0
    names = [fb.string(fb.table_at(root, 11, i), 0) for i in range(fb.vector(root, 11)[0])]
    assert names[:2] == ["H", "W"] and "ALIGN" in names
    # every dispatch: entry point = variant family, binary starts with the magic that tells it from SPIR-V
    for i in range(n_disp):
        d = fb.table_at(root, 8, i)
        entry = fb.string(d, 7)
        assert entry in {v["family"] for v in lib.variants()}
        bid = fb.u("I", fb.field(d, 0)) if fb.field(d, 0) else 0
        b = fb.table_at(root, 9, bid)
        nw, pw = fb.vector(b, 0)
        assert nw >= 10 and pw % 4 == 0
        assert fb.u("I", pw) == 0x43584E44 != 0x07230203
        pc = fb.table_at(d, 9)
        assert fb.u("H", fb.field(pc, 0)) == 8
        assert fb.vector(pc, 1)[0] == 2
        set0 = fb.table_at(d, 8, 0)
        nb, _ = fb.vector(set0, 1)
        assert 2 <= nb <= 6
        for k in range(nb):
            bind = fb.table_at(set0, 1, k)
            t = fb.u("I", fb.field(bind, 2)) if fb.field(bind, 2) else 0
            assert t < n_tensors
            assert (fb.u("H", fb.field(bind, 0)) if fb.field(bind, 0) else 0) == k


def _parse_only(data):
    import ctypes as C
    h = C.c_void_p()
    st = lib.L.dnxcu_model_create_from_dnx(data, len(data), -1, C.byref(h))
    return st, h


def test_reader_refuses_garbage_and_spirv_without_crashing():
    import ctypes as C
    for junk in (b"", b"\x00" * 7, b"\x10\x00\x00\x00dnxx" + b"\xff" * 64, b"\x08\x00\x00\x00nope" + b"\x00" * 32):
        st, h = _parse_only(junk)
        assert st < 0


def test_truncated_and_corrupted_files_are_refused():
    """Every prefix of a valid file, and the file with single bytes flipped, either parses to an equivalent model or
    is refused: the bounds checked reader never reads outside the buffer."""
    net = nets.tiny_unet()
    m = lib.Model(net, device=-1)
    data = m.write_dnx()
    for cut in list(range(0, 64)) + list(range(64, len(data), max(1, len(data) // 40))):
        st, h = _parse_only(data[:cut])
        if st == 0:
            lib.L.dnxcu_model_destroy(h)
    rs = np.random.RandomState(3)
    for _ in range(200):
        b = bytearray(data)
        pos = int(rs.randint(0, min(len(b), 4096)))
        b[pos] ^= 1 << int(rs.randint(0, 8))
        st, h = _parse_only(bytes(b))
        if st == 0:
            lib.L.dnxcu_model_destroy(h)
    m.close()
