"""`save` / `load`: the checkpoint file format is the reference's (anvil/interp.py:341-372,
anvil/backend/anvil_host.h:237-266): "EINW", version 2, tensor count, one key per tensor (shape hash
and element count), raw little-endian payloads. The reference interpreter printed
`loaded 0.0000 sum 11.7199` on the first run of tests/programs/save_load.anvil and
`loaded 1.0000 sum 11.7199` on the second. Here: the oracle does the same, the device does the same,
and each reads the file the other wrote."""
import io
import os
import struct

import pytest

from anvil_lang_b200 import kir
from oracle.kir_interp import Oracle
from util import GOLDEN

FIRST, SECOND = "loaded 0.0000 sum 11.7199\n", "loaded 1.0000 sum 11.7199\n"


def program(path):
    prog = kir.load(os.path.join(GOLDEN, "save_load.kir.json.gz"))
    for blk in kir.walk_blocks(prog.main):
        for st in blk.stmts:
            if isinstance(st, kir.RTCall) and "path" in st.args:
                st.args["path"] = path
    return prog


def run_oracle(path):
    out = io.StringIO()
    Oracle(program(path), out=out, seed=0).run()
    return out.getvalue()


def run_device(path):
    from anvil_lang_b200.program import DeviceProgram
    dp = DeviceProgram(program(path), seed=0)
    try:
        code, text = dp.run(capture=True)
        assert code == 0, dp.error
        return text
    finally:
        dp.close()


def test_oracle_saves_then_loads(tmp_path):
    f = str(tmp_path / "w.weights")
    assert run_oracle(f) == FIRST
    raw = open(f, "rb").read()
    magic, version, count = struct.unpack_from("<4sIQ", raw)
    assert (magic, version, count) == (b"EINW", 2, 4)
    keys = struct.unpack_from("<4Q", raw, 16)
    assert [k & 0xFFFFFFFF for k in keys] == [12, 4, 8, 2]
    assert len(raw) == 16 + 8 * 4 + 4 * (12 + 4 + 8 + 2)
    assert run_oracle(f) == SECOND


@pytest.mark.gpu
def test_device_saves_then_loads_and_files_are_interchangeable(tmp_path):
    f = str(tmp_path / "dev.weights")
    assert run_device(f) == FIRST
    assert run_device(f) == SECOND
    assert run_oracle(f) == SECOND                      # the oracle reads the device's file
    g = str(tmp_path / "cpu.weights")
    assert run_oracle(g) == FIRST
    assert run_device(g) == SECOND                      # the device reads the oracle's file
    a, b = open(f, "rb").read(), open(g, "rb").read()
    assert a[:48] == b[:48] and len(a) == len(b)        # same header and keys, same size
    with open(g, "r+b") as h:                           # a damaged file is refused, not half-loaded
        h.seek(20)
        h.write(b"\x01")
    assert run_device(g) == FIRST.replace("0.0000", "0.0000")
