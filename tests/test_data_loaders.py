"""Data-file runtime calls (`load_idx`, `load_csv`, `load_bytes`, `input`): the oracle's restatement of
anvil/interp.py:243-305 on files written here, and — on a GPU — the C-ABI loaders against the oracle.

The files are synthetic (seeded bytes in the IDX layout: 16-byte header + u8 payload, plain and gzip; a
CSV with a header line and mixed separators; a raw byte file); no dataset is involved."""
import gzip
import io
import os
import subprocess
import sys

import numpy as np
import pytest

from anvil_lang_b200 import kir
from anvil_lang_b200.kir import F32, I32, Buffer, RTCall
from oracle.kir_interp import Oracle, OracleRuntimeError
from kirbuild import nid
from util import ROOT


def write_files(d):
    rng = np.random.default_rng(11)
    pix = rng.integers(0, 256, size=6 * 28 * 28, dtype=np.uint8)
    lab = rng.integers(0, 10, size=6, dtype=np.uint8)
    with gzip.open(os.path.join(d, "images.idx.gz"), "wb") as f:
        f.write(bytes(16) + pix.tobytes())
    with open(os.path.join(d, "labels.idx"), "wb") as f:
        f.write(bytes(8) + lab.tobytes())
    vals = rng.standard_normal(12).astype(np.float32)
    with open(os.path.join(d, "table.csv"), "w") as f:
        f.write("a,b,c,d\n")
        rows = ["%.6g, %.6g;%.6g\t%.6g" % tuple(vals[i:i + 4]) for i in range(0, 12, 4)]
        f.write("\n".join(rows) + "\n-.5,+2e1,.25,7.\n")
    raw = rng.integers(0, 256, size=40, dtype=np.uint8)
    with open(os.path.join(d, "text.bin"), "wb") as f:
        f.write(raw.tobytes())
    return pix, lab, raw


def loader_program(d):
    X = Buffer(nid(), "X", (6, 28, 28), F32, "temp")
    y = Buffer(nid(), "y", (6,), I32, "temp")
    T = Buffer(nid(), "T", (4, 4), F32, "temp")
    B = Buffer(nid(), "B", (40,), I32, "temp")
    calls = [RTCall("load_idx", {"buf": X, "path": os.path.join(d, "images.idx.gz"), "header": 16, "gz": True}),
             RTCall("load_idx", {"buf": y, "path": os.path.join(d, "labels.idx"), "header": 8, "gz": False}),
             RTCall("load_csv", {"buf": T, "path": os.path.join(d, "table.csv"), "skip": 1}),
             RTCall("load_bytes", {"buf": B, "path": os.path.join(d, "text.bin")})]
    return kir.Program(kir.Block(calls), [X, y, T, B], "loaders"), (X, y, T, B)


@pytest.fixture(autouse=True)
def data_dir_is_the_temporary_directory(tmp_path, monkeypatch):
    monkeypatch.setenv("ANVIL_DATA", str(tmp_path))


def test_oracle_loaders(tmp_path):
    d = str(tmp_path)
    pix, lab, raw = write_files(d)
    prog, (X, y, T, B) = loader_program(d)
    o = Oracle(prog, out=io.StringIO(), seed=0).run()
    assert np.array_equal(o.arr(X)[:X.numel], pix.astype(np.float32))
    assert np.array_equal(o.arr(y)[:y.numel], lab.astype(np.int32))
    assert np.array_equal(o.arr(B)[:B.numel], raw.astype(np.int32))
    t = o.arr(T)[:16]
    assert np.allclose(t[12:], [-0.5, 20.0, 0.25, 7.0]) and np.isfinite(t).all()


def test_oracle_rejects_a_short_file(tmp_path):
    d = str(tmp_path)
    write_files(d)
    prog, (X, y, T, B) = loader_program(d)
    with open(os.path.join(d, "text.bin"), "ab") as f:
        f.write(b"x")
    with pytest.raises(OracleRuntimeError):
        Oracle(prog, out=io.StringIO(), seed=0).run()


def test_loader_programs_survive_serialisation(tmp_path):
    prog, _ = loader_program(str(tmp_path))
    again = kir.loads(kir.dumps(prog))
    assert [s.name for s in again.main.stmts] == ["load_idx", "load_idx", "load_csv", "load_bytes"]
    assert again.main.stmts[0].args["header"] == 16


@pytest.mark.gpu
def test_device_loaders_match_the_oracle(tmp_path):
    from anvil_lang_b200.program import DeviceProgram
    d = str(tmp_path)
    write_files(d)
    prog, bufs = loader_program(d)
    o = Oracle(prog, out=io.StringIO(), seed=0).run()
    dp = DeviceProgram(prog, seed=0)
    try:
        code, _ = dp.run(capture=True)
        assert code == 0, dp.error
        for b in bufs:
            got = dp.read(b).reshape(-1)
            assert np.array_equal(got, o.arr(b)[:b.numel]), b.name       # bit-exact, strtof == float() on these texts
    finally:
        dp.close()


@pytest.mark.gpu
def test_device_loader_reports_a_wrong_shape_and_honours_the_data_directory(tmp_path):
    from anvil_lang_b200.program import DeviceProgram
    d = str(tmp_path)
    write_files(d)
    prog, bufs = loader_program(os.path.join(d, "elsewhere"))       # paths that do not exist: found through ANVIL_DATA
    try:
        dp = DeviceProgram(prog, seed=0)
        code, _ = dp.run(capture=True)
        assert code == 0, dp.error
        dp.close()
        with open(os.path.join(d, "text.bin"), "ab") as f:
            f.write(b"x")
        dp = DeviceProgram(prog, seed=0)
        code, _ = dp.run(capture=True)
        assert code == 1 and "does not have the shape this program was compiled for" in dp.error
        dp.close()
    finally:
        pass


INPUT_CHILD = r"""
import sys
sys.path.insert(0, {root!r}); sys.path.insert(0, {tests!r})
from anvil_lang_b200 import kir
from anvil_lang_b200.kir import F32, Buffer, RTCall, Print, PrintItem
from anvil_lang_b200.program import DeviceProgram
from kirbuild import nid
v = Buffer(nid(), "v", (), F32, "temp")
stmts = []
for _ in range(3):
    stmts += [RTCall("input", {{"buf": v}}), Print([PrintItem("scalar", "", v, "", None)], "\n", False)]
prog = kir.Program(kir.Block(stmts), [v], "input")
dp = DeviceProgram(prog, seed=0)
code, _ = dp.run()
sys.exit(code)
"""


@pytest.mark.gpu
def test_input_reads_numbers_until_the_end_of_the_input():
    child = INPUT_CHILD.format(root=ROOT, tests=os.path.join(ROOT, "tests"))
    r = subprocess.run([sys.executable, "-c", child], input="x = 2.5 apples\n-7\n", capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    lines = r.stdout.split("\n")
    assert float(lines[0]) == 2.5 and float(lines[1]) == -7.0 and lines[2] == ""      # third read: end of input -> newline, exit 0


@pytest.mark.gpu
def test_device_npy_loader_honours_the_data_directory(tmp_path):
    """`.npy` files are relocated by ANVIL_DATA like the other data files (reference anvil/backend/anvil_host.h:199):
    the program names a directory that does not exist, the file is found in the data directory; f32, i64 and f16
    payloads are converted to 32 bits."""
    from anvil_lang_b200.program import DeviceProgram
    d = str(tmp_path)
    rng = np.random.default_rng(5)
    cases = [("w.npy", rng.standard_normal((3, 5)).astype(np.float32), F32, 0, 4),
             ("idx.npy", rng.integers(-1000, 1000, size=7).astype(np.int64), I32, 4, 8),
             ("h.npy", rng.standard_normal(9).astype(np.float16), F32, 2, 2)]
    bufs, calls = [], []
    for name, arr, dt, kind, size in cases:
        np.save(os.path.join(d, name), arr)
        with open(os.path.join(d, name), "rb") as f:            # the payload starts after the header
            f.seek(8)
            hlen = int.from_bytes(f.read(2), "little")
        b = Buffer(nid(), name[:-4], arr.shape, dt, "temp")
        bufs.append((b, arr))
        calls.append(RTCall("load_npy", {"buf": b, "path": os.path.join(d, "not_here", name), "offset": 10 + hlen,
                                         "kind": kind, "size": size}))
    prog = kir.Program(kir.Block(calls), [b for b, _ in bufs], "npy")
    dp = DeviceProgram(prog, seed=0)
    try:
        code, _ = dp.run(capture=True)
        assert code == 0, dp.error
        for b, arr in bufs:
            want = arr.reshape(-1).astype(np.int32 if b.dtype == I32 else np.float32)
            assert np.array_equal(dp.read(b).reshape(-1), want), b.name
    finally:
        dp.close()
