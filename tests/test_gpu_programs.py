"""Parity of the CUDA path with the reference interpreter's goldens, program by program.

Every fixture program runs on the device through the generated code and the C ABI; the printed
text must match the interpreter's (numbers to the reference's own 2e-3 print tolerance) and every
final tensor must match (i32 exactly, f32 to 1e-4 of the tensor's magnitude).

Two builds of each program: the default one (launch runs replayed as CUDA graphs, temporaries with disjoint lifetimes
sharing arena bytes — only tensors that still hold a value at the end are compared), and a plain one (no graphs,
every tensor in memory of its own — every tensor the interpreter holds at the end is compared)."""
import os

import pytest

from anvil_lang_b200 import kir
from anvil_lang_b200.program import DeviceProgram
from util import GOLDEN, check_arrays, device_program, golden_names, load_golden, outputs_match

pytestmark = pytest.mark.gpu

# tensors whose final value depends on float summation order amplified by training are compared
# through the printed losses instead
TRAINED = ("train_mlp", "train_cnn", "transformer_small")


@pytest.mark.parametrize("graphs", [True, False], ids=["graphs", "plain"])
@pytest.mark.parametrize("name", golden_names())
def test_program_matches_reference(name, graphs):
    prog, text, meta, arrays = load_golden(name)
    dp = device_program(prog, unshared_arena=not graphs, seed=0, graphs=graphs)
    try:
        assert graphs or not dp.plan.shared
        code, got = dp.run(capture=True)
        assert code == meta["exit"], dp.error
        if meta["exit"] == 1:
            assert "out of bounds" in dp.error and dp.error.startswith("anvil: runtime error:")
            assert got == text                    # everything printed before the fault, nothing after
            return
        ok, why = outputs_match(got, text)
        assert ok, why
        rel = 2e-3 if name in TRAINED else 1e-4
        bad = check_arrays(lambda b: dp.read(b).reshape(-1), prog, arrays, rel=rel, skip=dp.gen.dead_roots | dp.plan.clobbered)
        assert not bad, bad
    finally:
        dp.close()


def test_profile_table_has_the_reference_layout():
    """`--profile`: after the program's own output comes the native back end's table (runtime.s:1669-1671):
    a header, one row per launch unit that ran (share, milliseconds, calls, name), and the total."""
    import re
    from anvil_lang_b200 import cuda
    prog = kir.load(os.path.join(GOLDEN, "train_mlp.kir.json.gz"))
    plain_code, plain = cuda.run(prog, seed=0, capture=True)
    code, text = cuda.run(prog, seed=0, capture=True, profile=True)
    assert code == plain_code == 0
    assert text.startswith(plain)                                 # profiling does not change what the program prints
    table = text[len(plain):]
    lines = table.split("\n")
    assert lines[0] == "" and lines[1] == "  time%        ms      calls   kernel"
    rows = [ln for ln in lines[2:] if re.fullmatch(r" *\d+\.\d%  +\d+\.\d  +\d+   \S.*", ln)]
    assert len(rows) >= 10 and re.fullmatch(r" +\d+\.\d ms in kernels", lines[2 + len(rows)])
    shares = [float(r.split("%")[0]) for r in rows]
    assert abs(sum(shares) - 100.0) < 1.0
    calls = {r.split()[3]: int(r.split()[2]) for r in rows}
    assert max(calls.values()) >= 10                              # the training loop's kernels ran once per step


def test_check_stops_at_the_first_nan_and_says_where():
    """`--check`: log of a negative number makes a nan; the run stops after the kernel that wrote it with the
    reference's message head (anvil/interp.py:408-423) — `--check: nan in `name` at [indices]` — and the kernel."""
    from anvil_lang_b200 import cuda
    from anvil_lang_b200.kir import F32, Affine, Buffer, E, Kernel, KernelStmt, Store, Var
    from kirbuild import nid
    x = Buffer(nid(), "x", (3, 5), F32, "temp")
    y = Buffer(nid(), "y", (3, 5), F32, "temp")
    i, j = Var(nid(), "i", 3), Var(nid(), "j", 5)
    at = Affine(0, [(i, 5), (j, 1)])
    idx = E("un", F32, op="f32", a=[E("index", kir.I32, off=Affine(-7, [(i, 5), (j, 1)]))])      # negative for the first 7 elements
    k1 = Kernel(nid(), "k1", "fill", [i, j], [Store(x, at, E("bin", F32, op="sub", a=[E("const", F32, val=0.5), idx]), False)], None)
    k2 = Kernel(nid(), "k2", "log", [i, j], [Store(y, at, E("un", F32, op="log", a=[E("load", F32, buf=x, off=at)]), False)], None)
    prog = kir.Program(kir.Block([KernelStmt(k1), KernelStmt(k2)]), [x, y], "check")
    dp = DeviceProgram(prog, seed=0)
    try:
        assert dp.run(capture=True)[0] == 0                          # without --check the nans go unnoticed
        dp.rtlib.anvil_rt_check(dp.rt, 1)
        code, _ = dp.run(capture=True)
        assert code == 1
        head = dp.error.split("\n")
        assert head[0] == "anvil: runtime error: --check: nan in `y` at [1, 3]", dp.error    # x = 0.5 - (5i + j - 7) < 0 from element 8 on
        assert head[1] == "  made by `log`:" and head[2].startswith("  computing (k2):")
    finally:
        dp.close()
