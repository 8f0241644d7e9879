"""Parity of the CUDA path with the reference interpreter's goldens, program by program.

Every fixture program runs on the device through the generated code and the C ABI; the printed
text must match the interpreter's (numbers to the reference's own 2e-3 print tolerance) and every
final tensor must match (i32 exactly, f32 to 1e-4 of the tensor's magnitude)."""
import os

import pytest

from anvil_lang_b200 import kir
from anvil_lang_b200.program import DeviceProgram
from util import GOLDEN, check_arrays, golden_names, load_golden, outputs_match

pytestmark = pytest.mark.gpu

# tensors whose final value depends on float summation order amplified by training are compared
# through the printed losses instead
TRAINED = ("train_mlp", "train_cnn", "transformer_small")


@pytest.mark.parametrize("graphs", [True, False], ids=["graphs", "plain"])
@pytest.mark.parametrize("name", golden_names())
def test_program_matches_reference(name, graphs):
    prog, text, meta, arrays = load_golden(name)
    dp = DeviceProgram(prog, seed=0, graphs=graphs)
    try:
        code, got = dp.run(capture=True)
        assert code == meta["exit"], dp.error
        if meta["exit"] == 1:
            assert "out of bounds" in dp.error and dp.error.startswith("anvil: runtime error:")
            assert got == text                    # everything printed before the fault, nothing after
            return
        ok, why = outputs_match(got, text)
        assert ok, why
        rel = 2e-3 if name in TRAINED else 1e-4
        bad = check_arrays(lambda b: dp.read(b).reshape(-1), prog, arrays, rel=rel, skip=dp.gen.dead_roots)
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
