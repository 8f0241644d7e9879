"""Parity of the CUDA path with the reference interpreter's goldens, program by program.

Every fixture program runs on the device through the generated code and the C ABI; the printed
text must match the interpreter's (numbers to the reference's own 2e-3 print tolerance) and every
final tensor must match (i32 exactly, f32 to 1e-4 of the tensor's magnitude)."""
import pytest

from anvil_lang_b200.program import DeviceProgram
from util import check_arrays, golden_names, load_golden, outputs_match

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
