"""The IR data model: JSON round trip and the static analyses the emitter relies on."""
import pytest

from anvil_lang_b200 import kir
from anvil_lang_b200.backend import analysis as an
from util import golden_names, load_golden


@pytest.mark.parametrize("name", golden_names())
def test_json_round_trip(name):
    prog, _, _, _ = load_golden(name)
    text = kir.dumps(prog)
    again = kir.loads(text)
    assert kir.dumps(again) == text
    assert len(again.kernels()) == len(prog.kernels())


def test_injective_over():
    i, j = kir.Var(1, "i", 4), kir.Var(2, "j", 8)
    assert an.injective_over(kir.Affine(0, [(i, 8), (j, 1)]), [i, j])
    assert not an.injective_over(kir.Affine(0, [(i, 4), (j, 1)]), [i, j])      # rows overlap
    assert not an.injective_over(kir.Affine(0, [(i, 8)]), [i, j])              # j missing
    assert an.injective_over(kir.Affine(3, [(i, -8), (j, 1)]), [i, j])


def test_parallel_safe_flags_order_dependent_kernels():
    prog, _, _, _ = load_golden("gathers_views")
    flags = [an.parallel_safe(k) for k in prog.kernels()]
    assert all(flags)                                   # gathers and scatter-adds are parallel
    prog, _, _, _ = load_golden("train_mlp")
    assert an.hot_loop(prog) is not None


def test_hot_loop_is_the_batch_loop():
    prog = kir.load(__import__("os").path.join(__import__("util").ROOT, "anvil_lang_b200", "programs", "c3_mlp_adam.kir.json.gz"))
    hot = an.hot_loop(prog)
    assert hot.counter.name == "x_batch" and hot.stop == 234
