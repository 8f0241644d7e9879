"""Convolutions as implicit products (backend/implicit.py) on the CPU: the rewritten program prints the same
numbers and ends with the same parameters (to rounding: the window sum is re-associated), and the window tensor and
its gradient are gone from the arena of the CNN configuration."""
import io
import os

import numpy as np
import pytest

from anvil_lang_b200 import kir
from anvil_lang_b200.backend import emit, implicit, refuse
from oracle.kir_interp import Oracle
from util import GOLDEN, ROOT, outputs_match


@pytest.mark.parametrize("name,expect", [("train_cnn", 3), ("conv_pool", 1)])
def test_rewritten_program_computes_the_same(name, expect):
    path = os.path.join(GOLDEN, f"{name}.kir.json.gz")
    plain, folded = kir.load(path), kir.load(path)
    assert implicit.make_implicit(folded, refuse._host_reads(folded)) == expect
    assert implicit.make_implicit(folded, refuse._host_reads(folded)) == 0           # idempotent
    a = Oracle(plain, out=io.StringIO(), seed=0)
    a.run()
    b = Oracle(folded, out=io.StringIO(), seed=0)
    b.run()
    ok, why = outputs_match(b.out.getvalue(), a.out.getvalue(), rtol=1e-5, atol=1e-6)
    assert ok, why
    for r in plain.roots():
        if r.kind in ("param", "state", "var"):
            x, y = a.arr(r)[:r.numel], b.arr(r)[:r.numel]
            assert np.abs(x - y).max() <= 1e-5 * max(np.abs(x).max(), 1e-30), r.name


def test_cnn_configuration_holds_no_window_tensor():
    prog = kir.load(os.path.join(ROOT, "anvil_lang_b200", "programs", "c4_cnn_sgd.kir.json.gz"))
    before = {b.name for k in prog.kernels() for b in k.writes()}
    assert {"patches", "dpatches"} <= before
    src, gen = emit.generate(prog, 0)
    touched = {b.name for k in prog.kernels() for b in list(k.writes()) + list(k.reads())}
    assert "patches" not in touched and "dpatches" not in touched
    held = {b.name for b in prog.roots() if b.id not in gen.plan.unused}
    assert "patches" not in held and "dpatches" not in held
    notes = [n for n in gen.kernel_notes if n.startswith("gemm")]
    assert "gemm tc 1x15488x64x288 S1 pp" in notes                 # the second convolution is a tensor-core product gathering on load
    assert any(n.startswith("gemm tc 1x288x64x15488") for n in notes)    # and so is its weight gradient


def test_guarded_gather_form_of_the_scattered_gradient():
    prog = kir.load(os.path.join(ROOT, "anvil_lang_b200", "programs", "c4_cnn_sgd.kir.json.gz"))
    implicit.make_implicit(prog, refuse._host_reads(prog))
    folded = [k for k in prog.kernels() if k.label.endswith("+gathered")]
    assert len(folded) == 1
    k = folded[0]
    assert [v.extent for v in k.domain] == [128, 32, 13, 13] and sorted(v.extent for v in k.red.vars) == [3, 3, 64]
    text = kir.fmt_kernel(k)
    assert "if" in text and ">= 0" in text and "< 11" in text     # 0 <= y - u < 11 guards the shifted load
