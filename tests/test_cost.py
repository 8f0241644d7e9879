"""`anvil cost --cuda` (anvil_lang_b200/cost.py): the static half against the kernel-level cost model on the CPU, the
measured half on a GPU."""
import os
import re

import pytest

from anvil_lang_b200 import cost, kir
from anvil_lang_b200.backend import analysis as an
from util import GOLDEN, ROOT


def c3():
    return kir.load(os.path.join(ROOT, "anvil_lang_b200", "programs", "c3_mlp_adam.kir.json.gz"))


def test_static_cost_adds_up_per_source_line():
    prog = c3()
    c = cost.program_cost(prog)
    hot = an.hot_loop(prog)
    step = sum(an.kernel_flops(s.kernel) for s in hot.body.stmts if isinstance(s, kir.KernelStmt))
    steps = (hot.stop - hot.start) // hot.step
    assert c.flops >= step * steps and not c.unbounded
    assert sum(ln.flops for ln in c.lines.values()) == c.flops and sum(ln.bytes for ln in c.lines.values()) == c.bytes
    files = {f for f, _ in c.lines}
    assert "c3_mlp_adam.anvil" in files                          # kernels carry the line they came from
    text = cost.report(prog, "c3_mlp_adam.anvil")
    rows = [ln for ln in text.split("\n") if re.match(r" +\d+\.\d% ", ln)]
    assert rows and "minimize loss" in rows[0]                     # the training statement dominates
    assert "1,863,690 parameters" in text


def test_kernels_keep_their_source_line_through_the_rewrites():
    from anvil_lang_b200.backend import emit
    prog = c3()
    emit.generate(prog, 0)                                        # fused updates, fixed-order scatters
    assert all(k.src is not None for k in prog.kernels())


@pytest.mark.gpu
def test_measured_columns_on_the_device():
    prog = kir.load(os.path.join(GOLDEN, "train_mlp.kir.json.gz"))
    c = cost.program_cost(prog)
    ms = cost.measure(prog, c)
    assert ms > 0
    assert abs(sum(ln.ms for ln in c.lines.values()) - ms) <= 1e-6 * ms      # every launch unit's time lands on some line
    text = cost.report(prog, "train_mlp.anvil", measured_ms=ms, cost=c)
    assert "predicted    measured  of roof" in text
    rows = [ln for ln in text.split("\n") if re.match(r" +\d+\.\d% ", ln)]
    assert rows and all(re.search(r"\d+\.\d{3} ms +\d+\.\d{3} ms", r) for r in rows[:3])
