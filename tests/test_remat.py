"""Recomputing saved elementwise intermediates (backend/remat.py) on the CPU: the rewritten program must compute
bit-identical tensors, the activation's intermediates must no longer be stored, and the pass must be idempotent."""
import io
import os

import numpy as np
import pytest

from anvil_lang_b200 import kir
from anvil_lang_b200.backend import refuse, remat
from oracle.kir_interp import Oracle
from util import GOLDEN, ROOT


def run(prog):
    o = Oracle(prog, out=io.StringIO(), seed=0, mode="fast")
    o.run()
    return o


@pytest.mark.parametrize("name", ["transformer_small", "train_mlp"])
def test_rewritten_program_is_bit_identical(name):
    path = os.path.join(GOLDEN, f"{name}.kir.json.gz")
    plain, lean = kir.load(path), kir.load(path)
    n = remat.rematerialize(lean, refuse._host_reads(lean))
    if name == "transformer_small":
        assert n > 0
    assert remat.rematerialize(lean, refuse._host_reads(lean)) == 0        # idempotent
    a, b = run(plain), run(lean)
    assert a.out.getvalue() == b.out.getvalue()
    for r in plain.roots():
        if r.kind in ("param", "state"):
            assert np.array_equal(a.arr(r)[:r.numel], b.arr(r)[:r.numel], equal_nan=True), r.name


def test_gelu_keeps_only_its_result():
    prog = kir.load(os.path.join(ROOT, "anvil_lang_b200", "programs", "c5_transformer.kir.json.gz"))
    fwd = [k for k in prog.kernels() if k.label == "mul+tanh"]
    bwd = [k for k in prog.kernels() if k.label == "∂mul+∂add"]
    assert len(fwd) == 6 and all(len(k.stores) == 3 for k in fwd) and all(len(k.reads()) == 4 for k in bwd)
    assert remat.rematerialize(prog, refuse._host_reads(prog)) == 12             # two tensors per layer
    assert all(len(k.stores) == 1 for k in fwd)                                  # the activation itself
    assert all(len(k.reads()) == 2 for k in bwd)                                 # its gradient and its input


def test_tensors_the_host_reads_are_kept():
    prog = kir.load(os.path.join(GOLDEN, "transformer_small.kir.json.gz"))
    host = refuse._host_reads(prog)
    # pretend the host reads everything: nothing may be dropped
    every = {b.root.id for b in prog.buffers}
    assert remat.rematerialize(prog, host | every) == 0
