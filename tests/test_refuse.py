"""Producer / consumer re-fusion (backend/refuse.py) on the CPU: the rewritten program must compute bit-identical
tensors, the gradient of every Adam-updated matrix must no longer be stored, and the pass must be idempotent."""
import io
import os

import numpy as np
import pytest

from anvil_lang_b200 import dp, kir
from anvil_lang_b200.backend import refuse
from anvil_lang_b200.backend.analysis import hot_loop
from oracle.kir_interp import Oracle
from util import GOLDEN, ROOT


def run(prog, steps=None):
    o = Oracle(prog, out=io.StringIO(), seed=0, mode="fast")
    o.run()
    return o


@pytest.mark.parametrize("name", ["transformer_small", "train_mlp", "dp_mlp"])
def test_fused_program_is_bit_identical(name):
    path = os.path.join(GOLDEN, f"{name}.kir.json.gz")
    plain, fused = kir.load(path), kir.load(path)
    n = refuse.fuse_consumers(fused)
    if name == "transformer_small":
        assert n > 0
    a, b = run(plain), run(fused)
    assert a.out.getvalue() == b.out.getvalue()
    for r in plain.roots():
        if r.kind in ("param", "state"):
            assert np.array_equal(a.arr(r)[:r.numel], b.arr(r)[:r.numel], equal_nan=True), r.name


def test_adam_gradients_of_matrices_are_no_longer_stored():
    prog = kir.load(os.path.join(ROOT, "anvil_lang_b200", "programs", "c3_mlp_adam.kir.json.gz"))
    before = {b.root.name for k in prog.kernels() for b in k.writes()}
    assert "dnet.l1.W" in before and "dnet.l2.W" in before
    assert refuse.fuse_consumers(prog) == 2
    assert refuse.fuse_consumers(prog) == 0                          # idempotent
    after_w = {b.root.name for k in prog.kernels() for b in k.writes()}
    after_r = {b.root.name for k in prog.kernels() for b in k.reads()}
    assert "dnet.l1.W" not in after_w | after_r and "dnet.l2.W" not in after_w | after_r
    hot = hot_loop(prog)
    fused = [s.kernel for s in hot.body.stmts if isinstance(s, kir.KernelStmt) and "+" in s.kernel.name]
    assert len(fused) == 2
    for k in fused:                                                  # one kernel: product, both moments, the parameter
        assert k.red is not None and {s.buf.root.kind for s in k.stores} == {"state", "param"} and len(k.stores) == 3


def test_sharded_updates_fuse_too():
    prog = dp.shard(kir.load(os.path.join(ROOT, "anvil_lang_b200", "programs", "c3_mlp_adam.b128.kir.json.gz")), 2)
    assert refuse.fuse_consumers(prog) == 2
    hot = hot_loop(prog)
    kinds = [type(s).__name__ for s in hot.body.stmts]
    assert kinds.count("AllReduce") == 1
