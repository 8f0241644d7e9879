"""The arena plan (backend/analysis.plan_arena): temporaries with disjoint lifetimes share bytes.

Checked on the CPU, after the reference's own arena tests (tests/test_arena.py there: sharing keeps the output;
overlapping lifetimes never share bytes): (1) structurally — two tensors whose lifetimes overlap never overlap in
memory, nothing overlaps a tensor with memory of its own; (2) by execution — the oracle runs each fixture program
with ALL its tensors laid out in one flat array at the planned offsets, so a wrong lifetime shows as a wrong result
against the ordinary run; (3) the full-size transformer fits in 8 GB (31 GB with every tensor on its own)."""
import io
import os

import numpy as np
import pytest

from anvil_lang_b200 import kir
from anvil_lang_b200.backend import analysis as an
from anvil_lang_b200.backend import emit
from oracle.kir_interp import Oracle
from util import GOLDEN, ROOT, golden_names

PROGRAMS = ["train_mlp", "train_cnn", "transformer_small", "conv_pool", "control_flow", "softmax_ce", "reductions"]


def plan_of(prog):
    gen = emit.generate(prog, 0)[1]
    return gen.plan


@pytest.mark.parametrize("name", [n for n in PROGRAMS if n in golden_names()])
def test_shared_tensors_never_collide(name):
    prog = kir.load(os.path.join(GOLDEN, f"{name}.kir.json.gz"))
    plan = plan_of(prog)
    roots = {r.id: r for r in prog.roots()}
    spans = []
    for rid, r in roots.items():
        lo = plan.offsets[rid]
        spans.append((lo, lo + max(r.nbytes, 16), rid))
    own = [s for s in spans if s[2] not in plan.clobbered]
    shared = [s for s in spans if s[2] in plan.shared]
    for a in shared:                                            # a shared tensor never touches one with its own memory
        for b in own:
            assert a[1] <= b[0] or b[1] <= a[0], (roots[a[2]].name, roots[b[2]].name)
    for i, a in enumerate(shared):                              # two live at once never touch each other
        for b in shared[i + 1:]:
            la, lb = plan.spans[a[2]], plan.spans[b[2]]
            if la[0] <= lb[1] and lb[0] <= la[1]:
                assert a[1] <= b[0] or b[1] <= a[0], (roots[a[2]].name, la, roots[b[2]].name, lb)
    for i, a in enumerate(own):
        for b in own[i + 1:]:
            assert a[1] <= b[0] or b[1] <= a[0]


@pytest.mark.parametrize("name", [n for n in PROGRAMS if n in golden_names()])
def test_program_runs_the_same_inside_the_planned_arena(name):
    path = os.path.join(GOLDEN, f"{name}.kir.json.gz")
    plain_prog = kir.load(path)
    plan_of(plain_prog)                                         # the same IR rewrites (fixed-order scatters, fused updates)
    ref = Oracle(plain_prog, out=io.StringIO(), seed=0, mode="fast")
    ref.run()
    prog = kir.load(path)
    plan = plan_of(prog)                                        # (this also applies the emitter's IR rewrites to `prog`)
    o = Oracle(prog, out=io.StringIO(), seed=0, mode="fast")
    flat = np.zeros(plan.size // 4 + 16, np.float32)
    for r in prog.roots():                                      # every tensor becomes a view of the one flat array
        old = o.mem[r.id]
        at = plan.offsets[r.id] // 4
        view = flat[at:at + old.size].view(old.dtype)
        if r.id not in plan.clobbered:
            view[:] = old
        o.mem[r.id] = view
    o.run()
    assert o.out.getvalue() == ref.out.getvalue()
    by_id = {r.id: r for r in plain_prog.roots()}
    for r in prog.roots():
        if r.id in plan.clobbered or r.id not in by_id:
            continue
        assert np.array_equal(o.mem[r.id][:r.numel], ref.mem[r.id][:r.numel], equal_nan=True), r.name


def test_full_size_transformer_fits_in_eight_gigabytes():
    prog = kir.load(os.path.join(ROOT, "anvil_lang_b200", "programs", "c5_transformer.kir.json.gz"))
    plan = plan_of(prog)
    assert plan.size < 8 << 30
    assert plan.unshared_bytes > 1.9 * plan.shared_bytes       # the shared tensors fit in half of what they add up to
    names = {r.id: r.name for r in prog.roots()}
    grads_of_matrices = [rid for rid in plan.unused if names[rid].startswith("dnet.") and names[rid].endswith((".Wq", ".Wk", ".Wv", ".Wo", ".W"))]
    assert len(grads_of_matrices) >= 36                         # the weight gradients live in registers of the fused updates
    os.environ["ANVIL_B200_ARENA"] = "unshared"
    try:
        big = plan_of(kir.load(os.path.join(ROOT, "anvil_lang_b200", "programs", "c5_transformer.kir.json.gz")))
    finally:
        os.environ.pop("ANVIL_B200_ARENA", None)
    assert big.size > 3 * plan.size and not big.shared


def test_a_store_covers_its_tensor_only_as_a_bijection():
    from kirbuild import buf, nid, var
    from anvil_lang_b200.kir import F32, Affine, E, Kernel, Store
    t = buf("t", (4, 6))
    i, j, v = var("i", 4), var("j", 6), var("v", 24)
    one = E("const", F32, val=1.0)
    full = Kernel(nid(), "k", "", [i, j], [Store(t, Affine(0, [(i, 6), (j, 1)]), one)], None)
    collapsed = Kernel(nid(), "k", "", [v], [Store(t, Affine(0, [(v, 1)]), one)], None)
    transposed = Kernel(nid(), "k", "", [j, i], [Store(t, Affine(0, [(i, 6), (j, 1)]), one)], None)
    partial = Kernel(nid(), "k", "", [i], [Store(t, Affine(0, [(i, 6)]), one)], None)
    strided = Kernel(nid(), "k", "", [i, j], [Store(t, Affine(0, [(i, 6), (j, 0)]), one)], None)
    plus = Kernel(nid(), "k", "", [i, j], [Store(t, Affine(0, [(i, 6), (j, 1)]), one, True)], None)
    assert an.covers(full, full.stores[0]) and an.covers(collapsed, collapsed.stores[0]) and an.covers(transposed, transposed.stores[0])
    assert not an.covers(partial, partial.stores[0]) and not an.covers(strided, strided.stores[0]) and not an.covers(plus, plus.stores[0])
