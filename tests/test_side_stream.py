"""Kernels whose results the rest of a training step does not need run on a second stream (analysis.deferred_kernels,
the emitter's fork / join calls, the arena planner's longer lifetimes). CPU checks of the analysis and of the emitted
host code; the GPU parity tests run the programs both ways."""
import os
import re

from anvil_lang_b200 import kir
from anvil_lang_b200.backend import analysis as an
from anvil_lang_b200.backend import emit
from util import ROOT


def load(name):
    return kir.load(os.path.join(ROOT, "anvil_lang_b200", "programs", f"{name}.kir.json.gz"))


def test_deferred_kernels_write_what_nothing_later_touches():
    prog = load("c3_mlp_adam")
    ids = an.deferred_kernels(prog)
    assert ids
    hot = an.hot_loop(prog)
    stmts = hot.body.stmts
    for i, st in enumerate(stmts):
        if isinstance(st, kir.KernelStmt) and st.kernel.id in ids:
            k = st.kernel
            assert not k.uses_rand()
            w = {b.id for b in k.writes()}
            r = {b.id for b in k.reads()}
            assert all(b.kind in ("param", "state", "grad", "temp") for b in k.writes())
            for later in stmts[i + 1:]:
                lr, lw = an._stmt_roots(later)
                assert not (w & (lr | lw)) and not (r & lw)
    # the forward pass and the loss are needed by what follows: never deferred
    first = next(st.kernel for st in stmts if isinstance(st, kir.KernelStmt))
    assert first.id not in ids


def test_every_fork_is_joined_inside_its_graph(monkeypatch):
    prog = load("c5_transformer")
    src, g = emit.generate(prog, seed=0)
    assert len(g.side_ids) >= 30 and all(i in g.deferred for i in g.side_ids)
    # deferred contractions (weight gradients with their updates) are dealt to the two streams by accumulated work
    side_gemms = [i for i in g.side_ids if g.kernel_notes[g.kernel_index[i]].startswith("gemm")]
    assert side_gemms and 0.8 < g.dealt[1] / g.dealt[0] < 1.25
    for i in side_gemms:                                 # split-k partial sums of a second-stream product: second scratch region
        body = g.kernel_src[g.kernel_index[i]]
        if "_part" in body:
            assert f"A + {g.plan.side_scratch_off}UL" in body and f"A + {g.plan.scratch_off}UL" not in body
    blocks = re.findall(r"anvil_rt_graph_begin\(rt, \d+\).*?anvil_rt_graph_end\(rt, \d+\)", src, flags=re.S)
    forked = [b for b in blocks if "anvil_rt_fork" in b]
    assert forked
    for b in forked:
        assert b.rfind("anvil_rt_join(rt)") > b.rfind("anvil_rt_fork(rt)")
    # split reductions on the second stream keep their partial sums and tickets apart from the first stream's
    side_split = [i for i in g.side_ids if g.kernel_notes[g.kernel_index[i]].startswith("split col4")]
    assert side_split and g.plan.side_scratch_bytes >= 4 * 512 * 128
    body = g.kernel_src[g.kernel_index[side_split[0]]]
    first_off = g.member_slot.get(side_split[0], (0, 0))[0]
    assert "ANVIL_RT_SIDE_TICKETS_OFF" in body and f"A + {g.plan.side_scratch_off + first_off}UL" in body
    # ... and from one another when several of them share a launch: disjoint scratch ranges and ticket ranges
    groups = {}
    for i in side_split:
        if i in g.zgroup_of:
            groups.setdefault(g.zgroup_of[i], []).append(i)
    assert groups
    for ids, members in groups.items():
        spans = []
        ticks = []
        for i in members:
            kg = g.kernel_gens[i]
            soff, tick = g.member_slot[i]
            gx, S = kg.grid
            spans.append((soff, soff + 4 * kg.k.out_numel() * S))
            ticks.append((tick, tick + gx))
        for rng in (sorted(spans), sorted(ticks)):
            assert all(a[1] <= b[0] for a, b in zip(rng, rng[1:]))
        assert max(t[1] for t in ticks) <= 256 and max(sp[1] for sp in spans) <= g.plan.side_scratch_bytes
        assert len(ids) <= g.ZGROUP_MAX
    # a side-by-side launch appears once, at its last member, between a fork and the join
    z = {int(x) for x in re.findall(r"launch_group_(\d+)\(rt\)\); anvil_rt_back", src)}
    assert {i for i, n in enumerate(g.group_notes) if n.startswith("zgroup")} <= z      # (fused products may fork too)
    monkeypatch.setenv("ANVIL_B200_SIDE", "0")
    src0, g0 = emit.generate(load("c5_transformer"), seed=0)
    assert "anvil_rt_fork" not in src0 and not g0.side_ids


def test_what_a_deferred_kernel_reads_lives_until_the_join():
    prog = load("c5_transformer")
    src, g = emit.generate(prog, seed=0)
    uses, loops = an._flatten(g.prog, None, g.deferred)
    uses0, _ = an._flatten(g.prog, None, ())
    longer = 0
    for k in g.prog.kernels():
        if k.id in g.side_ids:
            for r in k.reads():
                assert uses[r.id][-1].pos >= uses0[r.id][-1].pos
                longer += uses[r.id][-1].pos > uses0[r.id][-1].pos
    assert longer > 0


def test_first_stream_groups_write_no_tensor_that_shares_bytes():
    """Kernels of one launch run concurrently, but lifetime sharing of arena bytes relies on the program's order: a
    first-stream member may therefore not write a tensor whose bytes another tensor had before."""
    from anvil_lang_b200 import dp
    from util import GOLDEN
    progs = [kir.load(os.path.join(GOLDEN, "transformer_small.kir.json.gz")), dp.shard(load("c5_transformer.b8"), 8)]
    seen = 0
    for prog in progs:
        src, g = emit.generate(prog, seed=0)
        assert g.plan.shared
        for kid, ids in g.zgroup_of.items():
            if ids[0] in g.side_ids:
                continue
            seen += 1
            k = g.kernels[g.kernel_index[kid]]
            assert not ({b.id for b in k.writes()} & g.plan.shared)
            for other in ids:                                   # and the members do not touch one another's results
                if other != kid:
                    o = g.kernels[g.kernel_index[other]]
                    assert not ({b.id for b in k.writes()} & ({b.id for b in o.reads()} | {b.id for b in o.writes()}))
    assert seen > 0
