"""Host-side checks of the code generator's contraction path (no GPU): which tcgen05 template a shape
takes, the split heuristics, and the two-phase epilogue (what `epi_loads` may fetch ahead of the stores)."""
import os
import re

import pytest

from anvil_lang_b200.backend import emit
from kirbuild import contraction_program


def gen(case, tc=None):
    old = os.environ.get("ANVIL_B200_TC")
    if tc is not None:
        os.environ["ANVIL_B200_TC"] = tc
    try:
        prog = contraction_program(*case)[0]
        src, g = emit.generate(prog, 0)[:2]
    finally:
        if old is None:
            os.environ.pop("ANVIL_B200_TC", None)
        else:
            os.environ["ANVIL_B200_TC"] = old
    return src, g.kernel_notes[0]


def test_template_choice_by_shape():
    tv = emit.tc_variant
    assert tv(True, 16384, 512, 2048) == "pp"          # 256-row shapes: resident CTA pairs
    assert tv(False, 512, 2048, 16384) == "pp"
    assert tv(True, 256, 64, 256) == "pp"              # narrow output: 64-column tiles
    assert tv(True, 128, 128, 64) == "ss"              # too few rows for a pair, short reduction
    assert tv(True, 200, 136, 512) == "ss32"
    assert tv(False, 200, 136, 512) == "ts"            # A read along m


def test_forced_variant_falls_back_when_the_shape_is_too_small():
    small = (128, 128, 64, 1, False, False, False, False, 1.0, False, False)
    src, note = gen(small, "pp")
    assert "gemm_tc_pair_persistent" not in src and note.startswith("gemm tc")


@pytest.mark.parametrize("case,bn,accs,split", [
    ((16384, 512, 2048, 1, False, False, True, False, 1.0, False, False), 256, 2, 1),   # chain 2048: two accumulators
    ((1024, 1024, 512, 1, False, False, False, False, 1.0, False, False), 128, 2, 2),   # 16 wide tiles on 74 slots: 32 narrow ones, split 2
    ((256, 64, 256, 6, False, False, False, False, 0.125, False, False), 64, 2, 2),
    ((384, 192, 512, 1, False, True, False, True, 1.0, False, False), 128, 2, 4),
])
def test_resident_pair_parameters(case, bn, accs, split):
    src, note = gen(case, "pp")                      # by name: two of the shapes are below the tensor-core FLOP threshold
    m = re.search(r"gemm_tc_pair_persistent<G\d+, (true|false), (true|false), (\d+), (\d+), (\d+)>", src)
    assert m, note
    assert (int(m.group(5)), int(m.group(4)), int(m.group(3))) == (bn, accs, split), (m.group(0), note)
    assert "__cluster_dims__(2, 1, 1)" in src
    grid = re.search(r"<<<dim3\((\d+), 1\), anvil::tc::PP_THREADS", src)
    assert grid and int(grid.group(1)) % 2 == 0 and int(grid.group(1)) <= 148


def test_accumulation_chain_is_capped():
    long_k = (512, 512, 65536, 1, True, False, False, False, 1.0, True, False)
    src, note = gen(long_k)
    split = int(re.search(r"S(\d+)", note).group(1))
    assert 65536 // split <= 4096, note


def nld(src):
    return [int(x) for x in re.findall(r"static constexpr int NLD = (\d+);", src)]


def test_two_phase_epilogue_preloads_the_accumulate_target():
    acc = (512, 512, 512, 1, False, False, False, False, 1.0, True, False)             # C += A B
    src, _ = gen(acc)
    assert nld(src) == [1]
    loads = src[src.index("void epi_loads"):src.index("void epi2")]
    assert re.search(r"ld\[0\] = b\d+\[", loads)
    body = src[src.index("void epi2"):]
    assert "+=" not in body[:body.index("};")] and "ld[0]" in body


def test_two_phase_epilogue_leaves_row_vectors_alone():
    bias = (512, 512, 512, 1, False, False, True, False, 1.0, False, True)              # bias[n] is not per element
    src, _ = gen(bias)
    assert nld(src) == [0]
    assert "prefetch_l2" not in src[src.index("void epi_touch"):src.index("static constexpr int NLD")]


def test_operand_prefetch_functors_exist_for_resident_pairs():
    src, _ = gen((512, 512, 512, 1, False, False, False, False, 1.0, False, False))
    assert "void a_touch(int m, int k, int bt)" in src and "void b_touch(int k, int n, int bt)" in src
    assert src.count("anvil::prefetch_l2(") >= 2


def test_continue_in_a_for_loop_still_advances_the_counter():
    """A `continue` inside a counted loop must reach the counter's advance (reference anvil/backend/cuda.py:445 puts
    it in the for statement's third clause); otherwise the host would launch the body for ever."""
    import os as _os
    from anvil_lang_b200 import kir
    from util import GOLDEN
    prog = kir.load(_os.path.join(GOLDEN, "control_flow.kir.json.gz"))
    src = emit.generate(prog, 0)[0]
    loops = [m for m in re.finditer(r"for \(long (i\d+) = lo\d+; i\d+ < hi\d+; ([^)]*\)?)\) \{", src)]
    with_continue = []
    for m in loops:
        depth, j = 1, m.end()
        while depth:
            depth += {"{": 1, "}": -1}.get(src[j], 0)
            j += 1
        body = src[m.end():j]
        if re.search(r"\bcontinue;", body):
            with_continue.append((m, body))
    assert with_continue, "the fixture has a `for` with `continue`"
    for m, body in with_continue:
        assert "anvil_b200_advance(rt," in m.group(0), m.group(0)       # the advance is the loop's third clause
        assert "anvil_rt_add_i32" not in body.split("continue;")[-1]      # not at the bottom of the body


def test_transformer_products_are_fused_side_by_side():
    """Per transformer block: the three products with the same left operand (h @ Wq, h @ Wk, h @ Wv) become one launch
    with the outputs side by side, so do their three weight gradients, and the three products that add up to the
    gradient of h become one launch over the concatenated reduction index (backend/hfuse.py)."""
    import os as _os
    from collections import Counter
    from anvil_lang_b200 import kir
    from util import ROOT
    prog = kir.load(_os.path.join(ROOT, "anvil_lang_b200", "programs", "c5_transformer.kir.json.gz"))
    src, g = emit.generate(prog, 0)
    notes = Counter(n for n in g.group_notes if n.startswith("gemm"))
    assert notes == {"gemm tc 1x16384x1536x512 S1 pp ncat3": 6, "gemm tc 1x16384x512x1536 S1 pp kcat3": 6,
                     "gemm tc 1x512x1536x16384 S6 pp ncat3": 6}
    units = [note for _, note, _ in g.hot_units]
    assert sum(1 for n in units if n.startswith("gemm tc 1x16384x512x512")) == 12       # Wo forward and its dX remain single
    assert "if (n < 512)" in src and "else if (n < 1024)" in src and "if (k < 512)" in src
    os.environ["ANVIL_B200_HGROUPS"] = "0"
    try:
        prog = kir.load(_os.path.join(ROOT, "anvil_lang_b200", "programs", "c5_transformer.kir.json.gz"))
        _, g0 = emit.generate(prog, 0)
    finally:
        os.environ.pop("ANVIL_B200_HGROUPS")
    assert not [n for n in g0.group_notes if n.startswith("gemm")] and len(g0.hot_units) == len(g.hot_units) + 36
