"""Parity of every LAUNCH UNIT of a training step: where the emitter runs several IR kernels as one launch (a fused
row group, contractions fused side by side, a fused attention run) that launch is compared with the oracle running
the same IR kernels one after the other, on inputs copied from the oracle. Tensors that a fused launch keeps on chip
are not compared (they are never written); everything it does write must match to 1e-4 of the tensor's magnitude
(i32 exactly). The program is the transformer at T = 256 with two heads of 64 (the attention template's tile), batch 2,
two layers; its IR and its first losses come from the reference front end and interpreter
(`make_golden.py traj c5_transformer 4 '{"BATCH": 2, "LAYERS": 2, "D": 128, "HEADS": 2, "T": 256, "STEPS": 4}' _t256`).
A second program has a band mask (`0.0 if j <= i + 64 else -1e9`, tests/programs/transformer_bandmask.anvil) instead of
the causal one: the attention template then runs every query tile over all keys and takes the mask from the IR's own
expression (`make_golden.py traj transformer_bandmask 3 '{... "STEPS": 3}' _t256`)."""
import io
import json
import os

import numpy as np
import pytest

from anvil_lang_b200 import kir
from anvil_lang_b200.backend.analysis import hot_loop
from anvil_lang_b200.program import DeviceProgram
from oracle.kir_interp import Oracle
from test_gpu_kernel_parity import run_to_loop
from util import GOLDEN, tensor_close

pytestmark = pytest.mark.gpu

PROGRAMS = ["c5_transformer_t256", "transformer_bandmask_t256"]


def build(name, min_mflop="0"):
    os.environ["ANVIL_B200_TC_MIN_MFLOP"] = min_mflop          # the small products take the tensor-core templates too
    try:
        prog = kir.load(os.path.join(GOLDEN, f"{name}.traj.kir.json.gz"))
        return prog, DeviceProgram(prog, seed=0, graphs=False)
    finally:
        os.environ.pop("ANVIL_B200_TC_MIN_MFLOP", None)


@pytest.mark.parametrize("name", PROGRAMS)
def test_fused_launch_units_match_their_kernels_run_one_by_one(name):
    prog, dp = build(name)
    hot = hot_loop(prog)
    o = Oracle(prog, out=io.StringIO(), seed=0, mode="fast")
    run_to_loop(o, prog, hot)
    nk = len(dp.gen.kernels)
    notes = [note for _, note, _ in dp.gen.hot_units]
    assert any(n.startswith("attention fwd") for n in notes) and any(n.startswith("attention bwd") for n in notes)
    assert any(n.startswith("attention") and n.endswith("causal") for n in notes) == (name == "c5_transformer_t256")
    assert any("ncat" in n for n in notes) and any("kcat" in n for n in notes) and any(n.startswith("rowgroup") for n in notes)
    bad = []
    try:
        for (kind, idx), note, ks in dp.gen.hot_units:
            touched = {}
            for k in ks:
                for b in list(k.reads()) + list(k.writes()):
                    touched[b.id] = b
            for b in touched.values():
                if b.id not in dp.gen.dead_roots:
                    dp.write(b, o.arr(b)[:max(b.numel, 1)])
            dp.rtlib.anvil_rt_set_stream(dp.rt, o.stream)
            for k in ks:
                o.kernel(k)
            dp.launch(idx if kind == "k" else nk + idx)
            written = {b.id: b for k in ks for b in k.writes()}
            for b in written.values():
                if b.id in dp.gen.dead_roots:
                    continue
                tol = 5e-3 if b.kind == "param" else 1e-4         # Adam's g / (|g| + eps), see test_gpu_kernel_parity
                ok, why = tensor_close(dp.read(b).reshape(-1), o.arr(b)[:b.numel], tol)
                if not ok:
                    bad.append(f"[{note}] {'+'.join(k.name for k in ks)[:60]} {b.name}{list(b.shape)}: {why}")
        dp.check_faults()
    finally:
        dp.close()
    assert not bad, "\n".join(bad[:20])


@pytest.mark.parametrize("name", PROGRAMS)
def test_first_losses_match_the_reference_interpreter(name):
    want = json.load(open(os.path.join(GOLDEN, f"{name}.losses.json")))["losses"]
    prog, dp = build(name)
    try:
        dp.rtlib.anvil_rt_capture(dp.rt, 1)
        dp.prologue()
        loss = dp.buffer("loss")
        got = []
        for _ in want:
            dp.step()
            got.append(float(dp.read(loss).reshape(-1)[0]))
        dp.check_faults()
    finally:
        dp.close()
    rel = np.abs(np.array(got) - np.array(want)) / np.abs(want)
    assert rel.max() <= 1e-4, (got, want)
