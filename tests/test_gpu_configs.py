"""Loss trajectories of the BASELINE configurations on the device.

Two comparisons, because ReLU / max-pool networks are not continuous in their rounding errors: when a
pre-activation lands within an ulp of zero, two correct f32 implementations that sum in a different
order put it on different sides of the kink, one mask element flips, and the trajectories separate
for good. The reference interpreter itself, re-run with its parameters perturbed by one ulp, drifts
from its own recorded trajectory by 5e-4 (C4, step 24) and 5e-3 (C3, step 68) — measured with the CPU
oracle. So:

  * windowed: every 10 steps the device state is re-synchronised from the oracle running alongside;
    inside each window every loss must match the oracle's to 1e-3 (the project's trajectory bar);
  * free-running from the program's own initialisation, against the reference interpreter's recorded
    losses (tests/golden/*.losses.json): the first 10 steps to 1e-3, all steps to 2e-2.
"""
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
from util import GOLDEN, ROOT

pytestmark = pytest.mark.gpu

CONFIGS = {
    "c1_mlp_sgd": (os.path.join(ROOT, "anvil_lang_b200", "programs", "c1_mlp_sgd.kir.json.gz"), 100, 100),
    "c3_mlp_adam": (os.path.join(ROOT, "anvil_lang_b200", "programs", "c3_mlp_adam.kir.json.gz"), 100, 40),
    "c4_cnn_sgd": (os.path.join(ROOT, "anvil_lang_b200", "programs", "c4_cnn_sgd.kir.json.gz"), 100, 30),
    "c5_transformer_small": (os.path.join(GOLDEN, "c5_transformer_small.traj.kir.json.gz"), 100, 50),
}


def free_running(prog, steps):
    dp = DeviceProgram(prog, seed=0)
    dp.rtlib.anvil_rt_capture(dp.rt, 1)
    try:
        dp.prologue()
        loss = dp.buffer("loss")
        out = []
        for _ in range(steps):
            dp.step()
            out.append(float(dp.read(loss).reshape(-1)[0]))
        dp.check_faults()
        return out
    finally:
        dp.close()


@pytest.mark.parametrize("cfg", sorted(CONFIGS))
def test_free_running_trajectory(cfg):
    path, steps, _ = CONFIGS[cfg]
    want = json.load(open(os.path.join(GOLDEN, f"{cfg}.losses.json")))["losses"][:steps]
    got = free_running(kir.load(path), len(want))
    rel = np.abs(np.array(got) - np.array(want)) / np.abs(want)
    assert rel[:10].max() <= 1e-3, rel[:10]
    assert rel.max() <= 2e-2, (int(rel.argmax()), float(rel.max()))


def test_full_size_c5_first_steps():
    """The benchmark's own workload (6 layers, D 512, T 256, batch 64) against the reference interpreter run at
    full size: two steps is what the interpreter finishes in five hours (tests/golden/c5_transformer.losses.json,
    made by `make_golden.py traj c5_transformer 2`)."""
    want = json.load(open(os.path.join(GOLDEN, "c5_transformer.losses.json")))["losses"]
    got = free_running(kir.load(os.path.join(ROOT, "anvil_lang_b200", "programs", "c5_transformer.kir.json.gz")), len(want))
    rel = np.abs(np.array(got) - np.array(want)) / np.abs(want)
    assert rel.max() <= 1e-4, (got, want)


@pytest.mark.parametrize("cfg", sorted(CONFIGS))
def test_windowed_trajectory(cfg):
    path, _, steps = CONFIGS[cfg]
    prog = kir.load(path)
    hot = hot_loop(prog)
    o = Oracle(prog, out=io.StringIO(), seed=0, mode="fast")
    run_to_loop(o, prog, hot)
    golden = json.load(open(os.path.join(GOLDEN, f"{cfg}.losses.json")))["losses"]
    loop_written = set()
    for st in hot.body.stmts:
        if isinstance(st, kir.KernelStmt):
            loop_written |= {b.id for b in st.kernel.writes()}
    dp = DeviceProgram(prog, seed=0)
    dp.rtlib.anvil_rt_capture(dp.rt, 1)
    try:
        dp.prologue()
        loss = dp.buffer("loss")
        worst = 0.0
        for step in range(steps):
            if step % 10 == 0:
                for b in prog.roots():
                    if b.numel and b is not hot.counter.root and (step == 0 or b.id in loop_written):
                        dp.write(b, o.arr(b)[:b.numel])
                dp.rtlib.anvil_rt_set_stream(dp.rt, o.stream)
            o.block(hot.body)
            o.arr(hot.counter)[0] += hot.step
            dp.step()
            want = float(o.arr(loss)[0])
            assert abs(want - golden[step]) <= 1e-3 * abs(golden[step])        # the oracle tracks the reference
            got = float(dp.read(loss).reshape(-1)[0])
            worst = max(worst, abs(got - want) / abs(want))
        dp.check_faults()
    finally:
        dp.close()
    assert worst <= 1e-3, worst


def test_transformer_full_size_first_steps():
    path = os.path.join(GOLDEN, "c5_transformer.losses.json")
    if not os.path.exists(path):
        pytest.skip("the full-size interpreter fixture takes hours to make and is not present")
    want = json.load(open(path))["losses"]
    prog = kir.load(os.path.join(ROOT, "anvil_lang_b200", "programs", "c5_transformer.kir.json.gz"))
    got = free_running(prog, len(want))
    rel = np.abs(np.array(got) - np.array(want)) / np.abs(want)
    assert rel.max() <= 1e-3, (got, want)
