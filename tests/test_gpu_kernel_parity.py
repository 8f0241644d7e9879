"""Kernel-by-kernel parity inside one training step: the oracle runs the program up to the training
loop and then one step kernel by kernel; before each kernel every tensor it touches is copied from the
oracle's memory to the device, the device runs that one kernel through the program library's launch
table, and its outputs are compared with the oracle's (i32 exactly, f32 to 1e-4 of the tensor's
magnitude). Errors therefore cannot hide behind, or leak into, neighbouring kernels."""
import io
import os

import numpy as np
import pytest

from anvil_lang_b200 import kir
from anvil_lang_b200.backend.analysis import hot_loop
from anvil_lang_b200.program import DeviceProgram
from oracle.kir_interp import Oracle
from util import GOLDEN, ROOT, tensor_close

pytestmark = pytest.mark.gpu

CASES = [
    ("c1", os.path.join(ROOT, "anvil_lang_b200", "programs", "c1_mlp_sgd.kir.json.gz"), 2),
    ("c3", os.path.join(ROOT, "anvil_lang_b200", "programs", "c3_mlp_adam.kir.json.gz"), 2),
    ("c4", os.path.join(ROOT, "anvil_lang_b200", "programs", "c4_cnn_sgd.kir.json.gz"), 1),
    ("c5_reduced", os.path.join(GOLDEN, "c5_transformer_small.traj.kir.json.gz"), 2),
    # the same reduced transformer with its (small) products forced onto the tensor-core templates
    ("c5_reduced_tc", os.path.join(GOLDEN, "c5_transformer_small.traj.kir.json.gz"), 2),
]


def run_to_loop(o, prog, hot):
    class Reached(Exception):
        pass

    def walk(block):
        for st in block.stmts:
            if st is hot:
                o.arr(hot.counter)[0] = hot.start
                raise Reached()
            if isinstance(st, kir.For):
                o.arr(st.counter)[0] = o.bound(st.start)
                walk(st.body)
            else:
                o.stmt(st)
    try:
        walk(prog.main)
    except Reached:
        pass


@pytest.mark.parametrize("name,path,steps", CASES, ids=[c[0] for c in CASES])
def test_each_kernel_of_a_step(name, path, steps):
    prog = kir.load(path)
    prog_text = " ".join(b.name for b in prog.buffers)
    hot = hot_loop(prog)
    o = Oracle(prog, out=io.StringIO(), seed=0, mode="fast")
    run_to_loop(o, prog, hot)
    if name.endswith("_tc"):
        os.environ["ANVIL_B200_TC_MIN_MFLOP"] = "0"
    try:
        dp = DeviceProgram(prog, seed=0, graphs=False)
    finally:
        os.environ.pop("ANVIL_B200_TC_MIN_MFLOP", None)
    if name.endswith("_tc"):
        assert any(n.startswith("gemm tc") for n in dp.gen.kernel_notes)
    bad = []
    try:
        for step in range(steps):
            for st in hot.body.stmts:
                if not isinstance(st, kir.KernelStmt):
                    continue
                k = st.kernel
                touched = {b.id: b for b in list(k.reads()) + list(k.writes())}
                for b in touched.values():
                    dp.write(b, o.arr(b)[:max(b.numel, 1)])
                dp.rtlib.anvil_rt_set_stream(dp.rt, o.stream)
                o.kernel(k)
                dp.launch(k)
                for b in k.writes():
                    # Adam divides by sqrt(v) + 1e-8: where a gradient is a sum that cancels to ~1e-9, the
                    # update g / (|g| + eps) turns the sum's rounding noise into a 1e-3 relative change of the
                    # parameter. The moments are linear (m) and quadratic (v) in the gradient: they keep 1e-4.
                    tol = 5e-3 if b.kind == "param" and "adam" in prog_text else 1e-4
                    ok, why = tensor_close(dp.read(b).reshape(-1), o.arr(b)[:b.numel], tol)
                    if not ok:
                        bad.append(f"step {step} {k.name} <{k.label}> [{dp.gen.kernel_notes[dp.gen.kernel_index[k.id]]}] "
                                   f"{b.name}{list(b.shape)}: {why}")
            o.arr(hot.counter)[0] += hot.step
        dp.check_faults()
    finally:
        dp.close()
    assert not bad, "\n".join(bad[:20])
