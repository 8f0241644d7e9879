"""Shared helpers for the tests: fixture loading and the comparison rules.

The comparison rule for program output is the reference's (tests/util.py:99-112 there): the text
must be identical once numbers are cut out, and the numbers must agree within a tolerance. The
per-tensor rule is the parity bar of this project: i32 tensors exactly, f32 tensors to 1e-4 of the
tensor's magnitude.
"""
import glob
import json
import os
import re

import numpy as np

from anvil_lang_b200 import kir

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")
NUM = re.compile(r"-?\d+\.\d+(?:e[+-]?\d+)?|-?\d+(?:e[+-]?\d+)?|-?inf|nan")


def golden_names(reference_tests=False):
    """Fixture programs with a recorded output: the project's own texts, or (reference_tests=True) the programs of the
    reference's CUDA tests, which run as child processes with their own standard input."""
    names = sorted(os.path.basename(p)[:-len(".kir.json.gz")] for p in glob.glob(os.path.join(GOLDEN, "*.kir.json.gz")))
    return [n for n in names if os.path.exists(os.path.join(GOLDEN, f"{n}.out.txt")) and n.startswith("ref_") == reference_tests]


def load_golden(name):
    prog = kir.load(os.path.join(GOLDEN, f"{name}.kir.json.gz"))
    with open(os.path.join(GOLDEN, f"{name}.out.txt")) as f:
        text = f.read()
    with open(os.path.join(GOLDEN, f"{name}.meta.json")) as f:
        meta = json.load(f)
    arrays = dict(np.load(os.path.join(GOLDEN, f"{name}.npz")))
    return prog, text, meta, arrays


def outputs_match(a: str, b: str, rtol=2e-3, atol=2e-3):
    ta, tb = NUM.split(a), NUM.split(b)
    if ta != tb:
        return False, f"text differs:\n--- got\n{a[:2000]}\n--- want\n{b[:2000]}"
    for x, y in zip(NUM.findall(a), NUM.findall(b)):
        if x == y:
            continue
        fx, fy = float(x), float(y)
        if not abs(fx - fy) <= atol + rtol * abs(fy):
            return False, f"{x} vs {y}"
    return True, ""


def tensor_close(got: np.ndarray, want: np.ndarray, rel=1e-4):
    """i32: exact. f32: max|a-b| <= rel * max(|want|, tiny), nan/inf positions equal."""
    got, want = np.asarray(got).reshape(-1), np.asarray(want).reshape(-1)
    if want.dtype.kind in "iu":
        return np.array_equal(got, want), "integer tensor differs"
    fin = np.isfinite(want)
    if not np.array_equal(fin, np.isfinite(got)):
        return False, "non-finite positions differ"
    if not np.array_equal(got[~fin], want[~fin], equal_nan=True):
        return False, "non-finite values differ"
    if not fin.any():
        return True, ""
    scale = max(float(np.abs(want[fin]).max()), 1e-30)
    err = float(np.abs(got[fin].astype(np.float64) - want[fin]).max())
    return err <= rel * scale, f"max error {err:.3e} vs scale {scale:.3e}"


def check_arrays(read, prog, arrays, rel=1e-4, skip=()):
    """`read(buffer) -> flat array`; compares against what make_golden.py stored. `skip`: names or
    root ids to leave out (temporaries that a fused kernel keeps in registers are never stored)."""
    bad = []
    for b in prog.roots():
        if b.name in skip or b.id in skip:
            continue
        full = arrays.get(f"b{b.id}_full")
        got = read(b)
        if full is not None:
            ok, why = tensor_close(got[:full.size], full, rel)
        else:
            head = arrays.get(f"b{b.id}_head")
            if head is None:
                continue
            ok, why = tensor_close(got[:head.size], head, rel)
            if ok:
                s = arrays[f"b{b.id}_stats"]
                g64 = got[:int(s[2])].astype(np.float64)
                ok = abs(g64.sum() - s[0]) <= 1e-4 * max(s[1], 1e-30)
                why = f"sum {g64.sum()} vs {s[0]}"
        if not ok:
            bad.append(f"{b.name}#{b.id}{list(b.shape)}: {why}")
    return bad


def device_program(prog, unshared_arena=False, **kw):
    """A DeviceProgram; `unshared_arena` builds it with every tensor in memory of its own (ANVIL_B200_ARENA=unshared),
    so that temporaries can still be read after the run (by default dead temporaries give their bytes to later ones)."""
    from anvil_lang_b200.program import DeviceProgram
    if unshared_arena:
        os.environ["ANVIL_B200_ARENA"] = "unshared"
    try:
        return DeviceProgram(prog, **kw)
    finally:
        os.environ.pop("ANVIL_B200_ARENA", None)
