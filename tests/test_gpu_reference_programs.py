"""The programs of the reference's own CUDA tests (its tests/test_cuda.py) on the device.

There each program is compiled to CUDA text, built as C++ with the launches emulated by loops, run as a child process
and its output compared with the interpreter's (`check_cuda`, `outputs_match`: same text, numbers within 2e-3). Here
the same programs — the hello / linear regression / attention / snake / checkers / transformer / diffusion examples
with the constants and substitutions those tests use, the split-reduction, scatter / gather, bounds-fault and assert
programs — arrive as the IR the reference front end made of them (tests/golden/ref_*.kir.json.gz, written by
`make_golden.py reftests` together with what the reference interpreter printed), run on the GPU as child processes
(`python -m anvil_lang_b200.cuda`) with the same standard input, and are held to the same comparison.

The two examples that read files train on seeded synthetic stand-ins (a pseudo-text, random digit-shaped images)
written by tests/programs/data/make_data.py, found through ANVIL_DATA."""
import json
import os
import shutil
import subprocess
import sys

import pytest

from util import GOLDEN, ROOT, golden_names, outputs_match

pytestmark = pytest.mark.gpu

NAMES = golden_names(reference_tests=True)


@pytest.fixture(scope="module")
def data_dir(tmp_path_factory):
    d = tmp_path_factory.mktemp("anvil_data")
    sys.path.insert(0, os.path.join(ROOT, "tests", "programs", "data"))
    import make_data
    shutil.copy(os.path.join(ROOT, "tests", "programs", "data", "corpus.txt"), d / "corpus.txt")
    make_data.write_digit_set(str(d))
    return str(d)


def run_child(name, data_dir, stdin):
    env = dict(os.environ, ANVIL_DATA=data_dir, PYTHONPATH=ROOT)
    return subprocess.run([sys.executable, "-m", "anvil_lang_b200.cuda", os.path.join(GOLDEN, f"{name}.kir.json.gz")],
                          input=stdin, capture_output=True, encoding="utf-8", errors="replace", timeout=900, env=env, cwd=ROOT)


@pytest.mark.parametrize("name", NAMES)
def test_reference_cuda_test_program(name, data_dir):
    want = open(os.path.join(GOLDEN, f"{name}.out.txt")).read()
    meta = json.load(open(os.path.join(GOLDEN, f"{name}.meta.json")))
    r = run_child(name, data_dir, meta.get("stdin", ""))
    if name == "ref_assert":                       # a failed `assert`: the message on stderr, a non-zero status, nothing printed after it
        assert r.returncode != 0 and "x is too big" in r.stderr and "unreachable" not in r.stdout
        return
    if meta["exit"] != 0:                          # the two bounds faults
        assert r.returncode != 0 and "out of bounds" in r.stderr, (r.returncode, r.stderr[-500:])
        if name == "ref_bounds_loop":
            assert r.stdout.split() == [str(i) for i in range(10)]
        else:
            assert "got 7" in r.stderr
        return
    assert r.returncode == 0, r.stderr[-2000:]
    ok, why = outputs_match(r.stdout, want)
    assert ok, why
