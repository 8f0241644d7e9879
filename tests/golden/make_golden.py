"""Generates the golden fixtures from the reference implementation itself.

Runs only where the reference checkout is present (pass its path with --reference, or set
ANVIL_REFERENCE): it imports the reference's front end and NumPy interpreter, and writes

  programs   tests/golden/<name>.kir.json.gz   the optimized IR of tests/programs/<name>.anvil
             tests/golden/<name>.out.txt       what the reference interpreter printed
             tests/golden/<name>.meta.json     exit status / error text
             tests/golden/<name>.npz           final contents of the program's tensors
  configs    anvil_lang_b200/programs/<cfg>.kir.json.gz     the IR of the benchmark configurations
  functions  anvil_lang_b200/programs/lowered/*.kir.json.gz the per-shape lowering of the standalone
             functions, and tests/golden/fn_<name>.npz with interpreter outputs at reduced sizes
  traj       tests/golden/<cfg>.losses.json    the first N training losses of a configuration

The fixtures are data produced BY the reference (not reference source); the tests compare the CPU
oracle and the CUDA path against them.
"""
from __future__ import annotations

import argparse
import glob
import io
import json
import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

FULL_LIMIT = 1 << 14          # tensors up to this many elements are stored whole
SAMPLE = 4096                 # larger ones: this many leading elements plus sums


def summarize(arr: np.ndarray) -> dict:
    out = {}
    if arr.size <= FULL_LIMIT:
        out["full"] = arr
    else:
        out["head"] = arr[:SAMPLE].copy()
        a64 = arr.astype(np.float64)
        out["stats"] = np.array([a64.sum(), np.abs(a64).sum(), float(arr.size)])
    return out


def run_reference(prog, seed=0, stdin=""):
    from anvil.interp import AnvilRuntimeError, Interpreter, ProgramExit
    out = io.StringIO()
    it = Interpreter(prog, out=out, seed=seed, inp=io.StringIO(stdin))
    meta = {"exit": 0, "error": ""}
    try:
        it.run()
    except ProgramExit as e:
        meta["exit"] = e.code
    except AnvilRuntimeError as e:
        meta["exit"] = 1
        meta["error"] = str(e)
    return out.getvalue(), meta, it


def do_programs(names):
    from anvil.driver import compile_file
    from anvil_lang_b200 import kir
    for path in sorted(glob.glob(os.path.join(ROOT, "tests", "programs", "*.anvil"))):
        name = os.path.splitext(os.path.basename(path))[0]
        if names and name not in names:
            continue
        t = time.time()
        c = compile_file(path)
        k = kir.from_anvil(c.program, f"tests/programs/{name}.anvil")
        kir.dump(k, os.path.join(HERE, f"{name}.kir.json.gz"))
        text, meta, it = run_reference(c.program)
        with open(os.path.join(HERE, f"{name}.out.txt"), "w") as f:
            f.write(text)
        with open(os.path.join(HERE, f"{name}.meta.json"), "w") as f:
            json.dump(meta, f)
        arrays = {}
        for b in k.roots():
            for key, v in summarize(it.mem[b.id][:max(b.numel, 1)]).items():
                arrays[f"b{b.id}_{key}"] = v
        np.savez_compressed(os.path.join(HERE, f"{name}.npz"), **arrays)
        print(f"{name}: {len(k.kernels())} kernels, exit {meta['exit']}, {time.time() - t:.1f}s")


CONFIGS = ["c1_mlp_sgd", "c3_mlp_adam", "c4_cnn_sgd", "c5_transformer"]


def do_configs():
    from anvil.driver import compile_file
    from anvil_lang_b200 import kir
    for name in CONFIGS:
        c = compile_file(os.path.join(ROOT, "anvil_lang_b200", "programs", f"{name}.anvil"))
        k = kir.from_anvil(c.program, f"{name}.anvil")
        kir.dump(k, os.path.join(ROOT, "anvil_lang_b200", "programs", f"{name}.kir.json.gz"))
        print(name, len(k.kernels()), "kernels")


def do_dp():
    """The same programs compiled for the global batch and for the per-rank batches of 2/4/8 ranks."""
    from anvil.driver import compile_file
    from anvil_lang_b200 import kir
    jobs = [(os.path.join(ROOT, "tests", "programs", "dp_mlp.anvil"), HERE, "dp_mlp", 32, (1, 2, 4)),
            (os.path.join(ROOT, "tests", "programs", "transformer_small.anvil"), HERE, "dp_transformer", 4, (1, 2)),
            (os.path.join(ROOT, "anvil_lang_b200", "programs", "c5_transformer.anvil"),
             os.path.join(ROOT, "anvil_lang_b200", "programs"), "c5_transformer", 64, (2, 4, 8)),
            (os.path.join(ROOT, "anvil_lang_b200", "programs", "c3_mlp_adam.anvil"),
             os.path.join(ROOT, "anvil_lang_b200", "programs"), "c3_mlp_adam", 256, (2, 4, 8))]
    for path, outdir, name, batch, worlds in jobs:
        for g in worlds:
            c = compile_file(path, consts={"BATCH": batch // g})
            k = kir.from_anvil(c.program, f"{name} (batch {batch // g})")
            kir.dump(k, os.path.join(outdir, f"{name}.b{batch // g}.kir.json.gz"))
            print(name, "batch", batch // g, len(k.kernels()), "kernels")


def do_traj(name, steps, consts=None, suffix=""):
    """The first `steps` values of `loss` in the training loop, read after each iteration."""
    from anvil import ir
    from anvil.driver import compile_file
    from anvil.interp import Interpreter
    from anvil_lang_b200 import kir
    from anvil_lang_b200.backend.analysis import hot_loop
    path = os.path.join(ROOT, "anvil_lang_b200", "programs", f"{name}.anvil")
    if not os.path.exists(path):                    # a test-only program
        path = os.path.join(ROOT, "tests", "programs", f"{name}.anvil")
    c = compile_file(path, consts=consts)
    k = kir.from_anvil(c.program, name)
    hot = hot_loop(k)
    if consts:                      # a variant of a configuration: its IR travels with the losses
        kir.dump(k, os.path.join(HERE, f"{name}{suffix}.traj.kir.json.gz"))
    loss = [b for b in c.program.buffers if b.name == "loss"][-1]
    losses, times = [], []

    class Stop(Exception):
        pass

    class Stepper(Interpreter):
        def exec_for(self, st: ir.For):
            if st.counter.id != hot.counter.id:
                return super().exec_for(st)
            cnt = self.arr(st.counter)
            cnt[0] = self.bound(st.start)
            stop = self.bound(st.stop)
            while cnt[0] < stop:
                t = time.time()
                self.exec_block(st.body)
                times.append(time.time() - t)
                losses.append(float(self.arr(loss)[0]))
                print(f"  step {len(losses)} loss {losses[-1]:.6f} ({times[-1]:.1f}s)", flush=True)
                if len(losses) >= steps:
                    raise Stop()
                cnt[0] += st.step

    it = Stepper(c.program, out=io.StringIO(), seed=0)
    try:
        it.run()
    except Stop:
        pass
    out = {"config": name, "consts": consts or {}, "seed": 0, "losses": losses,
           "seconds_per_step_reference_interpreter": float(np.median(times)),
           "numpy": np.__version__}
    with open(os.path.join(HERE, f"{name}{suffix}.losses.json"), "w") as f:
        json.dump(out, f, indent=1)
    return it, k, c


FUNCTIONS = {
    "rows": "fn rows(x: [n, d]) = softmax(x)\n",
    "ln": "fn ln(x: [n, d], g: [d], b: [d]) = layer_norm(x) * g + b\n",
    "lin": "fn lin(x: [n, d], W: [d, k], b: [k]):\n    y[i, k] = sum x[i, j] * W[j, k] + b[k]\n    return y\n",
}


def fn_inputs(name, small: bool, seed=0):
    """Seeded N(0,1) inputs of the standalone-function configuration (full or reduced size)."""
    rng = np.random.default_rng(seed)
    if name == "rows":
        n, d = (64, 4096) if small else (4096, 4096)
        return [rng.standard_normal((n, d), dtype=np.float32)]
    if name == "ln":
        n, d = (128, 1024) if small else (8192, 1024)
        return [rng.standard_normal((n, d), dtype=np.float32), np.ones(d, np.float32), np.zeros(d, np.float32)]
    n, d, k = (96, 1024, 256) if small else (8192, 1024, 4096)
    return [rng.standard_normal((n, d), dtype=np.float32),
            (rng.standard_normal((d, k), dtype=np.float32) * np.float32(0.02)),
            rng.standard_normal(k, dtype=np.float32)]


def do_functions():
    from anvil import pyapi as ref
    from anvil.interp import Interpreter
    from anvil_lang_b200 import kir
    from anvil_lang_b200 import pyapi as mine
    os.makedirs(mine.LOWERED_DIR, exist_ok=True)
    for name, src in FUNCTIONS.items():
        for small in (True, False):
            arrays = fn_inputs(name, small)
            _, sig = mine.arguments(arrays)
            lo = ref.lower(src, os.path.join(os.getcwd(), "<python>.anvil"), name, sig, seed=0)
            prog = kir.from_anvil(lo.prog, f"fn {name}")
            by_id = {b.id: b for b in prog.buffers}
            mlo = mine.Lowered(prog, [by_id[b.id] for b in lo.inputs],
                               [None if b is None else by_id[b.id] for b in lo.outputs], list(lo.consts), lo.tuple_result)
            mine.save_lowered(mlo, os.path.join(mine.LOWERED_DIR, mine.lowered_key(src, name, sig, 0) + ".kir.json.gz"))
            if small:
                it = Interpreter(lo.prog, out=io.StringIO(), seed=0)
                for b, a in zip(lo.inputs, arrays):
                    it.mem[b.root.id][:a.size] = a.reshape(-1)
                it.run()
                outs = {f"out{i}": it.arr(b)[:b.numel].reshape(b.shape).copy() for i, b in enumerate(lo.outputs)}
                np.savez_compressed(os.path.join(HERE, f"fn_{name}.npz"), **outs)
            print(name, "small" if small else "full", sig)


def reference_test_programs(reference: str):
    """The programs of the reference's own CUDA tests (its tests/test_cuda.py), read from the reference checkout at
    generation time: the example files with the substitutions and constants those tests use, and the program texts
    the tests define inline (found by walking the test module's syntax tree, so no text is restated here).
    Yields (fixture name, program text, path for diagnostics, constants, standard input)."""
    import ast

    def example(name, replace=()):
        path = os.path.join(reference, "examples", f"{name}.anvil")
        src = open(path).read()
        for old, new in replace:
            assert old in src, old
            src = src.replace(old, new)
        return src, path
    for name in ("hello", "linear_regression", "attention"):
        src, path = example(name)
        yield f"ref_{name}", src, path, None, ""
    src, path = example("snake", [("sleep(0.05)", "sleep(0.0)")])
    yield "ref_snake", src, path, {"EPISODES": 4}, ""
    src, path = example("checkers", [("sleep(0.15)", "sleep(0.0)"), ("{clock() - start:.1f}s", "{0 * start:.1f}s")])
    yield "ref_checkers", src, path, {"GAMES": 3, "MATCH": 2, "MAX_PLY": 30, "PLAY": 1, "PLAY_DEPTH": 2,
                                      "SAVE": "/nonexistent/c.weights"}, "3\n9\nx\n1\n1\n"
    # The two examples that read files get synthetic stand-ins of the same layout (the text the language model
    # trains on, the digit images of the diffusion model): tests/programs/data/make_data.py writes them from a seed.
    sys.path.insert(0, os.path.join(ROOT, "tests", "programs", "data"))
    import make_data
    corpus = os.path.join(ROOT, "tests", "programs", "data", "corpus.txt")
    make_data.write_corpus(corpus)
    src, path = example("transformer", [("{clock() - start:.1f}s", "{0 * start:.1f}s"), ("step % 250 == 249", "step % 5 == 4"),
                                        ('bytes("../README.md")', f'bytes("{corpus}")')])
    yield "ref_transformer", src, path, {"STEPS": 20, "BATCH": 4, "T": 8, "D": 16, "HEADS": 2, "SAMPLE": 10}, ""
    digits = "/tmp/anvil_synthetic_digits"
    os.makedirs(digits, exist_ok=True)
    make_data.write_digit_set(digits)
    src, path = example("diffusion", [("{clock() - start:.1f}s", "{0 * start:.1f}s"),
                                      ('idx("data/train-images-idx3-ubyte.gz")', f'idx("{digits}/train-images-idx3-ubyte.gz")'),
                                      ('idx("data/train-labels-idx1-ubyte.gz")', f'idx("{digits}/train-labels-idx1-ubyte.gz")')])
    yield "ref_diffusion", src, path, {"EPOCHS": 1, "T": 8, "H": 16, "BATCH": 3000, "PER_DIGIT": 1}, ""
    tree = ast.parse(open(os.path.join(reference, "tests", "test_cuda.py")).read())
    texts = {}
    for node in tree.body:                                   # module-level NAME = """program"""
        if isinstance(node, ast.Assign) and isinstance(node.value, ast.Constant) and isinstance(node.value.value, str):
            texts[node.targets[0].id] = node.value.value
    yield "ref_split", texts["SPLIT"], "<test>.anvil", None, ""
    for fn in (n for n in tree.body if isinstance(n, ast.FunctionDef)):
        strings = [c.value for c in ast.walk(fn) if isinstance(c, ast.Constant) and isinstance(c.value, str)
                   and "\n" in c.value and c.value != ast.get_docstring(fn)]
        if fn.name == "test_scatter_add_and_gather":
            yield "ref_scatter_gather", strings[0], "<test>.anvil", None, ""
        elif fn.name == "test_runtime_bounds_check":
            yield "ref_bounds_loop", strings[0], "<test>.anvil", None, ""
        elif fn.name == "test_gather_out_of_bounds_inside_a_kernel":
            yield "ref_bounds_gather", strings[0], "<test>.anvil", None, ""
        elif fn.name == "test_save_load_and_assert":
            yield "ref_assert", [s_ for s_ in strings if "assert x < 2" in s_][0], "<test>.anvil", None, ""


def do_reftests(reference, names):
    """Fixtures `ref_*`: the IR the reference front end makes of those programs, what its interpreter prints, the exit
    status and error text, and the standard input fed to it."""
    from anvil.driver import compile_text
    from anvil_lang_b200 import kir
    for name, src, path, consts, stdin in reference_test_programs(reference):
        if names and name not in names:
            continue
        t = time.time()
        c = compile_text(src, path=path, consts=consts)
        k = kir.from_anvil(c.program, f"{name} (reference tests/test_cuda.py)")
        kir.dump(k, os.path.join(HERE, f"{name}.kir.json.gz"))
        text, meta, it = run_reference(c.program, stdin=stdin)
        meta["stdin"] = stdin
        with open(os.path.join(HERE, f"{name}.out.txt"), "w") as f:
            f.write(text)
        with open(os.path.join(HERE, f"{name}.meta.json"), "w") as f:
            json.dump(meta, f)
        np.savez_compressed(os.path.join(HERE, f"{name}.npz"))            # text-level fixtures: no tensors kept
        print(f"{name}: {len(k.kernels())} kernels, exit {meta['exit']} {meta['error'][:60]!r}, "
              f"{os.path.getsize(os.path.join(HERE, f'{name}.kir.json.gz')) // 1024} KB, {time.time() - t:.1f}s", flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["programs", "configs", "functions", "traj", "dp", "reftests"])
    ap.add_argument("args", nargs="*")
    ap.add_argument("--reference", default=os.environ.get("ANVIL_REFERENCE", os.path.join(os.path.dirname(ROOT), "reference")))
    a = ap.parse_args()
    sys.path.insert(0, a.reference)
    os.environ.setdefault("ANVIL_CACHE", "/tmp/anvil_cache")
    sys.dont_write_bytecode = True
    if a.what == "programs":
        do_programs(a.args)
    elif a.what == "configs":
        do_configs()
    elif a.what == "functions":
        do_functions()
    elif a.what == "dp":
        do_dp()
    elif a.what == "reftests":
        do_reftests(a.reference, a.args)
    else:
        name, steps = a.args[0], int(a.args[1])
        consts = json.loads(a.args[2]) if len(a.args) > 2 else None
        suffix = a.args[3] if len(a.args) > 3 else ""
        do_traj(name, steps, consts, suffix)


if __name__ == "__main__":
    main()
