"""The C ABI without a GPU: libanvil_cuda.so loads and exports every function that
include/anvil_cuda.h declares; a generated program library exports the documented entry points."""
import ctypes
import os
import re

from anvil_lang_b200.backend import build, emit
from util import ROOT, load_golden


def declared_functions():
    text = open(os.path.join(ROOT, "include", "anvil_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = set(re.findall(r"\b(anvil_[a-z0-9_]+)\s*\(", text))
    return sorted(n for n in names if not n.endswith("_fn"))


def test_runtime_exports_every_declared_symbol():
    build.build_runtime()
    lib = ctypes.CDLL(build.RT_LIB)
    names = declared_functions()
    assert len(names) > 50
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_program_library_exports_its_entry_points():
    prog, _, _, _ = load_golden("train_mlp")
    src, gen = emit.generate(prog, 0)
    path = build.build_program(src)
    build.load_runtime()
    lib = ctypes.CDLL(path)
    for name in ("anvil_b200_main", "anvil_b200_step", "anvil_b200_step_fed", "anvil_b200_launch",
                 "anvil_b200_kernel_count", "anvil_b200_arena_bytes", "anvil_b200_seed"):
        assert hasattr(lib, name), name
    lib.anvil_b200_kernel_count.restype = ctypes.c_int
    assert lib.anvil_b200_kernel_count() == len(gen.kernels)


def test_function_library_exports_the_reference_abi():
    from anvil_lang_b200 import pyapi
    import glob
    f = sorted(glob.glob(os.path.join(pyapi.LOWERED_DIR, "*.kir.json.gz")))[0]
    lo = pyapi.load_lowered(f)
    src, _ = emit.generate(lo.prog, 0)
    lib = ctypes.CDLL(build.build_program(src))
    assert hasattr(lib, "anvil_entry")
    for b in lo.inputs + [o for o in lo.outputs if o is not None]:
        ctypes.c_void_p.in_dll(lib, f"anvil_{b.name}")        # raises if the slot is missing


def test_static_column_sum_refuses_bad_arguments_without_launching():
    """Status codes that are decided before any CUDA call: a missing output with columns to write (also when there
    are no rows: the sums are then zeros and still stored), a missing input with elements to read, negative sizes."""
    lib = build.load_runtime()
    f = lib.anvil_colsum_f32_static
    dummy = ctypes.c_void_p(0x1000)                           # never dereferenced: every call below is refused or empty
    assert f(dummy, 0, 8, None, None) == 1                    # no rows, columns, no output
    assert f(None, 4, 8, dummy, None) == 1                    # elements to read, no input
    assert f(dummy, -1, 8, dummy, None) == 1
    assert f(dummy, 4, -1, dummy, None) == 1
    assert f(None, 4, 0, None, None) == 0                     # nothing to do
