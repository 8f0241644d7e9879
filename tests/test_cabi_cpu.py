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
