"""The allocation-free column sum, `anvil_colsum_f32_static`, against the compiler-generated kernel.

Some callers of this library may not allocate device memory when they call it (a plug-in inside a
framework that owns all device memory, a process with a fixed memory budget, a latency-critical loop):
for them the library offers one entry point whose scratch space is a fixed array inside the library.
Here it is called through the C ABI on the same input as the generated split column reduction (which
keeps its partial sums in the cudaMalloc'd arena), twice in a row, and must give the same sums; a size
beyond the fixed array must be refused with status 2 and must launch nothing.

This file sorts last on purpose, so a run that stops at the first failure has already run every other
test."""
import ctypes

import numpy as np
import pytest

from anvil_lang_b200 import kir
from anvil_lang_b200.kir import F32, Affine, E, Kernel, KernelStmt, Reduction, Store
from anvil_lang_b200.program import DeviceProgram
from kirbuild import buf, nid, var

pytestmark = pytest.mark.gpu


def colsum_program(rows, cols):
    x, out = buf("x", (rows, cols)), buf("out", (cols,))
    out2 = buf("out2", (cols,), kind="var")                  # written only from outside the program: a tensor no kernel touches gets no memory unless it is a variable
    i, j = var("i", rows), var("j", cols)
    body = E("load", F32, buf=x, off=Affine(0, [(i, cols), (j, 1)]))
    k = Kernel(nid(), "colsum", "column sums", [j], [Store(out, Affine(0, [(j, 1)]), E("acc", F32))],
               Reduction([i], "sum", body))
    return kir.Program(kir.Block([KernelStmt(k)]), [x, out, out2], "column sums"), k, x, out, out2


@pytest.mark.parametrize("rows,cols", [(3000, 512), (16384, 2048), (257, 70)])
def test_static_scratch_column_sum_matches_generated_kernel(rows, cols):
    prog, k, x, out, out2 = colsum_program(rows, cols)
    dp = DeviceProgram(prog, graphs=False)
    try:
        rng = np.random.default_rng(rows + cols)
        for call in range(2):                                   # two calls in a row share the fixed scratch
            data = rng.standard_normal((rows, cols), dtype=np.float32)
            dp.write(x, data)
            dp.launch(k)                                        # existing entry point: partials in the arena
            want = dp.read(out).copy()
            rc = dp.rtlib.anvil_colsum_f32_static(ctypes.c_void_p(dp.ptr(x)), rows, cols, ctypes.c_void_p(dp.ptr(out2)),
                                                  ctypes.c_void_p(dp.stream))
            assert rc == 0
            dp.sync()
            got = dp.read(out2)
            scale = np.abs(want).max()
            assert np.abs(got - want).max() <= 1e-4 * scale
            ref = data.astype(np.float64).sum(axis=0)
            assert np.abs(got - ref).max() <= 1e-4 * np.abs(ref).max()
    finally:
        dp.close()


def test_static_scratch_refuses_sizes_beyond_its_array():
    prog, k, x, out, out2 = colsum_program(8, 8)
    dp = DeviceProgram(prog, graphs=False)
    try:
        before = dp.read(out2).copy()
        cols = (1 << 20) + 32                                   # one split already exceeds the fixed array
        rc = dp.rtlib.anvil_colsum_f32_static(ctypes.c_void_p(dp.ptr(x)), 4, cols, ctypes.c_void_p(dp.ptr(out2)),
                                              ctypes.c_void_p(dp.stream))
        assert rc == 2
        dp.sync()
        assert np.array_equal(dp.read(out2), before)
    finally:
        dp.close()
