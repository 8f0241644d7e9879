"""`export`: a lowered function with baked weights as lib<name>.so + <name>.h (reference: anvil/export.py:68-161).

Host side here (header text, wrapper code, the library builds with nvcc and exports the symbols); on a GPU the
library is loaded by a fresh process with nothing but ctypes and called like from C."""
import ctypes
import os
import subprocess
import sys

import numpy as np
import pytest

from anvil_lang_b200 import export, kir, pyapi
from anvil_lang_b200.kir import F32, Affine, Buffer, E, Kernel, KernelStmt, Reduction, Store, Var
from kirbuild import nid

M, K, N = 96, 128, 64


def lowered_linear():
    """y = relu(x W + b) with W and b baked in as constants."""
    rng = np.random.default_rng(5)
    W = Buffer(nid(), "W", (K, N), F32, "const", init=(rng.standard_normal(K * N) * 0.1).astype(np.float32))
    b = Buffer(nid(), "b", (N,), F32, "const", init=rng.standard_normal(N).astype(np.float32))
    x = Buffer(nid(), "input0", (M, K), F32, "input")
    y = Buffer(nid(), "output0", (M, N), F32, "output")
    i, j, k = Var(nid(), "i", M), Var(nid(), "j", N), Var(nid(), "k", K)
    body = E("bin", F32, op="mul", a=[E("load", F32, buf=x, off=Affine(0, [(i, K), (k, 1)])),
                                       E("load", F32, buf=W, off=Affine(0, [(k, N), (j, 1)]))])
    val = E("bin", F32, op="max", a=[E("bin", F32, op="add", a=[E("acc", F32), E("load", F32, buf=b, off=Affine(0, [(j, 1)]))]),
                                       E("const", F32, val=0.0)])
    kern = Kernel(nid(), "k1", "linear", [i, j], [Store(y, Affine(0, [(i, N), (j, 1)]), val, False)], Reduction([k], "sum", body))
    prog = kir.Program(kir.Block([KernelStmt(kern)]), [x, W, b, y], "exported linear")
    return pyapi.Lowered(prog, [x], [y], [], False), W.init.reshape(K, N), b.init


def test_header_and_wrapper_text():
    lo, _, _ = lowered_linear()
    h = export.header_text(lo, "digits_read")
    assert "int digits_read(const float *arg0, float *result0);" in h
    assert "arg0: float[96, 128]" in h and "result0: float[96, 64]" in h and "digits_read_last_error" in h
    proto, _ = export.signature(lo, "f")
    assert proto == "int f(const float *arg0, float *result0)"
    assert export.c_ident("9-lives") == "_9_lives"


def test_library_builds_and_exports_the_function(tmp_path):
    lo, _, _ = lowered_linear()
    lib, header = export.export(lo, "lin_relu", str(tmp_path))
    assert os.path.exists(header) and os.path.exists(os.path.join(str(tmp_path), "libanvil_cuda.so"))
    names = subprocess.run(["nm", "-D", "--defined-only", lib], capture_output=True, text=True).stdout
    assert " lin_relu" in names and "lin_relu_last_error" in names and "anvil_entry" in names
    src = open(os.path.join(str(tmp_path), "lin_relu.cu")).read()
    assert "export_init_" in src and src.count("anvil_rt_h2d(rt,") == 2          # W and b are uploaded once


CHILD = r"""
import ctypes, sys
import numpy as np
lib = ctypes.CDLL(sys.argv[1])
lib.lin_relu.restype = ctypes.c_int
lib.lin_relu.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
x = np.load(sys.argv[2]); y = np.empty((x.shape[0], int(sys.argv[4])), np.float32)
for _ in range(2):                                   # the second call reuses the context and the constants
    y[:] = -1
    rc = lib.lin_relu(x.ctypes.data, y.ctypes.data)
    assert rc == 0, rc
np.save(sys.argv[3], y)
"""


@pytest.mark.gpu
def test_exported_function_called_from_a_fresh_process(tmp_path):
    lo, W, b = lowered_linear()
    lib, _ = export.export(lo, "lin_relu", str(tmp_path))
    x = np.random.default_rng(6).standard_normal((M, K)).astype(np.float32)
    xin, yout = os.path.join(str(tmp_path), "x.npy"), os.path.join(str(tmp_path), "y.npy")
    np.save(xin, x)
    r = subprocess.run([sys.executable, "-c", CHILD, lib, xin, yout, str(N)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    want = np.maximum(x.astype(np.float64) @ W.astype(np.float64) + b, 0)
    got = np.load(yout)
    assert np.abs(got - want).max() <= 1e-5 * max(1.0, np.abs(want).max())
