"""`anvil.function` on the device: the standalone kernels of the BASELINE configuration
(row softmax f32[4096,4096], layer norm f32[8192,1024], Linear 8192x1024 -> 4096) through the
reference-facing call (NumPy arrays in, NumPy arrays out, host pointers through the `anvil_entry` ABI).
Reduced sizes are compared with the reference interpreter's outputs (tests/golden/fn_*.npz), full sizes
with float64 NumPy formulas; f32 tolerance 1e-4 of the output's magnitude."""
import os

import numpy as np
import pytest

from anvil_lang_b200 import pyapi
from util import GOLDEN

pytestmark = pytest.mark.gpu

SOURCES = {
    "rows": "fn rows(x: [n, d]) = softmax(x)\n",
    "ln": "fn ln(x: [n, d], g: [d], b: [d]) = layer_norm(x) * g + b\n",
    "lin": "fn lin(x: [n, d], W: [d, k], b: [k]):\n    y[i, k] = sum x[i, j] * W[j, k] + b[k]\n    return y\n",
}


def inputs(name, small, seed=0):
    rng = np.random.default_rng(seed)
    if name == "rows":
        n, d = (64, 4096) if small else (4096, 4096)
        return [rng.standard_normal((n, d), dtype=np.float32)]
    if name == "ln":
        n, d = (128, 1024) if small else (8192, 1024)
        return [rng.standard_normal((n, d), dtype=np.float32), np.ones(d, np.float32), np.zeros(d, np.float32)]
    n, d, k = (96, 1024, 256) if small else (8192, 1024, 4096)
    return [rng.standard_normal((n, d), dtype=np.float32), rng.standard_normal((d, k), dtype=np.float32) * np.float32(0.02),
            rng.standard_normal(k, dtype=np.float32)]


def formula(name, args):
    a = [x.astype(np.float64) for x in args]
    if name == "rows":
        e = np.exp(a[0] - a[0].max(axis=1, keepdims=True))
        return e / e.sum(axis=1, keepdims=True)
    if name == "ln":
        mu = a[0].mean(axis=1, keepdims=True)
        var = ((a[0] - mu) ** 2).mean(axis=1, keepdims=True)
        return (a[0] - mu) / np.sqrt(var + 1e-5) * a[1] + a[2]
    return a[0] @ a[1] + a[2]


def close(got, want, rel=1e-4):
    return np.abs(got.astype(np.float64) - want).max() <= rel * np.abs(want).max()


@pytest.mark.parametrize("name", sorted(SOURCES))
def test_reduced_size_matches_reference_interpreter(name):
    f = pyapi.function(SOURCES[name], name=name)
    args = inputs(name, True)
    got = f(*args)
    want = np.load(os.path.join(GOLDEN, f"fn_{name}.npz"))["out0"]
    assert got.shape == want.shape and got.dtype == np.float32
    assert close(got, want.astype(np.float64))
    again = f(*args)                                  # same version, second call
    assert np.array_equal(got, again)
    assert len(f.versions) == 1


@pytest.mark.parametrize("name", sorted(SOURCES))
def test_full_size_matches_float64_formula(name):
    f = pyapi.function(SOURCES[name], name=name)
    args = inputs(name, False)
    before = [a.copy() for a in args]
    got = f(*args)
    assert close(got, formula(name, args))
    assert all(np.array_equal(a, b) for a, b in zip(args, before))      # arguments are never written


def test_device_arrays_are_taken_without_a_host_copy():
    """Arguments that expose `__cuda_array_interface__` (torch tensors here) go device-to-device into the arena;
    the result equals the one computed from the same values passed as NumPy arrays, and mixing both works."""
    import torch
    f = pyapi.function(SOURCES["ln"], name="ln")
    args = inputs("ln", True)
    want = f(*args)
    dev = [torch.from_numpy(a).cuda() for a in args]
    got = f(*dev)
    assert np.array_equal(got, want)
    mixed = f(dev[0], args[1], dev[2])
    assert np.array_equal(mixed, want)
    assert len(f.versions) == 1                                    # same shapes and dtypes: the same compiled version
    assert all(torch.equal(d.cpu(), torch.from_numpy(a)) for d, a in zip(dev, args))     # arguments are never written
    with pytest.raises(TypeError):
        f(dev[0].double(), args[1], args[2])
