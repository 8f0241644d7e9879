"""`anvil.function` on B200: NumPy arrays in, NumPy arrays out, computed on the GPU.

Mirrors anvil/pyapi.py: `function(source, name, seed)` returns a `Function`; calling it with arrays
picks (or compiles) the version for that combination of shapes (:76-81, signature rules :212-234:
floats become f32, integers and bools i32, Python scalars and strings are compile-time constants).
The per-shape lowering itself (`lower`, :114-181) is the reference front end's job and is used
unchanged when the `anvil` package is importable. Where it is not, lowered programs are looked up
in a directory of `.kir.json.gz` files keyed by (source, name, signature, seed) that `save_lowered`
wrote on a machine that has the front end.

`Compiled` replaces anvil/pyapi.py:237-299. The reference links AArch64 assembly into a library
exporting `int anvil_entry(void)` and one `void *anvil_input{k}` / `anvil_output{k}` pointer slot
per used argument; the library built here exports the same symbols with the same meaning (host
pointers; the call copies inputs to the device arena, runs, and copies results back), so the
calling code is the reference's: set slots, call the entry, clear slots, under a lock.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import threading

import numpy as np

from . import kir
from .program import AnvilRuntimeError, DeviceProgram

LOWERED_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "programs", "lowered")


class DeviceArray:
    """A tensor argument that already lives in GPU memory (`__cuda_array_interface__`: torch, CuPy, Numba):
    it is copied device-to-device into the arena, with no trip through the host."""

    def __init__(self, obj):
        cai = obj.__cuda_array_interface__
        self.keep = obj
        self.shape = tuple(int(d) for d in cai["shape"])
        t = np.dtype(cai["typestr"])
        if t == np.float32:
            self.dtype = kir.F32
        elif t == np.int32:
            self.dtype = kir.I32
        else:
            raise TypeError(f"anvil: a device array of {t} cannot be passed without a copy (use float32 or int32)")
        if cai.get("strides") is not None:
            raise TypeError("anvil: a device array argument must be contiguous (row-major)")
        self.ptr = int(cai["data"][0])
        self.nbytes = 4 * int(np.prod(self.shape, dtype=np.int64))
        st = cai.get("stream")
        self.stream = int(st) if isinstance(st, int) and st > 2 else 0      # 1 / 2: the default streams


_TENSOR_KINDS = {"f": (np.float32, kir.F32), "i": (np.int32, kir.I32), "u": (np.int32, kir.I32), "b": (np.int32, kir.I32)}


def _constant_text(v) -> str:
    """How a Python scalar argument is spelled in the function's source: it is a compile-time constant and part
    of the signature (anvil/pyapi.py:216-221)."""
    if v is True or v is False:
        return "true" if v else "false"
    if isinstance(v, str):
        return '"' + v + '"'
    if isinstance(v, float) and v != v:
        return "nan"
    if isinstance(v, float) and v in (float("inf"), float("-inf")):
        return "inf" if v > 0 else "-inf"
    return repr(v)


def _host_tensor(a):
    arr = np.asarray(a)
    try:
        np_type, dtype = _TENSOR_KINDS[arr.dtype.kind]
    except KeyError:
        raise TypeError(f"anvil: cannot pass an array of {arr.dtype} (use floats or integers)") from None
    return np.ascontiguousarray(arr, dtype=np_type), dtype


def arguments(args):
    """Splits a call's arguments into tensors (NumPy arrays converted to f32 / i32, or `DeviceArray`s for objects that
    already live on the GPU) and the signature `(("tensor", shape, dtype) | ("const", text), ...)` that selects the
    compiled version — the same signature the reference computes (anvil/pyapi.py:212-234), so lowered programs
    stored under it are found by either implementation."""
    tensors, sig = [], []
    for a in args:
        if hasattr(a, "__cuda_array_interface__"):
            t = DeviceArray(a)
            shape, dtype = t.shape, t.dtype
        elif isinstance(a, (bool, int, float, str)) and not isinstance(a, np.generic):
            sig.append(("const", _constant_text(a)))
            continue
        else:
            t, dtype = _host_tensor(a)
            shape = tuple(map(int, t.shape))
        tensors.append(t)
        sig.append(("tensor", shape, dtype))
    return tensors, tuple(sig)


def lowered_key(source: str, name: str, sig, seed: int) -> str:
    return hashlib.sha256(repr((source, name, sig, seed)).encode()).hexdigest()[:20]


class Lowered:
    """A function as a program of its own (anvil/pyapi.py:101-111), in KIR."""

    def __init__(self, prog: kir.Program, inputs, outputs, consts, tuple_result):
        self.prog = prog
        self.inputs = inputs          # kir buffers in argument order (tensor arguments only)
        self.outputs = outputs        # kir buffers, None for a compile-time result
        self.consts = consts
        self.tuple_result = tuple_result


def lower(source: str, path: str, name: str | None, sig, seed: int = 0) -> Lowered:
    """Per-shape lowering through the reference front end, else from the shipped directory."""
    try:
        from anvil import pyapi as ref
    except ImportError:
        ref = None
    if ref is not None:
        if name is None:
            name = ref.Function(source, seed=seed).name
        lo = ref.lower(source if source.endswith("\n") else source + "\n", path, name, sig, seed=seed)
        prog = kir.from_anvil(lo.prog, f"fn {name}")
        by_id = {b.id: b for b in prog.buffers}
        ins = [by_id[b.id] for b in lo.inputs]
        outs = [None if b is None else by_id[b.id] for b in lo.outputs]
        return Lowered(prog, ins, outs, list(lo.consts), lo.tuple_result)
    f = os.path.join(LOWERED_DIR, lowered_key(source, name or "", sig, seed) + ".kir.json.gz")
    if not os.path.exists(f):
        raise AnvilRuntimeError("anvil: the Anvil front end is not importable and no lowered program is stored for "
                                f"this source and signature ({f})")
    return load_lowered(f)


def save_lowered(lo: Lowered, path: str):
    import gzip
    import json
    meta = {"inputs": [b.id for b in lo.inputs], "outputs": [None if b is None else b.id for b in lo.outputs],
            "consts": lo.consts, "tuple": lo.tuple_result, "kir": kir.dumps(lo.prog)}
    with gzip.GzipFile(path, "wb", mtime=0) as f:
        f.write(json.dumps(meta).encode())


def load_lowered(path: str) -> Lowered:
    import gzip
    import json
    with gzip.open(path, "rb") as f:
        meta = json.loads(f.read().decode())
    prog = kir.loads(meta["kir"])
    by_id = {b.id: b for b in prog.buffers}
    return Lowered(prog, [by_id[i] for i in meta["inputs"]], [None if i is None else by_id[i] for i in meta["outputs"]],
                   meta["consts"], meta["tuple"])


class Compiled:
    """One version of a Function: a GPU library for one combination of argument shapes."""

    def __init__(self, name, lowered: Lowered, seed: int, device: int = 0):
        self.name = name
        self.lowered = lowered
        self.prog = lowered.prog
        self.inputs = lowered.inputs
        self.outputs = lowered.outputs
        self.consts = lowered.consts
        self.tuple_result = lowered.tuple_result
        self.dp = DeviceProgram(self.prog, seed=seed, device=device, graphs=False)
        self.lib = self.dp.lib
        ctypes.c_void_p.in_dll(self.lib, "anvil_b200_rt").value = self.dp.rt
        self.entry = self.lib.anvil_entry
        self.entry.restype = ctypes.c_int
        self.entry.argtypes = []
        used = {r.id for r in self.prog.roots()}

        def slot(b):
            if b is None or b.root.id not in used:
                return None
            try:
                return ctypes.c_void_p.in_dll(self.lib, f"anvil_{b.name}")
            except ValueError:
                return None
        self.in_slots = [slot(b) for b in self.inputs]
        self.out_slots = [slot(b) for b in self.outputs]
        self.lock = threading.Lock()

    def call(self, arrays):
        results = [None if b is None else np.empty(b.shape, np.float32 if b.dtype == kir.F32 else np.int32)
                   for b in self.outputs]
        with self.lock:
            for s, a, b in zip(self.in_slots, arrays, self.inputs):
                if s is None:
                    continue
                if isinstance(a, DeviceArray):               # already on the GPU: device-to-device, the slot stays empty
                    self.dp._check(self.dp.rtlib.anvil_rt_d2d_async(self.dp.rt, self.dp.plan.off(b), a.ptr, a.nbytes, a.stream))
                else:
                    s.value = a.ctypes.data
            for s, r in zip(self.out_slots, results):
                if s is not None:
                    s.value = r.ctypes.data
            rc = self.entry()
            for s in self.in_slots + self.out_slots:
                if s is not None:
                    s.value = None
        if rc != 0:
            raise AnvilRuntimeError(self.dp.rtlib.anvil_rt_last_error(self.dp.rt).decode("utf-8", "replace"))
        consts = iter(self.consts)
        out = [next(consts) if r is None else (r[()] if r.ndim == 0 else r) for r in results]
        return tuple(out) if self.tuple_result else out[0]

    # device-resident calls: inputs already in the arena, results left there
    def run_resident(self):
        self.dp._check(self.lib.anvil_b200_main(self.dp.rt, 0))


class Function:
    """An Anvil function callable from Python on a B200: the counterpart of the reference's `Function`
    (anvil/pyapi.py:46-94) with `Compiled` swapped for the GPU dispatcher. One `Compiled` per signature is kept."""

    def __init__(self, source: str, name: str | None = None, seed: int = 0, device: int = 0):
        self.path, text = self._resolve(source)
        self.source = text if text.endswith("\n") else text + "\n"
        self.name, self.seed, self.device = name, seed, device
        self.versions: dict[tuple, Compiled] = {}

    @staticmethod
    def _resolve(source: str):
        """(`path` the diagnostics name, program text): `source` is either the text itself or the path of a .anvil file."""
        is_file = "\n" not in source and source.endswith(".anvil") and os.path.exists(source)
        if not is_file:
            return os.path.join(os.getcwd(), "<python>.anvil"), source
        with open(source, encoding="utf-8") as f:
            return os.path.abspath(source), f.read()

    def lower_sig(self, sig) -> Compiled:
        if sig not in self.versions:
            lowered = lower(self.source, self.path, self.name, sig, seed=self.seed)
            self.versions[sig] = Compiled(self.name, lowered, seed=self.seed, device=self.device)
        return self.versions[sig]

    def lower(self, *args) -> Compiled:
        """The compiled version these arguments would run, without running it."""
        _, sig = arguments(args)
        return self.lower_sig(sig)

    def __call__(self, *args):
        tensors, sig = arguments(args)
        return self.lower_sig(sig).call(tensors)


def function(source: str, name: str | None = None, seed: int = 0) -> Function:
    return Function(source, name=name, seed=seed)
