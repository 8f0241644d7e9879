"""Feeding a training loop from host memory.

A compiled program produces each step's inputs on the device (a batch gathered out of resident data
through the shuffled permutation, or tokens sampled by the program's random generator). A caller
whose data lives in host memory does the same work in NumPy, copies the result into the buffers
those kernels would have written (pinned memory, asynchronous copy on the program's stream) and
runs `DeviceProgram.step_fed()`, which skips them. The host-side arithmetic reproduces the device
kernels exactly (same permutation, same random numbers), so both ways train on identical batches.
"""
from __future__ import annotations

import ctypes

import numpy as np

from . import hostrng, kir
from .backend.analysis import hot_loop, input_producers


class Unsupported(Exception):
    pass


def pinned_array(rtlib, shape, dtype) -> np.ndarray:
    n = int(np.prod(shape)) * np.dtype(dtype).itemsize
    p = rtlib.anvil_rt_host_alloc(max(n, 16))
    if not p:
        raise MemoryError("anvil: could not allocate pinned host memory")
    buf = (ctypes.c_char * max(n, 16)).from_address(p)
    a = np.frombuffer(buf, dtype=dtype, count=int(np.prod(shape))).reshape(shape)
    a.flags.writeable = True
    return a


class HostFeeder:
    """Prepares the inputs of training step `i` on the host and copies them to the device."""

    def __init__(self, dp, rank: int = 0):
        self.dp = dp
        self.rank = rank
        self.hot = hot_loop(dp.prog)
        self.kernels, self.bufs = input_producers(dp.prog, self.hot)
        if not self.kernels:
            raise Unsupported("the training loop has no input-producing kernels")
        self.plans = [self._plan(k) for k in self.kernels]
        self.pinned = [pinned_array(dp.rtlib, p["shape"], p["dtype"]) for p in self.plans]
        self.bytes_per_step = sum(a.nbytes for a in self.pinned)
        self.rand_streams = sum(1 for k in self.kernels if k.uses_rand())

    def _plan(self, k: kir.Kernel) -> dict:
        if len(k.stores) != 1:
            raise Unsupported(f"{k.name}: several stores")
        st = k.stores[0]
        shape = tuple(v.extent for v in k.domain)
        dtype = np.int32 if st.buf.dtype == kir.I32 else np.float32
        if st.offset.bounds() != (0, kir.prod(shape) - 1) or st.buf.numel != kir.prod(shape):
            raise Unsupported(f"{k.name}: the store does not cover its buffer")
        e = st.value
        # tokens: i32(floor(C * rand0))
        if e.k == "un" and e.op == "i32" and e.a[0].k == "un" and e.a[0].op == "floor":
            m = e.a[0].a[0]
            if m.k == "bin" and m.op == "mul" and m.a[0].k == "const" and m.a[1].k == "rand" \
                    and m.a[1].salt == 0 and not m.a[1].open_low:
                base = k.rand_base[1] * self.rank if k.rand_base is not None else 0
                return {"mode": "randint", "hi": int(m.a[0].val), "shape": shape, "dtype": dtype, "buf": st.buf,
                        "base": base}
        # batch rows: data[perm[B * counter + i], j...]
        if e.k == "load":
            gs = e.off.gathers()
            if len(gs) == 1 and not e.off.scalars():
                g, row = gs[0]
                rank_buf = getattr(self.dp.prog, "rank_buf", None)
                all_srefs = g.offset.scalars()
                rank_terms = [(t, c) for t, c in all_srefs if rank_buf is not None and t.buf.root is rank_buf.root]
                srefs = [(t, c) for t, c in all_srefs if (t, c) not in rank_terms]
                rank_mult = rank_terms[0][1] if rank_terms else 0
                if len(srefs) == 1 and len(g.offset.var_terms()) == 1 and g.offset.var_terms()[0][0] is k.domain[0]:
                    rest = kir.Affine(e.off.const, e.off.var_terms())
                    lo_hi = rest.bounds()
                    inner = kir.prod(shape[1:])
                    if lo_hi == (0, inner - 1) and row == inner or (inner == 1 and row == 1):
                        return {"mode": "rows", "data": e.buf, "perm": g.buf, "counter": srefs[0][0].buf,
                                "mult": srefs[0][1], "const": g.offset.const + rank_mult * self.rank, "row": row,
                                "shape": shape, "dtype": dtype, "buf": st.buf}
        raise Unsupported(f"{k.name}: not a batch gather or a token sampler")

    def load_host_copies(self):
        """Reads the resident dataset and the current permutation once (after `prologue()`)."""
        for p in self.plans:
            if p["mode"] == "rows":
                p["host_data"] = self.dp.read(p["data"]).reshape(-1, p["row"]).copy()
                p["host_perm"] = self.dp.read(p["perm"]).reshape(-1).copy()

    def prepare(self, step: int, stream: int, seed: int):
        """Fills the pinned buffers with the inputs of loop iteration `step`; `stream` is the random
        stream number the first sampling kernel of that iteration would take."""
        s = stream
        for p, out in zip(self.plans, self.pinned):
            if p["mode"] == "randint":
                out[...] = hostrng.randint(p["shape"], 0, p["hi"], s, seed, base=p["base"])
                s += 1
            else:
                B = p["shape"][0]
                rows = p["host_perm"][p["mult"] * step + p["const"] + np.arange(B)]
                np.take(p["host_data"], rows, axis=0, out=out.reshape(B, -1))

    def push(self):
        for p, a in zip(self.plans, self.pinned):
            self.dp.copy_in_async(p["buf"], a.ctypes.data, a.nbytes)

    def close(self):
        for a in self.pinned:
            self.dp.rtlib.anvil_rt_host_free(a.ctypes.data)
        self.pinned = []
