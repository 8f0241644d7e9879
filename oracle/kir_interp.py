"""CPU oracle: a NumPy restatement of the reference interpreter's semantics for the kernel IR.

TEST INFRASTRUCTURE ONLY. Nothing in the shipped package imports this module; it is used by the
tests, by the smoke check and by the benchmark's CPU-baseline leg as the checker / timed baseline.

It follows the reference's NumPy interpreter (anvil/interp.py) function by function:
  rand_bits / lowbias32      anvil/interp.py:55-71    counter hash behind every random number
  format_tensor / fmt_f32    anvil/interp.py:74-115   print formats
  exec_stmt / exec_for       anvil/interp.py:152-211  control flow
  exec_print                 anvil/interp.py:213-239
  exec_rt                    anvil/interp.py:241-380  iota, shuffle, seed, save/load, nonzero, ...
  exec_kernel / run_kernel   anvil/interp.py:383-466  chunking, reduction first, then statements
  reduce                     anvil/interp.py:468-516
  eval / unary / binary      anvil/interp.py:519-632  scalar semantics (f32 arithmetic in NumPy)

Parity is pinned: tests/golden holds outputs of the reference interpreter itself (made by
tests/golden/make_golden.py in a container that has the reference), and the CPU test suite checks
this module against them.

`mode="faithful"` evaluates a reduction the way the reference does (materialise the broadcast body
over domain x reduction, then reduce; chunks of 4 Mi elements). `mode="fast"` additionally sends
sum-of-product bodies to `numpy.einsum` in float64, which gives the same values to ~1e-7 relative;
it exists so that parity checks at larger sizes finish, and is never the timed baseline.
"""
from __future__ import annotations

import io
import struct
import sys
import time

import numpy as np

from anvil_lang_b200 import kir
from anvil_lang_b200.kir import F32, I32

M32 = np.uint64(0xFFFFFFFF)
CHUNK = 1 << 22                       # anvil/interp.py:25
SHUFFLE_SALT = 7                      # anvil/interp.py:24
CKPT_HEAD = struct.Struct("<4sIQ")    # anvil/interp.py:26


class OracleRuntimeError(Exception):
    pass


class ProgramExit(Exception):
    def __init__(self, code):
        super().__init__(f"exit status {code}")
        self.code = code


class _Break(Exception):
    pass


class _Continue(Exception):
    pass


class _EndOfInput(Exception):
    pass


def lowbias32(x):
    """anvil/interp.py:55-62."""
    x = np.asarray(x).astype(np.uint32)
    x = x ^ (x >> np.uint32(16))
    x = ((x.astype(np.uint64) * np.uint64(0x7FEB352D)) & M32).astype(np.uint32)
    x = x ^ (x >> np.uint32(15))
    x = ((x.astype(np.uint64) * np.uint64(0x846CA68B)) & M32).astype(np.uint32)
    x = x ^ (x >> np.uint32(16))
    return x


def rand_bits(idx, stream: int, salt: int, seed: int):
    """32 random bits per element index (anvil/interp.py:68-71; anvil/backend/anvil_host.h:21-24)."""
    k = (stream * 0x85EBCA77 + salt * 0xC2B2AE3D + seed + 0x632BE5AB) & 0xFFFFFFFF
    h0 = (np.asarray(idx, dtype=np.uint64) * np.uint64(0x9E3779B1) + np.uint64(k)) & M32
    return lowbias32(lowbias32(h0))


def shuffle_inplace(p: np.ndarray, n: int, stream: int, seed: int):
    """Fisher-Yates with the draws of anvil/interp.py:309-320."""
    if n > 1:
        h = rand_bits(np.arange(n - 1), stream, SHUFFLE_SALT, seed)
        for k in range(n - 1):
            i = n - 1 - k
            j = int(h[k]) % (i + 1)
            p[i], p[j] = p[j], p[i]


def fmt_f32(v) -> str:
    """anvil/interp.py:74-80."""
    v = float(v)
    a = abs(v)
    if v == 0 or v != v or 1e-4 <= a < 1e6:
        return "%.4f" % v
    return "%.4e" % v


def fmt_elem(v, dtype) -> str:
    return "%d" % int(v) if dtype == I32 else fmt_f32(v)


def format_tensor(flat, shape, dtype) -> str:
    """anvil/interp.py:89-115: nested brackets, more than 1000 elements are summarised 3 ... 3."""
    rank = len(shape)
    if rank == 0:
        return fmt_elem(flat[0], dtype)
    numel = kir.prod(shape)
    if numel == 0:
        return "[]"
    summarize = numel > 1000
    strides = kir.row_major_strides(shape)

    def rec(off, d):
        n = shape[d]
        idxs = [0, 1, 2, None, n - 3, n - 2, n - 1] if (summarize and n > 6) else list(range(n))
        parts = []
        for i in idxs:
            if i is None:
                parts.append("...")
            elif d == rank - 1:
                parts.append(fmt_elem(flat[off + i], dtype))
            else:
                parts.append(rec(off + i * strides[d], d + 1))
        sep = ", " if d == rank - 1 else ",\n" + " " * (d + 1)
        return "[" + sep.join(parts) + "]"
    return rec(0, 0)


class Oracle:
    """Executes a `kir.Program` on NumPy arrays, one flat array per root buffer."""

    def __init__(self, prog: kir.Program, out=None, seed: int = 0, inp=None, mode: str = "faithful",
                 float_dtype=np.float32):
        self.prog = prog
        self.out = out if out is not None else sys.stdout
        self.inp = inp if inp is not None else io.StringIO("")
        self.mode = mode
        self.fdt = float_dtype
        self.mem: dict[int, np.ndarray] = {}
        for b in prog.buffers:                       # anvil/interp.py:127-135
            r = b.root
            if r.id in self.mem:
                continue
            arr = np.zeros(max(r.numel, 1), dtype=np.int32 if r.dtype == I32 else self.fdt)
            if r.init is not None:
                arr[:len(r.init)] = r.init
            self.mem[r.id] = arr
        self.seed = seed & 0xFFFFFFFF
        self.stream = 0
        self.t0 = time.perf_counter()
        self.kernel_count = 0
        self.on_kernel = None                        # hook(kernel) called after each kernel
        self.allreduce = None                        # hook(list of arrays): sum over ranks, in place

    def arr(self, b: kir.Buffer) -> np.ndarray:
        return self.mem[b.root.id]

    def rand_base(self, k: kir.Kernel) -> int:
        if k.rand_base is None:
            return 0
        b, coef = k.rand_base
        return coef * int(self.arr(b)[0])

    def tensor(self, b: kir.Buffer) -> np.ndarray:
        return self.arr(b)[:b.numel].reshape(b.shape)

    def run(self):
        try:
            self.block(self.prog.main)
        except _EndOfInput:
            pass
        if hasattr(self.out, "flush"):
            self.out.flush()
        return self

    # ------------------------------------------------------------------ statements
    def block(self, b: kir.Block):
        for st in b.stmts:
            self.stmt(st)

    def bound(self, x) -> int:
        return x if isinstance(x, int) else int(self.arr(x)[0])

    def stmt(self, st):
        if isinstance(st, kir.KernelStmt):
            self.kernel(st.kernel)
        elif isinstance(st, kir.For):                # anvil/interp.py:199-211
            c = self.arr(st.counter)
            c[0] = self.bound(st.start)
            stop = self.bound(st.stop)
            while c[0] < stop:
                try:
                    self.block(st.body)
                except _Break:
                    break
                except _Continue:
                    pass
                c[0] += st.step
        elif isinstance(st, kir.While):
            while True:
                self.block(st.cond_block)
                if self.arr(st.cond)[0] == 0:
                    break
                try:
                    self.block(st.body)
                except _Break:
                    break
                except _Continue:
                    continue
        elif isinstance(st, kir.If):
            self.block(st.then if self.arr(st.cond)[0] != 0 else st.orelse)
        elif isinstance(st, kir.AllReduce):
            if self.allreduce is None:
                raise OracleRuntimeError("the program has an all-reduce but no collective was given")
            self.allreduce([self.arr(b) for b in st.bufs])
        elif isinstance(st, kir.Break):
            raise _Break()
        elif isinstance(st, kir.Continue):
            raise _Continue()
        elif isinstance(st, kir.Print):
            self.print_(st)
        elif isinstance(st, kir.Check):
            v = int(np.asarray(self.affine(st.value, {}, None)).reshape(-1)[0])
            if not st.lo <= v <= st.hi:
                raise OracleRuntimeError(f"{st.message} (value {v})")
        elif isinstance(st, kir.RTCall):
            self.rtcall(st)
        else:
            raise NotImplementedError(type(st).__name__)

    def print_(self, st: kir.Print):
        parts = []
        for it in st.items:
            if it.kind == "text":
                parts.append(it.text)
            elif it.kind == "scalar":
                v = self.arr(it.buf)[0]
                if not it.fmt:
                    parts.append(fmt_elem(v, it.buf.dtype))
                elif it.buf.dtype == I32 or it.fmt.endswith("d"):
                    parts.append(it.fmt % int(v))
                else:
                    parts.append(it.fmt % float(v))
            elif it.kind == "chars":
                codes = self.arr(it.buf)[:it.buf.numel].astype(np.int64) & 0xFF
                parts.append(codes.astype(np.uint8).tobytes().decode("utf-8", errors="replace"))
            elif it.kind == "pick":
                k = int(self.arr(it.buf)[0])
                parts.append(it.choices[k] if 0 <= k < len(it.choices) else "?")
            else:
                b = it.buf
                parts.append(format_tensor(self.arr(b)[:b.numel], b.shape, b.dtype))
        text = "".join(parts) + st.end
        if st.err:
            sys.stderr.write(text)
        else:
            self.out.write(text)

    @staticmethod
    def data_path(path: str) -> str:
        """ANVIL_DATA, when set, replaces the directory of a data file (anvil/backend/anvil_host.h:134-141)."""
        import os
        d = os.environ.get("ANVIL_DATA")
        return os.path.join(d, os.path.basename(path)) if d else path

    def rtcall(self, st: kir.RTCall):
        a, n = st.args, st.name
        if n in ("load_idx", "load_bytes", "load_csv"):
            a = dict(a, path=self.data_path(a["path"]))
        if n == "seed":
            self.seed = a["value"] & 0xFFFFFFFF
            self.stream = 0
        elif n == "skip_rand":
            self.stream += 1
        elif n in ("iota", "iota_once"):
            b = a["buf"]
            self.arr(b)[:b.numel] = np.arange(b.numel, dtype=np.int32)
        elif n == "shuffle":
            b = a["buf"]
            stream = self.stream
            self.stream += 1
            shuffle_inplace(self.arr(b), b.numel, stream, self.seed)
        elif n == "clock":
            self.arr(a["buf"])[0] = time.perf_counter() - self.t0
        elif n == "exit":
            raise ProgramExit(a["value"])
        elif n == "nonzero":
            src, b = a["src"], a["buf"]
            idx = np.flatnonzero(self.arr(src)[:src.numel])[:b.numel]
            out = self.arr(b)
            out[:b.numel] = -1
            out[:len(idx)] = idx
        elif n == "show":
            g = a["glyphs"]
            data = self.arr(a["buf"])
            for r in range(a["rows"]):
                row = data[r * a["cols"]:(r + 1) * a["cols"]]
                self.out.write("".join(g[v] if 0 <= v < len(g) else "?" for v in row) + "\n")
        elif n == "sleep":
            time.sleep(max(0.0, float(self.arr(a["buf"])[0])))
        elif n == "input":
            import re
            line = self.inp.readline()
            if not line:
                self.out.write("\n")
                raise _EndOfInput()
            m = re.search(r"[-+]?(?:\d+(?:\.\d*)?|\.\d+)(?:[eE][-+]?\d+)?", line)
            self.arr(a["buf"])[0] = float(m.group(0)) if m else np.nan
        elif n == "save":                            # anvil/interp.py:341-350
            bufs = a["bufs"]
            try:
                with open(a["path"], "wb") as f:
                    f.write(CKPT_HEAD.pack(b"EINW", 2, len(bufs)))
                    f.write(struct.pack(f"<{len(bufs)}Q", *[b.root.ckpt_key for b in bufs]))
                    for b in bufs:
                        f.write(self.arr(b)[:b.numel].astype(np.int32 if b.dtype == I32 else np.float32).tobytes())
            except OSError:
                sys.stderr.write(f"anvil: cannot write {a['path']}\n")
        elif n == "load":                            # anvil/interp.py:351-372
            bufs = a["bufs"]
            ok = 0.0
            try:
                with open(a["path"], "rb") as f:
                    raw = f.read()
                sizes = [b.numel for b in bufs]
                head = CKPT_HEAD.size + 8 * len(bufs)
                magic, version, cnt = CKPT_HEAD.unpack_from(raw) if len(raw) >= CKPT_HEAD.size else (None, 0, 0)
                want = [b.root.ckpt_key for b in bufs] if version == 2 else sizes
                if len(raw) == head + 4 * sum(sizes) and magic == b"EINW" and version in (1, 2) and cnt == len(bufs) \
                        and list(struct.unpack_from(f"<{len(bufs)}Q", raw, CKPT_HEAD.size)) == want:
                    pos = head
                    for b in bufs:
                        self.arr(b)[:b.numel] = np.frombuffer(raw, np.int32 if b.dtype == I32 else np.float32,
                                                              b.numel, pos)
                        pos += 4 * b.numel
                    ok = 1.0
            except OSError:
                pass
            self.arr(a["buf"])[0] = ok
        elif n == "save_npy":
            b = a["buf"]
            with open(a["path"], "wb") as f:
                f.write(bytes(a["header"]))
                f.write(self.arr(b)[:b.numel].astype(np.int32 if b.dtype == I32 else np.float32).tobytes())
        elif n == "load_idx":                               # anvil/interp.py:243-251
            import gzip
            b = a["buf"]
            with open(a["path"], "rb") as f:
                magic = f.read(2)
            opener = gzip.open if magic == b"\x1f\x8b" else open
            with opener(a["path"], "rb") as f:
                f.read(a["header"])
                raw = np.frombuffer(f.read(b.numel), dtype=np.uint8)
            if raw.size != b.numel:
                raise OracleRuntimeError(f"data file {a['path']} does not have the shape this program was compiled for")
            self.arr(b)[:b.numel] = raw.astype(self.arr(b).dtype)
        elif n == "load_bytes":                             # anvil/interp.py:257-267
            b = a["buf"]
            try:
                raw = open(a["path"], "rb").read()
            except OSError:
                raise OracleRuntimeError(f"cannot open data file {a['path']}")
            if len(raw) != b.numel:
                raise OracleRuntimeError(f"data file {a['path']} does not have the shape this program was compiled for")
            self.arr(b)[:b.numel] = np.frombuffer(raw, dtype=np.uint8)
        elif n == "load_csv":                               # anvil/interp.py:289-305
            import re
            b = a["buf"]
            try:
                text = open(a["path"], encoding="utf-8", errors="replace").read()
            except OSError:
                raise OracleRuntimeError(f"cannot open data file {a['path']}")
            pos = 0
            for _ in range(a["skip"]):
                pos = text.index("\n", pos) + 1
            vals = re.findall(r"[+-]?(?:\d+\.?\d*|\.\d+)(?:[eE][+-]?\d+)?", text[pos:])
            if len(vals) < b.numel:
                raise OracleRuntimeError(f"data file {a['path']} does not have the shape this program was compiled for")
            self.arr(b)[:b.numel] = np.array([float(v) for v in vals[:b.numel]], dtype=np.float32)
        elif n == "load_npy" and not (a["kind"] & 16):
            b = a["buf"]
            data = np.load(a["path"], allow_pickle=False)
            if data.size != b.numel:
                raise OracleRuntimeError(f"data file {a['path']} does not have the shape this program was compiled for")
            self.arr(b)[:b.numel] = data.reshape(-1).astype(self.arr(b).dtype)
        else:
            raise NotImplementedError(f"runtime call {n}")

    # ------------------------------------------------------------------ kernels
    def kernel(self, k: kir.Kernel):
        """anvil/interp.py:383-406: a rand-using kernel takes the next stream number; kernels whose
        domain x reduction exceeds CHUNK are run in slices of the first domain var."""
        self.kernel_count += 1
        stream = None
        if k.uses_rand():
            stream = self.stream
            self.stream += 1
        D = list(k.domain)
        R = list(k.red.vars) if k.red else []
        total = kir.prod(v.extent for v in D + R)
        if total == 0:
            return
        if self.mode == "fast" and k.red is not None and k.red.op == "sum" and self._contraction(k, D, R, stream):
            pass
        elif total <= CHUNK or (not D and not R):
            self.run_kernel(k, D, R, None, stream)
        elif D:
            v0 = D[0]
            per = max(1, CHUNK // max(1, total // v0.extent))
            for s in range(0, v0.extent, per):
                self.run_kernel(k, D, R, (v0, s, min(v0.extent, s + per)), stream)
        else:
            self.run_kernel(k, D, R, None, stream, chunk_red=True)
        if self.on_kernel is not None:
            self.on_kernel(k)

    @staticmethod
    def grid(vars_, ranges):
        env, n = {}, len(vars_)
        for ax, v in enumerate(vars_):
            lo, hi = ranges.get(v, (0, v.extent))
            shape = [1] * n
            shape[ax] = hi - lo
            env[v] = np.arange(lo, hi, dtype=np.int64).reshape(shape)
        return env

    def run_kernel(self, k, D, R, chunk, stream, chunk_red=False, acc=None):
        """anvil/interp.py:435-466: the reduction over the whole (chunk of the) domain first, reading
        memory as it was before the kernel; then each statement over the domain, storing before the
        next statement is evaluated."""
        ranges = {}
        if chunk is not None:
            v0, lo, hi = chunk
            ranges[v0] = (lo, hi)
        allv = D + R
        env = self.grid(allv, ranges)
        dshape = tuple(ranges.get(v, (0, v.extent))[1] - ranges.get(v, (0, v.extent))[0] for v in D)
        fullshape = dshape + tuple(v.extent for v in R)
        if k.red is not None and acc is None:
            if chunk_red and R:
                acc = self.reduce_chunked(k, D, R, stream)
            else:
                ctx = {"env": env, "ndim": len(allv), "stream": stream, "rand_base": self.rand_base(k), "D": D, "lets": {}, "memo": {}}
                body = np.broadcast_to(self.eval(k.red.body, ctx), fullshape)
                acc = self.reduce(k.red.op, body, len(D))
        denv = {v: env[v].reshape(env[v].shape[:len(D)]) for v in D}
        sctx = {"env": denv, "ndim": len(D), "stream": stream, "rand_base": self.rand_base(k), "D": D, "lets": {}, "acc": acc, "memo": {}}
        for st in k.stmts:
            if isinstance(st, kir.Let):
                sctx["lets"][st.id] = self.eval(st.value, sctx)
                continue
            val = np.broadcast_to(self.eval(st.value, sctx), dshape)
            off = np.broadcast_to(self.affine(st.offset, denv, sctx), dshape)
            a = self.arr(st.buf)
            val = val.astype(a.dtype, copy=False)
            if st.accumulate:
                np.add.at(a, off.reshape(-1), val.reshape(-1))
            else:
                a[off.reshape(-1)] = val.reshape(-1)
            sctx["memo"] = {}                        # loads after a store read memory again

    @staticmethod
    def reduce(op, body, nd):
        """anvil/interp.py:468-482."""
        axes = tuple(range(nd, body.ndim))
        if op == "sum":
            return body.sum(axis=axes, dtype=body.dtype)
        if op == "max":
            return body.max(axis=axes)
        if op == "min":
            return body.min(axis=axes)
        if op == "prod":
            return body.prod(axis=axes, dtype=body.dtype)
        flat = body.reshape(body.shape[:nd] + (-1,))
        r = flat.argmax(axis=-1) if op == "argmax" else flat.argmin(axis=-1)
        return r.astype(np.int32)

    def reduce_chunked(self, k, D, R, stream):
        """anvil/interp.py:484-516: no domain to slice, so the first reduction var is sliced and the
        partial results are combined in order."""
        r0 = R[0]
        per = max(1, CHUNK // max(1, kir.prod(v.extent for v in R) // r0.extent))
        op = k.red.op
        acc = best = None
        for s in range(0, r0.extent, per):
            e = min(r0.extent, s + per)
            env2 = self.grid(D + R, {r0: (s, e)})
            shape2 = tuple(v.extent for v in D) + tuple((e - s) if v is r0 else v.extent for v in R)
            ctx = {"env": env2, "ndim": len(D + R), "stream": stream, "rand_base": self.rand_base(k), "D": D, "lets": {}, "memo": {}}
            body = np.broadcast_to(self.eval(k.red.body, ctx), shape2)
            if op in ("argmax", "argmin"):
                part = self.reduce("max" if op == "argmax" else "min", body, len(D))
                rest = kir.prod(v.extent for v in R[1:])
                pidx = self.reduce(op, body, len(D)) + s * rest
                if acc is None:
                    acc, best = part, pidx
                else:
                    better = part > acc if op == "argmax" else part < acc
                    acc = np.where(better, part, acc)
                    best = np.where(better, pidx, best)
                continue
            part = self.reduce(op, body, len(D))
            if acc is None:
                acc = part
            elif op == "sum":
                acc = acc + part
            elif op == "max":
                acc = np.maximum(acc, part)
            elif op == "min":
                acc = np.minimum(acc, part)
            else:
                acc = acc * part
        return best.astype(np.int32) if op in ("argmax", "argmin") else acc

    # ---- fast mode: sum of products through einsum (not the reference's method; see module docstring)
    def _contraction(self, k, D, R, stream) -> bool:
        factors = []

        def split(e):
            if e.k == "bin" and e.op == "mul" and e.dt == F32:
                split(e.a[0])
                split(e.a[1])
            else:
                factors.append(e)
        split(k.red.body)
        if len(factors) < 2 or kir.prod(v.extent for v in D + R) <= (1 << 16):
            return False
        if any(n.k == "rand" for f in factors for n in f.walk()):
            return False
        allv = D + R
        env = self.grid(allv, {})
        letters = "abcdefghijklmnopqrstuvwxyz"
        if len(allv) > len(letters):
            return False
        ops, subs = [], []
        for f in factors:
            ctx = {"env": env, "ndim": len(allv), "stream": stream, "rand_base": self.rand_base(k), "D": D, "lets": {}, "memo": {}}
            val = np.asarray(self.eval(f, ctx))
            if val.ndim == 0:
                val = val.reshape((1,) * len(allv))
            val = np.broadcast_to(val, np.broadcast_shapes(val.shape, (1,) * len(allv)))
            axes = [i for i in range(len(allv)) if val.shape[i] > 1]
            ops.append(val.reshape([val.shape[i] for i in axes]).astype(np.float64))
            subs.append("".join(letters[i] for i in axes))
        outsub = "".join(letters[i] for i in range(len(D)))
        used = set("".join(subs))
        scale = 1.0
        for i, v in enumerate(allv):                 # an index no factor depends on multiplies the sum
            if letters[i] not in used:
                if i < len(D):
                    outsub = outsub.replace(letters[i], "")
                else:
                    scale *= v.extent
        acc = np.einsum(",".join(subs) + "->" + outsub, *ops, optimize=True) * scale
        full = [letters[i] in outsub for i in range(len(D))]
        shape = [v.extent if full[i] else 1 for i, v in enumerate(D)]
        acc = np.broadcast_to(acc.reshape(shape), [v.extent for v in D]).astype(self.fdt)
        self.run_kernel(k, D, R, None, stream, acc=acc)
        return True

    # ------------------------------------------------------------------ expressions
    def affine(self, a: kir.Affine, env, ctx):
        """anvil/interp.py:519-534."""
        v = np.int64(a.const)
        for t, c in a.terms:
            if isinstance(t, kir.Var):
                v = v + c * env[t]
            elif isinstance(t, kir.SRef):
                v = v + c * np.int64(self.arr(t.buf)[0])
            else:
                off = self.affine(t.offset, env, ctx)
                g = self.arr(t.buf)[off].astype(np.int64)
                bad = (g < t.lo) | (g >= t.hi)
                if np.any(bad):
                    first = int(np.asarray(g)[bad].reshape(-1)[0])
                    raise OracleRuntimeError(f"index {first} out of bounds for a dimension of size {t.bound} "
                                             f"({t.where})")
                v = v + c * g
        return v

    def eval(self, e: kir.E, ctx):
        memo = ctx["memo"]
        hit = memo.get(id(e))
        if hit is not None:
            return hit
        r = self._eval(e, ctx)
        memo[id(e)] = r
        return r

    def _eval(self, e, ctx):
        fdt = self.fdt
        k = e.k
        if k == "const":
            return np.asarray(e.val, dtype=np.int32 if e.dt == I32 else fdt)
        if k == "load":
            idx = self.affine(e.off, ctx["env"], ctx)
            if any(c < 0 for t, c in e.off.terms if isinstance(t, kir.Var)):
                # A load under a range guard (`x[y - u] if 0 <= y - u < n else 0`, which the back end's implicit
                # convolution rewrite makes): NumPy evaluates both branches, so the index is clamped; the guard
                # discards the value. The reference's own IR never has a negative stride.
                idx = np.clip(idx, 0, self.arr(e.buf).size - 1)
            return self.arr(e.buf)[idx]
        if k == "index":
            return np.asarray(self.affine(e.off, ctx["env"], ctx), dtype=np.int32)
        if k == "acc":
            return ctx["acc"]
        if k == "let":
            return ctx["lets"][e.let.id]
        if k == "rand":                              # anvil/interp.py:549-559
            D = ctx["D"]
            idx = np.int64(ctx.get("rand_base", 0))
            for v, s in zip(D, kir.row_major_strides([v.extent for v in D])):
                g = ctx["env"][v]
                idx = idx + g.reshape(g.shape[:len(D)] + (1,) * (ctx["ndim"] - len(D))) * s
            bits = rand_bits(idx, ctx["stream"], e.salt, self.seed)
            hi = (bits >> np.uint32(8)).astype(np.float64)
            if e.open_low:
                hi = hi + 1.0
            return (hi * (2.0 ** -24)).astype(fdt)
        if k == "un":
            return self.unary(e.op, self.eval(e.a[0], ctx))
        if k == "bin":
            return self.binary(e.op, self.eval(e.a[0], ctx), self.eval(e.a[1], ctx), e.dt == I32)
        if k == "sel":
            c, a, b = (self.eval(x, ctx) for x in e.a)
            return np.where(c != 0, a, b).astype(np.int32 if e.dt == I32 else fdt)
        raise NotImplementedError(k)

    def unary(self, op, a):
        """anvil/interp.py:575-597."""
        fdt = self.fdt
        with np.errstate(all="ignore"):
            if op == "neg": return -a
            if op == "abs": return np.abs(a)
            if op == "exp": return np.exp(a.astype(fdt))
            if op == "log": return np.log(a.astype(fdt))
            if op == "sqrt": return np.sqrt(a.astype(fdt))
            if op == "rsqrt": return (1 / np.sqrt(a.astype(fdt))).astype(fdt)
            if op == "recip": return (1 / a.astype(fdt)).astype(fdt)
            if op == "tanh": return np.tanh(a.astype(fdt))
            if op == "sigmoid": return (1 / (1 + np.exp(-a.astype(fdt)))).astype(fdt)
            if op == "sin": return np.sin(a.astype(fdt))
            if op == "cos": return np.cos(a.astype(fdt))
            if op == "floor": return np.floor(a)
            if op == "ceil": return np.ceil(a)
            if op == "round": return np.round(a)
            if op == "sign": return np.sign(a).astype(a.dtype)
            if op == "not": return (a == 0).astype(fdt)
            if op == "f32": return a.astype(fdt)
            if op == "i32": return np.trunc(a).astype(np.int32) if a.dtype != np.int32 else a
            if op == "detach": return a
        raise NotImplementedError(op)

    def binary(self, op, a, b, isint):
        """anvil/interp.py:599-632: Python floor division / modulo, a zero integer divisor counts as 1,
        nan-propagating max/min, comparisons give 0.0 / 1.0."""
        fdt = self.fdt
        with np.errstate(all="ignore"):
            if op == "add": r = a + b
            elif op == "sub": r = a - b
            elif op == "mul": r = a * b
            elif op == "div": r = a.astype(fdt) / b.astype(fdt)
            elif op == "idiv":
                r = np.floor_divide(a, np.where(b == 0, 1, b)) if isint else np.floor(a / b)
            elif op == "mod":
                r = np.mod(a, np.where(b == 0, 1, b)) if isint else np.mod(a, b)
            elif op == "max": r = np.maximum(a, b)
            elif op == "min": r = np.minimum(a, b)
            elif op == "pow": r = np.power(a.astype(fdt), b.astype(fdt))
            elif op == "lt": r = a < b
            elif op == "le": r = a <= b
            elif op == "gt": r = a > b
            elif op == "ge": r = a >= b
            elif op == "eq": r = a == b
            elif op == "ne": r = a != b
            elif op == "and": r = (a != 0) & (b != 0)
            elif op == "or": r = (a != 0) | (b != 0)
            else:
                raise NotImplementedError(op)
        return np.asarray(r).astype(np.int32 if isint else fdt)


def run_to_string(prog: kir.Program, seed: int = 0, mode: str = "faithful", inp: str = "") -> str:
    buf = io.StringIO()
    Oracle(prog, out=buf, seed=seed, mode=mode, inp=io.StringIO(inp)).run()
    return buf.getvalue()
