"""Kernel IR consumed by the B200 back end ("KIR").

This is the back end's input contract: a plain-data restatement of Anvil's optimized kernel IR
(reference anvil/ir.py:62-98 buffers, :179-302 affine offsets, :387-511 scalar expressions,
:569-643 kernels, :647-737 program statements). A kernel is

    for d in domain:  acc = REDUCE_{r in red.vars} red.body ;  let ... ; store buf[offset] (=|+=) value

and every memory access is `buffer + affine offset` in elements, where an affine offset is
`c0 + sum ci*var_i + sum dj*scalar_j + sum ek*gather_k`.

Two ways in:
  * `from_anvil(prog)` converts a live `anvil.ir.Program` object (duck-typed: nothing from the
    Anvil package is imported here), and
  * `load(path)` / `loads(text)` read the JSON form that `dump`/`dumps` write, so that a program
    lowered on a machine with the Anvil front end can run on one without it.

The JSON keeps each kernel's expressions as a node table (children by index), so shared
subexpressions stay shared.
"""
from __future__ import annotations

import base64
import gzip
import json
from dataclasses import dataclass, field

import numpy as np

F32 = "f32"
I32 = "i32"

UNARY_OPS = ("neg", "abs", "exp", "log", "sqrt", "tanh", "sigmoid", "sin", "cos", "floor", "ceil",
             "round", "sign", "not", "f32", "i32", "detach", "rsqrt", "recip")
BINARY_OPS = ("add", "sub", "mul", "div", "max", "min", "pow", "idiv", "mod",
              "lt", "le", "gt", "ge", "eq", "ne", "and", "or")
COMPARISONS = ("lt", "le", "gt", "ge", "eq", "ne")
RED_OPS = ("sum", "max", "min", "prod", "argmax", "argmin")


def prod(xs) -> int:
    p = 1
    for x in xs:
        p *= int(x)
    return p


def row_major_strides(shape) -> list[int]:
    out, s = [], 1
    for d in reversed(list(shape)):
        out.append(s)
        s *= int(d)
    return out[::-1]


# ----------------------------------------------------------------------------- data model

@dataclass(eq=False)
class Buffer:
    """A statically shaped array. `kind` is one of param|state|data|temp|var|const|grad|scalar|
    input|output (reference anvil/ir.py:62-64). Aliases share `root`'s storage."""
    id: int
    name: str
    shape: tuple
    dtype: str = F32
    kind: str = "temp"
    init: np.ndarray | None = None      # initial contents of a const buffer (root only)
    ckpt_key: int = 0                   # what a checkpoint stores for it (reference anvil/ir.py:753-764)
    root: "Buffer" = None               # type: ignore[assignment]

    def __post_init__(self):
        self.shape = tuple(int(d) for d in self.shape)
        if self.root is None:
            self.root = self

    @property
    def numel(self) -> int:
        return prod(self.shape)

    @property
    def nbytes(self) -> int:
        return 4 * self.numel

    def __repr__(self):
        return f"{self.name}#{self.id}"


@dataclass(eq=False)
class Var:
    """A loop variable with a static extent."""
    id: int
    name: str
    extent: int

    def __repr__(self):
        return f"{self.name}<{self.extent}"


@dataclass(eq=False)
class SRef:
    """The run-time value of an i32 0-d buffer used inside an index (reference anvil/ir.py:120-136)."""
    buf: Buffer

    def key(self):
        return ("s", self.buf.root.id)


@dataclass(eq=False)
class Gather:
    """A data-dependent index: the i32 loaded from `buf[offset]`, which must satisfy lo <= v < hi
    (reference anvil/ir.py:139-170; lo/hi are `check_range()` evaluated at conversion time)."""
    buf: Buffer
    offset: "Affine"
    bound: int
    where: str
    lo: int
    hi: int

    def key(self):
        return ("g", self.buf.root.id, self.offset.key(), self.bound, self.lo, self.hi)


class Affine:
    """Immutable affine integer expression: const + sum coef*term, term in Var | SRef | Gather."""
    __slots__ = ("const", "terms")

    def __init__(self, const: int = 0, terms=()):
        self.const = int(const)
        self.terms = tuple((t, int(c)) for t, c in terms if c != 0)

    def key(self):
        ks = []
        for t, c in self.terms:
            ks.append((("v", t.id) if isinstance(t, Var) else t.key(), c))
        return (self.const, tuple(sorted(ks, key=repr)))

    def __eq__(self, o):
        return isinstance(o, Affine) and self.key() == o.key()

    def __hash__(self):
        return hash(self.key())

    def coef(self, v: Var) -> int:
        for t, c in self.terms:
            if t is v:
                return c
        return 0

    def var_terms(self):
        return [(t, c) for t, c in self.terms if isinstance(t, Var)]

    def scalars(self):
        return [(t, c) for t, c in self.terms if isinstance(t, SRef)]

    def gathers(self):
        return [(t, c) for t, c in self.terms if isinstance(t, Gather)]

    def vars(self) -> list[Var]:
        """Loop vars this offset depends on, including through gathered indices."""
        out = []
        for t, _ in self.terms:
            if isinstance(t, Var):
                if t not in out:
                    out.append(t)
            elif isinstance(t, Gather):
                for v in t.offset.vars():
                    if v not in out:
                        out.append(v)
        return out

    def is_plain(self) -> bool:
        """Only loop vars and a constant."""
        return all(isinstance(t, Var) for t, _ in self.terms)

    def bounds(self):
        """(min, max) over the var extents when the offset has no run-time terms, else None."""
        lo = hi = self.const
        for t, c in self.terms:
            if not isinstance(t, Var):
                return None
            span = c * (t.extent - 1)
            if span >= 0:
                hi += span
            else:
                lo += span
        return lo, hi

    def __repr__(self):
        parts = [str(self.const)] if self.const or not self.terms else []
        for t, c in self.terms:
            n = t.name if isinstance(t, Var) else (t.buf.name if isinstance(t, SRef) else f"{t.buf.name}[{t.offset!r}]")
            parts.append(n if c == 1 else f"{c}*{n}")
        return " + ".join(parts)


class E:
    """One scalar-expression node. `k` is the node kind:
    const(val) | load(buf, off) | index(off) | un(op, a0) | bin(op, a0, a1) | sel(a0=c, a1, a2) |
    acc | let(let) | rand(salt, open_low).   (reference anvil/ir.py:387-511)"""
    __slots__ = ("k", "dt", "op", "a", "val", "buf", "off", "let", "salt", "open_low", "_key")

    def __init__(self, k, dt, op=None, a=(), val=None, buf=None, off=None, let=None, salt=0, open_low=False):
        self.k, self.dt, self.op, self.a = k, dt, op, tuple(a)
        self.val, self.buf, self.off, self.let = val, buf, off, let
        self.salt, self.open_low = salt, open_low
        self._key = None

    def key(self):
        if self._key is None:
            k = self.k
            if k == "const":
                r = ("c", self.dt, repr(self.val))
            elif k == "load":
                r = ("ld", self.buf.root.id, self.off.key())
            elif k == "index":
                r = ("ix", self.off.key())
            elif k == "acc":
                r = ("acc", self.dt)
            elif k == "let":
                r = ("let", self.let.id)
            elif k == "rand":
                r = ("rand", self.salt, self.open_low)
            else:
                r = (k, self.op, self.dt) + tuple(x.key() for x in self.a)
            self._key = r
        return self._key

    def walk(self):
        """This node and everything below it, including the index loads of gathers."""
        yield self
        for x in self.a:
            yield from x.walk()

    def __repr__(self):
        return fmt_expr(self)


@dataclass(eq=False)
class Let:
    id: int
    name: str
    value: E


@dataclass(eq=False)
class Store:
    buf: Buffer
    offset: Affine
    value: E
    accumulate: bool = False


@dataclass(eq=False)
class Reduction:
    vars: list
    op: str
    body: E

    @property
    def dtype(self):
        return I32 if self.op in ("argmax", "argmin") else self.body.dt


@dataclass(eq=False)
class Kernel:
    id: int
    name: str
    label: str
    domain: list
    stmts: list
    red: Reduction | None = None
    rand_base: object = None   # (i32 0-d Buffer, coef): coef * buffer value is added to the element index of
                               # every random draw (a rank's slice of a global tensor)
    src: object = None         # (file path, line number, text of the line) of the source statement, when known
                               # (reference anvil/ir.py: `Kernel.span`); cost reports and --check messages use it

    @property
    def stores(self):
        return [s for s in self.stmts if isinstance(s, Store)]

    def exprs(self):
        if self.red is not None:
            yield self.red.body
        for s in self.stmts:
            yield s.value

    def uses_rand(self) -> bool:
        return any(n.k == "rand" for e in self.exprs() for n in e.walk())

    def loads(self):
        """Every (buffer, offset) read: expression loads, gather index loads, `+=` targets excluded."""
        out = []

        def aff(a: Affine):
            for g, _ in a.gathers():
                out.append((g.buf, g.offset))
                aff(g.offset)

        for e in self.exprs():
            for n in e.walk():
                if n.k == "load":
                    out.append((n.buf, n.off))
                    aff(n.off)
                elif n.k == "index":
                    aff(n.off)
        for s in self.stores:
            aff(s.offset)
        return out

    def reads(self) -> set:
        out = {b.root for b, _ in self.loads()}
        for a in self.offsets():
            for s, _ in a.scalars():
                out.add(s.buf.root)
        for s in self.stores:
            if s.accumulate:
                out.add(s.buf.root)
        return out

    def offsets(self):
        for e in self.exprs():
            for n in e.walk():
                if n.k in ("load", "index"):
                    yield n.off
                    yield from _nested(n.off)
        for s in self.stores:
            yield s.offset
            yield from _nested(s.offset)

    def writes(self) -> set:
        return {s.buf.root for s in self.stores}

    def out_numel(self) -> int:
        return prod(v.extent for v in self.domain)

    def red_numel(self) -> int:
        return prod(v.extent for v in self.red.vars) if self.red else 1


def _nested(a: Affine):
    for g, _ in a.gathers():
        yield g.offset
        yield from _nested(g.offset)


# ---- program statements (reference anvil/ir.py:647-737)

@dataclass(eq=False)
class KernelStmt:
    kernel: Kernel


@dataclass(eq=False)
class Block:
    stmts: list = field(default_factory=list)


@dataclass(eq=False)
class For:
    counter: Buffer
    start: object          # int | Buffer (i32 0-d)
    stop: object
    step: int
    body: Block


@dataclass(eq=False)
class While:
    cond_block: Block
    cond: Buffer
    body: Block


@dataclass(eq=False)
class If:
    cond: Buffer
    then: Block
    orelse: Block


@dataclass(eq=False)
class Break:
    pass


@dataclass(eq=False)
class Continue:
    pass


@dataclass(eq=False)
class PrintItem:
    kind: str              # text | scalar | tensor | pick | chars
    text: str = ""
    buf: Buffer | None = None
    fmt: str = ""
    choices: list | None = None


@dataclass(eq=False)
class Print:
    items: list
    end: str = "\n"
    err: bool = False


@dataclass(eq=False)
class Check:
    """Run-time assertion lo <= value <= hi, value an affine of run-time scalars."""
    value: Affine
    lo: int
    hi: int
    message: str           # already prefixed with the source location


@dataclass(eq=False)
class RTCall:
    name: str
    args: dict             # values: python scalars / str / bytes / Buffer / list[Buffer]


@dataclass(eq=False)
class AllReduce:
    """Sum the listed tensors over all ranks (data-parallel training; no reference counterpart: the
    reference has no multi-device code). The back end lays the tensors out contiguously and issues ONE
    collective over the span."""
    bufs: list


@dataclass(eq=False)
class Program:
    main: Block
    buffers: list
    name: str = "<program>"
    bucket: list = field(default_factory=list)     # tensors an AllReduce sums: laid out contiguously
    rank_buf: Buffer | None = None                 # i32 0-d: this process's rank in a data-parallel run

    def kernels(self) -> list[Kernel]:
        out = []
        for b in walk_blocks(self.main):
            for s in b.stmts:
                if isinstance(s, KernelStmt):
                    out.append(s.kernel)
        return out

    def roots(self) -> list[Buffer]:
        seen, out = set(), []
        for b in self.buffers:
            r = b.root
            if r.id not in seen:
                seen.add(r.id)
                out.append(r)
        return out


def walk_blocks(block: Block):
    yield block
    for s in block.stmts:
        if isinstance(s, For):
            yield from walk_blocks(s.body)
        elif isinstance(s, While):
            yield from walk_blocks(s.cond_block)
            yield from walk_blocks(s.body)
        elif isinstance(s, If):
            yield from walk_blocks(s.then)
            yield from walk_blocks(s.orelse)


# ----------------------------------------------------------------------------- pretty printing

_SYM = {"add": "+", "sub": "-", "mul": "*", "div": "/", "idiv": "//", "mod": "%", "pow": "**",
        "lt": "<", "le": "<=", "gt": ">", "ge": ">=", "eq": "==", "ne": "!=", "and": "and", "or": "or"}


def fmt_expr(e: E) -> str:
    k = e.k
    if k == "const":
        return repr(e.val)
    if k == "load":
        return f"{e.buf.name}{{{e.off!r}}}"
    if k == "index":
        return f"ix({e.off!r})"
    if k == "acc":
        return "acc"
    if k == "let":
        return e.let.name
    if k == "rand":
        return f"rand{'+' if e.open_low else ''}{e.salt}"
    if k == "un":
        return f"{e.op}({fmt_expr(e.a[0])})"
    if k == "bin":
        if e.op in ("max", "min"):
            return f"{e.op}({fmt_expr(e.a[0])}, {fmt_expr(e.a[1])})"
        return f"({fmt_expr(e.a[0])} {_SYM[e.op]} {fmt_expr(e.a[1])})"
    if k == "sel":
        return f"({fmt_expr(e.a[1])} if {fmt_expr(e.a[0])} else {fmt_expr(e.a[2])})"
    return f"<{k}>"


def fmt_kernel(k: Kernel) -> str:
    head = f"{k.name} [{' x '.join(map(repr, k.domain))}]"
    if k.red is not None:
        head += f" {k.red.op}_[{' x '.join(map(repr, k.red.vars))}] {fmt_expr(k.red.body)}"
    parts = []
    for s in k.stmts:
        if isinstance(s, Let):
            parts.append(f"let {s.name} = {fmt_expr(s.value)}")
        else:
            parts.append(f"{s.buf.name}{{{s.offset!r}}} {'+=' if s.accumulate else '='} {fmt_expr(s.value)}")
    return head + " :: " + "; ".join(parts) + (f"  <{k.label}>" if k.label else "")


# ----------------------------------------------------------------------------- from a live anvil.ir.Program

def _fnv_ckpt_key(name: str, dtype: str, shape) -> int:
    """Checkpoint key of a tensor: FNV-1a of `name-inside-model:dtype:shape` in the high 32 bits,
    element count in the low 32 (reference anvil/ir.py:753-764)."""
    inside = name.split(".", 1)[1] if "." in name else ""
    h = 2166136261
    for byte in f"{inside}:{dtype}:{','.join(map(str, shape))}".encode():
        h = ((h ^ byte) * 16777619) & 0xFFFFFFFF
    return ((h or 1) << 32) | prod(shape)


class _Importer:
    """Walks an `anvil.ir.Program` by attribute and class name only."""

    def __init__(self):
        self.bufs: dict[int, Buffer] = {}
        self.vars: dict[int, Var] = {}
        self.lets: dict[int, Let] = {}
        self.order: list[Buffer] = []
        self.next_id = 1

    def buffer(self, b) -> Buffer:
        hit = self.bufs.get(id(b))
        if hit is not None:
            return hit
        init = None
        if getattr(b, "init", None) is not None and b.storage is b:
            init = np.asarray(b.init, dtype=np.int32 if b.dtype == I32 else np.float32).reshape(-1)
        nb = Buffer(int(b.id), str(b.name), tuple(b.shape), b.dtype, b.kind, init,
                    _fnv_ckpt_key(str(b.name), b.dtype, tuple(int(d) for d in b.shape))
                    if prod(b.shape) < (1 << 32) else 0)
        self.bufs[id(b)] = nb
        self.order.append(nb)
        if b.storage is not b:
            nb.root = self.buffer(b.root)
        return nb

    def var(self, v) -> Var:
        hit = self.vars.get(id(v))
        if hit is None:
            hit = self.vars[id(v)] = Var(int(v.id), str(v.name), int(v.extent))
        return hit

    def affine(self, a) -> Affine:
        terms = []
        for t, c in a.terms.items():
            cn = type(t).__name__
            if cn == "Var":
                terms.append((self.var(t), c))
            elif cn == "ScalarRef":
                terms.append((SRef(self.buffer(t.buf)), c))
            elif cn == "Gather":
                # `rest` (the `+ t` of `ids[i] + t`) already sits in the enclosing offset's other
                # terms; it only narrows the range the gathered value may take.
                lo, hi = t.check_range()
                off = self.affine(t.load.offset)
                terms.append((Gather(self.buffer(t.load.buf), off, int(t.bound), str(t.where or ""),
                                     int(lo), int(hi)), c))
            else:
                raise NotImplementedError(f"affine term {cn}")
        return Affine(int(a.const), terms)

    def expr(self, e, memo) -> E:
        hit = memo.get(id(e))
        if hit is not None:
            return hit
        cn = type(e).__name__
        if cn == "Const":
            r = E("const", e.dtype, val=(float(e.value) if e.dtype == F32 else int(e.value)))
        elif cn == "Load":
            r = E("load", e.dtype, buf=self.buffer(e.buf), off=self.affine(e.offset))
        elif cn == "Index":
            r = E("index", I32, off=self.affine(e.affine))
        elif cn == "Unary":
            r = E("un", e.dtype, op=e.op, a=[self.expr(e.a, memo)])
        elif cn == "Binary":
            r = E("bin", e.dtype, op=e.op, a=[self.expr(e.a, memo), self.expr(e.b, memo)])
        elif cn == "Select":
            r = E("sel", e.dtype, a=[self.expr(e.c, memo), self.expr(e.a, memo), self.expr(e.b, memo)])
        elif cn == "Acc":
            r = E("acc", e.dtype)
        elif cn == "LetRef":
            r = E("let", e.dtype, let=self.lets[id(e.let)])
        elif cn == "Rand":
            r = E("rand", F32, salt=int(e.salt), open_low=bool(e.open_low))
        else:
            raise NotImplementedError(f"expression {cn}")
        memo[id(e)] = r
        return r

    def kernel(self, k) -> Kernel:
        memo: dict = {}
        domain = [self.var(v) for v in k.domain]
        red = None
        if k.red is not None:
            red = Reduction([self.var(v) for v in k.red.vars], k.red.op, self.expr(k.red.body, memo))
        stmts = []
        for s in k.stmts:
            if type(s).__name__ == "Let":
                nl = Let(self.next_id, str(s.name), self.expr(s.value, memo))
                self.next_id += 1
                self.lets[id(s)] = nl
                stmts.append(nl)
            else:
                stmts.append(Store(self.buffer(s.buf), self.affine(s.offset), self.expr(s.value, memo),
                                   bool(s.accumulate)))
        src = None
        span = getattr(k, "span", None)
        if span is not None and getattr(span, "file", None) is not None:
            try:
                text = span.file.line_text(span.line).strip()
            except Exception:
                text = ""
            src = (str(span.file.path).replace("\\", "/").rsplit("/", 1)[-1], int(span.line), text[:200])   # the file's name, not where it lay
        return Kernel(int(k.id), str(k.name or f"k{k.id}"), str(k.label or ""), domain, stmts, red, None, src)

    def bound(self, x):
        return int(x) if isinstance(x, int) else self.buffer(x)

    def block(self, b) -> Block:
        return Block([self.stmt(s) for s in b.stmts])

    def stmt(self, s):
        cn = type(s).__name__
        if cn == "KernelStmt":
            return KernelStmt(self.kernel(s.kernel))
        if cn == "For":
            return For(self.buffer(s.counter), self.bound(s.start), self.bound(s.stop), int(s.step), self.block(s.body))
        if cn == "While":
            return While(self.block(s.cond_block), self.buffer(s.cond), self.block(s.body))
        if cn == "If":
            return If(self.buffer(s.cond), self.block(s.then), self.block(s.orelse))
        if cn == "Break":
            return Break()
        if cn == "Continue":
            return Continue()
        if cn == "Print":
            items = [PrintItem(it.kind, it.text or "", self.buffer(it.buf) if it.buf is not None else None,
                               it.fmt or "", list(it.choices) if it.choices else None) for it in s.items]
            return Print(items, s.end, bool(s.err))
        if cn == "Check":
            loc = f"{s.span.location()}: " if getattr(s, "span", None) is not None else ""
            return Check(self.affine(s.value), int(s.lo), int(s.hi), loc + str(s.message))
        if cn == "RTCall":
            args = {}
            for key, v in s.args.items():
                if type(v).__name__ == "Buffer":
                    args[key] = self.buffer(v)
                elif isinstance(v, (list, tuple)) and v and type(v[0]).__name__ == "Buffer":
                    args[key] = [self.buffer(x) for x in v]
                elif isinstance(v, (bytes, bytearray)):
                    args[key] = bytes(v)
                elif isinstance(v, (list, tuple)):
                    args[key] = list(v)
                else:
                    args[key] = v
            return RTCall(str(s.name), args)
        raise NotImplementedError(f"statement {cn}")


def from_anvil(prog, name: str = "<program>") -> Program:
    """Convert an `anvil.ir.Program` (after `optimize_program`) into KIR."""
    imp = _Importer()
    for b in prog.buffers:
        imp.buffer(b)
    main = imp.block(prog.main)
    return Program(main, list(imp.order), name)


# ----------------------------------------------------------------------------- JSON form

class _Writer:
    def __init__(self):
        self.buf_ids: dict[int, int] = {}

    def aff(self, a: Affine):
        terms = []
        for t, c in a.terms:
            if isinstance(t, Var):
                terms.append(["v", t.id, c])
            elif isinstance(t, SRef):
                terms.append(["s", t.buf.id, c])
            else:
                terms.append(["g", t.buf.id, self.aff(t.offset), t.bound, t.where, t.lo, t.hi, c])
        return [a.const, terms]

    def kernel(self, k: Kernel):
        nodes: list = []
        index: dict = {}

        def put(e: E) -> int:
            key = e.key()
            hit = index.get(key)
            if hit is not None:
                return hit
            kids = [put(x) for x in e.a]
            if e.k == "const":
                v = e.val
                if isinstance(v, float) and (v != v or v in (float("inf"), float("-inf"))):
                    v = repr(v)
                n = ["const", e.dt, v]
            elif e.k == "load":
                n = ["load", e.dt, e.buf.id, self.aff(e.off)]
            elif e.k == "index":
                n = ["index", self.aff(e.off)]
            elif e.k == "acc":
                n = ["acc", e.dt]
            elif e.k == "let":
                n = ["let", e.dt, e.let.id]
            elif e.k == "rand":
                n = ["rand", e.salt, 1 if e.open_low else 0]
            else:
                n = [e.k, e.dt, e.op, kids]
            nodes.append(n)
            index[key] = len(nodes) - 1
            return len(nodes) - 1

        out = {"id": k.id, "name": k.name, "label": k.label,
               "domain": [[v.id, v.name, v.extent] for v in k.domain]}
        if k.red is not None:
            out["red"] = {"vars": [[v.id, v.name, v.extent] for v in k.red.vars], "op": k.red.op,
                          "body": put(k.red.body)}
        stmts = []
        for s in k.stmts:
            if isinstance(s, Let):
                stmts.append(["let", s.id, s.name, put(s.value)])
            else:
                stmts.append(["store", s.buf.id, self.aff(s.offset), put(s.value), 1 if s.accumulate else 0])
        out["stmts"] = stmts
        out["nodes"] = nodes
        if k.src is not None:
            out["src"] = list(k.src)
        return out

    def bound(self, x):
        return x if isinstance(x, int) else {"buf": x.id}

    def block(self, b: Block):
        return [self.stmt(s) for s in b.stmts]

    def stmt(self, s):
        if isinstance(s, KernelStmt):
            return {"t": "kernel", "k": self.kernel(s.kernel)}
        if isinstance(s, For):
            return {"t": "for", "counter": s.counter.id, "start": self.bound(s.start), "stop": self.bound(s.stop),
                    "step": s.step, "body": self.block(s.body)}
        if isinstance(s, While):
            return {"t": "while", "cond_block": self.block(s.cond_block), "cond": s.cond.id, "body": self.block(s.body)}
        if isinstance(s, If):
            return {"t": "if", "cond": s.cond.id, "then": self.block(s.then), "orelse": self.block(s.orelse)}
        if isinstance(s, Break):
            return {"t": "break"}
        if isinstance(s, Continue):
            return {"t": "continue"}
        if isinstance(s, Print):
            return {"t": "print", "end": s.end, "err": s.err,
                    "items": [{"kind": it.kind, "text": it.text, "buf": it.buf.id if it.buf is not None else None,
                               "fmt": it.fmt, "choices": it.choices} for it in s.items]}
        if isinstance(s, Check):
            return {"t": "check", "value": self.aff(s.value), "lo": s.lo, "hi": s.hi, "message": s.message}
        if isinstance(s, RTCall):
            args = {}
            for key, v in s.args.items():
                if isinstance(v, Buffer):
                    args[key] = {"buf": v.id}
                elif isinstance(v, list) and v and isinstance(v[0], Buffer):
                    args[key] = {"bufs": [x.id for x in v]}
                elif isinstance(v, bytes):
                    args[key] = {"bytes": base64.b64encode(v).decode()}
                else:
                    args[key] = v
            return {"t": "rtcall", "name": s.name, "args": args}
        raise NotImplementedError(type(s).__name__)


def dumps(prog: Program) -> str:
    w = _Writer()
    bufs = []
    for b in prog.buffers:
        d = {"id": b.id, "name": b.name, "shape": list(b.shape), "dtype": b.dtype, "kind": b.kind,
             "root": b.root.id, "ckpt_key": str(b.ckpt_key)}
        if b.init is not None:
            d["init"] = base64.b64encode(np.ascontiguousarray(b.init).tobytes()).decode()
        bufs.append(d)
    return json.dumps({"kir": 1, "name": prog.name, "buffers": bufs, "main": w.block(prog.main)},
                      separators=(",", ":"))


def dump(prog: Program, path: str):
    data = dumps(prog).encode()
    if path.endswith(".gz"):
        with gzip.GzipFile(path, "wb", mtime=0) as f:
            f.write(data)
    else:
        with open(path, "wb") as f:
            f.write(data)


class _Reader:
    def __init__(self, bufs):
        self.bufs = bufs
        self.vars: dict[int, Var] = {}
        self.lets: dict[int, Let] = {}

    def var(self, t) -> Var:
        hit = self.vars.get(t[0])
        if hit is None:
            hit = self.vars[t[0]] = Var(t[0], t[1], t[2])
        return hit

    def aff(self, a) -> Affine:
        terms = []
        for t in a[1]:
            if t[0] == "v":
                terms.append((self.vars[t[1]], t[2]))
            elif t[0] == "s":
                terms.append((SRef(self.bufs[t[1]]), t[2]))
            else:
                terms.append((Gather(self.bufs[t[1]], self.aff(t[2]), t[3], t[4], t[5], t[6]), t[7]))
        return Affine(a[0], terms)

    def kernel(self, d) -> Kernel:
        domain = [self.var(v) for v in d["domain"]]
        rvars = [self.var(v) for v in d["red"]["vars"]] if "red" in d else []
        for s in d["stmts"]:
            if s[0] == "let":
                self.lets[s[1]] = Let(s[1], s[2], None)     # value filled in below
        built: list = []
        for n in d["nodes"]:
            k = n[0]
            if k == "const":
                v = n[2]
                v = float(v) if n[1] == F32 else int(v)
                e = E("const", n[1], val=v)
            elif k == "load":
                e = E("load", n[1], buf=self.bufs[n[2]], off=self.aff(n[3]))
            elif k == "index":
                e = E("index", I32, off=self.aff(n[1]))
            elif k == "acc":
                e = E("acc", n[1])
            elif k == "let":
                e = E("let", n[1], let=self.lets[n[2]])
            elif k == "rand":
                e = E("rand", F32, salt=n[1], open_low=bool(n[2]))
            else:
                e = E(k, n[1], op=n[2], a=[built[i] for i in n[3]])
            built.append(e)
        red = None
        if "red" in d:
            red = Reduction(rvars, d["red"]["op"], built[d["red"]["body"]])
        stmts = []
        for s in d["stmts"]:
            if s[0] == "let":
                let = self.lets[s[1]]
                let.value = built[s[3]]
                stmts.append(let)
            else:
                stmts.append(Store(self.bufs[s[1]], self.aff(s[2]), built[s[3]], bool(s[4])))
        src = tuple(d["src"]) if d.get("src") else None
        return Kernel(d["id"], d["name"], d["label"], domain, stmts, red, None, src)

    def bound(self, x):
        return x if isinstance(x, int) else self.bufs[x["buf"]]

    def block(self, b) -> Block:
        return Block([self.stmt(s) for s in b])

    def stmt(self, s):
        t = s["t"]
        if t == "kernel":
            return KernelStmt(self.kernel(s["k"]))
        if t == "for":
            return For(self.bufs[s["counter"]], self.bound(s["start"]), self.bound(s["stop"]), s["step"],
                       self.block(s["body"]))
        if t == "while":
            return While(self.block(s["cond_block"]), self.bufs[s["cond"]], self.block(s["body"]))
        if t == "if":
            return If(self.bufs[s["cond"]], self.block(s["then"]), self.block(s["orelse"]))
        if t == "break":
            return Break()
        if t == "continue":
            return Continue()
        if t == "print":
            return Print([PrintItem(it["kind"], it["text"], self.bufs[it["buf"]] if it["buf"] is not None else None,
                                    it["fmt"], it["choices"]) for it in s["items"]], s["end"], s["err"])
        if t == "check":
            return Check(self.aff(s["value"]), s["lo"], s["hi"], s["message"])
        if t == "rtcall":
            args = {}
            for key, v in s["args"].items():
                if isinstance(v, dict) and "buf" in v:
                    args[key] = self.bufs[v["buf"]]
                elif isinstance(v, dict) and "bufs" in v:
                    args[key] = [self.bufs[i] for i in v["bufs"]]
                elif isinstance(v, dict) and "bytes" in v:
                    args[key] = base64.b64decode(v["bytes"])
                else:
                    args[key] = v
            return RTCall(s["name"], args)
        raise NotImplementedError(t)


def loads(text: str) -> Program:
    d = json.loads(text)
    if d.get("kir") != 1:
        raise ValueError("not a KIR file (or an unknown version)")
    bufs: dict[int, Buffer] = {}
    order = []
    for b in d["buffers"]:
        init = None
        if "init" in b:
            init = np.frombuffer(base64.b64decode(b["init"]), dtype=np.int32 if b["dtype"] == I32 else np.float32).copy()
        nb = Buffer(b["id"], b["name"], tuple(b["shape"]), b["dtype"], b["kind"], init, int(b["ckpt_key"]))
        bufs[nb.id] = nb
        order.append((nb, b["root"]))
    for nb, root in order:
        nb.root = bufs[root]
    r = _Reader(bufs)
    return Program(r.block(d["main"]), [nb for nb, _ in order], d.get("name", "<program>"))


def load(path: str) -> Program:
    if path.endswith(".gz"):
        with gzip.open(path, "rb") as f:
            return loads(f.read().decode())
    with open(path, "rb") as f:
        return loads(f.read().decode())
