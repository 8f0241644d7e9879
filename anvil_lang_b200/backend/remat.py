"""Recomputing a saved elementwise intermediate instead of storing it.

Reverse-mode differentiation saves every intermediate of the forward pass that the backward pass names. For an
activation function that leaves, per element, several tensors in memory that are cheap functions of one another
(anvil/prelude.anvil `gelu`, differentiated by anvil/autodiff.py):

    forward   u = 0.044715 * h * h;  store u;  t = tanh(0.79788 * (h + u * h));  store t;  g = 0.5 * h * (1 + t);  store g
    backward  dh = f(dg, h, t, u)                                                 loads dg, h, t, u

Both kernels run at the speed of HBM, and `u` and `t` cost one store and one load each per element although the
backward kernel holds `h`, from which they follow in a handful of operations. This pass rewrites the consumer to
compute the value from the producer's own inputs and drops the store:

    forward   store g only;        backward   u = 0.044715 * h * h;  t = tanh(...);  dh = f(dg, h, t, u)

The recomputed value is the same expression on the same f32 inputs, evaluated by the same instruction sequence (the
generated code is built without floating-point contraction), so results are bit-identical.

A stored tensor T of an elementwise kernel K is recomputed when
  * T is a temporary that only K writes, the host never reads, and K stores it plainly at the identity element;
  * its value reads tensors at the identity element only, is small (at most `MAX_NODES` nodes, one transcendental)
    and uses no random numbers;
  * every kernel that reads T sits after K in the same statement list, has no reduction, has K's domain (the same
    extents), reads T at the identity element only and writes none of the value's inputs;
  * nothing between K and such a reader writes one of the value's inputs;
  * the reader has to load at most one tensor more than it already does.
"""
from __future__ import annotations

import itertools

from .. import kir
from ..kir import Affine, E, Kernel, KernelStmt, Let, Store
from . import analysis as an

MAX_NODES = 24
TRANSCENDENTAL = ("tanh", "exp", "log", "sqrt", "sin", "cos", "pow", "sigmoid", "erf")


def _identity(domain) -> Affine:
    strides = kir.row_major_strides([v.extent for v in domain])
    return Affine(0, list(zip(domain, strides)))


class _Value:
    """A stored value of K with K's lets expanded: its nodes, inputs and whether it may be recomputed elsewhere."""

    def __init__(self, K: Kernel, value: E):
        self.K, self.value = K, value
        self.ident = _identity(K.domain)
        self.nodes, self.heavy, self.inputs, self.ok = 0, 0, {}, True
        self._seen: set = set()
        self._walk(value)

    def _walk(self, e: E):
        if id(e) in self._seen:
            return
        self._seen.add(id(e))
        self.nodes += 1
        if e.k == "load":
            if e.off != self.ident:
                self.ok = False
            self.inputs[e.buf.root.id] = e.buf.root
        elif e.k == "let":
            self._walk(e.let.value)
        elif e.k in ("acc", "rand", "index"):
            self.ok = False
        elif e.k in ("un", "bin") and e.op in TRANSCENDENTAL:
            self.heavy += 1
        for x in e.a:
            self._walk(x)

    def rebuilt(self, ident_c: Affine, memo: dict) -> E:
        """The same expression over another kernel's identity element, lets expanded."""
        def go(e: E) -> E:
            hit = memo.get(id(e))
            if hit is not None:
                return hit
            if e.k == "load":
                r = E("load", e.dt, buf=e.buf, off=ident_c)
            elif e.k == "let":
                r = go(e.let.value)
            elif e.a:
                r = E(e.k, e.dt, op=e.op, a=[go(x) for x in e.a])
            else:
                r = e
            memo[id(e)] = r
            return r
        return go(self.value)


def _replace_loads(C: Kernel, root_id: int, let: Let) -> None:
    memo: dict = {}

    def go(e: E) -> E:
        hit = memo.get(id(e))
        if hit is not None:
            return hit
        if e.k == "load" and e.buf.root.id == root_id:
            r = E("let", e.dt, let=let)
        elif e.a:
            a = [go(x) for x in e.a]
            r = e if all(x is y for x, y in zip(a, e.a)) else E(e.k, e.dt, op=e.op, a=a)
        else:
            r = e
        memo[id(e)] = r
        return r
    out = [let]
    for st in C.stmts:
        if isinstance(st, Let):
            st.value = go(st.value)
            out.append(st)
        else:
            out.append(Store(st.buf, st.offset, go(st.value), st.accumulate))
    C.stmts = out


def _may_write(st) -> set:
    """Root ids a statement between producer and reader may write (nested statements included; a runtime call or a
    collective counts as writing every tensor it names)."""
    out: set = set()
    if isinstance(st, KernelStmt):
        return {b.id for b in st.kernel.writes()}
    if isinstance(st, (kir.Print, kir.Check, kir.Break, kir.Continue)):
        return out
    if isinstance(st, kir.RTCall):
        for v in st.args.values():
            for x in (v if isinstance(v, list) else [v]):
                if isinstance(x, kir.Buffer):
                    out.add(x.root.id)
        return out
    if isinstance(st, kir.AllReduce):
        return {b.root.id for b in st.bufs}
    for name in ("body", "then", "orelse", "cond_block"):
        blk = getattr(st, name, None)
        if isinstance(blk, kir.Block):
            for inner in blk.stmts:
                out |= _may_write(inner)
    for name in ("counter",):
        b = getattr(st, name, None)
        if isinstance(b, kir.Buffer):
            out.add(b.root.id)
    return out


def rematerialize(prog: kir.Program, host_reads: set) -> int:
    """Rewrites `prog` in place; returns the number of stores dropped. Idempotent."""
    ids = itertools.count(max([b.id for b in prog.buffers] + [k.id for k in prog.kernels()]
                              + [st.id for k in prog.kernels() for st in k.stmts if isinstance(st, Let)]) + 19000)
    writers: dict = {}
    readers: dict = {}
    for k in prog.kernels():
        for b in k.writes():
            writers.setdefault(b.id, set()).add(k.id)
        for b in k.reads():
            readers.setdefault(b.id, set()).add(k.id)
    dropped = 0
    for blk in kir.walk_blocks(prog.main):
        stmts = blk.stmts
        where = {st.kernel.id: i for i, st in enumerate(stmts) if isinstance(st, KernelStmt)}
        for i, st in enumerate(stmts):
            if not isinstance(st, KernelStmt):
                continue
            K = st.kernel
            if K.red is not None or K.uses_rand() or K.rand_base is not None or not K.domain or len(K.stores) < 2:
                continue
            ident = _identity(K.domain)
            extents = [v.extent for v in K.domain]
            for s in list(K.stores):
                T = s.buf.root
                if (T.kind != "temp" or T.id in host_reads or writers.get(T.id) != {K.id} or s.accumulate
                        or s.offset != ident or sum(1 for x in K.stores if x.buf.root is T) != 1):
                    continue
                # the kernel's own value must not read T back (a later statement of K reading its own store)
                if any(b.root is T for b, _ in K.loads()):
                    continue
                val = _Value(K, s.value)
                if not val.ok or val.nodes > MAX_NODES or val.heavy > 1 or T.id in val.inputs:
                    continue
                users = readers.get(T.id, set())
                if not users or not all(u in where and where[u] > i for u in users):
                    continue
                good = True
                for u in users:
                    C = stmts[where[u]].kernel
                    if (C.red is not None or [v.extent for v in C.domain] != extents
                            or any(b.root is T and off != _identity(C.domain) for b, off in C.loads())
                            or any(b.id in val.inputs for b in C.writes())
                            or len(set(val.inputs) - ({b.id for b in C.reads()} - {T.id})) > 1):
                        good = False
                        break
                    if any(_may_write(mid) & set(val.inputs) for mid in stmts[i + 1:where[u]]):
                        good = False
                        break
                if not good:
                    continue
                for u in users:
                    C = stmts[where[u]].kernel
                    let = Let(next(ids), T.name, val.rebuilt(_identity(C.domain), {}))
                    _replace_loads(C, T.id, let)
                    if not an.parallel_safe(C):
                        raise AssertionError(f"rematerialising {T.name} made kernel {C.name} unsafe")
                    for r in val.inputs.values():
                        readers.setdefault(r.id, set()).add(C.id)
                K.stmts = [x for x in K.stmts if x is not s]
                readers.pop(T.id, None)
                writers.pop(T.id, None)
                dropped += 1
    return dropped
