"""Producer / consumer re-fusion: an elementwise kernel is folded into the kernel that makes its input.

The reference's optimizer fuses an elementwise consumer into its producer, but stops when the producer is a
matrix-product-like kernel and the merged statement list would exceed 8 expression nodes
(`GEMM_EPILOGUE = 8`, anvil/optimize.py:34, :838-841: on the CPU a longer epilogue costs the register tile). For
Adam on a weight matrix that leaves a pair (anvil/prelude.anvil:144-151 expanded by anvil/autodiff.py:409-491):

    P:  dW[k, j] = sum_i A[i, k] * dY[i, j];  store dW;  m = 0.9 m + 0.1 dW;  store m
    C:  v[ij] = 0.999 v[ij] + 0.001 dW[ij]^2;  W[ij] -= lr * (m[ij] / c1) / (sqrt(v[ij] / c2) + eps)

so the gradient goes to HBM and comes back, and `m` is read again. On a GPU the epilogue of a contraction runs out
of tensor memory through registers with room to spare, so the pair becomes ONE kernel here: C's statements are
appended to P's, C's loads of what P stored are replaced by the stored values, and a tensor that only C read (dW)
is no longer stored at all. The same rewrite joins the two elementwise halves an update is split into for data
parallel runs.

The fused kernel computes exactly what the pair computes, operation by operation (the generated code is built with
-fmad=false, and a value kept in a register is the f32 that would have been stored and re-loaded), so results are
bit-identical to the unfused program.

Legality:
  * P's stores all hit the row-major identity element of P's domain, none accumulates; C has no reduction, no random
    numbers, and its domain is P's domain or that domain collapsed into one index;
  * every access of C to a tensor P writes hits the identity element; C's stores are to identity elements too;
  * P moves down to C's place: no kernel in between may write what P reads or writes, or read what P writes;
  * the result must still be safe to run one element per thread (`analysis.parallel_safe`).
By default only consumers that update parameters or optimizer state are folded (`only_updates`).
"""
from __future__ import annotations

import itertools

from .. import kir
from ..kir import Affine, E, Kernel, KernelStmt, Let, Store, Var
from . import analysis as an

UPDATED_KINDS = ("param", "state")


def _identity(domain) -> Affine:
    strides = kir.row_major_strides([v.extent for v in domain])
    return Affine(0, list(zip(domain, strides)))


def _var_map(P: Kernel, C: Kernel):
    """C's domain vars expressed over P's: {var of C: [(var of P, coefficient), ...]} or None."""
    pn = [v for v in P.domain]
    if len(C.domain) == 1 and C.domain[0].extent == P.out_numel():
        return {C.domain[0]: list(zip(pn, kir.row_major_strides([v.extent for v in pn])))}
    if [v.extent for v in C.domain] == [v.extent for v in pn]:
        return {cv: [(pv, 1)] for cv, pv in zip(C.domain, pn)}
    return None


def _subst_affine(a: Affine, m: dict) -> Affine | None:
    const, terms = a.const, {}
    order = []
    for t, c in a.terms:
        if isinstance(t, Var):
            if t not in m:
                return None
            for pv, pc in m[t]:
                if pv not in terms:
                    order.append(pv)
                terms[pv] = terms.get(pv, 0) + c * pc
        elif isinstance(t, kir.Gather):
            inner = _subst_affine(t.offset, m)
            if inner is None:
                return None
            g = kir.Gather(t.buf, inner, t.bound, t.where, t.lo, t.hi)
            order.append(g)
            terms[g] = c
        else:
            order.append(t)
            terms[t] = terms.get(t, 0) + c
    return Affine(const, [(t, terms[t]) for t in order])


class _Merge:
    def __init__(self, P: Kernel, C: Kernel, ids):
        self.P, self.C, self.ids = P, C, ids
        self.vmap = _var_map(P, C)
        self.ident = _identity(P.domain)
        self.stored: dict = {}                    # root id -> value expression P stored at the identity element
        self.lets: dict = {}
        self.memo: dict = {}
        self.ok = self.vmap is not None

    def expr(self, e: E) -> E:
        hit = self.memo.get(id(e))
        if hit is not None:
            return hit
        if e.k == "load":
            off = _subst_affine(e.off, self.vmap)
            if off is None:
                self.ok = False
                off = e.off
            rid = e.buf.root.id
            if rid in self.stored:
                if off != self.ident:
                    self.ok = False               # reads an element another thread of P wrote
                r = self.stored[rid]
            else:
                r = E("load", e.dt, buf=e.buf, off=off)
        elif e.k == "index":
            off = _subst_affine(e.off, self.vmap)
            if off is None:
                self.ok = False
                off = e.off
            r = E("index", e.dt, off=off)
        elif e.k == "let":
            r = E("let", e.dt, let=self.lets[e.let.id])
        elif e.k in ("acc", "rand"):
            self.ok = False
            r = e
        elif e.a:
            r = E(e.k, e.dt, op=e.op, a=[self.expr(x) for x in e.a])
        else:
            r = e
        self.memo[id(e)] = r
        return r


def merge(P: Kernel, C: Kernel, ids, droppable: set) -> Kernel | None:
    """The fused kernel, or None when the pair does not have the shape described in the module docstring.
    `droppable`: root ids whose stores by P may be dropped (nothing but C reads them)."""
    if C.red is not None or C.uses_rand() or P.uses_rand() or C.rand_base is not None or not P.domain:
        return None
    mg = _Merge(P, C, ids)
    if not mg.ok:
        return None
    for st in P.stores:
        if st.accumulate or st.offset != mg.ident or st.buf.root.id in mg.stored:
            return None
        mg.stored[st.buf.root.id] = st.value
    if not any(b.root.id in mg.stored for b, _ in C.loads()):
        return None
    stmts = [st for st in P.stmts if not (isinstance(st, Store) and st.buf.root.id in droppable)]
    for st in C.stmts:
        if isinstance(st, Let):
            nl = Let(next(ids), st.name, mg.expr(st.value))
            mg.lets[st.id] = nl
            stmts.append(nl)
            continue
        off = _subst_affine(st.offset, mg.vmap)
        if off is None or off != mg.ident or st.accumulate:
            return None
        val = mg.expr(st.value)
        stmts.append(Store(st.buf, off, val, False))
        mg.stored[st.buf.root.id] = val           # a later read of it inside C sees this value
    if not mg.ok:
        return None
    fused = Kernel(next(ids), f"{P.name}+{C.name}", f"{P.label}+{C.label}" if C.label else P.label, list(P.domain), stmts,
                   P.red, P.rand_base, P.src)
    # two stores to one tensor (P's and C's) would make the second one the only live one: drop the first
    last = {}
    for i, st in enumerate(fused.stmts):
        if isinstance(st, Store):
            last[st.buf.root.id] = i
    fused.stmts = [st for i, st in enumerate(fused.stmts) if not isinstance(st, Store) or last[st.buf.root.id] == i]
    if not an.parallel_safe(fused):
        return None
    return fused


def _host_reads(prog: kir.Program) -> set:
    out = set()

    def note(b):
        if isinstance(b, kir.Buffer):
            out.add(b.root.id)
    for blk in kir.walk_blocks(prog.main):
        for st in blk.stmts:
            if isinstance(st, kir.For):
                note(st.counter); note(st.start); note(st.stop)
            elif isinstance(st, (kir.While, kir.If)):
                note(st.cond)
            elif isinstance(st, kir.Print):
                for it in st.items:
                    note(it.buf)
            elif isinstance(st, kir.Check):
                for t, _ in st.value.scalars():
                    note(t.buf)
            elif isinstance(st, kir.RTCall):
                for v in st.args.values():
                    note(v)
                    if isinstance(v, list):
                        for x in v:
                            note(x)
            elif isinstance(st, kir.AllReduce):
                for b in st.bufs:
                    note(b)
    for b in prog.buffers:
        if b.root.kind not in ("temp", "grad"):
            out.add(b.root.id)
    for b in getattr(prog, "bucket", []):
        out.add(b.root.id)
    return out


def fuse_consumers(prog: kir.Program, only_updates: bool = True) -> int:
    """Rewrites `prog` in place; returns the number of pairs fused. Idempotent."""
    ids = itertools.count(max([b.id for b in prog.buffers] + [k.id for k in prog.kernels()]
                              + [v.id for k in prog.kernels() for v in list(k.domain) + (list(k.red.vars) if k.red else [])]) + 9000)
    host = _host_reads(prog)
    readers: dict = {}
    for k in prog.kernels():
        for r in k.reads():
            readers.setdefault(r.id, set()).add(k.id)
    fused_n = 0
    for blk in kir.walk_blocks(prog.main):
        stmts = blk.stmts
        i = 0
        while i < len(stmts):
            if not isinstance(stmts[i], KernelStmt):
                i += 1
                continue
            P = stmts[i].kernel
            pw = {b.id for b in P.writes()}
            pr = {b.id for b in P.reads()}
            j, found = i + 1, None
            while j < len(stmts) and isinstance(stmts[j], KernelStmt):
                K = stmts[j].kernel
                kr, kw = {b.id for b in K.reads()}, {b.id for b in K.writes()}
                if kr & pw:
                    found = j                        # the first kernel that reads what P makes: the consumer, or the end
                    break
                if kw & (pr | pw):
                    break
                j += 1
            if found is None:
                i += 1
                continue
            C = stmts[found].kernel
            if only_updates and not any(s.buf.root.kind in UPDATED_KINDS for s in C.stores):
                i += 1
                continue
            droppable = {r for r in pw if r not in host and readers.get(r, set()) <= {C.id}}
            f = merge(P, C, ids, droppable)
            if f is None:
                i += 1
                continue
            stmts[found] = KernelStmt(f)
            del stmts[i]
            for r in f.reads():
                readers.setdefault(r.id, set()).add(f.id)
            fused_n += 1
            # do not advance: the statement now at i is examined next (the fused kernel may feed a further consumer
            # when its own turn comes)
    return fused_n
