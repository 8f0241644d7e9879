"""Fixed-order formulations of accumulating stores that collide.

`out[f(i)] += v(i)` where several domain points i reach the same element is run with atomicAdd by the
reference (anvil/backend/cuda.py:260-261), so the order of the f32 additions — and the last bits of
the result — change from run to run. Two IR-to-IR rewrites remove the atomics:

  * gathered target (`dE[x[b, t], d] += de[b, t, d]`, the embedding gradient): the kernel is inverted
    into a reduction over the points that carry the index, one output per target element:
        dE[r, d] += sum_{b, t} (x[b, t] == r) * de[b, t, d]
    The reduction runs through the ordinary fixed-order kernels: a contraction template when it is large enough (it is
    a product of a one-hot matrix with the values), the fixed-tree reduction kernels otherwise. Used when the indexed
    dimension has at most MAX_ROWS entries (the cost is rows x sources comparisons).
    An index outside [0, bound) matches no row and is dropped (the reference reports a fault there).

  * affine target with overlap (`dx[n, c, i + u, j + v] += dp[n, i, j, c, u, v]`, col2im): the
    smallest set of domain vars P that makes the store injective over the rest is peeled off, and the
    kernel is issued once per value of P, in order (9 launches for a 3 x 3 window); inside one launch
    every element is written by exactly one thread, so the `+=` is a plain read-modify-write.

Kernels whose accumulating stores are already exclusive, or add integers, are left alone. Anything
the two rewrites do not cover keeps its atomics; `remaining_atomics(prog)` lists those.
"""
from __future__ import annotations

import itertools

from .. import kir
from ..kir import F32, I32, Affine, E, Kernel, KernelStmt, Let, Reduction, Store, Var
from . import analysis as an

MAX_ROWS = 1 << 16
MAX_PHASES = 64


def _colliding(k: kir.Kernel):
    return [s for s in k.stores if s.accumulate and s.buf.dtype == F32 and not an.exclusive_store(k, s)]


def _subst_affine(a: Affine, m: dict) -> Affine:
    const, terms = a.const, []
    for t, c in a.terms:
        if isinstance(t, Var) and t in m:
            r = m[t]
            if isinstance(r, int):
                const += c * r
            else:
                terms.append((r, c))
        elif isinstance(t, kir.Gather):
            terms.append((kir.Gather(t.buf, _subst_affine(t.offset, m), t.bound, t.where, t.lo, t.hi), c))
        else:
            terms.append((t, c))
    return Affine(const, terms)


def _subst_expr(e: E, m: dict, memo: dict, lets: dict) -> E:
    hit = memo.get(id(e))
    if hit is not None:
        return hit
    if e.k == "load":
        r = E("load", e.dt, buf=e.buf, off=_subst_affine(e.off, m))
    elif e.k == "index":
        r = E("index", I32, off=_subst_affine(e.off, m))
    elif e.k == "let":
        r = E("let", e.dt, let=lets[e.let.id])
    elif e.a:
        r = E(e.k, e.dt, op=e.op, a=[_subst_expr(x, m, memo, lets) for x in e.a])
    else:
        r = e
    memo[id(e)] = r
    return r


def _copy_stmts(k: kir.Kernel, m: dict, ids):
    lets, memo, out = {}, {}, []
    for st in k.stmts:
        if isinstance(st, Let):
            nl = Let(next(ids), st.name, _subst_expr(st.value, m, memo, lets))
            lets[st.id] = nl
            out.append(nl)
        else:
            out.append(Store(st.buf, _subst_affine(st.offset, m), _subst_expr(st.value, m, memo, lets), st.accumulate))
    return out


def invert_gather(k: kir.Kernel, ids) -> Kernel | None:
    if k.red is not None or len(k.stmts) != 1 or k.uses_rand():
        return None
    st = k.stmts[0]
    gs = st.offset.gathers()
    if len(gs) != 1 or st.offset.scalars():
        return None
    g, cg = gs[0]
    if g.offset.gathers() or g.offset.scalars() or g.hi - g.lo > MAX_ROWS or g.lo != 0:
        return None
    src_vars = g.offset.vars()
    plain = [t for t, _ in st.offset.var_terms()]
    if any(v in src_vars for v in plain):
        return None
    other = [v for v in k.domain if v not in src_vars]
    if set(plain) - set(other):
        return None
    r = Var(next(ids), "row", g.hi)
    # one-hot(index == row) * value: a product, so that a large scatter (an embedding gradient) is recognised as the
    # contraction  one_hot[rows, points] @ values[points, d]  and runs on the tensor-core template (1.0 and 0.0 are exact
    # there). A select would be the same sum for finite values; a non-finite value now reaches every row of its column.
    hit = E("bin", F32, op="eq", a=[E("load", I32, buf=g.buf, off=g.offset), E("index", I32, off=Affine(0, [(r, 1)]))])
    body = E("bin", F32, op="mul", a=[hit, st.value])
    target = Affine(st.offset.const, [(r, cg)] + st.offset.var_terms())
    return Kernel(next(ids), k.name + "_inv", k.label, [r] + other,
                  [Store(st.buf, target, E("acc", F32), True)], Reduction([v for v in k.domain if v in src_vars], "sum", body), src=k.src)


def phase_split(k: kir.Kernel, ids) -> list | None:
    if k.red is not None or k.uses_rand():
        return None
    bad = _colliding(k)
    if any(s.offset.gathers() for s in bad):
        return None
    phase: list = []
    rest = list(k.domain)
    for v in sorted(k.domain, key=lambda v: v.extent):
        if all(an.injective_over(s.offset, rest) for s in bad):
            break
        phase.append(v)
        rest.remove(v)
    if not phase or not all(an.injective_over(s.offset, rest) for s in bad):
        return None
    if kir.prod(v.extent for v in phase) > MAX_PHASES:
        return None
    out = []
    for values in itertools.product(*[range(v.extent) for v in phase]):
        m = dict(zip(phase, values))
        out.append(Kernel(next(ids), f"{k.name}_p{'_'.join(map(str, values))}", k.label, rest, _copy_stmts(k, m, ids), None, src=k.src))
    return out


def make_deterministic(prog: kir.Program) -> kir.Program:
    """Rewrites `prog` in place; returns it."""
    ids = itertools.count(max([b.id for b in prog.buffers] + [k.id for k in prog.kernels()]
                              + [v.id for k in prog.kernels() for v in k.domain]) + 5000)
    for blk in kir.walk_blocks(prog.main):
        new = []
        for st in blk.stmts:
            if isinstance(st, KernelStmt) and _colliding(st.kernel):
                k = st.kernel
                inv = invert_gather(k, ids)
                if inv is not None:
                    new.append(KernelStmt(inv))
                    continue
                ph = phase_split(k, ids)
                if ph is not None:
                    new += [KernelStmt(x) for x in ph]
                    continue
            new.append(st)
        blk.stmts = new
    return prog


def remaining_atomics(prog: kir.Program) -> list:
    return [k for k in prog.kernels() if _colliding(k)]
