"""Convolutions as implicit products: the im2col tensor and its gradient are never materialised.

The reference lowers `Conv2d` through an explicit window tensor (anvil/prelude.anvil:84-87):

    patches[n, i, j, c, u, v] = x[n, c, i + u, j + v]                    (kept: its loads are not injective,
    out[n, o, ij]   = sum_cuv patches[n, ij, cuv] * W[o, cuv] + b[o]      anvil/optimize.py:674-675)
    dW[o, cuv]      = sum_{n, ij} dout[n, o, ij] * patches[n, ij, cuv]
    dpatches[n, ij, cuv] = sum_o dout[n, o, ij] * W[o, cuv]
    dx = 0;  dx[n, c, i + u, j + v] += dpatches[n, i, j, c, u, v]        (col2im)

so every step writes the 9x larger window tensor, reads it twice, writes its gradient and scatters it. The contraction
templates evaluate their operands through generated functors, so a gather costs nothing extra there. Two IR rewrites:

  * `inline_window_copies`: a kernel that only copies elements into a temporary (any affine gather pattern) is
    substituted into the kernels that read the temporary; index variables that the readers had collapsed (`ij`,
    `cuv`) are split back into the copy's own dimensions first, because the composed offset is affine only in those.
    When every reader has been rewritten the copy disappears, and with it the tensor.

  * `fold_product_scatters`: `T = product; D = 0; D[affine scatter] += T` becomes ONE reduction over D's own
    elements: each output coordinate that two variables reach (y = i + u) keeps the output coordinate, turns the short
    variable into a reduction variable (u), substitutes the long one (i = y - u) and guards the term with its range
    (0 <= y - u < extent), so that  dx[n, c, y, x] = sum_{o, u, v} [in range] dout[n, o, y - u, x - v] * W[o, c, u, v].
    It is a contraction with a guarded operand; nothing is scattered, no element is added to twice from different
    threads, and the order of the additions is fixed.

Both are exact re-associations only in the second case (the sum over o, u, v is added in one chain instead of first
over o and then over the window): results agree to rounding, not bit for bit.
"""
from __future__ import annotations

import itertools

from .. import kir
from ..kir import F32, I32, Affine, E, Kernel, KernelStmt, Let, Reduction, Store, Var
from . import analysis as an


# ----------------------------------------------------------------------------- generic rewriting
def subst_affine(a: Affine, m: dict) -> Affine:
    """`m`: Var -> list of (Var, coefficient) (an affine combination without constant), identity for other vars."""
    const, order, terms = a.const, [], {}

    def add(t, c):
        if t not in terms:
            order.append(t)
            terms[t] = 0
        terms[t] += c
    for t, c in a.terms:
        if isinstance(t, Var) and t in m:
            for nv, nc in m[t]:
                add(nv, c * nc)
        elif isinstance(t, kir.Gather):
            add(kir.Gather(t.buf, subst_affine(t.offset, m), t.bound, t.where, t.lo, t.hi), c)
        else:
            add(t, c)
    return Affine(const, [(t, terms[t]) for t in order])


def rewrite_expr(e: E, m: dict, load_hook, memo: dict, lets: dict) -> E:
    hit = memo.get(id(e))
    if hit is not None:
        return hit
    if e.k == "load":
        off = subst_affine(e.off, m)
        r = load_hook(e.buf, off, e.dt) if load_hook else None
        if r is None:
            r = E("load", e.dt, buf=e.buf, off=off)
    elif e.k == "index":
        r = E("index", I32, off=subst_affine(e.off, m))
    elif e.k == "let":
        r = E("let", e.dt, let=lets[e.let.id])
    elif e.a:
        r = E(e.k, e.dt, op=e.op, a=[rewrite_expr(x, m, load_hook, memo, lets) for x in e.a])
    else:
        r = e
    memo[id(e)] = r
    return r


def rewrite_kernel(k: Kernel, m: dict, domain, red_vars, ids, load_hook=None, name=None) -> Kernel:
    memo, lets, stmts = {}, {}, []
    red = None
    if k.red is not None:
        red = Reduction(list(red_vars), k.red.op, rewrite_expr(k.red.body, m, load_hook, memo, lets))
    for st in k.stmts:
        if isinstance(st, Let):
            nl = Let(next(ids), st.name, rewrite_expr(st.value, m, load_hook, memo, lets))
            lets[st.id] = nl
            stmts.append(nl)
        else:
            stmts.append(Store(st.buf, subst_affine(st.offset, m), rewrite_expr(st.value, m, load_hook, memo, lets), st.accumulate))
    return Kernel(next(ids), name or k.name, k.label, list(domain), stmts, red, k.rand_base, k.src)


def _ids(prog):
    return itertools.count(max([b.id for b in prog.buffers] + [k.id for k in prog.kernels()]
                               + [v.id for k in prog.kernels() for v in list(k.domain) + (list(k.red.vars) if k.red else [])]) + 20000)


def _dims_of_identity(k: Kernel, st: Store):
    """If `st` writes its tensor densely in the order of k's domain (offset = row-major identity of the domain, all
    of the tensor covered), the list of (var, stride, extent); else None."""
    if st.accumulate or not st.offset.is_plain() or st.offset.const != 0:
        return None
    strides = kir.row_major_strides([v.extent for v in k.domain])
    dims = []
    for v, s in zip(k.domain, strides):
        if v.extent > 1 and st.offset.coef(v) != s:
            return None
        dims.append((v, s, v.extent))
    if k.out_numel() != st.buf.root.numel:
        return None
    return dims


def _split_plan(off: Affine, dims):
    """How the vars of `off` (an offset into a tensor whose dense dims are `dims`: (producer var, stride, extent))
    map onto those dims: {var of off: [producer vars it spans, outermost first]} or None. A var spans dims d1..d2 when
    its coefficient is the stride of d2 and its extent the product of their extents."""
    if not off.is_plain() or off.const != 0:
        return None
    live = [d for d in dims if d[2] > 1]
    plan, covered = {}, set()
    for v, c in off.var_terms():
        if v.extent <= 1:
            continue
        hit = None
        for hi in range(len(live)):
            if live[hi][1] != c:
                continue
            ext, lo = 1, hi
            while lo >= 0:
                ext *= live[lo][2]
                if ext == v.extent:
                    hit = (lo, hi)
                    break
                if ext > v.extent:
                    break
                lo -= 1
            break
        if hit is None:
            return None
        span = live[hit[0]:hit[1] + 1]
        if any(d[0] in covered for d in span):
            return None
        covered |= {d[0] for d in span}
        plan[v] = [d[0] for d in span]
    if covered != {d[0] for d in live}:
        return None
    return plan


# ----------------------------------------------------------------------------- copies into readers
def _copy_kernel(k: Kernel):
    """(tensor, dims, value) when k only gathers elements into a temporary it covers densely."""
    if k.red is not None or len(k.stmts) != 1 or k.uses_rand() or not isinstance(k.stmts[0], Store):
        return None
    st = k.stmts[0]
    if st.buf.root.kind != "temp" or st.buf.dtype != F32:
        return None
    dims = _dims_of_identity(k, st)
    if dims is None:
        return None
    if st.value.k != "load" or not st.value.off.is_plain():
        return None                                      # only pure copies: anything computed is worth computing once
    if an.injective_over(st.value.off, k.domain):
        return None                                      # a plain permutation: the optimizer's business, nothing to gain
    return st.buf.root, dims, st.value


def inline_window_copies(prog: kir.Program, host_reads: set) -> int:
    ids = _ids(prog)
    done = 0
    for blk in kir.walk_blocks(prog.main):
        changed = True
        while changed:
            changed = False
            for pi, pst in enumerate(blk.stmts):
                if not isinstance(pst, KernelStmt):
                    continue
                info = _copy_kernel(pst.kernel)
                if info is None:
                    continue
                T, dims, value = info
                if T.id in host_reads:
                    continue
                P = pst.kernel
                p_reads = {b.id for b in P.reads()}
                here = [qi for qi, q in enumerate(blk.stmts)
                        if isinstance(q, KernelStmt) and q.kernel is not P and T in q.kernel.reads()]
                everywhere = [k for k in prog.kernels() if k is not P and T in k.reads()]
                writers = [k for k in prog.kernels() if k is not P and T in k.writes()]
                if writers or not here or len(here) != len(everywhere) or min(here) < pi:
                    continue
                # every reader sits in this block after P; nothing in between may write what P reads
                ok, new = True, {}
                for qi in here:
                    for mid in blk.stmts[pi + 1:qi]:
                        if not isinstance(mid, KernelStmt) or {b.id for b in mid.kernel.writes()} & p_reads:
                            ok = False
                    nk = _inline_into(blk.stmts[qi].kernel, P, T, dims, value, ids) if ok else None
                    if nk is None:
                        ok = False
                        break
                    new[qi] = nk
                if not ok:
                    continue
                for qi, nk in new.items():
                    blk.stmts[qi] = KernelStmt(nk)
                del blk.stmts[pi]
                done += 1
                changed = True
                break
    return done


def _inline_into(C: Kernel, P: Kernel, T, dims, value, ids) -> Kernel | None:
    """C with its loads of T replaced by P's value; C's vars that span several of T's dims are split."""
    offs = [n.off for e in C.exprs() for n in e.walk() if n.k == "load" and n.buf.root is T]
    if not offs or any(s.buf.root is T for s in C.stores):
        return None
    plans = [_split_plan(o, dims) for o in offs]
    if any(p is None for p in plans):
        return None
    plan = plans[0]
    for p in plans[1:]:                                  # all loads of T must agree on how C's vars map
        if {v: [d.id for d in ds] for v, ds in p.items()} != {v: [d.id for d in ds] for v, ds in plan.items()}:
            return None
    m, fresh_for = {}, {}                                # C var -> [(new var, coef)], producer var -> new var of C
    new_domain, new_red = [], []
    for group, out in ((C.domain, new_domain), (C.red.vars if C.red else [], new_red)):
        for v in group:
            if v in plan and len(plan[v]) > 1:
                parts = [Var(next(ids), pv.name, pv.extent) for pv in plan[v]]
                strides = kir.row_major_strides([p.extent for p in parts])
                m[v] = list(zip(parts, strides))
                out.extend(parts)
                for pv, nv in zip(plan[v], parts):
                    fresh_for[pv] = nv
            else:
                out.append(v)
                if v in plan:
                    fresh_for[plan[v][0]] = v
    p_map = {pv: [(fresh_for[pv], 1)] for pv, _, ext in dims if ext > 1}
    for pv, _, ext in dims:
        if ext <= 1:
            p_map[pv] = []                               # a dimension of extent 1 contributes nothing

    def hook(buf, off, dt):
        if buf.root is not T:
            return None
        return rewrite_expr(value, p_map, None, {}, {})
    nk = rewrite_kernel(C, m, new_domain, new_red, ids, hook)
    if not an.parallel_safe(nk) and an.parallel_safe(C):
        return None
    return nk


# ----------------------------------------------------------------------------- product + zero + scatter -> one reduction
def _scatter_kernel(k: Kernel):
    """(target tensor, scatter offset, source tensor, source offset) of `D[scatter] += T[offset]`."""
    if k.red is not None or len(k.stmts) != 1 or not isinstance(k.stmts[0], Store) or k.uses_rand():
        return None
    st = k.stmts[0]
    if not st.accumulate or st.value.k != "load" or not st.offset.is_plain() or not st.value.off.is_plain():
        return None
    if st.buf.dtype != F32 or st.offset.const != 0:
        return None
    return st.buf.root, st.offset, st.value.buf.root, st.value.off


def _is_zero_fill(k: Kernel, D) -> bool:
    if k.red is not None or len(k.stmts) != 1 or not isinstance(k.stmts[0], Store):
        return False
    st = k.stmts[0]
    return st.buf.root is D and st.value.k == "const" and float(st.value.val) == 0.0 and an.covers(k, st)


def fold_product_scatters(prog: kir.Program, host_reads: set) -> int:
    ids = _ids(prog)
    done = 0
    for blk in kir.walk_blocks(prog.main):
        si = 0
        while si < len(blk.stmts):
            st = blk.stmts[si]
            info = _scatter_kernel(st.kernel) if isinstance(st, KernelStmt) else None
            if info is None:
                si += 1
                continue
            D, scatter, T, t_off = info
            S = st.kernel
            gi = next((i for i in range(si - 1, -1, -1) if isinstance(blk.stmts[i], KernelStmt) and T in blk.stmts[i].kernel.writes()), None)
            zi = next((i for i in range(si - 1, -1, -1) if isinstance(blk.stmts[i], KernelStmt) and D in blk.stmts[i].kernel.writes()), None)
            if gi is None or zi is None or T.id in host_reads or T.kind not in ("temp", "grad"):
                si += 1
                continue
            G, Z = blk.stmts[gi].kernel, blk.stmts[zi].kernel
            others = [k for k in prog.kernels() if k not in (G, S) and (T in k.reads() or T in k.writes())]
            R = None if others or not _is_zero_fill(Z, D) else _fold(G, S, D, scatter, T, t_off, ids)
            if R is None:
                si += 1
                continue
            # R runs where S ran; between G and S nothing may write what G reads, between Z and S nothing may touch D
            g_reads = {b.id for b in G.reads()}
            lo = min(gi, zi)
            clean = True
            for i in range(lo + 1, si):
                if i in (gi, zi):
                    continue
                mid = blk.stmts[i]
                if not isinstance(mid, KernelStmt):
                    clean = False
                    break
                w = {b.id for b in mid.kernel.writes()}
                r = {b.id for b in mid.kernel.reads()}
                if (i > gi and w & g_reads) or (i > zi and D.id in (w | r)):
                    clean = False
                    break
            if not clean:
                si += 1
                continue
            blk.stmts[si] = KernelStmt(R)
            for i in sorted((gi, zi), reverse=True):
                del blk.stmts[i]
            si -= 1                                      # two statements before `si` are gone, one took its place
            done += 1
    return done


def _fold(G: Kernel, S: Kernel, D, scatter: Affine, T, t_off: Affine, ids) -> Kernel | None:
    if G.red is None or G.red.op != "sum" or len(G.stmts) != 1 or G.uses_rand():
        return None
    gst = G.stmts[0]
    if not isinstance(gst, Store) or gst.buf.root is not T or gst.value.k != "acc":
        return None
    g_dims = _dims_of_identity(G, gst)
    if g_dims is None:
        return None
    # T's dense dims in S's own vars: S reads T through an offset that must itself be a dense identity-like map
    s_dims = []
    strides_T = sorted(((c, v) for v, c in t_off.var_terms() if v.extent > 1), key=lambda x: -x[0])
    reach = 1
    for c, v in reversed(strides_T):
        if c != reach:
            return None
        reach *= v.extent
    if reach != T.numel or t_off.const != 0:
        return None
    s_dims = [(v, c, v.extent) for c, v in strides_T]              # outermost first
    # map G's domain vars onto S's vars through T's layout
    plan = _split_plan(gst.offset, s_dims)
    if plan is None:
        return None
    # D's own dims from its shape; which S vars reach each
    d_strides = kir.row_major_strides(D.shape)
    by_dim = {i: [] for i in range(len(D.shape))}
    for v, c in scatter.var_terms():
        if v.extent <= 1:
            continue
        if c not in d_strides:
            return None
        by_dim[d_strides.index(c)].append(v)
    out_vars, m_s, guards, extra_red = [], {}, [], []
    for di, ext in enumerate(D.shape):
        vs = sorted(by_dim[di], key=lambda v: -v.extent)
        y = Var(next(ids), f"y{di}", ext)
        out_vars.append(y)
        if not vs:
            if ext > 1:
                return None                              # an output coordinate nothing reaches: not a plain window scatter
            continue
        if sum(v.extent - 1 for v in vs) + 1 != ext:
            return None
        long_v, shorts = vs[0], vs[1:]
        combo = [(y, 1)]
        for sv in shorts:
            nv = Var(next(ids), sv.name, sv.extent)
            extra_red.append(nv)
            m_s[sv] = [(nv, 1)]
            combo.append((nv, -1))
        m_s[long_v] = combo
        if shorts:
            guards.append((Affine(0, combo), long_v.extent))
    for v in S.domain:
        if v.extent <= 1:
            m_s[v] = []
        elif v not in m_s:
            return None
    # G's vars -> S's vars (splitting collapsed ones) -> output / reduction vars
    m_g = {}
    for gv in G.domain:
        if gv.extent <= 1:
            m_g[gv] = []
            continue
        parts = plan.get(gv)
        if parts is None:
            return None
        strides = kir.row_major_strides([p.extent for p in parts])
        combo = []
        for pv, s in zip(parts, strides):
            combo += [(nv, s * c) for nv, c in m_s[pv]]
        m_g[gv] = combo
    red_vars = [Var(next(ids), v.name, v.extent) for v in G.red.vars]
    for old, new in zip(G.red.vars, red_vars):
        m_g[old] = [(new, 1)]
    body = rewrite_expr(G.red.body, m_g, None, {}, {})
    cond = None
    for aff, ext in guards:                              # 0 <= y - u < extent
        ix = E("index", I32, off=aff)
        for op, bound in (("ge", 0), ("lt", ext)):
            c = E("bin", F32, op=op, a=[ix, E("const", I32, val=bound)])
            cond = c if cond is None else E("bin", F32, op="and", a=[cond, c])
    if cond is not None:
        body = _guard_first_factor(body, cond, set(extra_red) | set(out_vars))
        if body is None:
            return None
    ident = Affine(0, list(zip(out_vars, d_strides)))
    return Kernel(next(ids), f"{G.name}+{S.name}", f"{G.label}+gathered", out_vars, [Store(D, ident, E("acc", F32), False)],
                  Reduction(red_vars + extra_red, "sum", body), None, G.src)


def _guard_first_factor(body: E, cond: E, guarded_vars: set) -> E | None:
    """The product with every factor that depends on a guarded index wrapped as `factor if in range else 0`:
    the product stays a product (so the contraction matcher still sees it), and an out-of-range load is never made."""
    from .contraction import _factors, _product, expr_vars
    fs: list = []
    _factors(body, fs)
    hit = False
    out = []
    for f in fs:
        if f.k != "const" and any(n.k == "load" and _reaches(n.off, cond) for n in f.walk()):
            out.append(E("sel", F32, a=[cond, f, E("const", F32, val=0.0)]))
            hit = True
        else:
            out.append(f)
    return _product(out) if hit else None


def _reaches(off: Affine, cond: E) -> bool:
    """Does this offset use a (negative) substituted coordinate that the guard talks about?"""
    neg = {t for t, c in off.terms if isinstance(t, Var) and c < 0}
    return bool(neg)


def make_implicit(prog: kir.Program, host_reads: set) -> int:
    """Both rewrites, in place; returns how many tensors disappeared. Idempotent."""
    return inline_window_copies(prog, host_reads) + fold_product_scatters(prog, host_reads)
