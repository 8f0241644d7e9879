"""Recognising attention in the IR: the runs of kernels that csrc/anvil_attn_sm100.cuh executes as one launch.

Forward (anvil/prelude.anvil:28-32 `softmax` inside the idiom of examples/transformer.anvil:34-36), seven kernels:

    t8[bh, i, j]  = alpha * sum_e q[.., i, e] * k[.., j, e]         contraction
    s             = t8 + mask(i, j)                                elementwise, the only reader of t8
    t9[r]         = max_j s[r, j];   e = exp(s - t9);   t10[r] = sum_j e[r, j];   out = e / t10        (softmax)
    o[.., i, e]   = sum_j out[bh, i, j] * v[.., j, e]               contraction whose A operand is `out`

Backward, five kernels:

    dout = sum_e do[.., i, e] * v[.., j, e];   de = dout * (1 / t10[r])      contraction with two stores
    dt10[r] = sum_j dout * (-out / t10[r]);    de += dt10[r];    ds = de * e
    dq[.., i, e] = alpha * sum_j ds[bh, i, j] * k[.., j, e]                  contraction whose A operand is `ds`

A run is taken only when every tensor in between is dense [batch x heads, T, T] (or [batch x heads, T]) in row-major
order, T = 256 and the head width is 64 (the template's tile), and the tensors the fusion no longer writes (t8, s, t9 /
dout, de, dt10) are read by nobody else. Which of e, out, t10, ds are still written is decided by who reads them later.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from .. import kir
from ..kir import F32
from . import contraction as ct

T_TILE, DH_TILE = 256, 64


@dataclass
class AttnGroup:
    mode: int                       # 0 forward, 1 backward
    kernels: list
    c1: object                      # contraction of product 1
    c2: object                      # contraction of product 2
    nbh: int
    post_kernel: object = None      # forward: the elementwise kernel that makes the score from product 1 (mask)
    post_load: object = None        # ... and its load of product 1's result
    causal: bool = False
    bufs: dict = field(default_factory=dict)      # role -> root buffer: e, p (probabilities), sum, max, r (row result), scores..
    live: dict = field(default_factory=dict)      # role -> still read by somebody outside the group


def _dense_rows(off: kir.Affine, row_vars, j, T) -> bool:
    """offset == T * rowmajor(row_vars) + j (j may be None for a per-row scalar: offset == rowmajor(row_vars))."""
    if not off.is_plain() or off.const != 0:
        return False
    strides = kir.row_major_strides([v.extent for v in row_vars])
    scale = T if j is not None else 1
    want = {v: s * scale for v, s in zip(row_vars, strides) if v.extent > 1}
    if j is not None:
        want[j] = 1
    got = {t: c for t, c in off.terms if t.extent > 1}
    return got == want


def _strip(e: kir.E) -> kir.E:
    while e.k == "un" and e.op == "detach":
        e = e.a[0]
    while e.k == "let":
        e = e.let.value
    return e


def _single_store(k):
    st = [s for s in k.stmts if isinstance(s, kir.Store)]
    return st[0] if len(st) == 1 and not st[0].accumulate else None


def _is_load(e, root=None):
    e = _strip(e)
    return e.k == "load" and (root is None or e.buf.root is root)


def _product1(k, need_stores):
    c = ct.match(k)
    if c is None or len(c.mvars) != 1 or len(c.nvars) != 1 or len(c.kvars) != 1:
        return None
    if (c.mvars[0].extent, c.nvars[0].extent, c.kvars[0].extent) != (T_TILE, T_TILE, DH_TILE) or not c.bvars:
        return None
    if list(k.domain) != list(c.bvars) + [c.mvars[0], c.nvars[0]]:
        return None
    stores = [s for s in k.stmts if isinstance(s, kir.Store)]
    if len(stores) != need_stores or any(s.accumulate or not _dense_rows(s.offset, list(c.bvars) + [c.mvars[0]], c.nvars[0], T_TILE)
                                         for s in stores):
        return None
    if not ct._contig(c.a, c.kvars[0]) or not ct._contig(c.b, c.kvars[0]):
        return None                                  # both operands are read along the head width
    return c


def _product2(k, root):
    """A contraction over the keys whose A operand is exactly the dense row result `root`."""
    c = ct.match(k)
    if c is None or len(c.mvars) != 1 or len(c.nvars) != 1 or len(c.kvars) != 1 or not c.bvars:
        return None
    if (c.mvars[0].extent, c.nvars[0].extent, c.kvars[0].extent) != (T_TILE, DH_TILE, T_TILE):
        return None
    a = _strip(c.a)
    if a.k != "load" or a.buf.root is not root:
        return None
    # bvars in domain order must index the dense tensor like product 1 did
    if not _dense_rows(a.off, list(c.bvars) + [c.mvars[0]], c.kvars[0], T_TILE):
        return None
    if any(n.k == "load" and n.buf.root is root for st in k.stmts for n in st.value.walk()):
        return None
    return c


def _row_kernel(k, T):
    """(row vars, j) of a kernel over [rows, j] or a reduction over j with domain [rows]."""
    if k.red is not None:
        if len(k.red.vars) != 1 or k.red.vars[0].extent != T:
            return None
        return list(k.domain), k.red.vars[0]
    if not k.domain or k.domain[-1].extent != T:
        return None
    return list(k.domain[:-1]), k.domain[-1]


def _causal_mask(e: kir.E, load, i, j) -> bool:
    """value == load + (0.0 if j <= i else C) with C <= -1e8 (in either operand order)."""
    e = _strip(e)
    if e.k != "bin" or e.op != "add":
        return False
    for x, y in ((e.a[0], e.a[1]), (e.a[1], e.a[0])):
        x, y = _strip(x), _strip(y)
        if x is load and y.k == "sel":
            c, a, b = (_strip(z) for z in y.a)
            if c.k == "bin" and c.op == "le" and c.a[0].k == "index" and c.a[1].k == "index" \
                    and c.a[0].off == kir.Affine(0, [(j, 1)]) and c.a[1].off == kir.Affine(0, [(i, 1)]) \
                    and a.k == "const" and float(a.val) == 0.0 and b.k == "const" and float(b.val) <= -1e8:
                return True
    return False


def match_forward(ks, i0):
    if i0 + 7 > len(ks):
        return None
    k0, k1, k2, k3, k4, k5, k6 = ks[i0:i0 + 7]
    c1 = _product1(k0, 1)
    if c1 is None:
        return None
    st0 = _single_store(k0)
    if st0 is None or _strip(st0.value).k != "acc":
        return None
    t8 = st0.buf.root
    nbh = kir.prod(v.extent for v in c1.bvars)
    # the mask: elementwise over the same dense tensor, one load of t8, no other loads
    st1 = _single_store(k1)
    if k1.red is not None or st1 is None or len(k1.domain) < 3 or k1.uses_rand():
        return None
    i1, j1 = k1.domain[-2], k1.domain[-1]
    if (i1.extent, j1.extent) != (T_TILE, T_TILE) or kir.prod(v.extent for v in k1.domain[:-2]) != nbh:
        return None
    loads = [n for n in st1.value.walk() if n.k == "load"]
    if len(loads) != 1 or loads[0].buf.root is not t8 or not _dense_rows(loads[0].off, list(k1.domain[:-1]), j1, T_TILE) \
            or not _dense_rows(st1.offset, list(k1.domain[:-1]), j1, T_TILE):
        return None
    s = st1.buf.root
    # softmax: max, exp, sum, divide
    shapes = [_row_kernel(k, T_TILE) for k in (k2, k3, k4, k5)]
    if any(x is None for x in shapes) or any(kir.prod(v.extent for v in rv) != nbh * T_TILE for rv, _ in shapes):
        return None
    (r2, j2), (r3, j3), (r4, j4), (r5, j5) = shapes
    st2, st3, st4, st5 = (_single_store(k) for k in (k2, k3, k4, k5))
    if None in (st2, st3, st4, st5):
        return None
    if k2.red is None or k2.red.op != "max" or not _is_load(k2.red.body, s) or not _dense_rows(_strip(k2.red.body).off, r2, j2, T_TILE) \
            or _strip(st2.value).k != "acc" or not _dense_rows(st2.offset, r2, None, T_TILE):
        return None
    t9 = st2.buf.root
    v3 = _strip(st3.value)
    if k3.red is not None or v3.k != "un" or v3.op != "exp":
        return None
    d3 = _strip(v3.a[0])
    if d3.k != "bin" or d3.op != "sub" or not _is_load(d3.a[0], s) or not _is_load(d3.a[1], t9) \
            or not _dense_rows(_strip(d3.a[0]).off, r3, j3, T_TILE) or not _dense_rows(_strip(d3.a[1]).off, r3, None, T_TILE) \
            or not _dense_rows(st3.offset, r3, j3, T_TILE):
        return None
    e = st3.buf.root
    if k4.red is None or k4.red.op != "sum" or not _is_load(k4.red.body, e) or not _dense_rows(_strip(k4.red.body).off, r4, j4, T_TILE) \
            or _strip(st4.value).k != "acc" or not _dense_rows(st4.offset, r4, None, T_TILE):
        return None
    t10 = st4.buf.root
    v5 = _strip(st5.value)
    if k5.red is not None or v5.k != "bin" or v5.op != "div" or not _is_load(v5.a[0], e) or not _is_load(v5.a[1], t10) \
            or not _dense_rows(_strip(v5.a[0]).off, r5, j5, T_TILE) or not _dense_rows(_strip(v5.a[1]).off, r5, None, T_TILE) \
            or not _dense_rows(st5.offset, r5, j5, T_TILE):
        return None
    out = st5.buf.root
    c2 = _product2(k6, out)
    if c2 is None or kir.prod(v.extent for v in c2.bvars) != nbh:
        return None
    if len({t8.id, s.id, t9.id, e.id, t10.id, out.id}) != 6:
        return None
    g = AttnGroup(0, ks[i0:i0 + 7], c1, c2, nbh, k1, loads[0], _causal_mask(st1.value, loads[0], i1, j1))
    g.bufs = {"scores": t8, "masked": s, "max": t9, "e": e, "sum": t10, "r": out}
    return g


def match_backward(ks, i0):
    if i0 + 5 > len(ks):
        return None
    k0, k1, k2, k3, k4 = ks[i0:i0 + 5]
    c1 = _product1(k0, 2)
    if c1 is None:
        return None
    nbh = kir.prod(v.extent for v in c1.bvars)
    stores = [s for s in k0.stmts if isinstance(s, kir.Store)]
    v_dout, v_de = _strip(stores[0].value), _strip(stores[1].value)
    if v_dout.k != "acc" or v_de.k != "bin" or v_de.op != "mul":
        return None
    dout, de = stores[0].buf.root, stores[1].buf.root
    rows0 = list(c1.bvars) + [c1.mvars[0]]
    inv = None
    for x, y in ((v_de.a[0], v_de.a[1]), (v_de.a[1], v_de.a[0])):
        x, y = _strip(x), _strip(y)
        if x.k == "acc" and y.k == "bin" and y.op == "div" and _strip(y.a[0]).k == "const" and float(_strip(y.a[0]).val) == 1.0 \
                and _is_load(y.a[1]) and _dense_rows(_strip(y.a[1]).off, rows0, None, T_TILE):
            inv = _strip(y.a[1]).buf.root
    if inv is None:
        return None
    t10 = inv
    shapes = [_row_kernel(k, T_TILE) for k in (k1, k2)]
    if any(x is None for x in shapes) or any(kir.prod(v.extent for v in rv) != nbh * T_TILE for rv, _ in shapes):
        return None
    (r1, j1), (r2, j2) = shapes
    # dt10[r] = sum_j dout * (neg(out) / t10[r])
    st1 = _single_store(k1)
    if k1.red is None or k1.red.op != "sum" or st1 is None or _strip(st1.value).k != "acc" or not _dense_rows(st1.offset, r1, None, T_TILE):
        return None
    b = _strip(k1.red.body)
    out = None
    if b.k == "bin" and b.op == "mul":
        for x, y in ((b.a[0], b.a[1]), (b.a[1], b.a[0])):
            x, y = _strip(x), _strip(y)
            if _is_load(x, dout) and _dense_rows(x.off, r1, j1, T_TILE) and y.k == "bin" and y.op == "div" \
                    and _strip(y.a[0]).k == "un" and _strip(y.a[0]).op == "neg" and _is_load(_strip(y.a[0]).a[0]) \
                    and _dense_rows(_strip(_strip(y.a[0]).a[0]).off, r1, j1, T_TILE) \
                    and _is_load(y.a[1], t10) and _dense_rows(_strip(y.a[1]).off, r1, None, T_TILE):
                out = _strip(_strip(y.a[0]).a[0]).buf.root
    if out is None:
        return None
    dt10 = st1.buf.root
    # de[r, j] += dt10[r]
    st2 = [s for s in k2.stmts if isinstance(s, kir.Store)]
    if k2.red is not None or len(st2) != 1 or not st2[0].accumulate or st2[0].buf.root is not de \
            or not _dense_rows(st2[0].offset, r2, j2, T_TILE) or not _is_load(st2[0].value, dt10) \
            or not _dense_rows(_strip(st2[0].value).off, r2, None, T_TILE):
        return None
    # ds = de * e (any dense factorisation of the domain)
    st3 = _single_store(k3)
    if k3.red is not None or st3 is None or k3.out_numel() != nbh * T_TILE * T_TILE:
        return None
    ident = kir.Affine(0, list(zip(k3.domain, kir.row_major_strides([v.extent for v in k3.domain]))))
    v3 = _strip(st3.value)
    if st3.offset != ident or v3.k != "bin" or v3.op != "mul":
        return None
    e = None
    for x, y in ((v3.a[0], v3.a[1]), (v3.a[1], v3.a[0])):
        if _is_load(x, de) and _strip(x).off == ident and _is_load(y) and _strip(y).off == ident:
            e = _strip(y).buf.root
    if e is None:
        return None
    ds = st3.buf.root
    c2 = _product2(k4, ds)
    if c2 is None or kir.prod(v.extent for v in c2.bvars) != nbh:
        return None
    if len({dout.id, de.id, dt10.id, ds.id, out.id, e.id, t10.id}) != 7:
        return None
    g = AttnGroup(1, ks[i0:i0 + 5], c1, c2, nbh)
    g.bufs = {"dp": dout, "de": de, "dsum": dt10, "r": ds, "p": out, "e": e, "sum": t10}
    return g


def find_attention(ks, readers, host_read, causal_e: set):
    """[(start, end, AttnGroup)] in a run of consecutive kernels. `readers`: root id -> ids of the kernels that read it;
    `causal_e`: root ids of exp tensors that a causal forward group wrote (zero above the diagonal); forward groups
    found here are added to it."""
    out, i = [], 0
    while i < len(ks):
        g = match_forward(ks, i) or match_backward(ks, i)
        if g is not None:
            inside = {k.id for k in g.kernels}

            def outside(root):
                return root.id in host_read or not (readers.get(root.id, set()) <= inside)
            dead_roles = ("scores", "masked", "max") if g.mode == 0 else ("dp", "de", "dsum")
            if any(outside(g.bufs[r]) for r in dead_roles if r != "max") \
                    or any(kk.id not in inside and g.bufs[r] in kk.writes() for r in g.bufs for kk in ks[i:i + len(g.kernels)]):
                g = None
            else:
                g.live = {r: outside(b) for r, b in g.bufs.items()}
                if g.mode == 0 and g.causal:
                    causal_e.add(g.bufs["e"].id)
                if g.mode == 1:
                    g.causal = g.bufs["e"].id in causal_e
        if g is None:
            i += 1
            continue
        out.append((i, i + len(g.kernels), g))
        i += len(g.kernels)
    return out
