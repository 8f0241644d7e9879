"""Recognising contractions: kernels of the form  out[.., m.., n..] (=|+=) f(sum_k A(b.., m.., k..) * B(b.., k.., n..)).

The reference has a matcher for its BLAS calls (anvil/backend/blas.py:113-198) that accepts exactly
`Load * Load` bodies with row-major operands. The matcher here works on dependence sets instead of
syntax, so that the products the optimizer really produces are all taken:

  * constant factors anywhere in the product are peeled into `alpha` (`0.125 * q * k`);
  * an operand is any expression over one side's index vars: an inlined `max(t, 0.0)`, a scaled
    load, a gathered row, a product of two loads that share their index vars;
  * index vars are classified by who uses them: A only -> M, B only -> N, both -> batch, and every
    reduction var is part of K. Several vars per class are flattened row-major in domain order, so
    the 4-d attention products and the summed-over-images convolution gradients are plain cases.

Everything else about the kernel (its statements, several stores, `+=`, in-place updates) stays in
the generated epilogue, so a match never changes what the kernel computes.
"""
from __future__ import annotations

from dataclasses import dataclass

from .. import kir
from ..kir import F32
from . import analysis as an


@dataclass
class Contraction:
    kernel: kir.Kernel
    mvars: list
    nvars: list
    kvars: list
    bvars: list
    a: kir.E               # operand expressions (products of the factors on each side)
    b: kir.E
    alpha: float
    a_kcontig: bool        # A is contiguous in memory along the innermost k var
    b_ncontig: bool        # B is contiguous along the innermost n var

    @property
    def M(self):
        return kir.prod(v.extent for v in self.mvars)

    @property
    def N(self):
        return kir.prod(v.extent for v in self.nvars)

    @property
    def K(self):
        return kir.prod(v.extent for v in self.kvars)

    @property
    def NB(self):
        return kir.prod(v.extent for v in self.bvars)

    @property
    def flops(self):
        return 2 * self.M * self.N * self.K * self.NB


def expr_vars(e: kir.E) -> set:
    out = set()
    for n in e.walk():
        if n.k in ("load", "index"):
            out.update(n.off.vars())
    return out


def _factors(e: kir.E, out: list):
    if e.k == "bin" and e.op == "mul" and e.dt == F32:
        _factors(e.a[0], out)
        _factors(e.a[1], out)
    else:
        out.append(e)


def _product(fs: list) -> kir.E:
    r = fs[0]
    for f in fs[1:]:
        r = kir.E("bin", F32, op="mul", a=[r, f])
    return r


def _contig(e: kir.E, v: kir.Var) -> bool:
    """Do the operand's loads walk memory with stride 1 along v?"""
    loads = [n for n in e.walk() if n.k == "load" and v in n.off.vars()]
    return bool(loads) and all(an.stride_of(n.off, v) == 1 for n in loads)


def match(k: kir.Kernel, min_flops: int = 1 << 21) -> Contraction | None:
    red = k.red
    if red is None or red.op != "sum" or red.body.dt != F32 or not k.domain:
        return None
    if k.uses_rand() or not an.parallel_safe(k):
        return None
    fs: list = []
    _factors(red.body, fs)
    alpha = 1.0
    ops = []
    for f in fs:
        if f.k == "const":
            alpha *= float(f.val)
        elif f.dt != F32:
            return None
        else:
            ops.append(f)
    if len(ops) < 2:
        return None
    K = set(red.vars)
    D = set(k.domain)
    deps = [expr_vars(f) for f in ops]
    if any(not (d & K) and not (d & D) for d in deps):
        return None                                    # a run-time scalar factor: leave it to the generic path
    if len(ops) > 5:
        return None
    # try every split of the factors into two sides (the first factor stays on side A) and keep the
    # first one that has M and N vars, no unused domain var, and both sides inside the reduction
    pick = None
    for mask in range(1, 1 << (len(ops) - 1)):
        side_b = [i + 1 for i in range(len(ops) - 1) if mask >> i & 1]
        side_a = [i for i in range(len(ops)) if i not in side_b]
        va = set().union(*[deps[i] for i in side_a])
        vb = set().union(*[deps[i] for i in side_b])
        if not (va & K) or not (vb & K):
            continue
        mvars = [v for v in k.domain if v in va and v not in vb]
        nvars = [v for v in k.domain if v in vb and v not in va]
        bvars = [v for v in k.domain if v in va and v in vb]
        if mvars and nvars and len(mvars) + len(nvars) + len(bvars) == len(k.domain):
            pick = (side_a, side_b, mvars, nvars, bvars)
            break
    if pick is None:
        return None
    side_a, side_b, mvars, nvars, bvars = pick
    kvars = list(red.vars)
    if kir.prod(v.extent for v in mvars) < 128 <= kir.prod(v.extent for v in nvars):
        # which factor is called A is arbitrary: the tiles are 128 rows of M by 64 or 128 columns of N,
        # so the short side goes to N
        side_a, side_b, mvars, nvars = side_b, side_a, nvars, mvars
    elif min(kir.prod(v.extent for v in mvars), kir.prod(v.extent for v in nvars)) >= 128:
        # both sides can be rows: let N run along the output's contiguous index, because the epilogue (and
        # the split-k finish) puts consecutive lanes on consecutive n — a weight gradient stored as
        # dW[n_features_in, n_features_out] with the factors the other way round had 32 sectors per store
        outs = [s_ for s_ in k.stmts if isinstance(s_, kir.Store)]
        if outs and outs[0].offset.is_plain() and outs[0].offset.coef(mvars[-1]) == 1 and outs[0].offset.coef(nvars[-1]) != 1:
            side_a, side_b, mvars, nvars = side_b, side_a, nvars, mvars
    c = Contraction(k, mvars, nvars, kvars, bvars, _product([ops[i] for i in side_a]),
                    _product([ops[i] for i in side_b]), alpha, False, False)
    if c.M < 32 or c.N < 32 or c.K < 8 or c.flops < min_flops:
        return None
    c.a_kcontig = _contig(c.a, kvars[-1])
    c.b_ncontig = _contig(c.b, nvars[-1])
    return c
