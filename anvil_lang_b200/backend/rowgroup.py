"""Row-group fusion: runs of kernels that all work row by row become ONE kernel.

The optimizer leaves `softmax` as four kernels (row max, exp, row sum, divide), `layer_norm` as three
and their gradients as three to six (anvil/prelude.anvil:28-43; anvil/optimize.py limits fusion to
kernels with the same domain). Each of them streams the same R x N tensor through HBM again. Here a
run of consecutive kernels is fused when every kernel is either

  * a row reduction:  out[r] = REDUCE_j f(r, j)   (domain [r], one reduction var j of extent N), or
  * a row-wise map:   out[r, j] = f(r, j)         (domain [r, j], or the collapsed form [v] with
                                                   v = r * N + j),

with affine offsets only. T = N / E threads own one row (E = 4 .. 16 elements each, in 128-bit groups
that are contiguous across threads), keep every row vector they produce in registers, combine their
partial results with a fixed shuffle / shared-memory tree, and go through the kernels in program
order. A tensor that a later kernel of the group reads at the element this thread wrote is taken
from the register instead of memory; a tensor that nothing outside the group ever reads is not
stored at all. Kernels keep their statement-level semantics (several stores, `+=`, in-place updates).

Legality (checked in `extend`): a tensor written inside the group may only be read, inside the group,
at exactly the element (or row) the writer's thread owns; anything else needs a grid-wide barrier
and ends the group.
"""
from __future__ import annotations

from dataclasses import dataclass

from .. import kir
from ..kir import F32
from . import analysis as an

THREADS = 256
RED_OPS = ("sum", "max", "min", "prod")


@dataclass
class RowForm:
    kernel: kir.Kernel
    kind: str                   # "red" | "map"
    rowvar: object              # Var or None (a single row)
    jvar: object                # Var along the row; for the collapsed form the one flat var
    R: int
    N: int
    collapsed: bool = False

    def canon(self, off: kir.Affine):
        """(coefficient of the row index, coefficient of j, constant) of an offset."""
        if self.collapsed:
            c = off.coef(self.jvar)
            return (c * self.N, c, off.const)
        a = off.coef(self.rowvar) if self.rowvar is not None else 0
        return (a, off.coef(self.jvar), off.const)


def _plain(k: kir.Kernel) -> bool:
    return all(a.is_plain() for a in k.offsets())


def row_form(k: kir.Kernel, N_hint: int | None = None) -> RowForm | None:
    if k.uses_rand() or not _plain(k) or not an.parallel_safe(k) or k.rand_base is not None:
        return None
    if any(n.k == "index" for e in k.exprs() for n in e.walk()):
        return None
    if k.red is not None:
        if k.red.op not in RED_OPS or k.red.body.dt != F32 or len(k.red.vars) != 1 or len(k.domain) > 1:
            return None
        j = k.red.vars[0]
        row = k.domain[0] if k.domain else None
        for n in k.red.body.walk():
            if n.k == "load" and j in n.off.vars() and n.off.coef(j) != 1:
                return None
        if any(s.buf.dtype != F32 for s in k.stores):
            return None
        return RowForm(k, "red", row, j, row.extent if row is not None else 1, j.extent)
    if any(s.buf.dtype != F32 for s in k.stores) or any(n.k == "load" and n.dt != F32 for e in k.exprs() for n in e.walk()):
        return None
    if len(k.domain) == 2:
        row, j = k.domain
        if any(a.coef(j) not in (0, 1) for a in k.offsets()):
            return None
        return RowForm(k, "map", row, j, row.extent, j.extent)
    if len(k.domain) == 1 and N_hint:
        v = k.domain[0]
        if v.extent % N_hint or any(a.coef(v) not in (0, 1) for a in k.offsets()):
            return None
        if any(a.coef(v) == 0 for a in k.offsets()):
            return None                                  # a scalar broadcast: rows are not separable here
        return RowForm(k, "map", None, v, v.extent // N_hint, N_hint, collapsed=True)
    return None


def threads_per_row(N: int) -> int | None:
    """T threads per row, E = N / T elements each (a multiple of 4, at most 16)."""
    for T in (32, 64, 128, 256):
        if N % T == 0 and (N // T) % 4 == 0 and N // T <= 16:
            return T
    return None


class Group:
    def __init__(self):
        self.forms: list[RowForm] = []
        self.writes: dict = {}          # root id -> set of canon keys written
        self.reads: dict = {}           # root id -> set of canon keys read

    @property
    def R(self):
        return self.forms[0].R

    @property
    def N(self):
        return self.forms[0].N

    def accesses(self, f: RowForm):
        k = f.kernel
        rd = [(b.root.id, f.canon(off)) for b, off in k.loads()]
        rd += [(s.buf.root.id, f.canon(s.offset)) for s in k.stores if s.accumulate]
        wr = [(s.buf.root.id, f.canon(s.offset)) for s in k.stores]
        return rd, wr

    def extend(self, f: RowForm) -> bool:
        if self.forms and (f.R != self.R or f.N != self.N):
            return False
        rd, wr = self.accesses(f)
        for root, key in rd:                             # read-after-write inside the group: same element only
            if root in self.writes and self.writes[root] != {key}:
                return False
        for root, key in wr:
            if root in self.reads and self.reads[root] != {key}:
                return False                             # write-after-read of other elements
            if root in self.writes and self.writes[root] != {key}:
                return False
            if key[1] not in (0, 1):
                return False
        own_w = {}
        for root, key in wr:
            own_w.setdefault(root, set()).add(key)
        for root, key in rd:                             # a kernel reading what it writes itself: same element
            if root in own_w and own_w[root] != {key}:
                return False
        self.forms.append(f)
        for root, key in rd:
            self.reads.setdefault(root, set()).add(key)
        for root, key in wr:
            self.writes.setdefault(root, set()).add(key)
        return True

    def worthwhile(self) -> bool:
        return len(self.forms) >= 2 and any(f.kind == "red" for f in self.forms) and threads_per_row(self.N) is not None


def find_groups(kernels: list[kir.Kernel]) -> list[tuple[int, int]]:
    """Index ranges [start, end) of fusable runs inside a run of consecutive kernels."""
    out = []
    i = 0
    n = len(kernels)
    while i < n:
        f0 = row_form(kernels[i])
        if f0 is None and i + 1 < n:                     # a collapsed map right before a row kernel
            nxt = row_form(kernels[i + 1])
            if nxt is not None:
                f0 = row_form(kernels[i], nxt.N)
                if f0 is not None and f0.R != nxt.R:
                    f0 = None
        if f0 is None:
            i += 1
            continue
        g = Group()
        g.extend(f0)
        j = i + 1
        while j < n:
            f = row_form(kernels[j], g.N)
            if f is None or not g.extend(f):
                break
            j += 1
        # drop trailing maps that gain nothing? keep them: they reuse registers
        if g.worthwhile():
            out.append((i, j))
            i = j
        else:
            i += 1
    return out
