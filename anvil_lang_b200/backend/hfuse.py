"""Horizontal fusion of contractions: several products that share an operand, or add into one output, run as ONE
launch of the resident tensor-core template.

The resident template pays a fixed price per launch (about 3 us until its first stage is full, 3-5 us for the last
epilogue, and a partly empty last round of tiles). A transformer block has three products  h @ Wq, h @ Wk, h @ Wv  of
16384 x 512 x 512 each (128 tiles on 74 resident clusters: two rounds, the second 73 % full), their three weight
gradients  h^T @ dq ...  and the three products that add up to the gradient of h. Side by side they fill the rounds
and pay the fixed price once:

  * "ncat": consecutive, mutually independent products with the same A operand, the same M and K, and outputs as wide
            as whole tiles become one product whose N is the concatenation: tile columns [N0, N0 + N1) read the
            second product's B and run its statements;
  * "kcat": `C = A0 @ B0; C += A1 @ B1; C += A2 @ B2` becomes one product over the concatenated reduction index
            (the sums differ from the sequence of three by rounding only: one chain instead of three added).

Nothing changes in the IR: the group is a launch unit of the emitter (like a fused row group), and each kernel keeps
its own launcher for kernel-by-kernel runs.
"""
from __future__ import annotations

from .. import kir
from . import contraction as ct

TILE_N = 128                   # outputs side by side must each be whole tiles wide (256-wide tiles when all are multiples of 256)
BLOCK_K = 32


def _sig(e: kir.E, roles: dict):
    """Structure of an operand expression with its index vars replaced by their role ("m0", "k1", ...)."""
    if e.k == "load":
        terms = []
        for t, c in e.off.terms:
            if not isinstance(t, kir.Var) or t not in roles:
                return None
            terms.append((roles[t], c))
        return ("ld", e.buf.root.id, e.off.const, tuple(sorted(terms)))
    if e.k == "const":
        return ("c", repr(e.val))
    if e.k in ("un", "bin", "sel"):
        kids = tuple(_sig(x, roles) for x in e.a)
        return None if any(x is None for x in kids) else (e.k, e.op, kids)
    return None


def _roles(c) -> dict:
    r = {}
    for tag, vs in (("m", c.mvars), ("n", c.nvars), ("k", c.kvars), ("b", c.bvars)):
        for i, v in enumerate(vs):
            r[v] = f"{tag}{i}:{v.extent}"
    return r


def _independent(ks) -> bool:
    for i, a in enumerate(ks):
        aw = {b.id for b in a.writes()}
        ar = {b.id for b in a.reads()}
        for b in ks[i + 1:]:
            bw = {x.id for x in b.writes()}
            br = {x.id for x in b.reads()}
            if aw & (bw | br) or bw & ar:
                return False
    return True


def _plain_acc_store(k: kir.Kernel):
    """(buffer root, offset signature inputs) when the kernel's only statement stores its accumulator."""
    if len(k.stmts) != 1 or not isinstance(k.stmts[0], kir.Store) or k.stmts[0].value.k != "acc":
        return None
    return k.stmts[0]


def find_hgroups(kernels, eligible) -> list:
    """[(start, end, kind)] over a run of consecutive kernels. `eligible(contraction)`: takes the resident template."""
    cs = []
    for k in kernels:
        c = ct.match(k)
        cs.append(c if c is not None and not c.bvars and eligible(c) else None)
    out, i, n = [], 0, len(kernels)
    while i < n:
        c0 = cs[i]
        if c0 is None:
            i += 1
            continue
        a0 = _sig(c0.a, _roles(c0))
        # ---- same A, outputs side by side
        j = i + 1
        if a0 is not None and c0.N % TILE_N == 0:
            while j < n and cs[j] is not None and j - i < 4:
                c = cs[j]
                if (c.M, c.K, c.alpha, c.a_kcontig) != (c0.M, c0.K, c0.alpha, c0.a_kcontig) or c.N % TILE_N \
                        or ct._contig(c.b, c.kvars[-1]) != ct._contig(c0.b, c0.kvars[-1]) \
                        or [v.extent for v in c.mvars] != [v.extent for v in c0.mvars] \
                        or [v.extent for v in c.kvars] != [v.extent for v in c0.kvars] \
                        or _sig(c.a, _roles(c)) != a0 or not _independent(kernels[i:j + 1]):
                    break
                j += 1
        if j - i >= 2:
            out.append((i, j, "ncat"))
            i = j
            continue
        # ---- one output, reduction ranges end to end
        st0 = _plain_acc_store(kernels[i])
        j = i + 1
        if st0 is not None and c0.K % BLOCK_K == 0:
            r0 = _roles(c0)
            t0 = _sig(kir.E("load", kir.F32, buf=st0.buf, off=st0.offset), r0)
            while j < n and cs[j] is not None and j - i < 4 and t0 is not None:
                c, st = cs[j], _plain_acc_store(kernels[j])
                if st is None or not st.accumulate or (c.M, c.N, c.alpha, c.a_kcontig) != (c0.M, c0.N, c0.alpha, c0.a_kcontig) \
                        or c.K % BLOCK_K or ct._contig(c.b, c.kvars[-1]) != ct._contig(c0.b, c0.kvars[-1]) \
                        or [v.extent for v in c.mvars] != [v.extent for v in c0.mvars] \
                        or [v.extent for v in c.nvars] != [v.extent for v in c0.nvars] \
                        or _sig(kir.E("load", kir.F32, buf=st.buf, off=st.offset), _roles(c)) != t0:
                    break
                # its operands must not be something the group writes
                written = {st0.buf.root.id}
                if {b.id for b, _ in kernels[j].loads()} & written:
                    break
                j += 1
        if j - i >= 2:
            out.append((i, j, "kcat"))
            i = j
            continue
        i += 1
    return out
