"""Static questions about a kernel that decide how it may be scheduled on the device.

`parallel_safe` restates the reference's rule for when every output element may run in its own
thread (anvil/backend/cuda.py:380-395, with `injective_over` :618-633 and `kernel_loads` :597-615).
The rest (contiguity, vector width, arena plan) has no reference counterpart: the reference always
runs one thread per output element with a scalar loop.
"""
from __future__ import annotations

from .. import kir

ALIGN = 256                  # arena alignment of every buffer, bytes


def injective_over(off: kir.Affine, vars_) -> bool:
    """Different values of `vars_` reach different offsets (mixed-radix argument: sorted by stride,
    each stride must exceed the span of all smaller ones). Every var of extent > 1 must appear."""
    items = []
    for v in vars_:
        if v.extent <= 1:
            continue
        c = off.coef(v)
        if c == 0:
            return False
        items.append((abs(c), v.extent))
    reach = 0
    for c, n in sorted(items):
        if c <= reach:
            return False
        reach += c * (n - 1)
    return True


def parallel_safe(k: kir.Kernel) -> bool:
    """Can every output element run in its own thread, in any order?"""
    written = {s.buf.root for s in k.stores}
    for s in k.stores:
        if s.accumulate:
            continue                                 # an atomic (or exclusive) add
        if s.offset.gathers():
            return False                             # duplicate indices: the last write wins
        if not injective_over(s.offset, k.domain):
            return False                             # several elements write one place
    for buf, off in k.loads():
        if buf.root in written:
            same = [s for s in k.stores if s.buf.root is buf.root]
            if any(s.accumulate or s.offset != off for s in same):
                return False                         # reads what other elements write
    return True


def exclusive_store(k: kir.Kernel, s: kir.Store) -> bool:
    """An accumulating store that no two output elements share: a plain read-modify-write. A gathered
    index whose checked range fits under the next larger stride (`out[10 * i + y[i]]`, y in [0, 10))
    counts as one more digit of the mixed-radix argument."""
    if s.offset.scalars():
        return False
    items = []
    for v in k.domain:
        if v.extent <= 1:
            continue
        c = s.offset.coef(v)
        if c == 0:
            return False
        items.append((abs(c), v.extent))
    for g, c in s.offset.gathers():
        if c == 0 or g.hi <= g.lo:
            return False
        items.append((abs(c), g.hi - g.lo))
    reach = 0
    for c, n in sorted(items):
        if c <= reach:
            return False
        reach += c * (n - 1)
    return True


def stride_of(off: kir.Affine, v: kir.Var) -> int | None:
    """Coefficient of `v` in `off`, or None when `v` also steers a gathered index."""
    for g, _ in off.gathers():
        if v in g.offset.vars():
            return None
    return off.coef(v)


def aligned4(off: kir.Affine, v: kir.Var) -> bool:
    """With `v` a multiple of 4, is the element offset a multiple of 4 (16-byte aligned access)?
    Needs every other contribution to be a multiple of 4: constants, other strides, and the
    coefficients of run-time terms."""
    if off.const % 4:
        return False
    for t, c in off.terms:
        if t is v:
            continue
        if c % 4:
            return False
    return True


def offset_fits_i32(off: kir.Affine) -> bool:
    b = off.bounds()
    return b is not None and -(1 << 31) < b[0] and b[1] < (1 << 31) - 1


def hot_loop(prog: kir.Program):
    """The `For` whose body does the most kernel work: the training loop. Returns the For or None."""
    best, best_w = None, 0

    def weight(block: kir.Block) -> int:
        w = 0
        for s in block.stmts:
            if isinstance(s, kir.KernelStmt):
                w += 1
            elif isinstance(s, kir.For):
                w += weight(s.body) * trips(s)
            elif isinstance(s, kir.While):
                w += weight(s.body) + weight(s.cond_block)
            elif isinstance(s, kir.If):
                w += max(weight(s.then), weight(s.orelse))
        return w

    def trips(f: kir.For) -> int:
        if isinstance(f.start, int) and isinstance(f.stop, int) and f.step > 0:
            return max(0, (f.stop - f.start + f.step - 1) // f.step)
        return 1

    def visit(block: kir.Block, mult: int):
        nonlocal best, best_w
        for s in block.stmts:
            if isinstance(s, kir.For):
                inner_loops = any(isinstance(x, (kir.For, kir.While)) for b in kir.walk_blocks(s.body) for x in b.stmts)
                w = weight(s.body) * trips(s) * mult
                if not inner_loops and trips(s) > 1 and w > best_w:
                    best, best_w = s, w
                visit(s.body, mult * trips(s))
            elif isinstance(s, kir.If):
                visit(s.then, mult)
                visit(s.orelse, mult)
    visit(prog.main, 1)
    return best


class ArenaPlan:
    """Byte offsets of every root buffer inside the runtime's arena. The header comes first, then a
    scratch region for split reductions, then the all-reduce bucket, then the region in which temporaries with
    disjoint lifetimes share bytes, then every other buffer in memory of its own."""

    def __init__(self, offsets: dict, size: int, scratch_off: int, scratch_bytes: int):
        self.offsets = offsets
        self.size = size
        self.scratch_off = scratch_off
        self.scratch_bytes = scratch_bytes
        self.shared: set = set()         # root ids whose bytes other tensors reuse once they are dead
        self.unused: set = set()         # root ids nothing touches (a gradient a fused update keeps in registers)
        self.shared_bytes = 0            # size of the shared region
        self.unshared_bytes = 0          # what its tensors would take with memory of their own
        self.spans: dict = {}            # root id -> (first, last) statement position of a shared tensor

    def off(self, b: kir.Buffer) -> int:
        return self.offsets[b.root.id]

    @property
    def clobbered(self) -> set:
        """Root ids whose contents are not meaningful after the program has run."""
        return self.shared | self.unused


def _stmt_roots(st) -> tuple[set, set]:
    """(root ids read, root ids written) by a statement and everything nested in it; a runtime call or a collective
    counts as reading and writing every tensor it names."""
    r: set = set()
    w: set = set()

    def buf(b, write=False):
        if isinstance(b, kir.Buffer):
            (w if write else r).add(b.root.id)
    if isinstance(st, kir.KernelStmt):
        return {b.id for b in st.kernel.reads()}, {b.id for b in st.kernel.writes()}
    if isinstance(st, kir.Print):
        for it in st.items:
            buf(it.buf)
    elif isinstance(st, kir.Check):
        for t, _ in st.value.scalars():
            buf(t.buf)
    elif isinstance(st, kir.RTCall):
        for v in st.args.values():
            for x in (v if isinstance(v, list) else [v]):
                buf(x); buf(x, True)
    elif isinstance(st, kir.AllReduce):
        for b in st.bufs:
            buf(b); buf(b, True)
    elif isinstance(st, kir.For):
        buf(st.start); buf(st.stop); buf(st.counter); buf(st.counter, True)
    elif isinstance(st, (kir.While, kir.If)):
        buf(st.cond)
    for name in ("body", "then", "orelse", "cond_block"):
        blk = getattr(st, name, None)
        if isinstance(blk, kir.Block):
            for inner in blk.stmts:
                r2, w2 = _stmt_roots(inner)
                r |= r2
                w |= w2
    return r, w


def deferred_kernels(prog: kir.Program) -> set:
    """Ids of kernels inside loops whose results nothing in the rest of their statement list needs: the rest neither
    reads nor writes what they write, and does not write what they read. They are the updates of biases, gains and
    their optimizer state at the end of a training step. Such a kernel may run on a second stream beside the kernels
    that follow it, as long as it has finished when the list ends. Kernels that draw random numbers (their stream
    position is ordered) are left out."""
    out: set = set()

    def visit(block: kir.Block, in_loop: bool):
        stmts = block.stmts
        if in_loop:
            later_r: set = set()
            later_w: set = set()
            for st in reversed(stmts):
                r, w = _stmt_roots(st)
                if isinstance(st, kir.KernelStmt):
                    k = st.kernel
                    if (not k.uses_rand() and k.rand_base is None
                            and not (w & (later_r | later_w)) and not (r & later_w)):
                        out.add(k.id)
                later_r |= r
                later_w |= w
        for st in stmts:
            if isinstance(st, kir.For):
                visit(st.body, True)
            elif isinstance(st, kir.While):
                visit(st.cond_block, True)
                visit(st.body, True)
            elif isinstance(st, kir.If):
                visit(st.then, in_loop)
                visit(st.orelse, in_loop)
    visit(prog.main, False)
    return out


SHARED_KINDS = ("temp", "grad")
FULL_WRITE_CALLS = ("nonzero", "input", "clock", "iota", "iota_once")
MIN_SHARED_BYTES = 4096                  # smaller tensors keep their own memory: nothing to gain


def covers(k: kir.Kernel, st: kir.Store) -> bool:
    """Does this store write EVERY element of its tensor, each exactly once? (The reference's planner asks for
    `domain extents == buffer shape` with the identity offset, anvil/backend/arena.py:46-57, which a collapsed loop nest
    no longer satisfies; a bijection of the domain onto the tensor is what is actually needed.)"""
    if st.accumulate or not st.offset.is_plain() or k.rand_base is not None:
        return False
    r = st.buf.root
    if k.out_numel() != r.numel or r.numel == 0:
        return False
    bounds = st.offset.bounds()
    return bounds == (0, r.numel - 1) and injective_over(st.offset, k.domain)


class _Use:
    __slots__ = ("pos", "chain", "write", "full", "after")

    def __init__(self, pos, chain, write, full, after=False):
        self.pos, self.chain, self.write, self.full, self.after = pos, chain, write, full, after


def _flatten(prog: kir.Program, fused_runs, deferred=()):
    """Every use of every root buffer with its statement position and the loops / branches around it, and the
    position ranges of the loops (the walk of anvil/backend/arena.py:36-98 over this IR). `fused_runs(kernels)` gives
    index ranges of consecutive kernels that the emitter runs as ONE kernel: they share a position, so nothing
    one of them reads can give its bytes to something another one writes. `deferred`: ids of kernels that may still be
    running on a second stream until the end of their run of kernels: what they touch is in use until then."""
    uses: dict = {}
    loops: list = []
    pos = 0

    def note(b, chain, write=False, full=False, after=False):
        if isinstance(b, kir.Buffer):
            uses.setdefault(b.root.id, []).append(_Use(pos, chain, write, full, after))

    def kernel_uses(k, chain, written_in_run):
        """`written_in_run`: tensors an earlier kernel of the same fused launch has written in full — a read of one of
        those is not a read of the tensor's initial contents, although it shares the statement position."""
        full = {st.buf.root.id for st in k.stores if covers(k, st)}
        for r in k.reads():
            note(r, chain, after=r.id in written_in_run)
        for r in k.writes():
            note(r, chain, True, r.id in full)
        written_in_run |= full

    def block(b: kir.Block, chain):
        nonlocal pos
        stmts = b.stmts
        i = 0
        while i < len(stmts):
            st = stmts[i]
            if isinstance(st, kir.KernelStmt):
                j = i
                while j < len(stmts) and isinstance(stmts[j], kir.KernelStmt):
                    j += 1
                run = [x.kernel for x in stmts[i:j]]
                starts = dict(fused_runs(run)) if fused_runs else {}
                q = 0
                while q < len(run):
                    pos += 1
                    end = starts.get(q, q + 1)
                    seen_full: set = set()
                    for k in run[q:end]:
                        kernel_uses(k, chain, seen_full)
                    q = end
                late = [k for k in run if k.id in deferred]
                if late:
                    pos += 1                         # the join
                    for k in late:
                        for r in list(k.reads()) + list(k.writes()):
                            note(r, chain)
                i = j
                continue
            stmt(st, chain)
            i += 1

    def stmt(st, chain):
        nonlocal pos
        pos += 1
        if isinstance(st, kir.For):
            start = pos
            note(st.start, chain); note(st.stop, chain)
            note(st.counter, chain, True)
            block(st.body, chain + (("loop", id(st)),))
            pos += 1
            loops.append((start, pos))
        elif isinstance(st, kir.While):
            start = pos
            inner = chain + (("loop", id(st)),)
            block(st.cond_block, inner)
            pos += 1
            note(st.cond, inner)
            block(st.body, inner)
            pos += 1
            loops.append((start, pos))
        elif isinstance(st, kir.If):
            note(st.cond, chain)
            block(st.then, chain + (("then", id(st)),))
            block(st.orelse, chain + (("else", id(st)),))
            pos += 1
        elif isinstance(st, kir.Print):
            for it in st.items:
                note(it.buf, chain)
        elif isinstance(st, kir.Check):
            for t, _ in st.value.scalars():
                note(t.buf, chain)
        elif isinstance(st, kir.RTCall):
            target = st.args.get("buf")
            for key, v in st.args.items():
                for x in (v if isinstance(v, list) else [v]):
                    if isinstance(x, kir.Buffer):
                        is_target = x is target and st.name not in ("save", "save_npy", "show", "sleep", "shuffle")
                        note(x, chain, is_target, is_target and st.name in FULL_WRITE_CALLS)
                        if st.name in ("load", "shuffle"):
                            note(x, chain, True, False)
        elif isinstance(st, kir.AllReduce):
            for b in st.bufs:
                note(b, chain, True, False)
    block(prog.main, ())
    return uses, loops


def _lifetime(us, loops):
    """[first, last] position over which a tensor holds a value somebody still needs, or None when it has to keep
    memory of its own: its first use must write all of it (nothing may rely on the initial zeros), and that write must
    be certain to have run before every other use (anvil/backend/arena.py:101-118)."""
    first = us[0].pos
    at_first = [u for u in us if u.pos == first]
    if any(not u.write and not u.after for u in at_first) or not any(u.full for u in at_first):
        return None
    chain = at_first[0].chain
    if any(u.chain[:len(chain)] != chain for u in us):
        return None
    lo, hi = first, us[-1].pos
    changed = True
    while changed:                                   # a lifetime that enters or leaves a loop covers the whole loop
        changed = False
        for a, b in loops:
            if lo <= b and a <= hi and not (a <= lo and hi <= b) and (a < lo or b > hi):
                lo, hi = min(lo, a), max(hi, b)
                changed = True
    return lo, hi


def plan_arena(prog: kir.Program, scratch_bytes: int = 0, header: int = 256 + 2 * 4 * 256, share: bool = True, fused_runs=None,
               keep=(), deferred=(), side_scratch_bytes: int = 0) -> ArenaPlan:
    """One arena for the whole program. Temporaries (`temp`, `grad`) whose first use writes all of them and whose
    lifetimes do not overlap share bytes (first fit by decreasing size, ids break ties: the layout is the same every
    run, like anvil/backend/arena.py:121-144); tensors nothing touches get no memory; every other root buffer
    gets its own zero-initialised, 256-byte aligned region (the reference gives each its own zeroed allocation,
    anvil/backend/cuda.py:416-421). `keep`: root ids that must not share (tensors the host reads or feeds).
    `deferred` / `side_scratch_bytes`: kernels that run on the second stream (see `deferred_kernels`) and the scratch
    space of their own that split reductions among them need (they run beside main-stream kernels that use the first)."""
    def up(n):
        return (n + ALIGN - 1) // ALIGN * ALIGN
    pos = up(header)
    scratch_off = pos
    pos += up(max(scratch_bytes, 4))
    side_scratch_off = pos
    pos += up(max(side_scratch_bytes, 4))
    offsets = {}
    bucket = [b.root for b in getattr(prog, "bucket", [])]
    bucket_off = pos
    for r in bucket:                                 # the all-reduce bucket is one contiguous span
        if r.id not in offsets:
            offsets[r.id] = pos
            pos += up(max(r.nbytes, 16))
    bucket_bytes = pos - bucket_off
    plan = ArenaPlan(offsets, 0, scratch_off, up(max(scratch_bytes, 4)))
    plan.bucket_off, plan.bucket_bytes = bucket_off, bucket_bytes
    plan.side_scratch_off, plan.side_scratch_bytes = side_scratch_off, up(max(side_scratch_bytes, 4))
    uses, loops = _flatten(prog, fused_runs, deferred)
    roots = prog.roots()
    items = []
    if share:
        for r in roots:
            if r.id in offsets or r.id in keep or r.kind not in SHARED_KINDS or r.nbytes < MIN_SHARED_BYTES or r.init is not None:
                continue
            us = uses.get(r.id)
            if not us:
                continue
            span = _lifetime(us, loops)
            if span is not None:
                items.append((r, span, up(r.nbytes)))
        items.sort(key=lambda it: (-it[2], it[1][0], it[0].id))
        placed: list = []                            # (lo, hi, offset, size)
        region = 0
        for r, (lo, hi), n in items:
            busy = sorted((off, off + sz) for l2, h2, off, sz in placed if l2 <= hi and lo <= h2)
            off = 0
            for s_, e_ in busy:
                if off + n <= s_:
                    break
                off = max(off, e_)
            placed.append((lo, hi, off, n))
            offsets[r.id] = pos + off
            plan.shared.add(r.id)
            plan.spans[r.id] = (lo, hi)
            region = max(region, off + n)
        plan.shared_bytes = region
        plan.unshared_bytes = sum(n for _, _, n in items)
        shared_base = pos
        pos += region
    for r in roots:
        if r.id in offsets:
            continue
        if r.id not in uses and r.kind in SHARED_KINDS and r.init is None and r.id not in keep:
            plan.unused.add(r.id)                    # nothing reads or writes it: no bytes of its own
            if share:
                offsets[r.id] = scratch_off          # (a valid address; DeviceProgram refuses to copy to or from it)
                continue
        offsets[r.id] = pos
        pos += up(max(r.nbytes, 16))
    plan.size = pos
    return plan


# ----------------------------------------------------------------------------- algorithmic work
FREE_UNARY = ("detach", "f32", "i32")


def kernel_flops(k: kir.Kernel) -> int:
    """Arithmetic of one kernel execution as the reference's cost model counts it
    (anvil/cost.py:22-37): every binary op, select and non-free unary op is 1, a reduction adds one
    accumulation per reduced element (so a multiply-add is 2)."""
    def ops(e: kir.E) -> int:
        seen, n = set(), 0
        stack = [e]
        while stack:
            x = stack.pop()
            if x.k in ("bin", "sel") or (x.k == "un" and x.op not in FREE_UNARY):
                n += 1
            stack.extend(x.a)
        return n
    per = 0
    if k.red is not None:
        per += k.red_numel() * (ops(k.red.body) + 1)
    per += sum(ops(st.value) for st in k.stmts)
    return k.out_numel() * per


def kernel_bytes(k: kir.Kernel) -> int:
    """Compulsory memory traffic of one kernel execution (anvil/cost.py:40-52): each tensor read
    counts once, but no more elements than its loads can reach; each store writes the domain once."""
    dom, red = k.out_numel(), k.red_numel()
    reach: dict = {}
    parts = ([(k.red.body, dom * red)] if k.red is not None else []) + [(st.value, dom) for st in k.stmts]
    roots = {}
    for e, n in parts:
        for x in e.walk():
            if x.k == "load":
                r = x.buf.root
                roots[r.id] = r
                reach[r.id] = reach.get(r.id, 0) + n
    read = sum(4 * min(roots[i].numel, n) for i, n in reach.items())
    return read + 4 * dom * len(k.stores)


def input_producers(prog: kir.Program, hot: kir.For):
    """The kernels at the head of the training loop that only produce the step's inputs: a batch
    gathered out of resident data through the shuffled permutation, or freshly sampled tokens.
    A caller that feeds batches from host memory copies into the buffers they write and skips them.
    Returns (kernels, buffers they write)."""
    ks, bufs = [], []
    if hot is None:
        return ks, bufs
    written_in_loop = set()
    for b in kir.walk_blocks(hot.body):
        for st in b.stmts:
            if isinstance(st, kir.KernelStmt):
                written_in_loop |= {r.id for r in st.kernel.writes()}
    for st in hot.body.stmts:
        if not isinstance(st, kir.KernelStmt):
            break
        k = st.kernel
        if k.red is not None or any(s.accumulate for s in k.stores):
            break
        reads = k.reads()
        if any(r.id in written_in_loop for r in reads):
            break                                    # depends on something the step computes
        if not k.uses_rand() and not any(r.numel > 1 for r in reads):
            break                                    # a constant fill, not an input
        ks.append(k)
        bufs += [s.buf.root for s in k.stores]
    return ks, bufs


def group_bytes(kernels, dead=()) -> int:
    """Compulsory traffic of a fused run of kernels: every tensor that comes from outside the run is
    read once, every tensor that outlives it is written once; what stays in registers moves nothing."""
    written, read, total = set(), {}, 0
    for k in kernels:
        dom, red = k.out_numel(), k.red_numel()
        for e, n in ([(k.red.body, dom * red)] if k.red is not None else []) + [(st.value, dom) for st in k.stmts]:
            for x in e.walk():
                if x.k == "load" and x.buf.root.id not in written:
                    r = x.buf.root
                    read[r.id] = max(read.get(r.id, 0), min(r.numel, n))
        for st in k.stores:
            r = st.buf.root
            if r.id not in written and r.id not in dead:
                total += 4 * dom
            written.add(r.id)
    return total + 4 * sum(read.values())
