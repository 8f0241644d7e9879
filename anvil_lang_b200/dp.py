"""Data-parallel training over the GPUs of one node: batch sharding with ONE all-reduce per step.

The reference has no multi-device code. The scheme here keeps the *global* computation identical to
the single-GPU program: rank r of G runs the program compiled for the local batch b = B / G, and
`shard()` rewrites it so that

  1. batch gathers read rows  perm[B * step + r * b + i]  (the rank's slice of the global batch) and
     the batch loop runs N / B times; r is read at run time from a 0-d tensor, so all ranks run the
     same compiled library;
  2. kernels that sample a step's inputs draw element r * b * rowlen + i of the global tensor
     (`Kernel.rand_base`), so the ranks' samples are slices of the single-GPU draw;
  3. every kernel that updates parameters or optimizer state is split at its reduction: the gradient
     goes to a buffer in a contiguous "bucket", the update becomes an elementwise kernel that reads
     1/G times the bucket; all updates move behind a single `kir.AllReduce` of the bucket (the loss
     rides along), so parameters stay bit-identical on every rank.

Parameter initialisation and the shuffle are untouched: same seed, same bits on every rank.
The collective itself is NCCL inside the runtime (`attach_native`, csrc/anvil_comm.cu), ordered on the program's stream;
`attach` routes it through a host program's `torch.distributed` group instead.
"""
from __future__ import annotations

import itertools

from . import kir
from .backend import analysis as an
from .kir import F32, Affine, E, Kernel, KernelStmt, Let, Store

UPDATED_KINDS = ("param", "state")


class ShardError(Exception):
    pass


def _rewrite(e: E, fn, memo: dict, lets: dict) -> E:
    """Rebuilds an expression bottom-up; `fn(node)` may return a replacement for leaves."""
    hit = memo.get(id(e))
    if hit is not None:
        return hit
    r = fn(e)
    if r is None:
        if e.k == "let":
            r = E("let", e.dt, let=lets[e.let.id])
        elif e.a:
            r = E(e.k, e.dt, op=e.op, a=[_rewrite(x, fn, memo, lets) for x in e.a])
        else:
            r = e
    memo[id(e)] = r
    return r


def _identity(domain) -> Affine:
    strides = kir.row_major_strides([v.extent for v in domain])
    return Affine(0, list(zip(domain, strides)))


def _require_mean_loss(kernels, loss_root):
    """Gradients are summed over ranks and scaled by 1/G, which equals the global-batch gradient only when the loss
    is a MEAN over the samples: the kernel that writes it must be a sum whose constant factor is 1 / (reduced elements)
    (`sum_i -1/n * out[i, y[i]]`, the form the front end gives `mean` and `cross_entropy`). A summed loss would get
    gradients G times too small, so it is refused."""
    from .backend.contraction import _factors
    writers = [k for k in kernels if any(s.buf.root is loss_root for s in k.stores)]
    if not writers:
        raise ShardError("the loss is not written by a kernel of the step")
    k = writers[-1]
    if k.red is None or k.red.op != "sum":
        raise ShardError(f"the loss ({k.name}) is not a sum over the batch")
    fs: list = []
    _factors(k.red.body, fs)
    c = 1.0
    for f in fs:
        if f.k == "const":
            c *= float(f.val)
        elif f.k == "un" and f.op == "neg" and f.a[0].k == "const":
            c *= -float(f.a[0].val)
    n = k.red_numel()
    if abs(abs(c) * n - 1.0) > 1e-4:
        raise ShardError(f"the loss ({k.name}) is not a mean: factor {c!r} over {n} elements; data-parallel gradient "
                         f"scaling needs a mean loss")


def shard(prog: kir.Program, world: int) -> kir.Program:
    """Rewrites `prog` (compiled for the local batch) in place for a run over `world` ranks. The
    result is the same for every rank: the rank is a run-time value in the 0-d tensor
    `prog.rank_buf`, which the caller sets (`DeviceProgram.set_rank`)."""
    if world == 1:
        return prog
    hot = an.hot_loop(prog)
    if hot is None:
        raise ShardError("the program has no training loop")
    ids = itertools.count(max([b.id for b in prog.buffers] + [k.id for k in prog.kernels()]) + 1000)
    inv = 1.0 / world
    rank_buf = kir.Buffer(next(ids), "dp.rank", (), kir.I32, "var")
    prog.buffers.append(rank_buf)
    prog.rank_buf = rank_buf

    # ---- 1, 2: the step's inputs
    producers, _ = an.input_producers(prog, hot)
    gathers_fixed = False
    for k in producers:
        b_local = k.domain[0].extent
        if k.uses_rand():
            k.rand_base = (rank_buf, b_local * kir.prod(v.extent for v in k.domain[1:]))
            continue
        for e in [n for x in k.exprs() for n in x.walk() if n.k == "load"]:
            for g, _ in e.off.gathers():
                srefs = g.offset.scalars()
                if len(srefs) == 1 and srefs[0][0].buf.root is hot.counter.root:
                    terms = [(t, c * world if isinstance(t, kir.SRef) else c) for t, c in g.offset.terms]
                    g.offset = Affine(g.offset.const, terms + [(kir.SRef(rank_buf), b_local)])
                    e._key = None
                    gathers_fixed = True
    if gathers_fixed:
        if not (isinstance(hot.start, int) and isinstance(hot.stop, int)):
            raise ShardError("the batch loop has run-time bounds")
        hot.stop = hot.start + (hot.stop - hot.start) // world

    # ---- 3: split updates from gradients, move them behind one all-reduce
    body = hot.body.stmts
    if not all(isinstance(s, (KernelStmt, kir.Print)) for s in body):
        raise ShardError("the training loop has control flow inside it")
    kernels = [s.kernel for s in body if isinstance(s, KernelStmt)]
    prints = [s for s in body if isinstance(s, kir.Print)]
    is_update = {k.id: any(s.buf.root.kind in UPDATED_KINDS for s in k.stores) for k in kernels}
    grads: list[kir.Buffer] = []
    first, updates = [], []
    for k in kernels:
        if not is_update[k.id]:
            first.append(k)
            continue
        if k.red is None:
            updates.append(k)
            continue
        g = kir.Buffer(next(ids), f"g.{k.name}", tuple(v.extent for v in k.domain), k.red.dtype, "grad")
        if g.dtype != F32:
            raise ShardError(f"{k.name}: an integer reduction feeds an update")
        prog.buffers.append(g)
        grads.append(g)
        ident = _identity(k.domain)
        first.append(Kernel(next(ids), k.name + "_g", k.label, k.domain, [Store(g, ident, E("acc", F32))], k.red, src=k.src))
        lets, memo, stmts = {}, {}, []

        def fn(n, g=g, ident=ident):
            if n.k == "acc":
                return E("bin", F32, op="mul", a=[E("const", F32, val=inv), E("load", F32, buf=g, off=ident)])
            return None
        for st in k.stmts:
            if isinstance(st, Let):
                nl = Let(next(ids), st.name, _rewrite(st.value, fn, memo, lets))
                lets[st.id] = nl
                stmts.append(nl)
            else:
                stmts.append(Store(st.buf, st.offset, _rewrite(st.value, fn, memo, lets), st.accumulate))
        updates.append(Kernel(next(ids), k.name + "_u", k.label, k.domain, stmts, None, src=k.src))

    # gradients that reach an update kernel through memory (written by non-update kernels)
    written_first = set()
    for k in first:
        written_first |= {b.id for b in k.writes()}
    grad_ids = {g.id for g in grads}
    exchanged: dict[int, kir.Buffer] = {}
    for k in updates:
        for r in k.reads():
            if r.id in written_first and r.id not in grad_ids and r.kind not in UPDATED_KINDS and r.numel > 0 \
                    and r.root is not hot.counter.root:
                if r.dtype != F32:
                    raise ShardError(f"{k.name} reads the integer tensor {r.name} computed by the step")
                exchanged[r.id] = r
    for i, k in enumerate(updates):
        if not any(r.id in exchanged for r in k.reads()):
            continue
        lets, memo, stmts = {}, {}, []

        def fn2(n):
            if n.k == "load" and n.buf.root.id in exchanged:
                return E("bin", F32, op="mul", a=[E("const", F32, val=inv), n])
            return None
        for st in k.stmts:
            if isinstance(st, Let):
                nl = Let(next(ids), st.name, _rewrite(st.value, fn2, memo, lets))
                lets[st.id] = nl
                stmts.append(nl)
            else:
                stmts.append(Store(st.buf, st.offset, _rewrite(st.value, fn2, memo, lets), st.accumulate))
        updates[i] = Kernel(k.id, k.name, k.label, k.domain, stmts, None, k.rand_base, k.src)

    # moving the updates to the end must not change what anything reads
    upd_writes = set()
    for k in updates:
        upd_writes |= {b.id for b in k.writes()}
    pos = {k.id: i for i, k in enumerate(kernels)}
    orig_of = {}
    for k in kernels:
        orig_of[k.name] = k
    for u in updates:
        base = orig_of.get(u.name.removesuffix("_u"), None)
        upos = pos.get(base.id if base is not None else u.id, 0)
        uw = {b.id for b in u.writes()}
        ur = {b.id for b in u.reads()}
        for k in kernels[upos + 1:]:
            if is_update[k.id]:
                # a later update with a reduction has its gradient half hoisted in front of the all-reduce: that
                # half must not read what this update writes (it would see the value from before the update)
                if k.red is not None:
                    red_reads = {n.buf.root.id for n in k.red.body.walk() if n.k == "load"}
                    for n in k.red.body.walk():
                        if n.k in ("load", "index"):
                            for a in [n.off] + list(kir._nested(n.off)):
                                red_reads |= {g.buf.root.id for g, _ in a.gathers()} | {s_.buf.root.id for s_, _ in a.scalars()}
                    if uw & red_reads:
                        raise ShardError(f"the gradient of {k.name} reads what the earlier update {u.name} writes")
                continue
            if uw & {b.id for b in k.reads()} or uw & {b.id for b in k.writes()} \
                    or (ur - set(exchanged) - grad_ids) & {b.id for b in k.writes()}:
                raise ShardError(f"{k.name} depends on the update {u.name} that would move behind it")

    bucket = grads + list(exchanged.values())
    tail = []
    loss = [b for b in prog.buffers if b.name == "loss" and b.root.id in written_first]
    if not loss:
        raise ShardError("no `loss` tensor is computed by the step: the 1/G scaling of the gradients assumes a mean loss")
    if loss:
        lb = loss[-1].root
        _require_mean_loss(first, lb)
        bucket.append(lb)
        zero = Affine(0)
        tail.append(Kernel(next(ids), "loss_mean", "mean over ranks", [],
                           [Store(lb, zero, E("bin", F32, op="mul", a=[E("const", F32, val=inv),
                                                                        E("load", F32, buf=lb, off=zero)]))], None))
    prog.bucket = bucket
    hot.body.stmts = ([KernelStmt(k) for k in first] + [kir.AllReduce(bucket)]
                      + [KernelStmt(k) for k in tail + updates] + prints)
    return prog


# ----------------------------------------------------------------------------- the collective on GPUs
_keep = []          # ctypes callbacks must outlive the programs that hold them


def attach_native(devprog, rank: int, world: int, id_file: str | None = None, timeout_s: float = 120.0):
    """Joins the runtime's own NCCL communicator (csrc/anvil_comm.cu): the program's `kir.AllReduce` becomes
    ncclAllReduce(sum, f32) in place on the arena's gradient bucket, ordered on the program's stream — no Python, no
    torch in the step. Only the 128-byte communicator id has to travel from rank 0 to the others once: through the
    default `torch.distributed` group when one is initialised, else through `id_file` (rank 0 writes it, the others wait
    for it), which is all a C host would need."""
    import ctypes
    import os
    import time
    buf = (ctypes.c_char * 128)()
    use_file = id_file is not None
    dist = None
    if not use_file:
        import torch.distributed as dist
        if not dist.is_initialized():
            raise RuntimeError("anvil: no process group and no id file to hand the communicator id around")
    if rank == 0:
        if devprog.rtlib.anvil_rt_comm_unique_id(buf, 128) != 0:
            raise RuntimeError("anvil: NCCL is not available (libnccl.so.2 could not be loaded)")
        if use_file:
            tmp = id_file + ".tmp"
            with open(tmp, "wb") as f:
                f.write(bytes(buf))
            os.replace(tmp, id_file)
    if use_file and rank != 0:
        t0 = time.time()
        while not os.path.exists(id_file):
            if time.time() - t0 > timeout_s:
                raise TimeoutError(f"anvil: rank 0 never wrote the communicator id to {id_file}")
            time.sleep(0.01)
        with open(id_file, "rb") as f:
            raw = f.read()
        ctypes.memmove(buf, raw, 128)
    if not use_file:
        box = [bytes(buf) if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        ctypes.memmove(buf, box[0], 128)
    devprog._check(devprog.rtlib.anvil_rt_comm_init(devprog.rt, rank, world, buf, 128))
    n = devprog.rtlib.anvil_rt_comm_nranks(devprog.rt)
    if n != world:
        raise RuntimeError(f"anvil: the communicator has {n} ranks, expected {world}")
    return n


def attach(devprog, device: int):
    """Binds a sharded `DeviceProgram` to the default `torch.distributed` process group (NCCL): the
    program runs on a torch-owned stream, and its `kir.AllReduce` becomes `dist.all_reduce(SUM)` on
    a tensor that aliases the arena's gradient bucket (in place, no staging copy). Kept for hosts that already own a
    process group and want its collective; `attach_native` is what `bench.py` and the command line use."""
    import ctypes

    import torch
    import torch.distributed as dist
    stream = torch.cuda.Stream(device=device)
    devprog._check(devprog.rtlib.anvil_rt_use_stream(devprog.rt, ctypes.c_void_p(stream.cuda_stream)))
    views = {}

    class _Span:
        def __init__(self, ptr, count):
            self.__cuda_array_interface__ = {"shape": (count,), "typestr": "<f4", "data": (ptr, False), "version": 2}

    def allreduce(user, ptr, count, cuda_stream):
        try:
            t = views.get((ptr, count))
            if t is None:
                t = views[(ptr, count)] = torch.as_tensor(_Span(ptr, count), device=f"cuda:{device}")
            with torch.cuda.stream(stream):
                dist.all_reduce(t)
            return 0
        except Exception as e:          # no exceptions across the C boundary
            import sys
            print(f"anvil: all-reduce failed: {e}", file=sys.stderr)
            return 1
    cb = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_long, ctypes.c_void_p)(allreduce)
    _keep.append((cb, stream, views))
    devprog.rtlib.anvil_rt_set_allreduce(devprog.rt, ctypes.cast(cb, ctypes.c_void_p), None)
    return stream
