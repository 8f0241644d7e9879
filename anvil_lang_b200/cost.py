"""`anvil cost --cuda`: what a program costs, statically and as measured on the GPU, per source line.

The static half restates the reference's report (anvil/cost.py:73-150): every kernel's FLOPs and compulsory memory
traffic (`analysis.kernel_flops` / `kernel_bytes`, the cost model of anvil/cost.py:22-52) times the number of times its
loop nest runs it, summed per source line, largest first. The measured half is new: the program runs once on the
device with every launch unit bracketed by CUDA events (`--profile`), the time of each unit is attributed to the
source lines of its kernels, and each line gets

    predicted   the time its FLOPs or its bytes need at the roofline (the slower of the two),
    measured    the time its kernels took,
    of roof     predicted / measured — how close the line runs to the hardware's limit.

Fused launch units (a softmax that is four source-level kernels but one launch) split their time over their kernels
in proportion to the predicted time of each.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field

from . import kir
from .backend import analysis as an

HBM_BYTES_PER_S = 6.5e12          # measured copy bandwidth of a B200 (the nominal figure is 7.7e12)
TENSOR_FLOPS_PER_S = 250e12       # 3xTF32: a third of the measured dense TF32 rate


@dataclass
class Line:
    flops: int = 0
    bytes: int = 0
    runs: int = 0
    kernels: set = field(default_factory=set)
    unbounded: bool = False
    text: str = ""
    ms: float = 0.0               # measured on the device (all runs)
    calls: int = 0


@dataclass
class Cost:
    flops: int = 0
    bytes: int = 0
    unbounded: bool = False
    lines: dict = field(default_factory=dict)        # (file, line) -> Line


def line_key(k: kir.Kernel):
    return (k.src[0], k.src[1]) if k.src else ("?", 0)


def program_cost(prog: kir.Program) -> Cost:
    """FLOPs and traffic of the whole run: a loop with constant bounds multiplies its body, a loop whose trip count
    is only known at run time counts once and marks the totals as lower bounds, both branches of an `if` count."""
    cost = Cost()

    def walk(block: kir.Block, times: int, unbounded: bool):
        for st in block.stmts:
            if isinstance(st, kir.KernelStmt):
                k = st.kernel
                f, m = an.kernel_flops(k) * times, an.kernel_bytes(k) * times
                cost.flops += f
                cost.bytes += m
                ln = cost.lines.setdefault(line_key(k), Line())
                ln.flops += f
                ln.bytes += m
                ln.runs = max(ln.runs, times)
                ln.kernels.add(k.id)
                ln.unbounded |= unbounded
                ln.text = k.src[2] if k.src else ""
            elif isinstance(st, kir.For):
                if isinstance(st.start, int) and isinstance(st.stop, int) and st.step > 0:
                    walk(st.body, times * max(0, -(-(st.stop - st.start) // st.step)), unbounded)
                else:
                    cost.unbounded = True
                    walk(st.body, times, True)
            elif isinstance(st, kir.While):
                cost.unbounded = True
                walk(st.cond_block, times, True)
                walk(st.body, times, True)
            elif isinstance(st, kir.If):
                walk(st.then, times, unbounded)
                walk(st.orelse, times, unbounded)
    walk(prog.main, 1, False)
    return cost


def roofline_seconds(flops: float, nbytes: float) -> float:
    return max(flops / TENSOR_FLOPS_PER_S, nbytes / HBM_BYTES_PER_S)


def human(n: float, unit: str = "") -> str:
    for scale, prefix in ((1e12, "T"), (1e9, "G"), (1e6, "M"), (1e3, "k")):
        if n >= scale:
            return f"{n / scale:.1f} {prefix}{unit}"
    return f"{n:.0f} {unit}".rstrip()


def measure(prog: kir.Program, cost: Cost, seed: int = 0, device: int = 0) -> float:
    """Runs the program on the GPU with per-unit timing and fills `ms` / `calls` of every line. Returns the
    milliseconds spent in kernels."""
    from .program import DeviceProgram
    dp = DeviceProgram(prog, seed=seed, device=device, graphs=False)
    try:
        dp.rtlib.anvil_rt_profile(dp.rt, 1)
        dp.run(capture=True)
        units = [[k] for k in dp.gen.kernels]
        by_idx = {idx: key for key, idx in dp.gen.groups.items()}
        kernel_of = {k.id: k for k in prog.kernels()}
        for gi in range(len(dp.gen.groups)):
            units.append([kernel_of[i] for i in by_idx[gi] if i in kernel_of])
        total = 0.0
        for slot, ks in enumerate(units):
            ms, calls = ctypes.c_double(), ctypes.c_long()
            if dp.rtlib.anvil_rt_profile_get(dp.rt, slot, ctypes.byref(ms), ctypes.byref(calls)) != 0 or not ks:
                continue
            total += ms.value
            weights = [roofline_seconds(an.kernel_flops(k), an.kernel_bytes(k)) or 1e-12 for k in ks]
            for k, w in zip(ks, weights):
                ln = cost.lines.get(line_key(k))
                if ln is not None:
                    ln.ms += ms.value * w / sum(weights)
                    ln.calls += calls.value
        return total
    finally:
        dp.close()


def report(prog: kir.Program, path: str, measured_ms: float | None = None, cost: Cost | None = None, shown: int = 15) -> str:
    """The text of `anvil cost` (static columns as in anvil/cost.py:116-150), with the measured columns when the
    program has been run (`measure`)."""
    c = cost or program_cost(prog)
    params = [b for b in prog.roots() if b.kind == "param"]
    nparams = sum(b.numel for b in params)
    ge = "≥ " if c.unbounded else ""
    out = [f"{path}: {nparams:,} parameters ({human(4 * nparams, 'B')})",
           f"the whole run: {ge}{human(c.flops, 'FLOP')}, {ge}{human(c.bytes, 'B')} of memory traffic "
           f"(at least {roofline_seconds(c.flops, c.bytes):.2g} s on a B200: {TENSOR_FLOPS_PER_S / 1e12:.0f} TFLOP/s as 3xTF32, "
           f"{HBM_BYTES_PER_S / 1e12:.1f} TB/s)"]
    if measured_ms is not None:
        out.append(f"measured on the device: {measured_ms / 1e3:.3g} s in kernels")
    out.append("")
    head = "  share      FLOP     traffic        runs"
    if measured_ms is not None:
        head += "   predicted    measured  of roof"
    out.append(head + "   line")
    rows = sorted(c.lines.items(), key=lambda kv: -(kv[1].ms if measured_ms is not None else kv[1].flops))
    n = 0
    for (f, line), ln in rows:
        weight = (ln.ms / measured_ms if measured_ms else 0) if measured_ms is not None else (ln.flops / c.flops if c.flops else 0)
        if n >= shown or (weight < 0.002 and n >= 5):
            break
        runs = ("≥ " if ln.unbounded else "") + f"{ln.runs:,}"
        row = f"  {weight:5.1%}  {human(ln.flops):>9}  {human(ln.bytes, 'B'):>10}  {runs:>10}"
        if measured_ms is not None:
            pred = 1e3 * roofline_seconds(ln.flops, ln.bytes)
            frac = f"{pred / ln.ms:7.0%}" if ln.ms > 0 else "      -"
            row += f"  {pred:8.3f} ms {ln.ms:8.3f} ms  {frac}"
        out.append(row + f"   {f + ':' + str(line):<16} {ln.text[:60]}")
        n += 1
    if len(rows) > n:
        rest = rows[n:]
        if measured_ms is not None:
            out.append(f"  {sum(ln.ms for _, ln in rest) / measured_ms if measured_ms else 0:5.1%}  (the other {len(rest)} lines)")
        else:
            rf = sum(ln.flops for _, ln in rest)
            out.append(f"  {rf / c.flops if c.flops else 0:5.1%}  {human(rf):>9}  (the other {len(rest)} lines)")
    return "\n".join(out)
