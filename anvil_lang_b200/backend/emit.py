"""The sm_100a emitter: a `kir.Program` becomes one CUDA C++ translation unit.

This is the counterpart of the reference's text emitter (anvil/backend/cuda.py: `KernelGen` :52-320
for kernels, `CudaGen` :348-594 for host code), redesigned for B200:

  * kernels are scheduled by class instead of always "one thread per output with a serial loop":
      eltwise      128-bit vectorised single pass over the flattened domain
      thread       short reductions (window max, 10-class argmax) stay in the thread
      coop(row)    the reduction index is contiguous in memory: lanes of a warp (or a whole CTA)
                   stride across it with 128-bit loads and combine with a fixed shuffle tree
      coop(col)    the output index is contiguous: threads along outputs, a second block dimension
                   along the reduction, shared-memory tree
      split        few outputs x long reduction: several CTAs per output write partial results to
                   arena scratch and a second kernel combines them in order
      serial       order-dependent kernels run on one thread (anvil/backend/cuda.py:380-395)
    All combination trees have a shape fixed by the launch geometry: results are bit-reproducible.
  * every tensor lives at a fixed offset of one device arena; a kernel receives the arena base and
    derives its pointers from compile-time offsets.
  * host control flow is emitted as C++ that calls the runtime's C ABI (include/anvil_cuda.h); it
    never touches device memory directly and synchronises only when the host needs a value
    (a printed scalar, an `if`/`while` condition, a run-time loop bound).
  * runs of kernel launches inside loops are recorded into CUDA graphs and replayed.
  * several IR kernels may become one launch: runs of row kernels (`rowgroup`), products that share an operand or an
    output (`hfuse`), attention runs (`attention`), and independent short kernels side by side (`plan_zgroups`);
    kernels whose results nothing later in their launch run needs go to a second stream (`analysis.deferred_kernels`).

Scalar expression semantics follow anvil/backend/cuda.py:110-199 (casts, wrap-around i32
arithmetic, comparison results 0.0/1.0, nan-propagating max/min).
"""
from __future__ import annotations

import math

from .. import kir
from ..kir import F32, I32
from . import analysis as an
from . import attention as at
from . import contraction as ct
from . import hfuse
from . import rowgroup as rg

THREADS = 256
MAX_BLOCKS = 148 * 8


def ctype(dt) -> str:
    return "int" if dt == I32 else "float"


def flit(v: float) -> str:
    """An f32 literal: the shortest decimal text that round-trips the double, with an `f` suffix, or the CUDA names
    of the special values."""
    v = float(v)
    if v != v:
        return "CUDART_NAN_F"
    if v in (math.inf, -math.inf):
        return "CUDART_INF_F" if v > 0 else "(-CUDART_INF_F)"
    text = repr(v)
    needs_point = not any(ch in text for ch in ".e")
    return text + (".0f" if needs_point else "f")


def c_string(s: str) -> str:
    out = []
    for ch in s.encode("utf-8"):
        c = chr(ch)
        if c == "\\":
            out.append("\\\\")
        elif c == '"':
            out.append('\\"')
        elif c == "\n":
            out.append("\\n")
        elif c == "\t":
            out.append("\\t")
        elif 32 <= ch < 127 and c != "?":
            out.append(c)
        else:
            out.append("\\%03o" % ch)
    return '"' + "".join(out) + '"'


RED_OP = {"sum": "anvil::OpSum", "prod": "anvil::OpProd", "max": "anvil::OpMax", "min": "anvil::OpMin"}


class Scope:
    """Builds the C++ for a kernel's expressions. `lanes` > 1 evaluates the body for that many
    consecutive values of `vv`; nodes that do not depend on `vv` are computed once."""

    def __init__(self, kg: "KernelGen", names: dict, lanes: int = 1, vv=None, ind: str = "        "):
        self.kg = kg
        self.names = names              # Var -> C identifier (lane l of vv is f"{name}_{l}")
        self.lanes = lanes
        self.vv = vv
        self.ind = ind
        self.lines: list[str] = []
        self.memo: dict = {}
        self.dep: dict = {}
        self.lets: dict = {}            # let id -> {lane: code}
        self.acc_name = "acc"           # C identifier that holds the kernel's reduction result
        self.acc_lanes = False          # one result per lane (`acc_0` ...): lanes run along an output var
        self.preloaded: dict = {}       # (root id, offset key) -> C expression holding that element already

    # ---- which nodes vary along the vectorised var
    def off_depends(self, a: kir.Affine) -> bool:
        return self.vv is not None and self.vv in a.vars()

    def depends(self, e: kir.E) -> bool:
        if self.lanes == 1:
            return False
        hit = self.dep.get(id(e))
        if hit is None:
            if e.k in ("load", "index"):
                hit = self.off_depends(e.off)
            elif e.k == "rand":
                hit = self.kg.rand_varies_with(self.vv)
            elif e.k == "let":
                hit = self.lets.get(e.let.id, {}).get("dep", False)
            elif e.k == "acc":
                hit = self.acc_lanes
            else:
                hit = any(self.depends(x) for x in e.a)
            self.dep[id(e)] = hit
        return hit

    def emit(self, s: str):
        self.lines.append(self.ind + s)

    def var(self, v: kir.Var, lane) -> str:
        n = self.names[v]
        if v is self.vv and self.lanes > 1:
            return f"{n}_{lane}"
        return n

    # ---- affine offsets
    def affine(self, a: kir.Affine, lane) -> str:
        wide = not an.offset_fits_i32(a)
        parts = [f"{a.const}{'L' if wide else ''}"] if a.const else []
        for t, c in a.terms:
            if isinstance(t, kir.Var):
                x = self.var(t, lane)
            elif isinstance(t, kir.SRef):
                x = self.sref(t)
            else:
                x = self.gather(t, lane)
            if wide:
                parts.append(f"(long){x}" if c == 1 else f"{c}L * {x}")
            else:
                parts.append(x if c == 1 else f"{c} * {x}")
        return " + ".join(parts) if parts else "0"

    def sref(self, t: kir.SRef) -> str:
        key = ("sref", t.buf.root.id)
        hit = self.memo.get(key)
        if hit is None:
            hit = self.kg.tmp()
            self.emit(f"const long {hit} = (long){self.kg.ptr(t.buf, False)}[0];")
            self.memo[key] = hit
        return hit

    def gather(self, g: kir.Gather, lane) -> str:
        dep = self.off_depends(g.offset)
        key = ("g", g.key(), lane if dep else None)
        hit = self.memo.get(key)
        if hit is None:
            hit = self.kg.tmp()
            code = self.kg.gen.fault(f"index out of bounds ({g.where or 'gather'}; dimension size {g.bound})")
            off = self.affine(g.offset, lane)
            self.emit(f"const long {hit} = anvil::gather_index({self.kg.ptr(g.buf, False)}, {off}, "
                      f"{g.lo}L, {g.hi}L, fault_, {code});")
            self.memo[key] = hit
        return hit

    # ---- expressions
    def ex(self, e: kir.E, lane=0) -> str:
        if e.k == "const":
            return flit(e.val) if e.dt == F32 else f"({int(e.val)})"
        if e.k == "acc":
            return f"{self.acc_name}_{lane}" if self.acc_lanes else self.acc_name
        if e.k == "let":
            d = self.lets[e.let.id]
            return d[lane if d["dep"] else None]
        dep = self.depends(e)
        key = (e.key(), lane if dep else None)
        hit = self.memo.get(key)
        if hit is not None:
            return hit
        s = self.build(e, lane)
        name = self.kg.tmp()
        self.emit(f"const {ctype(e.dt)} {name} = {s};")
        self.memo[key] = name
        return name

    def cast(self, e: kir.E, dt, lane) -> str:
        s = self.ex(e, lane)
        if e.dt == dt:
            return s
        return f"(float)({s})" if dt == F32 else f"anvil::f2i({s})"

    def build(self, e: kir.E, lane) -> str:
        k = e.k
        if k == "load":
            return self.load(e, lane)
        if k == "index":
            return f"(int)({self.affine(e.off, lane)})"
        if k == "rand":
            idx = self.kg.rand_index(self, lane)
            return f"anvil_rand((uint32_t)({idx}), stream_, {e.salt}u, seed_, {1 if e.open_low else 0})"
        if k == "un":
            return self.unary(e, lane)
        if k == "bin":
            return self.binary(e, lane)
        if k == "sel":
            c = self.ex(e.a[0], lane)
            if not any(n.k == "load" for br in (e.a[1], e.a[2]) for n in br.walk()):
                return f"(({c}) != 0 ? {self.cast(e.a[1], e.dt, lane)} : {self.cast(e.a[2], e.dt, lane)})"
            # a branch that reads memory is only evaluated when taken (`x if hit else 0.0` inside a long
            # reduction); with a condition shared by all lanes, one `if` serves all of them
            shared = self.lanes > 1 and self.depends(e) and not self.depends(e.a[0])
            lanes = list(range(self.lanes)) if shared else [lane]
            names = {l: self.kg.tmp("s") for l in lanes}
            self.emit(f"{ctype(e.dt)} " + ", ".join(names.values()) + ";")
            for branch, head in ((e.a[1], f"if (({c}) != 0) {{"), (e.a[2], "} else {")):
                self.emit(head)
                saved = dict(self.memo)
                self.ind += "    "
                for l in lanes:
                    self.emit(f"{names[l]} = {self.cast(branch, e.dt, l)};")
                self.ind = self.ind[:-4]
                self.memo = saved
            self.emit("}")
            for l in lanes:
                if l != lane:
                    self.memo[(e.key(), l)] = names[l]
            return names[lane]
        raise NotImplementedError(k)

    def load(self, e: kir.E, lane) -> str:
        if self.preloaded:
            hit = self.preloaded.get((e.buf.root.id, e.off.key()))
            if hit is not None:
                return hit
        p = self.kg.ptr(e.buf, False)
        if self.lanes % 4 == 0 and self.lanes >= 4 and self.depends(e) and an.stride_of(e.off, self.vv) == 1 \
                and an.aligned4(e.off, self.vv):
            vkey = ("vec", e.key(), lane // 4)           # lanes come in aligned groups of 4 consecutive elements
            q = self.memo.get(vkey)
            if q is None:
                q = self.kg.tmp("q")
                self.emit(f"const {ctype(e.dt)}4 {q} = anvil::ld4({p} + ({self.affine(e.off, lane - lane % 4)}));")
                self.memo[vkey] = q
            return f"{q}.{'xyzw'[lane % 4]}"
        return f"{p}[{self.affine(e.off, lane)}]"

    # Scalar operators as tables: `{a}` / `{b}` are the operand texts, `{fa}` the operand as a float. The semantics
    # are the interpreter's (anvil/interp.py:575-632): comparisons and logic give 0.0 / 1.0, integer arithmetic wraps,
    # max / min propagate nan, floor division and modulo follow Python, a zero integer divisor counts as 1.
    UNARY_ANY = {"detach": "{a}", "neg": "(-({a}))", "not": "(({a}) == 0 ? 1.0f : 0.0f)", "f32": "(float)({a})"}
    UNARY_BY_TYPE = {            # op -> (text for an i32 operand, text for an f32 operand)
        "abs": ("abs({a})", "fabsf({a})"), "i32": ("{a}", "anvil::f2i({a})"),
        "sign": ("anvil::isign({a})", "anvil::fsign({a})"),
        "floor": ("{a}", "floorf({a})"), "ceil": ("{a}", "ceilf({a})"), "round": ("{a}", "rintf({a})"),
    }
    UNARY_FLOAT = {"rsqrt": "(1.0f / sqrtf({fa}))", "recip": "(1.0f / ({fa}))", "sigmoid": "anvil::sigmoid({fa})",
                   "exp": "expf({fa})", "log": "logf({fa})", "sqrt": "sqrtf({fa})", "tanh": "tanhf({fa})",
                   "sin": "sinf({fa})", "cos": "cosf({fa})"}
    COMPARE = {"lt": "<", "le": "<=", "gt": ">", "ge": ">=", "eq": "==", "ne": "!="}
    LOGIC = {"and": "&&", "or": "||"}
    BINARY_I32 = {"add": "(int)((uint32_t)({a}) + (uint32_t)({b}))", "sub": "(int)((uint32_t)({a}) - (uint32_t)({b}))",
                  "mul": "(int)((uint32_t)({a}) * (uint32_t)({b}))", "idiv": "anvil::idiv({a}, {b})",
                  "mod": "anvil::imod({a}, {b})", "max": "anvil::imax({a}, {b})", "min": "anvil::imin({a}, {b})"}
    BINARY_F32 = {"add": "(({a}) + ({b}))", "sub": "(({a}) - ({b}))", "mul": "(({a}) * ({b}))", "div": "(({a}) / ({b}))",
                  "max": "anvil::fmax_nan({a}, {b})", "min": "anvil::fmin_nan({a}, {b})", "pow": "powf({a}, {b})",
                  "idiv": "floorf(({a}) / ({b}))", "mod": "anvil::fmod_py({a}, {b})"}

    def unary(self, e: kir.E, lane) -> str:
        operand = e.a[0]
        a = self.ex(operand, lane)
        integer = operand.dt == I32
        if e.op in self.UNARY_ANY:
            return self.UNARY_ANY[e.op].format(a=a)
        if e.op in self.UNARY_BY_TYPE:
            return self.UNARY_BY_TYPE[e.op][0 if integer else 1].format(a=a)
        return self.UNARY_FLOAT[e.op].format(fa=f"(float)({a})" if integer else a)

    def binary(self, e: kir.E, lane) -> str:
        lhs, rhs = e.a
        if e.op in self.LOGIC:
            return f"((({self.ex(lhs, lane)}) != 0 {self.LOGIC[e.op]} ({self.ex(rhs, lane)}) != 0) ? 1.0f : 0.0f)"
        if e.op in self.COMPARE:
            if lhs.dt == rhs.dt:                     # same type: compared as they are; mixed: both as floats
                a, b = self.ex(lhs, lane), self.ex(rhs, lane)
            else:
                a, b = self.cast(lhs, F32, lane), self.cast(rhs, F32, lane)
            return f"(({a}) {self.COMPARE[e.op]} ({b}) ? 1.0f : 0.0f)"
        if e.dt == I32:
            return self.BINARY_I32[e.op].format(a=self.ex(lhs, lane), b=self.ex(rhs, lane))
        return self.BINARY_F32[e.op].format(a=self.cast(lhs, F32, lane), b=self.cast(rhs, F32, lane))

    # ---- statements (anvil/backend/cuda.py:249-264)
    def statements(self):
        k = self.kg.k
        L = self.lanes
        for st in k.stmts:
            if isinstance(st, kir.Let):
                dep = self.depends(st.value)
                d = {"dep": dep}
                for lane in (range(L) if dep else [None]):
                    v = self.ex(st.value, lane if lane is not None else 0)
                    name = self.kg.tmp()
                    self.emit(f"const {ctype(st.value.dt)} {name} = {v};")
                    d[lane] = name
                self.lets[st.id] = d
                continue
            self.store(st)
            self.memo = {key: v for key, v in self.memo.items() if key[0] in ("sref",)}   # later loads re-read memory

    def store(self, st: kir.Store):
        k, L = self.kg.k, self.lanes
        p = self.kg.ptr(st.buf, True)
        dt = st.buf.dtype
        vec_ok = (L % 4 == 0 and L >= 4 and an.stride_of(st.offset, self.vv) == 1 and an.aligned4(st.offset, self.vv))
        vals = [self.cast(st.value, dt, lane) for lane in range(L)]
        exclusive = an.exclusive_store(k, st)
        if vec_ok and (not st.accumulate or exclusive):
            T4 = f"{ctype(dt)}4"
            for g in range(0, L, 4):
                off = self.affine(st.offset, g)
                v = vals[g:g + 4]
                if st.accumulate:
                    q = self.kg.tmp("q")
                    self.emit(f"{T4} {q} = anvil::ld4({p} + ({off}));")
                    self.emit(f"{q}.x += {v[0]}; {q}.y += {v[1]}; {q}.z += {v[2]}; {q}.w += {v[3]};")
                    self.emit(f"anvil::st4({p} + ({off}), {q});")
                else:
                    self.emit(f"anvil::st4({p} + ({off}), make_{T4}({', '.join(v)}));")
            return
        for lane in range(L):
            target = f"{p}[{self.affine(st.offset, lane)}]"
            old = self.preloaded.get((st.buf.root.id, st.offset.key())) if st.accumulate else None
            if old is not None:
                self.emit(f"{target} = ({old}) + ({vals[lane]});")
            elif st.accumulate:
                if exclusive or not self.kg.parallel:
                    self.emit(f"{target} += {vals[lane]};")
                else:
                    self.emit(f"atomicAdd(&{target}, {vals[lane]});")
            else:
                self.emit(f"{target} = {vals[lane]};")


class KernelGen:
    """One IR kernel -> one or two __global__ functions plus a host launcher."""

    def __init__(self, gen: "ProgramGen", k: kir.Kernel):
        self.gen = gen
        self.k = k
        self.n = 0
        self.ptrs: dict = {}            # root id -> (buffer, written?)
        self.parallel = an.parallel_safe(k)
        self.dom = {v: f"d{i}" for i, v in enumerate(k.domain)}
        self.red = {v: f"r{i}" for i, v in enumerate(k.red.vars)} if k.red else {}
        self.names = {**self.dom, **self.red}
        self.uses_rand = k.uses_rand()
        self.written = {s.buf.root.id for s in k.stores}
        self.strategy = ""
        self.notes = ""

    def tmp(self, prefix="t") -> str:
        self.n += 1
        return f"{prefix}{self.n}"

    def ptr(self, b: kir.Buffer, write: bool) -> str:
        r = b.root
        w = r.id in self.written
        self.ptrs[r.id] = (r, w)
        return f"b{r.id}"

    def rand_varies_with(self, vv) -> bool:
        return vv in self.k.domain

    def rand_index(self, scope: Scope, lane) -> str:
        strides = kir.row_major_strides([v.extent for v in self.k.domain])
        parts = [f"{s}u * (uint32_t){scope.var(v, lane)}" for v, s in zip(self.k.domain, strides)]
        if self.k.rand_base is not None:
            rb, coef = self.k.rand_base
            parts.append(f"{coef & 0xFFFFFFFF}u * (uint32_t){self.ptr(rb, False)}[0]")
        return " + ".join(parts) if parts else "0u"

    def pointer_decls(self) -> list[str]:
        out = []
        for rid, (r, w) in sorted(self.ptrs.items()):
            T = ctype(r.dtype)
            off = self.gen.plan.offsets[rid]
            if w:
                out.append(f"    {T} *b{rid} = ({T} *)(A + {off}UL);   // {r.name}{list(r.shape)}")
            else:
                out.append(f"    const {T} *__restrict__ b{rid} = (const {T} *)(A + {off}UL);   // {r.name}{list(r.shape)}")
        out.append("    anvil::Fault *fault_ = (anvil::Fault *)(A + ANVIL_RT_FAULT_OFF); (void)fault_;")
        if self.uses_rand:
            out.append("    const uint32_t stream_ = *(const uint32_t *)(A + ANVIL_RT_STREAM_OFF) + sdelta;")
        return out

    def head(self, name, threads) -> str:
        """Opens the kernel. Bodies index their CTA through bx_ / by_ / gdx_ (block index and grid width): a kernel that is a
        member of a side-by-side launch (`ZGroupGen`) is a device function that gets them as arguments, plus a thin
        __global__ wrapper so it can still be launched alone."""
        self.nthreads = threads
        if self.member:
            return (f"__device__ __forceinline__ void {name}_body(char *__restrict__ A, uint32_t sdelta, uint32_t seed_, "
                    f"const unsigned bx_, const unsigned by_, const unsigned gdx_, char *zsm_) {{")
        return (f"__global__ void __launch_bounds__({threads}) {name}(char *__restrict__ A, uint32_t sdelta, "
                f"uint32_t seed_) {{\n    const unsigned bx_ = blockIdx.x, by_ = blockIdx.y, gdx_ = gridDim.x; (void)by_; (void)gdx_;")

    @property
    def member(self) -> bool:
        return self.k.id in self.gen.member_slot

    def wrapper(self, name) -> str:
        return (f"__global__ void __launch_bounds__({self.nthreads}) {name}(char *__restrict__ A, uint32_t sdelta, uint32_t seed_) {{\n"
                f"    __shared__ __align__(16) char zsm_[{max(16, self.zsm_bytes)}];\n"
                f"    {name}_body(A, sdelta, seed_, blockIdx.x, blockIdx.y, gridDim.x, zsm_);\n}}")

    def comment(self, sched) -> str:
        k = self.k
        c = (f"// {k.name} | {k.label or 'kernel'} | {sched} | "
             + " x ".join(f"{v.name}<{v.extent}" for v in k.domain))
        if k.red is not None:
            c += f"  {k.red.op} over " + " x ".join(f"{v.name}<{v.extent}" for v in k.red.vars)
        return c

    # ---- index decode
    @staticmethod
    def decode(src: str, vars_, names, ind, vec_var=None, L=1) -> list[str]:
        """C lines that split the flat index `src` into `vars_` (row-major; the vectorised var counts
        extent/L positions and is scaled by L)."""
        ext = [(v.extent // L if v is vec_var else v.extent) for v in vars_]
        strides = kir.row_major_strides(ext)
        out = []
        for v, st, n in zip(vars_, strides, ext):
            idx = f"({src} / {st}u) % {n}u" if st != 1 else f"{src} % {n}u"
            if st * n >= kir.prod(ext):
                idx = f"{src} / {st}u" if st != 1 else src          # the outermost var needs no modulo
            scale = f" * {L}" if (v is vec_var and L > 1) else ""
            out.append(f"{ind}const int {names[v]} = (int)({idx}){scale};")
        return out

    def lane_vars(self, vv, L, ind) -> list[str]:
        if L == 1:
            return []
        n = self.names[vv]
        return [f"{ind}const int " + ", ".join(f"{n}_{l} = {n} + {l}" for l in range(L)) + ";"]

    # ---- strategy choice
    def choose(self):
        k = self.k
        ON, RN = k.out_numel(), k.red_numel()
        if not self.parallel:
            return ("serial",)
        if k.red is None:
            return ("eltwise", self.vec_width_domain())
        c = ct.match(k)
        if c is not None:
            return ("gemm", c)
        if k.red.op in ("argmax", "argmin") or RN <= 64:
            return ("thread",)
        rlast = k.red.vars[-1]
        dlast = k.domain[-1] if k.domain else None
        # which way do the loads that are re-read at every reduction step walk memory? (a load that
        # does not depend on the reduction vars is one value per output: it does not count)
        row = col = 0
        rset = set(k.red.vars)
        for n in k.red.body.walk():
            if n.k == "load" and rset & set(n.off.vars()):
                if an.stride_of(n.off, rlast) == 1:
                    row += 1
                elif dlast is not None and an.stride_of(n.off, dlast) == 1:
                    col += 1
        if dlast is None or row > col or ON == 1:
            L = self.vec_width_red()
            RY = 256 if RN >= 2048 * max(1, L // 2) else 32
            OX = THREADS // RY
            layout = "row"
        else:
            L, OX, RY, layout = 1, 32, 8, "col"
            if k.red.body.dt == F32 and self.vec_width_domain() == 4:
                groups = (ON // 4 + OX - 1) // OX         # each thread owns 4 consecutive outputs
                S = 1
                per_thread = RN // RY
                if groups < 148 and per_thread >= 64:
                    # enough CTAs for four per SM, each thread still adding eight rows or more
                    S = max(1, min(592 // groups, per_thread // 8, 128))
                return ("coop4", OX, RY, S)
        blocks = (ON + OX - 1) // OX
        S = 1
        per_thread = RN // (RY * L)
        if blocks < 148 and per_thread >= 64:
            S = max(1, min(296 // blocks, per_thread // 32, 64))
        return ("coop", layout, OX, RY, L, S)

    def vec_width_domain(self) -> int:
        k = self.k
        if not k.domain:
            return 1
        vv = k.domain[-1]
        if vv.extent % 4:
            return 1
        offs = list(k.offsets())
        for a in offs:
            st = an.stride_of(a, vv)
            if st is None or st not in (0, 1):
                return 1
            if st == 1 and not an.aligned4(a, vv):
                return 1
        if not any(an.stride_of(s.offset, vv) == 1 for s in k.stores):
            return 1
        return 4

    def vec_width_red(self) -> int:
        k = self.k
        vv = k.red.vars[-1]
        if vv.extent % 4:
            return 1
        for n in k.red.body.walk():
            if n.k in ("load", "index"):
                for a in [n.off] + list(kir._nested(n.off)):
                    st = an.stride_of(a, vv)
                    if st is None or st not in (0, 1):
                        return 1
                    if st == 1 and not an.aligned4(a, vv):
                        return 1
        return 4

    # ---- generation
    def generate(self):
        """Returns (device source, launcher body lines). The launcher receives `rt`, `A`, `st`
        (stream), `sdelta`, `seed`."""
        choice = self.choose()
        self.strategy = choice[0]
        self.zsm_bytes = 0
        self.grid = None
        base = f"k{self.k.id}"
        if choice[0] == "serial":
            return self.gen_serial(base)
        if choice[0] == "gemm":
            return self.gen_gemm(base, choice[1])
        if choice[0] == "eltwise":
            src, launch = self.gen_eltwise(base, choice[1])
        elif choice[0] == "thread":
            src, launch = self.gen_thread(base)
        elif choice[0] == "coop4":
            src, launch = self.gen_coop_col4(base, *choice[1:])
        else:
            return self.gen_coop(base, *choice[1:])
        if self.member:
            assert self.grid is not None
            src += "\n" + self.wrapper(base)
        return src, launch

    @property
    def side(self) -> bool:
        """Does this kernel run on the second stream, beside main-stream kernels? Then partial sums and tickets of a
        split reduction go to a scratch region and counters of their own."""
        return self.k.id in self.gen.side_ids

    @property
    def ticket_base(self) -> int:
        return self.gen.member_slot.get(self.k.id, (0, 0))[1]

    def scratch(self, nbytes: int) -> int:
        if self.member:                                  # members of one launch keep their partial sums apart
            off = self.gen.member_slot[self.k.id][0]
            if self.side:
                self.gen.side_scratch_bytes = max(self.gen.side_scratch_bytes, off + nbytes)
                return self.gen.plan.side_scratch_off + off
            self.gen.need_scratch(off + nbytes)
            return self.gen.plan.scratch_off + off
        if self.side:
            self.gen.side_scratch_bytes = max(self.gen.side_scratch_bytes, nbytes)
            return self.gen.plan.side_scratch_off
        self.gen.need_scratch(nbytes)
        return self.gen.plan.scratch_off

    def launch_line(self, name, blocks, threads) -> str:
        return (f"{name}<<<{blocks}, {threads}, 0, st>>>(A, sdelta, seed); anvil_rt_count_launches(rt, 1);")

    def gen_eltwise(self, base, L):
        k = self.k
        vv = k.domain[-1] if (L > 1 and k.domain) else None
        NT = k.out_numel() // L
        sc = Scope(self, self.names, L, vv)
        sc.statements()
        body = [f"    for (long tid = bx_ * {THREADS}L + threadIdx.x; tid < {NT}L; tid += (long)gdx_ * {THREADS}L) {{",
                f"        const {index_t(NT)} u = ({index_t(NT)})tid;"]
        body += self.decode("u", k.domain, self.names, "        ", vv, L)
        body += self.lane_vars(vv, L, "        ") if vv is not None else []
        src = [self.comment(f"elementwise, {L} element(s) per thread"), self.head(base, THREADS)]
        src += self.pointer_decls() + body + sc.lines + ["    }", "}"]
        blocks = max(1, min((NT + THREADS - 1) // THREADS, MAX_BLOCKS))
        self.grid = (blocks, 1)
        self.notes = f"eltwise x{L}"
        return "\n".join(src), [self.launch_line(base, blocks, THREADS)]

    def red_loops_serial(self, sc: Scope, ind: str) -> list[str]:
        """acc over the whole reduction inside one thread (fixed row-major order)."""
        red = self.k.red
        T = ctype(red.body.dt)
        out = []
        arg = red.op in ("argmax", "argmin")
        if arg:
            init = ("-CUDART_INF_F" if red.op == "argmax" else "CUDART_INF_F") if red.body.dt == F32 else \
                ("(-2147483647 - 1)" if red.op == "argmax" else "2147483647")
            out.append(f"{ind}{T} best = {init}; int acc = 0; long ridx = 0;")
        else:
            out.append(f"{ind}{T} acc = {RED_OP[red.op]}::id<{T}>();")
        inner = ind
        for v in red.vars:
            n = self.names[v]
            out.append(f"{inner}for (int {n} = 0; {n} < {v.extent}; {n}++) {{")
            inner += "    "
        saved_lines, saved_memo, saved_ind = sc.lines, dict(sc.memo), sc.ind
        sc.lines, sc.ind = [], inner
        val = sc.ex(red.body, 0)
        out += sc.lines
        sc.lines, sc.memo, sc.ind = saved_lines, saved_memo, saved_ind
        if arg:
            cmp = ">" if red.op == "argmax" else "<"
            out.append(f"{inner}if ({val} {cmp} best) {{ best = {val}; acc = (int)ridx; }}")
            out.append(f"{inner}ridx++;")
        else:
            out.append(f"{inner}acc = {RED_OP[red.op]}::f(acc, {val});")
        for _ in red.vars:
            inner = inner[:-4]
            out.append(f"{inner}}}")
        return out

    def gen_thread(self, base):
        k = self.k
        NT = k.out_numel()
        sc = Scope(self, self.names)
        red_lines = self.red_loops_serial(sc, "        ")
        sc.statements()
        body = [f"    for (long tid = bx_ * {THREADS}L + threadIdx.x; tid < {NT}L; tid += (long)gdx_ * {THREADS}L) {{",
                f"        const {index_t(NT)} u = ({index_t(NT)})tid;"]
        body += self.decode("u", k.domain, self.names, "        ")
        src = [self.comment("reduction inside the thread"), self.head(base, THREADS)]
        src += self.pointer_decls() + body + red_lines + sc.lines + ["    }", "}"]
        blocks = max(1, min((NT + THREADS - 1) // THREADS, MAX_BLOCKS))
        self.grid = (blocks, 1)
        self.notes = "thread"
        return "\n".join(src), [self.launch_line(base, blocks, THREADS)]

    def gen_serial(self, base):
        k = self.k
        sc = Scope(self, self.names)
        ind = "    "
        lines = []
        for v in k.domain:
            lines.append(f"{ind}for (int {self.names[v]} = 0; {self.names[v]} < {v.extent}; {self.names[v]}++) {{")
            ind += "    "
        sc.ind = ind
        if k.red is not None:
            lines += self.red_loops_serial(sc, ind)
        sc.statements()
        lines += sc.lines
        for _ in k.domain:
            ind = ind[:-4]
            lines.append(f"{ind}}}")
        src = [self.comment("one thread (order-dependent)"), self.head(base, 1)] + self.pointer_decls() + lines + ["}"]
        self.notes = "serial"
        return "\n".join(src), [self.launch_line(base, 1, 1)]

    def gen_coop(self, base, layout, OX, RY, L, S):
        k = self.k
        red = k.red
        ON, RN = k.out_numel(), k.red_numel()
        T = ctype(red.body.dt)
        OP = RED_OP[red.op]
        nthreads = OX * RY
        vv = red.vars[-1] if L > 1 else None
        RNL = RN // L                                    # reduction positions counted in lane groups
        chunk = (RNL + S - 1) // S
        ind = "    "
        lines = []
        if layout == "row":
            lines.append(f"{ind}const int ry = threadIdx.x % {RY}, ox = threadIdx.x / {RY};")
        else:
            lines.append(f"{ind}const int ox = threadIdx.x % {OX}, ry = threadIdx.x / {OX};")
        lines.append(f"{ind}const long o_ = bx_ * {OX}L + ox;")
        lines.append(f"{ind}const bool live = o_ < {ON}L;")
        lines.append(f"{ind}const {index_t(ON)} u = ({index_t(ON)})(live ? o_ : {ON - 1}L);")
        lines += self.decode("u", k.domain, self.names, ind)
        lines.append(f"{ind}{T} acc = {OP}::id<{T}>();")
        lines.append(f"{ind}const long rbeg = by_ * {chunk}L, rend = min({RNL}L, rbeg + {chunk}L);")
        lines.append("#pragma unroll 4")                 # several rows' loads in flight; the adds keep their order
        lines.append(f"{ind}for (long rr_ = rbeg + ry; rr_ < rend; rr_ += {RY}) {{")
        inner = ind + "    "
        lines.append(f"{inner}const {index_t(RNL)} rr = ({index_t(RNL)})rr_;")
        lines += self.decode("rr", red.vars, self.names, inner, vv, L)
        if vv is not None:
            lines += self.lane_vars(vv, L, inner)
        sc = Scope(self, self.names, L, vv, inner)
        vals = [sc.ex(red.body, lane) for lane in range(L)] if sc.depends(red.body) or L == 1 else None
        if vals is None:                                 # the body does not vary along the lanes
            v0 = sc.ex(red.body, 0)
            vals = [v0] * L
        lines += sc.lines
        for v in vals:
            lines.append(f"{inner}acc = {OP}::f(acc, {v});")
        lines.append(f"{ind}}}")
        # combine across ry with a tree whose shape depends only on (layout, RY)
        if layout == "row" and RY <= 32:
            o = RY // 2
            while o >= 1:
                lines.append(f"{ind}acc = {OP}::f(acc, __shfl_xor_sync(0xffffffffu, acc, {o}));")
                o //= 2
        elif layout == "row":
            lines.append(f"{ind}__shared__ {T} sm_[32];")
            lines.append(f"{ind}acc = anvil::block_reduce<{OP}>(acc, sm_);")
        else:
            lines.append(f"{ind}__shared__ {T} sm_[{RY}][{OX + 1}];")
            lines.append(f"{ind}sm_[ry][ox] = acc;")
            lines.append(f"{ind}__syncthreads();")
            s = RY // 2
            while s >= 1:
                lines.append(f"{ind}if (ry < {s}) sm_[ry][ox] = {OP}::f(sm_[ry][ox], sm_[ry + {s}][ox]);")
                lines.append(f"{ind}__syncthreads();")
                s //= 2
            lines.append(f"{ind}acc = sm_[0][ox];")
        tail = Scope(self, self.names, 1, None, ind + "    ")
        launch = []
        gx = (ON + OX - 1) // OX
        if S == 1:
            tail.statements()
            lines.append(f"{ind}if (ry == 0 && live) {{")
            lines += tail.lines
            lines.append(f"{ind}}}")
            src = [self.comment(f"cooperative reduction ({layout}, {OX} outputs x {RY} threads, {L} per load)"),
                   self.head(base, nthreads)] + self.pointer_decls() + lines + ["}"]
            launch.append(self.launch_line(base, f"dim3({gx}, 1)", nthreads))
            self.notes = f"coop {layout} {OX}x{RY} L{L}"
            return "\n".join(src), launch
        # split: partial results to scratch, second kernel combines them in order and runs the statements
        soff = self.scratch(4 * ON * S)
        lines.append(f"{ind}if (ry == 0 && live) (({T} *)(A + {soff}UL))[by_ * {ON}L + o_] = acc;")   # [slice][output]
        part = [self.comment(f"split reduction, part 1 of 2 ({layout}, {S} CTAs per output group)"),
                self.head(base + "_part", nthreads)] + self.pointer_decls() + lines + ["}"]
        # final
        saved = self.ptrs
        self.ptrs = {}
        fsc = Scope(self, self.names, 1, None, "        ")
        fsc.statements()
        fl = [f"    for (long tid = bx_ * {THREADS}L + threadIdx.x; tid < {ON}L; tid += (long)gdx_ * {THREADS}L) {{",
              f"        const {index_t(ON)} u = ({index_t(ON)})tid;"]
        fl += self.decode("u", k.domain, self.names, "        ")
        fl.append(f"        {T} acc = {OP}::id<{T}>();")
        fl.append("#pragma unroll 8")                    # slices are added in index order; the loads run ahead
        fl.append(f"        for (int p = 0; p < {S}; p++) acc = {OP}::f(acc, ((const {T} *)(A + {soff}UL))[p * {ON}L + tid]);")
        final = [self.comment("split reduction, part 2 of 2"), self.head(base, THREADS)] + self.pointer_decls() \
            + fl + fsc.lines + ["    }", "}"]
        self.ptrs = {**saved, **self.ptrs}
        launch.append(self.launch_line(base + "_part", f"dim3({gx}, {S})", nthreads))
        fb = max(1, min((ON + THREADS - 1) // THREADS, MAX_BLOCKS))
        launch.append(self.launch_line(base, fb, THREADS))
        self.notes = f"split {layout} {OX}x{RY} L{L} S{S}"
        return "\n".join(part) + "\n\n" + "\n".join(final), launch


    def gen_coop_col4(self, base, OX, RY, S):
        """Column-layout cooperative reduction where every thread owns 4 consecutive outputs: 128-bit
        loads along the output index, four accumulators, the same fixed trees as `gen_coop`."""
        k = self.k
        red = k.red
        ON, RN = k.out_numel(), k.red_numel()
        OP = RED_OP[red.op]
        vv = k.domain[-1]
        OG = ON // 4
        nthreads = OX * RY
        chunk = (RN + S - 1) // S
        ind = "    "
        lines = [f"{ind}const int ox = threadIdx.x % {OX}, ry = threadIdx.x / {OX};",
                 f"{ind}const long o_ = bx_ * {OX}L + ox;",
                 f"{ind}const bool live = o_ < {OG}L;",
                 f"{ind}const {index_t(OG)} u = ({index_t(OG)})(live ? o_ : {OG - 1}L);"]
        lines += self.decode("u", k.domain, self.names, ind, vv, 4) + self.lane_vars(vv, 4, ind)
        lines.append(f"{ind}float acc_0 = {OP}::id<float>(), acc_1 = acc_0, acc_2 = acc_0, acc_3 = acc_0;")
        lines.append(f"{ind}const long rbeg = by_ * {chunk}L, rend = min({RN}L, rbeg + {chunk}L);")
        lines.append("#pragma unroll 8")                 # several rows' loads in flight; the adds keep their order
        lines.append(f"{ind}for (long rr_ = rbeg + ry; rr_ < rend; rr_ += {RY}) {{")
        inner = ind + "    "
        lines.append(f"{inner}const {index_t(RN)} rr = ({index_t(RN)})rr_;")
        lines += self.decode("rr", red.vars, self.names, inner)
        sc = Scope(self, self.names, 4, vv, inner)
        dep = sc.depends(red.body)
        vals = [sc.ex(red.body, lane if dep else 0) for lane in range(4)]
        lines += sc.lines
        for i, v in enumerate(vals):
            lines.append(f"{inner}acc_{i} = {OP}::f(acc_{i}, {v});")
        lines.append(f"{ind}}}")
        W = 4 * OX + 4
        self.zsm_bytes = RY * W * 4 + 16
        if self.member:                                  # shared memory comes from the launch this kernel is a member of
            lines.append(f"{ind}float (*sm_)[{W}] = reinterpret_cast<float (*)[{W}]>(zsm_);")
        else:
            lines.append(f"{ind}__shared__ float sm_[{RY}][{W}];")
        for i in range(4):
            lines.append(f"{ind}sm_[ry][4 * ox + {i}] = acc_{i};")
        lines.append(f"{ind}__syncthreads();")
        s_ = RY // 2
        while s_ >= 1:
            lines.append(f"{ind}if (ry < {s_}) {{ " + " ".join(
                f"sm_[ry][4 * ox + {i}] = {OP}::f(sm_[ry][4 * ox + {i}], sm_[ry + {s_}][4 * ox + {i}]);" for i in range(4)) + " }")
            lines.append(f"{ind}__syncthreads();")
            s_ //= 2
        for i in range(4):
            lines.append(f"{ind}acc_{i} = sm_[0][4 * ox + {i}];")
        gx = (OG + OX - 1) // OX
        launch = []
        if S == 1:
            tail = Scope(self, self.names, 4, vv, ind + "    ")
            tail.acc_lanes = True
            tail.statements()
            lines.append(f"{ind}if (ry == 0 && live) {{")
            lines += tail.lines
            lines.append(f"{ind}}}")
            src = [self.comment(f"cooperative reduction (col, {OX} x 4 outputs x {RY} threads)"),
                   self.head(base, nthreads)] + self.pointer_decls() + lines + ["}"]
            launch.append(self.launch_line(base, f"dim3({gx}, 1)", nthreads))
            self.grid = (gx, 1)
            self.notes = f"coop col4 {OX}x{RY}"
            return "\n".join(src), launch
        # Split over S CTAs per output group, finished by whichever of them arrives last: every CTA writes its partial
        # sums to scratch and takes a ticket; the last one adds all S partials in a fixed order (slice ry takes partials
        # ry, ry + RY, ..., then the same shared-memory tree) and runs the statements. The result does not depend on which
        # CTA is last, and there is no second launch.
        soff = self.scratch(4 * ON * S)
        assert gx <= 256, "ticket counters"
        tree = []
        for i in range(4):
            tree.append(f"{ind}sm_[ry][4 * ox + {i}] = acc_{i};")
        tree.append(f"{ind}__syncthreads();")
        s_ = RY // 2
        while s_ >= 1:
            tree.append(f"{ind}if (ry < {s_}) {{ " + " ".join(
                f"sm_[ry][4 * ox + {i}] = {OP}::f(sm_[ry][4 * ox + {i}], sm_[ry + {s_}][4 * ox + {i}]);" for i in range(4)) + " }")
            tree.append(f"{ind}__syncthreads();")
            s_ //= 2
        for i in range(4):
            tree.append(f"{ind}acc_{i} = sm_[0][4 * ox + {i}];")
        lines.append(f"{ind}float *part_ = (float *)(A + {soff}UL);")
        lines.append(f"{ind}if (ry == 0 && live) *reinterpret_cast<float4 *>(part_ + by_ * {ON}L + o_ * 4) = make_float4(acc_0, acc_1, acc_2, acc_3);")
        last_decl = (f"{ind}unsigned &last_ = *reinterpret_cast<unsigned *>(zsm_ + {RY * W * 4});" if self.member
                     else f"{ind}__shared__ unsigned last_;")
        lines += [f"{ind}__threadfence();", last_decl, f"{ind}__syncthreads();",
                  f"{ind}unsigned *ticket_ = (unsigned *)(A + {'ANVIL_RT_SIDE_TICKETS_OFF' if self.side else 'ANVIL_RT_TICKETS_OFF'}) + {self.ticket_base}u + bx_;",
                  f"{ind}if (threadIdx.x == 0) last_ = atomicAdd(ticket_, 1u) == {S - 1}u;",
                  f"{ind}__syncthreads();", f"{ind}if (!last_) return;", f"{ind}__threadfence();"]
        for i in range(4):
            lines.append(f"{ind}acc_{i} = {OP}::id<float>();")
        lines.append(f"{ind}if (live) {{")
        lines.append("#pragma unroll 16")               # all of a thread's partials in flight at once: one trip to L2
        lines.append(f"{ind}    for (int p = ry; p < {S}; p += {RY}) {{")
        lines.append(f"{ind}        const float4 q_ = __ldcg(reinterpret_cast<const float4 *>(part_ + p * {ON}L + o_ * 4));")
        for i, c in enumerate("xyzw"):
            lines.append(f"{ind}        acc_{i} = {OP}::f(acc_{i}, q_.{c});")
        lines.append(f"{ind}    }}")
        lines.append(f"{ind}}}")
        lines.append(f"{ind}__syncthreads();")
        lines += tree
        lines.append(f"{ind}if (threadIdx.x == 0) *ticket_ = 0u;")
        tail = Scope(self, self.names, 4, vv, ind + "    ")
        tail.acc_lanes = True
        tail.statements()
        lines.append(f"{ind}if (ry == 0 && live) {{")
        lines += tail.lines
        lines.append(f"{ind}}}")
        src = [self.comment(f"split reduction finished by the last CTA (col, 4 outputs per thread, {S} CTAs per output group)"),
               self.head(base, nthreads)] + self.pointer_decls() + lines + ["}"]
        launch.append(self.launch_line(base, f"dim3({gx}, {S})", nthreads))
        self.grid = (gx, S)
        self.notes = f"split col4 {OX}x{RY} S{S}"
        return "\n".join(src), launch

    # ---- contractions
    def functor_method(self, sig: str, decodes: list, build) -> list[str]:
        """One __device__ method of a contraction functor: index decode, pointers, body."""
        saved = self.ptrs
        self.ptrs = {}
        sc = Scope(self, self.names, 1, None, "        ")
        ret = build(sc)
        decls = ["    " + ln for ln in self.pointer_decls()]
        out = [f"    __device__ __forceinline__ {sig} const {{"] + decls + decodes + sc.lines
        if ret is not None:
            out.append(f"        return {ret};")
        out.append("    }")
        self.ptrs = {**saved, **self.ptrs}
        return out

    def gen_gemm(self, base, c):
        k = self.k
        M, N, K, NB = c.M, c.N, c.K, c.NB
        fa, fb, fe = self.gemm_functors(c)
        tiles = ((M + 127) // 128) * ((N + 127) // 128)
        S = 1
        if tiles * NB < 148 and K >= 256:
            S = max(1, min(296 // (tiles * NB), K // 128, 32))
        AK, BNC = ("true" if c.a_kcontig else "false"), ("true" if c.b_ncontig else "false")
        fn = f"G{k.id}"
        if tc_eligible(c):
            return self.gen_gemm_tc(base, c, fn, fa, fb, fe, S)
        return self.gen_gemm_simt(base, c, fn, fa, fb, fe, S, tiles, AK, BNC)

    def gemm_functors(self, c):
        """The functor methods every contraction template takes: a / b (one operand element), epi (the statements on
        one accumulator), epi_touch (L2 prefetch of what they read), and the two-phase form epi_loads / epi2."""
        k = self.k
        M, N, K, NB = c.M, c.N, c.K, c.NB
        ind = "        "
        dm = self.decode("(uint32_t)m", c.mvars, self.names, ind)
        dn = self.decode("(uint32_t)n", c.nvars, self.names, ind)
        dk = self.decode("(uint32_t)k", c.kvars, self.names, ind)
        db = self.decode("(uint32_t)bt", c.bvars, self.names, ind) if c.bvars else []
        fa = self.functor_method("float a(int m, int k, int bt)", dm + dk + db, lambda sc: sc.ex(c.a, 0))
        fb = self.functor_method("float b(int k, int n, int bt)", dk + dn + db, lambda sc: sc.ex(c.b, 0))

        def epi(sc):
            sc.statements()
            return None
        fe = self.functor_method("void epi(int m, int n, int bt, float acc)", dm + dn + db, epi)

        def touch(sc):
            # L2 prefetch of what the statements read at element (m, n): residuals, `+=` targets. The
            # resident tensor-core template issues it one tile ahead of the epilogue that needs it.
            seen = set()
            reads = [(n.buf, n.off) for st in k.stmts for n in st.value.walk() if n.k == "load"]
            reads += [(st.buf, st.offset) for st in k.stmts if isinstance(st, kir.Store) and st.accumulate]
            for buf, off in reads:
                if not off.is_plain() or off.scalars() or (buf.root.id, off.key()) in seen:
                    continue
                vs = off.vars()
                if not (any(v in vs for v in c.mvars) and any(v in vs for v in c.nvars)):
                    continue                                 # a bias row or a per-row scalar: cached anyway
                seen.add((buf.root.id, off.key()))
                sc.emit(f"anvil::{self.prefetch}({self.ptr(buf, False)} + ({sc.affine(off, 0)}));")
            return None
        self.prefetch = "prefetch_l2"
        fe = fe + self.functor_method("void epi_touch(int m, int n, int bt)", dm + dn + db, touch)
        self.prefetch = "prefetch_l1"                        # the same lines into L1, right before the epilogue reads them
        fe = fe + self.functor_method("void epi_near(int m, int n, int bt)", dm + dn + db, touch)

        # Two-phase form of the statements: epi_loads fetches what they read at (m, n) — tensors this kernel
        # never writes, and the old value of an exclusive `+=` — and epi2 runs them on those values, so a
        # caller can issue the loads of several rows before the first store.
        # A per-element read may move in front of all stores when nothing can have written that element yet:
        # the tensor is never stored by this kernel, or every store to it is exclusive, hits exactly the element
        # read, and comes no earlier than the last statement that reads it (the old value of `+=`, the moments
        # of an Adam update).
        stores_of: dict = {}
        for si, st in enumerate(k.stmts):
            if isinstance(st, kir.Store):
                stores_of.setdefault(st.buf.root.id, []).append((si, st))
        reads: dict = {}                                     # (root, offset key) -> [buffer, offset, last reading statement]
        for si, st in enumerate(k.stmts):
            found = [(n.buf, n.off) for n in st.value.walk() if n.k == "load" and n.dt == F32]
            if isinstance(st, kir.Store) and st.accumulate and st.buf.dtype == F32:
                found.append((st.buf, st.offset))
            for buf, off in found:
                r = reads.setdefault((buf.root.id, off.key()), [buf, off, si])
                r[2] = max(r[2], si)
        pre: list = []
        for (root, okey), (buf, off, last_read) in reads.items():
            vs = off.vars()
            if not off.is_plain() or not (any(v in vs for v in c.mvars) and any(v in vs for v in c.nvars)):
                continue
            ok = all(sj >= last_read and st.offset.key() == okey and an.exclusive_store(k, st)
                     for sj, st in stores_of.get(root, []))
            other_reads = [key for key in reads if key[0] == root and key[1] != okey]
            if ok and not (stores_of.get(root) and other_reads) and len(pre) < 4:
                pre.append((buf, off, bool(stores_of.get(root))))
        nld = len(pre)

        def loads(sc):
            for i, (buf, off, _) in enumerate(pre):
                sc.emit(f"ld[{i}] = {self.ptr(buf, False)}[{sc.affine(off, 0)}];")
            return None

        def epi2(sc):
            sc.preloaded = {(buf.root.id, off.key()): f"ld[{i}]" for i, (buf, off, _) in enumerate(pre)}
            sc.statements()
            return None
        fe = fe + [f"    static constexpr int NLD = {nld};"]
        fe = fe + self.functor_method(f"void epi_loads(int m, int n, int bt, float (&ld)[{max(nld, 1)}])", dm + dn + db, loads)
        fe = fe + self.functor_method(f"void epi2(int m, int n, int bt, float acc, const float (&ld)[{max(nld, 1)}])", dm + dn + db, epi2)
        self.nld = nld
        return fa, fb, fe

    def gen_gemm_simt(self, base, c, fn, fa, fb, fe, S, tiles, AK, BNC):
        k = self.k
        M, N, K, NB = c.M, c.N, c.K, c.NB
        src = [self.comment(f"contraction M={M} N={N} K={K} batch={NB} (CUDA-core tiles, split {S})"),
               f"struct {fn} {{", "    char *__restrict__ A;",
               f"    static constexpr int M = {M}, N = {N}, K = {K}, NB = {NB};",
               f"    static constexpr float ALPHA = {flit(c.alpha)};"] + fa + fb + fe + ["};"]
        launch = []
        if S == 1:
            src += [f"__global__ void __launch_bounds__(256) {base}(char *__restrict__ A, uint32_t sdelta, uint32_t seed_) {{",
                    f"    anvil::gemm_simt_tile<{fn}, {AK}, {BNC}, 1>({fn}{{A}}, nullptr);", "}"]
            launch.append(self.launch_line(base, f"dim3({tiles}, {NB})", 256))
        else:
            soff = self.scratch(4 * M * N * NB * S)
            src += [f"__global__ void __launch_bounds__(256) {base}_part(char *__restrict__ A, uint32_t sdelta, uint32_t seed_) {{",
                    f"    anvil::gemm_simt_tile<{fn}, {AK}, {BNC}, {S}>({fn}{{A}}, (float *)(A + {soff}UL));", "}",
                    f"__global__ void __launch_bounds__(256) {base}(char *__restrict__ A, uint32_t sdelta, uint32_t seed_) {{",
                    f"    anvil::gemm_split_finish<{fn}, {S}>({fn}{{A}}, (const float *)(A + {soff}UL));", "}"]
            launch.append(self.launch_line(base + "_part", f"dim3({tiles}, {NB * S})", 256))
            fb_ = max(1, min((M * N * NB + 255) // 256, MAX_BLOCKS))
            launch.append(self.launch_line(base, fb_, 256))
        self.notes = f"gemm simt {NB}x{M}x{N}x{K} S{S}"
        self.contraction = c
        return "\n".join(src), launch


    def functor4(self, sig: str, c, operand, pre: list, kvars) -> list[str]:
        """`a4` / `b4`: four consecutive k of one operand row, 128-bit loads where the operand is
        contiguous and aligned along k."""
        saved = self.ptrs
        self.ptrs = {}
        vv = kvars[-1]
        ind = "        "
        if vv.extent % 4:
            # the innermost reduction index is not a multiple of 4 long (a 3 x 3 window): the four k are decoded one by one
            lines, vals = [], []
            for lane in range(4):
                names = dict(self.names)
                for v in kvars:
                    names[v] = f"{self.names[v]}_{lane}"
                lines += self.decode(f"(uint32_t)(k + {lane})", kvars, names, ind)
                sc = Scope(self, names, 1, None, ind)
                vals.append(sc.ex(operand, 0))
                lines += sc.lines
            decls = ["    " + ln for ln in self.pointer_decls()]
            out = [f"    __device__ __forceinline__ {sig} const {{"] + decls + pre + lines
            out += [f"{ind}v[{i}] = {x};" for i, x in enumerate(vals)] + ["    }"]
            self.ptrs = {**saved, **self.ptrs}
            return out
        dk = self.decode("((uint32_t)k >> 2)", kvars, self.names, ind, vv, 4) + self.lane_vars(vv, 4, ind)
        sc = Scope(self, self.names, 4, vv, ind)
        vals = [sc.ex(operand, lane) for lane in range(4)]
        decls = ["    " + ln for ln in self.pointer_decls()]
        out = [f"    __device__ __forceinline__ {sig} const {{"] + decls + pre + dk + sc.lines
        out += [f"{ind}v[{i}] = {x};" for i, x in enumerate(vals)] + ["    }"]
        self.ptrs = {**saved, **self.ptrs}
        return out

    def tc_operands(self, c, touch: bool):
        """a4 / b4 (four consecutive k of one operand row) and, for the resident template, a_touch / b_touch."""
        ind = "        "
        dm = self.decode("(uint32_t)m", c.mvars, self.names, ind)
        dn = self.decode("(uint32_t)n", c.nvars, self.names, ind)
        db = self.decode("(uint32_t)bt", c.bvars, self.names, ind) if c.bvars else []
        fa4 = self.functor4("void a4(int m, int k, int bt, float (&v)[4])", c, c.a, dm + db, c.kvars)
        fb4 = self.functor4("void b4(int k, int n, int bt, float (&v)[4])", c, c.b, dn + db, c.kvars)
        if touch:                                # L2 prefetch of the operand element (m, k) / (k, n): issued some blocks ahead
            dks = self.decode("(uint32_t)k", c.kvars, self.names, ind)

            def operand_touch(operand):
                def build(sc):
                    seen = set()
                    for nd in operand.walk():
                        if nd.k == "load" and nd.off.is_plain() and (nd.buf.root.id, nd.off.key()) not in seen:
                            seen.add((nd.buf.root.id, nd.off.key()))
                            sc.emit(f"anvil::prefetch_l2({self.ptr(nd.buf, False)} + ({sc.affine(nd.off, 0)}));")
                    return None
                return build
            fa4 = fa4 + self.functor_method("void a_touch(int m, int k, int bt)", dm + dks + db, operand_touch(c.a))
            fb4 = fb4 + self.functor_method("void b_touch(int k, int n, int bt)", dn + dks + db, operand_touch(c.b))
        return fa4, fb4

    def tc_struct(self, c, fn, fe, touch: bool) -> list[str]:
        fa4, fb4 = self.tc_operands(c, touch)
        return [f"struct {fn} {{", "    char *__restrict__ A;",
                f"    static constexpr int M = {c.M}, N = {c.N}, K = {c.K}, NB = {c.NB};",
                f"    static constexpr float ALPHA = {flit(c.alpha)};"] + fa4 + fb4 + fe + ["};"]

    def gen_gemm_tc(self, base, c, fn, fa, fb, fe, S):
        k = self.k
        M, N, K, NB = c.M, c.N, c.K, c.NB
        nstores = sum(1 for st in k.stmts if isinstance(st, kir.Store))
        variant = tc_variant(c.a_kcontig, M, N, K, nstores)
        fa4, fb4 = self.tc_operands(c, variant == "pp")
        pp = variant == "pp"
        pair = variant == "pair" or pp
        if pair:                                 # 256 x BN tile per cluster of two CTAs
            BN = 256 if N >= 256 else 128 if N >= 128 or not pp else 64
            if pp and BN == 256 and K <= 1024 and ((M + 255) // 256) * ((N + 255) // 256) * NB < 74:
                BN = 128                         # too few 256-wide tiles for the 74 clusters: narrower tiles before any k split
            tiles = ((M + 255) // 256) * ((N + BN - 1) // BN)
            slots = 74
        else:
            BN = 128 if N >= 128 else 64
            tiles = ((M + 127) // 128) * ((N + BN - 1) // BN)
            slots = 148
        S = 1
        if tiles * NB < slots and K >= 256:
            S = max(1, min(slots // (tiles * NB), K // 128, 32))
        S = max(S, (K + 4095) // 4096)           # one accumulation chain stays <= 4096 long (rounding, see the header)
        AK = "true" if c.a_kcontig else "false"
        BKC = "true" if ct._contig(c.b, c.kvars[-1]) else "false"
        src = [self.comment(f"contraction M={M} N={N} K={K} batch={NB} (tcgen05 3xTF32, {256 if pair else 128}x{BN} tiles, split {S})"),
               f"struct {fn} {{", "    char *__restrict__ A;",
               f"    static constexpr int M = {M}, N = {N}, K = {K}, NB = {NB};",
               f"    static constexpr float ALPHA = {flit(c.alpha)};"] + fa4 + fb4 + fe + ["};"]
        # A in tensor memory pays off when A is read along m (lane = row gives coalesced loads); a
        # k-contiguous A is read faster by the shared-memory variant's 8-lanes-per-row mapping
        ts = variant == "ts"
        tile_tail = ">"
        attrs = ""
        grid_x = 2 * tiles if pair else tiles
        grid_y = NB * S
        if pp:                                   # resident clusters walk over (tile, batch, split) items
            accs = 1 if (K + S - 1) // S <= 512 and BN == 256 else 2
            smem, threads, per_sm = f"anvil::tc::pp_smem_bytes({BN})", "anvil::tc::PP_THREADS", 1
            tile_fn = f"anvil::tc::gemm_tc_pair_persistent<{fn}, {AK}, {BKC}, "
            tile_tail = f", {accs}, {BN}>"
            attrs = "__cluster_dims__(2, 1, 1) "
            grid_x, grid_y = 2 * min(tiles * NB * S, 74), 1
        elif pair:
            smem, threads, per_sm = f"anvil::tc::pair_smem_bytes({BN})", "anvil::tc::THREADS", 1
            tile_fn = f"anvil::tc::gemm_tc_pair_tile<{fn}, {AK}, {BKC}, {BN}, "
            attrs = "__cluster_dims__(2, 1, 1) "
        elif ts:
            smem, threads, per_sm = f"anvil::tc::ts_smem_bytes({BN})", "anvil::tc::THREADS", 1
            tile_fn = f"anvil::tc::gemm_tc_ts_tile<{fn}, {BKC}, {BN}, "
        elif variant == "ss32":
            smem, threads, per_sm = f"anvil::tc::smem_bytes({BN})", "anvil::tc::THREADS", 1
            tile_fn = f"anvil::tc::gemm_tc_tile<{fn}, {AK}, {BKC}, {BN}, "
        else:
            smem, threads, per_sm = f"anvil::tc::smem2_bytes({BN})", "anvil::tc::THREADS2", 2
            tile_fn = f"anvil::tc::gemm_tc2_tile<{fn}, {AK}, {BKC}, {BN}, "
        status = "(uint32_t *)(A + ANVIL_RT_STATUS_OFF)"
        launch = []
        if S == 1:
            kname = base
            src += [f"__global__ void {attrs}__launch_bounds__({threads}, {per_sm}) {base}(char *__restrict__ A, uint32_t sdelta, uint32_t seed_) {{",
                    f"    {tile_fn}1{tile_tail}({fn}{{A}}, nullptr, {status});", "}"]
        else:
            kname = base + "_part"
            soff = self.scratch(4 * M * N * NB * S)
            src += [f"__global__ void {attrs}__launch_bounds__({threads}, {per_sm}) {kname}(char *__restrict__ A, uint32_t sdelta, uint32_t seed_) {{",
                    f"    {tile_fn}{S}{tile_tail}({fn}{{A}}, (float *)(A + {soff}UL), {status});", "}",
                    f"__global__ void __launch_bounds__(256) {base}(char *__restrict__ A, uint32_t sdelta, uint32_t seed_) {{",
                    f"    anvil::gemm_split_finish<{fn}, {S}>({fn}{{A}}, (const float *)(A + {soff}UL));", "}"]
        tma = pp and use_tma() and tma_kernel(self.gen, src, launch, kname, fn, c, c, AK, BKC, S, accs, BN, status,
                                              f"(float *)(A + {soff}UL)" if S > 1 else "nullptr",
                                              f"dim3({grid_x}, {grid_y})", smem)
        if not tma:
            launch.append(f"{{ static bool attr_ = false; if (!attr_) {{ cudaFuncSetAttribute({kname}, "
                          f"cudaFuncAttributeMaxDynamicSharedMemorySize, (int){smem}); attr_ = true; }} }}")
            launch.append(f"{kname}<<<dim3({grid_x}, {grid_y}), {threads}, {smem}, st>>>(A, sdelta, seed); anvil_rt_count_launches(rt, 1);")
        if S > 1:
            fb_ = max(1, min((M * N * NB + 255) // 256, MAX_BLOCKS))
            launch.append(self.launch_line(base, fb_, 256))
        self.notes = f"gemm tc {NB}x{M}x{N}x{K} S{S}" + (" A-tmem" if ts else " pp" if pp else " pair" if pair else "")
        self.contraction = c
        return "\n".join(src), launch


def os_environ(name: str, default: str) -> str:
    import os
    return os.environ.get(name, default)


def use_hoist() -> bool:
    """Moving second-stream launches up to just after what they depend on (the weight gradients of a layer beside the
    backward pass of the layers below) is built but off: measured on a B200 it does not shorten the step (14.37 against
    14.27 ms). A resident kernel's CTAs hold their SMs until their statically assigned tiles are done, so a second
    resident kernel gets SMs only as the first one's CTAs exit, wherever in the step it was launched. ANVIL_B200_HOIST=1
    turns it on."""
    import os
    return os.environ.get("ANVIL_B200_HOIST", "0") == "1"


def use_side_gemms() -> bool:
    import os
    return os.environ.get("ANVIL_B200_SIDE_GEMMS", "1") != "0"


def use_zgroups() -> bool:
    import os
    return os.environ.get("ANVIL_B200_ZGROUPS", "1") != "0"


def use_side_stream() -> bool:
    import os
    return os.environ.get("ANVIL_B200_SIDE", "1") != "0"


def use_attention() -> bool:
    import os
    return os.environ.get("ANVIL_B200_ATTENTION", "1") != "0" and os.environ.get("ANVIL_B200_TC", "1") in ("1", "pp")


def use_hgroups() -> bool:
    import os
    return os.environ.get("ANVIL_B200_HGROUPS", "1") != "0" and os.environ.get("ANVIL_B200_TC", "1") in ("1", "pp")


def tc_eligible_pp(c) -> bool:
    """Takes the resident pair template by the emitter's own choice."""
    nstores = sum(1 for st in c.kernel.stmts if isinstance(st, kir.Store))
    return tc_eligible(c) and tc_variant(c.a_kcontig, c.M, c.N, c.K, nstores) == "pp"


def fused_runs(kernels, attention_spans=()):
    """Index ranges of consecutive kernels that run as ONE launch (fused attention, horizontal contraction groups,
    fused row groups): the arena planner treats each as one statement."""
    out = [(a, b) for a, b, _ in attention_spans]
    more = list(rg.find_groups(kernels)) if use_row_groups() else []
    if use_hgroups():
        more += [(a, b) for a, b, _ in hfuse.find_hgroups(kernels, tc_eligible_pp)]
    for a, b in more:
        if not any(a < y and x < b for x, y in out):
            out.append((a, b))
    return out


def use_row_groups() -> bool:
    import os
    return os.environ.get("ANVIL_B200_ROWGROUPS", "1") != "0"


def use_tensor_cores() -> bool:
    import os
    return os.environ.get("ANVIL_B200_TC", "1") != "0"


def tc_eligible(c) -> bool:
    """Does this contraction take a tensor-core template? K must be a multiple of 4 (operands are converted four
    consecutive k at a time), the tile must not be mostly empty, and the product must be worth a tensor-core launch."""
    return use_tensor_cores() and c.K % 4 == 0 and c.M >= 96 and c.N >= 64 and c.K >= 64 and c.flops >= tc_min_flops()


def pp_launch_params(M, N, K, NB, max_bn=256):
    """(BN, split, accumulators, work items) of the resident pair template for a shape."""
    BN = 256 if N >= 256 and max_bn >= 256 else 128 if N >= 128 else 64
    if BN == 256 and K <= 1024 and ((M + 255) // 256) * ((N + 255) // 256) * NB < 74:
        BN = 128                         # too few 256-wide tiles for the 74 clusters: narrower tiles before any k split
    tiles = ((M + 255) // 256) * ((N + BN - 1) // BN)
    S = 1
    if tiles * NB < 74 and K >= 256:
        S = max(1, min(74 // (tiles * NB), K // 128, 32))
    S = max(S, (K + 4095) // 4096)       # one accumulation chain stays <= 4096 long (rounding, see the template's header)
    accs = 1 if (K + S - 1) // S <= 512 and BN == 256 else 2
    return BN, S, accs, tiles * NB * S


def use_tma() -> bool:
    """The TMA operand feed of the resident pair template is built and parity-tested but off by default: measured on a
    B200 it is slower than the converters' own loads (16384 x 512 x 512: 72 us against 49 us). The stage ring holds three
    66 KB stages (hi and lo tiles of both operands, 198 of 227 KB), so only one block's copy can be in flight while the
    tensor core works on one stage and the converters make lo for the next, and a copy takes longer than a block's MMAs;
    the load path keeps two blocks' operands in registers and asks L2 for four more. ANVIL_B200_TMA=1 turns it on."""
    import os
    return os.environ.get("ANVIL_B200_TMA", "0") == "1"


def tma_operand(c, operand, row_vars):
    """(root buffer, element offset, rows, row stride) when `operand` of contraction `c` can come by TMA: one plain load
    of a row-major matrix read along k with 16-byte aligned rows — no prologue, no gather, no batch."""
    if c.bvars or len(c.kvars) != 1 or operand.k != "load" or operand.dt != F32 or not operand.off.is_plain():
        return None
    off, kv = operand.off, c.kvars[0]
    if off.coef(kv) != 1 or off.const % 4 or c.K % 4:
        return None
    live = [v for v in row_vars if v.extent > 1]
    if not live or set(off.vars()) - set(live) - {kv}:
        return None
    stride = off.coef(live[-1])
    if stride <= 0 or stride % 4 or stride < c.K:
        return None
    for v, s_ in zip(live, kir.row_major_strides([v.extent for v in live])):
        if off.coef(v) != s_ * stride:
            return None                              # the row vars do not flatten into one row index
    return operand.buf.root, off.const, kir.prod(v.extent for v in live), stride


def tc_min_flops() -> int:
    """Products below this many FLOPs stay on the CUDA-core template: exact f32 products added in k order, no
    3xTF32 split, and nothing to gain from the tensor pipe at that size (a launch costs more than the arithmetic).
    ANVIL_B200_TC_MIN_MFLOP overrides the default of 128 MFLOP."""
    import os
    if os.environ.get("ANVIL_B200_TC", "1") in ("pp", "pair", "ts", "ss", "ss32"):
        return 0                                     # a template forced by name is taken at any size
    return int(float(os.environ.get("ANVIL_B200_TC_MIN_MFLOP", "128")) * 1e6)


def tc_variant(a_kcontig: bool, M: int, N: int, K: int, nstores: int = 1) -> str:
    """Which tcgen05 template a contraction takes (ANVIL_B200_TC=pp|pair|ss|ss32|ts forces one where it applies):
    "pp"   resident clusters of two CTAs on 256 x 256 tiles (tcgen05.mma.cta_group::2), converter / MMA /
           epilogue warps overlapping across tiles — needs M >= 256 and N >= 128; the default there
           (16384x2048x512: 232-245 TFLOP/s against 150-154 for "ss32");
    "pair" the same tile, one launch-time CTA pair per tile (kept for comparison);
    "ts"   A tiles in tensor memory — when A is read along m and the output is narrow;
    "ss"   operands in shared memory, 16-wide k blocks, two CTAs per SM — short reductions (K <= 128)
           on narrow outputs;
    "ss32" operands in shared memory, 32-wide k blocks, one CTA per SM — the remaining shapes."""
    import os
    v = os.environ.get("ANVIL_B200_TC", "1")
    pair_ok = M >= 256 and N >= 128
    pp_ok = M >= 256 and N >= 64
    if (v == "pair" and not pair_ok) or (v == "pp" and not pp_ok):
        v = "1"
    if v in ("pair", "pp", "ss", "ts", "ss32"):
        return v
    if pp_ok and K <= 128 and nstores >= 2 and a_kcontig:
        return "ss"                  # two blocks of main loop per tile and two outputs: all warps of "ss" store (34 vs 27 TFLOP/s)
    if pp_ok:
        return "pp"
    if not a_kcontig:
        return "ts"
    return "ss" if K <= 128 else "ss32"


class RowScope(Scope):
    """Scope of one kernel inside a fused row group: loads of elements an earlier kernel of the
    group produced come from registers, stores to tensors nothing else reads are dropped."""

    def __init__(self, gg: "RowGroupGen", form, lanes, ind):
        names = {}
        if form.rowvar is not None:
            names[form.rowvar] = "row"
        names[form.jvar] = "cv" if form.collapsed else "j"
        super().__init__(gg, names, lanes, form.jvar if lanes > 1 else None, ind)
        self.gg = gg
        self.form = form
        self.scalar_stores: list[str] = []

    def key(self, buf, off):
        return (buf.root.id,) + tuple(self.form.canon(off))

    def load(self, e: kir.E, lane) -> str:
        key = self.key(e.buf, e.off)
        hit = self.gg.fwd.get(key)
        if hit is not None:
            return hit[lane] if key[2] == 1 else hit[0]
        return super().load(e, lane)

    def store(self, st: kir.Store):
        key = self.key(st.buf, st.offset)
        L = self.lanes
        vec = key[2] == 1
        vals = [self.cast(st.value, st.buf.dtype, lane) for lane in (range(L) if vec else [0])]
        if st.accumulate:                                # read-modify-write of the element this thread owns
            prev = self.gg.fwd.get(key)
            p = self.kg.ptr(st.buf, True)
            out = []
            for i, v in enumerate(vals):
                old = prev[i] if prev is not None else f"{p}[{self.affine(st.offset, i)}]"
                name = self.kg.tmp()
                self.emit(f"const float {name} = ({old}) + ({v});")
                out.append(name)
            vals = out
        else:
            out = []
            for v in vals:                               # name the value so later phases can reuse it
                name = self.kg.tmp()
                self.emit(f"const float {name} = {v};")
                out.append(name)
            vals = out
        self.gg.fwd[key] = vals
        if st.buf.root.id in self.gg.dead:
            return
        p = self.kg.ptr(st.buf, True)
        if not vec:
            self.emit(f"if (tt == 0 && live) {p}[{self.affine(st.offset, 0)}] = {vals[0]};")
            return
        self.emit("if (live) {")
        if an.aligned4(st.offset, self.vv) and L % 4 == 0:
            for g in range(0, L, 4):
                self.emit(f"    anvil::st4({p} + ({self.affine(st.offset, g)}), make_float4({', '.join(vals[g:g + 4])}));")
        else:
            for lane in range(L):
                self.emit(f"    {p}[{self.affine(st.offset, lane)}] = {vals[lane]};")
        self.emit("}")


class RowGroupGen:
    """A fused row group (see rowgroup.py) -> one __global__ function and a launcher."""

    def __init__(self, gen: "ProgramGen", forms, dead: set):
        self.gen = gen
        self.forms = forms
        self.dead = dead
        self.n = 0
        self.ptrs: dict = {}
        self.fwd: dict = {}              # (root, a, b, const) -> list of C identifiers
        self.parallel = True
        self.uses_rand = False
        self.k = forms[0].kernel
        self.written = set()
        for f in forms:
            self.written |= {s.buf.root.id for s in f.kernel.stores}

    def tmp(self, prefix="t") -> str:
        self.n += 1
        return f"{prefix}{self.n}"

    def ptr(self, b: kir.Buffer, write: bool) -> str:
        r = b.root
        self.ptrs[r.id] = (r, r.id in self.written)
        return f"b{r.id}"

    def rand_varies_with(self, vv) -> bool:
        return False

    def generate(self, name: str):
        R, N = self.forms[0].R, self.forms[0].N
        T = rg.threads_per_row(N)
        E = N // T
        RB = rg.THREADS // T
        ind = "    "
        body = []
        for pi, f in enumerate(self.forms):
            k = self.k = f.kernel
            body.append(f"{ind}// ---- {k.name} <{k.label}>")
            if f.kind == "red":
                sc = RowScope(self, f, E, ind)
                dep = sc.depends(k.red.body)
                vals = [sc.ex(k.red.body, lane if dep else 0) for lane in range(E)]
                body += sc.lines
                OP = RED_OP[k.red.op]
                acc = f"acc{pi}"
                body.append(f"{ind}float {acc} = {OP}::id<float>();")
                for v in vals:
                    body.append(f"{ind}{acc} = {OP}::f({acc}, {v});")
                body.append(f"{ind}{acc} = anvil::row_reduce<{OP}, {T}>({acc}, red_);")
                tail = RowScope(self, f, 1, ind)
                tail.acc_name = acc
                tail.statements()
                body += tail.lines
            else:
                sc = RowScope(self, f, E, ind)
                sc.statements()
                body += sc.lines
        head = [f"// fused row group: {' + '.join(f.kernel.name for f in self.forms)} | {R} rows x {N} | "
                f"{T} threads per row, {E} elements each",
                f"__global__ void __launch_bounds__({rg.THREADS}) {name}(char *__restrict__ A, uint32_t sdelta, uint32_t seed_) {{"]
        decls = []
        for rid, (r, w) in sorted(self.ptrs.items()):
            Tn = ctype(r.dtype)
            off = self.gen.plan.offsets[rid]
            if w:
                decls.append(f"    {Tn} *b{rid} = ({Tn} *)(A + {off}UL);   // {r.name}{list(r.shape)}")
            else:
                decls.append(f"    const {Tn} *__restrict__ b{rid} = (const {Tn} *)(A + {off}UL);   // {r.name}{list(r.shape)}")
        decls += [f"    __shared__ float red_[8];",
                  f"    const int tt = threadIdx.x % {T};",
                  f"    const long row_ = blockIdx.x * {RB}L + threadIdx.x / {T};",
                  f"    const bool live = row_ < {R}L;",
                  f"    const int row = (int)(live ? row_ : {R - 1}L);"]
        wide = R * N >= (1 << 31)
        for i in range(E):
            decls.append(f"    const int j_{i} = ({i // 4} * {T} + tt) * 4 + {i % 4};")
        if any(f.collapsed for f in self.forms):
            ty = "long" if wide else "int"
            for i in range(E):
                decls.append(f"    const {ty} cv_{i} = ({ty})row * {N} + j_{i};")
            decls.append(f"    const {'long' if wide else 'int'} cv = cv_0; (void)cv;")
        decls.append("    const int j = j_0; (void)j;")
        src = "\n".join(head + decls + body + ["}"])
        blocks = (R + RB - 1) // RB
        launch = [f"{name}<<<{blocks}, {rg.THREADS}, 0, st>>>(A, sdelta, seed); anvil_rt_count_launches(rt, 1);"]
        return src, launch


def tma_kernel(gen, src: list, launch: list, kname: str, fn: str, ca, cb, AK, BKC, S, accs, BN, status, scratch, grid, smem) -> bool:
    """When an operand of the resident pair template can come by TMA (`tma_operand`), adds a second __global__ function
    `<kname>_tma` that takes the tensor maps as grid constants, and launch code that encodes the maps once per arena
    (anvil_rt_tensor_map) and falls back to the plain kernel if that fails. `ca` / `cb`: the contractions whose A / B
    operand the kernel reads (the same one, except for fused launches). Returns False when neither operand qualifies."""
    a = tma_operand(ca, ca.a, ca.mvars) if AK == "true" else None
    b = tma_operand(cb, cb.b, cb.nvars) if BKC == "true" and cb is not None else None
    if a is None and b is None:
        return False
    mask = (1 if a else 0) | (2 if b else 0)
    src += [f"__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(anvil::tc::PP_THREADS, 1) {kname}_tma(char *__restrict__ A, "
            f"uint32_t sdelta, uint32_t seed_, const __grid_constant__ CUtensorMap tma, const __grid_constant__ CUtensorMap tmb) {{",
            f"    anvil::tc::gemm_tc_pair_persistent<{fn}, {AK}, {BKC}, {S}, {accs}, {BN}, {mask}>({fn}{{A}}, {scratch}, {status}, &tma, &tmb);", "}"]
    enc = []
    if a:
        root, const, rows, stride = a
        enc.append(f"anvil_rt_tensor_map(rt, &tma_, {gen.plan.offsets[root.id] + 4 * const}UL, {rows}L, {ca.K}L, {stride}L, 128) == 0")
    if b:
        root, const, rows, stride = b
        enc.append(f"anvil_rt_tensor_map(rt, &tmb_, {gen.plan.offsets[root.id] + 4 * const}UL, {rows}L, {cb.K}L, {stride}L, {BN // 2}) == 0")
    launch += ["{ alignas(64) static CUtensorMap tma_, tmb_; static char *tm_base_ = nullptr; static bool tm_ok_ = false, attr_ = false;",
               f"  if (!attr_) {{ cudaFuncSetAttribute({kname}, cudaFuncAttributeMaxDynamicSharedMemorySize, (int){smem}); "
               f"cudaFuncSetAttribute({kname}_tma, cudaFuncAttributeMaxDynamicSharedMemorySize, (int){smem}); attr_ = true; }}",
               f"  if (tm_base_ != A) {{ tm_ok_ = {' && '.join(enc)}; tm_base_ = A; }}        // the maps hold the arena's address",
               f"  if (tm_ok_) {kname}_tma<<<{grid}, anvil::tc::PP_THREADS, {smem}, st>>>(A, sdelta, seed, tma_, tmb_);",
               f"  else {kname}<<<{grid}, anvil::tc::PP_THREADS, {smem}, st>>>(A, sdelta, seed);",
               "  anvil_rt_count_launches(rt, 1); }"]
    return True


class AttnGroupGen:
    """A recognised attention run (attention.py) -> one launch of anvil::attn::attn_fused over a functor made of the two
    products' own operand functors, the mask expression, and pointers to the dense row tensors."""

    def __init__(self, gen: "ProgramGen", g: "at.AttnGroup"):
        self.gen, self.g = gen, g

    def generate(self, name: str):
        gen, g = self.gen, self.g
        k1, k2 = g.kernels[0], g.kernels[-1]
        src = []
        kg1 = KernelGen(gen, k1)
        _, _, fe1 = kg1.gemm_functors(g.c1)
        src += [kg1.comment("product 1 of a fused attention launch")] + kg1.tc_struct(g.c1, f"{name}_p1", fe1, True) + [""]
        kg2 = KernelGen(gen, k2)
        _, _, fe2 = kg2.gemm_functors(g.c2)
        src += [kg2.comment("product 2 of a fused attention launch")] + kg2.tc_struct(g.c2, f"{name}_p2", fe2, True) + [""]
        T, DH = at.T_TILE, at.DH_TILE

        def base(root):
            return f"((float *)(A + {gen.plan.offsets[root.id]}UL))"

        def b(flag):
            return "true" if flag else "false"
        fn = "F_" + name
        f = [f"// fused attention ({'forward' if g.mode == 0 else 'backward'}): " + " + ".join(k.name for k in g.kernels),
             f"struct {fn} {{", "    char *__restrict__ A;",
             f"    static constexpr int T = {T}, DH = {DH}, NBH = {g.nbh}, MODE = {g.mode};",
             f"    static constexpr bool CAUSAL = {b(g.causal)}, STORE_R = {b(g.live['r'])}, STORE_E = {b(g.mode == 0 and g.live['e'])}, "
             f"STORE_SUM = {b(g.mode == 0 and g.live['sum'])}, STORE_MAX = {b(g.mode == 0 and g.live['max'])};",
             f"    static constexpr float ALPHA1 = {flit(g.c1.alpha)}, ALPHA2 = {flit(g.c2.alpha)};",
             f"    __device__ __forceinline__ void a1(int i, int k, int bh, float (&v)[4]) const {{ {name}_p1{{A}}.a4(i, k, bh, v); }}",
             f"    __device__ __forceinline__ void b1(int k, int j, int bh, float (&v)[4]) const {{ {name}_p1{{A}}.b4(k, j, bh, v); }}",
             f"    __device__ __forceinline__ void b2(int k, int n, int bh, float (&v)[4]) const {{ {name}_p2{{A}}.b4(k, n, bh, v); }}",
             f"    __device__ __forceinline__ void a1_touch(int i, int k, int bh) const {{ {name}_p1{{A}}.a_touch(i, k, bh); }}",
             f"    __device__ __forceinline__ void b1_touch(int k, int j, int bh) const {{ {name}_p1{{A}}.b_touch(k, j, bh); }}",
             f"    __device__ __forceinline__ void b2_touch(int k, int n, int bh) const {{ {name}_p2{{A}}.b_touch(k, n, bh); }}",
             f"    __device__ __forceinline__ void epi(int i, int n, int bh, float acc) const {{ {name}_p2{{A}}.epi(i, n, bh, acc); }}",
             f"    __device__ __forceinline__ float *r_row(int i, int bh) const {{ return {base(g.bufs['r'])} + ((long)bh * {T} + i) * {T}; }}",
             f"    __device__ __forceinline__ float *e_row(int i, int bh) const {{ return {base(g.bufs['e'])} + ((long)bh * {T} + i) * {T}; }}",
             f"    __device__ __forceinline__ float *sum_at(int i, int bh) const {{ return {base(g.bufs['sum'])} + (long)bh * {T} + i; }}"]
        if g.mode == 0:
            f.append(f"    __device__ __forceinline__ float *max_at(int i, int bh) const {{ return {base(g.bufs['max'])} + (long)bh * {T} + i; }}")
            f.append(f"    __device__ __forceinline__ const float *p_row(int i, int bh) const {{ return r_row(i, bh); }}")
            # the score from product 1's scaled accumulator: the elementwise kernel's expression with its load replaced
            pk = g.post_kernel
            kg = KernelGen(gen, pk)
            names = dict(kg.names)
            names[pk.domain[-2]], names[pk.domain[-1]] = "i", "j"
            sc = Scope(kg, names, 1, None, "        ")
            sc.preloaded = {(g.post_load.buf.root.id, g.post_load.off.key()): "acc"}
            dec = kg.decode("(uint32_t)bh", pk.domain[:-2], names, "        ")
            val = sc.ex([st for st in pk.stmts if isinstance(st, kir.Store)][0].value, 0)
            f += ["    __device__ __forceinline__ float post(float acc, int i, int j, int bh) const {"] \
                + ["    " + ln for ln in kg.pointer_decls()] + dec + sc.lines \
                + [f"        return {val};", "    }"]
        else:
            f.append(f"    __device__ __forceinline__ float *max_at(int i, int bh) const {{ return nullptr; }}")
            f.append(f"    __device__ __forceinline__ const float *p_row(int i, int bh) const {{ return {base(g.bufs['p'])} + ((long)bh * {T} + i) * {T}; }}")
            f.append("    __device__ __forceinline__ float post(float acc, int i, int j, int bh) const { return acc; }")
        f.append("};")
        status = "(uint32_t *)(A + ANVIL_RT_STATUS_OFF)"
        smem = f"anvil::attn::smem_bytes_att({T}, {DH})"
        f += [f"__global__ void __launch_bounds__(anvil::attn::THREADS_ATT, 1) {name}(char *__restrict__ A, uint32_t sdelta, uint32_t seed_) {{",
              f"    anvil::attn::attn_fused<{fn}>({fn}{{A}}, {status});", "}"]
        work = g.nbh * (T // 128)
        launch = [f"{{ static bool attr_ = false; if (!attr_) {{ cudaFuncSetAttribute({name}, "
                  f"cudaFuncAttributeMaxDynamicSharedMemorySize, (int){smem}); attr_ = true; }} }}",
                  f"{name}<<<{min(work, 148)}, anvil::attn::THREADS_ATT, {smem}, st>>>(A, sdelta, seed); anvil_rt_count_launches(rt, 1);"]
        note = f"attention {'fwd' if g.mode == 0 else 'bwd'} {g.nbh}x{T}x{T}x{DH}" + (" causal" if g.causal else "")
        return "\n".join(src + f), launch, note


class HGroupGen:
    """A horizontal group of contractions (see hfuse.py) -> one launch of the resident pair template over a functor
    that dispatches to the members' functors by tile column ("ncat") or by reduction block ("kcat")."""

    def __init__(self, gen: "ProgramGen", kernels, kind: str):
        self.gen, self.kernels, self.kind = gen, kernels, kind

    def generate(self, name: str):
        gen, ks, kind = self.gen, self.kernels, self.kind
        cs = [ct.match(k) for k in ks]
        src, names, nlds = [], [], []
        for i, (k, c) in enumerate(zip(ks, cs)):
            kg = KernelGen(gen, k)
            _, _, fe = kg.gemm_functors(c)
            fn = f"{name}_{i}"
            src += [kg.comment(f"member {i} of a fused launch")] + kg.tc_struct(c, fn, fe, True) + [""]
            names.append(fn)
            nlds.append(kg.nld)
        c0 = cs[0]
        M = c0.M
        N = sum(c.N for c in cs) if kind == "ncat" else c0.N
        K = sum(c.K for c in cs) if kind == "kcat" else c0.K
        nld = max(nlds) if kind == "ncat" else nlds[0]
        L = max(nld, 1)

        def dispatch(sig, call, sizes, var):
            """`if (var < s0) member0.call else if ...` with `var` rebased for each member."""
            out = [f"    __device__ __forceinline__ {sig} const {{"]
            base = 0
            for i, (fn, size) in enumerate(zip(names, sizes)):
                head = "if" if i == 0 else "else if"
                cond = f"{head} ({var} < {base + size})" if i < len(names) - 1 else ("else" if i else "")
                shifted = f"{var} - {base}" if base else var
                out.append(f"        {cond} {{ {fn}{{A}}.{call.format(v=shifted, L=max(nlds[i], 1))}; }}")
                base += size
            return out + ["    }"]
        kernel_name, name = name, "F_" + name               # the functor type; the __global__ function keeps the plain name
        f = [f"// {kind}: " + " | ".join(f"{k.name} <{k.label}>" for k in ks), f"struct {name} {{", "    char *__restrict__ A;",
             f"    static constexpr int M = {M}, N = {N}, K = {K}, NB = 1, NLD = {nld};",
             f"    static constexpr float ALPHA = {flit(c0.alpha)};"]
        first = names[0]
        if kind == "ncat":
            sizes = [c.N for c in cs]
            f += [f"    __device__ __forceinline__ void a4(int m, int k, int bt, float (&v)[4]) const {{ {first}{{A}}.a4(m, k, bt, v); }}",
                  f"    __device__ __forceinline__ void a_touch(int m, int k, int bt) const {{ {first}{{A}}.a_touch(m, k, bt); }}"]
            f += dispatch("void b4(int k, int n, int bt, float (&v)[4])", "b4(k, {v}, bt, v)", sizes, "n")
            f += dispatch("void b_touch(int k, int n, int bt)", "b_touch(k, {v}, bt)", sizes, "n")
            f += dispatch("void epi(int m, int n, int bt, float acc)", "epi(m, {v}, bt, acc)", sizes, "n")
            f += dispatch("void epi_touch(int m, int n, int bt)", "epi_touch(m, {v}, bt)", sizes, "n")
            f += dispatch("void epi_near(int m, int n, int bt)", "epi_near(m, {v}, bt)", sizes, "n")
            f += dispatch(f"void epi_loads(int m, int n, int bt, float (&ld)[{L}])",
                          "epi_loads(m, {v}, bt, reinterpret_cast<float (&)[{L}]>(ld))", sizes, "n")
            f += dispatch(f"void epi2(int m, int n, int bt, float acc, const float (&ld)[{L}])",
                          "epi2(m, {v}, bt, acc, reinterpret_cast<const float (&)[{L}]>(ld))", sizes, "n")
        else:
            sizes = [c.K for c in cs]
            f += dispatch("void a4(int m, int k, int bt, float (&v)[4])", "a4(m, {v}, bt, v)", sizes, "k")
            f += dispatch("void b4(int k, int n, int bt, float (&v)[4])", "b4({v}, n, bt, v)", sizes, "k")
            f += dispatch("void a_touch(int m, int k, int bt)", "a_touch(m, {v}, bt)", sizes, "k")
            f += dispatch("void b_touch(int k, int n, int bt)", "b_touch({v}, n, bt)", sizes, "k")
            f += [f"    __device__ __forceinline__ void epi(int m, int n, int bt, float acc) const {{ {first}{{A}}.epi(m, n, bt, acc); }}",
                  f"    __device__ __forceinline__ void epi_touch(int m, int n, int bt) const {{ {first}{{A}}.epi_touch(m, n, bt); }}",
                  f"    __device__ __forceinline__ void epi_near(int m, int n, int bt) const {{ {first}{{A}}.epi_near(m, n, bt); }}",
                  f"    __device__ __forceinline__ void epi_loads(int m, int n, int bt, float (&ld)[{L}]) const {{ {first}{{A}}.epi_loads(m, n, bt, ld); }}",
                  f"    __device__ __forceinline__ void epi2(int m, int n, int bt, float acc, const float (&ld)[{L}]) const {{ {first}{{A}}.epi2(m, n, bt, acc, ld); }}"]
        # The same methods as templates on the member index: the resident template looks the member of a whole k block
        # (kcat) or tile (ncat) up once and instantiates its loops per member (no branch inside an operand fetch).
        if len(names) <= 4:
            sizes = [c.N for c in cs] if kind == "ncat" else [c.K for c in cs]
            bases = [sum(sizes[:i]) for i in range(len(sizes))]

            def chain(var):
                out = "0"
                for i in range(1, len(sizes)):
                    out = f"({var} >= {bases[i]} ? {i} : {out})"
                return out

            def per_member(sig, call, own, shift):
                """own: every member has the method (else the first member's is used); shift: which argument is rebased."""
                out = [f"    template <int S> __device__ __forceinline__ {sig} const {{"]
                for i, fn in enumerate(names):
                    target = fn if own else first
                    args = call.format(v=(f"{shift} - {bases[i]}" if (own and bases[i]) else shift), L=max(nlds[i] if own else nlds[0], 1))
                    out.append(f"        {'if' if i == 0 else 'else if'} constexpr (S == {i}) {{ {target}{{A}}.{args}; }}")
                return out + ["    }"]
            f.append(f"    static constexpr int SEGS = {len(names)};")
            if kind == "ncat":
                f += [f"    __device__ __forceinline__ int op_seg(int k0, int n0) const {{ return {chain('n0')}; }}",
                      f"    __device__ __forceinline__ int epi_seg(int n0) const {{ return {chain('n0')}; }}"]
                f += per_member("void a4s(int m, int k, int bt, float (&v)[4])", "a4(m, k, bt, v)", False, "k")
                f += per_member("void a_touchs(int m, int k, int bt)", "a_touch(m, k, bt)", False, "k")
                f += per_member("void b4s(int k, int n, int bt, float (&v)[4])", "b4(k, {v}, bt, v)", True, "n")
                f += per_member("void b_touchs(int k, int n, int bt)", "b_touch(k, {v}, bt)", True, "n")
                f += per_member("void epi_touchs(int m, int n, int bt)", "epi_touch(m, {v}, bt)", True, "n")
                f += per_member("void epi_nears(int m, int n, int bt)", "epi_near(m, {v}, bt)", True, "n")
                f += per_member(f"void epi_loadss(int m, int n, int bt, float (&ld)[{L}])",
                                "epi_loads(m, {v}, bt, reinterpret_cast<float (&)[{L}]>(ld))", True, "n")
                f += per_member(f"void epi2s(int m, int n, int bt, float acc, const float (&ld)[{L}])",
                                "epi2(m, {v}, bt, acc, reinterpret_cast<const float (&)[{L}]>(ld))", True, "n")
            else:
                f += [f"    __device__ __forceinline__ int op_seg(int k0, int n0) const {{ return {chain('k0')}; }}",
                      "    __device__ __forceinline__ int epi_seg(int n0) const { return 0; }"]
                f += per_member("void a4s(int m, int k, int bt, float (&v)[4])", "a4(m, {v}, bt, v)", True, "k")
                f += per_member("void a_touchs(int m, int k, int bt)", "a_touch(m, {v}, bt)", True, "k")
                f += per_member("void b4s(int k, int n, int bt, float (&v)[4])", "b4({v}, n, bt, v)", True, "k")
                f += per_member("void b_touchs(int k, int n, int bt)", "b_touch({v}, n, bt)", True, "k")
                f += per_member("void epi_touchs(int m, int n, int bt)", "epi_touch(m, n, bt)", False, "n")
                f += per_member("void epi_nears(int m, int n, int bt)", "epi_near(m, n, bt)", False, "n")
                f += per_member(f"void epi_loadss(int m, int n, int bt, float (&ld)[{L}])", "epi_loads(m, n, bt, ld)", False, "n")
                f += per_member(f"void epi2s(int m, int n, int bt, float acc, const float (&ld)[{L}])", "epi2(m, n, bt, acc, ld)", False, "n")
        f.append("};")
        seg_bn = 256 if kind != "ncat" or all(c.N % 256 == 0 for c in cs) else 128      # a tile never straddles two members
        BN, S, accs, work = pp_launch_params(M, N, K, 1, seg_bn)
        AK = "true" if c0.a_kcontig else "false"
        BKC = "true" if ct._contig(c0.b, c0.kvars[-1]) else "false"
        status = "(uint32_t *)(A + ANVIL_RT_STATUS_OFF)"
        kname = kernel_name + ("_part" if S > 1 else "")
        smem = f"anvil::tc::pp_smem_bytes({BN})"
        scratch = "nullptr"
        soff = 0
        if S > 1:
            if all(k.id in gen.side_ids for k in ks):        # runs on the second stream, beside first-stream products
                gen.side_scratch_bytes = max(gen.side_scratch_bytes, 4 * M * N * S)
                soff = gen.plan.side_scratch_off
            else:
                gen.need_scratch(4 * M * N * S)
                soff = gen.plan.scratch_off
            scratch = f"(float *)(A + {soff}UL)"
        f += [f"__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(anvil::tc::PP_THREADS, 1) {kname}(char *__restrict__ A, uint32_t sdelta, uint32_t seed_) {{",
              f"    anvil::tc::gemm_tc_pair_persistent<{name}, {AK}, {BKC}, {S}, {accs}, {BN}>({name}{{A}}, {scratch}, {status});", "}"]
        launch = []
        if not (kind == "ncat" and use_tma() and tma_kernel(gen, f, launch, kname, name, c0, None, AK, BKC, S, accs, BN, status, scratch,
                                                          f"dim3({2 * min(work, 74)}, 1)", smem)):
            launch = [f"{{ static bool attr_ = false; if (!attr_) {{ cudaFuncSetAttribute({kname}, "
                      f"cudaFuncAttributeMaxDynamicSharedMemorySize, (int){smem}); attr_ = true; }} }}",
                      f"{kname}<<<dim3({2 * min(work, 74)}, 1), anvil::tc::PP_THREADS, {smem}, st>>>(A, sdelta, seed); anvil_rt_count_launches(rt, 1);"]
        if S > 1:
            f += [f"__global__ void __launch_bounds__(256) {kernel_name}_fin(char *__restrict__ A, uint32_t sdelta, uint32_t seed_) {{",
                  f"    anvil::gemm_split_finish<{name}, {S}>({name}{{A}}, (const float *)(A + {soff}UL));", "}"]
            fb_ = max(1, min((M * N + 255) // 256, MAX_BLOCKS))
            launch.append(f"{kernel_name}_fin<<<{fb_}, 256, 0, st>>>(A, sdelta, seed); anvil_rt_count_launches(rt, 1);")
        note = f"gemm tc 1x{M}x{N}x{K} S{S} pp {kind}{len(ks)}"
        return "\n".join(src + f), launch, note


def index_t(n: int) -> str:
    return "uint32_t" if n < (1 << 32) else "unsigned long long"


class ProgramGen:
    """Host side: the arena plan, one launcher per kernel, the program's control flow."""

    def __init__(self, prog: kir.Program, seed: int = 0):
        self.prog = prog
        self.seed = seed & 0xFFFFFFFF
        self.faults: list[str] = []
        self.scratch_bytes = 4
        self.side_scratch_bytes = 4
        self.deferred = an.deferred_kernels(prog) if use_side_stream() else set()
        self.side_ids: set = set()                   # deferred kernels that are launch units of their own: they run on the second stream
        self.dealt = [0, 0]                          # FLOPs of deferred contractions given to the first / second stream so far
        self.member_slot: dict = {}                  # kernel id -> (scratch offset, first ticket) inside its side-by-side launch
        self.zgroup_of: dict = {}                    # kernel id -> ids of the side-by-side launch it belongs to
        self.readers: dict = {}
        for k in prog.kernels():
            for r in k.reads():
                self.readers.setdefault(r.id, set()).add(k.id)
        self.causal_e: set = set()              # exp tensors written by causal fused attention (zero above the diagonal)
        self.plan = self.make_plan(0)
        self.kernel_index: dict[int, int] = {}
        self.kernels: list[kir.Kernel] = []
        self.kernel_src: list[str] = []
        self.kernel_gens: dict = {}
        self.launchers: list[str] = []
        self.kernel_notes: list[str] = []
        self.tables: list[str] = []
        self.n = 0
        self.graph_keys = 0
        self.hot = an.hot_loop(prog)
        self.hot_body: list[str] | None = None
        self.hot_counter = None
        self.hot_body_fed: list[str] | None = None
        self.feed_bufs: list = []
        self.feed_kernels: list = []
        self.groups: dict = {}                  # tuple of kernel ids -> launch-table index of the fused kernel
        self.group_src: list[str] = []
        self.group_launchers: list[str] = []
        self.group_notes: list[str] = []
        self.dead_roots: set = set()            # temporaries that live only in registers of a fused group (never stored)
        self.hot_units: list = []               # (launch-table index, note, [kernels]) of the training loop, in order
        self.record_units = False
        self.host_read = self._host_reads()

    def make_plan(self, scratch_bytes: int, side_scratch_bytes: int = 4):
        """The arena plan: lifetime sharing unless ANVIL_B200_ARENA=unshared. Tensors the host reads (printed values,
        loop conditions, checkpoints) or feeds (the step's inputs) keep their own memory, so they can be read between
        steps; row kernels that will run as one fused kernel count as one statement."""
        hot = an.hot_loop(self.prog)
        host = self._host_reads()
        keep = set(host)
        if hot is not None:
            keep |= {b.root.id for b in an.input_producers(self.prog, hot)[1]}
        def runs(ks):
            spans = at.find_attention(ks, self.readers, host, self.causal_e) if use_attention() else []
            return fused_runs(ks, spans)
        return an.plan_arena(self.prog, scratch_bytes, share=os_environ("ANVIL_B200_ARENA", "shared") != "unshared",
                             fused_runs=runs, keep=keep, deferred=self.deferred, side_scratch_bytes=side_scratch_bytes)

    def _host_reads(self) -> set:
        """Root ids of tensors that something other than a kernel reads."""
        out = set()

        def note(b):
            if isinstance(b, kir.Buffer):
                out.add(b.root.id)
        for blk in kir.walk_blocks(self.prog.main):
            for st in blk.stmts:
                if isinstance(st, kir.For):
                    note(st.counter); note(st.start); note(st.stop)
                elif isinstance(st, kir.While):
                    note(st.cond)
                elif isinstance(st, kir.If):
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
        for b in self.prog.buffers:
            if b.root.kind not in ("temp", "grad"):
                out.add(b.root.id)
        return out

    def add_group(self, kernels: list) -> int:
        """Launch-table index of the fused kernel for this run of row kernels."""
        key = tuple(k.id for k in kernels)
        hit = self.groups.get(key)
        if hit is not None:
            return hit
        forms, N = [], None
        for k in kernels:
            f = rg.row_form(k, N)
            if f is None and N is None:
                N = next(rg.row_form(x).N for x in kernels if rg.row_form(x) is not None)
                f = rg.row_form(k, N)
            N = f.N
            forms.append(f)
        ids = set(key)
        dead = set()
        written_so_far: dict = {}
        order_ok: dict = {}
        for f in forms:                                  # a tensor is private if every read follows a write of the same element
            k = f.kernel
            for b, off in k.loads():
                r = b.root.id
                if r not in written_so_far or f.canon(off) not in written_so_far[r]:
                    order_ok[r] = False
            for st in k.stores:
                r = st.buf.root.id
                if st.accumulate and (r not in written_so_far):
                    order_ok[r] = False
                written_so_far.setdefault(r, set()).add(f.canon(st.offset))
        for r in written_so_far:
            if r not in self.host_read and self.readers.get(r, set()) <= ids and order_ok.get(r, True):
                dead.add(r)
        self.dead_roots |= dead
        gg = RowGroupGen(self, forms, dead)
        name = f"g{len(self.groups)}_{kernels[0].id}"
        src, launch = gg.generate(name)
        idx = len(self.groups)
        self.groups[key] = idx
        self.group_src.append(src)
        self.group_notes.append(f"rowgroup x{len(kernels)} {forms[0].R}x{forms[0].N}")
        body = ["    char *A = (char *)anvil_rt_ptr(rt, 0);", "    cudaStream_t st = (cudaStream_t)anvil_rt_stream(rt);",
                "    uint32_t seed = anvil_rt_get_seed(rt);", "    uint32_t sdelta = 0;",
                f"    RT(anvil_rt_prof_begin(rt, PROF_GROUP0 + {idx}));"] + ["    " + ln for ln in launch] \
            + [f"    RT(anvil_rt_prof_end(rt, PROF_GROUP0 + {idx}));"] + self.check_lines(kernels) + ["    return 0;"]
        self.group_launchers.append(f"static int launch_group_{idx}(anvil_rt *rt) {{   // {' + '.join(k.name for k in kernels)}\n"
                                    + "\n".join(body) + "\n}")
        return idx

    ZGROUP_MAX = 8

    def plan_zgroups(self, side_kernels: list, neighbours: bool = False) -> None:
        """Side-stream kernels of one launch run become side-by-side launches of up to ZGROUP_MAX members: they are
        independent of everything after them (that is what put them on the second stream), so also of one another, and
        each is too short to fill the GPU or to hide its own latency chain (C5: a 16384 x 512 column sum with its Adam
        update is 16 us for 33 MB). A member must be generated as a device function, so only kernels without source yet
        are taken, and only the strategies whose bodies are written against bx_ / by_ / gdx_.
        `neighbours`: the list is a launch run of the first stream (None = something that cannot join); consecutive
        kernels join when none of them reads or writes what another writes (the bias-gradient sums of a data-parallel
        step, which go to the all-reduce bucket and so are not deferred) and none writes a tensor that shares arena
        bytes (lifetime sharing relies on the program's order between launches)."""
        cur: list = []

        def flush():
            if len(cur) >= 2:
                ids = tuple(k.id for k, _, _ in cur)
                soff = tick = 0
                for k, nbytes, gx in cur:
                    self.member_slot[k.id] = (soff, tick)
                    self.zgroup_of[k.id] = ids
                    soff += (nbytes + 255) // 256 * 256
                    tick += gx
            cur.clear()
        for k in side_kernels:
            if k is None or k.id in self.kernel_index or k.id in self.zgroup_of or (neighbours and (k.id in self.side_ids or k.uses_rand())):
                flush()
                continue
            if neighbours:
                r, w = {b.id for b in k.reads()}, {b.id for b in k.writes()}
                if w & self.plan.shared:                 # its output may live in bytes another member still reads: the
                    flush()                              # arena plan assumes the program's order between launches
                    continue
                for m, _, _ in cur:
                    mr, mw = {b.id for b in m.reads()}, {b.id for b in m.writes()}
                    if w & (mr | mw) or r & mw:
                        flush()
                        break
            choice = KernelGen(self, k).choose()
            if choice[0] == "coop4":
                OX, RY, S = choice[1:]
                gx = (k.out_numel() // 4 + OX - 1) // OX
                need = (4 * k.out_numel() * S if S > 1 else 0, gx if S > 1 else 0)
                ok = OX * RY == THREADS
            elif choice[0] in ("eltwise", "thread"):
                need, ok = (0, 0), True
            else:
                ok = False
            if not ok:
                flush()
                continue
            if len(cur) == self.ZGROUP_MAX or sum(g for _, _, g in cur) + need[1] > 256:
                flush()
            cur.append((k, need[0], need[1]))
        flush()

    def add_zgroup(self, kernels: list) -> int:
        """Launch-table index of the side-by-side launch of these (mutually independent) kernels."""
        key = ("z",) + tuple(k.id for k in kernels)
        hit = self.groups.get(key)
        if hit is not None:
            return hit
        idx = len(self.groups)
        name = f"z{idx}_{kernels[0].id}"
        gens = []
        for k in kernels:
            kg = self.kernel_gens[k.id]
            assert kg.member and kg.grid is not None and kg.nthreads == THREADS
            gens.append(kg)
        smem = max(16, max(kg.zsm_bytes for kg in gens))
        lines = [f"// side by side: {' | '.join(k.name for k in kernels)}",
                 f"__global__ void __launch_bounds__({THREADS}) {name}(char *__restrict__ A, uint32_t sdelta, uint32_t seed_) {{",
                 f"    __shared__ __align__(16) char zsm_[{smem}];", "    const unsigned b_ = blockIdx.x;"]
        off = 0
        for k, kg in zip(kernels, gens):
            gx, gy = kg.grid
            lines.append(f"    if (b_ < {off + gx * gy}u) {{ const unsigned l_ = b_ - {off}u; "
                         f"k{k.id}_body(A, 0u, seed_, l_ % {gx}u, l_ / {gx}u, {gx}u, zsm_); return; }}")
            off += gx * gy
        lines.append("}")
        self.groups[key] = idx
        self.group_src.append("\n".join(lines))
        self.group_notes.append(f"zgroup x{len(kernels)} " + "+".join(sorted({" ".join(kg.notes.split()[:2]) for kg in gens})))
        body = ["    char *A = (char *)anvil_rt_ptr(rt, 0);", "    cudaStream_t st = (cudaStream_t)anvil_rt_stream(rt);",
                "    uint32_t seed = anvil_rt_get_seed(rt);",
                f"    RT(anvil_rt_prof_begin(rt, PROF_GROUP0 + {idx}));",
                f"    {name}<<<{off}, {THREADS}, 0, st>>>(A, 0u, seed); anvil_rt_count_launches(rt, 1);",
                f"    RT(anvil_rt_prof_end(rt, PROF_GROUP0 + {idx}));"] + self.check_lines(kernels) + ["    return 0;"]
        self.group_launchers.append(f"static int launch_group_{idx}(anvil_rt *rt) {{   // {' | '.join(k.name for k in kernels)}\n"
                                    + "\n".join(body) + "\n}")
        return idx

    MAX_FAULT_CODES = 254

    def add_attention(self, g) -> int:
        """Launch-table index of the fused launch for a recognised attention run. Tensors that the fused kernel keeps in
        tensor memory (scores, masked scores, row maxima / the three softmax-gradient temporaries) are never stored."""
        key = ("a",) + tuple(k.id for k in g.kernels)
        hit = self.groups.get(key)
        if hit is not None:
            return hit
        idx = len(self.groups)
        src, launch, note = AttnGroupGen(self, g).generate(f"a{idx}_{g.kernels[0].id}")
        self.dead_roots |= {b.id for r, b in g.bufs.items() if not g.live[r]}
        self.groups[key] = idx
        self.group_src.append(src)
        self.group_notes.append(note)
        body = ["    char *A = (char *)anvil_rt_ptr(rt, 0);", "    cudaStream_t st = (cudaStream_t)anvil_rt_stream(rt);",
                "    uint32_t seed = anvil_rt_get_seed(rt);", "    uint32_t sdelta = 0;",
                f"    RT(anvil_rt_prof_begin(rt, PROF_GROUP0 + {idx}));"] + ["    " + ln for ln in launch] \
            + [f"    RT(anvil_rt_prof_end(rt, PROF_GROUP0 + {idx}));", "    return 0;"]
        self.group_launchers.append(f"static int launch_group_{idx}(anvil_rt *rt) {{   // {' + '.join(k.name for k in g.kernels)}\n"
                                    + "\n".join(body) + "\n}")
        return idx

    def add_hgroup(self, kernels: list, kind: str) -> int:
        """Launch-table index of the fused launch for a horizontal group of contractions."""
        key = ("h",) + tuple(k.id for k in kernels)
        hit = self.groups.get(key)
        if hit is not None:
            return hit
        idx = len(self.groups)
        src, launch, note = HGroupGen(self, kernels, kind).generate(f"h{idx}_{kernels[0].id}")
        self.groups[key] = idx
        self.group_src.append(src)
        self.group_notes.append(note)
        body = ["    char *A = (char *)anvil_rt_ptr(rt, 0);", "    cudaStream_t st = (cudaStream_t)anvil_rt_stream(rt);",
                "    uint32_t seed = anvil_rt_get_seed(rt);", "    uint32_t sdelta = 0;",
                f"    RT(anvil_rt_prof_begin(rt, PROF_GROUP0 + {idx}));"] + ["    " + ln for ln in launch] \
            + [f"    RT(anvil_rt_prof_end(rt, PROF_GROUP0 + {idx}));"] + self.check_lines(kernels) + ["    return 0;"]
        self.group_launchers.append(f"static int launch_group_{idx}(anvil_rt *rt) {{   // {' | '.join(k.name for k in kernels)}\n"
                                    + "\n".join(body) + "\n}")
        return idx

    def fault(self, message: str) -> int:
        """The code (1-based index into the program's message table) a kernel records for this bounds fault. The
        fault word holds one byte of code: once the table is full, further messages share a generic entry."""
        if message not in self.faults and len(self.faults) >= self.MAX_FAULT_CODES:
            message = "index out of bounds"
        if message not in self.faults:
            self.faults.append(message)
        return 1 + self.faults.index(message)

    def need_scratch(self, nbytes: int):
        self.scratch_bytes = max(self.scratch_bytes, nbytes)

    def label(self, hint: str) -> str:
        self.n += 1
        return f"{hint}{self.n}"

    def off(self, b: kir.Buffer) -> str:
        return f"{self.plan.off(b)}UL"

    # ---- kernels
    def add_kernel(self, k: kir.Kernel) -> int:
        hit = self.kernel_index.get(k.id)
        if hit is not None:
            return hit
        kg = KernelGen(self, k)
        src, launch = kg.generate()
        self.kernel_gens[k.id] = kg
        idx = len(self.kernels)
        self.kernel_index[k.id] = idx
        self.kernels.append(k)
        self.kernel_src.append(src)
        self.kernel_notes.append(kg.notes)
        body = ["    char *A = (char *)anvil_rt_ptr(rt, 0);", "    cudaStream_t st = (cudaStream_t)anvil_rt_stream(rt);",
                "    uint32_t seed = anvil_rt_get_seed(rt);"]
        body.append("    uint32_t sdelta = " + ("anvil_rt_next_stream_delta(rt);" if kg.uses_rand else "0;"))
        body.append(f"    RT(anvil_rt_prof_begin(rt, {idx}));")
        body += ["    " + ln for ln in launch]
        body.append(f"    RT(anvil_rt_prof_end(rt, {idx}));")
        body += self.check_lines([k])
        body.append("    return 0;")
        self.launchers.append(f"static int launch_{idx}(anvil_rt *rt) {{   // {k.name} {k.label}\n" + "\n".join(body) + "\n}")
        return idx

    def check_lines(self, kernels) -> list[str]:
        """--check: after a launch unit, every f32 tensor it wrote is scanned for nan / infinity (the reference
        does it kernel by kernel, anvil/interp.py:408-423); the message names the kernel that wrote the tensor."""
        out, seen = [], set()
        for k in kernels:
            desc = f"  made by `{k.label or 'a computation'}`:\n  computing ({k.name}):  {kir.fmt_kernel(k)}"
            for st in k.stores:
                r = st.buf.root
                if r.dtype != F32 or r.id in seen:
                    continue
                seen.add(r.id)
                shp = self.table("long", [str(d) for d in r.shape]) if r.shape else "nullptr"
                out.append(f"        RT(anvil_rt_check_tensor(rt, {self.off(r)}, {r.numel}L, {c_string(r.name)}, {shp}, "
                           f"{len(r.shape)}, {c_string(desc)}));")
        if not out:
            return []
        return ["    if (anvil_rt_checking(rt)) {"] + out + ["    }"]

    # ---- host control flow (anvil/backend/cuda.py:429-473)
    def block(self, b: kir.Block, ind: str, in_loop: bool, tail: list[str] | None = None, skip=()) -> list[str]:
        """`tail`: host calls to issue right after the block's last statement (the loop counter
        increment); they join the last launch run when the block ends with one."""
        out = []
        stmts = list(b.stmts)
        i = 0
        tail_done = False
        while i < len(stmts):
            st = stmts[i]
            if isinstance(st, kir.KernelStmt):
                j = i
                run = []
                calls = []
                run_kernels = []
                while j < len(stmts) and isinstance(stmts[j], kir.KernelStmt):
                    kj = stmts[j].kernel
                    if kj.id not in skip:
                        run_kernels.append(kj)
                    j += 1
                spans = rg.find_groups(run_kernels) if use_row_groups() else []
                starts = {a: b for a, b in spans}
                hstarts = {a: (b, kind) for a, b, kind in (hfuse.find_hgroups(run_kernels, tc_eligible_pp) if use_hgroups() else [])}
                astarts = {a: (b, g) for a, b, g in (at.find_attention(run_kernels, self.readers, self.host_read, self.causal_e)
                                                       if use_attention() else [])}
                if in_loop:
                    # Deferred kernels that stay launch units of their own go to the second stream (decided once, before
                    # the kernel's source exists). Deferred contractions (the weight gradients with their updates, at the
                    # end of a training step) are dealt to the two streams by accumulated work: two chains of resident
                    # kernels fill each other's partly empty last round of tiles.
                    def deal(ks_):
                        if not use_side_gemms() or any(x.id not in self.deferred or x.id in self.kernel_index for x in ks_):
                            return
                        fl = sum(an.kernel_flops(x) for x in ks_)
                        if os_environ("ANVIL_B200_SIDE_GEMMS", "1") == "all" or self.dealt[1] + fl <= self.dealt[0]:
                            self.dealt[1] += fl
                            self.side_ids.update(x.id for x in ks_)
                        else:
                            self.dealt[0] += fl
                    q = 0
                    while q < len(run_kernels):
                        if q in astarts:
                            q = astarts[q][0]
                        elif q in hstarts:
                            deal(run_kernels[q:hstarts[q][0]])
                            q = hstarts[q][0]
                        elif q in starts:
                            q = starts[q]
                        else:
                            kq = run_kernels[q]
                            if ct.match(kq) is not None:
                                deal([kq])
                            elif kq.id in self.deferred and kq.id not in self.kernel_index:
                                self.side_ids.add(kq.id)
                            q += 1
                if in_loop and use_zgroups():
                    self.plan_zgroups([kq for kq in run_kernels if kq.id in self.side_ids and ct.match(kq) is None])
                    # first-stream kernels: only neighbours that do not touch one another's results
                    q, singles = 0, []
                    while q < len(run_kernels):
                        if q in astarts:
                            q = astarts[q][0]
                        elif q in hstarts:
                            q = hstarts[q][0]
                        elif q in starts:
                            q = starts[q]
                        else:
                            singles.append(run_kernels[q])
                            q += 1
                            continue
                        singles.append(None)             # a fused launch stands between
                    self.plan_zgroups(singles, neighbours=True)
                for x in stmts[i:j]:
                    kj = x.kernel
                    self.add_kernel(kj)
                    if kj.id in skip and kj.uses_rand():      # fed from the host; its random stream is still consumed
                        calls.append("anvil_rt_set_stream(rt, anvil_rt_get_stream(rt) + 1u);")
                forked = False
                meta: dict = {}                      # index into calls -> (roots read, roots written, may move up: second stream, or tiny)

                def launch(text, ks_, side=False):
                    r_ = set().union(*[{b.id for b in x.reads()} for x in ks_])
                    w_ = set().union(*[{b.id for b in x.writes()} for x in ks_])
                    meta[len(calls)] = (r_, w_, side or all(x.out_numel() <= 1024 for x in ks_))
                    calls.append(text)
                q = 0
                while q < len(run_kernels):
                    if q in astarts:
                        end, g = astarts[q]
                        gi = self.add_attention(g)
                        launch(f"RT(launch_group_{gi}(rt));", g.kernels)
                        if self.record_units:
                            self.hot_units.append((("g", gi), self.group_notes[gi], g.kernels))
                        q = end
                    elif q in hstarts:
                        end, kind = hstarts[q]
                        ks = run_kernels[q:end]
                        gi = self.add_hgroup(ks, kind)
                        if all(x.id in self.side_ids for x in ks):
                            launch(f"RT(anvil_rt_fork(rt)); RT(launch_group_{gi}(rt)); anvil_rt_back(rt);", ks, True)
                            forked = True
                        else:
                            launch(f"RT(launch_group_{gi}(rt));", ks)
                        if self.record_units:
                            self.hot_units.append((("g", gi), self.group_notes[gi], ks))
                        q = end
                    elif q in starts:
                        ks = run_kernels[q:starts[q]]
                        gi = self.add_group(ks)
                        launch(f"RT(launch_group_{gi}(rt));", ks)
                        if self.record_units:
                            self.hot_units.append((("g", gi), self.group_notes[gi], ks))
                        q = starts[q]
                    else:
                        idx = self.kernel_index[run_kernels[q].id]
                        run.append(idx)
                        zg = self.zgroup_of.get(run_kernels[q].id)
                        by_id = {x.id: x for x in run_kernels}
                        if zg is not None and not all(i_ in by_id for i_ in zg):
                            zg = None                    # a member is fed from the host in this variant of the loop body: no shared launch
                        if zg is not None:               # runs when the last member of its side-by-side launch is reached
                            if run_kernels[q].id == zg[-1]:
                                ks = [by_id[i_] for i_ in zg]
                                gi = self.add_zgroup(ks)
                                if zg[0] in self.side_ids:
                                    launch(f"RT(anvil_rt_fork(rt)); RT(launch_group_{gi}(rt)); anvil_rt_back(rt);", ks, True)
                                    forked = True
                                else:
                                    launch(f"RT(launch_group_{gi}(rt));", ks)
                                if self.record_units:
                                    self.hot_units.append((("g", gi), self.group_notes[gi], ks))
                        elif run_kernels[q].id in self.side_ids:
                            launch(f"RT(anvil_rt_fork(rt)); RT(launch_{idx}(rt)); anvil_rt_back(rt);", [run_kernels[q]], True)
                            forked = True
                            if self.record_units:
                                self.hot_units.append((("k", idx), self.kernel_notes[idx], [run_kernels[q]]))
                        else:
                            launch(f"RT(launch_{idx}(rt));", [run_kernels[q]])
                            if self.record_units:
                                self.hot_units.append((("k", idx), self.kernel_notes[idx], [run_kernels[q]]))
                        q += 1
                if forked and use_hoist():
                    # A second-stream launch only has to follow what it depends on: it moves up past every launch it
                    # does not conflict with, so that it runs beside the first stream's chain instead of after it (the
                    # weight gradients of a layer beside the backward pass of the layers below). So do the tiny kernels of
                    # the first stream (the optimizer's step-dependent scalars, which every update waits for). A launch
                    # stays where it is when it writes a tensor that shares arena bytes (those are planned in program order).
                    order = [(calls[x], meta.get(x)) for x in range(len(calls))]
                    for x in range(len(order)):
                        m_ = order[x][1]
                        if m_ is None or not m_[2] or (m_[1] & self.plan.shared):
                            continue
                        y = x
                        while y > 0 and order[y - 1][1] is not None:
                            r2, w2, _ = order[y - 1][1]
                            if (m_[1] & (r2 | w2)) or (m_[0] & w2):
                                break
                            y -= 1
                        if y < x:
                            order.insert(y, order.pop(x))
                    calls[:] = [t_ for t_, _ in order]
                if forked:
                    calls.append("RT(anvil_rt_join(rt));")
                if j == len(stmts) and tail is not None:
                    calls += tail
                    tail_done = True
                if in_loop and len(calls) > 1:
                    key = self.graph_keys
                    self.graph_keys += 1
                    out.append(f"{ind}{{ int g_ = anvil_rt_graph_begin(rt, {key}); if (g_ < 0) return 1;")
                    out.append(f"{ind}  if (g_ != 0) {{")
                    out += [f"{ind}    {c}" for c in calls]
                    out.append(f"{ind}    if (g_ == 1) RT(anvil_rt_graph_end(rt, {key}));")
                    out.append(f"{ind}  }} }}")
                else:
                    out += [f"{ind}{c}" for c in calls]
                i = j
                continue
            out += self.stmt(st, ind, in_loop)
            i += 1
        if tail is not None and not tail_done:
            out += [f"{ind}{c}" for c in tail]
        return out

    def read_scalar(self, b: kir.Buffer, var: str, ind: str) -> list[str]:
        if b.dtype == I32:
            return [f"{ind}int32_t {var}; RT(anvil_rt_read_i32(rt, {self.off(b)}, &{var}));"]
        return [f"{ind}float {var}; RT(anvil_rt_read_f32(rt, {self.off(b)}, &{var}));"]

    def stmt(self, st, ind: str, in_loop: bool) -> list[str]:
        if isinstance(st, kir.For):
            return self.for_(st, ind)
        if isinstance(st, kir.While):
            c = self.label("c")
            out = [f"{ind}while (1) {{"] + self.block(st.cond_block, ind + "    ", True)
            out += [f"{ind}    RT(anvil_rt_check_faults(rt));"] + self.read_scalar(st.cond, c, ind + "    ")
            out += [f"{ind}    if ({c} == 0) break;"]
            return out + self.block(st.body, ind + "    ", True) + [f"{ind}}}"]
        if isinstance(st, kir.If):
            c = self.label("c")
            out = [f"{ind}{{", f"{ind}RT(anvil_rt_check_faults(rt));"] + self.read_scalar(st.cond, c, ind)
            out += [f"{ind}if ({c} != 0) {{"] + self.block(st.then, ind + "    ", in_loop)
            if st.orelse.stmts:
                out += [f"{ind}}} else {{"] + self.block(st.orelse, ind + "    ", in_loop)
            return out + [f"{ind}}}", f"{ind}}}"]
        if isinstance(st, kir.AllReduce):
            return [f"{ind}RT(anvil_rt_allreduce(rt, {self.plan.bucket_off}UL, {self.plan.bucket_bytes // 4}L));"]
        if isinstance(st, kir.Break):
            return [f"{ind}break;"]
        if isinstance(st, kir.Continue):
            return [f"{ind}continue;"]
        if isinstance(st, kir.Print):
            return self.print_(st, ind)
        if isinstance(st, kir.Check):
            out = [f"{ind}{{ RT(anvil_rt_check_faults(rt)); long v_ = {st.value.const}L;"]
            for t, c in st.value.terms:
                if isinstance(t, kir.SRef):
                    x = self.label("s")
                    out += self.read_scalar(t.buf, x, ind + "  ")
                    out.append(f"{ind}  v_ += {c}L * (long){x};")
            out.append(f"{ind}  if (v_ < {st.lo}L || v_ > {st.hi}L) return anvil_rt_oob(rt, {c_string(st.message)}, v_); }}")
            return out
        if isinstance(st, kir.RTCall):
            return [f"{ind}RT(anvil_rt_check_faults(rt));"] + [ind + ln for ln in self.rtcall(st)]
        raise NotImplementedError(type(st).__name__)

    def bound(self, x, var: str, ind: str) -> list[str]:
        if isinstance(x, int):
            return [f"{ind}long {var} = {x}L;"]
        t = self.label("b")
        return self.read_scalar(x, t, ind) + [f"{ind}long {var} = (long){t};"]

    def for_(self, st: kir.For, ind: str) -> list[str]:
        """The counter lives in the arena (kernels read it through scalar references); the host keeps
        a mirror for the loop test and advances the device copy with a stream-ordered add."""
        c = self.off(st.counter)
        body_writes_counter = any(st.counter.root in s.kernel.writes() for b in kir.walk_blocks(st.body)
                                  for s in b.stmts if isinstance(s, kir.KernelStmt))
        has_continue = any(isinstance(s, kir.Continue) for b in kir.walk_blocks(st.body) for s in b.stmts)
        lo, hi, i = self.label("lo"), self.label("hi"), self.label("i")
        out = [f"{ind}{{"]
        out += self.bound(st.start, lo, ind + "    ") + self.bound(st.stop, hi, ind + "    ")
        out.append(f"{ind}    RT(anvil_rt_set_i32(rt, {c}, (int32_t){lo}));")
        tail = [f"RT(anvil_rt_add_i32(rt, {c}, {st.step}));", "RT(anvil_rt_stream_commit(rt));"]
        if body_writes_counter or has_continue:
            # The advance sits in the for statement's third clause, so a `continue` in the body reaches it
            # (anvil/backend/cuda.py:445 does the same); a failing runtime call there ends the loop through `bad`.
            bad = self.label("bad")
            out.append(f"{ind}    int {bad} = 0;")
            out.append(f"{ind}    for (long {i} = {lo}; {i} < {hi}; {i} = anvil_b200_advance(rt, {c}, {st.step}, &{bad})) {{")
            out += self.block(st.body, ind + "        ", True)
            out.append(f"{ind}    }}")
            out.append(f"{ind}    if ({bad}) return 1;")
        else:
            is_hot = st is self.hot and not any(isinstance(s, kir.Break) for b in kir.walk_blocks(st.body) for s in b.stmts)
            body = self.block(st.body, ind + "        ", True, tail)
            if is_hot:
                self.record_units = True
                self.hot_body = self.block(st.body, "    ", True, tail)
                self.record_units = False
                feed_k, self.feed_bufs = an.input_producers(self.prog, st)
                self.feed_kernels = feed_k
                self.hot_body_fed = self.block(st.body, "    ", True, tail, skip={k.id for k in feed_k})
                self.hot_counter = st.counter
                out.append(f"{ind}    if (mode == 1) return 2;     // paused at the training loop")
            out.append(f"{ind}    for (long {i} = {lo}; {i} < {hi}; {i} += {st.step}) {{")
            out += body
            out.append(f"{ind}    }}")
        out.append(f"{ind}}}")
        return out

    def table(self, ctype_, items) -> str:
        name = self.label("tab")
        self.tables.append(f"static const {ctype_} {name}[] = {{{', '.join(items)}}};")
        return name

    def strings(self, strs) -> str:
        return self.table("char *const", [c_string(s) for s in strs])

    def print_(self, st: kir.Print, ind: str) -> list[str]:
        err = 1 if st.err else 0
        out = [f"{ind}RT(anvil_rt_check_faults(rt));"]
        for it in list(st.items) + [kir.PrintItem("text", st.end)]:
            if it.kind == "text":
                if it.text:
                    out.append(f"{ind}RT(anvil_rt_print_text(rt, {c_string(it.text)}, {err}));")
            elif it.kind == "scalar":
                isint = 1 if it.buf.dtype == I32 else 0
                fint = 1 if (it.fmt and it.fmt.endswith("d")) else 0
                out.append(f"{ind}RT(anvil_rt_print_scalar(rt, {self.off(it.buf)}, {isint}, {c_string(it.fmt or '')}, {fint}, {err}));")
            elif it.kind == "tensor":
                b = it.buf
                dims = self.table("long", [str(d) for d in b.shape] or ["0"])
                out.append(f"{ind}RT(anvil_rt_print_tensor(rt, {self.off(b)}, {1 if b.dtype == I32 else 0}, {len(b.shape)}, {dims}));")
            elif it.kind == "pick":
                out.append(f"{ind}RT(anvil_rt_print_pick(rt, {self.off(it.buf)}, {self.strings(it.choices)}, {len(it.choices)}, {err}));")
            elif it.kind == "chars":
                out.append(f"{ind}RT(anvil_rt_print_chars(rt, {self.off(it.buf)}, {it.buf.numel}L));")
            else:
                raise NotImplementedError(it.kind)
        return out

    def rtcall(self, st: kir.RTCall) -> list[str]:
        a, n = st.args, st.name
        b = a.get("buf")
        if n == "seed":
            return [f"anvil_rt_seed(rt, {a['value'] & 0xFFFFFFFF}u);"]
        if n == "skip_rand":
            return ["anvil_rt_set_stream(rt, anvil_rt_get_stream(rt) + 1u);"]
        if n in ("iota", "iota_once"):
            return [f"RT(anvil_rt_iota(rt, {self.off(b)}, {b.numel}L));"]
        if n == "shuffle":
            return [f"RT(anvil_rt_shuffle(rt, {self.off(b)}, {b.numel}L));"]
        if n == "clock":
            return [f"RT(anvil_rt_clock(rt, {self.off(b)}));"]
        if n == "nonzero":
            src = a["src"]
            return [f"RT(anvil_rt_nonzero(rt, {self.off(src)}, {src.numel}L, {self.off(b)}, {b.numel}L));"]
        if n == "show":
            return [f"RT(anvil_rt_show(rt, {self.off(b)}, {a['rows']}L, {a['cols']}L, {self.strings(a['glyphs'])}, {len(a['glyphs'])}));"]
        if n == "exit":
            return ["anvil_rt_flush(rt);", f"return 1000 + ({int(a['value'])} & 255);"]
        if n in ("save", "load"):
            tab = self.label("ckpt")
            entries = ", ".join(f"{{{self.off(x)}, {x.root.ckpt_key}ULL}}" for x in a["bufs"])
            self.tables.append(f"static const anvil_rt_ckpt {tab}[] = {{{entries}}};")
            if n == "save":
                return [f"RT(anvil_rt_save(rt, {c_string(a['path'])}, {tab}, {len(a['bufs'])}L));"]
            return [f"{{ float ok_; RT(anvil_rt_load(rt, {c_string(a['path'])}, {tab}, {len(a['bufs'])}L, &ok_)); "
                    f"RT(anvil_rt_set_f32(rt, {self.off(b)}, ok_)); }}"]
        if n == "save_npy":
            tab = self.table("unsigned char", [str(x) for x in bytes(a["header"])])
            return [f"RT(anvil_rt_save_npy(rt, {c_string(a['path'])}, {tab}, {len(a['header'])}L, {self.off(b)}, {4 * b.numel}L));"]
        if n == "load_npy":
            return [f"RT(anvil_rt_load_npy(rt, {c_string(a['path'])}, {self.off(b)}, {b.numel}L, {a['offset']}L, {a['kind']}, {a['size']}));"]
        if n == "load_idx":
            return [f"RT(anvil_rt_load_idx(rt, {c_string(a['path'])}, {self.off(b)}, {b.numel}L, {int(a['header'])}L, {1 if b.dtype == I32 else 0}));"]
        if n == "load_csv":
            return [f"RT(anvil_rt_load_csv(rt, {c_string(a['path'])}, {self.off(b)}, {b.numel}L, {int(a['skip'])}L));"]
        if n == "load_bytes":
            return [f"RT(anvil_rt_load_bytes(rt, {c_string(a['path'])}, {self.off(b)}, {b.numel}L));"]
        if n == "input":                                     # the end of the input ends the program with status 0
            return [f"{{ int eof_; RT(anvil_rt_input(rt, {self.off(b)}, &eof_)); if (eof_) {{ anvil_rt_flush(rt); return 1000; }} }}"]
        if n == "sleep":
            return [f"{{ float s_; RT(anvil_rt_read_f32(rt, {self.off(b)}, &s_)); anvil_rt_flush(rt); "
                    f"if (s_ > 0) usleep((useconds_t)(s_ * 1e6f)); }}"]
        return [f"return anvil_rt_set_error(rt, \"anvil: runtime call `{n}` is not supported by the B200 back end\");"]

    # ---- the translation unit
    def generate(self) -> str:
        main = self.block(self.prog.main, "    ", False)
        # kernels that needed scratch were generated against scratch_off; re-plan with the final size
        # (scratch sits before the buffers, so growing it moves every buffer: generate twice)
        return self._assemble(main)

    def _assemble(self, main) -> str:
        externs = [b for b in self.prog.roots() if b.kind in ("input", "output")]
        out = [f"// Generated by anvil-b200 from {self.prog.name}: sm_100a kernels over one device arena.",
               "#include <cuda.h>", "#include <cuda_runtime.h>", "#include <math_constants.h>", "#include <stdint.h>", "#include <unistd.h>",
               '#include "anvil_cuda.h"', '#include "anvil_device.cuh"', '#include "anvil_gemm_simt.cuh"', '#include "anvil_gemm_sm100.cuh"', '#include "anvil_attn_sm100.cuh"', "",
               "#define RT(call) do { if ((call) != 0) return 1; } while (0)", "",
               "// advances a loop counter that lives in the arena and returns its new value; on a failure the loop ends",
               "static long anvil_b200_advance(anvil_rt *rt, unsigned long off, int step, int *bad) {",
               "    int32_t v = 0;",
               "    if (anvil_rt_add_i32(rt, off, step) != 0 || anvil_rt_read_i32(rt, off, &v) != 0) { *bad = 1; return 0x7fffffffffffffffL; }",
               "    return (long)v;", "}", ""]
        out += self.tables + [""]
        # --profile: one row per launch unit, "name label strategy" like the native back end's "name label location"
        names = [f"{k.name:<6} {k.label[:34]:<34} {note}" for k, note in zip(self.kernels, self.kernel_notes)]
        by_idx = {idx: key for key, idx in self.groups.items()}
        kinds = {"h": "fused products", "a": "fused attention", "z": "side by side"}
        for gi, note in enumerate(self.group_notes):
            key = by_idx.get(gi, ())
            what = kinds.get(key[0], "fused rows") if key and isinstance(key[0], str) else "fused rows"
            names.append(f"{'g%d' % gi:<6} {what:<34} {note}")
        out.append(f"#define PROF_GROUP0 {len(self.kernels)}")
        out.append("static const char *const prof_names[] = {" + ", ".join(c_string(x) for x in names) + ("" if names else '""') + "};")
        out.append("")
        out.append("static const char *const fault_messages[] = {\"\", " + ", ".join(c_string(m) for m in self.faults)
                   + ("" if self.faults else "\"\"") + "};")
        out += ["", "// ---------------------------------------------------------------- kernels"]
        for src in self.kernel_src:
            out += [src, ""]
        for src in self.group_src:
            out += [src, ""]
        out += ["// ---------------------------------------------------------------- launchers"]
        out += self.launchers + self.group_launchers
        nk = len(self.kernels)
        n = nk + len(self.groups)
        out += ["", "typedef int (*launch_fn)(anvil_rt *);",
                "static const launch_fn launch_table[] = {" + ", ".join([f"launch_{i}" for i in range(nk)]
                                                                        + [f"launch_group_{i}" for i in range(len(self.groups))])
                + ("0" if n == 0 else "") + "};",
                f'extern "C" int anvil_b200_kernel_count(void) {{ return {nk}; }}',
                f'extern "C" unsigned long anvil_b200_arena_bytes(void) {{ return {self.plan.size}UL; }}',
                f'extern "C" unsigned int anvil_b200_seed(void) {{ return {self.seed}u; }}',
                'extern "C" int anvil_b200_launch(anvil_rt *rt, int idx) {',
                f"    if (idx < 0 || idx >= {n}) return anvil_rt_set_error(rt, \"anvil: no such kernel\");",
                "    return launch_table[idx](rt);", "}", ""]
        out += ['extern "C" int anvil_b200_main(anvil_rt *rt, int mode) {',
                f"    anvil_rt_fault_messages(rt, fault_messages, {len(self.faults) + 1});"]
        out += main
        out += ["    RT(anvil_rt_check_faults(rt));", f"    RT(anvil_rt_profile_report(rt, prof_names, {len(self.kernels) + len(self.groups)}));",
                "    anvil_rt_flush(rt);", "    return 0;", "}", ""]
        out += ['extern "C" int anvil_b200_step(anvil_rt *rt) {   // one iteration of the training loop']
        if self.hot_body is not None:
            out += self.hot_body + ["    return 0;", "}"]
        else:
            out += ["    return anvil_rt_set_error(rt, \"anvil: the program has no training loop\");", "}"]
        out += ['extern "C" int anvil_b200_step_fed(anvil_rt *rt) {   // the same, inputs already copied in by the caller']
        if self.hot_body_fed is not None:
            out += self.hot_body_fed + ["    return 0;", "}"]
        else:
            out += ["    return anvil_rt_set_error(rt, \"anvil: the program has no training loop\");", "}"]
        # anvil.function ABI (anvil/pyapi.py:237-299): pointer slots + anvil_entry, host arrays
        if externs:
            out += ["", "// ---------------------------------------------------------------- anvil.function entry"]
            for b in externs:
                out.append(f'extern "C" {{ void *anvil_{b.name} = 0; }}')
            out += ['extern "C" { anvil_rt *anvil_b200_rt = 0; }',
                    'extern "C" int anvil_entry(void) {', "    anvil_rt *rt = anvil_b200_rt;",
                    "    if (!rt) return 1;", f"    anvil_rt_seed(rt, {self.seed}u);"]
            for b in externs:
                if b.kind == "input":
                    if b.nbytes:                     # an empty array has nothing to copy (its host pointer may be dangling)
                        out.append(f"    if (anvil_{b.name}) RT(anvil_rt_h2d_staged(rt, {self.off(b)}, anvil_{b.name}, {b.nbytes}UL));")
            out.append("    RT(anvil_b200_main(rt, 0));")
            for b in externs:
                if b.kind == "output":
                    if b.nbytes:
                        out.append(f"    if (anvil_{b.name}) RT(anvil_rt_d2h_staged(rt, anvil_{b.name}, {self.off(b)}, {b.nbytes}UL));")
            out += ["    return anvil_rt_sync(rt);", "}"]
        return "\n".join(out) + "\n"


def generate(prog: kir.Program, seed: int = 0):
    """Returns (source text, ProgramGen). Generated twice when split reductions need scratch space,
    because the scratch region sits in front of the buffers."""
    if os_environ("ANVIL_B200_IMPLICIT", "1") != "0":
        from .implicit import make_implicit
        from .refuse import _host_reads
        make_implicit(prog, _host_reads(prog))       # window copies (im2col) and their scattered gradients fold into the products
    if os_environ("ANVIL_B200_DETERMINISTIC", "1") != "0":
        from .determinism import make_deterministic
        make_deterministic(prog)                     # colliding `+=` get a fixed order (idempotent)
    if os_environ("ANVIL_B200_REFUSE", "1") != "0":
        from .refuse import fuse_consumers
        fuse_consumers(prog)                         # optimizer updates join the kernel that makes their gradient (idempotent)
    if os_environ("ANVIL_B200_REMAT", "1") != "0":
        from .refuse import _host_reads
        from .remat import rematerialize
        rematerialize(prog, _host_reads(prog))       # saved elementwise intermediates are recomputed where they are read (idempotent)
    if os_environ("ANVIL_B200_REFUSE", "1") == "all":
        from .refuse import fuse_consumers
        fuse_consumers(prog, only_updates=False)     # every elementwise consumer joins the kernel that makes its input
    g = ProgramGen(prog, seed)
    src = g.generate()
    if g.scratch_bytes > g.plan.scratch_bytes or g.side_scratch_bytes > g.plan.side_scratch_bytes:
        need, side_need = g.scratch_bytes, g.side_scratch_bytes
        g = ProgramGen(prog, seed)
        g.plan = g.make_plan(need, side_need)
        g.scratch_bytes, g.side_scratch_bytes = need, side_need
        src = g.generate()
    return src, g
