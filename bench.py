"""Benchmark: train samples/s of a BASELINE configuration on N B200s, one JSON line on stdout.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c5|c3|c4|c1] [--impl b200|reference]

A step is one iteration of the program's training loop (forward, backward, optimizer update).
`value` times K steps on the device with CUDA events on the program's stream, inputs produced on
the device; `e2e` times the same steps through the host-fed path: inputs prepared in pinned host
memory, copied in every step, the loss copied back every step. The dominant kernel's roofline and a
CPU baseline (the oracle's NumPy restatement of the reference interpreter, on a bounded sample) ride
on the same line. `--impl reference` prints the CPU arm alone.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    "c5": ("c5_transformer", 64, "decoder-only char transformer 6L D512 H8 T256 vocab 256, f32, Adam lr 3e-4, global batch 64"),
    "c3": ("c3_mlp_adam", 256, "MLP 784-1024-1024-10, f32, cross_entropy, Adam lr 1e-3, batch 256"),
    "c4": ("c4_cnn_sgd", 128, "CNN conv3x3 1-32-64 + linear 1600-10, f32, SGD lr 0.05, batch 128"),
    "c1": ("c1_mlp_sgd", 64, "MLP 784-128-10, f32, cross_entropy, SGD lr 0.1, batch 64"),
}
L2_BYTES = 126 << 20
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the kernel templates, from ncu captures of single launches
# (the heaviest shape of the template in the transformer step; summaries of the captures are kept with the project's
# profiles). Keyed by template.
NCU_TRAFFIC_PER_LAUNCH = {"gemm tc": 208.6e6 + 24.9e6}          # 16384 x 512 x 2048 (+ bias + residual): 176 MB algorithmic


def load_program(name):
    from anvil_lang_b200 import kir
    return kir.load(os.path.join(ROOT, "anvil_lang_b200", "programs", f"{name}.kir.json.gz"))


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "source": "measured (MEASURED_PEAKS.json)"}
    return {"hbm_gbs": 6650.0, "source": "fallback"}


def measure_tf32_peak():
    """Dense TF32 matmul throughput measured like the driver measures bf16: torch.matmul 8192^3,
    best of 10, CUDA events. The 3xTF32 roof is a third of it."""
    try:
        import torch
        torch.backends.cuda.matmul.allow_tf32 = True
        a = torch.randn(8192, 8192, device="cuda")
        b = torch.randn(8192, 8192, device="cuda")
        for _ in range(3):
            a @ b
        best = 1e9
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            a @ b
            e1.record()
            e1.synchronize()
            best = min(best, e0.elapsed_time(e1))
        del a, b
        torch.cuda.empty_cache()
        return 2 * 8192 ** 3 / (best * 1e-3) / 1e12
    except Exception:
        return None


class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, device=0):
        self.path = tempfile.mktemp(suffix=".csv")
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={device}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return None
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        os.unlink(self.path)
        if not sm:
            return None
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons), "samples": len(sm)}


REDUCED = {          # whole training steps the reference interpreter finishes in seconds: the same program at a reduced size
    "c5_transformer": {"BATCH": 2, "LAYERS": 2, "D": 128, "HEADS": 2, "T": 256},
    "c3_mlp_adam": {}, "c4_cnn_sgd": {}, "c1_mlp_sgd": {},
}


def step_flops(prog):
    from anvil_lang_b200 import kir
    from anvil_lang_b200.backend import analysis as an
    hot = an.hot_loop(prog)
    return sum(an.kernel_flops(st.kernel) for st in hot.body.stmts if isinstance(st, kir.KernelStmt))


class ReferenceSteps:
    """The reference implementation itself (oracle/_ref: its front end and its NumPy interpreter, anvil/interp.py) running
    whole training steps of a configuration on the host. Configurations whose full-size step takes hours on the
    interpreter (the transformer: 8969 s per step, measured when the golden losses were made) run at a reduced size —
    same program text, smaller constants — and the time is scaled to the full size by the FLOP count of a step."""

    def __init__(self, name):
        ref = os.path.join(ROOT, "oracle", "_ref")
        if not os.path.isdir(os.path.join(ref, "anvil")):
            raise ImportError("oracle/_ref is absent")
        sys.path.insert(0, ref)
        sys.dont_write_bytecode = True
        os.environ.setdefault("ANVIL_CACHE", tempfile.mkdtemp(prefix="anvil_cache_"))
        from anvil import ir
        from anvil.driver import compile_file
        from anvil.interp import Interpreter
        from anvil_lang_b200 import kir
        from anvil_lang_b200.backend import analysis as an
        consts = REDUCED[name]
        c = compile_file(os.path.join(ROOT, "anvil_lang_b200", "programs", f"{name}.anvil"), consts=consts or None)
        k = kir.from_anvil(c.program, name)
        hot = an.hot_loop(k)
        self.scale = step_flops(load_program(name)) / step_flops(k)
        self.batch_scale = 1.0
        self.what = ("one whole training step on the reference interpreter (oracle/_ref) at full size" if not consts else
                     "one whole training step on the reference interpreter (oracle/_ref) at reduced size ("
                     + ", ".join(f"{a} {b}" for a, b in consts.items()) + f"), scaled to the full step by FLOP count x{self.scale:.0f}")
        outer = self

        class Pause(Exception):
            pass

        class Stepper(Interpreter):
            def exec_for(self, st: ir.For):
                if st.counter.id != hot.counter.id:
                    return super().exec_for(st)
                cnt = self.arr(st.counter)
                cnt[0] = self.bound(st.start)
                outer.body, outer.counter, outer.step_by = st.body, cnt, st.step
                raise Pause()
        self.it = Stepper(c.program, out=open(os.devnull, "w"), seed=0)
        try:
            self.it.run()
        except Pause:
            pass

    def step(self) -> float:
        """Seconds of one training step (at the size this object runs)."""
        t = time.perf_counter()
        self.it.exec_block(self.body)
        self.counter[0] += self.step_by
        return time.perf_counter() - t


def cpu_sample(name, batch, budget_s=20.0, steps=1):
    """The CPU baseline on a bounded sample: whole steps of the reference interpreter itself where oracle/_ref exists
    (`kind: "reference"`), else of the NumPy port in oracle/kir_interp.py on the first kernels of a step."""
    try:
        ref = ReferenceSteps(name)
    except Exception as e:
        return cpu_sample_port(name, batch, budget_s, why=str(e))
    secs = [ref.step() for _ in range(steps)]
    t = float(np.median(secs))
    return {"value": batch / (t * ref.scale), "unit": "samples/s", "cores": 1, "kind": "reference", "sample": ref.what,
            "sample_seconds": t, "scale": ref.scale}


def cpu_sample_port(name, batch, budget_s=20.0, why=""):
    """The oracle (NumPy restatement of the reference interpreter, reduction bodies
    materialised and summed like anvil/interp.py:435-466) runs the program's start-up and then the
    training step's kernels in order until `budget_s` seconds of kernel time have passed. Throughput
    for the whole step is extrapolated by the share of the step's FLOPs that the sample covered."""
    from anvil_lang_b200 import kir
    from anvil_lang_b200.backend import analysis as an
    from oracle.kir_interp import Oracle
    prog = load_program(name)
    hot = an.hot_loop(prog)
    o = Oracle(prog, out=open(os.devnull, "w"), seed=0)

    class Reached(Exception):
        pass

    def run_until_hot(block):
        for st in block.stmts:
            if st is hot:
                o.arr(hot.counter)[0] = hot.start if isinstance(hot.start, int) else o.bound(hot.start)
                raise Reached()
            if isinstance(st, kir.For):
                o.arr(st.counter)[0] = o.bound(st.start)
                run_until_hot(st.body)
            else:
                o.stmt(st)
    try:
        run_until_hot(prog.main)
    except Reached:
        pass
    kernels = [st.kernel for st in hot.body.stmts if isinstance(st, kir.KernelStmt)]
    total_flops = sum(an.kernel_flops(k) for k in kernels)
    done_flops, spent, n = 0, 0.0, 0
    for k in kernels:
        t = time.perf_counter()
        o.kernel(k)
        spent += time.perf_counter() - t
        done_flops += an.kernel_flops(k)
        n += 1
        if spent >= budget_s:
            break
    step_seconds = spent * total_flops / max(done_flops, 1)
    return {"value": batch / step_seconds, "unit": "samples/s", "cores": 1, "kind": "port",
            "sample": f"first {n} of {len(kernels)} kernels of one full-size training step "
                      f"({100.0 * done_flops / total_flops:.2f}% of its FLOPs, {spent:.1f} s), extrapolated by FLOP share"
                      + (f" (the reference copy was not usable: {why})" if why else ""),
            "sample_seconds": spent, "scale": total_flops / max(done_flops, 1)}


def reference_arm(args, name, batch, desc):
    """`--impl reference`: the CPU implementation alone. Each step is one bounded sample (a whole training step of the
    reference interpreter, at reduced size where the full size takes hours); `ms_per_step` is the time of a sample,
    `value` the configuration's throughput that follows from it."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    try:
        ref = ReferenceSteps(name)
        for _ in range(args.warmup):
            ref.step()
        secs = [ref.step() for _ in range(args.steps)]
        t = float(np.median(secs))
        last = {"value": batch / (t * ref.scale), "unit": "samples/s", "cores": 1, "kind": "reference", "sample": ref.what,
                "sample_seconds": t, "scale": ref.scale}
    except ImportError:
        vals = []
        for i in range(args.warmup + args.steps):
            last = cpu_sample_port(name, batch, budget_s=args.cpu_budget)
            if i >= args.warmup:
                vals.append(last["value"])
        last["value"] = float(np.median(vals))
        t = last["sample_seconds"]
    v = last["value"]
    line = {"impl": "reference", "metric": "train samples/s", "value": v, "unit": "samples/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * t, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic (the program's own seeded RNG, seed 0)",
            "config": {"workload": desc, "global_batch": batch}, "cpu_baseline": last,
            "e2e": {"value": v, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))
    return 0


C2_SOURCES = {       # the standalone `anvil.function` kernels of the second BASELINE configuration
    "rows": ("fn rows(x: [n, d]) = softmax(x)\n", "row softmax f32[4096,4096]"),
    "ln": ("fn ln(x: [n, d], g: [d], b: [d]) = layer_norm(x) * g + b\n", "layer norm f32[8192,1024]"),
    "lin": ("fn lin(x: [n, d], W: [d, k], b: [k]):\n    y[i, k] = sum x[i, j] * W[j, k] + b[k]\n    return y\n",
            "Linear f32[8192,1024] x [1024,4096] + bias"),
}


def c2_inputs(name):
    rng = np.random.default_rng(0)
    if name == "rows":
        return [rng.standard_normal((4096, 4096), dtype=np.float32)]
    if name == "ln":
        return [rng.standard_normal((8192, 1024), dtype=np.float32), np.ones(1024, np.float32), np.zeros(1024, np.float32)]
    return [rng.standard_normal((8192, 1024), dtype=np.float32), rng.standard_normal((1024, 4096), dtype=np.float32) * np.float32(0.02),
            rng.standard_normal(4096, dtype=np.float32)]


def time_training_config(name, batch, steps=20, warmup=3):
    """(device ms per step, end-to-end ms per step) of a training configuration on one GPU; L2 flushed between steps
    when a step's traffic would fit in it."""
    from anvil_lang_b200 import kir
    from anvil_lang_b200.backend import analysis as an
    from anvil_lang_b200.feed import HostFeeder, Unsupported, pinned_array
    from anvil_lang_b200.program import DeviceProgram
    prog = load_program(name)
    dp = DeviceProgram(prog, seed=0)
    try:
        dp.rtlib.anvil_rt_capture(dp.rt, 1)
        dp.prologue()
        hot = an.hot_loop(prog)
        loss = dp.buffer("loss")
        step_bytes = sum(an.kernel_bytes(st.kernel) for st in hot.body.stmts if isinstance(st, kir.KernelStmt))
        flush = step_bytes < 2 * L2_BYTES
        for _ in range(warmup):
            dp.step()
        dp.sync()
        ms = 0.0
        for _ in range(steps):
            if flush:
                flush_l2(dp)
            dp.timer_begin()
            dp.step()
            ms += dp.timer_end()
        e2e = None
        try:
            feeder = HostFeeder(dp, 0)
            feeder.load_host_copies()
            host_loss = pinned_array(dp.rtlib, (1,), np.float32)
            counter = int(dp.read(hot.counter).reshape(-1)[0])
            stream = int(dp.rtlib.anvil_rt_get_stream(dp.rt))
            times = []
            for i in range(steps + 2):
                t0 = time.perf_counter()
                feeder.prepare(counter, stream, dp.seed)
                feeder.push()
                dp.step_fed()
                dp.copy_out_async(host_loss.ctypes.data, loss, 4)
                dp.sync()
                times.append(time.perf_counter() - t0)
                counter += hot.step
                stream += feeder.rand_streams
            e2e = 1e3 * float(np.mean(times[2:]))
        except Unsupported:
            pass
        return {"ms_per_step": ms / steps, "samples_per_s": batch * steps / (ms * 1e-3),
                "e2e_ms_per_step": e2e, "e2e_samples_per_s": (batch / (e2e * 1e-3)) if e2e else None,
                "l2": "flushed between timed steps" if flush else "step traffic exceeds L2"}
    finally:
        dp.close()


def time_function_config(name):
    """A standalone function: device microseconds of a call with the arguments resident in the arena, and milliseconds of
    the reference-facing call (NumPy arrays in pageable host memory in, NumPy array out)."""
    from anvil_lang_b200 import pyapi
    src, what = C2_SOURCES[name]
    f = pyapi.function(src, name=name)
    args = c2_inputs(name)
    out = f(*args)                                       # compiles / loads, first call
    comp = f.lower(*args)
    dp = comp.dp
    for _ in range(3):
        comp.run_resident()
    dp.sync()
    best = 1e9
    for _ in range(10):
        flush_l2(dp)
        dp.timer_begin()
        comp.run_resident()
        best = min(best, dp.timer_end())
    times = []
    for _ in range(5):
        t0 = time.perf_counter()
        out = f(*args)
        times.append(time.perf_counter() - t0)
    nbytes_in, nbytes_out = sum(a.nbytes for a in args), out.nbytes
    return {"what": what, "device_us": 1e3 * best, "e2e_ms": 1e3 * float(np.median(times)),
            "h2d_bytes": nbytes_in, "d2h_bytes": nbytes_out}


def other_configs():
    """The BASELINE configurations besides the headline one, each device-timed and end to end (one GPU)."""
    out = {}
    for key in ("c1", "c3", "c4"):
        name, batch, desc = WORKLOADS[key]
        try:
            out[key] = dict(time_training_config(name, batch), workload=desc)
        except Exception as e:                           # a secondary measurement must not lose the headline line
            out[key] = {"error": str(e)[:200]}
    for name in C2_SOURCES:
        try:
            out["c2_" + name] = time_function_config(name)
        except Exception as e:
            out["c2_" + name] = {"error": str(e)[:200]}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="c5", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--cpu-budget", type=float, default=20.0)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-configs", action="store_true", help="skip the other BASELINE configurations")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    name, batch, desc = WORKLOADS[args.workload]
    if args.impl == "reference":
        return reference_arm(args, name, batch, desc)

    from anvil_lang_b200 import dp as dpmod
    from anvil_lang_b200 import kir
    from anvil_lang_b200.backend import analysis as an
    from anvil_lang_b200.feed import HostFeeder, Unsupported, pinned_array
    from anvil_lang_b200.program import DeviceProgram

    world = int(os.environ.get("WORLD_SIZE", "1")) if args.gpus > 1 else 1
    rank = int(os.environ.get("RANK", "0")) if world > 1 else 0
    device = int(os.environ.get("LOCAL_RANK", "0")) if world > 1 else 0
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(device)
        if rank == 0:                                    # the communicator's own report (ranks, transport) goes to stderr
            os.environ.setdefault("NCCL_DEBUG", "INFO")
            os.environ.setdefault("NCCL_DEBUG_SUBSYS", "INIT")
            os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{device}"))
        if batch % world:
            raise SystemExit(f"global batch {batch} does not divide over {world} GPUs")
        prog = dpmod.shard(load_program(f"{name}.b{batch // world}"), world)
    else:
        prog = load_program(name)

    dp = DeviceProgram(prog, seed=0, device=device)
    dp.set_rank(rank)
    comm = None
    if world > 1:
        nranks = dpmod.attach_native(dp, rank, world)        # NCCL inside the runtime; the id travelled through the process group
        comm = {"backend": "nccl in libanvil_cuda.so (ncclAllReduce on the program's stream)", "nranks": nranks}
    dp.rtlib.anvil_rt_capture(dp.rt, 1)                 # the program's own prints stay off stdout
    dp.prologue()
    loss = dp.buffer("loss")
    hot = an.hot_loop(prog)
    kernels = [st.kernel for st in hot.body.stmts if isinstance(st, kir.KernelStmt)]
    step_bytes = sum(an.kernel_bytes(k) for k in kernels)
    flush = step_bytes < 2 * L2_BYTES                   # working set may sit in L2: evict it between steps
    W, K = args.warmup, args.steps

    def barrier():
        dp.sync()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if dist is None:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=f"cuda:{device}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for _ in range(W):
        dp.step()
    barrier()
    dp.rtlib.anvil_rt_capture(dp.rt, 1)                 # (re)starting capture drops the text so far

    # ---- device-resident steps, CUDA events on the program's stream, max over ranks
    clocks = ClockSampler(device) if rank == 0 else None
    launches0 = dp.launches
    t_wall = time.perf_counter()
    if not flush:
        dp.timer_begin()
        for _ in range(K):
            dp.step()
        ms = dp.timer_end()
    else:
        ms = 0.0
        for _ in range(K):
            flush_l2(dp)
            dp.timer_begin()
            dp.step()
            ms += dp.timer_end()
    barrier()
    wall = time.perf_counter() - t_wall
    ms = max_over_ranks(ms)
    launches = dp.launches - launches0
    last_loss = float(dp.read(loss).reshape(-1)[0])
    value = batch * K / (ms * 1e-3)

    # ---- end to end: inputs from pinned host memory every step, loss back to the host every step
    try:
        feeder = HostFeeder(dp, rank)
        feeder.load_host_copies()
        host_loss = pinned_array(dp.rtlib, (1,), np.float32)
        seed = dp.seed
        counter = int(dp.read(hot.counter).reshape(-1)[0])
        stream = int(dp.rtlib.anvil_rt_get_stream(dp.rt))

        def fed_step(read_loss):
            nonlocal counter, stream
            feeder.prepare(counter, stream, seed)
            feeder.push()
            dp.step_fed()
            if read_loss:
                dp.copy_out_async(host_loss.ctypes.data, loss, 4)
                dp.sync()
            counter += hot.step
            stream += feeder.rand_streams
        for i in range(2):                               # warm the fed path (its own launch graphs)
            fed_step(False)
        barrier()
        t0 = time.perf_counter()
        for i in range(K):
            fed_step(True)
        barrier()
        t_e2e = max_over_ranks(time.perf_counter() - t0)
        e2e = {"value": batch * K / t_e2e, "unit": "samples/s", "h2d_bytes_per_step": feeder.bytes_per_step * world,
               "d2h_bytes_per_step": 4 * world, "ms_per_step": 1e3 * t_e2e / K, "loss": float(host_loss[0])}
    except Unsupported as e:
        e2e = {"value": None, "unit": "samples/s", "why": str(e)}
    clk = clocks.stop() if clocks is not None else None

    # ---- the dominant kernel and its roofline (rank 0; a collective cannot be timed alone)
    if dist is not None:
        dist.barrier()
    if rank != 0:
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        return 0
    nk = len(dp.gen.kernels)
    rows = []                                            # (ms, note, kernels of the unit)
    for (kind, idx), unote, ks in dp.gen.hot_units:
        rows.append((dp.time_kernel(idx if kind == "k" else nk + idx, 3), unote, ks))
    total_k = sum(r[0] for r in rows)
    # A kernel = one __global__ template; its launches differ in shape and statements only. Launch units are grouped by
    # the template they run (the first words of their strategy note); the dominant kernel is the template with the most
    # time in the step, and its roofline is that of its launches taken together: their algorithmic FLOPs (or bytes)
    # over their summed CUDA-event time.
    def template_of(unote):
        w = unote.split()
        return " ".join(w[:2]) if w[0] in ("gemm", "attention", "split", "coop", "eltwise", "rowgroup") else w[0]
    by_template: dict = {}
    for t, unote, ks in rows:
        by_template.setdefault(template_of(unote), []).append((t, unote, ks))
    top_name, top_rows = max(by_template.items(), key=lambda kv: sum(r[0] for r in kv[1]))
    top_ms = sum(r[0] for r in top_rows)
    peaks = measured_peaks()
    tf32 = measure_tf32_peak()
    tensor_peak = (tf32 / 3.0) if tf32 else 1590.0 / 2 / 3
    tensor_src = ("torch.matmul tf32 8192^3 best of 10 (cuBLAS), measured in this run: %.0f TFLOP/s, / 3 for 3xTF32; the tensor "
                  "pipe's own issue ceiling for kind::tf32, measured with a stand-alone issue loop, is 991 TFLOP/s" % tf32) if tf32 \
        else "fallback: half the bf16 fallback peak / 3"
    unit_flops = lambda ks: sum(an.kernel_flops(k_) for k_ in ks)
    common = {"kernel": f"{top_name} (all {len(top_rows)} launches of the template in one step)", "launches_per_step": len(top_rows),
              "avg_launch_ms": top_ms / len(top_rows), "share_of_step": top_ms / total_k}
    shapes: dict = {}
    for t, unote, ks in top_rows:
        g = shapes.setdefault(" ".join(unote.split()[:3]) + " <" + "+".join(sorted({k_.label for k_ in ks}))[:40] + ">", [0.0, 0, 0.0, 0.0])
        g[0] += t; g[1] += 1; g[2] += unit_flops(ks); g[3] += an.group_bytes(ks, dp.gen.dead_roots)
    if top_name.startswith("gemm"):
        flops = sum(unit_flops(ks) for _, _, ks in top_rows)
        achieved = flops / (top_ms * 1e-3) / 1e12
        roof = {"bound": "tensor", "achieved": achieved, "peak": tensor_peak, "unit": "TFLOP/s", "frac": achieved / tensor_peak,
                "traffic": NCU_TRAFFIC_PER_LAUNCH.get(top_name), **common, "peak_source": tensor_src,
                "by_shape": {k_: {"ms": round(v[0], 3), "launches": v[1], "TFLOP/s": round(v[2] / (v[0] * 1e-3) / 1e12, 1)}
                             for k_, v in sorted(shapes.items(), key=lambda kv: -kv[1][0])[:10]}}
    else:
        nbytes = sum(an.group_bytes(ks, dp.gen.dead_roots) for _, _, ks in top_rows)
        achieved = nbytes / (top_ms * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "traffic": NCU_TRAFFIC_PER_LAUNCH.get(top_name), **common,
                "peak_source": peaks["source"]}
    classes = {}
    for t, unote, _ in rows:
        c = template_of(unote)
        classes[c] = classes.get(c, 0.0) + t
    roof["step_ms_by_class"] = {c: round(v, 3) for c, v in sorted(classes.items(), key=lambda kv: -kv[1])}
    step_flops_all = sum(an.kernel_flops(k_) for k_ in kernels)
    roof["whole_step"] = {"flops": step_flops_all, "achieved": step_flops_all / (ms / K * 1e-3) / 1e12, "unit": "TFLOP/s",
                          "frac": step_flops_all / (ms / K * 1e-3) / 1e12 / tensor_peak,
                          "note": "all FLOPs of a step (contractions are 94 % of them) over the step time, against the 3xTF32 roof"}

    cpu = None if (args.no_cpu or world > 1) else cpu_sample(name, batch, budget_s=args.cpu_budget)
    line = {"metric": "train samples/s", "value": value, "unit": "samples/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic (the program's own seeded RNG, seed 0)",
            "config": {"workload": desc, "global_batch": batch, "parallelism": f"dp{world}",
                       "l2": ("per-step traffic %.0f MB exceeds the 126 MB L2, no flush" % (step_bytes / 1e6)) if not flush
                       else "L2 flushed with a 256 MB write between timed steps"},
            "e2e": e2e, "gpu_launches": int(launches), "clocks": clk, "roofline": roof, "cpu_baseline": cpu,
            "wall_ms_per_step": 1e3 * wall / K, "last_loss": last_loss}
    if comm is not None:
        line["comm"] = comm
    if world == 1 and not args.no_configs and args.workload == "c5":
        dp.close()
        line["configs"] = other_configs()
    print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    dp.close()
    return 0


_flush_buf = {}


def flush_l2(dp):
    """Evicts L2 by writing 256 MB of device memory with torch (outside the timed events)."""
    import torch
    if "t" not in _flush_buf:
        _flush_buf["t"] = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _flush_buf["t"].zero_()
    torch.cuda.synchronize()


if __name__ == "__main__":
    sys.exit(main())
