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
# dram__bytes_read.sum + dram__bytes_write.sum of one launch, from the ncu captures summarised under
# profiles/ (gemm_tc_pp_16384x512x2048.md, c5_transformer_step_launches.md), keyed by the kernel's strategy note
NCU_TRAFFIC = {"gemm tc 1x16384x512x2048": 141.8e6 + 13.9e6, "gemm tc 1x512x512x16384": 67.3e6 + 5.0e6,
               "gemm tc 1x16384x512x512": 34.6e6 + 0.6e6}


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


def cpu_sample(name, batch, budget_s=20.0):
    """The CPU baseline: the oracle (NumPy restatement of the reference interpreter, reduction bodies
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
                      f"({100.0 * done_flops / total_flops:.2f}% of its FLOPs, {spent:.1f} s), extrapolated by FLOP share"}


def reference_arm(args, name, batch, desc):
    """`--impl reference`: the CPU implementation alone. Each step is one bounded sample."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    vals, last = [], None
    for i in range(args.warmup + args.steps):
        last = cpu_sample(name, batch, budget_s=args.cpu_budget)
        if i >= args.warmup:
            vals.append(last["value"])
    v = float(np.median(vals))
    last["value"] = v
    line = {"impl": "reference", "metric": "train samples/s", "value": v, "unit": "samples/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * batch / v, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic (program RNG, seed 0)",
            "config": {"workload": desc, "global_batch": batch}, "cpu_baseline": last,
            "e2e": {"value": v, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="c5", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--cpu-budget", type=float, default=20.0)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
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
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{device}"))
        if batch % world:
            raise SystemExit(f"global batch {batch} does not divide over {world} GPUs")
        prog = dpmod.shard(load_program(f"{name}.b{batch // world}"), world)
    else:
        prog = load_program(name)

    dp = DeviceProgram(prog, seed=0, device=device)
    dp.set_rank(rank)
    if world > 1:
        dpmod.attach(dp, device)
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
    # Launches of the same generated kernel (same template, shape and statements; only the tensors differ) are
    # one kernel: the dominant one is the group with the largest total time, and the roofline is that of its
    # average launch.
    groups: dict = {}
    for t, unote, ks in rows:
        key = (" ".join(unote.split()[:3]) if unote.startswith("gemm") else unote, "+".join(k_.label for k_ in ks))
        g = groups.setdefault(key, [0.0, 0, ks, unote])
        g[0] += t
        g[1] += 1
    (_, _), (grp_ms, grp_n, top_ks, note) = max(groups.items(), key=lambda kv: kv[1][0])
    top_ms = grp_ms / grp_n
    top = top_ks[0]
    peaks = measured_peaks()
    common = {"kernel": f"{top.name} {top.label} [{note}]", "launches_per_step": grp_n, "avg_launch_ms": top_ms,
              "share_of_step": grp_ms / total_k}
    if note.startswith("gemm"):
        tf32 = measure_tf32_peak()
        flops = an.kernel_flops(top)
        achieved = flops / (top_ms * 1e-3) / 1e12
        peak = (tf32 / 3.0) if tf32 else 1590.0 / 2 / 3
        gemm_ms = sum(t for t, unote, _ in rows if unote.startswith("gemm"))
        gemm_flops = sum(an.kernel_flops(ks[0]) for _, unote, ks in rows if unote.startswith("gemm"))
        roof = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "traffic": next((v for k_, v in NCU_TRAFFIC.items() if note.startswith(k_)), None), **common,
                "all_contractions": {"share_of_step": gemm_ms / total_k, "achieved": gemm_flops / (gemm_ms * 1e-3) / 1e12},
                "peak_source": "torch.matmul tf32 8192^3 best of 10, measured in this run, / 3 for 3xTF32" if tf32
                else "fallback: half the bf16 fallback peak / 3"}
    else:
        nbytes = an.group_bytes(top_ks, dp.gen.dead_roots)
        achieved = nbytes / (top_ms * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "traffic": None, **common, "peak_source": peaks["source"]}
    classes = {}
    for t, unote, _ in rows:
        c = " ".join(unote.split()[:2])
        classes[c] = classes.get(c, 0.0) + t
    roof["step_ms_by_class"] = {c: round(v, 3) for c, v in sorted(classes.items(), key=lambda kv: -kv[1])}

    cpu = None if (args.no_cpu or world > 1) else cpu_sample(name, batch, budget_s=args.cpu_budget)
    line = {"metric": "train samples/s", "value": value, "unit": "samples/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic (the program's own seeded RNG, seed 0)",
            "config": {"workload": desc, "global_batch": batch, "parallelism": f"dp{world}",
                       "l2": ("per-step traffic %.0f MB exceeds the 126 MB L2, no flush" % (step_bytes / 1e6)) if not flush
                       else "L2 flushed with a 256 MB write between timed steps"},
            "e2e": e2e, "gpu_launches": int(launches), "clocks": clk, "roofline": roof, "cpu_baseline": cpu,
            "wall_ms_per_step": 1e3 * wall / K, "last_loss": last_loss}
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
