"""`anvil run --cuda` on B200: the drop-in for the reference's CUDA back end module.

Same entry points as anvil/backend/cuda.py:636-663 — `generate(prog, seed) -> str` and
`build(source, exe, emulate)` raising `CudaToolchainError` — plus `run`, which is what
`cli.build_cuda` + `subprocess.run([exe])` do in the reference (anvil/cli.py:127-136, 305-320).
`prog` may be a live `anvil.ir.Program` (unmodified, straight from `driver.compile_file`) or an
already converted `kir.Program`.

Differences that follow from running in-process on a device arena: `build` produces a shared
library, not an executable, and `emulate=True` is refused (there is no CPU path in this back end).
"""
from __future__ import annotations

import sys

from . import kir
from .backend import build as _build
from .backend import emit as _emit
from .backend.build import CudaToolchainError  # noqa: F401  (part of the interface)
from .program import AnvilRuntimeError, DeviceProgram  # noqa: F401


def as_kir(prog, name: str = "<program>") -> kir.Program:
    if isinstance(prog, kir.Program):
        return prog
    src = getattr(prog, "source", None)
    if src is not None and hasattr(src, "display_path"):
        name = src.display_path()
    return kir.from_anvil(prog, name)


def generate(prog, seed: int = 0) -> str:
    """The program as one sm_100a CUDA C++ translation unit."""
    return _emit.generate(as_kir(prog), seed)[0]


def build(source: str, exe: str, emulate: bool = False):
    """Compile generated source with nvcc for sm_100a into the shared library `exe`."""
    if emulate:
        raise CudaToolchainError("the B200 back end has no CPU emulation: run on a GPU, or use the "
                                 "reference interpreter (`anvil run --interp`)")
    _build.build_runtime()
    _build.build_program(source, exe)


def run(prog, seed: int = 0, capture: bool = False, device: int = 0, graphs: bool = True, profile: bool = False,
        check: str | None = None):
    """Compile (cached) and execute on the device. Returns the exit status — 0, 1 after a run-time
    error (message on stderr, as `anvil: runtime error: ...`), or the value of a failed `assert` —
    and, with capture=True, the text the program printed."""
    dp = DeviceProgram(as_kir(prog), seed=seed, device=device, graphs=graphs)
    try:
        if profile:                                      # `anvil run --profile` (anvil/cli.py:43): per-kernel table at the end
            dp.rtlib.anvil_rt_profile(dp.rt, 1)
        if check:                                        # `anvil run --check[=inf]` (anvil/interp.py:408-423)
            dp.rtlib.anvil_rt_check(dp.rt, 2 if check == "inf" else 1)
        code, text = dp.run(capture=capture)
        if code == 1 and dp.error:
            sys.stdout.flush()
            print(dp.error, file=sys.stderr)
        return (code, text) if capture else code
    finally:
        dp.close()


def main(argv=None) -> int:
    """`python -m anvil_lang_b200.cuda file.anvil [--seed N]` (needs the Anvil front end importable),
    or `... file.kir.json[.gz]` for a program lowered elsewhere."""
    import argparse
    ap = argparse.ArgumentParser(prog="anvil-b200")
    ap.add_argument("file")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--emit", action="store_true", help="print the generated CUDA instead of running")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--profile", action="store_true", help="time every kernel and print a breakdown at exit")
    ap.add_argument("--check", nargs="?", const="nan", choices=["nan", "inf"], help="stop at the first nan (or infinity) a kernel writes")
    ap.add_argument("--cost", action="store_true", help="`anvil cost --cuda`: the static FLOP / traffic estimate per source "
                    "line beside the time measured on the device and its share of the roofline")
    ap.add_argument("--gpus", type=int, default=int(__import__("os").environ.get("ANVIL_GPUS", "1")),
                    help="data-parallel run over this many GPUs of the node (also ANVIL_GPUS); needs the program compiled "
                    "for the per-rank batch, see anvil_lang_b200.dp")
    args = ap.parse_args(argv)
    if args.file.endswith((".json", ".json.gz")):
        prog = kir.load(args.file)
    else:
        from anvil.driver import compile_file          # the reference front end
        prog = as_kir(compile_file(args.file, seed=args.seed).program, args.file)
    if args.emit:
        print(generate(prog, args.seed))
        return 0
    if args.cost:
        from . import cost as _cost
        c = _cost.program_cost(prog)                     # before the emitter rewrites the program: the source's own kernels
        ms = _cost.measure(prog, c, seed=args.seed)
        print(_cost.report(prog, args.file, measured_ms=ms, cost=c))
        return 0
    if args.gpus > 1:
        return run_data_parallel(prog, args, argv)
    return run(prog, seed=args.seed, graphs=not args.no_graphs, profile=args.profile, check=args.check)


def run_data_parallel(prog, args, argv) -> int:
    """`--gpus N` / ANVIL_GPUS: one process per GPU. The first call starts N copies of this command with the
    rendezvous in the environment (RANK, WORLD_SIZE, LOCAL_RANK, MASTER_ADDR = 127.0.0.1, a free MASTER_PORT) and
    returns rank 0's exit status; each copy shards the program (`dp.shard`: the program must have been compiled for
    the per-rank batch), joins the NCCL process group and runs. Only rank 0 prints."""
    import os
    import subprocess
    if "RANK" not in os.environ:
        import socket
        sock = socket.socket()
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
        sock.close()
        cmd = [sys.executable, "-m", "anvil_lang_b200.cuda"] + list(argv if argv is not None else sys.argv[1:])
        procs = [subprocess.Popen(cmd, env=dict(os.environ, RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE=str(args.gpus),
                                                 MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), ANVIL_GPUS=str(args.gpus)))
                 for r in range(args.gpus)]
        codes = [p.wait() for p in procs]
        return codes[0] if codes[0] != 0 else max(codes)
    import torch
    import torch.distributed as dist
    from . import dp as _dp
    rank, world, dev = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{dev}"))
    try:
        sharded = _dp.shard(as_kir(prog), world)
        devprog = DeviceProgram(sharded, seed=args.seed, device=dev, graphs=not args.no_graphs)
        try:
            devprog.set_rank(rank)
            _dp.attach_native(devprog, rank, world)
            code, _ = devprog.run(capture=rank != 0)
            if code == 1 and devprog.error and rank == 0:
                print(devprog.error, file=sys.stderr)
            return code
        finally:
            devprog.close()
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    sys.exit(main())
