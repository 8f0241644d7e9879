"""One rank of a data-parallel run on the CPU oracle (gloo). Usage: dp_worker.py KIR WORLD OUT
Environment: RANK, WORLD_SIZE, MASTER_ADDR, MASTER_PORT."""
import io
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from anvil_lang_b200 import dp, kir  # noqa: E402
from oracle.kir_interp import Oracle  # noqa: E402


def main():
    path, world, out_path = sys.argv[1], int(sys.argv[2]), sys.argv[3]
    rank = int(os.environ["RANK"])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    prog = dp.shard(kir.load(path), world)
    out = io.StringIO()
    o = Oracle(prog, out=out, seed=0)
    o.arr(prog.rank_buf)[0] = rank

    def allreduce(arrays):
        for a in arrays:
            t = torch.from_numpy(a)
            dist.all_reduce(t)
    o.allreduce = allreduce
    o.run()
    params = {b.name: o.arr(b)[:b.numel].tolist() for b in prog.roots() if b.kind == "param"}
    gathered = [None] * world
    dist.all_gather_object(gathered, {"text": out.getvalue(), "params": params})
    if rank == 0:
        same = all(g["params"] == gathered[0]["params"] for g in gathered)
        with open(out_path, "w") as f:
            json.dump({"text": gathered[0]["text"], "params": params, "identical_across_ranks": same}, f)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
