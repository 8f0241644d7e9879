"""One rank of a data-parallel run on GPUs (NCCL), launched by torch.distributed.run.
Usage: dp_gpu_worker.py KIR STEPS — rank 0 prints `DPLOSSES [..]`."""
import os, sys, json
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch, torch.distributed as dist
from anvil_lang_b200 import kir, dp as dpmod
from anvil_lang_b200.program import DeviceProgram
rank, world, dev = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(dev)
dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{dev}"))
path, steps = sys.argv[1], int(sys.argv[2])
prog = dpmod.shard(kir.load(path), world)
p = DeviceProgram(prog, device=dev); p.set_rank(rank)
if os.environ.get("ANVIL_DP_COLLECTIVE", "native") == "native": dpmod.attach_native(p, rank, world)
else: dpmod.attach(p, dev)
p.rtlib.anvil_rt_capture(p.rt, 1)
p.prologue(); loss = p.buffer("loss"); out = []
for i in range(steps):
    p.step(); out.append(float(p.read(loss).reshape(-1)[0]))
if rank == 0: print("DPLOSSES", json.dumps(out))
dist.barrier(); dist.destroy_process_group()
