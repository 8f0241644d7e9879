"""Data parallelism on real GPUs: 2 ranks over NCCL must reproduce the reference interpreter's
global-batch losses (needs at least 2 GPUs; skipped otherwise)."""
import json
import os
import re
import subprocess
import sys

import numpy as np
import pytest

from util import GOLDEN, ROOT

pytestmark = pytest.mark.gpu


def gpu_count():
    try:
        out = subprocess.run(["nvidia-smi", "-L"], capture_output=True, text=True, timeout=30).stdout
        return len([ln for ln in out.splitlines() if ln.startswith("GPU ")])
    except Exception:
        return 0


def run_two_ranks(kir_name, steps, collective, port):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", ANVIL_DP_COLLECTIVE=collective)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(ROOT, "tests", "dp_gpu_worker.py"),
           os.path.join(GOLDEN, f"{kir_name}.kir.json.gz"), str(steps)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    m = re.search(r"DPLOSSES (\[.*\])", r.stdout)
    assert m, (r.stdout[-2000:], r.stderr[-6000:])
    return json.loads(m.group(1))


@pytest.mark.skipif(gpu_count() < 2, reason="needs 2 GPUs")
def test_runtime_collective_is_bit_reproducible():
    """NCCL inside the runtime with the algorithm, protocol and channel count pinned: two separate 2-rank runs give the
    same losses bit for bit, and the same values as the collective routed through torch.distributed."""
    a = run_two_ranks("dp_transformer.b2", 6, "native", 29541)
    b = run_two_ranks("dp_transformer.b2", 6, "native", 29542)
    assert a == b
    c = run_two_ranks("dp_transformer.b2", 6, "torch", 29543)
    assert np.allclose(a, c, rtol=1e-5)


@pytest.mark.skipif(gpu_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("kir_name,golden,steps", [("dp_mlp.b16", "dp_mlp", 8), ("dp_transformer.b2", "transformer_small", 6)])
def test_two_ranks_match_global_batch(kir_name, golden, steps):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29533", os.path.join(ROOT, "tests", "dp_gpu_worker.py"),
           os.path.join(GOLDEN, f"{kir_name}.kir.json.gz"), str(steps)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    m = re.search(r"DPLOSSES (\[.*\])", r.stdout)
    assert m, (r.stdout[-2000:], r.stderr[-6000:])
    got = json.loads(m.group(1))
    want = [float(x) for x in re.findall(r"loss (\d+\.\d+)", open(os.path.join(GOLDEN, f"{golden}.out.txt")).read())][:steps]
    assert np.allclose(got, want, rtol=1e-3), (got, want)
