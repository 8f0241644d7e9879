"""Data parallelism on CPU ranks (gloo): the sharded per-rank programs, summed with one all-reduce
per step, must reproduce the single-process run at the global batch, and leave bit-identical
parameters on every rank."""
import json
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

from anvil_lang_b200 import dp, kir
from util import GOLDEN, ROOT, outputs_match


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def run_ranks(kir_path, world, tmp_path):
    out = str(tmp_path / "dp.json")
    port = free_port()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   OMP_NUM_THREADS="1")
        procs.append(subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "dp_worker.py"), kir_path, str(world), out],
                                      env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT))
    for p in procs:
        text, _ = p.communicate(timeout=600)
        assert p.returncode == 0, text.decode()[-3000:]
    return json.load(open(out))


@pytest.mark.parametrize("world,batch", [(2, 16), (4, 8)])
def test_mlp_ranks_match_global_batch(world, batch, tmp_path):
    got = run_ranks(os.path.join(GOLDEN, f"dp_mlp.b{batch}.kir.json.gz"), world, tmp_path)
    want = open(os.path.join(GOLDEN, "dp_mlp.out.txt")).read()          # the reference interpreter, batch 32
    ok, why = outputs_match(got["text"], want, rtol=1e-4, atol=1e-5)
    assert ok, why
    assert got["identical_across_ranks"]


def test_transformer_ranks_match_global_batch(tmp_path):
    got = run_ranks(os.path.join(GOLDEN, "dp_transformer.b2.kir.json.gz"), 2, tmp_path)
    want = open(os.path.join(GOLDEN, "transformer_small.out.txt")).read()
    ok, why = outputs_match(got["text"], want, rtol=1e-4, atol=1e-5)
    assert ok, why
    assert got["identical_across_ranks"]


def test_shard_structure():
    prog = kir.load(os.path.join(ROOT, "anvil_lang_b200", "programs", "c3_mlp_adam.b128.kir.json.gz"))
    dp.shard(prog, 2)
    from anvil_lang_b200.backend.analysis import hot_loop
    hot = hot_loop(prog)
    kinds = [type(s).__name__ for s in hot.body.stmts]
    assert kinds.count("AllReduce") == 1 and hot.stop == 234
    at = kinds.index("AllReduce")
    before = [s.kernel for s in hot.body.stmts[:at]]
    after = [s.kernel for s in hot.body.stmts[at + 1:] if isinstance(s, kir.KernelStmt)]
    assert not any(st.buf.root.kind in ("param", "state") for k in before for st in k.stores)
    assert all(k.red is None for k in after)
    assert sum(b.nbytes for b in prog.bucket) == 4 * (784 * 1024 + 1024 + 1024 * 1024 + 1024 + 1024 * 10 + 10 + 1)
