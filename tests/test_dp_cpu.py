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


def _dp_mlp():
    return kir.load(os.path.join(GOLDEN, "dp_mlp.b16.kir.json.gz"))


def test_a_summed_loss_is_refused():
    """The 1/G scaling of the summed gradients is only right for a MEAN loss: with the loss's 1/n factor removed
    (a batch sum) sharding must raise instead of training with gradients G times too small."""
    from anvil_lang_b200.backend.analysis import hot_loop
    prog = _dp_mlp()
    hot = hot_loop(prog)
    k = [s.kernel for s in hot.body.stmts if isinstance(s, kir.KernelStmt)
         and any(st.buf.name == "loss" for st in s.kernel.stores)][-1]
    consts = [n for n in k.red.body.walk() if n.k == "const"]
    assert consts
    for c in consts:
        c.val, c._key = -1.0, None
    with pytest.raises(dp.ShardError, match="not a mean"):
        dp.shard(prog, 2)


def test_a_gradient_that_reads_an_earlier_update_is_refused():
    """Updates move behind the all-reduce while the gradient half of a later update stays in front of it: if that
    gradient reads a parameter an earlier update wrote, it would see the stale value, so sharding must raise."""
    from anvil_lang_b200.backend.analysis import hot_loop
    from anvil_lang_b200.kir import F32, Affine, E
    prog = _dp_mlp()
    hot = hot_loop(prog)
    ks = [s.kernel for s in hot.body.stmts if isinstance(s, kir.KernelStmt)]
    upd = [k for k in ks if any(st.buf.root.kind == "param" for st in k.stores)]
    assert len(upd) >= 2 and upd[-1].red is not None
    earlier_param = [st.buf for st in upd[0].stores if st.buf.root.kind == "param"][0]
    last = upd[-1]
    last.red.body = E("bin", F32, op="mul", a=[last.red.body, E("load", F32, buf=earlier_param, off=Affine(0))])
    with pytest.raises(dp.ShardError, match="reads what the earlier update"):
        dp.shard(prog, 2)
