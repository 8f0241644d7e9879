"""Hand-built KIR programs for kernel-level tests (no front end needed)."""
import itertools

import numpy as np

from anvil_lang_b200 import kir
from anvil_lang_b200.kir import F32, I32, Affine, Buffer, E, Kernel, KernelStmt, Let, Reduction, Store, Var

_ids = itertools.count(1000)


def nid():
    return next(_ids)


def buf(name, shape, dtype=F32, kind="temp"):
    return Buffer(nid(), name, tuple(shape), dtype, kind)


def var(name, n):
    return Var(nid(), name, n)


def load(b, terms, const=0):
    return E("load", b.dtype, buf=b, off=Affine(const, terms))


def const(v):
    return E("const", F32, val=float(v))


def binop(op, a, b):
    return E("bin", F32, op=op, a=[a, b])


def contraction_program(M, N, K, batch=1, ta=False, tb=False, bias=False, relu_a=False, alpha=1.0,
                        accumulate=False, relu_out=False, extra=""):
    """C[b, m, n] (=|+=) epi(alpha * sum_k A[b, m, k] * B[b, k, n]); ta/tb store the operand transposed.
    extra = "adam_m": a second store  Mo = 0.9 * Mo + 0.1 * acc  (a weight gradient with the first Adam moment fused);
    extra = "residual": the result is added to what C holds through a plain in-place statement  C = C + acc (+ bias)."""
    A = buf("A", (batch, K, M) if ta else (batch, M, K))
    B = buf("B", (batch, N, K) if tb else (batch, K, N))
    C = buf("C", (batch, M, N))
    Mo = buf("Mo", (batch, M, N))
    bias_b = buf("bias", (N,))
    b_, m, n, k = var("b", batch), var("m", M), var("n", N), var("k", K)
    a_ld = load(A, [(b_, M * K), (k, M), (m, 1)] if ta else [(b_, M * K), (m, K), (k, 1)])
    b_ld = load(B, [(b_, N * K), (n, K), (k, 1)] if tb else [(b_, N * K), (k, N), (n, 1)])
    if relu_a:
        a_ld = binop("max", a_ld, const(0.0))
    body = binop("mul", a_ld, b_ld)
    if alpha != 1.0:
        body = binop("mul", const(alpha), body)
    val = E("acc", F32)
    if bias:
        val = binop("add", val, load(bias_b, [(n, 1)]))
    if relu_out:
        val = binop("max", val, const(0.0))
    dom = ([b_] if batch > 1 else []) + [m, n]
    off = Affine(0, [(b_, M * N), (m, N), (n, 1)] if batch > 1 else [(m, N), (n, 1)])
    if extra == "residual":
        val = binop("add", E("load", F32, buf=C, off=off), val)
    stmts = [Store(C, off, val, accumulate)]
    if extra == "adam_m":
        stmts.append(Store(Mo, off, binop("add", binop("mul", const(0.9), E("load", F32, buf=Mo, off=off)),
                                          binop("mul", const(0.1), E("acc", F32)))))
    if batch == 1:                       # drop the batch var from operand offsets
        for e in body.walk():
            if e.k == "load":
                e.off = Affine(e.off.const, [(t, c) for t, c in e.off.terms if t is not b_])
                e._key = None
    kern = Kernel(nid(), f"k{nid()}", "test contraction", dom, stmts, Reduction([k], "sum", body))
    prog = kir.Program(kir.Block([KernelStmt(kern)]), [A, B, C, bias_b, Mo], "contraction test")
    return prog, kern, A, B, C, bias_b


def contraction_reference(a, b, c0, bias, M, N, K, batch, ta, tb, use_bias, relu_a, alpha, accumulate, relu_out, extra=""):
    """float64 result of `contraction_program`'s kernel for C (the value `acc` takes is `contraction_acc`)."""
    r = contraction_acc(a, b, M, N, K, batch, ta, tb, relu_a, alpha)
    if use_bias:
        r = r + bias.astype(np.float64)
    if relu_out:
        r = np.maximum(r, 0)
    if accumulate or extra == "residual":
        r = r + c0.astype(np.float64).reshape(batch, M, N)
    return r


def contraction_acc(a, b, M, N, K, batch, ta, tb, relu_a, alpha):
    a = a.astype(np.float64).reshape((batch, K, M) if ta else (batch, M, K))
    b = b.astype(np.float64).reshape((batch, N, K) if tb else (batch, K, N))
    if ta:
        a = a.transpose(0, 2, 1)
    if tb:
        b = b.transpose(0, 2, 1)
    if relu_a:
        a = np.maximum(a, 0)
    return alpha * np.matmul(a, b)
