"""The contraction templates against float64 matmul, through generated code and the C ABI.

Covers both templates (tcgen05 3xTF32 tiles and the CUDA-core tiles), operand transposes, batch,
ragged M / N / K tails, split-k, operand prologue, bias / relu / alpha / += epilogues. Tolerance:
1e-5 of the output's magnitude (the project bar is 1e-4; 3xTF32 and f32 FMA both sit near 1e-6)."""
import os

import numpy as np
import pytest

from anvil_lang_b200.program import DeviceProgram
from kirbuild import contraction_acc, contraction_program, contraction_reference

pytestmark = pytest.mark.gpu

CASES = [
    # M, N, K, batch, ta, tb, bias, relu_a, alpha, accumulate, relu_out
    (128, 128, 64, 1, False, False, False, False, 1.0, False, False),
    (256, 256, 256, 1, False, False, True, False, 1.0, False, True),
    (384, 192, 512, 1, False, True, False, True, 1.0, False, False),
    (200, 136, 100, 1, True, False, False, False, 0.125, False, False),      # ragged tails, K % 32 != 0
    (512, 512, 4096, 1, True, False, False, False, 1.0, True, False),        # split-k, += into C
    (256, 64, 256, 6, False, False, False, False, 0.125, False, False),      # batched, 64-wide tile
    (256, 256, 64, 4, False, True, False, False, 1.0, False, False),
    (130, 70, 36, 2, True, True, True, False, 1.0, False, False),
    (300, 300, 72, 2, True, False, True, False, 1.0, False, False),           # ragged in every direction, two tile columns
    (1024, 1024, 1024, 1, False, False, True, False, 1.0, False, False),
    (16384, 512, 2048, 1, False, False, True, False, 1.0, False, False),       # a transformer MLP product (A is 134 MB)
    (256, 64, 256, 512, False, False, False, False, 1.0, False, False),        # attention P·V over 512 (batch, head) pairs
    (256, 256, 64, 300, False, True, False, False, 0.125, False, False),       # Q·K^T shape: two k blocks per item, 4-5 items per cluster
]


# Shapes of the full-size transformer step (M = batch x T = 16384, D = 512) that the list above does not reach, with
# the epilogues they carry there. They run with the emitter's own choice and on the resident pairs.
#   M, N, K, batch, ta, tb, bias, relu_a, alpha, accumulate, relu_out, extra
BIG_CASES = [
    (512, 512, 16384, 1, True, False, False, False, 1.0, False, False, "adam_m"),     # dW of Wq/Wk/Wv/Wo: A read along m, split-k
    (2048, 512, 16384, 1, True, False, False, False, 1.0, False, False, "adam_m"),    # dW of the MLP's second matrix
    (512, 2048, 16384, 1, True, False, False, False, 1.0, False, False, "adam_m"),    # dW of the MLP's first matrix
    (16384, 512, 512, 1, False, True, False, False, 1.0, True, False, ""),             # dX through W^T, `+=` into dh
    (16384, 512, 512, 1, False, False, False, False, 1.0, False, False, "residual"),   # x = x + o @ Wo
    (16384, 256, 512, 1, False, False, True, False, 1.0, False, False, ""),            # logits
]


def run_case(case, tc):
    """tc: True (the emitter's choice), "pp" (resident CTA pairs walking over the tiles), "pair" (two CTAs of a cluster on one 256-row tile, cta_group::2; shapes too
    small for it take the emitter's choice), "ts" (A tiles in tensor memory), "ss" (operands in shared memory, two CTAs
    per SM), "ss32" (operands in shared memory, one CTA per SM, 32-wide k blocks), False (CUDA cores)."""
    M, N, K, batch, ta, tb, bias, relu_a, alpha, accumulate, relu_out = case[:11]
    extra = case[11] if len(case) > 11 else ""
    os.environ["ANVIL_B200_TC"] = {True: "1", False: "0"}.get(tc, tc)
    try:
        prog, kern, A, B, C, bias_b = contraction_program(*case)
        dp = DeviceProgram(prog, graphs=False)
    finally:
        os.environ.pop("ANVIL_B200_TC", None)
    note = dp.gen.kernel_notes[0]
    rng = np.random.default_rng(7)
    a = rng.standard_normal(A.numel, dtype=np.float32)
    b = rng.standard_normal(B.numel, dtype=np.float32)
    c0 = rng.standard_normal(C.numel, dtype=np.float32)
    bv = rng.standard_normal(N, dtype=np.float32)
    Mo = [x for x in prog.buffers if x.name == "Mo"][0]
    m0 = rng.standard_normal(Mo.numel, dtype=np.float32)
    dp.write(A, a); dp.write(B, b); dp.write(C, c0); dp.write(bias_b, bv); dp.write(Mo, m0)
    dp.launch(kern)
    dp.check_faults()
    got = dp.read(C).astype(np.float64)
    got_m = dp.read(Mo).astype(np.float64)
    dp.close()
    want = contraction_reference(a, b, c0, bv, M, N, K, batch, ta, tb, bias, relu_a, alpha, accumulate, relu_out, extra)
    err = np.abs(got - want).max() / max(np.abs(want).max(), 1e-30)
    if extra == "adam_m":                                  # the moment is linear in the product: same bar
        want_m = 0.9 * m0.astype(np.float64).reshape(batch, M, N) + 0.1 * contraction_acc(a, b, M, N, K, batch, ta, tb, relu_a, alpha)
        err = max(err, np.abs(got_m - want_m).max() / max(np.abs(want_m).max(), 1e-30))
    else:                                                  # no kernel touches Mo here: it has no memory and reads as zeros
        assert not got_m.any()
    return err, note


@pytest.mark.parametrize("variant", ["pp", "pair", "ts", "ss", "ss32"])
@pytest.mark.parametrize("case", CASES, ids=lambda c: "x".join(map(str, c[:4])))
def test_tensor_core_contraction(case, variant):
    err, note = run_case(case, tc=variant)
    # the tensor core's accumulator rounds toward zero at each of the K/8 accumulates: the error grows with K
    assert err < (1e-5 if case[2] <= 1024 else 3e-5), (err, note)


@pytest.mark.parametrize("case", CASES[:8], ids=lambda c: "x".join(map(str, c[:4])))
def test_cuda_core_contraction(case):
    err, note = run_case(case, tc=False)
    assert "simt" in note or "coop" in note or "thread" in note
    assert err < 1e-5, (err, note)


def test_large_shapes_take_the_tensor_core_template():
    _, note = run_case(CASES[9], tc=True)               # 1024^3
    assert note.startswith("gemm tc")
    _, note = run_case(CASES[1], tc=True)               # 33 MFLOP: below the tensor-core threshold
    assert note.startswith("gemm simt")


@pytest.mark.parametrize("variant", [True, "pp"])
@pytest.mark.parametrize("case", BIG_CASES, ids=lambda c: "x".join(map(str, c[:3])) + ("_" + c[11] if c[11] else ""))
def test_full_size_transformer_products(case, variant):
    err, note = run_case(case, tc=variant)
    assert note.startswith("gemm tc"), note
    assert err < 3e-5, (err, note)


def test_tma_operand_feed():
    """Plain row-major operands read along k arrive by TMA (cp.async.bulk.tensor, one 16-byte column of the tile per copy,
    no multicast) and serve as the hi operand as they are; the converters only make the lo tile. The tensor map must
    encode for the shape and the product must match float64. Both variants are timed on the same data and the times
    printed: the feed is opt-in (ANVIL_B200_TMA=1) because with three 66 KB stages only one copy is in flight and it
    measured slower (72 us against 49 us) than the converters' own register-prefetched loads."""
    import ctypes
    case = BIG_CASES[3]                                  # 16384 x 512 x 512, both operands read along k, += into C
    times = {}
    for tma in ("1", "0"):
        os.environ["ANVIL_B200_TMA"] = tma
        os.environ["ANVIL_B200_TC"] = "pp"
        try:
            prog, kern, A, B, C, bias_b = contraction_program(*case)
            dp = DeviceProgram(prog, graphs=False)
        finally:
            os.environ.pop("ANVIL_B200_TMA", None)
            os.environ.pop("ANVIL_B200_TC", None)
        assert ("_tma<<<" in dp.source) == (tma == "1")
        if tma == "1":
            buf = (ctypes.c_char * 192)()
            at = (ctypes.addressof(buf) + 63) // 64 * 64
            rc = dp.rtlib.anvil_rt_tensor_map(dp.rt, ctypes.c_void_p(at), dp.plan.off(A), 16384, 512, 512, 128)
            assert rc == 0, dp.rtlib.anvil_rt_last_error(dp.rt)
        rng = np.random.default_rng(3)
        a = rng.standard_normal(A.numel, dtype=np.float32)
        b = rng.standard_normal(B.numel, dtype=np.float32)
        c0 = rng.standard_normal(C.numel, dtype=np.float32)
        dp.write(A, a); dp.write(B, b); dp.write(C, c0)
        dp.launch(kern)
        dp.check_faults()
        got = dp.read(C).astype(np.float64)
        want = contraction_reference(a, b, c0, None, *case[:3], 1, False, True, False, False, 1.0, True, False)
        assert np.abs(got - want).max() / np.abs(want).max() < 1e-5
        times[tma] = min(dp.time_kernel(kern, 5) for _ in range(3))
        dp.close()
    print(f"16384x512x512 +=: TMA feed {times['1'] * 1e3:.1f} us, converter loads {times['0'] * 1e3:.1f} us")
    assert times["1"] <= 3 * times["0"]
