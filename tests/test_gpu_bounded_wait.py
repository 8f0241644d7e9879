"""The failure path of the contraction templates' waits, made to happen on purpose and harmlessly: a kernel waits
with a limit of about a millisecond on a barrier nothing arrives on (the same `mbar_wait` the tcgen05 templates
use), gives up, records the time-out in the arena's status word and returns. The host must see the status, the
next fault check must report it, and the context must keep working afterwards."""
import ctypes

import numpy as np
import pytest

from anvil_lang_b200.program import AnvilRuntimeError, DeviceProgram
from test_zz_no_alloc import colsum_program

pytestmark = pytest.mark.gpu

STATUS_OFF, TIMEOUT = 32, 0x7C05


def test_a_wait_that_runs_out_reports_and_returns():
    prog, k, x, out, _ = colsum_program(512, 64)
    dp = DeviceProgram(prog, graphs=False)
    try:
        status, waited = ctypes.c_uint32(0), ctypes.c_longlong(0)
        limit = 2_000_000                                       # about 1 ms of SM clocks
        dp._check(dp.rtlib.anvil_rt_selftest_wait(dp.rt, limit, ctypes.byref(status), ctypes.byref(waited)))
        assert status.value == TIMEOUT
        assert limit <= waited.value < 50 * limit               # it gave up right after the limit
        with pytest.raises(AnvilRuntimeError, match="gave up waiting on a barrier"):
            dp.check_faults()
        dp._check(dp.rtlib.anvil_rt_zero(dp.rt, STATUS_OFF, 4))
        dp.check_faults()                                       # cleared
        data = np.random.default_rng(1).standard_normal((512, 64), dtype=np.float32)
        dp.write(x, data)                                       # the context still runs kernels
        dp.launch(k)
        got = dp.read(out)
        assert np.abs(got - data.astype(np.float64).sum(0)).max() <= 1e-4 * np.abs(got).max()
    finally:
        dp.close()
