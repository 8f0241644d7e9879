"""A compiled program on one B200: arena, constants, and the entry points of its shared library.

This is the in-process replacement for what the reference does with a child process
(`subprocess.run([exe])`, anvil/cli.py:317-320): `DeviceProgram.run()` executes the program's host
control flow (generated C++) against libanvil_cuda.so and returns its exit status; stdout text is
either printed or captured. The same object gives tests and the benchmark kernel-level access
(`launch`), the training loop one iteration at a time (`prologue`, `step`), and typed reads/writes
of any tensor through explicit device copies.
"""
from __future__ import annotations

import ctypes

import numpy as np

from . import kir
from .backend import build, emit


class AnvilRuntimeError(Exception):
    pass


class DeviceProgram:
    def __init__(self, prog: kir.Program, seed: int = 0, device: int = 0, graphs: bool = True, lib_path: str | None = None):
        self.prog = prog
        self.seed = seed & 0xFFFFFFFF
        self.source, self.gen = emit.generate(prog, seed)
        self.plan = self.gen.plan
        self.lib_path = lib_path or build.build_program(self.source)
        self.rtlib = build.load_runtime()
        self.lib = build.load_program(self.lib_path)
        self.rt = self.rtlib.anvil_rt_create(device)
        if not self.rt:
            raise AnvilRuntimeError("anvil: could not create a runtime context")
        self._check(self.rtlib.anvil_rt_arena(self.rt, self.plan.size))
        self.rtlib.anvil_rt_graphs(self.rt, 1 if graphs else 0)
        self.reset()

    # ---- plumbing
    def _check(self, status: int):
        if status != 0:
            raise AnvilRuntimeError(self.rtlib.anvil_rt_last_error(self.rt).decode("utf-8", "replace") or f"status {status}")

    def close(self):
        if getattr(self, "rt", None):
            self.rtlib.anvil_rt_destroy(self.rt)
            self.rt = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def reset(self):
        """Zero every tensor, write the constants, restart the random stream (a fresh process in the
        reference: anvil/backend/cuda.py:415-421)."""
        self._check(self.rtlib.anvil_rt_zero(self.rt, 0, self.plan.size))
        self.rtlib.anvil_rt_seed(self.rt, self.seed)
        self.rtlib.anvil_rt_set_stream(self.rt, 0)
        for r in self.prog.roots():
            if r.init is not None and len(r.init):
                a = np.ascontiguousarray(r.init)
                self._check(self.rtlib.anvil_rt_h2d(self.rt, self.plan.off(r), a.ctypes.data, a.nbytes))
        # the device copy of the stream counter was zeroed with the arena
        self.rtlib.anvil_rt_arena_bytes(self.rt)
        self._check(self.rtlib.anvil_rt_sync(self.rt))

    def set_rank(self, rank: int):
        """The rank of this process in a data-parallel run (after every `reset`)."""
        if self.prog.rank_buf is not None:
            self._check(self.rtlib.anvil_rt_set_i32(self.rt, self.plan.off(self.prog.rank_buf), int(rank)))
            self._check(self.rtlib.anvil_rt_sync(self.rt))

    # ---- tensors
    def read(self, b: kir.Buffer) -> np.ndarray:
        out = np.empty(max(b.numel, 1), dtype=np.int32 if b.dtype == kir.I32 else np.float32)
        if b.root.id in self.plan.unused:            # a tensor no kernel touches has no memory: it reads as zeros
            out[:] = 0
            return out[:b.numel].reshape(b.shape)
        self._check(self.rtlib.anvil_rt_d2h(self.rt, out.ctypes.data, self.plan.off(b), out.nbytes))
        return out[:b.numel].reshape(b.shape)

    def write(self, b: kir.Buffer, value):
        a = np.ascontiguousarray(value, dtype=np.int32 if b.dtype == kir.I32 else np.float32).reshape(-1)
        if a.size != max(b.root.numel, 1) and a.size != b.numel:
            raise ValueError(f"{b.name}: expected {b.numel} elements, got {a.size}")
        if b.root.id in self.plan.unused:            # no kernel touches it: nothing to write to
            return
        self._check(self.rtlib.anvil_rt_h2d(self.rt, self.plan.off(b), a.ctypes.data, a.nbytes))

    def buffer(self, name: str) -> kir.Buffer:
        hits = [b for b in self.prog.buffers if b.name == name]
        if not hits:
            raise KeyError(name)
        return hits[-1]

    # ---- execution
    def run(self, capture: bool = False):
        """Runs the whole program. Returns (exit status, captured stdout or None). A run-time error
        (bounds fault, failed check) gives status 1 with the message in `self.error`; a failed
        `assert` gives the program's own exit value."""
        self.error = ""
        self.rtlib.anvil_rt_capture(self.rt, 1 if capture else 0)
        rc = self.lib.anvil_b200_main(self.rt, 0)
        text = self.rtlib.anvil_rt_captured(self.rt).decode("utf-8", "replace") if capture else None
        if rc >= 1000:
            return rc - 1000, text
        if rc != 0:
            self.error = self.rtlib.anvil_rt_last_error(self.rt).decode("utf-8", "replace")
            self.rtlib.anvil_rt_sync(self.rt)
            return 1, text
        return 0, text

    def prologue(self):
        """Runs the program up to the first iteration of its training loop."""
        rc = self.lib.anvil_b200_main(self.rt, 1)
        if rc != 2:
            self._check(rc if rc else 1)

    def step(self):
        self._check(self.lib.anvil_b200_step(self.rt))

    def step_fed(self):
        """One training iteration whose input tensors (`self.gen.feed_bufs`) the caller has already
        written, e.g. with `copy_in_async` from pinned host memory."""
        self._check(self.lib.anvil_b200_step_fed(self.rt))

    def copy_in_async(self, b: kir.Buffer, host_ptr: int, nbytes: int):
        self._check(self.rtlib.anvil_rt_h2d_async(self.rt, self.plan.off(b), host_ptr, nbytes))

    def copy_out_async(self, host_ptr: int, b: kir.Buffer, nbytes: int):
        self._check(self.rtlib.anvil_rt_d2h_async(self.rt, host_ptr, self.plan.off(b), nbytes))

    def launch(self, kernel: kir.Kernel | int):
        idx = kernel if isinstance(kernel, int) else self.gen.kernel_index[kernel.id]
        self._check(self.lib.anvil_b200_launch(self.rt, idx))

    def sync(self):
        self._check(self.rtlib.anvil_rt_sync(self.rt))

    def check_faults(self):
        self._check(self.rtlib.anvil_rt_check_faults(self.rt))

    def timer_begin(self):
        self._check(self.rtlib.anvil_rt_timer_begin(self.rt))

    def timer_end(self) -> float:
        """Milliseconds on the device since `timer_begin` (CUDA events on the program's stream)."""
        ms = ctypes.c_float()
        self._check(self.rtlib.anvil_rt_timer_end(self.rt, ctypes.byref(ms)))
        return float(ms.value)

    def time_kernel(self, kernel, repeats: int = 1) -> float:
        """Mean device milliseconds of one kernel's launcher (all its passes), timed alone."""
        idx = kernel if isinstance(kernel, int) else self.gen.kernel_index[kernel.id]
        ms = ctypes.c_float()
        fn = ctypes.cast(self.lib.anvil_b200_launch, ctypes.c_void_p)
        self._check(self.rtlib.anvil_rt_time_launch(self.rt, fn, idx, repeats, ctypes.byref(ms)))
        return float(ms.value)

    @property
    def launches(self) -> int:
        return int(self.rtlib.anvil_rt_launch_count(self.rt))

    @property
    def stream(self) -> int:
        return int(self.rtlib.anvil_rt_stream(self.rt) or 0)

    def ptr(self, b: kir.Buffer) -> int:
        return int(self.rtlib.anvil_rt_ptr(self.rt, self.plan.off(b)))
