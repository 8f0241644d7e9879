"""Building and loading: nvcc for sm_100a, in-tree outputs, ctypes bindings.

The counterpart of `cuda.build` / `cli.build_cuda` in the reference (anvil/backend/cuda.py:644-663,
anvil/cli.py:127-136): there the generated file is compiled to an executable and run as a child
process; here it becomes a shared library next to libanvil_cuda.so and is driven in-process.
Nothing here falls back to a CPU path: a missing compiler or library raises `CudaToolchainError`.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
INCLUDE = os.path.join(ROOT, "include")
BUILD_DIR = os.environ.get("ANVIL_B200_BUILD") or os.path.join(PKG, "_build")
RT_LIB = os.path.join(BUILD_DIR, "libanvil_cuda.so")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


class CudaToolchainError(Exception):
    pass


def nvcc() -> str:
    exe = shutil.which("nvcc") or ("/usr/local/cuda/bin/nvcc" if os.path.exists("/usr/local/cuda/bin/nvcc") else None)
    if exe is None:
        raise CudaToolchainError("nvcc not found: the B200 back end needs the CUDA toolkit")
    return exe


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise CudaToolchainError(f"{os.path.basename(cmd[0])} failed:\n{r.stderr[-6000:]}")
    return r


def _stamp(paths) -> str:
    h = hashlib.sha256()
    for p in paths:
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:16]


def runtime_sources():
    return [os.path.join(CSRC, "anvil_rt.cu"), os.path.join(CSRC, "anvil_colsum_static.cu"), os.path.join(CSRC, "anvil_selftest.cu"),
            os.path.join(CSRC, "anvil_comm.cu"),
            os.path.join(CSRC, "anvil_gemm_sm100.cuh"), os.path.join(CSRC, "anvil_rng.h"),
            os.path.join(INCLUDE, "anvil_cuda.h")]


def build_runtime(force: bool = False) -> str:
    """libanvil_cuda.so from csrc/ (rebuilt when a source changed)."""
    os.makedirs(BUILD_DIR, exist_ok=True)
    srcs = [p for p in runtime_sources() if os.path.exists(p)]
    stamp = _stamp(srcs)
    stamp_file = RT_LIB + ".stamp"
    if not force and os.path.exists(RT_LIB) and os.path.exists(stamp_file) and open(stamp_file).read() == stamp:
        return RT_LIB
    cus = [p for p in srcs if p.endswith(".cu")]
    cmd = [nvcc(), "-shared", "-Xcompiler", "-fPIC", "-O3", "-std=c++17", "-lineinfo", *ARCH_FLAGS,
           "-I", INCLUDE, "-I", CSRC, "-o", RT_LIB, *cus, "-lz", "-lpthread", "-ldl"]
    _run(cmd)
    with open(stamp_file, "w") as f:
        f.write(stamp)
    return RT_LIB


def program_flags():
    # -fmad=false: f32 arithmetic is done operation by operation, like the NumPy interpreter that
    # defines the results; IEEE division and square root are nvcc's defaults without fast-math.
    return ["-O3", "-std=c++17", "-lineinfo", "-fmad=false", "-w", *ARCH_FLAGS, "-I", INCLUDE, "-I", CSRC]


def build_program(source: str, path: str | None = None) -> str:
    """Compile generated source to a shared library; cached by content hash under the build dir."""
    os.makedirs(BUILD_DIR, exist_ok=True)
    deps = _stamp([os.path.join(CSRC, "anvil_device.cuh"), os.path.join(CSRC, "anvil_rng.h"),
                   os.path.join(CSRC, "anvil_gemm_simt.cuh"), os.path.join(CSRC, "anvil_gemm_sm100.cuh"),
                   os.path.join(CSRC, "anvil_attn_sm100.cuh"), os.path.join(INCLUDE, "anvil_cuda.h")])
    key = hashlib.sha256((source + deps).encode()).hexdigest()[:16]
    lib = path or os.path.join(BUILD_DIR, f"prog-{key}.so")
    if os.path.exists(lib) and path is None:
        return lib
    cu = os.path.join(BUILD_DIR, f"prog-{key}.cu")
    with open(cu, "w") as f:
        f.write(source)
    tmp = lib + f".tmp{os.getpid()}"
    _run([nvcc(), "-shared", "-Xcompiler", "-fPIC", *program_flags(), "-o", tmp, cu])
    os.replace(tmp, lib)
    return lib


_rt_handle = None


def load_runtime() -> ctypes.CDLL:
    """libanvil_cuda.so with its symbols visible to program libraries loaded afterwards."""
    global _rt_handle
    if _rt_handle is not None:
        return _rt_handle
    if not os.path.exists(RT_LIB):
        build_runtime()
    lib = ctypes.CDLL(RT_LIB, mode=ctypes.RTLD_GLOBAL)
    c = ctypes
    P, Z, I, L, U = c.c_void_p, c.c_size_t, c.c_int, c.c_long, c.c_uint32
    sig = {
        "anvil_rt_create": (P, [I]), "anvil_rt_destroy": (None, [P]), "anvil_rt_arena": (I, [P, Z]),
        "anvil_rt_ptr": (P, [P, Z]), "anvil_rt_arena_bytes": (Z, [P]), "anvil_rt_stream": (P, [P]),
        "anvil_rt_use_stream": (I, [P, P]), "anvil_rt_fork": (I, [P]), "anvil_rt_back": (I, [P]), "anvil_rt_join": (I, [P]),
        "anvil_rt_side_stream": (I, [P, I]), "anvil_rt_last_error": (c.c_char_p, [P]),
        "anvil_rt_set_error": (I, [P, c.c_char_p]),
        "anvil_rt_load_idx": (I, [P, c.c_char_p, Z, L, L, I]), "anvil_rt_load_csv": (I, [P, c.c_char_p, Z, L, L]),
        "anvil_rt_load_bytes": (I, [P, c.c_char_p, Z, L]), "anvil_rt_input": (I, [P, Z, c.POINTER(I)]),
        "anvil_rt_d2d_async": (I, [P, Z, P, Z, P]),
        "anvil_rt_profile": (None, [P, I]), "anvil_rt_check": (None, [P, I]),
        "anvil_rt_profile_get": (I, [P, I, c.POINTER(c.c_double), c.POINTER(L)]),
        "anvil_rt_h2d": (I, [P, Z, P, Z]), "anvil_rt_d2h": (I, [P, P, Z, Z]),
        "anvil_rt_h2d_async": (I, [P, Z, P, Z]), "anvil_rt_d2h_async": (I, [P, P, Z, Z]),
        "anvil_rt_h2d_staged": (I, [P, Z, P, Z]), "anvil_rt_d2h_staged": (I, [P, P, Z, Z]),
        "anvil_rt_zero": (I, [P, Z, Z]), "anvil_rt_sync": (I, [P]),
        "anvil_rt_host_alloc": (P, [Z]), "anvil_rt_host_free": (None, [P]),
        "anvil_rt_set_i32": (I, [P, Z, c.c_int32]), "anvil_rt_set_f32": (I, [P, Z, c.c_float]),
        "anvil_rt_add_i32": (I, [P, Z, c.c_int32]),
        "anvil_rt_read_i32": (I, [P, Z, c.POINTER(c.c_int32)]), "anvil_rt_read_f32": (I, [P, Z, c.POINTER(c.c_float)]),
        "anvil_rt_seed": (None, [P, U]), "anvil_rt_get_seed": (U, [P]), "anvil_rt_get_stream": (U, [P]),
        "anvil_rt_set_stream": (None, [P, U]), "anvil_rt_next_stream_delta": (U, [P]),
        "anvil_rt_stream_commit": (I, [P]),
        "anvil_rt_rand_bits": (U, [U, U, U, U]), "anvil_rt_rand": (c.c_float, [U, U, U, U, I]),
        "anvil_rt_iota": (I, [P, Z, L]), "anvil_rt_shuffle": (I, [P, Z, L]),
        "anvil_rt_nonzero": (I, [P, Z, L, Z, L]), "anvil_rt_clock": (I, [P, Z]),
        "anvil_rt_capture": (I, [P, I]), "anvil_rt_captured": (c.c_char_p, [P]),
        "anvil_rt_print_text": (I, [P, c.c_char_p, I]), "anvil_rt_flush": (I, [P]),
        "anvil_rt_check_faults": (I, [P]),
        "anvil_rt_graphs": (None, [P, I]), "anvil_rt_launch_count": (L, [P]),
        "anvil_rt_timer_begin": (I, [P]), "anvil_rt_timer_end": (I, [P, c.POINTER(c.c_float)]),
        "anvil_rt_time_launch": (I, [P, P, I, I, c.POINTER(c.c_float)]),
        "anvil_rt_set_allreduce": (None, [P, P, P]), "anvil_rt_allreduce": (I, [P, Z, L]),
        "anvil_rt_comm_unique_id": (I, [P, Z]), "anvil_rt_comm_init": (I, [P, I, I, P, Z]),
        "anvil_rt_comm_nranks": (I, [P]), "anvil_rt_comm_destroy": (I, [P]),
        "anvil_colsum_f32_static": (I, [P, L, L, P, P]),
        "anvil_rt_selftest_wait": (I, [P, c.c_longlong, c.POINTER(U), c.POINTER(c.c_longlong)]),
        "anvil_rt_tensor_map": (I, [P, P, Z, L, L, L, I]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _rt_handle = lib
    return lib


def load_program(path: str) -> ctypes.CDLL:
    load_runtime()
    lib = ctypes.CDLL(path)
    c = ctypes
    lib.anvil_b200_kernel_count.restype = c.c_int
    lib.anvil_b200_arena_bytes.restype = c.c_ulong
    lib.anvil_b200_seed.restype = c.c_uint
    lib.anvil_b200_launch.restype = c.c_int
    lib.anvil_b200_launch.argtypes = [c.c_void_p, c.c_int]
    lib.anvil_b200_main.restype = c.c_int
    lib.anvil_b200_main.argtypes = [c.c_void_p, c.c_int]
    lib.anvil_b200_step.restype = c.c_int
    lib.anvil_b200_step.argtypes = [c.c_void_p]
    lib.anvil_b200_step_fed.restype = c.c_int
    lib.anvil_b200_step_fed.argtypes = [c.c_void_p]
    return lib
