"""`anvil export` for the B200 back end: a lowered Anvil function as a C library and header.

Mirrors anvil/export.py:68-161 (the reference builds `lib<name>.dylib` + `<name>.h` from its native back end):
everything the function reads from the rest of the program is already constant data in the lowered program
(`Buffer.init`), so it is written into the library as arrays and uploaded to the device arena on the first call;
the exported function has the reference's shape

    int <name>(const float *arg0, ..., float *result0, ...);      /* row-major arrays, 0 on success */

Calls from several threads take turns (one device arena per library), as in the reference. The library links
against `libanvil_cuda.so`, a copy of which is placed beside it (rpath `$ORIGIN`).

    from anvil_lang_b200 import export, pyapi
    lowered = pyapi.load_lowered("fn.kir.json.gz")           # or pyapi.lower(...) with the Anvil front end
    lib, header = export.export(lowered, "digits_read", "build/")
"""
from __future__ import annotations

import os
import re
import shutil

import numpy as np

from . import kir
from .backend import build as _build
from .backend import emit as _emit


def c_ident(s: str) -> str:
    s = re.sub(r"[^A-Za-z0-9_]", "_", s)
    return s if s and not s[0].isdigit() else "_" + s


def c_type(dtype) -> str:
    return "int32_t" if dtype == kir.I32 else "float"


def signature(lowered, name: str) -> tuple[str, list[str]]:
    """The C prototype and one comment per argument (shape, like the reference's header)."""
    args, notes = [], []
    for i, b in enumerate(lowered.inputs):
        args.append(f"const {c_type(b.dtype)} *arg{i}")
        notes.append(f"arg{i}: {c_type(b.dtype)}{list(b.shape)}")
    for i, b in enumerate(lowered.outputs):
        if b is None:
            raise ValueError("a result that is a compile-time constant cannot be exported: return it from C directly")
        args.append(f"{c_type(b.dtype)} *result{i}")
        notes.append(f"result{i}: {c_type(b.dtype)}{list(b.shape)}")
    return f"int {name}({', '.join(args)})", notes


def header_text(lowered, name: str) -> str:
    proto, notes = signature(lowered, name)
    guard = c_ident(name).upper() + "_H"
    lines = [f"/* {name}: an Anvil function compiled for NVIDIA B200 (sm_100a). Arrays are row-major.",
             " * Returns 0 on success; after a failure " + name + "_last_error() gives the message."]
    lines += [f" *   {n}" for n in notes]
    lines += [" */", f"#ifndef {guard}", f"#define {guard}", "#include <stdint.h>", "#ifdef __cplusplus", 'extern "C" {', "#endif",
              proto + ";", f"const char *{name}_last_error(void);", "#ifdef __cplusplus", "}", "#endif", "#endif", ""]
    return "\n".join(lines)


def wrapper_source(lowered, gen, name: str) -> str:
    """Constant data + the exported function, appended to the generated translation unit."""
    prog = lowered.prog
    out = ["", "// ---------------------------------------------------------------- exported function", "#include <mutex>"]
    uploads = []
    for r in prog.roots():
        if r.init is None or not len(r.init):
            continue
        words = np.ascontiguousarray(r.init, dtype=np.float32 if r.dtype == kir.F32 else np.int32).view(np.uint32).reshape(-1)
        rows = [", ".join(f"0x{w:08x}u" for w in words[i:i + 12]) for i in range(0, len(words), 12)]
        out.append(f"static const uint32_t export_init_{r.id}[] = {{   // {r.name}{list(r.shape)}\n    " + ",\n    ".join(rows) + "};")
        uploads.append(f"        if (anvil_rt_h2d(rt, {gen.plan.off(r)}UL, export_init_{r.id}, {4 * len(words)}UL)) return 1;")
    proto, _ = signature(lowered, name)
    out += ["static std::mutex export_lock;", "static anvil_rt *export_rt = 0;",
            f'extern "C" const char *{name}_last_error(void) {{ return export_rt ? anvil_rt_last_error(export_rt) : "anvil: no CUDA device context"; }}',
            f'extern "C" {proto} {{', "    std::lock_guard<std::mutex> guard(export_lock);",
            "    if (!export_rt) {                               // first call: context, zeroed arena, constants",
            "        anvil_rt *rt = anvil_rt_create(0);", "        if (!rt) return 1;",
            f"        if (anvil_rt_arena(rt, {gen.plan.size}UL)) {{ export_rt = rt; return 1; }}"]
    out += uploads
    out += ["        export_rt = rt;", "        anvil_b200_rt = rt;", "    }"]
    used = {r.id for r in prog.roots()}
    for i, b in enumerate(lowered.inputs):
        if b.root.id in used:
            out.append(f"    anvil_{b.name} = (void *)arg{i};")
    for i, b in enumerate(lowered.outputs):
        out.append(f"    anvil_{b.name} = (void *)result{i};")
    out.append("    const int rc = anvil_entry();")
    for b in list(lowered.inputs) + list(lowered.outputs):
        if b.root.id in used:
            out.append(f"    anvil_{b.name} = 0;")
    out += ["    return rc;", "}", ""]
    return "\n".join(out)


def export(lowered, name: str, outdir: str, seed: int = 0) -> tuple[str, str]:
    """Writes `<outdir>/lib<name>.so` (+ a copy of libanvil_cuda.so) and `<outdir>/<name>.h`."""
    name = c_ident(name)
    os.makedirs(outdir, exist_ok=True)
    src, gen = _emit.generate(lowered.prog, seed)
    src += wrapper_source(lowered, gen, name)
    rt = _build.build_runtime()
    shutil.copy2(rt, os.path.join(outdir, os.path.basename(rt)))
    cu = os.path.join(outdir, f"{name}.cu")
    with open(cu, "w") as f:
        f.write(src)
    lib = os.path.join(outdir, f"lib{name}.so")
    _build._run([_build.nvcc(), "-shared", "-Xcompiler", "-fPIC", *_build.program_flags(), "-o", lib, cu,
                 "-L", outdir, "-lanvil_cuda", "-Xlinker", "-rpath=$ORIGIN"])
    header = os.path.join(outdir, f"{name}.h")
    with open(header, "w") as f:
        f.write(header_text(lowered, name))
    return lib, header
