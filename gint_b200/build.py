"""Build libgint_b200.so (the CUDA kernels + C ABI) in-tree with nvcc for sm_100a.

    python -m gint_b200.build [--force] [--jobs N] [--no-jump-table] [-D MACRO=VALUE ...]

Pipeline, per interpreter kernel in ``gint_b200/csrc/kernels/*.cu``:

    nvcc -ptx                      CUDA C++  -> PTX (compute_100a)
    gint_b200.ptx_dispatch         the dispatch switch's compare tree -> one ``brx.idx`` jump table
    nvcc -cubin                    PTX -> sm_100a machine code (ptxas)
    .incbin                        the cubin becomes a byte array in an object file

then ``gint_capi.cu`` (host code) is compiled and everything is linked into ``gint_b200/libgint_b200.so`` with the CUDA
runtime linked statically. nvcc cross-compiles without a GPU, so this also runs on a CPU-only machine. A unit is rebuilt
when it or any header is newer than its output.
"""
from __future__ import annotations

import argparse
import concurrent.futures
import glob
import os
import shutil
import subprocess
import sys
import time

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
KERNELS = os.path.join(CSRC, "kernels")
OBJ_DIR = os.path.join(CSRC, "build")
LIB_PATH = os.path.join(PKG_DIR, "libgint_b200.so")
def _dispatch_count(family: str = "plain") -> int:
    """GINT_N_DISPATCH_PLAIN / _RF / _VEC of csrc/gint_opcodes.h: the 106 opcodes of the format + the internal ones + the fused
    handlers; the kernel families with opcodes of their own (registers in shared memory, vector layout) dispatch on more."""
    import re
    with open(os.path.join(CSRC, "gint_opcodes.h")) as f:
        return int(re.search(rf"#define GINT_N_DISPATCH_{family.upper()} (\d+)", f.read()).group(1))


N_OPS = _dispatch_count()
N_KEYS = 9 * N_OPS   # (GINT_MAX_STACK + 1) * GINT_N_DISPATCH

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-lineinfo", "-O3", "-std=c++17",
          "-fmad=false"]   # the bytecode's FMul/FAdd must stay separate roundings; FMA is its own opcode


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; cannot build libgint_b200.so")
    return exe


STEP_TIMEOUT_S = 900    # a compiler step that runs this long is stuck (ptxas on an unlucky control-flow graph): fail, do not hang


def _run(cmd: list[str], what: str) -> str:
    try:
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=STEP_TIMEOUT_S)
    except subprocess.TimeoutExpired:
        raise RuntimeError(f"{what} did not finish within {STEP_TIMEOUT_S} s:\n{' '.join(cmd)}")
    if r.returncode != 0:
        raise RuntimeError(f"{what} failed:\n{' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    return r.stderr + r.stdout


def _newest_header() -> float:
    hdrs = glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "hot_handlers.json")) + \
        glob.glob(os.path.join(PKG_DIR, "..", "include", "*.h")) + [os.path.join(PKG_DIR, "ptx_dispatch.py"), __file__]
    return max(os.path.getmtime(h) for h in hdrs)


def _build_kernel(src: str, extra: list[str], jump_table: bool, cluster: bool = True) -> tuple[str, str]:
    """CUDA C++ -> PTX -> (jump-table rewrite) -> cubin -> object with the cubin as a byte array."""
    from . import hot_handlers, ptx_dispatch
    stem = os.path.basename(src)[:-3]                       # gint_direct_p4_k1
    sym = stem.replace("gint_", "gint_cubin_").replace("_p", "_").replace("_k", "_")   # gint_cubin_direct_4_1
    ptx, cubin, obj = (os.path.join(OBJ_DIR, stem + ext) for ext in (".ptx", ".cubin", ".o"))
    t0 = time.time()
    _run([_nvcc(), "-arch=compute_100a", "-ptx"] + COMMON + extra + [src, "-o", ptx], f"nvcc -ptx {stem}")
    log = ""
    if jump_table:
        # the register-file kernels' hot handlers are long fused register-operand sequences: cluster them whatever their length
        family = "rf" if stem.startswith("gint_rf") else "vec" if stem.startswith("gint_vec") else "plain"
        n_ops = _dispatch_count(family)
        text, stats = ptx_dispatch.rewrite(open(ptx).read(), 9 * n_ops, n_ops, cluster=cluster, hot=hot_handlers.load(family),
                                           hot_any_size=family == "rf")
        with open(ptx, "w") as f:
            f.write(text)
        log += f"jump table: {stats['cases']} cases over {stats['keys']} keys, {stats['clustered']} small handlers clustered\n"
    t1 = time.time()
    # -fmad=false again: ptxas would otherwise contract the adjacent mul.rn.f32x2 / add.rn.f32x2 of a fused handler into an fma
    log += _run([_nvcc(), "-arch=sm_100a", "-cubin", "-lineinfo", "-fmad=false", "-Xptxas", "-v", ptx, "-o", cubin], f"ptxas {stem}")
    log += f"build time: nvcc -ptx {t1 - t0:.0f} s, ptxas {time.time() - t1:.0f} s\n"
    asm = os.path.join(OBJ_DIR, stem + ".S")
    with open(asm, "w") as f:
        f.write(f'.section .rodata\n.balign 64\n.global {sym}\n{sym}:\n.incbin "{cubin}"\n.global {sym}_end\n{sym}_end:\n.byte 0\n'
                '.section .note.GNU-stack,"",@progbits\n')
    _run(["gcc", "-c", asm, "-o", obj], f"as {stem}")
    return stem, log


def build(force: bool = False, jobs: int | None = None, verbose: bool = False, extra_flags: list[str] | None = None,
          jump_table: bool = True, cluster: bool = True) -> str:
    os.makedirs(OBJ_DIR, exist_ok=True)
    extra = list(extra_flags or [])
    stamp = os.path.join(OBJ_DIR, "flags.txt")
    flags_now = " ".join(extra) + f" jt={jump_table} cluster={cluster}"
    if not os.path.exists(stamp) or open(stamp).read() != flags_now:
        force = True
    hdr_time = _newest_header()
    kernels = sorted(glob.glob(os.path.join(KERNELS, "*.cu")))
    todo, objs = [], []
    for src in kernels:
        obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), hdr_time):
            todo.append(src)
    logs = []
    capi_src = os.path.join(CSRC, "gint_capi.cu")
    capi_obj = os.path.join(OBJ_DIR, "gint_capi.o")
    objs.append(capi_obj)
    capi_todo = force or not os.path.exists(capi_obj) or os.path.getmtime(capi_obj) < max(os.path.getmtime(capi_src), hdr_time)
    with concurrent.futures.ThreadPoolExecutor(max_workers=jobs or os.cpu_count() or 4) as ex:
        futs = [ex.submit(_build_kernel, s, extra, jump_table, cluster) for s in todo]
        if capi_todo:
            futs.append(ex.submit(lambda: ("gint_capi", _run([_nvcc()] + ARCH + COMMON + ["-Xcompiler", "-fPIC", "-c", capi_src, "-o", capi_obj],
                                                              "nvcc gint_capi"))))
        for f in concurrent.futures.as_completed(futs):
            logs.append(f.result())
    if todo or capi_todo or not os.path.exists(LIB_PATH):
        _run([_nvcc(), "-shared", "-o", LIB_PATH] + objs, "link")
    with open(stamp, "w") as f:
        f.write(flags_now)
    if verbose:
        for name, log in sorted(logs):
            for line in log.splitlines():
                if "registers" in line or "jump table" in line or "build time" in line or ("spill" in line and "0 bytes spill stores" not in line):
                    print(f"[{name}] {line.strip()}")
    return LIB_PATH


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--jobs", type=int, default=None)
    ap.add_argument("--no-jump-table", action="store_true", help="keep nvcc's compare-tree dispatch (for A/B measurements)")
    ap.add_argument("--no-cluster", action="store_true", help="leave the small handlers where the compiler put them (for A/B measurements)")
    ap.add_argument("-D", dest="defines", action="append", default=[])
    opts = ap.parse_args()
    path = build(force=opts.force, jobs=opts.jobs, verbose=True, extra_flags=[f"-D{d}" for d in opts.defines],
                 jump_table=not opts.no_jump_table, cluster=not opts.no_cluster)
    print(path)


if __name__ == "__main__":
    sys.exit(main())
