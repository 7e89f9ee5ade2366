"""Build libgint_b200.so (the CUDA kernels + C ABI) in-tree with nvcc for sm_100a.

    python -m gint_b200.build [--force] [--jobs N]

Every translation unit under ``gint_b200/csrc`` is compiled to an object file in ``gint_b200/csrc/build`` and
linked into ``gint_b200/libgint_b200.so``. nvcc cross-compiles without a GPU, so this also runs on a CPU-only
machine. A unit is rebuilt when it or any header is newer than its object.
"""
from __future__ import annotations

import argparse
import concurrent.futures
import glob
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
OBJ_DIR = os.path.join(CSRC, "build")
LIB_PATH = os.path.join(PKG_DIR, "libgint_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-fmad=false",            # the bytecode's FMul/FAdd must stay separate roundings; FMA is its own opcode
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; cannot build libgint_b200.so")
    return exe


def _newest_header() -> float:
    hdrs = glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh")) + \
        glob.glob(os.path.join(PKG_DIR, "..", "include", "*.h"))
    return max(os.path.getmtime(h) for h in hdrs)


def _compile(src: str, obj: str, extra: list[str]) -> str:
    cmd = [_nvcc()] + NVCC_FLAGS + extra + ["-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {os.path.basename(src)}:\n{r.stdout}\n{r.stderr}")
    return r.stderr


def build(force: bool = False, jobs: int | None = None, verbose: bool = False, extra_flags: list[str] | None = None) -> str:
    os.makedirs(OBJ_DIR, exist_ok=True)
    extra = list(extra_flags or [])
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    hdr_time = _newest_header()
    todo, objs = [], []
    for src in srcs:
        obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), hdr_time):
            todo.append((src, obj))
    logs = []
    if todo:
        with concurrent.futures.ThreadPoolExecutor(max_workers=jobs or os.cpu_count() or 4) as ex:
            futs = {ex.submit(_compile, s, o, extra): s for s, o in todo}
            for f in concurrent.futures.as_completed(futs):
                logs.append((os.path.basename(futs[f]), f.result()))
    if todo or not os.path.exists(LIB_PATH):
        cmd = [_nvcc(), "-shared", "-o", LIB_PATH] + objs
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    if verbose:
        for name, log in sorted(logs):
            for line in log.splitlines():
                if "registers" in line or "spill" in line and "0 bytes spill stores" not in line:
                    print(f"[{name}] {line.strip()}")
    return LIB_PATH


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--jobs", type=int, default=None)
    ap.add_argument("-D", dest="defines", action="append", default=[])
    opts = ap.parse_args()
    path = build(force=opts.force, jobs=opts.jobs, verbose=True, extra_flags=[f"-D{d}" for d in opts.defines])
    print(path)


if __name__ == "__main__":
    sys.exit(main())
