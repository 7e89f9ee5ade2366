#!/usr/bin/env python
"""Install the unmodified reference (eliphatfs/gint) into ``baseline/_ref`` and build ITS interpreter kernels for sm_100.

    python baseline/build_ref.py [--reference /path/to/gint/checkout] [--force]

What it makes (all under ``baseline/_ref/``, which is kept out of version control):

    gint/                                the reference package, byte for byte
    gint/host/cuda/gint.fatbin.xz        geval_s7 / geval_l12 assembled for sm_100 (what gint/host/cuda/executor_impl.py:18-19 opens)
    tests/                               the reference's own unittest modules (run unmodified by tests/test_gpu_reference_suite.py)
    BUILD_INFO.json                      how it was installed, compiler versions, registers per kernel

The reference's build (generate.sh:1-18, gint/scripts/gen_llir.py:53-78) is llvmlite IR -> ``llvm-link`` libdevice -> ``clang -O3``
-> PTX -> ``nvcc -fatbin``. ``llvm-link`` and ``clang`` are not needed: llvmlite carries the same LLVM with the NVPTX target, so
the same steps run in-process (parse the emitted IR, link the reference's own ``nvptx.libdevice.10.bc``, new-pass-manager O3,
emit PTX) and ``ptxas`` assembles the PTX. Nothing of this repository's interpreter is involved: these are the kernels this
repository's kernels are measured against.

The package is installed with pip first (``pip install --no-index --no-build-isolation --no-deps --target``); that needs the
reference's build backend (hatchling). Where it is absent the package tree is copied as it is -- the project is pure Python plus
the one data file built here, so the result is the same tree a wheel would unpack.
"""
from __future__ import annotations

import argparse
import json
import lzma
import os
import re
import shutil
import subprocess
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
DEFAULT_REFERENCE = "/root/reference"


def _log(msg: str) -> None:
    print(f"[build_ref] {msg}", file=sys.stderr, flush=True)


def install_package(reference: str) -> str:
    """Returns how the package got there ("pip" or "tree copy (<why>)")."""
    if os.path.isdir(os.path.join(REF_DIR, "gint")):
        shutil.rmtree(os.path.join(REF_DIR, "gint"))
    os.makedirs(REF_DIR, exist_ok=True)
    how = None
    with tempfile.TemporaryDirectory() as tmp:
        src = os.path.join(tmp, "reference")     # the checkout may be read-only and a build writes into its tree
        shutil.copytree(reference, src, ignore=shutil.ignore_patterns(".git", "__pycache__"))
        cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps", "--find-links", "/opt/wheelhouse",
               "--target", REF_DIR, src]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode == 0 and os.path.isdir(os.path.join(REF_DIR, "gint")):
            how = "pip"
        else:
            tail = (r.stderr or r.stdout).strip().splitlines()[-1:] or ["pip failed"]
            how = f"tree copy (pip install failed: {tail[0][:160]})"
    if how != "pip":
        shutil.copytree(os.path.join(reference, "gint"), os.path.join(REF_DIR, "gint"), ignore=shutil.ignore_patterns("__pycache__"))
    tests_dst = os.path.join(REF_DIR, "tests")
    if os.path.isdir(tests_dst):
        shutil.rmtree(tests_dst)
    shutil.copytree(os.path.join(reference, "tests"), tests_dst, ignore=shutil.ignore_patterns("__pycache__"))
    return how


def build_ptx() -> tuple[str, dict]:
    """The reference's two kernels as PTX text, by its own generator and its own libdevice bitcode."""
    sys.path.insert(0, REF_DIR)
    import llvmlite.binding as llvm
    from gint.kernel.interpreter.main import build_interpreter_main_nvptx   # the reference's generator (main.py:277-294)
    import gint.kernel.platforms as platforms

    t0 = time.time()
    ir_text = build_interpreter_main_nvptx().emit()
    if isinstance(ir_text, bytes):
        ir_text = ir_text.decode()
    t_emit = time.time() - t0
    for init in ("initialize_all_targets", "initialize_all_asmprinters"):
        getattr(llvm, init)()
    target = llvm.Target.from_triple("nvptx64-nvidia-cuda")
    # PTX 8.0 / sm_90 is the newest pair this LLVM offers that CUDA 12.9's ptxas takes for every later architecture; the
    # kernels use nothing newer than sm_70 features (generate.sh:4 builds them with --cc 70)
    tm = target.create_target_machine(cpu="sm_90", features="+ptx80", opt=3)
    mod = llvm.parse_assembly(ir_text)
    libdevice = os.path.join(os.path.dirname(os.path.abspath(platforms.__file__)), "nvptx.libdevice.10.bc")
    with open(libdevice, "rb") as f:
        lib = llvm.parse_bitcode(f.read())
    lib.triple = mod.triple
    lib.data_layout = mod.data_layout
    mod.link_in(lib, preserve=False)
    mod.verify()
    t1 = time.time()
    pto = llvm.create_pipeline_tuning_options(speed_level=3, size_level=0)
    pb = llvm.create_pass_builder(tm, pto)
    pm = pb.getModulePassManager()
    pm.run(mod, pb)
    t_opt = time.time() - t1
    ptx = tm.emit_assembly(mod)
    # only-needed: drop what llvm-link --only-needed would not have pulled in (unreferenced libdevice functions are internalised
    # away by O3 when they are not kernels; what is left is the two entries and their callees)
    entries = re.findall(r"\.entry\s+(\w+)", ptx)
    unresolved = sorted(set(re.findall(r"\.extern\s+\.func[^;]*?(__nv_\w+)", ptx)))
    info = {"llvm": ".".join(map(str, llvm.llvm_version_info)), "emit_s": round(t_emit, 1), "opt_s": round(t_opt, 1), "entries": entries,
            "unresolved_libdevice": unresolved, "ptx_bytes": len(ptx)}
    return ptx, info


def assemble(ptx: str) -> tuple[bytes, dict]:
    with tempfile.TemporaryDirectory() as tmp:
        p = os.path.join(tmp, "gint.ptx")
        c = os.path.join(tmp, "gint.cubin")
        with open(p, "w") as f:
            f.write(ptx)
        ptxas = shutil.which("ptxas") or "/usr/local/cuda/bin/ptxas"
        t0 = time.time()
        r = subprocess.run([ptxas, "-arch=sm_100", "-lineinfo", "-v", p, "-o", c], capture_output=True, text=True)   # generate.sh:12
        if r.returncode != 0:
            raise RuntimeError("ptxas failed:\n" + r.stderr[-4000:])
        regs = {}
        cur = None
        for line in r.stderr.splitlines():
            m = re.search(r"Compiling entry function '(\w+)'", line)
            if m:
                cur = m.group(1)
            m = re.search(r"Used (\d+) registers", line)
            if m and cur:
                regs[cur] = int(m.group(1))
            m = re.search(r"(\d+) bytes spill stores", line)
            if m and cur:
                regs[cur + "_spill_store_bytes"] = int(m.group(1))
        with open(c, "rb") as f:
            cubin = f.read()
        ver = subprocess.run([ptxas, "--version"], capture_output=True, text=True).stdout.strip().splitlines()[-1]
        return cubin, {"ptxas": ver, "ptxas_s": round(time.time() - t0, 1), "registers": regs, "cubin_bytes": len(cubin)}


def build(reference: str = DEFAULT_REFERENCE, force: bool = False) -> str | None:
    """Returns the path of the installed tree, or None when no reference checkout is there to install from."""
    fatbin = os.path.join(REF_DIR, "gint", "host", "cuda", "gint.fatbin.xz")
    if os.path.exists(fatbin) and os.path.exists(os.path.join(REF_DIR, "BUILD_INFO.json")) and not force:
        return REF_DIR
    if not os.path.isdir(os.path.join(reference, "gint")):
        return None
    info = {"reference": reference, "when": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime())}
    info["install"] = install_package(reference)
    _log(f"package: {info['install']}")
    ptx, i = build_ptx()
    info.update(i)
    _log(f"PTX: {i['ptx_bytes']} bytes, entries {i['entries']}, emit {i['emit_s']} s, O3 {i['opt_s']} s")
    if i["unresolved_libdevice"]:
        raise RuntimeError(f"libdevice symbols left unresolved: {i['unresolved_libdevice']}")
    cubin, i = assemble(ptx)
    info.update(i)
    _log(f"cubin: {i['cubin_bytes']} bytes, registers {i['registers']}")
    with lzma.open(fatbin, "wb", preset=6) as f:     # cuModuleLoadData takes a cubin as well as a fatbin (driver.py:162-169)
        f.write(cubin)
    with open(os.path.join(REF_DIR, "BUILD_INFO.json"), "w") as f:
        json.dump(info, f, indent=1)
    return REF_DIR


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=DEFAULT_REFERENCE)
    ap.add_argument("--force", action="store_true")
    o = ap.parse_args()
    out = build(o.reference, o.force)
    print(out if out else "no reference checkout: nothing built")


if __name__ == "__main__":
    main()
