import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session", autouse=True)
def _built_libraries():
    """Both shared libraries are built in-tree before any test runs (nvcc cross-compiles without a GPU)."""
    from oracle import oracle
    oracle.build()
    from gint_b200 import build as b
    if not os.path.exists(b.LIB_PATH):
        b.build()


# ------------------------------------------------------------------------------------------------ helpers shared by tests

def infos_as_dicts(program):
    return [vars(t) for t in program.tensor_infos]


def oracle_run_workload(wl, threads: int = 4):
    """Run a workload (built on the CPU) through the oracle, in place; eager pre-steps included."""
    from oracle import oracle
    if wl.pre is not None:
        wl.pre(wl.tensors)
    for st in wl.steps:
        oracle.execute(st.program.bytecode, infos_as_dicts(st.program), [wl.tensors[r] for r in st.roles], st.grid_dim,
                       input_indices=st.program.input_indices, threads=threads)


def bits_equal(a: torch.Tensor, b: torch.Tensor) -> bool:
    """Bit-for-bit equality, except that any NaN matches any NaN (payloads differ between x86 and the GPU)."""
    a = a.detach().cpu().contiguous()
    b = b.detach().cpu().contiguous()
    if a.shape != b.shape or a.dtype != b.dtype:
        return False
    if a.dtype in (torch.float32, torch.float16, torch.bfloat16):
        an, bn = torch.isnan(a), torch.isnan(b)
        if not torch.equal(an, bn):
            return False
        view = {torch.float32: torch.int32, torch.float16: torch.int16, torch.bfloat16: torch.int16}[a.dtype]
        return torch.equal(a.view(view)[~an], b.view(view)[~bn])
    return torch.equal(a, b)


def mismatch_report(a: torch.Tensor, b: torch.Tensor, limit: int = 5) -> str:
    a = a.detach().cpu().reshape(-1)
    b = b.detach().cpu().reshape(-1)
    bad = (a != b) & ~(torch.isnan(a) & torch.isnan(b)) if a.is_floating_point() else (a != b)
    idx = torch.nonzero(bad).reshape(-1)[:limit].tolist()
    return f"{int(bad.sum())} mismatches of {a.numel()}; first: " + ", ".join(f"[{i}] {a[i].item()!r} vs {b[i].item()!r}" for i in idx)
