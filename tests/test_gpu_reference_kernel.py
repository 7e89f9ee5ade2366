"""GPU parity against the reference's OWN device code: the same int32 streams and the same seeded inputs go through the
unmodified reference executor and its ``geval_s7`` / ``geval_l12`` kernels (built for sm_100 from the reference's generator by
``baseline/build_ref.py``) and through ``B200Executor``.

Integer and index programs must agree bit for bit. Float programs must agree within the benchmark's tolerances
(rtol 1e-5 / atol 1e-6; 1e-4 for the 4x4 inverse); programs made of add / sub / mul / div / fma / moves only are additionally
required to agree bit for bit, because both sides round every operation separately (the reference emits explicit
``fmul`` / ``fadd`` and ``llvm.fma`` only for FMA and FMAImm, arith.py:15-30). Where the two sides use different approximations
(the reference lowers FSqrt / FRSqrt / FExp / FLog through ``sqrt.approx`` / ``rsqrt.approx`` / ``ex2.approx`` / ``lg2.approx``; this
build calls the CUDA math library) the distance is bounded by the tolerance written in the case.

The whole module is skipped where ``baseline/_ref`` is absent.
"""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from baseline import ref_harness  # noqa: E402
from cases import build_cases, to_interfaces  # noqa: E402
from conftest import bits_equal, mismatch_report  # noqa: E402
from gint_b200 import get_executor  # noqa: E402
from gint_b200.workloads import FULL_SIZES, make_workload  # noqa: E402

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not ref_harness.available(), reason=ref_harness.why_unavailable() or "reference not installed")]

CASES = build_cases()

# Programs whose every operation is exactly rounded on both sides (or is an integer / index / move operation): bit-for-bit.
# The others contain FSqrt, FRSqrt, FExp, ... or narrow-type conversions of such results: tolerance.
APPROX = ("rmsnorm_bf16", "fused_idioms", "special_math", "alu_mix")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


@pytest.mark.parametrize("case", CASES, ids=lambda c: c.name)
def test_case_matches_reference_kernel(case):
    g = torch.Generator().manual_seed(42)
    host = case.make(g)
    ours = [t.cuda() for t in host]
    theirs = [t.cuda() for t in host]
    if case.view:
        host, ours, theirs = case.view(host), case.view(ours), case.view(theirs)
    pd = case.program.get_program(*to_interfaces(host), **case.kwargs)
    if pd.stats.max_stack > 8:
        pytest.skip("deeper than any reference kernel's stack: undefined there (main.py:245-248)")
    case.program(*ours, grid_dim=case.grid_dim, cuda_stream=_stream(), **case.kwargs)
    ref_prog = ref_harness.wrap_program_data(pd.program, pd.input_infos, pd.input_indices)
    ref_harness.execute(ref_prog, theirs, case.grid_dim, _stream())
    torch.cuda.synchronize()
    approx = (not case.exact) or case.name.startswith(APPROX)
    for i in case.outputs:
        if case.name.startswith("int_mix") and i == 3:
            # IDiv / IRem by zero: undefined in the reference (LLVM sdiv / srem, arith_int.py:42-51); this build defines them
            # (quotient -1, remainder = dividend). Compared where the divisor is not zero.
            keep = host[1].view(torch.int32) != 0
            assert keep.sum() > 0
            assert bits_equal(ours[i].cpu()[keep], theirs[i].cpu()[keep]), f"{case.name} output {i}: " + mismatch_report(ours[i].cpu()[keep], theirs[i].cpu()[keep])
            continue
        if approx:
            torch.testing.assert_close(ours[i].float().cpu(), theirs[i].float().cpu(), rtol=max(case.rtol, 2e-5), atol=max(case.atol, 2e-5))
        else:
            assert bits_equal(ours[i], theirs[i]), f"{case.name} output {i}: " + mismatch_report(ours[i], theirs[i])


NAMED = [("add", 4096, 1), ("add", 1000, 1), ("rmsnorm", 64, 4096), ("rmsnorm", 7, 256), ("rmsnorm", 5, 200), ("bmm4x4", 1000, 16),
         ("bmm4x4", 33, 16), ("inv4x4", 1000, 16), ("inv4x4", 33, 16), ("graph", 96, 1024), ("graph", 10, 256)] + \
        [(n, *FULL_SIZES[n]) for n in ("add", "rmsnorm", "bmm4x4", "inv4x4", "graph")]


@pytest.mark.parametrize("name,leading,inner", NAMED)
def test_named_program_matches_reference_kernel(name, leading, inner):
    """The five benchmark programs, small and at full size, on identical device buffers."""
    ours = make_workload(name, leading, inner, device="cuda")
    theirs = make_workload(name, leading, inner, device="cuda")
    ours.run(get_executor(), _stream())
    ref_harness.run_workload(theirs, _stream())
    torch.cuda.synchronize()
    for role in ours.outputs:
        a, b = ours.tensors[role], theirs.tensors[role]
        if name in ("add", "bmm4x4", "inv4x4"):      # add / mul / sub / div and moves: same roundings on both sides
            assert bits_equal(a, b), f"{name}.{role}: " + mismatch_report(a, b)
        else:                                         # rsqrt (and exp in the graph) are approximations that differ
            torch.testing.assert_close(a, b, rtol=ours.rtol, atol=ours.atol)


def test_reference_build_is_the_reference():
    """The kernels compared against come from the reference's generator: two entries, its register counts, no spills."""
    import json
    with open(os.path.join(ref_harness.REF_DIR, "BUILD_INFO.json")) as f:
        info = json.load(f)
    assert sorted(info["entries"]) == ["geval_l12", "geval_s7"]
    assert info["unresolved_libdevice"] == []
    assert info["registers"].get("geval_s7_spill_store_bytes", 0) == 0 and info["registers"].get("geval_l12_spill_store_bytes", 0) == 0
