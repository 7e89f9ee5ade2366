"""The bytecode format contract: opcode numbers, stack effects and program analysis agree with the reference.

Golden data: gint_b200/data/opcodes.json is a dump of the reference's own INSNS / _EFFECTS / VARIANTS tables
(gint/kernel/interpreter/main.py:34-38,61-168; gint/host/analyzer.py:24-135), made by tests/golden/make_golden.py.
The analysis cases restate the reference's tests/test_analyzer.py:10-83.
"""
import json
import os

import numpy as np
import pytest

from gint_b200 import opcodes
from gint_b200.host.analyzer import analyze_bytecode, known_opcodes, select_pool_size, stack_effect
from gint_b200.host.executor import VARIANTS, ProgramData, c_analyze, select_variant
from gint_b200.host import frontend as fe
from gint_b200.programs import load_records
from oracle import oracle

GOLDEN = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "gint_b200", "data", "opcodes.json")


@pytest.fixture(scope="module")
def golden():
    with open(GOLDEN) as f:
        return json.load(f)


def test_opcode_numbers_match_reference(golden):
    assert opcodes.OPCODES == golden["opcodes"]
    assert opcodes.N_OPCODES == len(golden["opcodes"]) == 106


def test_stack_effects_match_reference(golden):
    ref = {int(k): tuple(v) for k, v in golden["stack_effects"].items()}
    assert opcodes.STACK_EFFECTS == ref
    assert known_opcodes() == frozenset(ref)
    assert stack_effect(opcodes.FMA) == (3, -2)


def test_constants_match_reference(golden):
    assert opcodes.REG_WIDTH == golden["reg_width"] == 4
    assert opcodes.MAX_N_TENSORS == golden["max_n_tensors"] == 8
    assert {k: tuple(v) for k, v in golden["variants"].items()} == VARIANTS


def test_c_header_table_matches_python():
    # gint_opcodes.h is what both the kernels and the C-ABI pre-decoder use
    path = os.path.join(os.path.dirname(os.path.dirname(__file__)), "gint_b200", "csrc", "gint_opcodes.h")
    import re
    rows = re.findall(r"X\((\w+), (\d+), (-?\d+), (-?\d+)\)", open(path).read())
    internal = [r for r in rows if int(r[1]) >= opcodes.N_OPCODES]   # the kernels' internal opcodes sit above the format's 106
    RF = ("RLoad", "RStore", "RLoadP", "RLoadS", "RemapVN")          # ... those of the register-file and vector-layout kernels after the fused handlers
    assert all(r[0].startswith(("Pf", "Bcast_")) or r[0].endswith("Fast") or r[0].endswith("Rows") or r[0] in RF for r in internal)
    # numbered consecutively after the format's
    plain = sorted(int(r[1]) for r in internal if r[0] not in RF)
    assert plain == list(range(opcodes.N_OPCODES, opcodes.N_OPCODES + len(plain)))
    assert {r[0]: int(r[1]) for r in internal if r[0] in RF} == {"RLoad": 150, "RStore": 151, "RLoadP": 152, "RLoadS": 153, "RemapVN": 180}
    rows = [r for r in rows if int(r[1]) < opcodes.N_OPCODES]
    assert len(rows) == opcodes.N_OPCODES
    for name, num, md, net in rows:
        assert opcodes.OPCODES[name] == int(num)
        assert opcodes.STACK_EFFECTS[int(num)] == (int(md), int(net))


def _bc(*pairs):
    return np.array(pairs, dtype=np.int32).reshape(-1)


def test_analyzer_simple_program():
    bc = _bc([fe.LoadImm, 0], [fe.LoadImm, 0], [fe.FAdd, 0], [fe.Dup, 0], [fe.FMul, 0], [fe.Pop, 0], [fe.Halt, 0])
    st = analyze_bytecode(bc)
    assert (st.num_instructions, st.max_stack, st.max_reg_idx, st.min_pool_size) == (6, 2, -1, 2)
    assert st.regs_used == frozenset()


def test_analyzer_registers_and_pool():
    bc = _bc([fe.LoadImm, 0], [fe.FStoreReg0 + 3, 0], [fe.LoadImm, 0], [fe.LoadImm, 0], [fe.FLoadReg0 + 3, 0], [fe.Halt, 0])
    st = analyze_bytecode(bc)
    assert st.max_reg_idx == 3 and st.regs_used == frozenset({3})
    assert st.max_stack == 3
    assert st.min_pool_size == 3 + 4


def test_analyzer_errors_like_reference():
    with pytest.raises(ValueError, match="unknown opcode"):
        analyze_bytecode(_bc([999, 0], [0, 0]))
    with pytest.raises(ValueError, match="needs depth 2"):
        analyze_bytecode(_bc([fe.LoadImm, 0], [fe.FAdd, 0], [0, 0]))


def test_select_variant_rules():
    # s7: stack <= 7 and registers 0..3; else l12 (gint/host/executor.py:131-149)
    small = _bc([fe.LoadImm, 0], [fe.FStoreReg0 + 3, 0], [0, 0])
    big_reg = _bc([fe.LoadImm, 0], [fe.FStoreReg0 + 4, 0], [0, 0])
    deep = _bc(*([[fe.LoadImm, 0]] * 8), [0, 0])
    assert select_variant(small) == "s7"
    assert select_variant(big_reg) == "l12"
    assert select_variant(deep) == "l12"
    assert select_variant(ProgramData(small, [])) == "s7"


def test_three_analyzers_agree_on_every_golden_program():
    """Python analyzer == C-ABI gint_analyze == oracle's analyze, on every recorded program."""
    for name, rec in load_records().items():
        bc = np.asarray(rec["bytecode"], dtype=np.int32)
        py = analyze_bytecode(bc)
        c = c_analyze(bc)
        o = oracle.analyze(bc)
        if name == "execute_everything":
            # The reference's own smoke program (tests/test_frontend.py:46-163) reaches depth 9 at its third dup2, one
            # more than any reference kernel holds (main.py:34-38); there the push is `unreachable` (main.py:245-248).
            # Both C implementations refuse it instead of running undefined behaviour.
            assert py.max_stack == 9
            assert c["status"] == -4 and c["error_index"] == 64
            assert o["status"] == -3
            continue
        assert c["status"] == 0 and o["status"] == 0, name
        for k_py, k_c in (("num_instructions", "num_instructions"), ("max_stack", "max_stack"), ("max_reg_idx", "max_reg_idx"),
                          ("min_pool_size", "min_pool_size")):
            assert getattr(py, k_py) == c[k_c] == o[k_c], (name, k_py)
        assert c["pool_size"] == o["pool_size"] == select_pool_size(py), name
        assert len(bc) // 2 == py.num_instructions + 1, name   # all recorded programs end with exactly one Halt


def test_pool_geometry_of_the_named_programs():
    recs = load_records()
    pool = lambda n: c_analyze(np.asarray(recs[n]["bytecode"], dtype=np.int32))["pool_size"]
    assert pool("add_n1048576") == 4
    assert pool("rmsnorm_r16384_n4096") == 4
    assert pool("bmm4x4_b4194304") == 7
    assert pool("inv4x4_b4194304") == 12
    assert pool("graph_fused_r65536_n1024") == 4
    # the reference would run these on s7, s7, s7, l12, s7
    variant = lambda n: select_variant(np.asarray(recs[n]["bytecode"], dtype=np.int32))
    assert [variant(n) for n in ("add_n1048576", "rmsnorm_r16384_n4096", "bmm4x4_b4194304", "inv4x4_b4194304",
                                 "graph_fused_r65536_n1024")] == ["s7", "s7", "s7", "l12", "s7"]


def test_every_opcode_is_executed_by_a_parity_case():
    """All 106 opcodes of the format appear in the programs that the GPU parity tests run against the oracle (the case list
    plus the random programs), so no handler goes untested."""
    import torch
    from cases import build_cases, to_interfaces
    from fuzz import FuzzProgram
    seen = set()
    for case in build_cases():
        host = case.make(torch.Generator().manual_seed(42))
        if case.view:
            host = case.view(host)
        pd = case.program.get_program(*to_interfaces(host), **case.kwargs)
        seen.update(int(op) for op in np.asarray(pd.program).reshape(-1, 2)[:, 0])
    for seed in range(24):     # the parameters of test_gpu_parity.py::test_random_programs_bit_exact
        depth, regs = [(3, 1), (4, 0), (6, 1), (7, 4), (8, 4), (4, 8), (5, 7), (2, 2)][seed % 8]
        for family in ("float", "int"):
            pd = FuzzProgram(seed, family, depth, regs, length=60 + 7 * seed, rows=33, cols=36).get_program()
            seen.update(int(op) for op in np.asarray(pd.program).reshape(-1, 2)[:, 0])
    missing = sorted(set(range(opcodes.N_OPCODES)) - seen)
    assert not missing, [opcodes.NAMES[m] for m in missing]


def test_hot_handler_table_is_current():
    """gint_b200/csrc/hot_handlers.json (the profile behind the kernels' code layout) equals a fresh derivation from the
    recorded programs with the library as built: it has to be regenerated when opcode numbers or the pre-decoder change."""
    import json
    from gint_b200 import hot_handlers
    with open(hot_handlers.TABLE) as f:
        committed = json.load(f)
    assert committed == hot_handlers.derive(), "run `python -m gint_b200.hot_handlers` and rebuild"
    assert len(hot_handlers.load()) == len(committed["keys"]) > 100
