"""Batched candidate execution (``gint_execute_batch`` / ``gint_b200.feeder.BatchRunner``): every candidate of a batch gives the
bits that the same program gives when it is launched by itself; invalid candidates are skipped and reported."""
import numpy as np
import pytest
import torch

from conftest import bits_equal, mismatch_report
from gint_b200 import get_executor, opcodes as O
from gint_b200.feeder import BatchRunner, contiguous_f32_info
from gint_b200.host.executor import BaseExecutableProgram, ProgramData, _convert_arg
from gint_b200.host.frontend import _bytes4, _f32_bits

pytestmark = pytest.mark.gpu
N_IN, SIZE = 2, 128


def candidate(rng, body_len: int) -> list:
    """load a; load b; <body_len stack-valid float instructions>; fold; store; halt -- padded with Nops to a fixed length."""
    bc, depth = [[O.LoadGlobal1DF32, 0], [O.LoadGlobal1DF32, 1]], 2
    binary = [O.FAdd, O.FMul, O.FSub, O.FRSub, O.FGt, O.FLt]
    for _ in range(body_len):
        kinds = ["imm", "dup"] if depth < 6 else []
        kinds += ["unary", "perm", "immop"] if depth >= 1 else []
        kinds += ["binary", "binary", "swap"] if depth >= 2 else []
        k = kinds[rng.integers(len(kinds))]
        if k == "imm":
            bc.append([O.LoadImm, _f32_bits(float(rng.normal()))]); depth += 1
        elif k == "dup":
            bc.append([O.Dup, 0]); depth += 1
        elif k == "unary":
            bc.append([O.FNeg, 0])
        elif k == "perm":
            bc.append([O.FPermW, _bytes4(*rng.integers(0, 4, 4).tolist())])
        elif k == "immop":
            bc.append([O.FMulImm, _f32_bits(float(rng.normal()))])
        elif k == "binary":
            bc.append([int(binary[rng.integers(len(binary))]), 0]); depth -= 1
        else:
            bc.append([O.Swap, 0])
    while depth > 1:
        bc.append([O.FAdd, 0]); depth -= 1
    bc.append([O.StoreGlobal1DF32, 2])
    return bc


class Raw(BaseExecutableProgram):
    def __init__(self, bc):
        super().__init__()
        self._pd = ProgramData(np.asarray(bc, dtype=np.int32).reshape(-1), [contiguous_f32_info(SIZE)] * (N_IN + 1))

    def get_program(self, *a, **k):
        return self._pd

    def cache_policy(self, *a, **k):
        return None


def test_batch_matches_single_launches_and_skips_invalid_candidates():
    rng = np.random.default_rng(5)
    words = 2 * 40
    progs = []
    for i in range(300):
        bc = candidate(rng, int(rng.integers(0, 24)))
        bc += [[O.Nop, 0]] * (words // 2 - 1 - len(bc)) + [[O.Halt, 0]]
        progs.append(bc)
    bad_underflow, bad_opcode, bad_no_halt = 17, 101, 250
    progs[bad_underflow] = [[O.FAdd, 0]] + [[O.Nop, 0]] * (words // 2 - 2) + [[O.Halt, 0]]
    progs[bad_opcode] = [[999, 0]] + [[O.Nop, 0]] * (words // 2 - 2) + [[O.Halt, 0]]
    progs[bad_no_halt] = [[O.Nop, 0]] * (words // 2)
    codes = np.asarray(progs, dtype=np.int32).reshape(len(progs), words)
    g = torch.Generator().manual_seed(1)
    a, b = torch.randn(SIZE, generator=g).cuda(), torch.randn(SIZE, generator=g).cuda()
    out = torch.full((len(progs), SIZE), 42.0, device="cuda")
    runner = BatchRunner(N_IN, SIZE)
    for call in range(2):                                   # the second call reuses the context's scratch
        got = runner.run(codes, [a, b], out)
        torch.cuda.synchronize()
        assert got.shape == (len(progs), SIZE)
        st = runner.last_status
        assert st[bad_underflow] == -3 and st[bad_opcode] == -2 and st[bad_no_halt] == -5
        assert (np.delete(st, [bad_underflow, bad_opcode, bad_no_halt]) == 0).all()
    ex = get_executor()
    single = torch.zeros(SIZE, device="cuda")
    for i in list(range(0, 300, 7)) + [299]:
        if i in (bad_underflow, bad_opcode, bad_no_halt):
            continue
        ex.execute(Raw(progs[i]), [_convert_arg(t) for t in (a, b, single)], 1)
        torch.cuda.synchronize()
        assert bits_equal(out[i], single), f"candidate {i}: " + mismatch_report(out[i], single)
    for i in (bad_underflow, bad_opcode, bad_no_halt):      # skipped: rows untouched
        assert torch.equal(out[i], torch.full((SIZE,), 42.0, device="cuda"))


def test_batch_argument_checks():
    runner = BatchRunner(N_IN, SIZE)
    a = torch.zeros(SIZE, device="cuda")
    out = torch.zeros(4, SIZE, device="cuda")
    assert runner.run(np.zeros((0, 10), dtype=np.int32), [a, a], out).shape[0] == 0
    with pytest.raises(ValueError):
        runner.run(np.zeros((2, 10), dtype=np.int32), [a], out)
    with pytest.raises(ValueError):
        runner.run(np.zeros((8, 10), dtype=np.int32), [a, a], out)
