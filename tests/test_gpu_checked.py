"""The bounds-checking kernel (``gint_execute_checked``): same results as the ordinary kernels for valid programs; an access
outside the tensor view that was passed is skipped and reported with its kind, tensor slot, logical program and instruction.

The out-of-range cases use descriptors that claim 256 elements for a tensor view of 128; the view sits inside a larger
allocation, so the refused addresses are ordinary device memory (the test checks that it stays untouched)."""
import numpy as np
import pytest
import torch

import cases as C
from conftest import bits_equal, mismatch_report
from gint_b200 import get_executor
from gint_b200.host.executor import BaseExecutableProgram, ProgramData, ProgramTensorInfo, _convert_arg

pytestmark = pytest.mark.gpu


class Claims256(BaseExecutableProgram):
    """c = a + b over two 128-element tiles, whatever the tensors' real extents are."""

    def get_program(self, a, b, c) -> ProgramData:
        bc = [15, 0, 15, 1, 2, 0, 16, 2, 0, 0]     # LoadGlobal1DF32 a; LoadGlobal1DF32 b; FAdd; StoreGlobal1DF32 c; Halt
        return ProgramData(np.array(bc, dtype=np.int32), [ProgramTensorInfo(4, [], [], [256, 1], [1, 0], [2, 1], [128, 0]) for _ in range(3)])

    def cache_policy(self, *args, **kw):
        return None


def test_valid_programs_run_clean_and_equal():
    ex = get_executor()
    ex.device_status()       # clear whatever an earlier test left
    for case in [c for c in C.build_cases() if c.name in ("vector_add_s12345", "basic_expr1_s1000_p18", "bmm4x4_B1000", "int_mix_n5000",
                                                          "dtype_tiles_2dw_t33_w6", "advance_walk", "indirect_arith")]:
        g = torch.Generator().manual_seed(3)
        host = case.make(g)
        plain = [t.cuda() for t in host]
        checked = [t.cuda() for t in host]
        if case.view:
            plain, checked = case.view(plain), case.view(checked)
        case.program(*plain, grid_dim=case.grid_dim, **case.kwargs)
        ex.execute_checked(case.program, [_convert_arg(t) for t in checked], case.grid_dim, **case.kwargs)
        st = ex.device_status()
        assert st["code"] == 0 and st["count"] == 0, (case.name, st)
        for i in case.outputs:
            assert bits_equal(checked[i], plain[i]), f"{case.name} output {i}: " + mismatch_report(checked[i], plain[i])


def test_store_outside_the_view_is_refused_and_reported():
    ex = get_executor()
    ex.device_status()
    a, b = torch.randn(256, device="cuda"), torch.randn(256, device="cuda")
    backing = torch.full((512,), 7.0, device="cuda")
    c = backing[:128]                                             # the program believes it has 256 elements
    ex.execute_checked(Claims256(), [_convert_arg(t) for t in (a, b, c)], 2)
    st = ex.device_status()
    assert st["what"] == "store out of range" and st["slot"] == 2 and st["logical_program"] == 1 and st["instruction"] == 3
    assert st["count"] == 128                                     # every element of the second tile
    assert backing.data_ptr() + 128 * 4 <= st["address"] < backing.data_ptr() + 256 * 4
    torch.testing.assert_close(c, a[:128] + b[:128])
    assert torch.equal(backing[128:], torch.full((384,), 7.0, device="cuda"))     # nothing beyond the view was written
    assert ex.device_status()["code"] == 0                        # reading cleared it


def test_load_outside_the_view_yields_zero_and_is_reported():
    ex = get_executor()
    ex.device_status()
    backing = torch.randn(512, device="cuda")
    a = backing[:128]
    b, c = torch.randn(256, device="cuda"), torch.zeros(256, device="cuda")
    ex.execute_checked(Claims256(), [_convert_arg(t) for t in (a, b, c)], 2)
    st = ex.device_status(clear=False)
    assert st["what"] == "load out of range" and st["slot"] == 0 and st["logical_program"] == 1 and st["instruction"] == 0 and st["count"] == 128
    assert ex.device_status()["count"] == 128                    # not cleared by the first read
    torch.testing.assert_close(c[:128], a + b[:128])
    assert torch.equal(c[128:], b[128:])                          # the refused loads contributed 0.0
