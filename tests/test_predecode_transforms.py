"""The host pre-decoder's program transformations (early-issued loads, fused handlers) are checked on the CPU by undoing
them: expanding every fused handler into its members and replaying the ring of early-issued loads must give back the
original instruction list (with an immediately repeated load folded into Dup), for every recorded program and for random
programs."""
import ctypes

import numpy as np
import pytest

from fuzz import FuzzProgram
from gint_b200 import opcodes as O
from gint_b200.host import capi
from gint_b200.host.utils import fill_tensor_info
from gint_b200.programs import load_records, recorded

PF_TAKE, PF_ISSUE_1D, PF_TAKE_ISSUE_1D, PF_SKIP, LOAD_1D_FAST, STORE_1D_FAST, PF_ISSUE_1D_FAST, PF_TAKE_ISSUE_1D_FAST, STAGE_ROWS, LOAD_STAGED_ROWS = range(106, 116)
BCAST, LOAD_2DW_FAST, STORE_2DW_FAST = 116, 120, 121   # Bcast_0..3
RLOAD, RSTORE, RLOADP, RLOADS = 150, 151, 152, 153     # virtual registers in shared memory: operand = 512 * register number (+ selectors)
REMAP_VN = 180                                         # vector layout -> natural layout (vector-layout kernels)


def fused_table():
    lib = capi.load_library()
    buf = (ctypes.c_int32 * (64 * 10))()
    n = lib.gint_debug_fused_table(buf, 64)
    assert n > 0
    return {buf[10 * k]: [buf[10 * k + 2 + j] for j in range(buf[10 * k + 1])] for k in range(n)}


def transform(bytecode, infos, early, fuse):
    lib = capi.load_library()
    code = np.ascontiguousarray(np.asarray(bytecode, dtype=np.int32).reshape(-1))
    ti = capi.HTensorInfo()
    fill_tensor_info(ti, infos)
    n_max = code.size // 2 + 16
    ops = (ctypes.c_int32 * n_max)()
    operands = (ctypes.c_uint32 * n_max)()
    n = lib.gint_debug_transform(code.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)), code.size, ctypes.byref(ti), len(infos),
                                 int(early), int(fuse), ops, operands, n_max)
    assert n > 0, n
    return list(zip(ops[:n], operands[:n]))


def normalised(bytecode):
    """What the kernels run with both passes off, plus the Dup fold the early-issue pass applies."""
    out = []
    for op, operand in np.asarray(bytecode, dtype=np.int64).reshape(-1, 2):
        op, operand = int(op), int(operand) & 0xFFFFFFFF
        if op == O.DupBroadcastW:
            s = operand - (1 << 32) if operand >= 1 << 31 else operand
            operand = min(max(s, 0), 3)
        elif op in (O.FPermW, O.FShuf2):
            operand = sum(min((operand >> (8 * w)) & 0xFF, 3) << (8 * w) for w in range(4))
        out.append((op, operand))
        if op == O.Halt:
            break
    return out


def fold_repeated_loads(prog):
    loads = {O.LoadGlobal1DF32, O.LoadGlobal1DF16, O.LoadGlobal1DBF16, O.LoadGlobal1DU8, O.LoadGlobal2DTF32, O.LoadGlobal2DTF16,
             O.LoadGlobal2DTBF16, O.LoadGlobal2DTU8, O.LoadGlobal2DWF32, O.LoadGlobal2DWF16, O.LoadGlobal2DWBF16, O.LoadGlobal2DWU8}
    out = []
    for op, operand in prog:
        if out and op in loads and out[-1] == (op, operand):    # compares with the already folded predecessor
            out.append((O.Dup, 0))
        else:
            out.append((op, operand))
    return out


def undo(prog, table):
    # 1. fused handlers -> members (operands come from the absorbed instructions that follow)
    flat = []
    i = 0
    while i < len(prog):
        op, operand = prog[i]
        if op in table:
            members = table[op]
            for j, m in enumerate(members):
                assert j == 0 or prog[i + j][0] == -1
                flat.append((m, prog[i + j][1]))
            i += len(members)
        else:
            assert op != -1
            flat.append((op, operand))
            i += 1
    flat = [(op, operand) for op, operand in flat if op != REMAP_VN]     # changes where values sit, not what they are
    # 1b. DupBroadcastW with a built-in lane index -> the format's instruction with an operand
    flat = [(O.DupBroadcastW, op - BCAST) if BCAST <= op < BCAST + 4 else (op, operand) for op, operand in flat]
    # 1c. registers in shared memory -> the format's per-register opcodes; permutations and shuffles folded into a register load
    # come apart again (selectors: 2 bits each in the operand -> one byte each)
    def sel_bytes(bits):
        return sum(((bits >> (2 * w)) & 3) << (8 * w) for w in range(4))

    def shuffle(operand):
        return [(O.FLoadReg0 + (operand & 0xFFF) // 512, 0), (O.FLoadReg0 + ((operand >> 12) & 0xFFF) // 512, 0)], (O.FShuf2, sel_bytes(operand >> 24))

    back, i = [], 0
    while i < len(flat):
        op, operand = flat[i]
        nxt = [f[0] for f in flat[i + 1:i + 4]]
        same_pair = i + 1 < len(flat) and flat[i + 1][0] == RLOADS and (flat[i + 1][1] ^ operand) & 0xFFFFFF == 0
        if op == RLOADS and same_pair and nxt[1:3] == [RSTORE, RSTORE]:
            # two shuffles of one register pair, then two register stores: the Dup2 form (stores in the original order)
            loads, s1 = shuffle(operand)
            _, s2 = shuffle(flat[i + 1][1])
            back += loads + [(O.Dup2, 0), s1, flat[i + 3], s2, flat[i + 2]]
            i += 4
        elif op == RLOADS and len(nxt) == 3 and nxt[1] == RLOADS and nxt[0] == nxt[2] and nxt[0] in (O.StoreGlobal2DWF32, STORE_2DW_FAST) and \
                (flat[i + 2][1] ^ operand) & 0xFFFFFF == 0:
            loads, s1 = shuffle(operand)
            _, s2 = shuffle(flat[i + 2][1])
            back += loads + [(O.Dup2, 0), s1, flat[i + 1], s2, flat[i + 3]]
            i += 4
        elif op == RLOADS:
            loads, s1 = shuffle(operand)
            back += loads + [s1]
            i += 1
        elif op == RLOADP:
            back += [(O.FLoadReg0 + (operand & 0xFFFF) // 512, 0), (O.FPermW, sel_bytes(operand >> 16))]
            i += 1
        else:
            back.append((op, operand))
            i += 1
    flat = [(O.FLoadReg0 + operand // 512, 0) if op == RLOAD else (O.FStoreReg0 + operand // 512, 0) if op == RSTORE else (op, operand)
            for op, operand in back]
    # 2. fast accesses -> the generic opcodes they specialise
    generic = {LOAD_1D_FAST: O.LoadGlobal1DF32, STORE_1D_FAST: O.StoreGlobal1DF32, PF_ISSUE_1D_FAST: PF_ISSUE_1D,
               PF_TAKE_ISSUE_1D_FAST: PF_TAKE_ISSUE_1D, LOAD_2DW_FAST: O.LoadGlobal2DWF32, STORE_2DW_FAST: O.StoreGlobal2DWF32}
    # (their operand is {8 * slot in bits 26..31, byte offset of the tile in bits 0..25})
    flat = [(generic[op], ((operand & 0x03FFFFFF) // 4) << 4 | operand >> 29) if op in generic else (op, operand) for op, operand in flat]
    # staged row blocks: the copy at the program start disappears, the row loads get their tensor slot and column back
    # (operand of LoadStagedRows: log2 chunks per row in bits 0..1, chunk of the row in bits 2..3, slot in bits 4..6)
    flat = [(O.LoadGlobal2DWF32, (((operand >> 2) & 3) * 4) << 4 | (operand >> 4) & 7) if op == LOAD_STAGED_ROWS else (op, operand)
            for op, operand in flat if op != STAGE_ROWS]
    # 3. replay the ring of early-issued loads
    out, ring = [], []
    for op, operand in flat:
        if op == PF_ISSUE_1D:
            ring.append((O.LoadGlobal1DF32, operand))
        elif op == PF_SKIP:
            pass
        elif op == PF_TAKE:
            out.append(ring.pop(0))
        elif op == PF_TAKE_ISSUE_1D:
            out.append(ring.pop(0))
            ring.append((O.LoadGlobal1DF32, operand))
        else:
            out.append((op, operand))
    assert not ring, "loads were issued but never taken"
    return out


def zero_operands(prog):
    """Operands of instructions that ignore them are not preserved by fused handlers."""
    uses = set(range(O.LoadImm, O.LoadGlobal1DU8 + 1)) | {O.FApprox, O.FPermW, O.FShuf2} | set(range(O.LoadGlobal1DF32Indirect, O.DupBroadcastW + 1))
    return [(op, operand if op in uses else 0) for op, operand in prog]


@pytest.mark.parametrize("early,fuse", [(0, 0), (1, 0), (0, 1), (1, 1)])
def test_transforms_are_invertible_on_recorded_programs(early, fuse):
    table = fused_table()
    for name, rec in load_records().items():
        if name == "execute_everything":
            continue
        prog = recorded(name)
        got = transform(prog.bytecode, prog.tensor_infos, early, fuse)
        want = normalised(prog.bytecode)
        if early:
            want = fold_repeated_loads(want)
        assert zero_operands(undo(got, table)) == zero_operands(want), name


@pytest.mark.parametrize("family", ["float", "int"])
def test_transforms_are_invertible_on_random_programs(family):
    table = fused_table()
    for seed in range(40):
        depth, regs = [(3, 1), (4, 0), (6, 1), (7, 4), (8, 4), (4, 8), (5, 7), (2, 2)][seed % 8]
        prog = FuzzProgram(seed, family, depth, regs, length=80 + 5 * seed, rows=33, cols=36)
        pd = prog.get_program()
        got = transform(pd.program, pd.input_infos, 1, 1)
        want = fold_repeated_loads(normalised(pd.program))
        assert zero_operands(undo(got, table)) == zero_operands(want), seed


def test_register_file_stream_is_invertible_and_shorter():
    """The 4x4 inverse (8 registers, stack depth 5: the 12-slot pool) qualifies for the kernels that keep the registers in shared
    memory; its stream there undoes to the same program and needs less than half the dispatches."""
    table = fused_table()
    prog = recorded("inv4x4_b4194304")
    for early in (2, 3):
        got = transform(prog.bytecode, prog.tensor_infos, early, 1)
        want = normalised(prog.bytecode)
        if early & 1:
            want = fold_repeated_loads(want)
        assert zero_operands(undo(got, table)) == zero_operands(want)
        members = [m for op, _ in got for m in (table[op] if op in table else [op])]
        assert not any(O.FLoadReg0 <= m <= O.FStoreReg7 for m in members) and members.count(RSTORE) == 16
        # 56 register loads: 25 carry their lane permutation, 15 are plain, 16 went into 12 shuffles (4 shuffles of a register
        # pair, and 4 pairs that the program duplicated on the stack to shuffle them twice)
        assert (members.count(RLOADP), members.count(RLOADS), members.count(RLOAD)) == (25, 12, 15)
        assert O.FPermW in members and O.FShuf2 not in members      # permutations of computed values stay
    assert sum(1 for op, _ in transform(prog.bytecode, prog.tensor_infos, 3, 1) if op != -1) <= 45
    assert sum(1 for op, _ in transform(prog.bytecode, prog.tensor_infos, 1, 1) if op != -1) >= 160
    # programs whose pool is smaller than 12 slots keep their registers in the pool
    lib = capi.load_library()
    small = recorded("rmsnorm_r64_n4096")
    code = np.ascontiguousarray(np.asarray(small.bytecode, dtype=np.int32).reshape(-1))
    ti = capi.HTensorInfo()
    fill_tensor_info(ti, small.tensor_infos)
    assert lib.gint_debug_transform(code.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)), code.size, ctypes.byref(ti), len(small.tensor_infos),
                                    3, 1, None, None, 4096) == 0


def _rf_qualifies(bytecode):
    lib = capi.load_library()
    code = np.ascontiguousarray(np.asarray(bytecode, dtype=np.int32).reshape(-1))
    infos = [capi_info()]
    ti = capi.HTensorInfo()
    fill_tensor_info(ti, infos)
    n = lib.gint_debug_transform(code.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)), code.size, ctypes.byref(ti), 1, 2, 0, None, None, 4096)
    assert n >= 0, n
    return n > 0


def capi_info():
    from gint_b200.host import frontend as fe
    return fe.ProgramTensorInfo(4, [], [], [128, 1], [1, 0], [1, 1], [0, 0])


def test_register_file_needs_an_unobservable_overlap():
    """In the 12-slot pool register 7 IS stack slot 4 (register n = pool[11 - n]). A program that can see this keeps the pool
    layout; one that cannot may keep its registers elsewhere."""
    from gint_b200.host import frontend as fe
    one = [fe.LoadImm, 0x3F800000]
    push5, pop5 = [one] * 5, [[fe.Pop, 0]] * 5
    tail = [[fe.StoreGlobal1DF32, 0], [0, 0]]
    # register 7 is written, the stack then grows over it, and it is read afterwards: the overlap is visible
    seen = [one, [fe.FStoreReg7, 0]] + push5 + pop5 + [[fe.FLoadReg7, 0]] + tail
    assert not _rf_qualifies(seen)
    # the same with the register written after the stack has shrunk again
    unseen = push5 + pop5 + [one, [fe.FStoreReg7, 0], [fe.FLoadReg7, 0]] + tail
    assert _rf_qualifies(unseen)
    # a stack value that a register store would clobber
    clobber = push5 + [one, [fe.FStoreReg7, 0]] + [[fe.FAdd, 0]] * 4 + tail
    assert not _rf_qualifies(clobber)
    # a register read before it is written reads the zero the pool starts with: stays in the pool
    unwritten = push5 + pop5 + [[fe.FLoadReg7, 0]] + tail
    assert not _rf_qualifies(unwritten)
    # stack deeper than the 7 slots of the register-file kernels
    deep = [one, [fe.FStoreReg7, 0]] + [one] * 8 + [[fe.Pop, 0]] * 7 + tail
    assert not _rf_qualifies(deep)


def _vec_stream(bytecode, infos):
    """The stream for the vector-layout kernels (early-issue pass + layout analysis, no fusion), or [] if the program does not qualify."""
    lib = capi.load_library()
    code = np.ascontiguousarray(np.asarray(bytecode, dtype=np.int32).reshape(-1))
    ti = capi.HTensorInfo()
    fill_tensor_info(ti, infos)
    ops, operands = (ctypes.c_int32 * 4096)(), (ctypes.c_uint32 * 4096)()
    n = lib.gint_debug_transform(code.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)), code.size, ctypes.byref(ti), len(infos), 5, 0, ops, operands, 4096)
    assert n >= 0, n
    return [(ops[i], operands[i]) for i in range(n)]


def test_vector_layout_stream_of_the_row_programs():
    """RMSNorm and the conductor graph's fused program: every tile access is a full aligned 1-D tile, everything between them is
    element-wise, and the one place that looks across lanes -- the warp reduction of the sum of squares -- gets ONE RemapVN in front
    of it. What the reduction leaves is provably the same in all lanes and width values (after WarpAllReduceSum and the two
    FPermW / FAdd steps), so the second pass may multiply vector-layout tiles with it. The stream undoes to the same program."""
    table = fused_table()
    for name in ("rmsnorm_r16384_n4096", "graph_fused_r65536_n1024", "graph_fused_r96_n1024"):
        prog = recorded(name)
        got = _vec_stream(prog.bytecode, prog.tensor_infos)
        ops = [op for op, _ in got]
        assert ops.count(REMAP_VN) == 1 and ops[ops.index(REMAP_VN) + 1] == O.WarpAllReduceSum, name
        assert zero_operands(undo(got, table)) == zero_operands(fold_repeated_loads(normalised(prog.bytecode))), name
    # the row-sum program and short rows would qualify, but a handful of loads does not pay for the rearrangement; ragged rows have
    # masked tiles
    for name in ("graph_rowsum_r65536_n1024", "rmsnorm_r7_n256", "rmsnorm_r5_n200", "add_n1048576", "bmm4x4_b4194304"):
        prog = recorded(name)
        assert _vec_stream(prog.bytecode, prog.tensor_infos) == [], name


def test_vector_layout_analysis_refuses_what_it_cannot_prove():
    from gint_b200.host import frontend as fe
    n_tiles = 16
    infos = [fe.ProgramTensorInfo(4, [], [], [128 * n_tiles, 1], [1, 0], [1, 1], [0, 0]) for _ in range(2)]

    def program(per_tile):
        bc = []
        for i in range(n_tiles):
            bc += [[fe.LoadGlobal1DF32, 16 * 128 * i + 0]] + per_tile + [[fe.StoreGlobal1DF32, 16 * 128 * i + 1]]
        return np.array(bc + [[0, 0]], dtype=np.int32)

    def count(per_tile):
        return [op for op, _ in _vec_stream(program(per_tile), infos)].count(REMAP_VN)

    assert _vec_stream(program([[fe.FMulImm, 0x40000000]]), infos) != [] and count([[fe.FMulImm, 0x40000000]]) == 0      # element-wise: no rearrangement
    assert _vec_stream(program([[fe.LoadImm, 0x3F800000], [fe.FAdd, 0]]), infos) != []                                   # a uniform operand mixes with anything
    # a value that differs per width value (here: 1, 2, 3, 4) means other elements in the two layouts
    assert _vec_stream(program([[fe.LoadImm4F, 0x04030201], [fe.FMul, 0]]), infos) == []
    # a lane permutation of tile data needs the natural layout, and the fast store behind it the vector layout again
    assert _vec_stream(program([[fe.FPermW, 0x00010203]]), infos) == []
    # ... but a permutation that feeds a reduction is fine: one rearrangement per tile, which is too many to pay off
    assert _vec_stream(program([[fe.Dup, 0], [fe.FPermW, 0x00010203], [fe.WarpAllReduceSum, 0], [fe.Pop, 0]]), infos) == []
    # a width-uniform value made from a reduction: sum over lanes, then over the four width values, then used as a scale
    reduce_all = [[fe.Dup, 0], [fe.WarpAllReduceSum, 0], [fe.Dup, 0], [fe.FPermW, 0x01000302], [fe.FAdd, 0], [fe.Dup, 0], [fe.FPermW, 0x02030001], [fe.FAdd, 0], [fe.FMul, 0]]
    bc = [[fe.LoadGlobal1DF32, 0]] + reduce_all[1:-1] + [[fe.FStoreReg0, 0]]
    for i in range(n_tiles):
        bc += [[fe.LoadGlobal1DF32, 16 * 128 * i + 0], [fe.FLoadReg0, 0], [fe.FMul, 0], [fe.StoreGlobal1DF32, 16 * 128 * i + 1]]
    got = [op for op, _ in _vec_stream(np.array(bc + [[0, 0]], dtype=np.int32), infos)]
    assert got.count(REMAP_VN) == 1
    # the same with only ONE of the two width steps: the scale still differs between width values, the program keeps its layout
    half = [[fe.LoadGlobal1DF32, 0], [fe.WarpAllReduceSum, 0], [fe.Dup, 0], [fe.FPermW, 0x01000302], [fe.FAdd, 0], [fe.FStoreReg0, 0]]
    for i in range(n_tiles):
        half += [[fe.LoadGlobal1DF32, 16 * 128 * i + 0], [fe.FLoadReg0, 0], [fe.FMul, 0], [fe.StoreGlobal1DF32, 16 * 128 * i + 1]]
    assert _vec_stream(np.array(half + [[0, 0]], dtype=np.int32), infos) == []


def test_named_programs_get_the_expected_shape():
    """The conductor's RMSNorm lowering: 363 instructions become about a hundred dispatches."""
    table = fused_table()
    prog = recorded("rmsnorm_r16384_n4096")
    plain = transform(prog.bytecode, prog.tensor_infos, 0, 0)
    both = transform(prog.bytecode, prog.tensor_infos, 1, 1)
    dispatches = sum(1 for op, _ in both if op != -1)
    assert len(plain) == 363
    assert dispatches < 130
    takes = (PF_TAKE_ISSUE_1D, PF_TAKE_ISSUE_1D_FAST, PF_TAKE)
    assert sum(sum(m in takes for m in (table[op] if op in table else [op])) for op, _ in both) == 96
    assert dispatches < 80     # two reduction steps, or a whole scale-and-store chunk, per dispatch
    # every tile of this program is full, unit-stride and 16-byte aligned: only the fast forms remain
    members = [m for op, _ in both for m in (table[op] if op in table else [op])]
    assert PF_TAKE_ISSUE_1D not in members and PF_ISSUE_1D not in members and O.StoreGlobal1DF32 not in members
    assert members.count(STORE_1D_FAST) == 32
    # ring depth: 8 loads ahead for this long-row streaming program, 4 for the conductor graph's 1024-wide rows
    assert [op for op, _ in both[:9]].count(PF_ISSUE_1D_FAST) == 8
    graph = recorded("graph_fused_r65536_n1024")
    assert [op for op, _ in transform(graph.bytecode, graph.tensor_infos, 1, 1)[:9]].count(PF_ISSUE_1D_FAST) == 4
    # a store between two loads of the same tensor keeps the second load where it is
    from gint_b200.host import frontend as fe
    bc = [[fe.LoadGlobal1DF32, 0], [fe.StoreGlobal1DF32, 16 * 128 + 0], [fe.LoadGlobal1DF32, 16 * 128 + 0], [fe.StoreGlobal1DF32, 1], [0, 0]]
    infos = [fe.ProgramTensorInfo(4, [], [], [256, 1], [1, 0], [1, 1], [0, 0]) for _ in range(2)]
    got = transform(np.array(bc, dtype=np.int32), infos, 1, 0)
    assert [op for op, _ in got].count(LOAD_1D_FAST) == 1      # the second load was not moved across the store


def test_fast_accesses_need_full_aligned_tiles():
    from gint_b200.host import frontend as fe

    def ops_for(n, off=0, stride=1):
        bc = [[fe.LoadGlobal1DF32, 16 * off + 0], [fe.LoadGlobal1DF32, 16 * off + 1], [fe.FAdd, 0], [fe.StoreGlobal1DF32, 16 * off + 2], [0, 0]]
        infos = [fe.ProgramTensorInfo(4, [], [], [n, stride], [1, 0], [(n + 127) // 128, 1], [128, 0]) for _ in range(3)]
        return [op for op, _ in transform(np.array(bc, dtype=np.int32), infos, 1, 0)]

    assert ops_for(1024) == [PF_ISSUE_1D_FAST, PF_ISSUE_1D_FAST, PF_SKIP, PF_TAKE, PF_TAKE, fe.FAdd, STORE_1D_FAST, 0]
    assert STORE_1D_FAST not in ops_for(1000) and PF_ISSUE_1D_FAST not in ops_for(1000)      # ragged last tile
    assert STORE_1D_FAST not in ops_for(1024 + 2, off=2)                                    # tile starts off a 16-byte boundary
    assert STORE_1D_FAST not in ops_for(1024, stride=2)                                     # not unit-stride


def test_small_matrix_operands_are_staged_as_row_blocks():
    """bmm4x4: A and B (32 matrices of 16 floats back to back per logical program) are copied to shared memory once and all
    20 row loads read from there; a ragged batch keeps its masked row loads."""
    table = fused_table()
    prog = recorded("bmm4x4_b4194304")
    got = transform(prog.bytecode, prog.tensor_infos, 1, 1)
    members = [m for op, _ in got for m in (table[op] if op in table else [op])]
    assert members.count(STAGE_ROWS) == 2 and members.count(LOAD_STAGED_ROWS) == 20 and O.LoadGlobal2DWF32 not in members
    assert [op for op, _ in got[:2]] == [STAGE_ROWS, STAGE_ROWS]
    ragged = recorded("bmm4x4_b1000")
    members = [m for op, _ in transform(ragged.bytecode, ragged.tensor_infos, 1, 1) for m in (table[op] if op in table else [op])]
    assert STAGE_ROWS not in members and members.count(O.LoadGlobal2DWF32) == 20
