/*
 * gint_opcodes.h -- opcode numbers and stack effects of the gint bytecode format, as an X-macro.
 *
 * Numbering follows the reference's INSNS table (gint/kernel/interpreter/main.py:61-168); the
 * (minimum depth, net effect) pairs follow its analyzer (gint/host/analyzer.py:24-135).
 * X(name, opcode, min_depth, net_effect)
 */
#ifndef GINT_OPCODES_H
#define GINT_OPCODES_H

#define GINT_N_OPCODES 106
#define GINT_MAX_STACK 8
#define GINT_NUM_REGS 8

#define GINT_OPCODE_LIST(X) \
    X(Halt, 0, 0, 0) \
    X(Nop, 1, 0, 0) \
    X(FAdd, 2, 2, -1) \
    X(FMul, 3, 2, -1) \
    X(FMA, 4, 3, -2) \
    X(FSub, 5, 2, -1) \
    X(FRSub, 6, 2, -1) \
    X(FNeg, 7, 1, 0) \
    X(FDiv, 8, 2, -1) \
    X(FRDiv, 9, 2, -1) \
    X(FRem, 10, 2, -1) \
    X(LoadImm, 11, 0, 1) \
    X(FAddImm, 12, 1, 0) \
    X(FMulImm, 13, 1, 0) \
    X(FMAImm, 14, 1, 0) \
    X(LoadGlobal1DF32, 15, 0, 1) \
    X(StoreGlobal1DF32, 16, 1, -1) \
    X(LoadGlobal1DF16, 17, 0, 1) \
    X(StoreGlobal1DF16, 18, 1, -1) \
    X(LoadGlobal1DBF16, 19, 0, 1) \
    X(StoreGlobal1DBF16, 20, 1, -1) \
    X(LoadGlobal1DU8, 21, 0, 1) \
    X(Pop, 22, 1, -1) \
    X(Pop2, 23, 2, -2) \
    X(Dup, 24, 1, 1) \
    X(DupX1, 25, 2, 1) \
    X(DupX2, 26, 3, 1) \
    X(Dup2, 27, 2, 2) \
    X(FGt, 28, 2, -1) \
    X(FLt, 29, 2, -1) \
    X(FGe, 30, 2, -1) \
    X(FLe, 31, 2, -1) \
    X(FEq, 32, 2, -1) \
    X(FNe, 33, 2, -1) \
    X(FApprox, 34, 2, -1) \
    X(Select, 35, 3, -2) \
    X(WarpAllReduceSum, 36, 1, 0) \
    X(WarpAllReduceMax, 37, 1, 0) \
    X(WarpAllReduceMin, 38, 1, 0) \
    X(WarpAllReduceProd, 39, 1, 0) \
    X(FSqrt, 40, 1, 0) \
    X(FSin, 41, 1, 0) \
    X(FCos, 42, 1, 0) \
    X(FTan, 43, 1, 0) \
    X(FArcSin, 44, 1, 0) \
    X(FArcCos, 45, 1, 0) \
    X(FArcTan, 46, 1, 0) \
    X(FArcTan2, 47, 2, -1) \
    X(FPow, 48, 2, -1) \
    X(FExp, 49, 1, 0) \
    X(FExp2, 50, 1, 0) \
    X(FLog, 51, 1, 0) \
    X(FLog2, 52, 1, 0) \
    X(FRSqrt, 53, 1, 0) \
    X(FErf, 54, 1, 0) \
    X(Swap, 55, 2, 0) \
    X(IAdd, 56, 2, -1) \
    X(IMul, 57, 2, -1) \
    X(ISub, 58, 2, -1) \
    X(IDiv, 59, 2, -1) \
    X(IRem, 60, 2, -1) \
    X(IShl, 61, 2, -1) \
    X(IShr, 62, 2, -1) \
    X(IAnd, 63, 2, -1) \
    X(IOr, 64, 2, -1) \
    X(IXor, 65, 2, -1) \
    X(LoadGlobal1DF32Indirect, 66, 1, 0) \
    X(StoreGlobal1DF32Indirect, 67, 2, -2) \
    X(LoadImm4F, 68, 0, 1) \
    X(LoadImm4I, 69, 0, 1) \
    X(LoadGlobal2DTF32, 70, 0, 1) \
    X(StoreGlobal2DTF32, 71, 1, -1) \
    X(LoadGlobal2DTF16, 72, 0, 1) \
    X(StoreGlobal2DTF16, 73, 1, -1) \
    X(LoadGlobal2DTBF16, 74, 0, 1) \
    X(StoreGlobal2DTBF16, 75, 1, -1) \
    X(LoadGlobal2DTU8, 76, 0, 1) \
    X(LoadGlobal2DWF32, 77, 0, 1) \
    X(StoreGlobal2DWF32, 78, 1, -1) \
    X(LoadGlobal2DWF16, 79, 0, 1) \
    X(StoreGlobal2DWF16, 80, 1, -1) \
    X(LoadGlobal2DWBF16, 81, 0, 1) \
    X(StoreGlobal2DWBF16, 82, 1, -1) \
    X(LoadGlobal2DWU8, 83, 0, 1) \
    X(AdvanceBlock2D, 84, 0, 0) \
    X(AdvanceBase, 85, 0, 0) \
    X(DupBroadcastW, 86, 1, 1) \
    X(FLoadReg0, 87, 0, 1) \
    X(FLoadReg1, 88, 0, 1) \
    X(FLoadReg2, 89, 0, 1) \
    X(FLoadReg3, 90, 0, 1) \
    X(FLoadReg4, 91, 0, 1) \
    X(FLoadReg5, 92, 0, 1) \
    X(FLoadReg6, 93, 0, 1) \
    X(FLoadReg7, 94, 0, 1) \
    X(FStoreReg0, 95, 1, -1) \
    X(FStoreReg1, 96, 1, -1) \
    X(FStoreReg2, 97, 1, -1) \
    X(FStoreReg3, 98, 1, -1) \
    X(FStoreReg4, 99, 1, -1) \
    X(FStoreReg5, 100, 1, -1) \
    X(FStoreReg6, 101, 1, -1) \
    X(FStoreReg7, 102, 1, -1) \
    X(FRcp, 103, 1, 0) \
    X(FPermW, 104, 1, 0) \
    X(FShuf2, 105, 2, -1)

/*
 * Internal opcodes. They never appear in a gint bytecode stream; the host pre-decoder (gint_capi.cu) introduces them when
 * it turns tile loads into "issue early, take later" pairs over a ring of staging slots in shared memory (see
 * exec_all / tile_issue in gint_interp.cuh):
 *   PfTake               push the four values waiting in the ring's current slot, advance the ring
 *   PfIssue1D            start the 1-D tile load described by the operand into the current slot, advance (program prologue)
 *   PfTakeIssue1D        PfTake, then start the load described by the operand into the slot just emptied
 *   PfSkip               advance the ring by `operand` slots without touching them (after a prologue shorter than the ring)
 * and when it can prove, from a program's descriptors, that a 1-D f32 access is always a full unit-stride tile that starts
 * on a 16-byte boundary (given a 16-byte aligned base pointer, which is checked at every launch):
 *   LoadGlobal1DF32Fast / StoreGlobal1DF32Fast   the same access without shape, stride or mask handling
 *   PfIssue1DFast / PfTakeIssue1DFast            PfIssue1D / PfTakeIssue1D likewise: one 16-byte copy per lane
 * and for a tensor that a program only reads through 2DW row loads, whose 32 rows per logical program are short (4, 8 or 16
 * floats) and lie back to back in memory (one lane = one small matrix):
 *   StageRows        copy the whole 32-row block into shared memory with fully coalesced 16-byte copies (program start)
 *   LoadStagedRows   the row load, served from that copy
 * (a row load by itself is a 16-byte access per lane at the row stride: 16 L1 wavefronts per warp where 4 would do)
 */
/*
 * DupBroadcastW with the lane index built into the opcode (no operand is read at run time). The format's DupBroadcastW carries
 * its lane index in the operand word, so a handler has to select the value among four at run time; the index is a constant
 * of the program, and with it in the opcode the handler is two register moves per tile:
 *   Bcast_k    push (T[k], T[k], T[k], T[k])
 * (The same was tried for FPermW and FShuf2, split into two steps of 16 index pairs each: four moves per tile instead of a
 * dozen selects, but a program with many different permutations then jumps between several times as many distinct handlers,
 * and the instruction cache misses cost more than the selects had -- the 4x4 inverse ran 2.2 times slower.)
 */
/* ... and for a tensor whose 2DW rows the host can prove full, 16-byte aligned and never masked, for every logical program
 * (given a 16-byte aligned base pointer, checked at every launch):
 *   LoadGlobal2DWF32Fast / StoreGlobal2DWF32Fast   one 128-bit access per lane, no shape, mask or alignment handling
 */
/*
 * Virtual registers kept in shared memory (the kernels built with GINT_RF, see gint_interp.cuh). A program that needs the
 * 12-slot pool only because of its eight virtual registers runs with a pool that holds just its operand stack; the registers
 * live in a per-warp block of shared memory and the register number travels in the operand word, so one handler serves all
 * eight registers and sequences such as "load register, permute, load register, multiply" can be fused whatever registers
 * they name:
 *   RLoad    push register (operand / 512)      -- operand = 512 * register number
 *   RStore   pop into register (operand / 512)
 *   RLoadP   push a lane permutation of a register: RLoad, FPermW in one (the register area keeps the four width values of a
 *            lane in four planes, so a permutation is the same four loads from other planes and costs no selects)
 *   RLoadS   push a shuffle of two registers: RLoad a, RLoad b, FShuf2 in one
 * The host introduces them (gint_capi.cu: rf_transform) only where the reference's overlap of stack and registers in one
 * pool cannot be observed by the program.
 */
#define GINT_INTERNAL_OPCODE_LIST(X) \
    X(PfTake, 106, 0, 1) X(PfIssue1D, 107, 0, 0) X(PfTakeIssue1D, 108, 0, 1) X(PfSkip, 109, 0, 0) \
    X(LoadGlobal1DF32Fast, 110, 0, 1) X(StoreGlobal1DF32Fast, 111, 1, -1) X(PfIssue1DFast, 112, 0, 0) X(PfTakeIssue1DFast, 113, 0, 1) \
    X(StageRows, 114, 0, 0) X(LoadStagedRows, 115, 0, 1) \
    X(Bcast_0, 116, 1, 1) X(Bcast_1, 117, 1, 1) X(Bcast_2, 118, 1, 1) X(Bcast_3, 119, 1, 1) \
    X(LoadGlobal2DWF32Fast, 120, 0, 1) X(StoreGlobal2DWF32Fast, 121, 1, -1)
/* the register-file kernels' own opcodes: numbered after the fused handlers of the ordinary kernels (gint_fused.h), so that
 * nothing in the ordinary kernels -- numbering, dispatch keys, generated code -- depends on them */
#define GINT_RF_OPCODE_LIST(X) X(RLoad, 150, 0, 1) X(RStore, 151, 1, -1) X(RLoadP, 152, 0, 1) X(RLoadS, 153, 0, 1)
/* opcodes a kernel dispatches on: the 106 of the format, the 16 internal ones and the 28 fused handlers of gint_fused.h; in
 * the register-file kernels also RLoad / RStore and the register-operand fused handlers */
/* the vector-layout kernels' own opcode (GINT_VEC, see gint_interp.cuh): in those kernels a 1-D tile that the host proved
 * full, unit-stride and aligned lives in the pool with lane l holding elements 4l..4l+3 (one 16-byte access per lane) instead of
 * elements l, l+32, l+64, l+96. Element-wise work does not care; an instruction that looks across lanes or width values does,
 * and the host puts this in front of it (gint_capi.cu: vec_transform):
 *   RemapVN   rearrange the top of the stack from the vector layout into the natural one (through shared memory) */
#define GINT_VEC_OPCODE_LIST(X) X(RemapVN, 180, 1, 0)
#define GINT_N_DISPATCH_PLAIN 150
#define GINT_N_DISPATCH_RF 176
#define GINT_N_DISPATCH_VEC 181
#if defined(GINT_RF)
#define GINT_N_DISPATCH GINT_N_DISPATCH_RF
#elif defined(GINT_VEC)
#define GINT_N_DISPATCH GINT_N_DISPATCH_VEC
#else
#define GINT_N_DISPATCH GINT_N_DISPATCH_PLAIN
#endif

enum gint_opcode {
#define GINT_X_ENUM(name, num, md, net) OP_##name = num,
    GINT_OPCODE_LIST(GINT_X_ENUM)
    GINT_INTERNAL_OPCODE_LIST(GINT_X_ENUM)
    GINT_RF_OPCODE_LIST(GINT_X_ENUM)
    GINT_VEC_OPCODE_LIST(GINT_X_ENUM)
#undef GINT_X_ENUM
};

#endif /* GINT_OPCODES_H */
