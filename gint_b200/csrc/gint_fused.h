/*
 * gint_fused.h -- fused handlers ("superinstructions"): fixed sequences of bytecode instructions that the interpreter
 * executes with a single dispatch.
 *
 * Every interpreted instruction pays for one fetch and one indirect branch, about as much as the work of a simple
 * instruction itself. The host pre-decoder (gint_capi.cu) therefore replaces the most common instruction sequences by one
 * internal opcode each; the kernel's handler for such an opcode is generated at compile time by running the handlers of
 * the listed instructions back to back at their (static) stack depths. Semantics do not change: the same operations run
 * in the same order on the same slots; only the dispatches in between disappear.
 *
 * The sequences below are the idioms of the gint frontend and conductor lowerings: the chunk bodies of row reductions and
 * of scale-and-store loops, SiLU, and the inner step and row end of the 4x4 matmul.
 * 1-D loads appear in the two flavours the early-issue transformation (gint_capi.cu) produces for provably full, aligned
 * tiles before fusion runs: taken from the ring while the next one is started, and taken without a successor.
 *
 * In the pre-decoded stream a fused instruction occupies one entry, plus one entry for every member after the first
 * that reads an operand word.
 *
 * X(number, length, op0, op1, ...). Numbers continue the internal opcode space of gint_opcodes.h.
 */
#ifndef GINT_FUSED_H
#define GINT_FUSED_H

#include "gint_opcodes.h"

#define GINT_FUSED_FIRST 122

/* one entry per load flavour L for the 1-D idioms */
#define GINT_FUSED_1D(X, base, L)                                                        \
    X(base + 0, 4, L, OP_Dup, OP_FMul, OP_FAdd)             /* acc += x*x             */ \
    X(base + 1, 3, L, OP_Dup, OP_FMul)                      /* x*x                    */ \
    X(base + 2, 4, OP_Dup, L, OP_Swap, OP_FMul)             /* s, s*x                 */ \
    X(base + 3, 3, L, OP_FMul, OP_StoreGlobal1DF32Fast)     /* store(top * w)         */ \
    X(base + 4, 2, L, OP_FMul)                                                           \
    X(base + 5, 2, L, OP_FAdd)                                                           \
    X(base + 6, 3, L, OP_FAdd, OP_StoreGlobal1DF32Fast)

#define GINT_FUSED_LIST(X)                                                               \
    GINT_FUSED_1D(X, GINT_FUSED_FIRST + 0, OP_PfTakeIssue1DFast)                         \
    GINT_FUSED_1D(X, GINT_FUSED_FIRST + 7, OP_PfTake)                                    \
    X(GINT_FUSED_FIRST + 14, 5, OP_Dup, OP_FNeg, OP_FExp, OP_FAddImm, OP_FRDiv)          /* SiLU      */ \
    X(GINT_FUSED_FIRST + 15, 5, OP_Pop, OP_FAdd, OP_FAdd, OP_FAdd, OP_StoreGlobal2DWF32)   /* bmm row end */ \
    X(GINT_FUSED_FIRST + 16, 5, OP_Pop, OP_FAdd, OP_FAdd, OP_FAdd, OP_StoreGlobal2DWF32Fast) \
    X(GINT_FUSED_FIRST + 17, 2, OP_FMul, OP_FAdd)                                        \
    X(GINT_FUSED_FIRST + 18, 2, OP_FMul, OP_StoreGlobal1DF32Fast)                        \
    /* whole chunk bodies: two reduction steps; scale by s and by w, store; the same without the store; SiLU, add, store */ \
    X(GINT_FUSED_FIRST + 19, 8, OP_PfTakeIssue1DFast, OP_Dup, OP_FMul, OP_FAdd, OP_PfTakeIssue1DFast, OP_Dup, OP_FMul, OP_FAdd) \
    X(GINT_FUSED_FIRST + 20, 7, OP_Dup, OP_PfTakeIssue1DFast, OP_Swap, OP_FMul, OP_PfTakeIssue1DFast, OP_FMul, OP_StoreGlobal1DF32Fast) \
    X(GINT_FUSED_FIRST + 21, 6, OP_Dup, OP_PfTakeIssue1DFast, OP_Swap, OP_FMul, OP_PfTakeIssue1DFast, OP_FMul) \
    X(GINT_FUSED_FIRST + 22, 8, OP_Dup, OP_FNeg, OP_FExp, OP_FAddImm, OP_FRDiv, OP_PfTakeIssue1DFast, OP_FAdd, OP_StoreGlobal1DF32Fast) \
    X(GINT_FUSED_FIRST + 23, 4, OP_PfTakeIssue1DFast, OP_FAdd, OP_PfTakeIssue1DFast, OP_FAdd)                \
    /* inner step of the 4x4 product over staged rows, one per broadcast lane */         \
    X(GINT_FUSED_FIRST + 24, 4, OP_Bcast_0, OP_LoadStagedRows, OP_FMul, OP_Swap)         \
    X(GINT_FUSED_FIRST + 25, 4, OP_Bcast_1, OP_LoadStagedRows, OP_FMul, OP_Swap)         \
    X(GINT_FUSED_FIRST + 26, 4, OP_Bcast_2, OP_LoadStagedRows, OP_FMul, OP_Swap)         \
    X(GINT_FUSED_FIRST + 27, 4, OP_Bcast_3, OP_LoadStagedRows, OP_FMul, OP_Swap)

#define GINT_N_FUSED 28
#define GINT_N_DISPATCH_ALL (GINT_FUSED_FIRST + GINT_N_FUSED)   /* 150 */

/*
 * Register-operand forms, for the kernels that keep the virtual registers in shared memory (GINT_RF) and the streams made for
 * them. RLoad / RStore / RLoadP / RLoadS carry register numbers and lane selectors in their operand words, so ONE handler
 * serves a sequence whatever registers and lane permutations it names -- with the registers in the pool every combination
 * would need a handler of its own. The sequences are the building blocks of the small-matrix programs (gint/host/matrix.py:
 * products of two permuted registers, accumulated or subtracted; shuffles of register pairs; shuffled pairs stored as rows).
 * Numbered after RLoad / RStore (gint_opcodes.h).
 */
#define GINT_RF_FUSED_FIRST 154
#define GINT_RF_PP OP_RLoadP, OP_RLoadP, OP_FMul      /* perm(r[a]) * perm(r[b]) */
#define GINT_RF_P1 OP_RLoadP, OP_RLoad, OP_FMul       /* perm(r[a]) * r[b]       */
#define GINT_RF_1P OP_RLoad, OP_RLoadP, OP_FMul       /* r[a] * perm(r[b])       */
#define GINT_RF_FUSED_LIST(X)                                                            \
    X(GINT_RF_FUSED_FIRST + 0, 3, GINT_RF_PP)                                            \
    X(GINT_RF_FUSED_FIRST + 1, 3, GINT_RF_P1)                                            \
    X(GINT_RF_FUSED_FIRST + 2, 3, GINT_RF_1P)                                            \
    X(GINT_RF_FUSED_FIRST + 3, 4, GINT_RF_PP, OP_FAdd)                                   \
    X(GINT_RF_FUSED_FIRST + 4, 4, GINT_RF_PP, OP_FSub)                                   \
    X(GINT_RF_FUSED_FIRST + 5, 4, GINT_RF_PP, OP_FRSub)                                  \
    X(GINT_RF_FUSED_FIRST + 6, 4, GINT_RF_P1, OP_FAdd)                                   \
    X(GINT_RF_FUSED_FIRST + 7, 4, GINT_RF_P1, OP_FSub)                                   \
    X(GINT_RF_FUSED_FIRST + 8, 4, GINT_RF_P1, OP_FRSub)                                  \
    X(GINT_RF_FUSED_FIRST + 9, 5, GINT_RF_PP, OP_FRSub, OP_RStore)                       \
    X(GINT_RF_FUSED_FIRST + 10, 6, GINT_RF_P1, OP_FSub, OP_RLoad, OP_FMul)               \
    X(GINT_RF_FUSED_FIRST + 11, 3, OP_RLoadS, OP_RLoadS, OP_FMul)                        \
    X(GINT_RF_FUSED_FIRST + 12, 4, OP_RLoadS, OP_RLoadS, OP_RStore, OP_RStore)           \
    X(GINT_RF_FUSED_FIRST + 13, 4, OP_RLoadS, OP_StoreGlobal2DWF32Fast, OP_RLoadS, OP_StoreGlobal2DWF32Fast) \
    X(GINT_RF_FUSED_FIRST + 14, 2, OP_RLoad, OP_FMul)                                    \
    X(GINT_RF_FUSED_FIRST + 15, 3, OP_FMul, OP_FRSub, OP_RStore)                         \
    X(GINT_RF_FUSED_FIRST + 16, 2, OP_FMul, OP_FRSub)                                    \
    X(GINT_RF_FUSED_FIRST + 17, 2, OP_FMul, OP_FSub)                                     \
    X(GINT_RF_FUSED_FIRST + 18, 2, OP_FRSub, OP_RStore)                                  \
    X(GINT_RF_FUSED_FIRST + 19, 2, OP_LoadStagedRows, OP_RStore)                         \
    X(GINT_RF_FUSED_FIRST + 20, 2, OP_RStore, OP_RStore)                                 \
    X(GINT_RF_FUSED_FIRST + 21, 3, OP_Dup, OP_FPermW, OP_FAdd)
#define GINT_N_RF_FUSED 22

/* is `op` a fused handler (of either list)? */
#define GINT_IS_FUSED(op) (((op) >= GINT_FUSED_FIRST && (op) < GINT_FUSED_FIRST + GINT_N_FUSED) || \
                           ((op) >= GINT_RF_FUSED_FIRST && (op) < GINT_RF_FUSED_FIRST + GINT_N_RF_FUSED))
#define GINT_MAX_FUSED_LEN 8

/* does the instruction read its operand word? (fused handlers fetch operands only for those that do) */
#define GINT_OP_USES_OPERAND(op)                                                                                           \
    (((op) >= OP_LoadImm && (op) <= OP_LoadGlobal1DU8) || (op) == OP_FApprox || ((op) >= OP_LoadGlobal1DF32Indirect && (op) <= OP_DupBroadcastW) || \
     (op) == OP_FPermW || (op) == OP_FShuf2 || (op) == OP_PfIssue1D || (op) == OP_PfTakeIssue1D || (op) == OP_PfSkip || ((op) >= OP_LoadGlobal1DF32Fast && (op) <= OP_LoadStagedRows) || \
     (op) == OP_LoadGlobal2DWF32Fast || (op) == OP_StoreGlobal2DWF32Fast || ((op) >= OP_RLoad && (op) <= OP_RLoadS))

#endif /* GINT_FUSED_H */
