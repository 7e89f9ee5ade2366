/*
 * gint_oracle.c -- lane-accurate CPU restatement of the gint device interpreter.
 *
 * TEST INFRASTRUCTURE ONLY. This file is the checker the GPU kernels are compared against; it is never
 * part of the product path and the product never falls back to it.
 *
 * The reference (eliphatfs/gint) has no CPU execution path for bytecode: its only device code is an
 * llvmlite-generated NVPTX kernel. This file restates that kernel's algorithm in plain C, one logical
 * program (= one 32-lane warp x 4 "width" values per stack slot) at a time, following:
 *
 *   kernel skeleton / dispatch      gint/kernel/interpreter/main.py:171-260
 *   machine state (unified pool)    gint/kernel/interpreter/state.py:11-78
 *   operand fetch, pc += 2          gint/kernel/interpreter/instruction.py:19-36
 *   tensor descriptor decode        gint/kernel/interpreter/instructions/load_tensor_infos.py:14-54
 *   descriptor layout (608 bytes)   gint/kernel/interpreter/structs.py:6-30
 *   global load/store, advance      gint/kernel/interpreter/instructions/load_store.py:9-321
 *   float ALU                       gint/kernel/interpreter/instructions/arith.py:7-66
 *   integer ALU                     gint/kernel/interpreter/instructions/arith_int.py:7-75
 *   immediates                      gint/kernel/interpreter/instructions/immediate.py:7-61
 *   stack / width-lane moves        gint/kernel/interpreter/instructions/move.py:7-135
 *   compare / select                gint/kernel/interpreter/instructions/predication.py:8-73
 *   virtual registers, FRcp         gint/kernel/interpreter/instructions/reg.py:7-67
 *   warp all-reduce                 gint/kernel/interpreter/instructions/reduction.py:7-30,
 *                                   gint/kernel/platforms/nvptx.py:89-104 (butterfly 16,8,4,2,1)
 *   special math                    gint/kernel/interpreter/instructions/special.py:7-87,
 *                                   gint/kernel/platforms/nvptx.py:106-129
 *   stack effects per opcode        gint/host/analyzer.py:24-135
 *   kernel variant selection        gint/host/executor.py:131-149
 *
 * Pinning: the restatement is checked (tests/test_oracle.py) against the known-answer tests the
 * reference keeps for this path (packed immediates, integer add, gather, scatter:
 * tests/test_frontend.py:166-208,245-291) and, on bytecode streams produced by running the reference's
 * own frontend/conductor (tests/golden/programs.json), against the torch-eager expressions the
 * reference's tests use as their oracle.
 *
 * Arithmetic notes. Float add/mul/sub/div are single IEEE operations with no contraction (build with
 * -ffp-contract=off); FMA/FMAImm use fmaf. Transcendentals use libm, so they agree with the GPU's
 * libdevice only to a few ulp. Integer ops are exact two's complement; shifts by >= 32 give 0 and
 * division by zero gives -1 / remainder by zero gives the dividend (the values the GPU path defines).
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define GINT_MAX_TENSORS 8
#define WARP 32
#define REGW 4
#define MAX_POOL 12

typedef struct {
    int64_t base_ptr[GINT_MAX_TENSORS];
    int32_t elm_size[GINT_MAX_TENSORS];
    int32_t batch_strides[GINT_MAX_TENSORS][4];
    int32_t batch_shape[GINT_MAX_TENSORS][4];
    int32_t block_shape_stride_1[GINT_MAX_TENSORS][2];
    int32_t block_shape_stride_2[GINT_MAX_TENSORS][2];
    int32_t block_grid_dims[GINT_MAX_TENSORS][2];
    int32_t block_grid_steps[GINT_MAX_TENSORS][2];
} oracle_tensor_info; /* 608 bytes, gint/kernel/interpreter/structs.py:19-30 */

typedef struct {
    int32_t num_instructions;
    int32_t max_stack;
    int32_t max_reg_idx;
    int32_t min_pool_size;
    int32_t regs_used_mask;
    int32_t error_index; /* instruction index of the first error, -1 if none */
} oracle_stats;

enum {
    ORACLE_OK = 0,
    ORACLE_ERR_UNKNOWN_OPCODE = -1,
    ORACLE_ERR_STACK_UNDERFLOW = -2,
    ORACLE_ERR_STACK_OVERFLOW = -3,
    ORACLE_ERR_NO_HALT = -4,
    ORACLE_ERR_BAD_ARG = -5,
};

#define N_OPCODES 106

/* (min depth, net effect) per opcode; gint/host/analyzer.py:24-135 */
static const int8_t EFFECTS[N_OPCODES][2] = {
    /*0 Halt*/ {0, 0}, /*1 Nop*/ {0, 0}, /*2 FAdd*/ {2, -1}, /*3 FMul*/ {2, -1}, /*4 FMA*/ {3, -2},
    /*5 FSub*/ {2, -1}, /*6 FRSub*/ {2, -1}, /*7 FNeg*/ {1, 0}, /*8 FDiv*/ {2, -1}, /*9 FRDiv*/ {2, -1},
    /*10 FRem*/ {2, -1}, /*11 LoadImm*/ {0, 1}, /*12 FAddImm*/ {1, 0}, /*13 FMulImm*/ {1, 0}, /*14 FMAImm*/ {1, 0},
    /*15 Ld1DF32*/ {0, 1}, /*16 St1DF32*/ {1, -1}, /*17 Ld1DF16*/ {0, 1}, /*18 St1DF16*/ {1, -1},
    /*19 Ld1DBF16*/ {0, 1}, /*20 St1DBF16*/ {1, -1}, /*21 Ld1DU8*/ {0, 1},
    /*22 Pop*/ {1, -1}, /*23 Pop2*/ {2, -2}, /*24 Dup*/ {1, 1}, /*25 DupX1*/ {2, 1}, /*26 DupX2*/ {3, 1}, /*27 Dup2*/ {2, 2},
    /*28 FGt*/ {2, -1}, /*29 FLt*/ {2, -1}, /*30 FGe*/ {2, -1}, /*31 FLe*/ {2, -1}, /*32 FEq*/ {2, -1}, /*33 FNe*/ {2, -1},
    /*34 FApprox*/ {2, -1}, /*35 Select*/ {3, -2},
    /*36-39 WarpAllReduce Sum,Max,Min,Prod*/ {1, 0}, {1, 0}, {1, 0}, {1, 0},
    /*40 FSqrt*/ {1, 0}, /*41 FSin*/ {1, 0}, /*42 FCos*/ {1, 0}, /*43 FTan*/ {1, 0}, /*44 FArcSin*/ {1, 0},
    /*45 FArcCos*/ {1, 0}, /*46 FArcTan*/ {1, 0}, /*47 FArcTan2*/ {2, -1}, /*48 FPow*/ {2, -1}, /*49 FExp*/ {1, 0},
    /*50 FExp2*/ {1, 0}, /*51 FLog*/ {1, 0}, /*52 FLog2*/ {1, 0}, /*53 FRSqrt*/ {1, 0}, /*54 FErf*/ {1, 0},
    /*55 Swap*/ {2, 0},
    /*56-65 IAdd,IMul,ISub,IDiv,IRem,IShl,IShr,IAnd,IOr,IXor*/
    {2, -1}, {2, -1}, {2, -1}, {2, -1}, {2, -1}, {2, -1}, {2, -1}, {2, -1}, {2, -1}, {2, -1},
    /*66 Ld1DF32Indirect*/ {1, 0}, /*67 St1DF32Indirect*/ {2, -2}, /*68 LoadImm4F*/ {0, 1}, /*69 LoadImm4I*/ {0, 1},
    /*70 Ld2DTF32*/ {0, 1}, /*71 St2DTF32*/ {1, -1}, /*72 Ld2DTF16*/ {0, 1}, /*73 St2DTF16*/ {1, -1},
    /*74 Ld2DTBF16*/ {0, 1}, /*75 St2DTBF16*/ {1, -1}, /*76 Ld2DTU8*/ {0, 1},
    /*77 Ld2DWF32*/ {0, 1}, /*78 St2DWF32*/ {1, -1}, /*79 Ld2DWF16*/ {0, 1}, /*80 St2DWF16*/ {1, -1},
    /*81 Ld2DWBF16*/ {0, 1}, /*82 St2DWBF16*/ {1, -1}, /*83 Ld2DWU8*/ {0, 1},
    /*84 AdvanceBlock2D*/ {0, 0}, /*85 AdvanceBase*/ {0, 0}, /*86 DupBroadcastW*/ {1, 1},
    /*87-94 FLoadReg0-7*/ {0, 1}, {0, 1}, {0, 1}, {0, 1}, {0, 1}, {0, 1}, {0, 1}, {0, 1},
    /*95-102 FStoreReg0-7*/ {1, -1}, {1, -1}, {1, -1}, {1, -1}, {1, -1}, {1, -1}, {1, -1}, {1, -1},
    /*103 FRcp*/ {1, 0}, /*104 FPermW*/ {1, 0}, /*105 FShuf2*/ {2, -1},
};

/* Static walk of a straight-line program; gint/host/analyzer.py:187-238. */
int gint_oracle_analyze(const int32_t *code, int n_words, oracle_stats *out)
{
    int depth = 0, max_d = 0, max_reg = -1, n = 0, min_pool = 0, mask = 0, halted = 0;
    if (!code || !out || n_words < 0 || (n_words & 1)) return ORACLE_ERR_BAD_ARG;
    memset(out, 0, sizeof(*out));
    out->error_index = -1;
    for (int i = 0; i + 1 < n_words; i += 2) {
        int op = code[i];
        if (op == 0) { halted = 1; break; }
        if (op < 0 || op >= N_OPCODES) { out->error_index = n; return ORACLE_ERR_UNKNOWN_OPCODE; }
        if (depth < EFFECTS[op][0]) { out->error_index = n; return ORACLE_ERR_STACK_UNDERFLOW; }
        if (op >= 87 && op <= 102) {
            int r = (op - 87) & 7;
            mask |= 1 << r;
            if (r > max_reg) max_reg = r;
        }
        int post = depth + EFFECTS[op][1];
        int peak = post > depth ? post : depth;
        if (peak > max_d) max_d = peak;
        if (peak + max_reg + 1 > min_pool) min_pool = peak + max_reg + 1;
        depth = post;
        n++;
    }
    out->num_instructions = n;
    out->max_stack = max_d;
    out->max_reg_idx = max_reg;
    out->min_pool_size = min_pool;
    out->regs_used_mask = mask;
    if (!halted) return ORACLE_ERR_NO_HALT;
    if (max_d > 8) return ORACLE_ERR_STACK_OVERFLOW;
    return ORACLE_OK;
}

/*
 * Pool geometry. The reference has two kernels: s7 (pool 7, 4 regs, stack 7) and l12 (pool 12, 8 regs,
 * stack 8), gint/kernel/interpreter/main.py:34-38, chosen by max stack depth and highest register index
 * separately (gint/host/executor.py:131-149). Register n is pool[P-1-n] (state.py:38-41), so the pool
 * size is observable only when stack and registers overlap. This build uses pools of 4, 7 or 12 slots:
 * the smallest with max_stack + (max_reg_idx + 1) <= P, else 12 (the reference's largest layout).
 */
int gint_oracle_pool_size(const oracle_stats *st)
{
    int need = st->max_stack + st->max_reg_idx + 1;
    if (need <= 4) return 4;
    if (need <= 7) return 7;
    return 12;
}

typedef union { float f; uint32_t u; int32_t i; } word_t;

static inline float bits_to_f(uint32_t u) { word_t w; w.u = u; return w.f; }
static inline uint32_t f_to_bits(float f) { word_t w; w.f = f; return w.u; }

static inline float half_to_f(uint16_t h) { _Float16 v; memcpy(&v, &h, 2); return (float)v; }
static inline uint16_t f_to_half(float f)
{
    if (f != f) return 0x7FFF; /* cvt.rn.f16.f32 canonical NaN */
    _Float16 v = (_Float16)f; uint16_t h; memcpy(&h, &v, 2); return h;
}
static inline float bf16_to_f(uint16_t h) { return bits_to_f((uint32_t)h << 16); }
static inline uint16_t f_to_bf16(float f)
{
    uint32_t u = f_to_bits(f);
    if (f != f) return 0x7FFF; /* cvt.rn.bf16.f32 canonical NaN */
    u += 0x7FFFu + ((u >> 16) & 1u); /* round to nearest even */
    return (uint16_t)(u >> 16);
}

/* llvm.maximum / llvm.minimum: NaN if either is NaN, -0 < +0 (nvptx.py:97-100) */
static inline float max_nan(float a, float b)
{
    if (a != a || b != b) return bits_to_f(0x7FFFFFFFu);
    if (a == 0.0f && b == 0.0f) return bits_to_f(f_to_bits(a) & f_to_bits(b));
    return a > b ? a : b;
}
static inline float min_nan(float a, float b)
{
    if (a != a || b != b) return bits_to_f(0x7FFFFFFFu);
    if (a == 0.0f && b == 0.0f) return bits_to_f(f_to_bits(a) | f_to_bits(b));
    return a < b ? a : b;
}

typedef float slot_t[WARP][REGW];

typedef struct {
    char *ptr[GINT_MAX_TENSORS];
    int32_t shape1[GINT_MAX_TENSORS], stride1[GINT_MAX_TENSORS];
    int32_t shape2[GINT_MAX_TENSORS], stride2[GINT_MAX_TENSORS];
    int32_t adv[GINT_MAX_TENSORS];
} block_info; /* BlockTensorInfo, load_tensor_infos.py:6-11 */

/* load_tensor_infos.py:23-46 -- all index arithmetic is 32-bit unsigned, the byte offset is 64-bit. */
static void decode_tensor_infos(const oracle_tensor_info *ti, int n_tensors, uint32_t bidx, block_info *bi)
{
    memset(bi, 0, sizeof(*bi));
    for (int t = 0; t < n_tensors && t < GINT_MAX_TENSORS; t++) {
        uint32_t r = bidx;
        uint32_t gd1 = (uint32_t)ti->block_grid_dims[t][0], gd2 = (uint32_t)ti->block_grid_dims[t][1];
        uint32_t st1 = (uint32_t)ti->block_grid_steps[t][0], st2 = (uint32_t)ti->block_grid_steps[t][1];
        uint32_t s1 = (uint32_t)ti->block_shape_stride_1[t][1], s2 = (uint32_t)ti->block_shape_stride_2[t][1];
        uint32_t b1 = gd1 ? r % gd1 : 0; r = gd1 ? r / gd1 : 0;
        uint32_t b2 = gd2 ? r % gd2 : 0; r = gd2 ? r / gd2 : 0;
        uint32_t off = b1 * st1 * s1 + b2 * st2 * s2;
        for (int j = 0; j < 4; j++) {
            uint32_t sz = (uint32_t)ti->batch_shape[t][j];
            uint32_t idx = sz ? r % sz : 0; r = sz ? r / sz : 0;
            off += (uint32_t)ti->batch_strides[t][j] * idx;
        }
        bi->ptr[t] = (char *)(intptr_t)ti->base_ptr[t] + (uint64_t)off * (uint64_t)(uint32_t)ti->elm_size[t];
        bi->shape1[t] = (int32_t)((uint32_t)ti->block_shape_stride_1[t][0] - b1 * st1);
        bi->stride1[t] = (int32_t)s1;
        bi->shape2[t] = (int32_t)((uint32_t)ti->block_shape_stride_2[t][0] - b2 * st2);
        bi->stride2[t] = (int32_t)s2;
        bi->adv[t] = 0;
    }
}

enum { DT_F32, DT_F16, DT_BF16, DT_U8 };
static const int DT_SIZE[4] = {4, 2, 2, 1};

static inline float mem_load(const char *p, int dt)
{
    switch (dt) {
    case DT_F32: { float v; memcpy(&v, p, 4); return v; }
    case DT_F16: { uint16_t h; memcpy(&h, p, 2); return half_to_f(h); }
    case DT_BF16: { uint16_t h; memcpy(&h, p, 2); return bf16_to_f(h); }
    default: return (float)*(const uint8_t *)p;
    }
}
static inline void mem_store(char *p, int dt, float v)
{
    switch (dt) {
    case DT_F32: memcpy(p, &v, 4); break;
    case DT_F16: { uint16_t h = f_to_half(v); memcpy(p, &h, 2); break; }
    case DT_BF16: { uint16_t h = f_to_bf16(v); memcpy(p, &h, 2); break; }
    default: break;
    }
}

/* layout: 0 = 1D, 1 = 2DT, 2 = 2DW.  load_store.py:76-158 */
static void tile_access(block_info *bi, int32_t operand, int layout, int dt, int is_store, slot_t v)
{
    int arg = operand & 0xf;
    int32_t off = (int32_t)((uint32_t)operand >> 4); /* lshr */
    int esz = DT_SIZE[dt];
    if (arg >= GINT_MAX_TENSORS) return;
    char *base = bi->ptr[arg];
    for (int lane = 0; lane < WARP; lane++) {
        for (int w = 0; w < REGW; w++) {
            int ok;
            int64_t idx;
            if (layout == 0) {
                int32_t e = lane + off + WARP * w;
                ok = e < bi->shape1[arg];
                idx = (int64_t)(int32_t)((uint32_t)(lane + off) * (uint32_t)bi->stride1[arg]) +
                      (int64_t)w * (int64_t)(int32_t)((uint32_t)bi->stride1[arg] * WARP);
            } else {
                int32_t t = layout == 1 ? lane + off : lane + bi->adv[arg];
                int32_t j0 = layout == 1 ? bi->adv[arg] : off;
                ok = t < bi->shape1[arg] && (j0 + w) < bi->shape2[arg];
                idx = (int64_t)(int32_t)((uint32_t)t * (uint32_t)bi->stride1[arg] + (uint32_t)j0 * (uint32_t)bi->stride2[arg]) +
                      (int64_t)w * (int64_t)bi->stride2[arg];
            }
            if (is_store) {
                if (ok) mem_store(base + idx * esz, dt, v[lane][w]);
            } else {
                v[lane][w] = ok ? mem_load(base + idx * esz, dt) : 0.0f;
            }
        }
    }
}

/* binary_cond_tree over 4 elements, move.py:58-66: (i < 2 ? (i < 1 ? v0 : v1) : (i < 3 ? v2 : v3)) */
static inline int tree_sel(int32_t i) { return i < 2 ? (i < 1 ? 0 : 1) : (i < 3 ? 2 : 3); }

static float special_unary(int op, float x)
{
    switch (op) {
    case 40: return sqrtf(x);
    case 41: return sinf(x);
    case 42: return cosf(x);
    case 43: return tanf(x);
    case 44: return asinf(x);
    case 45: return acosf(x);
    case 46: return atanf(x);
    case 49: return expf(x);
    case 50: return exp2f(x);
    case 51: return logf(x);
    case 52: return log2f(x);
    case 53: return 1.0f / sqrtf(x);
    case 54: return erff(x);
    }
    return x;
}

static inline int32_t int_binary(int op, int32_t t, int32_t s)
{
    uint32_t ut = (uint32_t)t, us = (uint32_t)s;
    switch (op) {
    case 56: return (int32_t)(ut + us);
    case 57: return (int32_t)(ut * us);
    case 58: return (int32_t)(ut - us);
    case 59: if (s == 0) return -1; if (t == INT32_MIN && s == -1) return INT32_MIN; return t / s;
    case 60: if (s == 0) return t; if (t == INT32_MIN && s == -1) return 0; return t % s;
    case 61: return us >= 32 ? 0 : (int32_t)(ut << us);
    case 62: return us >= 32 ? 0 : (int32_t)(ut >> us);
    case 63: return (int32_t)(ut & us);
    case 64: return (int32_t)(ut | us);
    case 65: return (int32_t)(ut ^ us);
    }
    return 0;
}

/* One logical program (= one warp of the reference kernel). */
static int run_program(const int32_t *code, int n_words, const oracle_tensor_info *ti, int n_tensors,
                       uint32_t bidx, int P)
{
    slot_t pool[MAX_POOL];
    slot_t tmp, tmp2;
    block_info bi;
    int sp = 0;
    memset(pool, 0, sizeof(pool));
    decode_tensor_infos(ti, n_tensors, bidx, &bi);

#define TOP(k) pool[sp - 1 - (k)]
#define FOR_LW for (int l = 0; l < WARP; l++) for (int w = 0; w < REGW; w++)
#define BINARY(expr) do { FOR_LW { float T = TOP(0)[l][w], S = TOP(1)[l][w]; (void)T; (void)S; tmp[l][w] = (expr); } \
                          sp -= 1; memcpy(TOP(0), tmp, sizeof(slot_t)); } while (0)
#define UNARY(expr) do { FOR_LW { float T = TOP(0)[l][w]; TOP(0)[l][w] = (expr); } } while (0)

    for (int pc = 0; pc + 1 < n_words; pc += 2) {
        int op = code[pc];
        int32_t operand = code[pc + 1];
        if (op < 0 || op >= N_OPCODES) return ORACLE_ERR_UNKNOWN_OPCODE;
        if (sp < EFFECTS[op][0]) return ORACLE_ERR_STACK_UNDERFLOW;
        if (sp + EFFECTS[op][1] > P || (op == 27 && sp + 2 > P)) return ORACLE_ERR_STACK_OVERFLOW;
        switch (op) {
        case 0: return ORACLE_OK;
        case 1: break;
        case 2: BINARY(T + S); break;
        case 3: BINARY(T * S); break;
        case 4: /* FMA: fma(T, S, U), pops 3; arith.py:27-30 */
            FOR_LW tmp[l][w] = fmaf(TOP(0)[l][w], TOP(1)[l][w], TOP(2)[l][w]);
            sp -= 2; memcpy(TOP(0), tmp, sizeof(slot_t));
            break;
        case 5: BINARY(T - S); break;
        case 6: BINARY(S - T); break;
        case 7: UNARY(-T); break;
        case 8: BINARY(T / S); break;
        case 9: BINARY(S / T); break;
        case 10: BINARY(fmodf(T, S)); break;
        case 11: FOR_LW pool[sp][l][w] = bits_to_f((uint32_t)operand); sp++; break;
        case 12: { float imm = bits_to_f((uint32_t)operand); UNARY(T + imm); break; }
        case 13: { float imm = bits_to_f((uint32_t)operand); UNARY(T * imm); break; }
        case 14: { /* f16x2: low half = mul, high half = add; immediate.py:29-36 */
            float mul = half_to_f((uint16_t)((uint32_t)operand & 0xFFFF)), add = half_to_f((uint16_t)((uint32_t)operand >> 16));
            UNARY(fmaf(T, mul, add));
            break;
        }
        case 15: tile_access(&bi, operand, 0, DT_F32, 0, pool[sp]); sp++; break;
        case 16: tile_access(&bi, operand, 0, DT_F32, 1, TOP(0)); sp--; break;
        case 17: tile_access(&bi, operand, 0, DT_F16, 0, pool[sp]); sp++; break;
        case 18: tile_access(&bi, operand, 0, DT_F16, 1, TOP(0)); sp--; break;
        case 19: tile_access(&bi, operand, 0, DT_BF16, 0, pool[sp]); sp++; break;
        case 20: tile_access(&bi, operand, 0, DT_BF16, 1, TOP(0)); sp--; break;
        case 21: tile_access(&bi, operand, 0, DT_U8, 0, pool[sp]); sp++; break;
        case 22: sp -= 1; break;
        case 23: sp -= 2; break;
        case 24: memcpy(pool[sp], TOP(0), sizeof(slot_t)); sp++; break;
        case 25: /* DupX1 [a,b] -> [b,a,b] */
            memcpy(tmp, TOP(0), sizeof(slot_t)); memcpy(tmp2, TOP(1), sizeof(slot_t));
            memcpy(pool[sp - 2], tmp, sizeof(slot_t)); memcpy(pool[sp - 1], tmp2, sizeof(slot_t)); memcpy(pool[sp], tmp, sizeof(slot_t));
            sp++;
            break;
        case 26: { /* DupX2 [a,b,c] -> [c,a,b,c] */
            slot_t v3;
            memcpy(tmp, TOP(0), sizeof(slot_t)); memcpy(tmp2, TOP(1), sizeof(slot_t)); memcpy(v3, TOP(2), sizeof(slot_t));
            memcpy(pool[sp - 3], tmp, sizeof(slot_t)); memcpy(pool[sp - 2], v3, sizeof(slot_t));
            memcpy(pool[sp - 1], tmp2, sizeof(slot_t)); memcpy(pool[sp], tmp, sizeof(slot_t));
            sp++;
            break;
        }
        case 27: /* Dup2 [a,b] -> [a,b,a,b] */
            memcpy(pool[sp], TOP(1), sizeof(slot_t)); memcpy(pool[sp + 1], TOP(0), sizeof(slot_t)); sp += 2;
            break;
        case 28: BINARY(T > S ? 1.0f : 0.0f); break;
        case 29: BINARY(T < S ? 1.0f : 0.0f); break;
        case 30: BINARY(T >= S ? 1.0f : 0.0f); break;
        case 31: BINARY(T <= S ? 1.0f : 0.0f); break;
        case 32: BINARY(T == S ? 1.0f : 0.0f); break;
        case 33: BINARY(T != S ? 1.0f : 0.0f); break; /* unordered: true on NaN */
        case 34: { float eps = bits_to_f((uint32_t)operand); BINARY(fabsf(T - S) < eps ? 1.0f : 0.0f); break; }
        case 35: /* Select: T > 0 ? S : U, pops 3; predication.py:64-73 */
            FOR_LW tmp[l][w] = TOP(0)[l][w] > 0.0f ? TOP(1)[l][w] : TOP(2)[l][w];
            sp -= 2; memcpy(TOP(0), tmp, sizeof(slot_t));
            break;
        case 36: case 37: case 38: case 39:
            for (int w = 0; w < REGW; w++) {
                float red[WARP], nxt[WARP];
                for (int l = 0; l < WARP; l++) red[l] = TOP(0)[l][w];
                for (int mask = 16; mask >= 1; mask >>= 1) {
                    for (int l = 0; l < WARP; l++) {
                        float a = red[l], b = red[l ^ mask];
                        nxt[l] = op == 36 ? a + b : op == 37 ? max_nan(a, b) : op == 38 ? min_nan(a, b) : a * b;
                    }
                    memcpy(red, nxt, sizeof(red));
                }
                for (int l = 0; l < WARP; l++) TOP(0)[l][w] = red[l];
            }
            break;
        case 40: case 41: case 42: case 43: case 44: case 45: case 46:
        case 49: case 50: case 51: case 52: case 53: case 54:
            UNARY(special_unary(op, T));
            break;
        case 47: BINARY(atan2f(T, S)); break;
        case 48: BINARY(powf(T, S)); break;
        case 55: memcpy(tmp, TOP(0), sizeof(slot_t)); memcpy(TOP(0), TOP(1), sizeof(slot_t)); memcpy(TOP(1), tmp, sizeof(slot_t)); break;
        case 56: case 57: case 58: case 59: case 60: case 61: case 62: case 63: case 64: case 65:
            BINARY(bits_to_f((uint32_t)int_binary(op, (int32_t)f_to_bits(T), (int32_t)f_to_bits(S))));
            break;
        case 66: case 67: { /* gather / scatter, load_store.py:266-288 */
            int arg = operand & 0xf;
            if (arg < GINT_MAX_TENSORS) {
                for (int l = 0; l < WARP; l++) for (int w = 0; w < REGW; w++) {
                    int32_t idx = (int32_t)f_to_bits(TOP(0)[l][w]);
                    int ok = idx < bi.shape1[arg];
                    char *p = bi.ptr[arg] + (int64_t)(int32_t)((uint32_t)idx * (uint32_t)bi.stride1[arg]) * 4;
                    if (op == 66) tmp[l][w] = ok ? mem_load(p, DT_F32) : 0.0f;
                    else if (ok) mem_store(p, DT_F32, TOP(1)[l][w]);
                }
            }
            if (op == 66) memcpy(TOP(0), tmp, sizeof(slot_t)); else sp -= 2;
            break;
        }
        case 68: FOR_LW pool[sp][l][w] = (float)(int8_t)((uint32_t)operand >> (8 * w)); sp++; break;
        case 69: FOR_LW pool[sp][l][w] = bits_to_f((uint32_t)(int32_t)(int8_t)((uint32_t)operand >> (8 * w))); sp++; break;
        case 70: tile_access(&bi, operand, 1, DT_F32, 0, pool[sp]); sp++; break;
        case 71: tile_access(&bi, operand, 1, DT_F32, 1, TOP(0)); sp--; break;
        case 72: tile_access(&bi, operand, 1, DT_F16, 0, pool[sp]); sp++; break;
        case 73: tile_access(&bi, operand, 1, DT_F16, 1, TOP(0)); sp--; break;
        case 74: tile_access(&bi, operand, 1, DT_BF16, 0, pool[sp]); sp++; break;
        case 75: tile_access(&bi, operand, 1, DT_BF16, 1, TOP(0)); sp--; break;
        case 76: tile_access(&bi, operand, 1, DT_U8, 0, pool[sp]); sp++; break;
        case 77: tile_access(&bi, operand, 2, DT_F32, 0, pool[sp]); sp++; break;
        case 78: tile_access(&bi, operand, 2, DT_F32, 1, TOP(0)); sp--; break;
        case 79: tile_access(&bi, operand, 2, DT_F16, 0, pool[sp]); sp++; break;
        case 80: tile_access(&bi, operand, 2, DT_F16, 1, TOP(0)); sp--; break;
        case 81: tile_access(&bi, operand, 2, DT_BF16, 0, pool[sp]); sp++; break;
        case 82: tile_access(&bi, operand, 2, DT_BF16, 1, TOP(0)); sp--; break;
        case 83: tile_access(&bi, operand, 2, DT_U8, 0, pool[sp]); sp++; break;
        case 84: if ((operand & 0xf) < GINT_MAX_TENSORS) bi.adv[operand & 0xf] += operand >> 4; break;       /* ashr */
        case 85: if ((operand & 0xf) < GINT_MAX_TENSORS) bi.ptr[operand & 0xf] += (int64_t)(operand >> 4); break; /* bytes */
        case 86: { int k = tree_sel(operand); FOR_LW pool[sp][l][w] = TOP(0)[l][k]; sp++; break; }
        case 87: case 88: case 89: case 90: case 91: case 92: case 93: case 94: {
            int k = P - 1 - (op - 87);
            if (k < 0) return ORACLE_ERR_BAD_ARG;
            memcpy(tmp, pool[k], sizeof(slot_t)); memcpy(pool[sp], tmp, sizeof(slot_t)); sp++;
            break;
        }
        case 95: case 96: case 97: case 98: case 99: case 100: case 101: case 102: {
            int k = P - 1 - (op - 95);
            if (k < 0) return ORACLE_ERR_BAD_ARG;
            memcpy(tmp, TOP(0), sizeof(slot_t)); sp--; memcpy(pool[k], tmp, sizeof(slot_t));
            break;
        }
        case 103: UNARY(1.0f / T); break;
        case 104: /* FPermW: out[w] = T[idx_w]; move.py:77-104 */
            FOR_LW tmp[l][w] = TOP(0)[l][tree_sel((int32_t)(((uint32_t)operand >> (8 * w)) & 0xFF))];
            memcpy(TOP(0), tmp, sizeof(slot_t));
            break;
        case 105: /* FShuf2: vec2 = T, vec1 = S -> (vec1[x], vec1[y], vec2[z], vec2[w]); move.py:107-135 */
            FOR_LW {
                int k = tree_sel((int32_t)(((uint32_t)operand >> (8 * w)) & 0xFF));
                tmp[l][w] = w < 2 ? TOP(1)[l][k] : TOP(0)[l][k];
            }
            sp -= 1; memcpy(TOP(0), tmp, sizeof(slot_t));
            break;
        }
    }
    return ORACLE_ERR_NO_HALT;
}

/*
 * Execute `grid_dim` logical programs on HOST memory (descriptor base pointers are host addresses).
 * pool_size: 4, 7, 12, or 0 to choose by gint_oracle_pool_size().
 * n_threads > 1 splits the logical programs into contiguous ranges, one pthread each; programs whose warps
 * race on memory then race here too.
 */
typedef struct {
    const int32_t *code; int n_words; const oracle_tensor_info *ti; int n_tensors;
    uint32_t lo, hi; int P; int rc;
} job_t;

static void *job_main(void *arg)
{
    job_t *j = (job_t *)arg;
    for (uint32_t b = j->lo; b < j->hi; b++) {
        int r = run_program(j->code, j->n_words, j->ti, j->n_tensors, b, j->P);
        if (r != ORACLE_OK) j->rc = r;
    }
    return NULL;
}

int gint_oracle_execute_range(const int32_t *code, int n_words, const oracle_tensor_info *ti, int n_tensors,
                              uint32_t first, uint32_t count, int pool_size, int n_threads);

int gint_oracle_execute(const int32_t *code, int n_words, const oracle_tensor_info *ti, int n_tensors,
                        uint32_t grid_dim, int pool_size, int n_threads)
{
    return gint_oracle_execute_range(code, n_words, ti, n_tensors, 0u, grid_dim, pool_size, n_threads);
}

/* Logical programs [first, first + count) only: what one rank of a sharded launch executes. */
int gint_oracle_execute_range(const int32_t *code, int n_words, const oracle_tensor_info *ti, int n_tensors,
                              uint32_t first, uint32_t count, int pool_size, int n_threads)
{
    const uint32_t grid_dim = count;
    oracle_stats st;
    int rc = gint_oracle_analyze(code, n_words, &st);
    if (rc != ORACLE_OK) return rc;
    if (n_tensors < 0 || n_tensors > GINT_MAX_TENSORS) return ORACLE_ERR_BAD_ARG;
    int P = pool_size ? pool_size : gint_oracle_pool_size(&st);
    if (P < 1 || P > MAX_POOL) return ORACLE_ERR_BAD_ARG;
    if (n_threads < 1) n_threads = 1;
    if (n_threads > 64) n_threads = 64;
    if ((uint32_t)n_threads > grid_dim) n_threads = grid_dim ? (int)grid_dim : 1;
    job_t jobs[64];
    pthread_t th[64];
    uint32_t chunk = (grid_dim + (uint32_t)n_threads - 1) / (uint32_t)n_threads;
    for (int t = 0; t < n_threads; t++) {
        uint32_t lo = (uint32_t)t * chunk, hi = lo + chunk;
        if (lo > grid_dim) lo = grid_dim;
        if (hi > grid_dim) hi = grid_dim;
        jobs[t] = (job_t){code, n_words, ti, n_tensors, first + lo, first + hi, P, ORACLE_OK};
    }
    if (n_threads == 1) {
        job_main(&jobs[0]);
        return jobs[0].rc;
    }
    for (int t = 0; t < n_threads; t++)
        if (pthread_create(&th[t], NULL, job_main, &jobs[t]) != 0) { job_main(&jobs[t]); th[t] = 0; }
    int err = ORACLE_OK;
    for (int t = 0; t < n_threads; t++) {
        if (th[t]) pthread_join(th[t], NULL);
        if (jobs[t].rc != ORACLE_OK) err = jobs[t].rc;
    }
    return err;
}

/*
 * Indirect mode (flag > 0 in the reference kernel, main.py:179-194): logical program i runs
 * codes[i] with descriptors tis[i]; `n_tensors` is the maximum over the batch (executor_impl.py:192).
 */
int gint_oracle_execute_indirect(const int32_t *const *codes, const int32_t *n_words, const oracle_tensor_info *const *tis,
                                 int n_tensors, uint32_t grid_dim, int pool_size)
{
    for (uint32_t b = 0; b < grid_dim; b++) {
        oracle_stats st;
        int rc = gint_oracle_analyze(codes[b], n_words[b], &st);
        if (rc != ORACLE_OK) return rc;
        rc = run_program(codes[b], n_words[b], tis[b], n_tensors, b, pool_size ? pool_size : 12);
        if (rc != ORACLE_OK) return rc;
    }
    return ORACLE_OK;
}

int gint_oracle_sizeof_tensor_info(void) { return (int)sizeof(oracle_tensor_info); }
