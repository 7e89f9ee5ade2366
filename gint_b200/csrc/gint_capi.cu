/*
 * gint_capi.cu -- host side of libgint_b200.so: program analysis and pre-decoding, the per-device context,
 * and the launch entry points declared in include/gint_b200.h.
 *
 * It replaces the reference's Python executor (gint/host/cuda/executor_impl.py, gint/host/cuda/driver.py):
 * instead of a device-side descriptor buffer refreshed by a 608-byte host-to-device copy before every launch
 * (executor_impl.py:66-72), descriptors travel as kernel parameters, so a launch is a single cudaLaunchKernel
 * with no allocation and no copy and every captured launch in a CUDA graph is self-contained.
 */
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <mutex>
#include <string>
#include <atomic>
#include <array>
#include <map>
#include <vector>

#include "../../include/gint_b200.h"
#include "gint_fused.h"
#include "gint_opcodes.h"
#include "gint_types.h"
#include "gint_variants.h"

using gint::IndirectArgs;
using gint::IndirectEntry;
using gint::LaunchArgs;

namespace {

struct OpEffect { int8_t min_depth, net; };
const OpEffect kEffects[GINT_FUSED_FIRST] = {     // the format's opcodes, then the internal ones (numbered consecutively)
#define GINT_X_EFF(name, num, md, net) {md, net},
    GINT_OPCODE_LIST(GINT_X_EFF)
    GINT_INTERNAL_OPCODE_LIST(GINT_X_EFF)
#undef GINT_X_EFF
};
static_assert(sizeof(kEffects) / sizeof(kEffects[0]) == GINT_FUSED_FIRST, "internal opcodes must be numbered consecutively up to the fused handlers");

bool is_tensor_op(int op)
{
    return (op >= OP_LoadGlobal1DF32 && op <= OP_LoadGlobal1DU8) || op == OP_LoadGlobal1DF32Indirect ||
           op == OP_StoreGlobal1DF32Indirect || (op >= OP_LoadGlobal2DTF32 && op <= OP_AdvanceBase);
}

/* Static walk (gint/host/analyzer.py:187-238) + pool geometry choice (replaces gint/host/executor.py:131-149). */
int analyze(const int32_t *code, int n_words, gint_bytecode_stats *st)
{
    if (!code || !st || n_words < 0 || (n_words & 1)) return GINT_ERR_INVALID_ARGUMENT;
    memset(st, 0, sizeof(*st));
    st->error_index = -1;
    st->max_reg_idx = -1;
    int depth = 0, n = 0;
    bool halted = false;
    for (int i = 0; i + 1 < n_words; i += 2) {
        const int op = code[i];
        if (op == OP_Halt) { halted = true; break; }
        if (op < 0 || op >= GINT_N_OPCODES) { st->error_index = n; return GINT_ERR_UNKNOWN_OPCODE; }
        if (depth < kEffects[op].min_depth) { st->error_index = n; return GINT_ERR_STACK_UNDERFLOW; }
        if (op >= OP_FLoadReg0 && op <= OP_FStoreReg7) {
            const int r = (op - OP_FLoadReg0) & 7;
            st->regs_used_mask |= 1 << r;
            if (r > st->max_reg_idx) st->max_reg_idx = r;
        }
        const int post = depth + kEffects[op].net;
        const int peak = post > depth ? post : depth;
        if (peak > GINT_MAX_STACK) { st->error_index = n; return GINT_ERR_STACK_OVERFLOW; }
        if (peak > st->max_stack) st->max_stack = peak;
        if (peak + st->max_reg_idx + 1 > st->min_pool_size) st->min_pool_size = peak + st->max_reg_idx + 1;
        depth = post;
        n++;
    }
    st->num_instructions = n;
    if (!halted) { st->error_index = n; return GINT_ERR_NO_HALT; }
    /* Register n lives in pool[P-1-n] (gint/kernel/interpreter/state.py:38-41), so P is observable only if stack
     * and registers overlap. Smallest pool that keeps them apart; otherwise the reference's largest layout. */
    const int need = st->max_stack + st->max_reg_idx + 1;
    st->pool_size = need <= 4 ? 4 : need <= 7 ? 7 : 12;
    return GINT_OK;
}

uint32_t clamp_lane_bytes(uint32_t operand)
{
    uint32_t r = 0;
    for (int w = 0; w < 4; w++) {
        uint32_t b = (operand >> (8 * w)) & 0xFFu;
        r |= (b > 3u ? 3u : b) << (8 * w);
    }
    return r;
}

/* One instruction of the normalised program: opcode (format or internal), operand as the kernel wants it. */
struct Insn { int op; uint32_t operand; };

/* Validate and normalise: width-lane selectors are clamped to 0..3, which is what the reference's compare tree computes for
 * any operand (gint/kernel/interpreter/instructions/move.py:58-66). The list ends with the Halt. */
int normalise(const int32_t *code, int n_words, int n_tensors, std::vector<Insn> *out)
{
    gint_bytecode_stats st;
    int rc = analyze(code, n_words, &st);
    if (rc != GINT_OK) return rc;
    out->clear();
    for (int i = 0; i < st.num_instructions; i++) {
        const int op = code[2 * i];
        uint32_t operand = (uint32_t)code[2 * i + 1];
        if (is_tensor_op(op) && (int)(operand & 15u) >= n_tensors) return GINT_ERR_INVALID_ARGUMENT;
        if (op == OP_DupBroadcastW) {
            const int32_t s = (int32_t)operand;
            operand = s < 0 ? 0u : s > 3 ? 3u : (uint32_t)s;
        } else if (op == OP_FPermW || op == OP_FShuf2) {
            operand = clamp_lane_bytes(operand);
        }
        out->push_back(Insn{op, operand});
    }
    out->push_back(Insn{OP_Halt, 0u});
    return GINT_OK;
}

struct FusedDef { int num, len; int ops[GINT_MAX_FUSED_LEN]; };
const FusedDef kFused[GINT_N_FUSED + GINT_N_RF_FUSED] = {   // the ordinary fused handlers, then the register-operand forms (RF streams only)
#define GINT_X_FDEF(num, len, ...) {num, len, {__VA_ARGS__}},
    GINT_FUSED_LIST(GINT_X_FDEF)
    GINT_RF_FUSED_LIST(GINT_X_FDEF)
#undef GINT_X_FDEF
};
const FusedDef &fused_def(int op)
{
    return kFused[op >= GINT_RF_FUSED_FIRST ? GINT_N_FUSED + (op - GINT_RF_FUSED_FIRST) : op - GINT_FUSED_FIRST];
}
constexpr int OP_CARRIER = -1;        // an instruction absorbed into the fused handler before it: only its operand is used
constexpr int OP_CARRIER_UNUSED = -2; // the same, for a member that reads no operand: it gets no stream entry

int net_effect(int op)
{
    if (op == OP_CARRIER || op == OP_CARRIER_UNUSED) return 0;
    if (GINT_IS_FUSED(op)) {
        int net = 0;
        const FusedDef &f = fused_def(op);
        for (int j = 0; j < f.len; j++) net += net_effect(f.ops[j]);
        return net;
    }
    if (op == OP_RLoad || op == OP_RLoadP || op == OP_RLoadS) return 1;
    if (op == OP_RStore) return -1;
    if (op == OP_RemapVN) return 0;
    return kEffects[op].net;
}

/* Replace known instruction sequences by fused handlers (gint_fused.h): greedy, longest match first. The absorbed
 * instructions stay in the stream as operand carriers. */
void fuse_sequences(std::vector<Insn> *prog, bool rf = false)
{
    std::vector<Insn> &p = *prog;
    const int n_defs = rf ? GINT_N_FUSED + GINT_N_RF_FUSED : GINT_N_FUSED;   // the register-operand forms: RF streams only
    for (size_t i = 0; i < p.size();) {
        int best = -1;
        for (int k = 0; k < n_defs; k++) {
            const FusedDef &f = kFused[k];
            if (i + (size_t)f.len > p.size() || (best >= 0 && f.len <= kFused[best].len)) continue;
            bool match = true;
            for (int j = 0; j < f.len && match; j++) match = p[i + (size_t)j].op == f.ops[j];
            if (match) best = k;
        }
        if (best < 0) { i++; continue; }
        p[i].op = kFused[best].num;
        for (int j = 1; j < kFused[best].len; j++)
            p[i + (size_t)j].op = GINT_OP_USES_OPERAND(kFused[best].ops[j]) ? OP_CARRIER : OP_CARRIER_UNUSED;
        i += (size_t)kFused[best].len;
    }
}

/* Stream layout, skewed for threaded dispatch: entry 0 = {0, opcode of insn 0}; entry i+1 = {operand of insn i, opcode of
 * insn i+1}; the opcode after the final Halt is Halt again. The stack depth before every instruction is static
 * (straight-line code) and is baked into the handlers, not the stream. Members of a fused sequence that read no operand
 * get no entry. */
void emit_stream(const std::vector<Insn> &full, std::vector<uint2> *out, std::vector<int> *depth_out = nullptr)
{
    std::vector<Insn> prog;
    prog.reserve(full.size());
    for (const Insn &in : full)
        if (in.op != OP_CARRIER_UNUSED) prog.push_back(in);
    const size_t n = prog.size();
    out->clear();
    out->reserve(n + 4);
    out->push_back(make_uint2(0u, (uint32_t)prog[0].op));
    for (size_t i = 0; i < n; i++) {
        const int next = i + 1 < n ? prog[i + 1].op : OP_Halt;
        out->push_back(make_uint2(prog[i].operand, next == OP_CARRIER ? (uint32_t)OP_Halt : (uint32_t)next));
    }
    out->push_back(make_uint2(0u, OP_Halt));  // handlers fetch one entry ahead
    if (out->size() & 1) out->push_back(make_uint2(0u, OP_Halt));
    if (depth_out) {
        depth_out->assign(n, 0);
        int depth = 0;
        for (size_t i = 0; i < n; i++) { (*depth_out)[i] = depth; depth += net_effect(prog[i].op); }
    }
}

int predecode(const int32_t *code, int n_words, int n_tensors, std::vector<uint2> *out, std::vector<int> *depth_out = nullptr)
{
    std::vector<Insn> prog;
    int rc = normalise(code, n_words, n_tensors, &prog);
    if (rc != GINT_OK) return rc;
    emit_stream(prog, out, depth_out);
    return GINT_OK;
}

bool writes_tensor(int op)
{
    return op == OP_StoreGlobal1DF32 || op == OP_StoreGlobal1DF16 || op == OP_StoreGlobal1DBF16 || op == OP_StoreGlobal1DF32Indirect ||
           op == OP_StoreGlobal2DTF32 || op == OP_StoreGlobal2DTF16 || op == OP_StoreGlobal2DTBF16 || op == OP_StoreGlobal2DWF32 ||
           op == OP_StoreGlobal2DWF16 || op == OP_StoreGlobal2DWBF16 || op == OP_StoreGlobal1DF32Fast || op == OP_StoreGlobal2DWF32Fast;
}

/*
 * Early-issue transformation. The interpreter consumes every loaded value in the next instruction or two, so as written
 * a program keeps one tile load per logical program in flight and waits out the full memory latency each time. The
 * bytecode is straight-line, though: which tiles it will load, and in which order, is known here. Eligible loads
 * (f32, 1-D layout) are numbered 0, 1, 2, ... in program order; load n is STARTED where load n-D is consumed (the
 * first D in a prologue) into staging slot n mod D of the warp's ring in shared memory, and at its original place only a
 * read of that slot remains
 * (PfTake / PfTakeIssue, gint_opcodes.h). A load keeps its place when starting it early could change what it reads:
 *   - a store or scatter to the SAME tensor slot, or an AdvanceBlock2D / AdvanceBase on it, lies in between (checked here);
 *   - a store to ANOTHER slot lies in between and the two tensors overlap in memory: that depends on the base pointers
 *     of the launch, so the pairs (loaded slot, stored slot) are recorded and checked against address ranges at launch
 *     time (launch_direct); on any overlap the untransformed stream runs instead.
 * Also folded here: a load that immediately repeats the previous instruction's load becomes Dup.
 */
/* Ring depth for a program: the deep ring pays for programs that stream long rows -- at least 48 1-D loads and at least 2
 * of 5 instructions accessing memory (measured on RMSNorm rows of 4096: 110 us with 8 slots at 5 blocks per SM against
 * 121 us with 4 slots at 6) -- and costs the others occupancy through its shared memory (the conductor graph's 1024-wide
 * rows, two tiles per warp: 344 us with 8 slots against 332 us with 4). */
int choose_ring_slots(const std::vector<Insn> &prog)
{
    int n_loads = 0, n_mem = 0;
    for (const Insn &in : prog) {
        n_loads += in.op == OP_LoadGlobal1DF32;
        n_mem += is_tensor_op(in.op) && in.op != OP_AdvanceBlock2D && in.op != OP_AdvanceBase;
    }
    return n_loads >= 48 && 5 * n_mem >= 2 * (int)prog.size() ? gint::kRingSlotsDeep : gint::kRingSlotsShallow;
}

struct EarlyIssue {
    std::vector<Insn> prog;
    uint8_t alias_slots[GINT_MAX_TENSORS] = {};   // bit b of [a]: loads of slot a were moved across stores to slot b
    int n_early = 0;
};

void early_issue_transform(const std::vector<Insn> &in, int D, EarlyIssue *out)
{
    std::vector<Insn> prog = in;
    for (size_t i = 1; i < prog.size(); i++) {
        const int op = prog[i].op;
        const bool is_load = (op >= OP_LoadGlobal1DF32 && op <= OP_LoadGlobal1DU8 && !writes_tensor(op)) ||
                             (op >= OP_LoadGlobal2DTF32 && op <= OP_LoadGlobal2DWU8 && !writes_tensor(op));
        if (is_load && prog[i - 1].op == op && prog[i - 1].operand == prog[i].operand) prog[i] = Insn{OP_Dup, 0u};
    }
    struct Member { size_t site; uint32_t operand; };
    std::vector<Member> ring;
    for (size_t i = 0; i < prog.size(); i++) {
        const int op = prog[i].op;
        /* 1-D tile loads only: for 2DW rows (one 16-byte access per thread, mostly L1 hits) the staging round trip costs
         * more than it hides (measured on the batched 4x4 programs) */
        if (op != OP_LoadGlobal1DF32) continue;
        const int slot = (int)(prog[i].operand & 15u);
        const size_t n = ring.size();
        const size_t from = n >= (size_t)D ? ring[n - (size_t)D].site + 1 : 0;   // first instruction the load would move across
        bool hazard = false;
        for (size_t j = from; j < i && !hazard; j++) {
            const int oj = prog[j].op;
            const int sj = (int)(prog[j].operand & 15u);
            if ((writes_tensor(oj) || oj == OP_AdvanceBlock2D || oj == OP_AdvanceBase) && sj == slot) hazard = true;
        }
        if (hazard) continue;
        for (size_t j = from; j < i; j++)
            if (writes_tensor(prog[j].op)) out->alias_slots[slot] |= (uint8_t)(1u << (prog[j].operand & 7u));
        ring.push_back(Member{i, prog[i].operand});
    }
    out->n_early = (int)ring.size();
    out->prog.clear();
    if (ring.empty()) { out->prog = prog; return; }
    const size_t R = ring.size();
    for (size_t n = 0; n < (size_t)D && n < R; n++) out->prog.push_back(Insn{OP_PfIssue1D, ring[n].operand});   // prologue: fill the ring
    if (R < (size_t)D) out->prog.push_back(Insn{OP_PfSkip, (uint32_t)((size_t)D - R)});   // ... and step over the unused slots, back to slot 0
    size_t next = 0;
    for (size_t i = 0; i < prog.size(); i++) {
        if (next < R && ring[next].site == i) {
            if (next + (size_t)D < R) {
                const Member &f = ring[next + (size_t)D];
                out->prog.push_back(Insn{OP_PfTakeIssue1D, f.operand});
            } else {
                out->prog.push_back(Insn{OP_PfTake, 0u});
            }
            next++;
        } else {
            out->prog.push_back(prog[i]);
        }
    }
}

/*
 * Fast accesses. A 1-D f32 access can skip all shape, stride and mask handling when, for every logical program of the
 * grid, it covers a full unit-stride tile whose first byte is 16-byte aligned. With the descriptors of program creation
 * this is decidable up to the alignment of the base pointer: the tile's first element is at
 *   base + (b1*grid_step1*stride1 + b2*grid_step2*stride2 + sum(batch_index*batch_stride) + off) * 4
 * and its extent along dimension 1 is shape1 - b1*grid_step1 (descriptor decode, gint_interp.cuh: decode_tiles), so it is
 * enough that every step that can be non-zero is a multiple of 4 elements, that off is, and that off + 128 fits the
 * smallest extent. Slots that the program moves (AdvanceBase / AdvanceBlock2D) are left alone. The slots that fast
 * accesses rely on are returned as a mask; a launch whose base pointer for one of them is not 16-byte aligned runs the
 * plain stream instead.
 */
uint32_t apply_fast_accesses(std::vector<Insn> *prog, const gint_tensor_info &ti, int n_tensors)
{
    bool ok[GINT_MAX_TENSORS];
    int64_t min_extent[GINT_MAX_TENSORS];
    for (int t = 0; t < GINT_MAX_TENSORS; t++) {
        ok[t] = false;
        min_extent[t] = 0;
        if (t >= n_tensors) continue;
        const int64_t shape1 = ti.block_shape_stride_1[t][0], stride1 = ti.block_shape_stride_1[t][1];
        const int64_t stride2 = ti.block_shape_stride_2[t][1];
        const int64_t gd1 = (uint32_t)ti.block_grid_dims[t][0], gd2 = (uint32_t)ti.block_grid_dims[t][1];
        const int64_t gs1 = ti.block_grid_steps[t][0], gs2 = ti.block_grid_steps[t][1];
        bool good = ti.elm_size[t] == 4 && stride1 == 1 && gd1 >= 1 && gd2 >= 1 && gs1 >= 0;
        if (good && gd1 != 1 && (gs1 * stride1) % 4 != 0) good = false;
        if (good && gd2 != 1 && (gs2 * stride2) % 4 != 0) good = false;
        for (int j = 0; good && j < 4; j++)
            if (ti.batch_shape[t][j] != 1 && ti.batch_strides[t][j] % 4 != 0) good = false;
        ok[t] = good;
        min_extent[t] = shape1 - (gd1 - 1) * gs1;
    }
    for (const Insn &in : *prog)
        if (in.op == OP_AdvanceBlock2D || in.op == OP_AdvanceBase) ok[in.operand & 7u] = false;
    uint32_t used = 0;
    for (Insn &in : *prog) {
        int fast;
        switch (in.op) {
        case OP_LoadGlobal1DF32: fast = OP_LoadGlobal1DF32Fast; break;
        case OP_StoreGlobal1DF32: fast = OP_StoreGlobal1DF32Fast; break;
        case OP_PfIssue1D: fast = OP_PfIssue1DFast; break;
        case OP_PfTakeIssue1D: fast = OP_PfTakeIssue1DFast; break;
        default: continue;
        }
        const int slot = (int)(in.operand & 15u);
        const int64_t off = (int64_t)(in.operand >> 4);
        if (slot >= n_tensors || slot >= 8 || !ok[slot] || (off & 3) != 0 || off + 128 > min_extent[slot] || off * 4 >= (1 << 26)) continue;
        in.op = fast;
        in.operand = ((uint32_t)slot << 29) | (uint32_t)(off * 4);   // {8 * slot, byte offset}: see fast_tile_address in gint_interp.cuh
        used |= 1u << slot;
    }
    return used;
}

/*
 * Staged row blocks. In the small-matrix programs one lane owns one matrix: a 2DW row load is a 16-byte access per lane at
 * the row stride (64 bytes for a 4x4 matrix), which costs 16 L1 wavefronts per warp request where 512 contiguous bytes
 * cost 4, and the rows of an operand are loaded again for every output row. When a tensor slot is only read, only through
 * LoadGlobal2DWF32, and its 32 rows per logical program are R = 4, 8 or 16 floats long and lie back to back (row stride R,
 * unit column stride, always 32 valid rows, 16-byte aligned given an aligned base pointer), the whole 32 x R block is
 * copied into shared memory once, at the start of the program, with fully coalesced copies (StageRows) and every row load
 * reads from there (LoadStagedRows, one conflict-free 16-byte shared-memory access per lane). Returns the slots staged;
 * *area_bytes receives the shared memory needed per tile. Loads of those slots now happen before every store of the
 * program, so the stored slots are recorded as alias partners (checked against the launch's address ranges).
 */
uint32_t apply_row_staging(std::vector<Insn> *prog, const gint_tensor_info &ti, int n_tensors, uint32_t *area_bytes, uint8_t *alias_slots)
{
    *area_bytes = 0;
    int lq_of[GINT_MAX_TENSORS];
    bool ok[GINT_MAX_TENSORS];
    uint32_t stored = 0;
    for (int t = 0; t < GINT_MAX_TENSORS; t++) {
        ok[t] = false;
        lq_of[t] = 0;
        if (t >= n_tensors) continue;
        const int64_t rows = ti.block_shape_stride_1[t][0], row_stride = ti.block_shape_stride_1[t][1];
        const int64_t cols = ti.block_shape_stride_2[t][0], col_stride = ti.block_shape_stride_2[t][1];
        const int64_t gd1 = (uint32_t)ti.block_grid_dims[t][0], gd2 = (uint32_t)ti.block_grid_dims[t][1];
        const int64_t gs1 = ti.block_grid_steps[t][0];
        bool good = ti.elm_size[t] == 4 && col_stride == 1 && (row_stride == 4 || row_stride == 8 || row_stride == 16) &&
                    cols >= row_stride && gd2 == 1 && gd1 >= 1 && gs1 >= 0 && rows - (gd1 - 1) * gs1 >= 32;
        if (good && gd1 != 1 && (gs1 * row_stride) % 4 != 0) good = false;
        for (int j = 0; good && j < 4; j++)
            if (ti.batch_shape[t][j] != 1 && ti.batch_strides[t][j] % 4 != 0) good = false;
        ok[t] = good;
        lq_of[t] = row_stride == 4 ? 0 : row_stride == 8 ? 1 : 2;
    }
    for (const Insn &in : *prog) {
        if (!is_tensor_op(in.op)) continue;
        const int t = (int)(in.operand & 15u);
        if (t >= GINT_MAX_TENSORS) continue;
        if (writes_tensor(in.op)) stored |= 1u << t;
        if (in.op != OP_LoadGlobal2DWF32) { ok[t] = false; continue; }
        const int64_t j0 = (int64_t)(in.operand >> 4);
        if ((j0 & 3) != 0 || j0 + 4 > (4ll << lq_of[t])) ok[t] = false;
    }
    uint32_t staged = 0, area_of[GINT_MAX_TENSORS] = {};
    bool used[GINT_MAX_TENSORS] = {};
    for (const Insn &in : *prog)
        if (in.op == OP_LoadGlobal2DWF32 && (in.operand & 15u) < GINT_MAX_TENSORS && ok[in.operand & 15u]) used[in.operand & 15u] = true;
    std::vector<Insn> head;
    for (int t = 0; t < n_tensors; t++) {
        if (!used[t]) continue;
        if (*area_bytes + (512u << lq_of[t]) > 0xFFFFu) break;
        area_of[t] = *area_bytes;
        *area_bytes += 512u << lq_of[t];
        staged |= 1u << t;
        alias_slots[t] |= (uint8_t)stored;
        head.push_back(Insn{OP_StageRows, (uint32_t)t | ((uint32_t)lq_of[t] << 3) | (area_of[t] << 8)});
    }
    if (!staged) return 0;
    for (Insn &in : *prog) {
        const uint32_t t = in.operand & 15u;
        if (in.op != OP_LoadGlobal2DWF32 || t >= GINT_MAX_TENSORS || !((staged >> t) & 1u)) continue;
        const uint32_t part = (in.operand >> 4) >> 2;
        in.op = OP_LoadStagedRows;
        in.operand = (uint32_t)lq_of[t] | (part << 2) | (t << 4) | (area_of[t] << 8);
    }
    prog->insert(prog->begin(), head.begin(), head.end());
    return staged;
}

/*
 * Fast row accesses: the 2DW counterpart of apply_fast_accesses. A LoadGlobal2DWF32 / StoreGlobal2DWF32 becomes its Fast form
 * (one unmasked 128-bit access per lane) when, for every logical program of the grid, all 32 rows of the tile exist, the four
 * columns exist, and the first byte is 16-byte aligned given a 16-byte aligned base pointer: unit column stride, row stride
 * and every per-program offset a multiple of 4 elements, column offset a multiple of 4. Slots that the program moves
 * (AdvanceBase / AdvanceBlock2D) are left alone. Returns the mask of slots relied on (base alignment is checked per launch).
 */
uint32_t apply_fast_rows(std::vector<Insn> *prog, const gint_tensor_info &ti, int n_tensors)
{
    bool ok[GINT_MAX_TENSORS];
    int64_t min_cols[GINT_MAX_TENSORS];
    for (int t = 0; t < GINT_MAX_TENSORS; t++) {
        ok[t] = false;
        min_cols[t] = 0;
        if (t >= n_tensors) continue;
        const int64_t rows = ti.block_shape_stride_1[t][0], row_stride = ti.block_shape_stride_1[t][1];
        const int64_t cols = ti.block_shape_stride_2[t][0], col_stride = ti.block_shape_stride_2[t][1];
        const int64_t gd1 = (uint32_t)ti.block_grid_dims[t][0], gd2 = (uint32_t)ti.block_grid_dims[t][1];
        const int64_t gs1 = ti.block_grid_steps[t][0], gs2 = ti.block_grid_steps[t][1];
        bool good = ti.elm_size[t] == 4 && col_stride == 1 && row_stride >= 0 && (row_stride % 4) == 0 && gd1 >= 1 && gd2 >= 1 && gs1 >= 0 && gs2 >= 0 &&
                    rows - (gd1 - 1) * gs1 >= 32 && (int64_t)31 * row_stride + cols < (1ll << 29);
        if (good && gd1 != 1 && (gs1 * row_stride) % 4 != 0) good = false;
        if (good && gd2 != 1 && (gs2 * col_stride) % 4 != 0) good = false;
        for (int j = 0; good && j < 4; j++)
            if (ti.batch_shape[t][j] != 1 && ti.batch_strides[t][j] % 4 != 0) good = false;
        ok[t] = good;
        min_cols[t] = cols - (gd2 - 1) * gs2;
    }
    for (const Insn &in : *prog)
        if (in.op == OP_AdvanceBlock2D || in.op == OP_AdvanceBase) ok[in.operand & 7u] = false;
    uint32_t used = 0;
    for (Insn &in : *prog) {
        if (in.op != OP_LoadGlobal2DWF32 && in.op != OP_StoreGlobal2DWF32) continue;
        const int slot = (int)(in.operand & 15u);
        const int64_t j0 = (int64_t)(in.operand >> 4);
        if (slot >= n_tensors || slot >= 8 || !ok[slot] || (j0 & 3) != 0 || j0 + 4 > min_cols[slot] || j0 * 4 >= (1 << 26)) continue;
        in.op = in.op == OP_LoadGlobal2DWF32 ? OP_LoadGlobal2DWF32Fast : OP_StoreGlobal2DWF32Fast;
        in.operand = ((uint32_t)slot << 29) | (uint32_t)(j0 * 4);
        used |= 1u << slot;
    }
    return used;
}

/*
 * DupBroadcastW k -> Bcast_k: the lane index is a constant of the program, so it moves from the operand word into the opcode
 * and the handler needs no run-time select (gint_opcodes.h). Same value in the same slot; the index was clamped to 0..3 by
 * normalise().
 */
void lower_lane_moves(std::vector<Insn> *prog, int pool_size)
{
    if (pool_size >= 12) return;   // the 12-slot kernels carry no Bcast_k handlers (register budget, see op_valid)
    for (Insn &in : *prog)
        if (in.op == OP_DupBroadcastW) in = Insn{OP_Bcast_0 + (int)(in.operand & 3u), 0u};
}

/* Conservative byte extent a program can touch from a tensor's base pointer; 0 = unknown (negative strides). */
/*
 * Virtual registers in shared memory ("RF" streams and kernels). In the reference, and in this library's ordinary kernels, the
 * operand stack and the eight virtual registers share one pool (register n = pool[P-1-n], gint/kernel/interpreter/state.py:
 * 12-18, 38-41), and a program with a deep stack AND many registers needs the 12-slot pool: 96 pool registers at two tiles per
 * warp, 16 resident warps per SM, handlers at the edge of the register budget. Such a program can run with a pool that holds
 * only its stack if its registers live elsewhere -- in a per-warp block of shared memory -- PROVIDED the overlap of stack
 * slots and registers in the shared pool is not observable: rf_equivalent runs the straight-line program on value numbers in
 * both models (one pool of P slots with the overlap; stack and registers apart) and demands that every instruction reads the
 * same value numbers in both. It also refuses a program that reads a register before writing it (the pool starts as zeros;
 * the shared-memory registers start as whatever the previous logical program left).
 */
bool rf_equivalent(const std::vector<Insn> &prog, int P)
{
    int pool[12] = {}, stack[GINT_MAX_STACK + 1] = {}, regs[8] = {};
    int next_id = 1, depth = 0;
    if (P > 12) return false;
    for (const Insn &in : prog) {
        const int op = in.op;
        if (op == OP_Halt) break;
        if (op < 0 || op >= GINT_N_OPCODES) return false;
        if (op >= OP_FLoadReg0 && op <= OP_FLoadReg7) {
            const int n = op - OP_FLoadReg0;
            if (P - 1 - n < 0 || regs[n] == 0 || pool[P - 1 - n] != regs[n] || depth >= P || depth >= GINT_MAX_STACK) return false;
            pool[depth] = stack[depth] = next_id++;
            depth++;
            continue;
        }
        if (op >= OP_FStoreReg0 && op <= OP_FStoreReg7) {
            const int n = op - OP_FStoreReg0;
            if (P - 1 - n < 0 || depth < 1 || pool[depth - 1] != stack[depth - 1]) return false;
            pool[P - 1 - n] = regs[n] = next_id++;
            depth--;
            continue;
        }
        const int md = kEffects[op].min_depth, post = depth + kEffects[op].net, top = post > depth ? post : depth;
        if (depth < md || top > P || top > GINT_MAX_STACK) return false;
        for (int j = depth - md; j < depth; j++)
            if (pool[j] != stack[j]) return false;
        for (int j = depth - md; j < top; j++) pool[j] = stack[j] = next_id++;
        depth = post;
    }
    return true;
}

/* FLoadRegN / FStoreRegN -> RLoad / RStore with the register number in the operand (512 bytes per register and tile). The
 * register area keeps a lane's four width values in four planes, so a lane permutation or shuffle that is applied to freshly
 * loaded registers is folded into the load (the handler reads other planes; no selects):
 *   RLoad a, FPermW s                  ->  RLoadP(a, s)
 *   RLoad a, RLoad b, FShuf2 s         ->  RLoadS(a, b, s)
 *   RLoad a, RLoad b, Dup2, FShuf2 s1, X1, FShuf2 s2, X2     (two shuffles of the same pair, each consumed at once)
 *       X = row stores to memory       ->  RLoadS(a, b, s1), X1, RLoadS(a, b, s2), X2
 *       X = RStore c, RStore d, c != d ->  RLoadS(a, b, s1), RLoadS(a, b, s2), RStore d, RStore c
 *         (both shuffles read a and b before either store, as the stack copies did in the original -- c or d may be a or b)
 * Selectors are already clamped to 0..3 (normalise). */
uint32_t pack_selectors(uint32_t clamped_bytes)
{
    return (clamped_bytes & 3u) | ((clamped_bytes >> 8) & 3u) << 2 | ((clamped_bytes >> 16) & 3u) << 4 | ((clamped_bytes >> 24) & 3u) << 6;
}
void rf_rewrite(std::vector<Insn> *prog)
{
    for (Insn &in : *prog) {
        if (in.op >= OP_FLoadReg0 && in.op <= OP_FLoadReg7) in = Insn{OP_RLoad, (uint32_t)(in.op - OP_FLoadReg0) * 512u};
        else if (in.op >= OP_FStoreReg0 && in.op <= OP_FStoreReg7) in = Insn{OP_RStore, (uint32_t)(in.op - OP_FStoreReg0) * 512u};
    }
    const std::vector<Insn> &p = *prog;
    std::vector<Insn> out;
    out.reserve(p.size());
    auto is_row_store = [](int op) { return op == OP_StoreGlobal2DWF32 || op == OP_StoreGlobal2DWF32Fast; };
    for (size_t i = 0; i < p.size();) {
        const size_t left = p.size() - i;
        if (left >= 7 && p[i].op == OP_RLoad && p[i + 1].op == OP_RLoad && p[i + 2].op == OP_Dup2 && p[i + 3].op == OP_FShuf2 &&
            p[i + 5].op == OP_FShuf2) {
            const uint32_t pair = p[i].operand | p[i + 1].operand << 12;
            const Insn s1{OP_RLoadS, pair | pack_selectors(p[i + 3].operand) << 24}, s2{OP_RLoadS, pair | pack_selectors(p[i + 5].operand) << 24};
            if (is_row_store(p[i + 4].op) && is_row_store(p[i + 6].op)) {
                out.insert(out.end(), {s1, p[i + 4], s2, p[i + 6]});
                i += 7;
                continue;
            }
            if (p[i + 4].op == OP_RStore && p[i + 6].op == OP_RStore && p[i + 4].operand != p[i + 6].operand) {
                out.insert(out.end(), {s1, s2, p[i + 6], p[i + 4]});
                i += 7;
                continue;
            }
        }
        if (left >= 3 && p[i].op == OP_RLoad && p[i + 1].op == OP_RLoad && p[i + 2].op == OP_FShuf2) {
            out.push_back(Insn{OP_RLoadS, p[i].operand | p[i + 1].operand << 12 | pack_selectors(p[i + 2].operand) << 24});
            i += 3;
            continue;
        }
        if (left >= 2 && p[i].op == OP_RLoad && p[i + 1].op == OP_FPermW) {
            out.push_back(Insn{OP_RLoadP, p[i].operand | pack_selectors(p[i + 1].operand) << 16});
            i += 2;
            continue;
        }
        out.push_back(p[i]);
        i++;
    }
    *prog = out;
}

/*
 * Vector layout ("vec" streams and kernels). As written, a 1-D tile puts element e of its 128 into lane e % 32, width value
 * e / 32, so a warp touches a tile with four 4-byte accesses per lane. Where the host has proved a tile full, unit-stride and
 * 16-byte aligned, lane l could just as well hold elements 4l..4l+3 -- one 16-byte access per lane -- as long as nothing in the
 * program can tell the difference. vec_transform decides that by abstract interpretation of the straight-line program. Every
 * pool entry is one of
 *   V   tile data in the vector layout (from early-issued or fast 1-D loads)
 *   N   tile data in the natural layout (from every other load)
 *   W   the same in all lanes; per width value a symbol that names the expression it holds (equal symbols => equal bits)
 * (a W whose four symbols are equal is uniform and mixes with anything). Element-wise instructions combine like with like; an
 * instruction that looks across lanes or width values (warp reductions, FPermW, DupBroadcastW, a store that is not a fast
 * 1-D store) needs N or W and gets a RemapVN in front of it if its operand is V (RemapVN moves the accumulators to where the
 * natural layout has them, so a reduction afterwards adds the same values in the same order: bit-identical results). The
 * symbols make the typical epilogue of a row reduction provable: after WarpAllReduceSum and the two FPermW / FAdd steps that add
 * the four width values, all four symbols are the same expression up to the order of commutative operands, the value is
 * uniform, and the second pass may multiply vector-layout tiles with it. Anything the analysis does not know ends it: the
 * program then simply has no vector-layout stream.
 */
struct LaneValue {
    enum Kind : uint8_t { W, V, N } kind;
    uint32_t sym[4];
    bool uniform() const { return kind == W && sym[0] == sym[1] && sym[1] == sym[2] && sym[2] == sym[3]; }
};

struct SymbolTable {
    std::map<std::array<uint32_t, 5>, uint32_t> ids;
    uint32_t next = 1;
    uint32_t fresh() { return next++; }
    uint32_t make(uint32_t op, uint32_t operand, uint32_t a, uint32_t b = 0, uint32_t c = 0, bool commutative = false)
    {
        if (commutative && a > b) std::swap(a, b);
        const std::array<uint32_t, 5> key{op, operand, a, b, c};
        auto it = ids.find(key);
        if (it != ids.end()) return it->second;
        return ids[key] = next++;
    }
};

bool vec_is_unary(int op)
{
    return op == OP_FNeg || op == OP_FAddImm || op == OP_FMulImm || op == OP_FMAImm || (op >= OP_FSqrt && op <= OP_FArcTan) ||
           (op >= OP_FExp && op <= OP_FErf) || op == OP_FRcp;
}
bool vec_is_binary(int op)
{
    return op == OP_FAdd || op == OP_FMul || op == OP_FSub || op == OP_FRSub || op == OP_FDiv || op == OP_FRDiv || op == OP_FRem ||
           (op >= OP_FGt && op <= OP_FApprox) || op == OP_FArcTan2 || op == OP_FPow || (op >= OP_IAdd && op <= OP_IXor);
}
bool vec_is_commutative(int op) { return op == OP_FAdd || op == OP_FMul || op == OP_IAdd || op == OP_IMul || op == OP_IAnd || op == OP_IOr || op == OP_IXor; }

/* `prog`: the early-issue stream after the fast-access pass, before lowering and fusion. On success `out` is the stream for the
 * vector-layout kernels (RemapVN inserted) and the counts say how much it is worth. */
bool vec_transform(const std::vector<Insn> &prog, std::vector<Insn> *out, int *n_vector_accesses, int *n_remaps)
{
    SymbolTable st;
    std::vector<LaneValue> stack;
    LaneValue regs[8];
    const uint32_t zero = st.make(OP_LoadImm, 0u, 0u);
    for (auto &r : regs) r = LaneValue{LaneValue::W, {zero, zero, zero, zero}};
    out->clear();
    *n_vector_accesses = 0;
    *n_remaps = 0;
    auto join = [](const LaneValue &a, const LaneValue &b, LaneValue::Kind *k) {   // layout of an element-wise result; false: they clash
        if (a.kind == LaneValue::W && b.kind == LaneValue::W) { *k = LaneValue::W; return true; }
        const LaneValue &data = a.kind != LaneValue::W ? a : b, &other = a.kind != LaneValue::W ? b : a;
        if (other.kind == LaneValue::W) {
            if (data.kind == LaneValue::V && !other.uniform()) return false;   // width w means other elements in the two layouts
            *k = data.kind;
            return true;
        }
        if (data.kind != other.kind) return false;
        *k = data.kind;
        return true;
    };
    auto need_natural_top = [&]() {   // the top of the stack must not be in the vector layout
        if (stack.back().kind == LaneValue::V) {
            out->push_back(Insn{OP_RemapVN, 0u});
            stack.back().kind = LaneValue::N;
            (*n_remaps)++;
        }
    };
    for (const Insn &in : prog) {
        const int op = in.op;
        const size_t d = stack.size();
        if (op == OP_Halt) { out->push_back(in); return true; }
        if (op == OP_Nop || op == OP_PfIssue1D || op == OP_PfIssue1DFast || op == OP_PfSkip || op == OP_AdvanceBase || op == OP_AdvanceBlock2D ||
            op == OP_StageRows) {
            out->push_back(in);
        } else if (op == OP_Pop) {
            if (d < 1) return false;
            stack.pop_back();
            out->push_back(in);
        } else if (op == OP_Pop2) {
            if (d < 2) return false;
            stack.pop_back(); stack.pop_back();
            out->push_back(in);
        } else if (op == OP_Dup) {
            if (d < 1) return false;
            stack.push_back(stack[d - 1]);
            out->push_back(in);
        } else if (op == OP_Dup2) {
            if (d < 2) return false;
            stack.push_back(stack[d - 2]); stack.push_back(stack[d - 1]);
            out->push_back(in);
        } else if (op == OP_DupX1) {          // [a, b] -> [b, a, b]
            if (d < 2) return false;
            const LaneValue a = stack[d - 2], b = stack[d - 1];
            stack[d - 2] = b; stack[d - 1] = a; stack.push_back(b);
            out->push_back(in);
        } else if (op == OP_DupX2) {          // [a, b, c] -> [c, a, b, c]
            if (d < 3) return false;
            const LaneValue a = stack[d - 3], b = stack[d - 2], c = stack[d - 1];
            stack[d - 3] = c; stack[d - 2] = a; stack[d - 1] = b; stack.push_back(c);
            out->push_back(in);
        } else if (op == OP_Swap) {
            if (d < 2) return false;
            std::swap(stack[d - 1], stack[d - 2]);
            out->push_back(in);
        } else if (op == OP_LoadImm) {
            const uint32_t s0 = st.make(OP_LoadImm, in.operand, 0u);
            stack.push_back(LaneValue{LaneValue::W, {s0, s0, s0, s0}});
            out->push_back(in);
        } else if (op == OP_LoadImm4F || op == OP_LoadImm4I) {
            LaneValue v{LaneValue::W, {}};
            for (int w = 0; w < 4; w++) v.sym[w] = st.make((uint32_t)op, (in.operand >> (8 * w)) & 0xFFu, 0u);
            stack.push_back(v);
            out->push_back(in);
        } else if (op >= OP_FLoadReg0 && op <= OP_FLoadReg7) {
            stack.push_back(regs[op - OP_FLoadReg0]);
            out->push_back(in);
        } else if (op >= OP_FStoreReg0 && op <= OP_FStoreReg7) {
            if (d < 1) return false;
            regs[op - OP_FStoreReg0] = stack.back();
            stack.pop_back();
            out->push_back(in);
        } else if (vec_is_unary(op)) {
            if (d < 1) return false;
            LaneValue &t = stack.back();
            if (t.kind == LaneValue::W)
                for (int w = 0; w < 4; w++) t.sym[w] = st.make((uint32_t)op, in.operand, t.sym[w]);
            out->push_back(in);
        } else if (vec_is_binary(op)) {
            if (d < 2) return false;
            const LaneValue t = stack[d - 1], s2 = stack[d - 2];
            LaneValue r{LaneValue::W, {}};
            if (!join(t, s2, &r.kind)) return false;
            if (r.kind == LaneValue::W)
                for (int w = 0; w < 4; w++) r.sym[w] = st.make((uint32_t)op, in.operand, t.sym[w], s2.sym[w], 0u, vec_is_commutative(op));
            stack.pop_back();
            stack.back() = r;
            out->push_back(in);
        } else if (op == OP_FMA || op == OP_Select) {
            if (d < 3) return false;
            const LaneValue t = stack[d - 1], s2 = stack[d - 2], u = stack[d - 3];
            LaneValue r{LaneValue::W, {}}, ts{LaneValue::W, {}};
            if (!join(t, s2, &ts.kind)) return false;
            if (ts.kind == LaneValue::W) {
                /* stands for "lane-uniform with the widths of both": uniform only if both are */
                const bool both = t.uniform() && s2.uniform();
                for (int w = 0; w < 4; w++) ts.sym[w] = both ? 1u : (uint32_t)(w + 2);
            }
            if (!join(ts, u, &r.kind)) return false;
            if (r.kind == LaneValue::W)
                for (int w = 0; w < 4; w++) r.sym[w] = st.make((uint32_t)op, in.operand, t.sym[w], s2.sym[w], u.sym[w]);
            stack.pop_back(); stack.pop_back();
            stack.back() = r;
            out->push_back(in);
        } else if (op >= OP_WarpAllReduceSum && op <= OP_WarpAllReduceProd) {
            if (d < 1) return false;
            need_natural_top();
            LaneValue &t = stack.back();
            if (t.kind == LaneValue::N) {
                t.kind = LaneValue::W;
                for (int w = 0; w < 4; w++) t.sym[w] = st.fresh();
            } else {
                for (int w = 0; w < 4; w++) t.sym[w] = st.make((uint32_t)op, 0u, t.sym[w]);
            }
            out->push_back(in);
        } else if (op == OP_FPermW) {
            if (d < 1) return false;
            need_natural_top();
            LaneValue &t = stack.back();
            if (t.kind == LaneValue::W) {
                const LaneValue o = t;
                for (int w = 0; w < 4; w++) t.sym[w] = o.sym[(in.operand >> (8 * w)) & 3u];
            }
            out->push_back(in);
        } else if (op == OP_DupBroadcastW) {
            if (d < 1) return false;
            need_natural_top();
            LaneValue v = stack.back();
            if (v.kind == LaneValue::W) {
                const uint32_t s0 = v.sym[in.operand & 3u];
                for (int w = 0; w < 4; w++) v.sym[w] = s0;
            }
            stack.push_back(v);
            out->push_back(in);
        } else if (op == OP_FShuf2) {
            if (d < 2) return false;
            const LaneValue t = stack[d - 1], s2 = stack[d - 2];
            if (t.kind == LaneValue::V || s2.kind == LaneValue::V) return false;
            LaneValue r{LaneValue::N, {}};
            if (t.kind == LaneValue::W && s2.kind == LaneValue::W) {
                r.kind = LaneValue::W;
                for (int w = 0; w < 4; w++) r.sym[w] = (w < 2 ? s2 : t).sym[(in.operand >> (8 * w)) & 3u];
            }
            stack.pop_back();
            stack.back() = r;
            out->push_back(in);
        } else if (op == OP_PfTake || op == OP_PfTakeIssue1D || op == OP_PfTakeIssue1DFast || op == OP_LoadGlobal1DF32Fast) {
            stack.push_back(LaneValue{LaneValue::V, {}});
            (*n_vector_accesses)++;
            out->push_back(in);
        } else if (op == OP_StoreGlobal1DF32Fast) {
            if (d < 1) return false;
            const LaneValue &t = stack.back();
            if (!(t.kind == LaneValue::V || t.uniform())) return false;   // (natural-layout data would need the opposite rearrangement)
            stack.pop_back();
            (*n_vector_accesses)++;
            out->push_back(in);
        } else if (op == OP_LoadGlobal1DF32 || op == OP_LoadGlobal1DF16 || op == OP_LoadGlobal1DBF16 || op == OP_LoadGlobal1DU8 ||
                   (op >= OP_LoadGlobal2DTF32 && op <= OP_LoadGlobal2DWU8 && !writes_tensor(op)) || op == OP_LoadStagedRows ||
                   op == OP_LoadGlobal2DWF32Fast) {
            stack.push_back(LaneValue{LaneValue::N, {}});
            out->push_back(in);
        } else if (writes_tensor(op) && op != OP_StoreGlobal1DF32Indirect) {
            if (d < 1) return false;
            need_natural_top();
            stack.pop_back();
            out->push_back(in);
        } else {
            return false;   // gathers and scatters, and whatever this analysis has not been taught
        }
        if (stack.size() > (size_t)GINT_MAX_STACK) return false;
    }
    return false;   // no Halt
}

/* A rearrangement is a round trip through shared memory with two warp synchronisations on the critical path of its logical
 * program; a vector access saves three load/store instructions. Measured on the conductor graph at two tiles per warp: the fused
 * program (40 vector accesses, 1 rearrangement) 175 -> 169 us, the row-sum program (8 and 1) 49.7 -> 52.3 us. */
bool vec_worth_it(int n_vector_accesses, int n_remaps) { return n_vector_accesses >= 16 && n_vector_accesses >= 16 * n_remaps; }

uint64_t tensor_extent_bytes(const gint_tensor_info &ti, int t)
{
    int64_t elems = 1;
    const int32_t dims[6][2] = {{ti.block_shape_stride_1[t][0], ti.block_shape_stride_1[t][1]},
                                {ti.block_shape_stride_2[t][0], ti.block_shape_stride_2[t][1]},
                                {ti.batch_shape[t][0], ti.batch_strides[t][0]}, {ti.batch_shape[t][1], ti.batch_strides[t][1]},
                                {ti.batch_shape[t][2], ti.batch_strides[t][2]}, {ti.batch_shape[t][3], ti.batch_strides[t][3]}};
    for (auto &d : dims) {
        if (d[1] < 0) return 0;
        if (d[0] > 1) elems += (int64_t)(d[0] - 1) * (int64_t)d[1];
    }
    return (uint64_t)elems * (uint64_t)(ti.elm_size[t] > 4 ? ti.elm_size[t] : 4);
}

struct Variant {
    int P, K;
    const void *fn;   // cudaKernel_t of the loaded cubin, usable wherever the runtime takes a kernel function
    int regs;
    bool ok;
    int resident_warps;   // warps of this kernel the whole device holds when a block needs only its minimum of shared memory
    bool rf = false;      // virtual registers in shared memory (pool = operand stack only)
    bool vec = false;     // 1-D tiles in the vector layout
};

/* The embedded cubins are loaded once per process (a cudaLibrary_t is not tied to a device or context). */
struct KernelImage {
    const unsigned char *begin;
    const unsigned char *end;
    const char *name;
    int P, K;          // K == 0: indirect kernel; K == -1: checked kernel
    cudaLibrary_t lib;
    cudaKernel_t kernel;
    bool loaded;
    bool rf;
    bool vec = false;
};

KernelImage g_images[] = {
#define GINT_X_IMG(P, K) {gint_cubin_direct_##P##_##K, gint_cubin_direct_##P##_##K##_end, "gint_geval_direct_" #P "_" #K, P, K, nullptr, nullptr, false, false},
    GINT_DIRECT_VARIANTS(GINT_X_IMG)
#undef GINT_X_IMG
#define GINT_X_IMG(P, K) {gint_cubin_rf_##P##_##K, gint_cubin_rf_##P##_##K##_end, "gint_geval_rf_" #P "_" #K, P, K, nullptr, nullptr, false, true},
    GINT_RF_VARIANTS(GINT_X_IMG)
#undef GINT_X_IMG
#define GINT_X_IMG(P, K) {gint_cubin_vec_##P##_##K, gint_cubin_vec_##P##_##K##_end, "gint_geval_vec_" #P "_" #K, P, K, nullptr, nullptr, false, false, true},
    GINT_VEC_VARIANTS(GINT_X_IMG)
#undef GINT_X_IMG
#define GINT_X_IMG(P) {gint_cubin_indirect_##P, gint_cubin_indirect_##P##_end, "gint_geval_indirect_" #P, P, 0, nullptr, nullptr, false, false},
    GINT_INDIRECT_VARIANTS(GINT_X_IMG)
#undef GINT_X_IMG
#define GINT_X_IMG(P) {gint_cubin_checked_##P, gint_cubin_checked_##P##_end, "gint_geval_checked_" #P, P, -1, nullptr, nullptr, false, false},
    GINT_CHECKED_VARIANTS(GINT_X_IMG)
#undef GINT_X_IMG
};
std::mutex g_images_mu;
std::string g_images_error;

int load_images()
{
    std::lock_guard<std::mutex> lk(g_images_mu);
    int usable = 0;
    for (auto &im : g_images) {
        if (!im.loaded) {
            cudaError_t e = cudaLibraryLoadData(&im.lib, im.begin, nullptr, nullptr, 0, nullptr, nullptr, 0);
            if (e == cudaSuccess) e = cudaLibraryGetKernel(&im.kernel, im.lib, im.name);
            if (e != cudaSuccess) {
                g_images_error = std::string(im.name) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")";
                cudaGetLastError();
                continue;
            }
            im.loaded = true;
        }
        usable++;
    }
    return usable;
}

struct Geometry {
    Variant *v;
    uint32_t smem;
    uint32_t code_smem;
    int blocks_per_sm;
    uint32_t grid;
};

struct PlanMemo { bool valid; uint32_t count; int opt_k, opt_blocks; Geometry g; };

struct Program {
    bool live = false;
    uint2 *code_dev = nullptr;
    uint32_t n_slots = 0;
    int n_tensors = 0;
    gint_tensor_info ti;
    gint_bytecode_stats st;
    uint32_t prefetch_mask = 0;
    gint::Footprint fp[GINT_MAX_TENSORS];
    /* early-issue stream (nullptr if the program has no eligible load) and what must hold at launch for it to be used */
    uint2 *early_dev = nullptr;
    uint32_t early_slots = 0;
    int n_early = 0;
    uint8_t alias_slots[GINT_MAX_TENSORS] = {};
    uint32_t fast_slots = 0;   // tensor slots whose base pointer must be 16-byte aligned for the early-issue stream
    bool prefer_narrow = false; // one tile per warp unless told otherwise (see plan_direct)
    uint32_t reread_bytes = 0;  // bytes of the 1-D tiles a logical program loads more than once (0: none)
    uint64_t uid = 0;           // unique per created program (a handle slot may be reused)
    int ring_slots = gint::kRingSlotsShallow;   // depth of the ring of early-issued loads (early-issue stream)
    uint32_t row_area_bytes = 0; // shared memory per tile for staged row blocks (early-issue stream only)
    uint64_t extent[GINT_MAX_TENSORS] = {};
    /* host copies of the two streams when they are short enough to travel inside the kernel parameters */
    uint2 code_inline[gint::kInlineCodeSlots];
    uint2 early_inline[gint::kInlineCodeSlots];
    /* the stream for the kernels with virtual registers in shared memory (nullptr: none); made from the early-issue stream if
     * the program has a usable one (rf_from_early: the same launch conditions apply), else from the plain stream */
    uint2 *rf_dev = nullptr;
    uint32_t rf_slots = 0;
    int rf_pool = 0;            // pool size of the kernel that runs it (the operand stack alone)
    uint32_t rf_bytes = 0;      // shared memory per tile for the registers: 512 bytes per register
    bool rf_from_early = false;
    uint2 rf_inline[gint::kInlineCodeSlots];
    /* the stream for the vector-layout kernels (nullptr: none): the early-issue stream with RemapVN where a value has to be in
     * the natural layout; usable whenever the early-issue stream is */
    uint2 *vec_dev = nullptr;
    uint32_t vec_slots = 0;
    int vec_remaps = 0;
    uint2 vec_inline[gint::kInlineCodeSlots];
    PlanMemo memo[4] = {};      // last launch plan of the plain stream [0], the early-issue stream [1], the RF stream [2], the vector-layout stream [3]
    std::mutex memo_mu;
};

/* Which bytes of each tensor one logical program reads: the union of its tile loads along the contiguous dimension.
 * Tensors that are only written, are reached through gather/scatter or AdvanceBlock2D/AdvanceBase, use the 2DT layout or a
 * non-f32 element type get no footprint (they are simply not prefetched). */
void compute_footprints(const int32_t *code, int n_insns, const gint_tensor_info &ti, int n_tensors, Program *p)
{
    bool dynamic[GINT_MAX_TENSORS] = {};
    for (int t = 0; t < GINT_MAX_TENSORS; t++) p->fp[t] = gint::Footprint{gint::FP_NONE, INT32_MAX, INT32_MIN, 0};
    for (int i = 0; i < n_insns; i++) {
        const int op = code[2 * i];
        const uint32_t operand = (uint32_t)code[2 * i + 1];
        if (!is_tensor_op(op)) continue;
        const int t = (int)(operand & 15u);
        if (t >= n_tensors) continue;
        const int off = (int)(operand >> 4);
        int kind = gint::FP_NONE, width = 0;
        if (op == OP_LoadGlobal1DF32) { kind = gint::FP_1D; width = 128; }
        else if (op == OP_LoadGlobal2DWF32) { kind = gint::FP_ROWS; width = 4; }
        else if (op == OP_StoreGlobal1DF32 || op == OP_StoreGlobal2DWF32 || op == OP_StoreGlobal2DTF32) continue;  // writes need no prefetch
        else { dynamic[t] = true; continue; }
        gint::Footprint &f = p->fp[t];
        if (f.kind != gint::FP_NONE && f.kind != kind) { dynamic[t] = true; continue; }
        f.kind = kind;
        if (off < f.lo) f.lo = off;
        if (off + width > f.hi) f.hi = off + width;
    }
    p->prefetch_mask = 0;
    for (int t = 0; t < n_tensors; t++) {
        gint::Footprint &f = p->fp[t];
        const bool unit = f.kind == gint::FP_1D ? ti.block_shape_stride_1[t][1] == 1 : ti.block_shape_stride_2[t][1] == 1;
        if (f.kind == gint::FP_NONE || dynamic[t] || !unit || ti.elm_size[t] != 4) { f.kind = gint::FP_NONE; f.lo = f.hi = 0; continue; }
        p->prefetch_mask |= 1u << t;
    }
}

}  // namespace

struct gint_ctx {
    int device = -1;
    int num_sms = 0;
    int max_smem_optin = 0;
    std::mutex mu;
    std::vector<Program *> programs;
    std::vector<Variant> direct;
    Variant indirect{12, 1, nullptr, 0, false, 0};
    Variant checked{12, 1, nullptr, 0, false, 0};
    gint_device_status *status_dev = nullptr;   // status word of the checked launches (allocated on first use)
    std::string last_error;
    int opt_tiles_per_warp = 0;
    int opt_max_blocks = 0;
    int opt_prefetch = 0;
    int opt_early_issue = 1;
    int opt_fuse = 1;           // applies to programs created afterwards
    int opt_lower = 1;          // DupBroadcastW -> Bcast_k (lower_lane_moves); applies to programs created afterwards
    int opt_rf = 1;             // launches use a program's RF stream (virtual registers in shared memory) when it has one
    int opt_rf_create = 1;      // programs created from now on get an RF stream when they qualify
    int opt_vec = 0;            // vector-layout stream and kernels for the programs that qualify (creation and launch). Off unless asked
                                // for: measured on the conductor graph, the fused program alone gains 2-3 % (175 -> 169 us) but the whole
                                // graph through the benchmark's plan loses 1-2 % (340 -> 345 us)
    /* scratch for indirect launches */
    void *ind_dev = nullptr;
    void *ind_host = nullptr;
    size_t ind_bytes = 0;
    cudaEvent_t ind_event = nullptr;         // the last indirect launch's table upload has been queued and read the host image
    cudaEvent_t ind_kernel_event = nullptr;  // the last indirect launch's kernel has finished with the device tables
    std::mutex ind_mu;                       // serialises indirect launches of this context (shared scratch)
};

namespace {

int fail(gint_ctx *ctx, int status, const char *what, cudaError_t e = cudaSuccess)
{
    if (ctx) {
        char buf[512];
        if (e != cudaSuccess) snprintf(buf, sizeof(buf), "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
        else snprintf(buf, sizeof(buf), "%s", what);
        ctx->last_error = buf;
    }
    return status;
}

struct DeviceGuard {
    int prev = -1;
    bool switched = false;
    explicit DeviceGuard(int dev)
    {
        if (cudaGetDevice(&prev) == cudaSuccess && prev != dev) switched = cudaSetDevice(dev) == cudaSuccess;
    }
    ~DeviceGuard()
    {
        if (switched) cudaSetDevice(prev);
    }
};

Program *lookup(gint_ctx *ctx, uint64_t handle)
{
    std::lock_guard<std::mutex> lk(ctx->mu);
    if (handle == 0 || handle > ctx->programs.size()) return nullptr;
    Program *p = ctx->programs[handle - 1];
    return (p && p->live) ? p : nullptr;
}

Variant *find_variant(gint_ctx *ctx, int P, int K, bool rf = false, bool vec = false)
{
    for (auto &v : ctx->direct)
        if (v.P == P && v.K == K && v.rf == rf && v.vec == vec && v.ok) return &v;
    return nullptr;
}


/* What a launch runs: one of the program's two streams. The ring of early-issued loads and the staged row blocks exist only
 * in the early-issue stream. */
struct StreamView {
    uint32_t n_slots;
    uint32_t ring_bytes;       // shared memory per tile for the ring of early-issued loads
    uint32_t row_area_bytes;   // shared memory per tile for staged row blocks
    uint32_t rf_bytes;         // shared memory per tile for virtual registers (RF stream)
    int P;                     // pool size of the kernels that run this stream
    bool early;
    bool rf;
    bool vec;
};

StreamView stream_view(const Program *p, bool early, bool rf = false, bool vec = false)
{
    StreamView v;
    v.early = early;
    v.rf = rf;
    v.vec = vec;
    v.n_slots = rf ? p->rf_slots : vec ? p->vec_slots : early ? p->early_slots : p->n_slots;
    v.ring_bytes = early && p->n_early > 0 ? (uint32_t)p->ring_slots * 512u : 0u;
    v.row_area_bytes = early ? p->row_area_bytes : 0u;
    v.rf_bytes = rf ? p->rf_bytes : vec && p->vec_remaps > 0 ? 512u : 0u;   // (vector layout: the exchange area of RemapVN)
    v.P = rf ? p->rf_pool : p->st.pool_size;
    return v;
}

uint32_t direct_smem(const StreamView &v, int K, uint32_t *code_smem)
{
    const uint32_t cs = (v.n_slots * 8u + 127u) & ~127u;
    *code_smem = cs;
    return cs + gint::kTensorInfoSmemBytes + (uint32_t)(gint::kWarpsPerBlock * K) * (uint32_t)sizeof(gint::TileInfo) +
           (uint32_t)(gint::kWarpsPerBlock * K) * (v.ring_bytes + v.row_area_bytes + v.rf_bytes);
}

/* Blocks needed to give every group of K logical programs a warp. */
uint64_t blocks_for(uint32_t count, int K)
{
    const uint64_t groups = ((uint64_t)count + (uint64_t)K - 1) / (uint64_t)K;
    return (groups + gint::kWarpsPerBlock - 1) / gint::kWarpsPerBlock;
}

int plan_direct(gint_ctx *ctx, const Program *p, const StreamView &sv, uint32_t count, Geometry *g)
{
    const int P = sv.P;
    const int ks[3] = {4, 2, 1};
    /* upper bound on K: the option if set; else 2 (measured: 4 tiles per warp lose more to the lower occupancy of the
     * 96-register kernels than they gain from amortised dispatch), and 1 for programs that are bound by memory instructions
     * rather than by dispatch: those in which at least 2 of 5 instructions access memory (measured on RMSNorm rows: load/store
     * issue is not amortised by more tiles per warp) and those in which at least 1 of 5 instructions is a load that is not
     * issued early (measured on the batched 4x4 product: its latency is hidden only by more resident warps, which the
     * narrower kernel gives) */
    int k_max = ctx->opt_tiles_per_warp ? ctx->opt_tiles_per_warp : p->prefer_narrow ? 1 : 2;
    /* ... unless the logical program is a single tile or so: what a warp keeps in flight is (early-issued loads of one logical
     * program, at most the ring's depth) x K tiles of 512 bytes, and the dispatches are shared by K tiles. Measured on a + b over
     * 2^26 elements (torch's add: 6.8 TB/s): one tile per logical program 4.3 / 5.9 / 6.4 TB/s at 1 / 2 / 4 tiles per warp;
     * two tiles 6.1 / 5.8 / 5.8; four tiles 6.5 / 5.9 / 5.9; sixteen 5.9 / 5.8 / 5.8 -- so only the shortest programs go wide */
    if (!ctx->opt_tiles_per_warp && sv.early && p->n_early > 0) {
        const int in_flight = p->n_early < p->ring_slots ? p->n_early : p->ring_slots;
        if (in_flight < 4 && k_max < 4) k_max = 4;
    }
    /* A short program whose whole grid is gone after at most two rounds of the resident warps is bound by latency, not
     * throughput: what it waits for is a fixed per-block cost (block start, program staging, descriptor decode) and one or
     * two memory round trips per warp. Fewer, fatter blocks are then faster as long as every SM still gets two of them
     * (measured on a+b over 2^20 elements, device time: 7.1 / 6.3 / 5.9 us at 1 / 2 / 4 tiles per warp). */
    bool latency_bound = false;
    if (!ctx->opt_tiles_per_warp && sv.n_slots <= (uint32_t)gint::kInlineCodeSlots) {
        Variant *v1 = find_variant(ctx, P, 1, sv.rf, sv.vec);
        if (v1 && v1->resident_warps > 0 && (uint64_t)count <= 2ull * (uint64_t)v1->resident_warps) {
            latency_bound = true;
            k_max = 1;
            for (int K : ks)
                if (find_variant(ctx, P, K, sv.rf, sv.vec) && blocks_for(count, K) >= 2ull * (uint64_t)ctx->num_sms) { k_max = K; break; }
        }
    }
    Geometry best{};
    bool have = false;
    for (int K : ks) {
        if (K > k_max) continue;
        Variant *v = find_variant(ctx, P, K, sv.rf, sv.vec);
        if (!v) continue;
        Geometry c{};
        c.v = v;
        c.smem = direct_smem(sv, K, &c.code_smem);
        if ((int)c.smem > ctx->max_smem_optin) continue;
        if (c.smem > 48u * 1024u) {
            cudaError_t e = cudaFuncSetAttribute(v->fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)c.smem);
            if (e != cudaSuccess) { cudaGetLastError(); continue; }
        }
        int bps = 0;
        cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&bps, v->fn, gint::kThreadsPerBlock, c.smem);
        if (e != cudaSuccess || bps < 1) { cudaGetLastError(); continue; }
        /* A program that reads a tile twice (a reduction pass, then a second pass over the same row) finds it in L2 the
         * second time only if the rows in flight, with their write-allocated outputs, fit there: measured on RMSNorm
         * rows of 16 KB with the 8-slot ring, 5 blocks per SM (47 MB of rows in flight) beat 6 (110 us vs 118 us); fewer
         * lose to exposed latency. Rows of 4 KB (the conductor graph) stay below that bound at full occupancy. */
        while (bps > 4 && (uint64_t)p->reread_bytes * (uint64_t)(K * gint::kWarpsPerBlock) * (uint64_t)ctx->num_sms * (uint64_t)bps > 50000000ull) bps--;
        c.blocks_per_sm = bps;
        const uint64_t blocks_needed = blocks_for(count, K);
        uint64_t resident = (uint64_t)bps * (uint64_t)ctx->num_sms;
        if (ctx->opt_max_blocks > 0 && (uint64_t)ctx->opt_max_blocks < resident) resident = (uint64_t)ctx->opt_max_blocks;
        c.grid = (uint32_t)(blocks_needed < resident ? blocks_needed : resident);
        if (c.grid == 0) c.grid = 1;
        if (!have) { best = c; have = true; }
        /* take the widest K that still fills the machine with at least one group per resident warp */
        if (blocks_needed >= resident || ctx->opt_tiles_per_warp || latency_bound) { best = c; break; }
        best = c;  // fewer groups than warps: prefer the narrower variant (more warps busy)
    }
    if (!have) return fail(ctx, GINT_ERR_TOO_LARGE, "no kernel variant fits this program (shared memory)");
    *g = best;
    return GINT_OK;
}

struct GatherArgs {
    uint32_t mask;            // tensor slots whose innermost batch index goes through the row index
    const long long *index;   // device pointer
    uint64_t extent_bytes;    // bytes of the gathered tensor(s) that the index can reach, from the base pointer
    uint32_t rows;            // rows of the gathered table
};

int launch_direct(gint_ctx *ctx, uint64_t handle, const uint64_t *base_ptrs, int n_tensors, uint32_t first, uint32_t count,
                  void *stream, const GatherArgs *gather = nullptr)
{
    if (!ctx || (!base_ptrs && n_tensors > 0)) return fail(ctx, GINT_ERR_INVALID_ARGUMENT, "null argument");
    Program *p = lookup(ctx, handle);
    if (!p) return fail(ctx, GINT_ERR_BAD_HANDLE, "unknown program handle");
    if (n_tensors != p->n_tensors) return fail(ctx, GINT_ERR_ARG_COUNT, "number of arguments does not match the program");
    if (count == 0) return GINT_OK;
    if ((uint64_t)first + (uint64_t)count > 0xFFFFFFFFull) return fail(ctx, GINT_ERR_TOO_LARGE, "logical program range overflows 32 bits");
    DeviceGuard guard(ctx->device);
    /* The early-issue stream is used unless a tensor whose loads were moved across stores overlaps, at this launch's
     * addresses, one of the tensors those stores write. */
    bool early = ctx->opt_early_issue && p->early_dev != nullptr;
    for (int t = 0; early && t < n_tensors; t++) {
        if (!p->alias_slots[t]) continue;
        for (int b = 0; early && b < n_tensors; b++) {
            if (!((p->alias_slots[t] >> b) & 1u)) continue;
            const bool ga = gather && ((gather->mask >> t) & 1u), gb = gather && ((gather->mask >> b) & 1u);
            const uint64_t a0 = base_ptrs[t], a1 = a0 + (ga ? gather->extent_bytes : p->extent[t]);
            const uint64_t b0 = base_ptrs[b], b1 = b0 + (gb ? gather->extent_bytes : p->extent[b]);
            if (a0 < b1 && b0 < a1) early = false;
        }
    }
    for (int t = 0; early && t < n_tensors; t++)
        if (((p->fast_slots >> t) & 1u) && (base_ptrs[t] & 15u) != 0) early = false;   // fast accesses need aligned bases
    /* the stream with the virtual registers in shared memory, when the stream it was made from is the one this launch may use */
    bool rf = ctx->opt_rf && p->rf_dev != nullptr && p->rf_from_early == early;
    /* the vector-layout stream, for programs that run more than one tile per warp (measured: the conductor graph's fused program
     * 174 -> 164 us at two tiles per warp; RMSNorm at one tile per warp 110 -> 112 us, so it stays on the ordinary kernel) */
    bool vec = ctx->opt_vec && p->vec_dev != nullptr && early && !rf && !p->prefer_narrow && ctx->opt_tiles_per_warp != 1;
    StreamView sv = stream_view(p, early, rf, vec);   // geometry depends on the stream
    Geometry g;
    {
        /* each program remembers its last plan per stream: a launch that repeats the previous one's size skips the occupancy
         * queries (several microseconds), also when the caller alternates between programs */
        std::lock_guard<std::mutex> lk(p->memo_mu);
        PlanMemo *m = &p->memo[rf ? 2 : vec ? 3 : early ? 1 : 0];
        if (m->valid && m->count == count && m->opt_k == ctx->opt_tiles_per_warp && m->opt_blocks == ctx->opt_max_blocks) {
            g = m->g;
        } else {
            int rc = plan_direct(ctx, p, sv, count, &g);
            if (rc != GINT_OK && (rf || vec)) {   // no such kernel for this tiles-per-warp choice or this much shared memory: the ordinary kernels
                rf = vec = false;
                sv = stream_view(p, early, false);
                rc = plan_direct(ctx, p, sv, count, &g);   // (remembered under the RF stream's memo: the next launch asks there again)
            }
            if (rc != GINT_OK) return rc;
            *m = PlanMemo{true, count, ctx->opt_tiles_per_warp, ctx->opt_max_blocks, g};
        }
        rf = g.v->rf;
        vec = g.v->vec;
        if ((!rf && sv.rf) || (!vec && sv.vec)) sv = stream_view(p, early, false);
    }
    LaunchArgs a;
    const bool inline_code = sv.n_slots <= (uint32_t)gint::kInlineCodeSlots;
    a.code = inline_code ? nullptr : (rf ? p->rf_dev : vec ? p->vec_dev : early ? p->early_dev : p->code_dev);
    a.n_slots = sv.n_slots;
    a.n_tensors = (uint32_t)p->n_tensors;
    a.first = first;
    a.end = first + count;
    a.code_smem_bytes = g.code_smem;
    a.prefetch_mask = ctx->opt_prefetch ? p->prefetch_mask : 0u;
    a.zero = 0;
    a.row_area_bytes = sv.row_area_bytes;
    a.ring_bytes = sv.ring_bytes;
    a.rf_bytes = sv.rf_bytes;
    a.gather_mask = gather ? gather->mask : 0u;
    a.gather_index = gather ? gather->index : nullptr;
    a.gather_rows = gather ? gather->rows : 0u;
    a.chk_status = nullptr;
    if (a.prefetch_mask)
        for (int t = 0; t < GINT_MAX_TENSORS; t++) a.fp[t] = p->fp[t];
    a.ti = p->ti;
    for (int i = 0; i < n_tensors; i++) a.ti.base_ptr[i] = (int64_t)base_ptrs[i];
    if (inline_code) memcpy(a.inline_code, rf ? p->rf_inline : vec ? p->vec_inline : early ? p->early_inline : p->code_inline, sizeof(a.inline_code));
    void *args[1] = {&a};
    cudaError_t e = cudaLaunchKernel(g.v->fn, dim3(g.grid), dim3(gint::kThreadsPerBlock), args, g.smem, (cudaStream_t)stream);
    if (e != cudaSuccess) return fail(ctx, GINT_ERR_CUDA, "cudaLaunchKernel", e);
    return GINT_OK;
}

}  // namespace

/* ------------------------------------------------------------------------------------------------ */
/* Allocation-free indirect launches: the per-launch tables live in a fixed device array instead of context-owned
 * scratch that is grown with cudaMalloc.                                                                          */

#define GINT_STATIC_MAX_PROGRAMS 64
#define GINT_STATIC_MAX_GRID 4096

struct StaticScratch {
    gint_tensor_info ti[GINT_STATIC_MAX_PROGRAMS];        // per-program descriptor blocks, base pointers filled in
    gint::IndirectEntry table[GINT_STATIC_MAX_GRID];       // per-logical-program {code, descriptors, length}
};

/* 166 KiB that every GPU which loads this library holds until the process exits. In host code this name is only a
 * stand-in for the device object: it must never be handed to a kernel; the device address comes from
 * cudaGetSymbolAddress (static_scratch_for_device below). */
static __device__ __align__(256) unsigned char g_static_scratch[sizeof(StaticScratch)];

namespace {

constexpr int kMaxDevices = 64;
void *g_static_scratch_dev[kMaxDevices];          // device address of g_static_scratch, per device; nullptr = not set up
unsigned char g_static_host[sizeof(StaticScratch)];  // host image of the tables for the call in progress
std::mutex g_static_mu;                            // one allocation-free launch at a time: set-up, table upload and kernel launch

/* Once per device, with that device current: resolve the device address of the scratch array. The caller holds g_static_mu,
 * so two threads making their first call at the same time do the set-up once and neither sees a half-made entry. Nothing has
 * to be cleared: every call writes each table entry that its kernel reads before that kernel is queued. */
int static_scratch_for_device(gint_ctx *ctx, void **out)
{
    if (ctx->device < 0 || ctx->device >= kMaxDevices) return fail(ctx, GINT_ERR_INVALID_ARGUMENT, "device ordinal out of range");
    if (!g_static_scratch_dev[ctx->device]) {
        void *ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess || !ptr) return fail(ctx, GINT_ERR_CUDA, "cudaGetSymbolAddress(static scratch)", e);
        g_static_scratch_dev[ctx->device] = ptr;
    }
    *out = g_static_scratch_dev[ctx->device];
    return GINT_OK;
}

/* The indirect entry points upload their tables from a host image that the next call overwrites; a captured copy would read
 * that image again at every replay. They therefore refuse a stream that is being captured. */
int refuse_capture(gint_ctx *ctx, cudaStream_t stream, const char *who)
{
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    cudaError_t e = cudaStreamIsCapturing(stream, &st);
    if (e != cudaSuccess) { cudaGetLastError(); return fail(ctx, GINT_ERR_CUDA, "cudaStreamIsCapturing", e); }
    if (st != cudaStreamCaptureStatusNone) {
        std::string msg = std::string(who) + ": the stream is being captured; indirect launches cannot be part of a CUDA graph";
        return fail(ctx, GINT_ERR_INVALID_ARGUMENT, msg.c_str());
    }
    return GINT_OK;
}

}  // namespace

/* ================================================================================================ */

extern "C" {

int gint_version(void) { return 100; }

const char *gint_status_string(int status)
{
    switch (status) {
    case GINT_OK: return "ok";
    case GINT_ERR_INVALID_ARGUMENT: return "invalid argument";
    case GINT_ERR_UNKNOWN_OPCODE: return "unknown opcode";
    case GINT_ERR_STACK_UNDERFLOW: return "stack underflow";
    case GINT_ERR_STACK_OVERFLOW: return "stack overflow";
    case GINT_ERR_NO_HALT: return "program is not terminated by Halt";
    case GINT_ERR_BAD_HANDLE: return "bad program handle";
    case GINT_ERR_ARG_COUNT: return "number of arguments does not match the program";
    case GINT_ERR_CUDA: return "CUDA error";
    case GINT_ERR_NO_DEVICE: return "no usable device or kernel image";
    case GINT_ERR_TOO_LARGE: return "program or batch too large";
    case GINT_ERR_OUT_OF_MEMORY: return "out of memory";
    }
    return "unknown status";
}

int gint_sizeof_tensor_info(void) { return (int)sizeof(gint_tensor_info); }

int gint_analyze(const int32_t *code, int n_words, gint_bytecode_stats *out) { return analyze(code, n_words, out); }

int gint_predecode(const int32_t *code, int n_words, uint32_t *out_keys, int max_keys)
{
    std::vector<uint2> pre;
    std::vector<int> depths;
    int rc = predecode(code, n_words, GINT_MAX_TENSORS, &pre, &depths);
    if (rc != GINT_OK) return rc;
    gint_bytecode_stats st;
    analyze(code, n_words, &st);
    const int n = st.num_instructions + 1;
    if (out_keys) {
        if (max_keys < n) return GINT_ERR_INVALID_ARGUMENT;
        for (int i = 0; i < n; i++) out_keys[i] = (uint32_t)depths[(size_t)i] * GINT_N_OPCODES + pre[(size_t)i].y;
    }
    return n;
}

int gint_create(int device, gint_ctx **out)
{
    if (!out) return GINT_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) {
        cudaGetLastError();
        return GINT_ERR_NO_DEVICE;
    }
    DeviceGuard guard(device);
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) { cudaGetLastError(); return GINT_ERR_NO_DEVICE; }
    gint_ctx *ctx = new gint_ctx();
    ctx->device = device;
    ctx->num_sms = prop.multiProcessorCount;
    ctx->max_smem_optin = (int)prop.sharedMemPerBlockOptin;
    if (load_images() == 0) {  // the library carries sm_100a code only
        delete ctx;
        return GINT_ERR_NO_DEVICE;
    }
    for (auto &im : g_images) {
        if (!im.loaded) continue;
        if (im.K == 0) ctx->indirect.fn = (const void *)im.kernel;
        else if (im.K < 0) ctx->checked.fn = (const void *)im.kernel;
        else ctx->direct.push_back(Variant{im.P, im.K, (const void *)im.kernel, 0, false, 0, im.rf, im.vec});
    }
    int usable = 0;
    for (auto &v : ctx->direct) {
        cudaFuncAttributes attr;
        cudaError_t e = cudaFuncGetAttributes(&attr, v.fn);
        if (e == cudaSuccess) {
            v.regs = attr.numRegs;
            v.ok = true;
            usable++;
            int bps = 0;
            if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&bps, v.fn, gint::kThreadsPerBlock, 2048) == cudaSuccess)
                v.resident_warps = bps * ctx->num_sms * gint::kWarpsPerBlock;
            else cudaGetLastError();
        } else cudaGetLastError();
    }
    if (ctx->indirect.fn) {
        cudaFuncAttributes attr;
        if (cudaFuncGetAttributes(&attr, ctx->indirect.fn) == cudaSuccess) { ctx->indirect.regs = attr.numRegs; ctx->indirect.ok = true; }
        else cudaGetLastError();
    }
    if (ctx->checked.fn) {
        cudaFuncAttributes attr;
        if (cudaFuncGetAttributes(&attr, ctx->checked.fn) == cudaSuccess) { ctx->checked.regs = attr.numRegs; ctx->checked.ok = true; }
        else cudaGetLastError();
    }
    if (usable == 0) {
        delete ctx;
        return GINT_ERR_NO_DEVICE;
    }
    *out = ctx;
    return GINT_OK;
}

void gint_destroy(gint_ctx *ctx)
{
    if (!ctx) return;
    {
        DeviceGuard guard(ctx->device);
        for (Program *p : ctx->programs) {
            if (p) {
                if (p->code_dev) cudaFree(p->code_dev);
                if (p->early_dev) cudaFree(p->early_dev);
                if (p->rf_dev) cudaFree(p->rf_dev);
                if (p->vec_dev) cudaFree(p->vec_dev);
                delete p;
            }
        }
        if (ctx->status_dev) cudaFree(ctx->status_dev);
        if (ctx->ind_dev) cudaFree(ctx->ind_dev);
        if (ctx->ind_host) cudaFreeHost(ctx->ind_host);
        if (ctx->ind_event) cudaEventDestroy(ctx->ind_event);
        if (ctx->ind_kernel_event) cudaEventDestroy(ctx->ind_kernel_event);
    }
    delete ctx;
}

const char *gint_last_error(gint_ctx *ctx) { return ctx ? ctx->last_error.c_str() : "no context"; }

int gint_program_create(gint_ctx *ctx, const int32_t *code, int n_words, const gint_tensor_info *ti, int n_tensors,
                        uint64_t *out_handle)
{
    if (!ctx || !code || !out_handle || (!ti && n_tensors > 0)) return fail(ctx, GINT_ERR_INVALID_ARGUMENT, "null argument");
    if (n_tensors < 0 || n_tensors > GINT_MAX_TENSORS) return fail(ctx, GINT_ERR_INVALID_ARGUMENT, "at most 8 tensors");
    std::vector<uint2> pre;
    {
        std::vector<Insn> plain;
        int rc = normalise(code, n_words, n_tensors, &plain);
        if (rc != GINT_OK) return fail(ctx, rc, gint_status_string(rc));
        gint_bytecode_stats st0;
        analyze(code, n_words, &st0);
        if (ctx->opt_lower) lower_lane_moves(&plain, st0.pool_size);
        if (ctx->opt_fuse) fuse_sequences(&plain);
        emit_stream(plain, &pre);
    }
    Program *p = new Program();
    {
        static std::atomic<uint64_t> next_uid{1};
        p->uid = next_uid.fetch_add(1);
    }
    analyze(code, n_words, &p->st);
    p->n_tensors = n_tensors;
    p->n_slots = (uint32_t)pre.size();
    memset(&p->ti, 0, sizeof(p->ti));
    if (ti) p->ti = *ti;
    for (int t = 0; t < GINT_MAX_TENSORS; t++) p->ti.base_ptr[t] = 0;
    compute_footprints(code, p->st.num_instructions, p->ti, n_tensors, p);
    std::vector<uint2> early, rfs, vecs;
    {
        std::vector<Insn> prog;
        normalise(code, n_words, n_tensors, &prog);
        /* virtual registers in shared memory: for programs that need the 12-slot pool although their stack fits 7 slots */
        const int rf_pool = 7;
        const bool rf_ok = ctx->opt_rf_create && p->st.pool_size == 12 && p->st.max_stack <= rf_pool && p->st.max_reg_idx >= 0 &&
                           (find_variant(ctx, rf_pool, 1, true) || find_variant(ctx, rf_pool, 2, true)) && rf_equivalent(prog, p->st.pool_size);
        auto make_rf = [&](std::vector<Insn> from, bool from_early) {
            rf_rewrite(&from);
            if (ctx->opt_lower) lower_lane_moves(&from, rf_pool);
            if (ctx->opt_fuse) fuse_sequences(&from, true);
            emit_stream(from, &rfs);
            p->rf_pool = rf_pool;
            p->rf_bytes = (uint32_t)(p->st.max_reg_idx + 1) * 512u;
            p->rf_from_early = from_early;
        };
        EarlyIssue ei;
        p->ring_slots = choose_ring_slots(prog);
        early_issue_transform(prog, p->ring_slots, &ei);
        uint32_t row_area = 0, staged = 0;
        int n_staged_loads = 0;
        if (ei.n_early == 0) {   // (a program with a ring of early-issued loads keeps its cp.async groups to itself)
            staged = apply_row_staging(&ei.prog, p->ti, n_tensors, &row_area, ei.alias_slots);
            for (const Insn &in : ei.prog) n_staged_loads += in.op == OP_LoadStagedRows;
        }
        /* fast row accesses are tried on a copy: they count only if the early stream is used at all */
        uint32_t fast_rows = 0;
        {
            std::vector<Insn> probe = ei.prog;
            fast_rows = apply_fast_rows(&probe, p->ti, n_tensors);
        }
        bool usable = ei.n_early > 0 || staged != 0 || fast_rows != 0;
        /* A slot that the program moves (AdvanceBase / AdvanceBlock2D) reaches beyond the extent its descriptor gives, so
         * the launch-time overlap check cannot bound it: a program that pairs such a slot with a moved load keeps the
         * stream as written. */
        uint32_t advanced = 0;
        for (const Insn &in : prog)
            if (in.op == OP_AdvanceBlock2D || in.op == OP_AdvanceBase) advanced |= 1u << (in.operand & 7u);
        for (int t = 0; t < n_tensors; t++) {
            p->extent[t] = tensor_extent_bytes(p->ti, t);
            p->alias_slots[t] = ei.alias_slots[t];
            if (ei.alias_slots[t] && (p->extent[t] == 0 || ((advanced >> t) & 1u))) usable = false;
            for (int b = 0; b < n_tensors; b++)
                if ((ei.alias_slots[t] >> b) & 1u) { if (tensor_extent_bytes(p->ti, b) == 0 || ((advanced >> b) & 1u)) usable = false; }
        }
        if (usable) {
            p->fast_slots = apply_fast_accesses(&ei.prog, p->ti, n_tensors) | apply_fast_rows(&ei.prog, p->ti, n_tensors) | staged;
            p->row_area_bytes = row_area;
            if (rf_ok) make_rf(ei.prog, true);
            if (ctx->opt_vec && p->st.pool_size == 4 && (find_variant(ctx, 4, 1, false, true) || find_variant(ctx, 4, 2, false, true))) {
                std::vector<Insn> v;
                int n_vector = 0, n_remaps = 0;
                if (vec_transform(ei.prog, &v, &n_vector, &n_remaps) && vec_worth_it(n_vector, n_remaps)) {
                    if (ctx->opt_lower) lower_lane_moves(&v, p->st.pool_size);
                    if (ctx->opt_fuse) fuse_sequences(&v);
                    emit_stream(v, &vecs);
                    p->vec_remaps = n_remaps;
                }
            }
            if (ctx->opt_lower) lower_lane_moves(&ei.prog, p->st.pool_size);
            if (ctx->opt_fuse) fuse_sequences(&ei.prog);
            emit_stream(ei.prog, &early);
            p->n_early = ei.n_early;
        } else {
            for (int t = 0; t < n_tensors; t++) p->alias_slots[t] = 0;
            n_staged_loads = 0;
            if (rf_ok) make_rf(prog, false);
        }
        int n_mem = 0, n_loads = 0;
        for (const Insn &in : prog) {
            if (!is_tensor_op(in.op) || in.op == OP_AdvanceBlock2D || in.op == OP_AdvanceBase) continue;
            n_mem++;
            if (!writes_tensor(in.op)) n_loads++;
        }
        {
            std::vector<uint32_t> seen, again;
            for (const Insn &in : prog) {
                if (in.op != OP_LoadGlobal1DF32) continue;   // row passes; the 4x4 programs' repeated row loads are L1 hits
                bool known = false, counted = false;
                for (uint32_t s : seen) known = known || s == in.operand;
                for (uint32_t s : again) counted = counted || s == in.operand;
                if (known && !counted) again.push_back(in.operand);
                if (!known) seen.push_back(in.operand);
            }
            p->reread_bytes = (uint32_t)again.size() * 512u;
        }
        const int n_insns = (int)prog.size(), n_direct = n_loads - (usable ? ei.n_early + n_staged_loads : 0);
        /* One tile per warp for programs bound by memory instructions (2 of 5 instructions access memory), and for programs
         * with many loads that are neither issued early nor staged WHEN the wider kernel costs occupancy (pools of 7 and 12:
         * 96 and 128 registers at two tiles against 64 and 95 at one). With the 4-slot pool two tiles per warp cost one block
         * per SM (72 against 64 registers) and double the loads each warp keeps in flight: measured on the bf16 RMSNorm of
         * the reference's tests (2DT tiles, no early issue), 180 us at two tiles per warp against 221 us at one. */
        p->prefer_narrow = 5 * n_mem >= 2 * n_insns || (p->st.pool_size >= 7 && 5 * n_direct >= n_insns);
    }
    p->early_slots = (uint32_t)early.size();
    p->rf_slots = (uint32_t)rfs.size();
    p->vec_slots = (uint32_t)vecs.size();
    for (int i = 0; i < gint::kInlineCodeSlots; i++) {
        p->code_inline[i] = (size_t)i < pre.size() ? pre[(size_t)i] : make_uint2(0u, OP_Halt);
        p->early_inline[i] = (size_t)i < early.size() ? early[(size_t)i] : make_uint2(0u, OP_Halt);
        p->rf_inline[i] = (size_t)i < rfs.size() ? rfs[(size_t)i] : make_uint2(0u, OP_Halt);
        p->vec_inline[i] = (size_t)i < vecs.size() ? vecs[(size_t)i] : make_uint2(0u, OP_Halt);
    }
    {
        DeviceGuard guard(ctx->device);
        cudaError_t e = cudaMalloc(&p->code_dev, pre.size() * sizeof(uint2));
        if (e != cudaSuccess) { delete p; return fail(ctx, GINT_ERR_OUT_OF_MEMORY, "cudaMalloc(program)", e); }
        e = cudaMemcpy(p->code_dev, pre.data(), pre.size() * sizeof(uint2), cudaMemcpyHostToDevice);
        if (e != cudaSuccess) { cudaFree(p->code_dev); delete p; return fail(ctx, GINT_ERR_CUDA, "cudaMemcpy(program)", e); }
        if (!early.empty()) {
            e = cudaMalloc(&p->early_dev, early.size() * sizeof(uint2));
            if (e == cudaSuccess) e = cudaMemcpy(p->early_dev, early.data(), early.size() * sizeof(uint2), cudaMemcpyHostToDevice);
            if (e != cudaSuccess) {
                if (p->early_dev) cudaFree(p->early_dev);
                cudaFree(p->code_dev);
                delete p;
                return fail(ctx, GINT_ERR_OUT_OF_MEMORY, "cudaMalloc/cudaMemcpy(early-issue program)", e);
            }
        }
        if (!rfs.empty()) {
            e = cudaMalloc(&p->rf_dev, rfs.size() * sizeof(uint2));
            if (e == cudaSuccess) e = cudaMemcpy(p->rf_dev, rfs.data(), rfs.size() * sizeof(uint2), cudaMemcpyHostToDevice);
            if (e != cudaSuccess) {
                if (p->rf_dev) cudaFree(p->rf_dev);
                if (p->early_dev) cudaFree(p->early_dev);
                cudaFree(p->code_dev);
                delete p;
                return fail(ctx, GINT_ERR_OUT_OF_MEMORY, "cudaMalloc/cudaMemcpy(register-file program)", e);
            }
        }
        if (!vecs.empty()) {
            e = cudaMalloc(&p->vec_dev, vecs.size() * sizeof(uint2));
            if (e == cudaSuccess) e = cudaMemcpy(p->vec_dev, vecs.data(), vecs.size() * sizeof(uint2), cudaMemcpyHostToDevice);
            if (e != cudaSuccess) {
                if (p->vec_dev) cudaFree(p->vec_dev);
                if (p->rf_dev) cudaFree(p->rf_dev);
                if (p->early_dev) cudaFree(p->early_dev);
                cudaFree(p->code_dev);
                delete p;
                return fail(ctx, GINT_ERR_OUT_OF_MEMORY, "cudaMalloc/cudaMemcpy(vector-layout program)", e);
            }
        }
    }
    p->live = true;
    std::lock_guard<std::mutex> lk(ctx->mu);
    ctx->programs.push_back(p);
    *out_handle = (uint64_t)ctx->programs.size();
    return GINT_OK;
}

int gint_program_destroy(gint_ctx *ctx, uint64_t handle)
{
    if (!ctx) return GINT_ERR_INVALID_ARGUMENT;
    Program *p = nullptr;
    {
        std::lock_guard<std::mutex> lk(ctx->mu);
        if (handle == 0 || handle > ctx->programs.size() || !ctx->programs[handle - 1]) return fail(ctx, GINT_ERR_BAD_HANDLE, "unknown program handle");
        p = ctx->programs[handle - 1];
        ctx->programs[handle - 1] = nullptr;
    }
    DeviceGuard guard(ctx->device);
    /* the program may still be running on some stream: cudaFree waits for the device */
    if (p->code_dev) cudaFree(p->code_dev);
    if (p->early_dev) cudaFree(p->early_dev);
    if (p->rf_dev) cudaFree(p->rf_dev);
    if (p->vec_dev) cudaFree(p->vec_dev);
    delete p;
    return GINT_OK;
}

int gint_program_launch_info(gint_ctx *ctx, uint64_t handle, uint32_t grid_dim, gint_launch_info *out)
{
    if (!ctx || !out) return fail(ctx, GINT_ERR_INVALID_ARGUMENT, "null argument");
    Program *p = lookup(ctx, handle);
    if (!p) return fail(ctx, GINT_ERR_BAD_HANDLE, "unknown program handle");
    DeviceGuard guard(ctx->device);
    Geometry g;
    const bool early = ctx->opt_early_issue && p->early_dev != nullptr;
    const bool rf = ctx->opt_rf && p->rf_dev != nullptr && p->rf_from_early == early;
    const bool vec = ctx->opt_vec && p->vec_dev != nullptr && early && !rf && !p->prefer_narrow && ctx->opt_tiles_per_warp != 1;
    StreamView sv = stream_view(p, early, rf, vec);
    int rc = plan_direct(ctx, p, sv, grid_dim ? grid_dim : 1, &g);
    if (rc != GINT_OK && (rf || vec)) {
        sv = stream_view(p, early, false);
        rc = plan_direct(ctx, p, sv, grid_dim ? grid_dim : 1, &g);
    }
    if (rc != GINT_OK) return rc;
    memset(out, 0, sizeof(*out));
    out->pool_size = g.v->P;
    out->tiles_per_warp = g.v->K;
    out->warps_per_block = gint::kWarpsPerBlock;
    out->grid_blocks = (int32_t)g.grid;
    out->smem_bytes = (int32_t)g.smem;
    out->regs_per_thread = g.v->regs;
    out->blocks_per_sm = g.blocks_per_sm;
    out->num_sms = ctx->num_sms;
    out->early_loads = p->n_early;
    out->registers_in_smem = g.v->rf ? p->st.max_reg_idx + 1 : 0;
    out->vector_layout = g.v->vec ? 1 : 0;
    return GINT_OK;
}

int gint_execute(gint_ctx *ctx, uint64_t handle, const uint64_t *base_ptrs, int n_tensors, uint32_t grid_dim, void *cuda_stream)
{
    return launch_direct(ctx, handle, base_ptrs, n_tensors, 0u, grid_dim, cuda_stream);
}

int gint_execute_range(gint_ctx *ctx, uint64_t handle, const uint64_t *base_ptrs, int n_tensors, uint32_t first, uint32_t count,
                       void *cuda_stream)
{
    return launch_direct(ctx, handle, base_ptrs, n_tensors, first, count, cuda_stream);
}

int gint_execute_gathered(gint_ctx *ctx, uint64_t handle, const uint64_t *base_ptrs, int n_tensors, uint32_t grid_dim, uint32_t gather_mask,
                          const int64_t *row_index, uint32_t table_rows, uint64_t gathered_extent_bytes, void *cuda_stream)
{
    if (!ctx) return GINT_ERR_INVALID_ARGUMENT;
    if (gather_mask == 0) return launch_direct(ctx, handle, base_ptrs, n_tensors, 0u, grid_dim, cuda_stream);
    if (!row_index || table_rows == 0) return fail(ctx, GINT_ERR_INVALID_ARGUMENT, "gathered rows need a row index and a table with at least one row");
    if (n_tensors < 0 || n_tensors > GINT_MAX_TENSORS || (gather_mask >> n_tensors) != 0) return fail(ctx, GINT_ERR_INVALID_ARGUMENT, "gather mask names a slot the program does not have");
    GatherArgs ga{gather_mask, reinterpret_cast<const long long *>(row_index), gathered_extent_bytes, table_rows};
    return launch_direct(ctx, handle, base_ptrs, n_tensors, 0u, grid_dim, cuda_stream, &ga);
}

int gint_execute_checked(gint_ctx *ctx, uint64_t handle, const uint64_t *base_ptrs, const uint64_t *lo, const uint64_t *hi, int n_tensors,
                         uint32_t grid_dim, void *cuda_stream)
{
    if (!ctx || ((!base_ptrs || !lo || !hi) && n_tensors > 0)) return fail(ctx, GINT_ERR_INVALID_ARGUMENT, "null argument");
    Program *p = lookup(ctx, handle);
    if (!p) return fail(ctx, GINT_ERR_BAD_HANDLE, "unknown program handle");
    if (n_tensors != p->n_tensors) return fail(ctx, GINT_ERR_ARG_COUNT, "number of arguments does not match the program");
    if (!ctx->checked.ok) return fail(ctx, GINT_ERR_NO_DEVICE, "checked kernel image not usable on this device");
    if (grid_dim == 0) return GINT_OK;
    DeviceGuard guard(ctx->device);
    cudaStream_t stream = (cudaStream_t)cuda_stream;
    {
        int rc = refuse_capture(ctx, stream, "gint_execute_checked");
        if (rc != GINT_OK) return rc;
    }
    {
        std::lock_guard<std::mutex> lk(ctx->mu);
        if (!ctx->status_dev) {
            cudaError_t e = cudaMalloc(&ctx->status_dev, sizeof(gint_device_status));
            if (e == cudaSuccess) e = cudaMemset(ctx->status_dev, 0, sizeof(gint_device_status));
            if (e != cudaSuccess) { ctx->status_dev = nullptr; return fail(ctx, GINT_ERR_OUT_OF_MEMORY, "cudaMalloc(device status)", e); }
        }
    }
    const StreamView sv = stream_view(p, false);      // the program as written
    uint32_t code_smem = 0;
    const uint32_t smem = direct_smem(sv, 1, &code_smem);
    if ((int)smem > ctx->max_smem_optin) return fail(ctx, GINT_ERR_TOO_LARGE, "program too long for the checked kernel (shared memory)");
    cudaError_t e;
    if (smem > 48u * 1024u) {
        e = cudaFuncSetAttribute(ctx->checked.fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(ctx, GINT_ERR_CUDA, "cudaFuncSetAttribute(checked)", e);
    }
    int bps = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&bps, ctx->checked.fn, gint::kThreadsPerBlock, smem);
    if (e != cudaSuccess || bps < 1) return fail(ctx, GINT_ERR_CUDA, "occupancy query (checked)", e);
    uint64_t blocks = blocks_for(grid_dim, 1);
    const uint64_t resident = (uint64_t)bps * (uint64_t)ctx->num_sms;
    if (blocks > resident) blocks = resident;
    LaunchArgs a;
    memset(&a, 0, sizeof(a));
    a.code = p->code_dev;
    a.n_slots = sv.n_slots;
    a.n_tensors = (uint32_t)p->n_tensors;
    a.first = 0;
    a.end = grid_dim;
    a.code_smem_bytes = code_smem;
    a.ti = p->ti;
    for (int i = 0; i < n_tensors; i++) {
        a.ti.base_ptr[i] = (int64_t)base_ptrs[i];
        a.chk_lo[i] = lo[i];
        a.chk_hi[i] = hi[i];
    }
    a.chk_status = ctx->status_dev;
    void *args[1] = {&a};
    e = cudaLaunchKernel(ctx->checked.fn, dim3((unsigned)blocks), dim3(gint::kThreadsPerBlock), args, smem, stream);
    if (e != cudaSuccess) return fail(ctx, GINT_ERR_CUDA, "cudaLaunchKernel(checked)", e);
    return GINT_OK;
}

int gint_device_status_read(gint_ctx *ctx, gint_device_status *out, int clear)
{
    if (!ctx || !out) return fail(ctx, GINT_ERR_INVALID_ARGUMENT, "null argument");
    memset(out, 0, sizeof(*out));
    if (!ctx->status_dev) return GINT_OK;     // no checked launch so far
    DeviceGuard guard(ctx->device);
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaMemcpy(out, ctx->status_dev, sizeof(*out), cudaMemcpyDeviceToHost);
    if (e == cudaSuccess && clear) e = cudaMemset(ctx->status_dev, 0, sizeof(*out));
    if (e != cudaSuccess) return fail(ctx, GINT_ERR_CUDA, "reading the device status", e);
    return GINT_OK;
}

int gint_execute_plan(gint_ctx *ctx, const gint_plan_step *steps, int n_steps, void *cuda_stream)
{
    if (!ctx || (!steps && n_steps > 0) || n_steps < 0) return fail(ctx, GINT_ERR_INVALID_ARGUMENT, "null or negative plan");
    for (int i = 0; i < n_steps; i++) {
        const gint_plan_step &st = steps[i];
        if (st.grid_dim == 0) continue;
        if (st.n_tensors < 0 || st.n_tensors > GINT_MAX_TENSORS) return fail(ctx, GINT_ERR_INVALID_ARGUMENT, "plan step: tensor count out of range");
        const int rc = launch_direct(ctx, st.handle, st.base_ptrs, st.n_tensors, 0u, st.grid_dim, cuda_stream);
        if (rc != GINT_OK) {
            char msg[320];
            snprintf(msg, sizeof msg, "plan step %d of %d: %s", i, n_steps, ctx->last_error.c_str());
            ctx->last_error = msg;
            return rc;
        }
    }
    return GINT_OK;
}

int gint_execute_indirect(gint_ctx *ctx, const uint64_t *handles, int n_programs, const uint64_t *base_ptrs, const int32_t *indices,
                          uint32_t grid_dim, void *cuda_stream)
{
    if (!ctx || !handles || !base_ptrs || !indices || n_programs <= 0) return fail(ctx, GINT_ERR_INVALID_ARGUMENT, "null argument");
    if (grid_dim == 0) return GINT_OK;
    if (!ctx->indirect.ok) return fail(ctx, GINT_ERR_NO_DEVICE, "indirect kernel image not usable on this device");
    std::vector<Program *> progs((size_t)n_programs);
    int max_tensors = 0;
    uint32_t max_slots = 0;
    for (int i = 0; i < n_programs; i++) {
        progs[(size_t)i] = lookup(ctx, handles[i]);
        if (!progs[(size_t)i]) return fail(ctx, GINT_ERR_BAD_HANDLE, "unknown program handle");
        if (progs[(size_t)i]->n_tensors > max_tensors) max_tensors = progs[(size_t)i]->n_tensors;
        if (progs[(size_t)i]->n_slots > max_slots) max_slots = progs[(size_t)i]->n_slots;
    }
    /* each warp keeps its own program in shared memory */
    const uint32_t code_smem = (max_slots * 8u + 127u) & ~127u;
    const uint32_t smem = (uint32_t)gint::kWarpsPerBlock * ((uint32_t)sizeof(gint::TileInfo) + (uint32_t)gint::kTensorInfoSmemBytes + code_smem);
    if ((int)smem > ctx->max_smem_optin) return fail(ctx, GINT_ERR_TOO_LARGE, "a program of this batch is too long for indirect mode (shared memory)");
    for (uint32_t i = 0; i < grid_dim; i++)
        if (indices[i] < 0 || indices[i] >= n_programs) return fail(ctx, GINT_ERR_INVALID_ARGUMENT, "program index out of range");

    DeviceGuard guard(ctx->device);
    cudaStream_t stream = (cudaStream_t)cuda_stream;
    {
        int rc = refuse_capture(ctx, stream, "gint_execute_indirect");
        if (rc != GINT_OK) return rc;
    }
    /* One indirect launch of a context at a time builds its tables: the scratch (host image and device copy) is shared by
     * every call, and its layout depends on n_programs. */
    std::lock_guard<std::mutex> ind_lock(ctx->ind_mu);
    /* scratch layout: [n_programs x gint_tensor_info | grid_dim x IndirectEntry] */
    const size_t ti_bytes = (size_t)n_programs * sizeof(gint_tensor_info);
    const size_t need = ti_bytes + (size_t)grid_dim * sizeof(IndirectEntry);
    if (need > ctx->ind_bytes) {
        if (ctx->ind_event) cudaEventSynchronize(ctx->ind_event);
        if (ctx->ind_kernel_event) cudaEventSynchronize(ctx->ind_kernel_event);   // the previous kernel still reads the old scratch
        if (ctx->ind_dev) { cudaFree(ctx->ind_dev); ctx->ind_dev = nullptr; }
        if (ctx->ind_host) { cudaFreeHost(ctx->ind_host); ctx->ind_host = nullptr; }
        ctx->ind_bytes = 0;
        const size_t cap = need < 65536 ? 65536 : need * 2;
        cudaError_t e = cudaMalloc(&ctx->ind_dev, cap);
        if (e != cudaSuccess) return fail(ctx, GINT_ERR_OUT_OF_MEMORY, "cudaMalloc(indirect scratch)", e);
        e = cudaMallocHost(&ctx->ind_host, cap);
        if (e != cudaSuccess) { cudaFree(ctx->ind_dev); ctx->ind_dev = nullptr; return fail(ctx, GINT_ERR_OUT_OF_MEMORY, "cudaMallocHost(indirect scratch)", e); }
        ctx->ind_bytes = cap;
    }
    if (!ctx->ind_event) {
        cudaError_t e = cudaEventCreateWithFlags(&ctx->ind_event, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ctx->ind_kernel_event, cudaEventDisableTiming);
        if (e != cudaSuccess) return fail(ctx, GINT_ERR_CUDA, "cudaEventCreate", e);
    } else {
        cudaEventSynchronize(ctx->ind_event);  // the previous launch's upload has left the staging buffer
        /* ... and the previous launch's KERNEL, possibly on another stream, must be done with the device copy of the
         * tables before this upload overwrites them: this stream waits for it (a no-op on the same stream) */
        cudaError_t e = cudaStreamWaitEvent(stream, ctx->ind_kernel_event, 0);
        if (e != cudaSuccess) return fail(ctx, GINT_ERR_CUDA, "cudaStreamWaitEvent(indirect)", e);
    }
    gint_tensor_info *h_ti = (gint_tensor_info *)ctx->ind_host;
    IndirectEntry *h_tab = (IndirectEntry *)((char *)ctx->ind_host + ti_bytes);
    const gint_tensor_info *d_ti = (const gint_tensor_info *)ctx->ind_dev;
    for (int i = 0; i < n_programs; i++) {
        h_ti[i] = progs[(size_t)i]->ti;
        for (int t = 0; t < progs[(size_t)i]->n_tensors; t++) h_ti[i].base_ptr[t] = (int64_t)base_ptrs[(size_t)i * GINT_MAX_TENSORS + (size_t)t];
    }
    for (uint32_t i = 0; i < grid_dim; i++) {
        h_tab[i].code = progs[(size_t)indices[i]]->code_dev;
        h_tab[i].ti = d_ti + indices[i];
        h_tab[i].n_slots = progs[(size_t)indices[i]]->n_slots;
        h_tab[i].patch_slot = 0;
        h_tab[i].patch_ptr = 0;
    }
    cudaError_t e = cudaMemcpyAsync(ctx->ind_dev, ctx->ind_host, need, cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) return fail(ctx, GINT_ERR_CUDA, "cudaMemcpyAsync(indirect tables)", e);
    cudaEventRecord(ctx->ind_event, stream);

    IndirectArgs a;
    a.table = (const IndirectEntry *)((const char *)ctx->ind_dev + ti_bytes);
    a.n_tensors = (uint32_t)max_tensors;
    a.grid_dim = grid_dim;
    a.code_smem_bytes = code_smem;
    a.reserved = 0;
    if (smem > 48u * 1024u) {
        e = cudaFuncSetAttribute(ctx->indirect.fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(ctx, GINT_ERR_CUDA, "cudaFuncSetAttribute(indirect)", e);
    }
    int bps = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&bps, ctx->indirect.fn, gint::kThreadsPerBlock, smem);
    if (e != cudaSuccess || bps < 1) return fail(ctx, GINT_ERR_CUDA, "occupancy query (indirect)", e);
    uint64_t blocks = ((uint64_t)grid_dim + gint::kWarpsPerBlock - 1) / gint::kWarpsPerBlock;
    const uint64_t resident = (uint64_t)bps * (uint64_t)ctx->num_sms;
    if (blocks > resident) blocks = resident;
    void *args[1] = {&a};
    e = cudaLaunchKernel(ctx->indirect.fn, dim3((unsigned)blocks), dim3(gint::kThreadsPerBlock), args, smem, stream);
    /* recorded whether or not the launch succeeded: the next call waits on this event and it must not be left unrecorded */
    cudaEventRecord(ctx->ind_kernel_event, stream);
    if (e != cudaSuccess) return fail(ctx, GINT_ERR_CUDA, "cudaLaunchKernel(indirect)", e);
    return GINT_OK;
}

int gint_execute_batch(gint_ctx *ctx, const int32_t *codes, int n_programs, int n_words, const gint_tensor_info *ti, int n_tensors,
                       const uint64_t *base_ptrs, int out_slot, uint64_t out_stride_bytes, int32_t *status_out, void *cuda_stream)
{
    if (!ctx || !codes || !ti || !base_ptrs || n_programs < 0 || n_words <= 0 || (n_words & 1)) return fail(ctx, GINT_ERR_INVALID_ARGUMENT, "null or malformed argument");
    if (n_tensors < 1 || n_tensors > GINT_MAX_TENSORS || out_slot < 0 || out_slot >= n_tensors) return fail(ctx, GINT_ERR_INVALID_ARGUMENT, "tensor count or output slot out of range");
    if (n_programs == 0) return GINT_OK;
    if (!ctx->indirect.ok) return fail(ctx, GINT_ERR_NO_DEVICE, "indirect kernel image not usable on this device");
    /* every candidate is pre-decoded into a slice of `stride` entries: its instructions, the lead entry and the tail */
    const uint32_t stride = (uint32_t)((n_words / 2 + 4 + 1) & ~1);
    const uint32_t code_smem = (stride * 8u + 127u) & ~127u;
    const uint32_t smem = (uint32_t)gint::kWarpsPerBlock * ((uint32_t)sizeof(gint::TileInfo) + (uint32_t)gint::kTensorInfoSmemBytes + code_smem);
    if ((int)smem > ctx->max_smem_optin) return fail(ctx, GINT_ERR_TOO_LARGE, "candidate programs too long for indirect mode (shared memory)");

    DeviceGuard guard(ctx->device);
    cudaStream_t stream = (cudaStream_t)cuda_stream;
    {
        int rc = refuse_capture(ctx, stream, "gint_execute_batch");
        if (rc != GINT_OK) return rc;
    }
    std::lock_guard<std::mutex> ind_lock(ctx->ind_mu);
    /* scratch layout: [one gint_tensor_info, padded to 640 | n_programs x IndirectEntry | n_programs x stride x uint2] */
    const size_t ti_bytes = 640, tab_bytes = (size_t)n_programs * sizeof(IndirectEntry);
    const size_t code_off = (ti_bytes + tab_bytes + 15) & ~(size_t)15;
    const size_t need = code_off + (size_t)n_programs * stride * sizeof(uint2);
    if (need > ctx->ind_bytes) {
        if (ctx->ind_event) cudaEventSynchronize(ctx->ind_event);
        if (ctx->ind_kernel_event) cudaEventSynchronize(ctx->ind_kernel_event);
        if (ctx->ind_dev) { cudaFree(ctx->ind_dev); ctx->ind_dev = nullptr; }
        if (ctx->ind_host) { cudaFreeHost(ctx->ind_host); ctx->ind_host = nullptr; }
        ctx->ind_bytes = 0;
        const size_t cap = need < 65536 ? 65536 : need * 2;
        cudaError_t e = cudaMalloc(&ctx->ind_dev, cap);
        if (e != cudaSuccess) return fail(ctx, GINT_ERR_OUT_OF_MEMORY, "cudaMalloc(batch scratch)", e);
        e = cudaMallocHost(&ctx->ind_host, cap);
        if (e != cudaSuccess) { cudaFree(ctx->ind_dev); ctx->ind_dev = nullptr; return fail(ctx, GINT_ERR_OUT_OF_MEMORY, "cudaMallocHost(batch scratch)", e); }
        ctx->ind_bytes = cap;
    }
    if (!ctx->ind_event) {
        cudaError_t e = cudaEventCreateWithFlags(&ctx->ind_event, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ctx->ind_kernel_event, cudaEventDisableTiming);
        if (e != cudaSuccess) return fail(ctx, GINT_ERR_CUDA, "cudaEventCreate", e);
    } else {
        cudaEventSynchronize(ctx->ind_event);
        cudaError_t e = cudaStreamWaitEvent(stream, ctx->ind_kernel_event, 0);
        if (e != cudaSuccess) return fail(ctx, GINT_ERR_CUDA, "cudaStreamWaitEvent(batch)", e);
    }
    gint_tensor_info *h_ti = (gint_tensor_info *)ctx->ind_host;
    IndirectEntry *h_tab = (IndirectEntry *)((char *)ctx->ind_host + ti_bytes);
    uint2 *h_code = (uint2 *)((char *)ctx->ind_host + code_off);
    const char *d_base = (const char *)ctx->ind_dev;
    *h_ti = *ti;
    for (int t = 0; t < n_tensors; t++) h_ti->base_ptr[t] = (int64_t)base_ptrs[t];
    std::vector<uint2> pre;
    int n_valid = 0;
    for (int i = 0; i < n_programs; i++) {
        IndirectEntry &en = h_tab[i];
        en.code = (const uint2 *)(d_base + code_off) + (size_t)i * stride;
        en.ti = (const gint_tensor_info *)d_base;
        en.patch_slot = (uint32_t)out_slot + 1u;
        en.patch_ptr = base_ptrs[out_slot] + (uint64_t)i * out_stride_bytes;
        const int rc = predecode(codes + (size_t)i * (size_t)n_words, n_words, n_tensors, &pre);
        if (status_out) status_out[i] = rc;
        if (rc != GINT_OK || pre.size() > stride) {
            if (status_out && rc == GINT_OK) status_out[i] = GINT_ERR_TOO_LARGE;
            en.n_slots = 0;                 // the warp skips this candidate; its output row is left as it is
            continue;
        }
        en.n_slots = (uint32_t)pre.size();
        memcpy(h_code + (size_t)i * stride, pre.data(), pre.size() * sizeof(uint2));
        n_valid++;
    }
    cudaError_t e = cudaMemcpyAsync(ctx->ind_dev, ctx->ind_host, need, cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) return fail(ctx, GINT_ERR_CUDA, "cudaMemcpyAsync(batch tables)", e);
    cudaEventRecord(ctx->ind_event, stream);
    if (n_valid == 0) { cudaEventRecord(ctx->ind_kernel_event, stream); return GINT_OK; }

    IndirectArgs a;
    a.table = (const IndirectEntry *)(d_base + ti_bytes);
    a.n_tensors = (uint32_t)n_tensors;
    a.grid_dim = (uint32_t)n_programs;
    a.code_smem_bytes = code_smem;
    a.reserved = 0;
    if (smem > 48u * 1024u) {
        e = cudaFuncSetAttribute(ctx->indirect.fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(ctx, GINT_ERR_CUDA, "cudaFuncSetAttribute(indirect)", e);
    }
    int bps = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&bps, ctx->indirect.fn, gint::kThreadsPerBlock, smem);
    if (e != cudaSuccess || bps < 1) return fail(ctx, GINT_ERR_CUDA, "occupancy query (indirect)", e);
    uint64_t blocks = ((uint64_t)n_programs + gint::kWarpsPerBlock - 1) / gint::kWarpsPerBlock;
    const uint64_t resident = (uint64_t)bps * (uint64_t)ctx->num_sms;
    if (blocks > resident) blocks = resident;
    void *args[1] = {&a};
    e = cudaLaunchKernel(ctx->indirect.fn, dim3((unsigned)blocks), dim3(gint::kThreadsPerBlock), args, smem, stream);
    cudaEventRecord(ctx->ind_kernel_event, stream);
    if (e != cudaSuccess) return fail(ctx, GINT_ERR_CUDA, "cudaLaunchKernel(batch)", e);
    return GINT_OK;
}

int gint_execute_indirect_static(gint_ctx *ctx, const uint64_t *handles, int n_programs, const uint64_t *base_ptrs,
                                 const int32_t *indices, uint32_t grid_dim, void *cuda_stream)
{
    if (!ctx || !handles || !base_ptrs || !indices || n_programs <= 0) return fail(ctx, GINT_ERR_INVALID_ARGUMENT, "null argument");
    if (n_programs > GINT_STATIC_MAX_PROGRAMS)
        return fail(ctx, GINT_ERR_TOO_LARGE, "gint_execute_indirect_static: more than 64 programs in one launch");
    if (grid_dim > GINT_STATIC_MAX_GRID)
        return fail(ctx, GINT_ERR_TOO_LARGE, "gint_execute_indirect_static: more than 4096 logical programs in one launch");
    if (grid_dim == 0) return GINT_OK;
    if (!ctx->indirect.ok) return fail(ctx, GINT_ERR_NO_DEVICE, "indirect kernel image not usable on this device");
    Program *progs[GINT_STATIC_MAX_PROGRAMS];
    int max_tensors = 0;
    uint32_t max_slots = 0;
    for (int i = 0; i < n_programs; i++) {
        progs[i] = lookup(ctx, handles[i]);
        if (!progs[i]) return fail(ctx, GINT_ERR_BAD_HANDLE, "unknown program handle");
        if (progs[i]->n_tensors > max_tensors) max_tensors = progs[i]->n_tensors;
        if (progs[i]->n_slots > max_slots) max_slots = progs[i]->n_slots;
    }
    for (uint32_t i = 0; i < grid_dim; i++)
        if (indices[i] < 0 || indices[i] >= n_programs) return fail(ctx, GINT_ERR_INVALID_ARGUMENT, "program index out of range");
    const uint32_t code_smem = (max_slots * 8u + 127u) & ~127u;
    const uint32_t smem = (uint32_t)gint::kWarpsPerBlock * ((uint32_t)sizeof(gint::TileInfo) + (uint32_t)gint::kTensorInfoSmemBytes + code_smem);
    if ((int)smem > ctx->max_smem_optin) return fail(ctx, GINT_ERR_TOO_LARGE, "a program of this batch is too long for indirect mode (shared memory)");

    DeviceGuard guard(ctx->device);
    cudaStream_t stream = (cudaStream_t)cuda_stream;
    int rc = refuse_capture(ctx, stream, "gint_execute_indirect_static");
    if (rc != GINT_OK) return rc;
    /* Held from set-up to the kernel launch: the host image is shared, and the uploads and the launch of one call must not be
     * interleaved with another thread's. */
    std::lock_guard<std::mutex> lk(g_static_mu);
    void *scratch = nullptr;
    rc = static_scratch_for_device(ctx, &scratch);  // first call on a device: resolves the array's device address
    if (rc != GINT_OK) return rc;
    const StaticScratch *d = reinterpret_cast<const StaticScratch *>(scratch);
    cudaError_t e;
    {
        StaticScratch *h = reinterpret_cast<StaticScratch *>(g_static_host);
        for (int i = 0; i < n_programs; i++) {
            h->ti[i] = progs[i]->ti;
            for (int t = 0; t < progs[i]->n_tensors; t++) h->ti[i].base_ptr[t] = (int64_t)base_ptrs[(size_t)i * GINT_MAX_TENSORS + (size_t)t];
        }
        for (uint32_t i = 0; i < grid_dim; i++) {
            h->table[i].code = progs[indices[i]]->code_dev;
            h->table[i].ti = d->ti + indices[i];
            h->table[i].n_slots = progs[indices[i]]->n_slots;
            h->table[i].patch_slot = 0;
            h->table[i].patch_ptr = 0;
        }
        /* Two copies of exactly the used parts. The source is ordinary (pageable) host memory: the runtime stages it and
         * returns once the host image may be reused by the next call. */
        e = cudaMemcpyAsync(scratch, h, (size_t)n_programs * sizeof(gint_tensor_info), cudaMemcpyHostToDevice, stream);
        if (e == cudaSuccess)
            e = cudaMemcpyAsync((char *)scratch + offsetof(StaticScratch, table), h->table, (size_t)grid_dim * sizeof(IndirectEntry),
                                cudaMemcpyHostToDevice, stream);
    }
    if (e != cudaSuccess) return fail(ctx, GINT_ERR_CUDA, "cudaMemcpyAsync(static indirect tables)", e);

    IndirectArgs a;
    a.table = d->table;
    a.n_tensors = (uint32_t)max_tensors;
    a.grid_dim = grid_dim;
    a.code_smem_bytes = code_smem;
    a.reserved = 0;
    if (smem > 48u * 1024u) {
        e = cudaFuncSetAttribute(ctx->indirect.fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(ctx, GINT_ERR_CUDA, "cudaFuncSetAttribute(indirect)", e);
    }
    int bps = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&bps, ctx->indirect.fn, gint::kThreadsPerBlock, smem);
    if (e != cudaSuccess || bps < 1) return fail(ctx, GINT_ERR_CUDA, "occupancy query (indirect)", e);
    uint64_t blocks = ((uint64_t)grid_dim + gint::kWarpsPerBlock - 1) / gint::kWarpsPerBlock;
    const uint64_t resident = (uint64_t)bps * (uint64_t)ctx->num_sms;
    if (blocks > resident) blocks = resident;
    void *args[1] = {&a};
    e = cudaLaunchKernel(ctx->indirect.fn, dim3((unsigned)blocks), dim3(gint::kThreadsPerBlock), args, smem, stream);
    if (e != cudaSuccess) return fail(ctx, GINT_ERR_CUDA, "cudaLaunchKernel(indirect, static tables)", e);
    return GINT_OK;
}

int gint_debug_transform(const int32_t *code, int n_words, const gint_tensor_info *ti, int n_tensors, int early_issue, int fuse,
                         int32_t *out_ops, uint32_t *out_operands, int max_insns)
{
    std::vector<Insn> prog;
    int rc = normalise(code, n_words, n_tensors, &prog);
    if (rc != GINT_OK) return rc;
    if (early_issue & 1) {
        gint_bytecode_stats st;
        analyze(code, n_words, &st);
        EarlyIssue ei;
        early_issue_transform(prog, choose_ring_slots(prog), &ei);
        prog = ei.prog;
        if (ti) {
            gint_tensor_info t0 = *ti;
            uint32_t row_area = 0, staged = 0;
            if (ei.n_early == 0) staged = apply_row_staging(&prog, t0, n_tensors, &row_area, ei.alias_slots);
            uint32_t rows_fast = 0;
            {
                std::vector<Insn> probe = prog;
                rows_fast = apply_fast_rows(&probe, t0, n_tensors);
            }
            if (ei.n_early > 0 || staged || rows_fast) {
                apply_fast_accesses(&prog, t0, n_tensors);
                apply_fast_rows(&prog, t0, n_tensors);
            }
        }
    }
    if (early_issue & 4) {   // the stream for the vector-layout kernels, if the program qualifies (needs the early-issue pass)
        gint_bytecode_stats st0;
        analyze(code, n_words, &st0);
        std::vector<Insn> v;
        int n_vector = 0, n_remaps = 0;
        if (!(early_issue & 1) || st0.pool_size != 4 || !vec_transform(prog, &v, &n_vector, &n_remaps) || !vec_worth_it(n_vector, n_remaps)) return 0;
        prog = v;
    }
    if (early_issue & 2) {   // the stream for the kernels with virtual registers in shared memory, if the program qualifies
        gint_bytecode_stats st0;
        analyze(code, n_words, &st0);
        std::vector<Insn> plain;
        normalise(code, n_words, n_tensors, &plain);
        if (!(st0.pool_size == 12 && st0.max_stack <= 7 && st0.max_reg_idx >= 0 && rf_equivalent(plain, st0.pool_size))) return 0;
        rf_rewrite(&prog);
        if (fuse) {
            lower_lane_moves(&prog, 7);
            fuse_sequences(&prog, true);
        }
    } else if (fuse) {
        gint_bytecode_stats st0;
        analyze(code, n_words, &st0);
        lower_lane_moves(&prog, st0.pool_size);
        fuse_sequences(&prog);
    }
    if ((int)prog.size() > max_insns) return GINT_ERR_INVALID_ARGUMENT;
    for (size_t i = 0; i < prog.size(); i++) {
        if (out_ops) out_ops[i] = prog[i].op == OP_CARRIER_UNUSED ? OP_CARRIER : prog[i].op;
        if (out_operands) out_operands[i] = prog[i].operand;
    }
    return (int)prog.size();
}

int gint_debug_fused_table(int32_t *out, int max_entries)
{
    if (!out || max_entries < GINT_N_FUSED + GINT_N_RF_FUSED) return GINT_ERR_INVALID_ARGUMENT;
    for (int k = 0; k < GINT_N_FUSED + GINT_N_RF_FUSED; k++) {
        int32_t *row = out + (size_t)k * (2 + GINT_MAX_FUSED_LEN);
        row[0] = kFused[k].num;
        row[1] = kFused[k].len;
        for (int j = 0; j < GINT_MAX_FUSED_LEN; j++) row[2 + j] = j < kFused[k].len ? kFused[k].ops[j] : -1;
    }
    return GINT_N_FUSED + GINT_N_RF_FUSED;
}

int gint_set_option(gint_ctx *ctx, const char *name, int value)
{
    if (!ctx || !name) return GINT_ERR_INVALID_ARGUMENT;
    if (strcmp(name, "tiles_per_warp") == 0) {
        if (value != 0 && value != 1 && value != 2 && value != 4) return fail(ctx, GINT_ERR_INVALID_ARGUMENT, "tiles_per_warp must be 0, 1, 2 or 4");
        ctx->opt_tiles_per_warp = value;
        return GINT_OK;
    }
    if (strcmp(name, "fuse") == 0) {
        ctx->opt_fuse = value != 0;
        return GINT_OK;
    }
    if (strcmp(name, "lower") == 0) {
        ctx->opt_lower = value != 0;
        return GINT_OK;
    }
    if (strcmp(name, "early_issue") == 0) {
        ctx->opt_early_issue = value != 0;
        return GINT_OK;
    }
    if (strcmp(name, "register_file") == 0) {   // virtual registers in shared memory: programs created and launches made from now on
        ctx->opt_rf = ctx->opt_rf_create = value != 0;
        return GINT_OK;
    }
    if (strcmp(name, "vector_layout") == 0) {   // programs created and launches made from now on
        ctx->opt_vec = value != 0;
        return GINT_OK;
    }
    if (strcmp(name, "prefetch") == 0) {
        ctx->opt_prefetch = value != 0;
        return GINT_OK;
    }
    if (strcmp(name, "max_blocks") == 0) {
        ctx->opt_max_blocks = value < 0 ? 0 : value;
        return GINT_OK;
    }
    return fail(ctx, GINT_ERR_INVALID_ARGUMENT, "unknown option");
}

}  // extern "C"
