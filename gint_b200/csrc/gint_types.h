/*
 * gint_types.h -- structures shared by the interpreter kernels (gint_interp.cuh) and the host side (gint_capi.cu).
 */
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/gint_b200.h"
#include "gint_opcodes.h"

namespace gint {

typedef unsigned long long u64;

constexpr int kWarpsPerBlock = 4;
constexpr int kThreadsPerBlock = kWarpsPerBlock * 32;
constexpr int kTensorInfoSmemBytes = 640;  // 608-byte descriptor block, padded to a 128-byte multiple
constexpr int kNumKeys = (GINT_MAX_STACK + 1) * GINT_N_DISPATCH;

/* Slots of the ring of early-issued loads: how many tile loads per logical program are in flight ahead of their use. The
 * host chooses per program: 8 for programs that stream long rows (many loads, mostly memory instructions), 4 otherwise. */
constexpr int kRingSlotsShallow = 4, kRingSlotsDeep = 8;

/* Minimum resident blocks per SM requested from the compiler (caps registers per thread): the pool itself takes 4*P*K
 * registers; addresses and interpreter state take about 40 more. */
#ifndef GINT_MIN_BLOCKS_WIDE
#define GINT_MIN_BLOCKS_WIDE 4   /* for the widest pool (12 slots x 2 tiles = 96 pool registers) */
#endif
#ifndef GINT_MIN_BLOCKS
#define GINT_MIN_BLOCKS(P, K) ((P) * (K) <= 7 ? 8 : (P) * (K) <= 8 ? 7 : (P) * (K) <= 16 ? 5 : GINT_MIN_BLOCKS_WIDE)
#endif

/* Per logical program, decoded once into shared memory (the reference's BlockTensorInfo,
 * load_tensor_infos.py:6-11, plus a flags word): 256 bytes. */
struct __align__(16) TileInfo {
    u64 ptr[GINT_MAX_TENSORS];   // base pointer with the per-program offset applied
    int2 s1[GINT_MAX_TENSORS];   // (shape1 clamped to this program's tile, stride1)
    int2 s2[GINT_MAX_TENSORS];   // (shape2 clamped, stride2)
    int adv[GINT_MAX_TENSORS];   // AdvanceBlock2D accumulator
    int flags[GINT_MAX_TENSORS]; // kVecRows: 2DW rows are 16-byte vectorisable
};
constexpr int kVecRows = 1;

/* What a program reads from one tensor, per logical program, found by a static walk over its (straight-line) bytecode:
 * the element range [lo, hi) relative to the tile origin along the contiguous dimension. */
enum { FP_NONE = 0, FP_1D = 1, FP_ROWS = 2 };
struct Footprint {
    int32_t kind;  // FP_1D: 1-D tiles, elements [lo, hi) of the block; FP_ROWS: 2DW tiles, columns [lo, hi) of each of the 32 rows
    int32_t lo, hi;
    int32_t reserved;
};

constexpr int kInlineCodeSlots = 24;   // stream entries that fit into the parameter block (programs of up to ~20 instructions)

struct LaunchArgs {
    const uint2 *code;        // pre-decoded {operand, next opcode} entries; n_slots of them, padded with Halt; nullptr: inline_code
    uint32_t n_slots;         // entries staged into shared memory (even, so the copy is a 16-byte multiple)
    uint32_t n_tensors;
    uint32_t first;           // first logical program of this launch
    uint32_t end;             // one past the last logical program
    uint32_t code_smem_bytes; // shared-memory bytes reserved for the program
    uint32_t prefetch_mask;   // bit t set: prefetch tensor t's footprint into L2 when a tile's descriptors are decoded
    uint32_t zero;            // always 0; a zero the assembler cannot see (fma_barrier in gint_interp.cuh)
    uint32_t row_area_bytes;  // shared-memory bytes per tile for staged row blocks (StageRows), 0 if the program has none
    uint32_t ring_bytes;      // shared-memory bytes per tile for the ring of early-issued loads, 0 if the stream has none
    uint32_t rf_bytes;        // shared-memory bytes per tile for virtual registers (kernels built with GINT_RF; 512 per register), else 0
    Footprint fp[GINT_MAX_TENSORS];
    gint_tensor_info ti;      // descriptor block, base pointers patched per call: travels as a kernel parameter
    uint2 inline_code[kInlineCodeSlots];   // the program itself when it has at most kInlineCodeSlots entries (code == nullptr)
    /* checked launches only (gint_execute_checked): declared byte range [lo, hi) of every tensor and the status word */
    u64 chk_lo[GINT_MAX_TENSORS], chk_hi[GINT_MAX_TENSORS];
    void *chk_status;
    /* gathered rows (gint_execute_gathered): for the tensor slots in gather_mask the index along the innermost batch dimension
     * is replaced by gather_index[that index] before it is multiplied by the batch stride */
    const long long *gather_index;
    uint32_t gather_mask;
    uint32_t gather_rows;     // rows of the gathered table: a negative index counts from the end, anything else is clamped into range
};

struct IndirectEntry {
    const uint2 *code;              // pre-decoded program of this logical program
    const gint_tensor_info *ti;     // its descriptor block in device memory
    uint32_t n_slots;               // entries in `code`; 0: nothing to run (an invalid candidate of a batch)
    uint32_t patch_slot;            // 1 + tensor slot whose base pointer is replaced by patch_ptr for this logical program; 0: none
    u64 patch_ptr;                  // (batches of candidate programs share one descriptor block and differ in one pointer)
};


struct IndirectArgs {
    const IndirectEntry *table;
    uint32_t n_tensors;       // maximum over the batch (executor_impl.py:192)
    uint32_t grid_dim;
    uint32_t code_smem_bytes; // shared-memory bytes reserved per warp for its program
    uint32_t reserved;        // always 0; doubles as the zero the assembler cannot see (fma_barrier in gint_interp.cuh)
};

}  // namespace gint
