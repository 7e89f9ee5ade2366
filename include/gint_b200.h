/*
 * gint_b200.h -- C ABI of the B200-native gint bytecode executor (libgint_b200.so).
 *
 * The reference (eliphatfs/gint) has no C ABI: its executor is Python over the CUDA driver bindings.
 * Each entry point below replaces one piece of that Python executor; the citation names the reference
 * code it stands in for. Plain pointers and sizes only; every function returns GINT_OK (0) or a negative
 * gint_status, never throws and never aborts. Device pointers are passed as uint64_t, the CUDA stream as
 * the raw CUstream / cudaStream_t handle (what torch.cuda.current_stream().cuda_stream holds).
 *
 * Threading: a gint_ctx may be used from several host threads; program creation/destruction take an
 * internal lock, launches are lock-free. One gint_ctx per device.
 */
#ifndef GINT_B200_H
#define GINT_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GINT_MAX_TENSORS 8  /* gint/kernel/platforms/common.py:63 (MAX_N_TENSORS) */

/*
 * Tensor descriptor block, byte-identical to the reference's host struct HTensorInfo
 * (gint/kernel/interpreter/structs.py:19-30): struct-of-arrays over 8 tensor slots, 608 bytes.
 * batch_strides / batch_shape are in REVERSED order (index 0 = innermost batch dim), padded with
 * stride 0 / shape 1 (gint/host/utils.py:6-27).
 */
typedef struct gint_tensor_info {
    int64_t base_ptr[GINT_MAX_TENSORS];
    int32_t elm_size[GINT_MAX_TENSORS];
    int32_t batch_strides[GINT_MAX_TENSORS][4];
    int32_t batch_shape[GINT_MAX_TENSORS][4];
    int32_t block_shape_stride_1[GINT_MAX_TENSORS][2];
    int32_t block_shape_stride_2[GINT_MAX_TENSORS][2];
    int32_t block_grid_dims[GINT_MAX_TENSORS][2];
    int32_t block_grid_steps[GINT_MAX_TENSORS][2];
} gint_tensor_info;

typedef enum gint_status {
    GINT_OK = 0,
    GINT_ERR_INVALID_ARGUMENT = -1,  /* null pointer, bad count, odd word count ... */
    GINT_ERR_UNKNOWN_OPCODE = -2,    /* gint/host/analyzer.py:205-208 raises ValueError */
    GINT_ERR_STACK_UNDERFLOW = -3,   /* gint/host/analyzer.py:209-213 raises ValueError */
    GINT_ERR_STACK_OVERFLOW = -4,    /* deeper than any kernel geometry (8) */
    GINT_ERR_NO_HALT = -5,           /* stream not terminated by opcode 0 */
    GINT_ERR_BAD_HANDLE = -6,
    GINT_ERR_ARG_COUNT = -7,         /* gint/host/cuda/executor_impl.py:93-94 raises ValueError */
    GINT_ERR_CUDA = -8,              /* a CUDA runtime call failed; see gint_last_error() */
    GINT_ERR_NO_DEVICE = -9,         /* no usable sm_100 device / kernel image */
    GINT_ERR_TOO_LARGE = -10,        /* program or batch exceeds a documented limit */
    GINT_ERR_OUT_OF_MEMORY = -11
} gint_status;

/* Result of the static walk over a straight-line program (gint/host/analyzer.py:137-158, BytecodeStats). */
typedef struct gint_bytecode_stats {
    int32_t num_instructions; /* up to, not including, the first Halt */
    int32_t max_stack;
    int32_t max_reg_idx;      /* -1 if no virtual register is touched */
    int32_t min_pool_size;
    int32_t regs_used_mask;   /* bit n set = register n touched */
    int32_t error_index;      /* instruction index of the first error, -1 if none */
    int32_t pool_size;        /* pool geometry this library runs the program with: 4, 7 or 12 */
    int32_t reserved;
} gint_bytecode_stats;

/* How a program will be / was launched; for tests and benchmarks. */
typedef struct gint_launch_info {
    int32_t pool_size;        /* 4, 7, 12 */
    int32_t tiles_per_warp;   /* logical programs interpreted together by one warp: 1, 2 or 4 */
    int32_t warps_per_block;
    int32_t grid_blocks;
    int32_t smem_bytes;
    int32_t regs_per_thread;
    int32_t blocks_per_sm;
    int32_t num_sms;
    int32_t early_loads;      /* tile loads per logical program that are started ahead of their use (early issue) */
    int32_t registers_in_smem; /* virtual registers kept in shared memory (the pool then holds the operand stack alone); 0: in the pool */
    int32_t vector_layout;    /* 1: full 1-D tiles live in the pool with lane l holding elements 4l..4l+3 (16-byte accesses) */
    int32_t reserved[5];
} gint_launch_info;

/* What a checked launch (gint_execute_checked) found; all zero = nothing. The FIRST event is described, `count` counts all. */
typedef enum gint_device_code {
    GINT_DEVICE_OK = 0,
    GINT_DEVICE_LOAD_OUT_OF_RANGE = 1,    /* a tile load or gather outside the tensor's declared byte range: skipped, value 0 */
    GINT_DEVICE_STORE_OUT_OF_RANGE = 2,   /* a tile store or scatter outside it: skipped */
    GINT_DEVICE_INSTRUCTION_BUDGET = 3,   /* more instructions executed than the program holds (a dispatch error): stopped */
    GINT_DEVICE_BAD_DISPATCH = 4          /* no handler for an (opcode, stack depth) pair; `address` holds the key: stopped */
} gint_device_code;

typedef struct gint_device_status {
    int32_t code;             /* gint_device_code of the first event */
    int32_t slot;             /* tensor slot of the access, -1 if not applicable */
    uint32_t logical_program; /* logical program (warp tile) in which it happened */
    uint32_t instruction;     /* index of the instruction in the bytecode stream */
    uint64_t address;         /* the address that was refused */
    uint32_t lane;            /* lane of the warp (0..31) */
    uint32_t count;           /* number of events in all */
} gint_device_status;

typedef struct gint_ctx gint_ctx;

/* ---- host-only helpers: no GPU needed ---------------------------------------------------------- */

/* Library version (major*10000 + minor*100 + patch). */
int gint_version(void);

/* Human-readable name of a status code. */
const char *gint_status_string(int status);

/* sizeof(gint_tensor_info); lets a binding check its struct layout (608). */
int gint_sizeof_tensor_info(void);

/* Static analysis of a bytecode stream. Replaces analyze_bytecode (gint/host/analyzer.py:187-238) and
 * select_variant (gint/host/executor.py:131-149). n_words = 2 * number of instructions. */
int gint_analyze(const int32_t *code, int n_words, gint_bytecode_stats *out);

/* Pre-decode a stream into the kernel's internal form (for tests): out_keys[i] receives the dispatch key of
 * instruction i (stack depth * number of opcodes + opcode). Returns the instruction count incl. Halt, or < 0. */
int gint_predecode(const int32_t *code, int n_words, uint32_t *out_keys, int max_keys);

/* The instruction list the kernels actually run for a program, after the optional early-issue and fusion passes (for
 * tests; no GPU needed): out_ops[i] is a format opcode, an internal opcode (>= 106) or -1 for an instruction absorbed into
 * the fused handler before it. With early_issue != 0 the descriptors in `ti` also decide which 1-D accesses become their
 * "fast" forms (provably full, aligned tiles). early_issue is a bit set: 1 = the early-issue pass, 2 = the stream for the
 * kernels that keep the virtual registers in shared memory (FLoadRegN / FStoreRegN become RLoad / RStore with the register in
 * the operand; returns 0 if the program does not qualify for them), 4 = the stream for the vector-layout kernels (with 1; RemapVN
 * inserted where a value must be in the natural layout; 0 if the program does not qualify). Returns the number of instructions
 * (including the Halt) or < 0. */
int gint_debug_transform(const int32_t *code, int n_words, const gint_tensor_info *ti, int n_tensors, int early_issue, int fuse,
                         int32_t *out_ops, uint32_t *out_operands, int max_insns);

/* The fused-handler table: rows of 10 ints {opcode number, length, 8 member opcodes (padded with -1)}. Returns the row count. */
int gint_debug_fused_table(int32_t *out, int max_entries);

/* ---- context ------------------------------------------------------------------------------------ */

/* Create the executor state for one device, using that device's primary context (the one PyTorch uses).
 * Replaces CudaExecutor.__init__ / geval_func_handle (gint/host/cuda/executor_impl.py:14-37) and
 * current_context/fatbin_load (gint/host/cuda/driver.py:84-95,162-169). */
int gint_create(int device, gint_ctx **out);
void gint_destroy(gint_ctx *ctx);

/* Message of the last failure on this context (thread-unsafe convenience, never NULL). */
const char *gint_last_error(gint_ctx *ctx);

/* ---- programs ----------------------------------------------------------------------------------- */

/* Validate, pre-decode and upload a program together with its static descriptor template
 * (base_ptr values are ignored here). Replaces the cache-miss half of CudaExecutor.execute,
 * _build_cacheline (gint/host/cuda/executor_impl.py:76-133) and fill_tensor_info's consumer.
 * Allocates device memory; call outside stream capture. */
int gint_program_create(gint_ctx *ctx, const int32_t *code, int n_words, const gint_tensor_info *ti,
                        int n_tensors, uint64_t *out_handle);
int gint_program_destroy(gint_ctx *ctx, uint64_t handle);

/* Geometry the library would use to launch `handle` over grid_dim logical programs. */
int gint_program_launch_info(gint_ctx *ctx, uint64_t handle, uint32_t grid_dim, gint_launch_info *out);

/* ---- launches ----------------------------------------------------------------------------------- */

/* Launch the interpreter over logical programs [0, grid_dim). base_ptrs[i] is the device address for
 * descriptor slot i. Asynchronous on `cuda_stream`; performs no allocation and no host<->device copy
 * (descriptors travel as kernel parameters), so it is legal during stream capture and every captured
 * launch is self-contained. Replaces the cache-hit half of CudaExecutor.execute
 * (gint/host/cuda/executor_impl.py:63-74: base-pointer patch, 608-byte H2D copy, cuLaunchKernel). */
int gint_execute(gint_ctx *ctx, uint64_t handle, const uint64_t *base_ptrs, int n_tensors, uint32_t grid_dim,
                 void *cuda_stream);

/* Same, restricted to logical programs [first, first + count) of the program's grid: the primitive used to
 * shard one program over several GPUs by its leading dimension (each rank passes base pointers biased by its
 * shard's byte offset). No counterpart in the reference, which is single-GPU. */
int gint_execute_range(gint_ctx *ctx, uint64_t handle, const uint64_t *base_ptrs, int n_tensors, uint32_t first,
                       uint32_t count, void *cuda_stream);

/* gint_execute with every global-memory access checked: `lo[i]` / `hi[i]` give the byte range [lo, hi) that descriptor slot i
 * may touch (the tensor view the caller handed over). The program runs as written, on a slower kernel (one logical program
 * per warp, no early-issued loads, no fused handlers); an access outside its tensor's range is not performed (a load yields
 * 0) and is recorded in a status word that gint_device_status_read returns. The reference has no counterpart: an invalid
 * program is undefined behaviour there (gint/kernel/interpreter/main.py:245-248) and the only tool is an external memory
 * checker; this is the bounds-checking debug mode for program and descriptor development. Allocates the status word on first
 * use; not for stream capture. */
int gint_execute_checked(gint_ctx *ctx, uint64_t handle, const uint64_t *base_ptrs, const uint64_t *lo, const uint64_t *hi,
                         int n_tensors, uint32_t grid_dim, void *cuda_stream);

/* Wait for the device, copy the status word of the checked launches so far into *out and, if `clear` is not 0, reset it. */
int gint_device_status_read(gint_ctx *ctx, gint_device_status *out, int clear);

/* gint_execute with gathered rows: for every descriptor slot in `gather_mask`, the index along the tensor's INNERMOST batch
 * dimension -- b = 0 .. batch_shape-1, normally multiplied by the batch stride -- is first looked up in the device array
 * row_index[b] (int64). Logical program b thus works on row row_index[b] of the tensor at base_ptrs[slot]: `table[index]` is
 * read (or written) in place, without the separate gather kernel and the intermediate copy that the reference needs for the
 * same graph (its conductor leaves aten.index.Tensor to torch eager, gint/conductor/op_registry.py:1058-1132; the interpreter's
 * own gather opcode, 66, picks single elements). table_rows = rows of the table: a negative index counts from the end, as in
 * torch; an index that is still out of range (an error in torch) is clamped to the nearest row, so no access leaves the
 * table. gathered_extent_bytes = bytes of the table from its base pointer (used by the launch-time overlap check in place
 * of the descriptor's extent). Offsets are 32-bit element counts like every other descriptor term. No counterpart in the
 * reference. Same launch properties as gint_execute. */
int gint_execute_gathered(gint_ctx *ctx, uint64_t handle, const uint64_t *base_ptrs, int n_tensors, uint32_t grid_dim,
                          uint32_t gather_mask, const int64_t *row_index, uint32_t table_rows, uint64_t gathered_extent_bytes,
                          void *cuda_stream);

/* One step of a plan: a program, the device addresses of its tensors and its logical grid. */
typedef struct gint_plan_step {
    uint64_t handle;
    uint64_t base_ptrs[GINT_MAX_TENSORS];
    int32_t n_tensors;
    uint32_t grid_dim;
} gint_plan_step;

/* Launch a list of programs back to back on one stream with a single call: what a compiled graph is once it has been
 * lowered -- the conductor's `execute` closure walks such a list in Python, one executor call and one 608-byte upload
 * per subgraph (gint/conductor/compiler.py:1442-1485; the reference measured 36-90 us of CPU dispatch per call against a
 * 62 us kernel, docs/conductor.md:94). Steps run in order (stream order); the call stops at the first step that fails,
 * returns its status and names the step in gint_last_error. Same properties as gint_execute: no allocation, no copy,
 * legal during stream capture. A step with grid_dim 0 is skipped. */
int gint_execute_plan(gint_ctx *ctx, const gint_plan_step *steps, int n_steps, void *cuda_stream);

/* One launch in which logical program i runs programs[indices[i]] with that program's own tensors.
 * base_ptrs holds n_programs rows of GINT_MAX_TENSORS addresses. Replaces CudaExecutor.execute_indirect
 * (gint/host/cuda/executor_impl.py:135-201). Uses context-owned scratch for the per-warp tables and may grow it
 * (allocation) on a call with a larger batch than any before. Indirect launches of one context are serialised: a call
 * holds a context lock while it builds and queues its tables, and its upload waits (on the GPU, through an event) for
 * the previous indirect kernel of the context, whichever stream that ran on, so calls from several threads or streams
 * cannot overwrite tables that are still being read. Not for stream capture: the tables are uploaded from a host image
 * that the next call overwrites, so a stream that is being captured is refused with GINT_ERR_INVALID_ARGUMENT. Of the
 * launch entry points only gint_execute, gint_execute_range and gint_execute_plan may be captured. */
int gint_execute_indirect(gint_ctx *ctx, const uint64_t *handles, int n_programs, const uint64_t *base_ptrs,
                          const int32_t *indices, uint32_t grid_dim, void *cuda_stream);

/* A batch of candidate programs, one launch: candidate i (the n_words int32 words at codes + i * n_words) runs as ONE logical
 * program over the tensors of `base_ptrs` with the descriptors of `ti`, except that the base pointer of descriptor slot
 * `out_slot` is base_ptrs[out_slot] + i * out_stride_bytes (every candidate writes its own output row). Replaces the batch
 * path of the reference's superoptimizer example (examples/superopt/executor.py:100-186: per candidate a 608-byte descriptor
 * block is packed in Python, then bytecode, blocks and two pointer tables are uploaded and geval is launched with flag 1;
 * its profile puts 55 % of the batch time into that packing loop, examples/superopt/bench/README.md:92-120): here the
 * candidates are analysed and pre-decoded in C, ONE descriptor block is shared and the per-candidate pointer travels in the
 * table entry. A candidate that fails the analysis (unknown opcode, stack underflow or overflow, no Halt) is skipped -- its
 * output row is left as it is -- and its gint_status is stored in status_out[i] (0 for the others; status_out may be NULL).
 * Shares the context's indirect scratch and its serialisation (see gint_execute_indirect); may allocate; not for capture. */
int gint_execute_batch(gint_ctx *ctx, const int32_t *codes, int n_programs, int n_words, const gint_tensor_info *ti, int n_tensors,
                       const uint64_t *base_ptrs, int out_slot, uint64_t out_stride_bytes, int32_t *status_out, void *cuda_stream);

/* Indirect launch that allocates nothing. No counterpart in the reference (whose execute_indirect allocates and frees
 * on every call). Same arguments and same results as gint_execute_indirect, but the per-launch tables (one descriptor
 * block per program, one {program, descriptors} entry per logical program) are written into a fixed 166 KiB array that
 * lives in the library's device image, not into context scratch that grows with cudaMalloc. It exists for callers that
 * are not allowed to allocate device memory when they launch: processes whose whole device-memory budget has been handed
 * to another allocator (a framework's caching pool, a partitioned inference server), control loops with a hard deadline
 * that cannot absorb the device-wide stall an allocation may cause, and deployments where the set of permitted driver
 * calls is audited and cudaMalloc / cudaFree are not on the list. This call performs no cudaMalloc, cudaFree, cudaMallocHost
 * or any other allocating routine, on the device or in a library.
 *   Limits: n_programs <= 64 and grid_dim <= 4096; anything larger is refused with GINT_ERR_TOO_LARGE (and a message in
 *     gint_last_error) before any work is queued. Use gint_execute_indirect for larger batches.
 *   Set-up: the first call on a device resolves the array's device address (cudaGetSymbolAddress, which may load the
 *     library's device code); make that first call before any stream capture begins in the process and outside
 *     latency-critical sections. Set-up and the rest of the call run under one process-wide lock, so first calls from
 *     several threads are safe.
 *   Capture: like gint_execute_indirect this call uploads its tables from a host image that the next call overwrites, so
 *     it refuses a stream that is being captured (GINT_ERR_INVALID_ARGUMENT).
 *   Sharing: every call on a device, from any context or thread, uses the same array, and the array keeps the previous
 *     call's tables until they are overwritten. Each call rewrites every entry it is going to read (nothing has to start
 *     at zero), but two of these launches that can overlap on the GPU -- different streams without an ordering between
 *     them -- race on the tables: the second upload may replace entries the first kernel has not read yet. Issue them
 *     on one stream, or order the streams with events. */
int gint_execute_indirect_static(gint_ctx *ctx, const uint64_t *handles, int n_programs, const uint64_t *base_ptrs,
                                 const int32_t *indices, uint32_t grid_dim, void *cuda_stream);

/* ---- tuning knobs (benchmarks / tests) ---------------------------------------------------------- */

/* Knobs for later launches: "tiles_per_warp" (0 = automatic, else upper bound 1/2/4), "early_issue" (1 = start tile
 * loads ahead of their use when safe, default; 0 = keep loads where they are), "fuse" (1 = replace known instruction
 * sequences by fused handlers, default; applies to programs created afterwards), "prefetch" (L2 footprint prefetch,
 * default 0), "max_blocks" (cap on the persistent grid, 0 = none), "lower" (1 = lane indices of DupBroadcastW move into the
 * opcode, default; programs created afterwards), "register_file" (1 = programs that need the 12-slot pool only for their
 * virtual registers keep those in shared memory and run on a kernel whose pool is the operand stack alone, default),
 * "vector_layout" (1 = programs created from now on whose full 1-D tiles can live in the pool as four consecutive elements
 * per lane run on the kernels that access them with one 16-byte access per lane; default 0: no measurable gain on the
 * benchmark programs). */
int gint_set_option(gint_ctx *ctx, const char *name, int value);

#ifdef __cplusplus
}
#endif
#endif /* GINT_B200_H */
