/*
 * gint_interp.cuh -- the gint stack-machine interpreter as hand-written CUDA C++ for sm_100a.
 *
 * What it replaces: the reference's llvmlite-generated kernels geval_s7 / geval_l12
 * (gint/kernel/interpreter/main.py:171-294 and everything under gint/kernel/interpreter/instructions/).
 * Semantics are kept per opcode; the execution strategy is new:
 *
 *   - The program is pre-decoded on the host into {dispatch key, operand} pairs, where the key already
 *     combines the opcode with the (statically known) stack depth, and is staged ONCE per thread block into
 *     shared memory. Every warp reads it with warp-uniform addresses, so dispatch never diverges. The
 *     reference re-reads opcode and operand from global memory in every warp (instruction.py:19-36).
 *   - The operand stack and the virtual registers live in registers: every handler is instantiated per stack
 *     depth, so all pool indices are compile-time constants (the reference gets the same effect by cloning
 *     its dispatch block per depth, main.py:201-257).
 *   - One warp interprets K logical programs ("tiles") side by side (K = 1, 2 or 4): one fetch/decode/branch
 *     is amortised over K x 128 values and K independent memory streams are in flight per warp.
 *   - The four width lanes of a slot are held as two packed f32x2 registers; add/sub/mul/fma use the
 *     Blackwell packed-f32x2 instructions, halving FP issue.
 *   - Tile loads/stores take a 128-bit path when the descriptor allows it (2DW rows) and an unpredicated
 *     4 x 128-byte coalesced path for full unit-stride 1-D tiles.
 *   - The grid is persistent: blocks loop over groups of K logical programs.
 *
 * Tensor cores are not used: none of the opcodes is a contraction.
 */
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <utility>

#include "../../include/gint_b200.h"
#include "gint_fused.h"
#include "gint_opcodes.h"
#include "gint_types.h"

/* GINT_GUARD: debugging aid for changes to the dispatch machinery. Every handler decrements an instruction budget (the
 * number of stream entries) and the interpreter returns when it runs out, so a mis-wired jump table cannot spin forever. */
#ifdef GINT_CHECKED
#define GINT_GUARD 1
#define GINT_GUARD_TRIPPED gint::chk_record(GINT_DEVICE_INSTRUCTION_BUDGET, -1, 0ull)
#else
#define GINT_GUARD_TRIPPED
#endif
#ifdef GINT_GUARD
#define GINT_GUARD_STEP                                                                                               \
    {                                                                                                                 \
        uint32_t left;                                                                                                \
        asm volatile("sub.u32 %%gbudget, %%gbudget, 1; mov.u32 %0, %%gbudget;" : "=r"(left));                         \
        if ((int)left < 0) { GINT_GUARD_TRIPPED; return; }                                                            \
    }
#else
#define GINT_GUARD_STEP
#endif

namespace gint {

/* ------------------------------------------------------------------------------------------------ */
/* checked build (GINT_CHECKED): every global-memory access of a program is compared with the byte range its tensor was
 * declared to occupy; an access outside it is NOT performed and the first such event is recorded in a status word that the
 * host reads (gint_device_status in gint_b200.h). Compiled into one extra kernel (kernels/gint_checked_p12.cu); in the
 * ordinary kernels GINT_CHK is the constant true and leaves no trace in the code.                                    */
#ifdef GINT_CHECKED
struct CheckState {
    u64 lo[GINT_MAX_TENSORS], hi[GINT_MAX_TENSORS];   // declared byte range [lo, hi) of every tensor slot
    gint_device_status *status;
    uint32_t code_base;                               // shared-memory address of the staged program
    uint32_t logical[kWarpsPerBlock];                 // first logical program of the group each warp is interpreting
};
static __shared__ CheckState g_chk;

__device__ __forceinline__ void chk_record(int code, int slot, u64 address)
{
    gint_device_status *st = g_chk.status;
    if (atomicCAS(&st->code, 0, code) == 0) {
        uint32_t gc;
        asm volatile("mov.b32 %0, %%gc;" : "=r"(gc));
        st->slot = slot;
        st->address = address;
        st->logical_program = g_chk.logical[threadIdx.x >> 5];
        st->instruction = (gc - g_chk.code_base) / 8u - 3u;   // %gc points three entries past the instruction in progress
        st->lane = threadIdx.x & 31;
    }
    atomicAdd(&st->count, 1u);
}
__device__ __forceinline__ bool chk_access(int slot, const void *p, int bytes, bool store)
{
    const u64 a = reinterpret_cast<u64>(p);
    if (a >= g_chk.lo[slot] && a + (u64)bytes <= g_chk.hi[slot]) return true;
    chk_record(store ? GINT_DEVICE_STORE_OUT_OF_RANGE : GINT_DEVICE_LOAD_OUT_OF_RANGE, slot, a);
    return false;
}
#define GINT_CHK(slot, p, bytes, store) gint::chk_access((slot), (p), (bytes), (store))
#else
#define GINT_CHK(slot, p, bytes, store) true
#endif

/* ------------------------------------------------------------------------------------------------ */
/* packed f32x2 helpers                                                                              */

struct Slot { u64 a, b; };  // a = width lanes (0,1), b = width lanes (2,3)

__device__ __forceinline__ u64 pack2(float x, float y)
{
    u64 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(x), "f"(y));
    return r;
}
__device__ __forceinline__ void unpack2(u64 v, float &x, float &y)
{
    asm("mov.b64 {%0, %1}, %2;" : "=f"(x), "=f"(y) : "l"(v));
}
__device__ __forceinline__ u64 add2(u64 x, u64 y)
{
    u64 r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(x), "l"(y));
    return r;
}
__device__ __forceinline__ u64 sub2(u64 x, u64 y)
{
    u64 r;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(x), "l"(y));
    return r;
}
__device__ __forceinline__ u64 mul2(u64 x, u64 y)
{
    u64 r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(x), "l"(y));
    return r;
}
__device__ __forceinline__ u64 fma2(u64 x, u64 y, u64 z)
{
    u64 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(x), "l"(y), "l"(z));
    return r;
}
__device__ __forceinline__ Slot make_slot(float v0, float v1, float v2, float v3)
{
    Slot s;
    s.a = pack2(v0, v1);
    s.b = pack2(v2, v3);
    return s;
}
__device__ __forceinline__ void slot_get(const Slot &s, float (&v)[4])
{
    unpack2(s.a, v[0], v[1]);
    unpack2(s.b, v[2], v[3]);
}
__device__ __forceinline__ Slot splat(float x)
{
    Slot s;
    s.a = pack2(x, x);
    s.b = s.a;
    return s;
}

/* llvm.maximum / llvm.minimum of the reference (nvptx.py:97-100): NaN if either input is NaN */
__device__ __forceinline__ float max_nan(float x, float y)
{
    float r;
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(x), "f"(y));
    return r;
}
__device__ __forceinline__ float min_nan(float x, float y)
{
    float r;
    asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(x), "f"(y));
    return r;
}

/* ------------------------------------------------------------------------------------------------ */
/* rarely used, code-heavy math: one out-of-line copy shared by every stack depth                    */

static __device__ __noinline__ float slow_math(int op, float t, float s)
{
    switch (op) {
    case OP_FRem: return fmodf(t, s);
    case OP_FArcSin: return asinf(t);
    case OP_FArcCos: return acosf(t);
    case OP_FArcTan: return atanf(t);
    case OP_FArcTan2: return atan2f(t, s);
    case OP_FPow: return powf(t, s);
    case OP_FErf: return erff(t);
    case OP_FTan: return __tanf(t);
    case OP_FLog: return logf(t);
    case OP_FLog2: return log2f(t);
    case OP_IDiv: {
        int a = __float_as_int(t), b = __float_as_int(s);
        int r = b == 0 ? -1 : (a == INT32_MIN && b == -1) ? INT32_MIN : a / b;
        return __int_as_float(r);
    }
    case OP_IRem: {
        int a = __float_as_int(t), b = __float_as_int(s);
        int r = b == 0 ? a : (a == INT32_MIN && b == -1) ? 0 : a % b;
        return __int_as_float(r);
    }
    }
    return t;
}

/* ------------------------------------------------------------------------------------------------ */
/* scalar per-element semantics                                                                      */

template <int OP> __device__ __forceinline__ float scalar_binary(float t, float s, uint32_t operand)
{
    if constexpr (OP == OP_FDiv) return __fdiv_rn(t, s);
    else if constexpr (OP == OP_FRDiv) return __fdiv_rn(s, t);
    else if constexpr (OP == OP_FGt) return t > s ? 1.0f : 0.0f;
    else if constexpr (OP == OP_FLt) return t < s ? 1.0f : 0.0f;
    else if constexpr (OP == OP_FGe) return t >= s ? 1.0f : 0.0f;
    else if constexpr (OP == OP_FLe) return t <= s ? 1.0f : 0.0f;
    else if constexpr (OP == OP_FEq) return t == s ? 1.0f : 0.0f;
    else if constexpr (OP == OP_FNe) return t != s ? 1.0f : 0.0f;  // unordered: true on NaN
    else if constexpr (OP == OP_FApprox) return fabsf(__fsub_rn(t, s)) < __uint_as_float(operand) ? 1.0f : 0.0f;
    else if constexpr (OP == OP_IAdd) return __int_as_float(__float_as_int(t) + __float_as_int(s));
    else if constexpr (OP == OP_IMul) return __int_as_float(__float_as_int(t) * __float_as_int(s));
    else if constexpr (OP == OP_ISub) return __int_as_float(__float_as_int(t) - __float_as_int(s));
    else if constexpr (OP == OP_IShl) {
        uint32_t n = __float_as_uint(s);
        return __uint_as_float(n >= 32 ? 0u : __float_as_uint(t) << n);
    } else if constexpr (OP == OP_IShr) {
        uint32_t n = __float_as_uint(s);
        return __uint_as_float(n >= 32 ? 0u : __float_as_uint(t) >> n);
    } else if constexpr (OP == OP_IAnd) return __uint_as_float(__float_as_uint(t) & __float_as_uint(s));
    else if constexpr (OP == OP_IOr) return __uint_as_float(__float_as_uint(t) | __float_as_uint(s));
    else if constexpr (OP == OP_IXor) return __uint_as_float(__float_as_uint(t) ^ __float_as_uint(s));
    else return slow_math(OP, t, s);  // FRem, FArcTan2, FPow, IDiv, IRem
}

template <int OP> __device__ __forceinline__ float scalar_unary(float t)
{
    if constexpr (OP == OP_FSqrt) return __fsqrt_rn(t);
    else if constexpr (OP == OP_FSin) return __sinf(t);   // the reference maps FSin/FCos/FTan to the fast variants
    else if constexpr (OP == OP_FCos) return __cosf(t);   // (nvptx.py:108-110)
    else if constexpr (OP == OP_FExp) return expf(t);
    else if constexpr (OP == OP_FExp2) return exp2f(t);
    else if constexpr (OP == OP_FRSqrt) return rsqrtf(t);
    else if constexpr (OP == OP_FRcp) return __frcp_rn(t);
    else return slow_math(OP, t, 0.0f);  // FTan, FArcSin, FArcCos, FArcTan, FLog, FLog2, FErf
}

/* ------------------------------------------------------------------------------------------------ */
/* memory                                                                                            */

enum { DT_F32 = 0, DT_F16 = 1, DT_BF16 = 2, DT_U8 = 3 };
enum { LAY_1D = 0, LAY_2DT = 1, LAY_2DW = 2 };

template <int DT> struct ElemSize { static constexpr int value = DT == DT_F32 ? 4 : DT == DT_U8 ? 1 : 2; };

template <int DT> __device__ __forceinline__ float load_elem(const char *p)
{
    if constexpr (DT == DT_F32) return *reinterpret_cast<const float *>(p);
    else if constexpr (DT == DT_F16) return __half2float(*reinterpret_cast<const __half *>(p));
    else if constexpr (DT == DT_BF16) return __bfloat162float(*reinterpret_cast<const __nv_bfloat16 *>(p));
    else return (float)*reinterpret_cast<const unsigned char *>(p);
}
template <int DT> __device__ __forceinline__ void store_elem(char *p, float v)
{
    if constexpr (DT == DT_F32) *reinterpret_cast<float *>(p) = v;
    else if constexpr (DT == DT_F16) *reinterpret_cast<__half *>(p) = __float2half_rn(v);
    else if constexpr (DT == DT_BF16) *reinterpret_cast<__nv_bfloat16 *>(p) = __float2bfloat16_rn(v);
}

/*
 * One 32 x 4 tile access for one logical program.
 *   1D  (load_store.py:76-101):   element e = off + lane + 32*w on dim 1, active iff e < shape1
 *   2DT (load_store.py:104-150):  t = lane + off on dim 1, j = adv + w on dim 2
 *   2DW (load_store.py:153-158):  t = lane + adv on dim 1, j = off + w on dim 2
 * Inactive loads give 0.0 (load_store.py:12). off = operand >> 4 (logical), slot = operand & 15.
 * Index arithmetic is 32-bit, the byte offset is sign-extended to 64 bits, as in the reference's GEPs.
 */
template <int LAYOUT, int DT, bool STORE>
__device__ __forceinline__ void tile_rw(const TileInfo *ti, uint32_t operand, int lane, float (&v)[4])
{
    constexpr int ESZ = ElemSize<DT>::value;
    const int arg = operand & 15;
    const int off = (int)(operand >> 4);
    char *base = reinterpret_cast<char *>(ti->ptr[arg]);
    const int2 s1 = ti->s1[arg];

    if constexpr (LAYOUT == LAY_1D) {
        const int e = lane + off;
        if constexpr (DT == DT_F32) {
            if (s1.y == 1) {  // unit stride: four fully coalesced 128-byte warp accesses
                float *p = reinterpret_cast<float *>(base) + e;
                if (off + 128 <= s1.x) {
#pragma unroll
                    for (int w = 0; w < 4; w++) {
                        if (GINT_CHK(arg, p + 32 * w, 4, STORE)) {
                            if constexpr (STORE) p[32 * w] = v[w];
                            else v[w] = p[32 * w];
                        } else if constexpr (!STORE) v[w] = 0.0f;
                    }
                } else {
#pragma unroll
                    for (int w = 0; w < 4; w++) {
                        const bool ok = e + 32 * w < s1.x && GINT_CHK(arg, p + 32 * w, 4, STORE);
                        if constexpr (STORE) { if (ok) p[32 * w] = v[w]; }
                        else v[w] = ok ? p[32 * w] : 0.0f;
                    }
                }
                return;
            }
        }
        char *p = base + (long long)(e * s1.y) * ESZ;
        const long long pstep = (long long)(s1.y * 32) * ESZ;
#pragma unroll
        for (int w = 0; w < 4; w++) {
            const bool ok = e + 32 * w < s1.x && GINT_CHK(arg, p, ESZ, STORE);
            if constexpr (STORE) { if (ok) store_elem<DT>(p, v[w]); }
            else v[w] = ok ? load_elem<DT>(p) : 0.0f;
            p += pstep;
        }
    } else {
        const int2 s2 = ti->s2[arg];
        const int adv = ti->adv[arg];
        const int t = LAYOUT == LAY_2DT ? lane + off : lane + adv;
        const int j0 = LAYOUT == LAY_2DT ? adv : off;
        const bool tok = t < s1.x;
        if constexpr (DT == DT_F32 && LAYOUT == LAY_2DW) {
            // one 128-bit access per thread: rows of 4 consecutive floats, 16-byte aligned
            if ((ti->flags[arg] & kVecRows) && (j0 & 3) == 0 && j0 + 4 <= s2.x) {
                float4 *p = reinterpret_cast<float4 *>(base + (long long)(t * s1.y + j0) * 4);
                const bool vok = tok && GINT_CHK(arg, p, 16, STORE);
                if constexpr (STORE) {
                    if (vok) *p = make_float4(v[0], v[1], v[2], v[3]);
                } else {
                    float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (vok) r = *p;
                    v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
                }
                return;
            }
        }
        char *p = base + (long long)(t * s1.y + j0 * s2.y) * ESZ;
        const long long pstep = (long long)s2.y * ESZ;
#pragma unroll
        for (int w = 0; w < 4; w++) {
            const bool ok = tok && (j0 + w < s2.x) && GINT_CHK(arg, p, ESZ, STORE);
            if constexpr (STORE) { if (ok) store_elem<DT>(p, v[w]); }
            else v[w] = ok ? load_elem<DT>(p) : 0.0f;
            p += pstep;
        }
    }
}

/* gather / scatter of f32 elements by i32 indices taken from the stack (load_store.py:266-288):
 * active iff idx < shape1 (signed; negative indices are not rejected, as in the reference). */
template <bool STORE>
__device__ __forceinline__ void tile_indirect(const TileInfo *ti, uint32_t operand, const float (&idx)[4], float (&v)[4])
{
    const int arg = operand & 15;
    char *base = reinterpret_cast<char *>(ti->ptr[arg]);
    const int2 s1 = ti->s1[arg];
#pragma unroll
    for (int w = 0; w < 4; w++) {
        const int i = __float_as_int(idx[w]);
        float *p = reinterpret_cast<float *>(base + (long long)(i * s1.y) * 4);
        const bool ok = i < s1.x && GINT_CHK(arg, p, 4, STORE);
        if constexpr (STORE) { if (ok) *p = v[w]; }
        else v[w] = ok ? *p : 0.0f;
    }
}

/* ------------------------------------------------------------------------------------------------ */
/* descriptor decode (load_tensor_infos.py:14-54): lane (8k + t) decodes tensor t of tile k           */

template <int K>
__device__ __forceinline__ void decode_tiles(const gint_tensor_info *__restrict__ ti, int n_tensors, uint32_t first_idx,
                                             uint32_t end_idx, TileInfo *tiles, int lane, uint32_t gather_mask = 0u,
                                             const long long *__restrict__ gather_index = nullptr, uint32_t gather_rows = 0u)
{
    const int k = lane >> 3, t = lane & 7;
    if (k < K) {
        /* A group at the end of the range may have fewer than K logical programs: the spare tiles repeat the last one
         * (same loads, same values, same stores from the same threads), so that no handler needs to know about them. */
        const uint32_t bidx = min(first_idx + (uint32_t)k, end_idx - 1u);
        u64 ptr = 0;
        int2 s1 = make_int2(INT32_MIN, 0);  // x < INT32_MIN never holds: every access of this slot is masked
        int2 s2 = make_int2(INT32_MIN, 0);
        int flags = 0;
        if (t < n_tensors && bidx < end_idx) {
            const int2 bs1 = *reinterpret_cast<const int2 *>(ti->block_shape_stride_1[t]);
            const int2 bs2 = *reinterpret_cast<const int2 *>(ti->block_shape_stride_2[t]);
            const int2 gd = *reinterpret_cast<const int2 *>(ti->block_grid_dims[t]);
            const int2 gs = *reinterpret_cast<const int2 *>(ti->block_grid_steps[t]);
            uint32_t r = bidx;
            uint32_t b1 = 0, b2 = 0;
            if ((uint32_t)gd.x != 1u) { b1 = r % (uint32_t)gd.x; r = r / (uint32_t)gd.x; }
            if ((uint32_t)gd.y != 1u && r != 0u) { b2 = r % (uint32_t)gd.y; r = r / (uint32_t)gd.y; }
            uint32_t off = b1 * (uint32_t)gs.x * (uint32_t)bs1.y + b2 * (uint32_t)gs.y * (uint32_t)bs2.y;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint32_t sz = (uint32_t)ti->batch_shape[t][j];
                if (j == 0 && ((gather_mask >> t) & 1u)) {
                    /* gathered rows: the innermost batch index selects an entry of the row index, which takes its place
                     * (tensor[index[b]] without the copy; 64-bit index values, 32-bit offset arithmetic like every other term) */
                    const uint32_t q = sz != 1u ? r / sz : r;
                    const uint32_t b = sz != 1u ? r - q * sz : 0u;
                    /* torch's indexing rule for a negative index (counts from the end); an index that is still out of range --
                     * an error in torch -- is clamped to the nearest row so that no access leaves the table */
                    long long row = gather_index[b];
                    if (row < 0) row += (long long)gather_rows;
                    row = row < 0 ? 0 : row >= (long long)gather_rows ? (long long)gather_rows - 1 : row;
                    off += (uint32_t)ti->batch_strides[t][0] * (uint32_t)row;
                    r = q;
                    continue;
                }
                if (sz != 1u && r != 0u) {
                    const uint32_t q = r / sz;
                    off += (uint32_t)ti->batch_strides[t][j] * (r - q * sz);
                    r = q;
                }
            }
            ptr = (u64)ti->base_ptr[t] + (u64)off * (u64)(uint32_t)ti->elm_size[t];
            s1 = make_int2((int)((uint32_t)bs1.x - b1 * (uint32_t)gs.x), bs1.y);
            s2 = make_int2((int)((uint32_t)bs2.x - b2 * (uint32_t)gs.y), bs2.y);
            if (bs2.y == 1 && (bs1.y & 3) == 0 && (ptr & 15) == 0) flags |= kVecRows;
        }
        TileInfo *o = tiles + k;
        o->ptr[t] = ptr;
        o->s1[t] = s1;
        o->s2[t] = s2;
        o->adv[t] = 0;
        o->flags[t] = flags;
    }
    __syncwarp();
}

/* ------------------------------------------------------------------------------------------------ */
/* the register pool                                                                                  */
/*
 * The operand stack and the virtual registers are 2*P*K 64-bit PTX registers %gs0 .. %gs(2PK-1), declared once at the
 * top of the kernel and touched only from inline asm, by name. Slot s of tile k is the pair
 * (%gs[(s*K+k)*2], %gs[(s*K+k)*2+1]) = width lanes (0,1) and (2,3). Keeping them out of the C++ value world matters:
 * as C++ variables they are loop-carried through a ~950-way switch, and the compiler's phi copies for every slot on
 * every path (which ptxas does not coalesce across the jump table) cost more than the handlers themselves.
 */

template <int P, int K> __device__ __forceinline__ void pool_declare()
{
    asm volatile(".reg .b64 %%gs<%0>;" ::"n"(2 * P * K));
}

/* A packed pair assembled from two lanes of a slot chosen by immediate operands (Bcast_k, gint_opcodes.h): the four lanes of the
 * source slot are named a0..a3 inside a PTX scope -- register moves only, no selects. */
template <int DST, int SRC_LO, int SRC_HI, int I, int J> __device__ __forceinline__ void r_pick()
{
    asm volatile("{\n\t.reg .b32 a<4>;\n\tmov.b64 {a0, a1}, %%gs%1;\n\tmov.b64 {a2, a3}, %%gs%2;\n\tmov.b64 %%gs%0, {a%3, a%4};\n\t}"
                 ::"n"(DST), "n"(SRC_LO), "n"(SRC_HI), "n"(I), "n"(J));
}

template <int I> __device__ __forceinline__ void r_get(float &x, float &y)
{
    asm volatile("mov.b64 {%0, %1}, %%gs%2;" : "=f"(x), "=f"(y) : "n"(I));
}
template <int I> __device__ __forceinline__ void r_set(float x, float y)
{
    asm volatile("mov.b64 %%gs%2, {%0, %1};" ::"f"(x), "f"(y), "n"(I));
}
template <int I> __device__ __forceinline__ void r_set64(u64 v)
{
    asm volatile("mov.b64 %%gs%1, %0;" ::"l"(v), "n"(I));
}
template <int D, int A> __device__ __forceinline__ void r_mov()
{
    if constexpr (D != A) asm volatile("mov.b64 %%gs%0, %%gs%1;" ::"n"(D), "n"(A));
}
template <int A, int B> __device__ __forceinline__ void r_swap()
{
    asm volatile("{ .reg .b64 t; mov.b64 t, %%gs%0; mov.b64 %%gs%0, %%gs%1; mov.b64 %%gs%1, t; }" ::"n"(A), "n"(B));
}
template <int D, int A, int B> __device__ __forceinline__ void r_add2()
{
    asm volatile("add.rn.f32x2 %%gs%0, %%gs%1, %%gs%2;" ::"n"(D), "n"(A), "n"(B));
}
template <int D, int A, int B> __device__ __forceinline__ void r_sub2()
{
    asm volatile("sub.rn.f32x2 %%gs%0, %%gs%1, %%gs%2;" ::"n"(D), "n"(A), "n"(B));
}
template <int D, int A, int B> __device__ __forceinline__ void r_mul2()
{
    asm volatile("mul.rn.f32x2 %%gs%0, %%gs%1, %%gs%2;" ::"n"(D), "n"(A), "n"(B));
}
template <int D, int A, int B, int C> __device__ __forceinline__ void r_fma2()
{
    asm volatile("fma.rn.f32x2 %%gs%0, %%gs%1, %%gs%2, %%gs%3;" ::"n"(D), "n"(A), "n"(B), "n"(C));
}
template <int D> __device__ __forceinline__ void r_add2_imm(u64 imm)
{
    asm volatile("add.rn.f32x2 %%gs%0, %%gs%0, %1;" ::"n"(D), "l"(imm));
}
template <int D> __device__ __forceinline__ void r_mul2_imm(u64 imm)
{
    asm volatile("mul.rn.f32x2 %%gs%0, %%gs%0, %1;" ::"n"(D), "l"(imm));
}
template <int D> __device__ __forceinline__ void r_fma2_imm(u64 m, u64 c)
{
    asm volatile("fma.rn.f32x2 %%gs%0, %%gs%0, %1, %2;" ::"n"(D), "l"(m), "l"(c));
}
template <int D> __device__ __forceinline__ void r_neg2()
{
    asm volatile("xor.b64 %%gs%0, %%gs%0, 0x8000000080000000;" ::"n"(D));
}

/* index of the low (h = 0) / high (h = 1) pair of slot `slot`, tile `k` */
template <int K> __host__ __device__ constexpr int gs(int slot, int k, int h) { return (slot * K + k) * 2 + h; }

template <int K, int SLOT, int KI> __device__ __forceinline__ void slot_read(float (&v)[4])
{
    r_get<gs<K>(SLOT, KI, 0)>(v[0], v[1]);
    r_get<gs<K>(SLOT, KI, 1)>(v[2], v[3]);
}
template <int K, int SLOT, int KI> __device__ __forceinline__ void slot_write(const float (&v)[4])
{
    r_set<gs<K>(SLOT, KI, 0)>(v[0], v[1]);
    r_set<gs<K>(SLOT, KI, 1)>(v[2], v[3]);
}
template <int K, int D, int A, int KI> __device__ __forceinline__ void slot_mov()
{
    r_mov<gs<K>(D, KI, 0), gs<K>(A, KI, 0)>();
    r_mov<gs<K>(D, KI, 1), gs<K>(A, KI, 1)>();
}
template <int K, int A, int B, int KI> __device__ __forceinline__ void slot_swap()
{
    r_swap<gs<K>(A, KI, 0), gs<K>(B, KI, 0)>();
    r_swap<gs<K>(A, KI, 1), gs<K>(B, KI, 1)>();
}

/* ------------------------------------------------------------------------------------------------ */
/* one instruction at one stack depth, for one of the warp's K tiles                                 */

struct Ctx {
    TileInfo *tiles;   // this warp's K tile descriptors (shared memory)
    int lane;
    uint32_t hidden;   // shared-memory address of slot 0, tile 0 of the warp's load staging area, plus 4 * lane
    uint32_t ring_mask; // bytes of the warp's ring of early-issued loads (4 or 8 slots of K x 512 bytes) minus 1
    uint32_t rows;     // shared-memory address of this warp's staged row blocks (tile 0); tile k is rows_stride bytes further
    uint32_t rows_stride;
    const LaunchArgs *args;   // the launch parameters (direct mode), for the kernels that derive the four values above on demand
};

/* The widest kernels (12 slots x 2 tiles = 96 pool registers) have about a dozen registers left for everything else, and the
 * handlers with the most temporaries (runtime lane selects) spilled. They do not keep hidden / ring_mask / rows / rows_stride
 * in registers between handlers: the few handlers that need them recompute them from the launch parameters (constant bank)
 * and the warp index. */
template <int P, int K> __host__ __device__ constexpr bool lean_ctx() { return P * K >= 24; }

/* shared-memory address of the first byte after the block's tile descriptors (see geval_direct_body for the layout) */
template <int K> __device__ __forceinline__ uint32_t cx_after_tiles(const Ctx &cx, uint32_t warp)
{
    return (uint32_t)__cvta_generic_to_shared(cx.tiles) + ((uint32_t)kWarpsPerBlock - warp) * (uint32_t)(K * sizeof(TileInfo));
}
template <int P, int K> __device__ __forceinline__ uint32_t cx_ring_mask(const Ctx &cx)
{
    if constexpr (lean_ctx<P, K>()) return (uint32_t)K * cx.args->ring_bytes - 1u;
    else return cx.ring_mask;
}
template <int P, int K> __device__ __forceinline__ uint32_t cx_rows_stride(const Ctx &cx)
{
    if constexpr (lean_ctx<P, K>()) return cx.args->row_area_bytes;
    else return cx.rows_stride;
}
template <int P, int K> __device__ __forceinline__ uint32_t cx_hidden(const Ctx &cx)
{
    if constexpr (lean_ctx<P, K>()) {
        const uint32_t warp = threadIdx.x >> 5;
        return cx_after_tiles<K>(cx, warp) + warp * (uint32_t)K * cx.args->ring_bytes + (uint32_t)cx.lane * 4u;
    } else return cx.hidden;
}
template <int P, int K> __device__ __forceinline__ uint32_t cx_rows(const Ctx &cx)
{
    if constexpr (lean_ctx<P, K>()) {
        const uint32_t warp = threadIdx.x >> 5;
        return cx_after_tiles<K>(cx, warp) + (uint32_t)(kWarpsPerBlock * K) * cx.args->ring_bytes + warp * (uint32_t)K * cx.args->row_area_bytes;
    } else return cx.rows;
}

template <int OP> struct OpInfo;
#define GINT_X_INFO(name, num, md, net) \
    template <> struct OpInfo<num> { static constexpr int min_depth = md; static constexpr int net_effect = net; };
GINT_OPCODE_LIST(GINT_X_INFO)
GINT_INTERNAL_OPCODE_LIST(GINT_X_INFO)
GINT_RF_OPCODE_LIST(GINT_X_INFO)
GINT_VEC_OPCODE_LIST(GINT_X_INFO)
#undef GINT_X_INFO

template <int OP, int SP, int P, int K_ = 1> __host__ __device__ constexpr bool op_valid();

/* Fused handlers (gint_fused.h): a sequence's stack effect and validity follow from its members. */
template <int... OPS> struct Seq {
    static constexpr int n = sizeof...(OPS);
    /* stream entries the sequence occupies: one, plus one for every member after the first that reads an operand word */
    static __host__ __device__ constexpr int entries()
    {
        constexpr int ops[] = {OPS..., 0};
        int m = 1;
        for (int j = 1; j < n; j++) m += GINT_OP_USES_OPERAND(ops[j]) ? 1 : 0;
        return m;
    }
    /* 1-based index, among those extra entries, of the entry that carries member j's operand (j >= 1, operand-reading) */
    static __host__ __device__ constexpr int entry_of(int j)
    {
        constexpr int ops[] = {OPS..., 0};
        int e = 0;
        for (int i = 1; i <= j; i++) e += GINT_OP_USES_OPERAND(ops[i]) ? 1 : 0;
        return e;
    }
};
template <int NUM> struct FusedSeq;
#define GINT_X_FSEQ(num, len, ...) template <> struct FusedSeq<num> { using type = Seq<__VA_ARGS__>; static_assert(Seq<__VA_ARGS__>::n == len, "length"); };
GINT_FUSED_LIST(GINT_X_FSEQ)
GINT_RF_FUSED_LIST(GINT_X_FSEQ)
#undef GINT_X_FSEQ
static_assert(GINT_FUSED_FIRST + GINT_N_FUSED == GINT_N_DISPATCH_PLAIN && GINT_RF_FUSED_FIRST + GINT_N_RF_FUSED == GINT_N_DISPATCH_RF,
              "gint_fused.h and gint_opcodes.h disagree");

template <typename S> struct SeqInfo;
template <> struct SeqInfo<Seq<>> {
    static constexpr int net = 0, min_depth = 0;
    template <int SP, int P, int K_> static constexpr bool valid() { return true; }
};
template <int OP0, int... REST> struct SeqInfo<Seq<OP0, REST...>> {
    using Tail = SeqInfo<Seq<REST...>>;
    static constexpr int net = OpInfo<OP0>::net_effect + Tail::net;
    static constexpr int tail_need = Tail::min_depth - OpInfo<OP0>::net_effect;
    static constexpr int min_depth = OpInfo<OP0>::min_depth > tail_need ? OpInfo<OP0>::min_depth : tail_need;
    template <int SP, int P, int K_> static constexpr bool valid()
    {
        if constexpr (!op_valid<OP0, SP, P, K_>()) return false;
        else return Tail::template valid<SP + OpInfo<OP0>::net_effect, P, K_>();
    }
};
#define GINT_X_FINFO(num, len, ...)                                                                        \
    template <> struct OpInfo<num> {                                                                       \
        static constexpr int min_depth = SeqInfo<Seq<__VA_ARGS__>>::min_depth;                             \
        static constexpr int net_effect = SeqInfo<Seq<__VA_ARGS__>>::net;                                  \
    };
GINT_FUSED_LIST(GINT_X_FINFO)
GINT_RF_FUSED_LIST(GINT_X_FINFO)
#undef GINT_X_FINFO

template <int OP, int SP, int P, int K_> __host__ __device__ constexpr bool op_valid()
{
    if constexpr (GINT_IS_FUSED(OP)) {
#ifndef GINT_RF
        if (OP >= GINT_RF_FUSED_FIRST) return false;
#endif
        return SP >= 0 && SeqInfo<typename FusedSeq<OP>::type>::template valid<SP, P, K_>();
    } else {
        constexpr int limit = P < GINT_MAX_STACK ? P : GINT_MAX_STACK;
        if (SP > limit || SP < OpInfo<OP>::min_depth) return false;
        if (SP + OpInfo<OP>::net_effect > limit) return false;
        if (OP == OP_DupX2 && SP + 1 > limit) return false;
        /* The 12-slot two-tile kernel has no Bcast_k handlers (the host keeps DupBroadcastW in programs that need 12 slots):
         * with them it no longer fits its 128 registers and the assembler moves pool registers to local memory, which every
         * program pays for. The one-tile 12-slot kernels (direct, indirect, checked) keep them: they also run the streams of
         * programs with smaller pools, in which DupBroadcastW has become Bcast_k. */
        if (OP >= OP_Bcast_0 && OP <= OP_Bcast_3 && P * K_ >= 24) return false;
#ifndef GINT_VEC
        if (OP == OP_RemapVN) return false;
#endif
#ifdef GINT_RF
        /* virtual registers in shared memory: the pool is the operand stack alone, registers are reached through RLoad / RStore */
        if (OP >= OP_FLoadReg0 && OP <= OP_FStoreReg7) return false;
#else
        if (OP >= OP_RLoad && OP <= OP_RLoadS) return false;
        if (OP >= OP_FLoadReg0 && OP <= OP_FLoadReg7 && (P - 1 - (OP - OP_FLoadReg0)) < 0) return false;
        if (OP >= OP_FStoreReg0 && OP <= OP_FStoreReg7 && (P - 1 - (OP - OP_FStoreReg0)) < 0) return false;
#endif
        return true;
    }
}

/* 4-way select by a 2-bit index; indices are clamped to 0..3 by the host pre-decoder, which makes this equal to
 * the reference's compare tree (move.py:58-66) */
__device__ __forceinline__ float sel4(const float (&v)[4], uint32_t i)
{
    const float lo = (i & 1u) ? v[1] : v[0];
    const float hi = (i & 1u) ? v[3] : v[2];
    return (i & 2u) ? hi : lo;
}

template <int OP> __host__ __device__ constexpr bool is_scalar_binary()
{
    return OP == OP_FDiv || OP == OP_FRDiv || OP == OP_FRem || (OP >= OP_FGt && OP <= OP_FApprox) || OP == OP_FArcTan2 ||
           OP == OP_FPow || (OP >= OP_IAdd && OP <= OP_IXor);
}
template <int OP> __host__ __device__ constexpr bool is_scalar_unary()
{
    return OP == OP_FSqrt || OP == OP_FSin || OP == OP_FCos || OP == OP_FTan || OP == OP_FArcSin || OP == OP_FArcCos ||
           OP == OP_FArcTan || OP == OP_FExp || OP == OP_FExp2 || OP == OP_FLog || OP == OP_FLog2 || OP == OP_FRSqrt ||
           OP == OP_FErf || OP == OP_FRcp;
}
template <int OP> struct MemOp { static constexpr bool is = false; };
#define GINT_MEMOP(name, lay, dt, st) \
    template <> struct MemOp<OP_##name> { static constexpr bool is = true; static constexpr int layout = lay; static constexpr int dtype = dt; static constexpr bool store = st; };
GINT_MEMOP(LoadGlobal1DF32, LAY_1D, DT_F32, false) GINT_MEMOP(StoreGlobal1DF32, LAY_1D, DT_F32, true)
GINT_MEMOP(LoadGlobal1DF16, LAY_1D, DT_F16, false) GINT_MEMOP(StoreGlobal1DF16, LAY_1D, DT_F16, true)
GINT_MEMOP(LoadGlobal1DBF16, LAY_1D, DT_BF16, false) GINT_MEMOP(StoreGlobal1DBF16, LAY_1D, DT_BF16, true)
GINT_MEMOP(LoadGlobal1DU8, LAY_1D, DT_U8, false)
GINT_MEMOP(LoadGlobal2DTF32, LAY_2DT, DT_F32, false) GINT_MEMOP(StoreGlobal2DTF32, LAY_2DT, DT_F32, true)
GINT_MEMOP(LoadGlobal2DTF16, LAY_2DT, DT_F16, false) GINT_MEMOP(StoreGlobal2DTF16, LAY_2DT, DT_F16, true)
GINT_MEMOP(LoadGlobal2DTBF16, LAY_2DT, DT_BF16, false) GINT_MEMOP(StoreGlobal2DTBF16, LAY_2DT, DT_BF16, true)
GINT_MEMOP(LoadGlobal2DTU8, LAY_2DT, DT_U8, false)
GINT_MEMOP(LoadGlobal2DWF32, LAY_2DW, DT_F32, false) GINT_MEMOP(StoreGlobal2DWF32, LAY_2DW, DT_F32, true)
GINT_MEMOP(LoadGlobal2DWF16, LAY_2DW, DT_F16, false) GINT_MEMOP(StoreGlobal2DWF16, LAY_2DW, DT_F16, true)
GINT_MEMOP(LoadGlobal2DWBF16, LAY_2DW, DT_BF16, false) GINT_MEMOP(StoreGlobal2DWBF16, LAY_2DW, DT_BF16, true)
GINT_MEMOP(LoadGlobal2DWU8, LAY_2DW, DT_U8, false)
#undef GINT_MEMOP

/*
 * Start a 1-D tile load whose values are not needed yet. The warp copies the tile with cp.async into a slot of its ring of
 * staging slots in shared memory and commits the copies as one group; nothing here waits for memory. A slot holds the tile
 * in ELEMENT order (element e of the tile at byte 4e of the slot's 512 bytes; K tiles back to back; the current slot is
 * tracked in the named register %gring):
 *   - a full unit-stride tile whose first byte is 16-byte aligned is ONE 16-byte copy per lane (lane l moves elements
 *     4l..4l+3), i.e. one instruction and four conflict-free shared-memory wavefronts per 512 bytes;
 *   - anything else is four 4-byte copies per lane (lane l moves elements l, l+32, l+64, l+96: consecutive lanes write
 *     consecutive words), masked elements being zero-filled by the copy itself (source size 0).
 * PfTake later waits for exactly this group (cp.async groups complete in order, and at that point D-1 newer groups are in
 * flight), synchronises the warp -- a lane consumes words that other lanes copied -- and reads its four values, elements
 * l + 32w, with four conflict-free 4-byte loads. Same addressing and masking rules as tile_rw.
 * `slot` is the shared-memory address of the slot's tile 0 plus 4 * lane.
 */
__device__ __forceinline__ void cp_async_f32(uint32_t dst, const void *src, bool ok)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(ok ? 4 : 0) : "memory");
}
template <int K, int KI>
__device__ __forceinline__ void tile_issue(const TileInfo *ti, uint32_t operand, const Ctx &cx, uint32_t slot)
{
    const int arg = operand & 15;
    const int off = (int)(operand >> 4);
    const int lane = cx.lane;
    char *base = reinterpret_cast<char *>(ti->ptr[arg]);
    const int2 s1 = ti->s1[arg];
#ifdef GINT_VEC
    const uint32_t dst = slot - (uint32_t)(lane * 12) + (uint32_t)(KI * 512);   // (`slot` carries 16 * lane here)
#else
    const uint32_t dst = slot + (uint32_t)(KI * 512);
#endif
    const int e = lane + off;
    if (s1.y == 1 && off + 128 <= s1.x) {  // full unit-stride tile
        const char *p0 = base + (long long)off * 4;
        if ((reinterpret_cast<u64>(p0) & 15) == 0) {
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + (uint32_t)(lane * 12)), "l"(p0 + lane * 16) : "memory");
        } else {
            const char *p = p0 + lane * 4;
            asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n\t"
                         "cp.async.ca.shared.global [%0+128], [%1+128], 4;\n\t"
                         "cp.async.ca.shared.global [%0+256], [%1+256], 4;\n\t"
                         "cp.async.ca.shared.global [%0+384], [%1+384], 4;" ::"r"(dst), "l"(p) : "memory");
        }
        return;
    }
    const char *p = base + (long long)(e * s1.y) * 4;
    const long long pstep = (long long)(s1.y * 32) * 4;
#pragma unroll
    for (int w = 0; w < 4; w++) {
        const bool ok = e + 32 * w < s1.x;
        cp_async_f32(dst + 128 * w, ok ? p + w * pstep : base, ok);
    }
}
/* Operand of the fast accesses, as the host pre-decoder writes it (gint_capi.cu: apply_fast_accesses): byte offset of the
 * tile from the tensor's tile pointer in bits 0..25, 8 * tensor slot in bits 26..31 -- the byte offset of the slot's
 * pointer in TileInfo::ptr. */
__device__ __forceinline__ char *fast_tile_address(const TileInfo *ti, uint32_t operand)
{
    const u64 base = *reinterpret_cast<const u64 *>(reinterpret_cast<const char *>(ti->ptr) + (operand >> 26));
    return reinterpret_cast<char *>(base) + (operand & 0x03FFFFFFu);
}
/* The same for a tile that the host proved full, unit-stride and 16-byte aligned: no shape, stride or mask handling. */
template <int K, int KI>
__device__ __forceinline__ void tile_issue_fast(const TileInfo *ti, uint32_t operand, const Ctx &cx, uint32_t slot)
{
    const char *p = fast_tile_address(ti, operand) + cx.lane * 16;
#ifdef GINT_VEC
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(slot + (uint32_t)(KI * 512)), "l"(p) : "memory");
#else
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(slot + (uint32_t)(KI * 512 + cx.lane * 12)), "l"(p) : "memory");
#endif
}
template <int K, int SLOT, int KI> __device__ __forceinline__ void take_hidden(uint32_t slot)
{
    const uint32_t src = slot + (uint32_t)(KI * 512);
#ifdef GINT_VEC
    asm volatile("ld.shared.v2.b64 {%%gs%0, %%gs%1}, [%2];" ::"n"(gs<K>(SLOT, KI, 0)), "n"(gs<K>(SLOT, KI, 1)), "r"(src) : "memory");
    return;
#endif
    asm volatile("{\n\t.reg .b32 t<4>;\n\t"
                 "ld.shared.b32 t0, [%2];\n\tld.shared.b32 t1, [%2+128];\n\tld.shared.b32 t2, [%2+256];\n\tld.shared.b32 t3, [%2+384];\n\t"
                 "mov.b64 %%gs%0, {t0, t1};\n\tmov.b64 %%gs%1, {t2, t3};\n\t}" ::"n"(gs<K>(SLOT, KI, 0)), "n"(gs<K>(SLOT, KI, 1)), "r"(src) : "memory");
}

/* four values of a tile in element order at `at` (+ 128 w): the natural layout's read */
template <int K, int SLOT, int KI> __device__ __forceinline__ void take_natural(uint32_t at)
{
    asm volatile("{\n\t.reg .b32 t<4>;\n\t"
                 "ld.shared.b32 t0, [%2];\n\tld.shared.b32 t1, [%2+128];\n\tld.shared.b32 t2, [%2+256];\n\tld.shared.b32 t3, [%2+384];\n\t"
                 "mov.b64 %%gs%0, {t0, t1};\n\tmov.b64 %%gs%1, {t2, t3};\n\t}" ::"n"(gs<K>(SLOT, KI, 0)), "n"(gs<K>(SLOT, KI, 1)), "r"(at) : "memory");
}

template <int K, int SLOT, int KI> __device__ __forceinline__ void put_vector(uint32_t at)
{
    asm volatile("st.shared.v2.b64 [%2], {%%gs%0, %%gs%1};" ::"n"(gs<K>(SLOT, KI, 0)), "n"(gs<K>(SLOT, KI, 1)), "r"(at) : "memory");
}

/* Staged row blocks (StageRows / LoadStagedRows). Row m of the block (lane m's row) has q = 2^lq chunks of 16 bytes; chunk r
 * of row m is kept at chunk position m*q + (r ^ ((m >> (3 - lq)) & (q - 1))) of the copy, so that the eight lanes a 16-byte
 * shared-memory access serves per wavefront hit eight different 16-byte bank groups, whichever chunk they ask for. */
__device__ __forceinline__ uint32_t staged_row_position(uint32_t m, uint32_t r, uint32_t lq)
{
    return (m << lq) + (r ^ ((m >> (3u - lq)) & ((1u << lq) - 1u)));
}
template <int K, int SLOT, int KI> __device__ __forceinline__ void take_rows(uint32_t at)
{
    asm volatile("ld.shared.v2.b64 {%%gs%0, %%gs%1}, [%2];" ::"n"(gs<K>(SLOT, KI, 0)), "n"(gs<K>(SLOT, KI, 1)), "r"(at) : "memory");
}

/* %grf as a value (kernels built with GINT_RF). Not volatile: the register is written once, before the first handler runs, so
 * the compiler may merge the reads of the K tiles and of the members of a fused sequence. */
__device__ __forceinline__ uint32_t rf_base()
{
    uint32_t v = 0;
#ifdef GINT_RF
    asm("mov.b32 %0, %%grf;" : "=r"(v));
#endif
    return v;
}

template <int OP, int SP, int P, int K, int KI>
__device__ __forceinline__ void exec_tile(const uint32_t operand, const Ctx &cx)
{
    constexpr int T = SP - 1;  // top of stack; T-1 = second ("S"), T-2 = third ("U")
#define LO(slot) gs<K>((slot), KI, 0)
#define HI(slot) gs<K>((slot), KI, 1)
    /* ---- float ALU (arith.py:15-66): binary handlers compute fn(T, S) ---- */
    if constexpr (OP == OP_Nop || OP == OP_Pop || OP == OP_Pop2) {
    } else if constexpr (OP == OP_FAdd) {
        r_add2<LO(T - 1), LO(T), LO(T - 1)>();
        r_add2<HI(T - 1), HI(T), HI(T - 1)>();
    } else if constexpr (OP == OP_FMul) {
        r_mul2<LO(T - 1), LO(T), LO(T - 1)>();
        r_mul2<HI(T - 1), HI(T), HI(T - 1)>();
    } else if constexpr (OP == OP_FSub) {
        r_sub2<LO(T - 1), LO(T), LO(T - 1)>();
        r_sub2<HI(T - 1), HI(T), HI(T - 1)>();
    } else if constexpr (OP == OP_FRSub) {
        r_sub2<LO(T - 1), LO(T - 1), LO(T)>();
        r_sub2<HI(T - 1), HI(T - 1), HI(T)>();
    } else if constexpr (OP == OP_FMA) {  // fma(T, S, U)
        r_fma2<LO(T - 2), LO(T), LO(T - 1), LO(T - 2)>();
        r_fma2<HI(T - 2), HI(T), HI(T - 1), HI(T - 2)>();
    } else if constexpr (OP == OP_FNeg) {
        r_neg2<LO(T)>();
        r_neg2<HI(T)>();
    } else if constexpr (is_scalar_binary<OP>()) {
        float t[4], s[4];
        slot_read<K, T, KI>(t);
        slot_read<K, T - 1, KI>(s);
#pragma unroll
        for (int w = 0; w < 4; w++) s[w] = scalar_binary<OP>(t[w], s[w], operand);
        slot_write<K, T - 1, KI>(s);
    } else if constexpr (is_scalar_unary<OP>()) {
        float t[4];
        slot_read<K, T, KI>(t);
#pragma unroll
        for (int w = 0; w < 4; w++) t[w] = scalar_unary<OP>(t[w]);
        slot_write<K, T, KI>(t);
    }
    /* ---- immediates (immediate.py:7-61) ---- */
    else if constexpr (OP == OP_LoadImm) {
        const u64 v = pack2(__uint_as_float(operand), __uint_as_float(operand));
        r_set64<LO(SP)>(v);
        r_set64<HI(SP)>(v);
    } else if constexpr (OP == OP_FAddImm) {
        const u64 imm = pack2(__uint_as_float(operand), __uint_as_float(operand));
        r_add2_imm<LO(T)>(imm);
        r_add2_imm<HI(T)>(imm);
    } else if constexpr (OP == OP_FMulImm) {
        const u64 imm = pack2(__uint_as_float(operand), __uint_as_float(operand));
        r_mul2_imm<LO(T)>(imm);
        r_mul2_imm<HI(T)>(imm);
    } else if constexpr (OP == OP_FMAImm) {  // f16x2: low half = multiplier, high half = addend
        const float m = __half2float(__ushort_as_half((unsigned short)(operand & 0xFFFFu)));
        const float c = __half2float(__ushort_as_half((unsigned short)(operand >> 16)));
        const u64 m2 = pack2(m, m), c2 = pack2(c, c);
        r_fma2_imm<LO(T)>(m2, c2);
        r_fma2_imm<HI(T)>(m2, c2);
    } else if constexpr (OP == OP_LoadImm4F) {
        r_set<LO(SP)>((float)(signed char)(operand), (float)(signed char)(operand >> 8));
        r_set<HI(SP)>((float)(signed char)(operand >> 16), (float)(signed char)(operand >> 24));
    } else if constexpr (OP == OP_LoadImm4I) {
        r_set<LO(SP)>(__int_as_float((int)(signed char)(operand)), __int_as_float((int)(signed char)(operand >> 8)));
        r_set<HI(SP)>(__int_as_float((int)(signed char)(operand >> 16)), __int_as_float((int)(signed char)(operand >> 24)));
    }
    /* ---- stack moves (move.py:7-55), rightmost = top ---- */
    else if constexpr (OP == OP_Dup) {
        slot_mov<K, SP, T, KI>();
    } else if constexpr (OP == OP_DupX1) {  // [a, b] -> [b, a, b]
        slot_mov<K, SP, T, KI>();
        slot_swap<K, T, T - 1, KI>();
    } else if constexpr (OP == OP_DupX2) {  // [a, b, c] -> [c, a, b, c]
        slot_mov<K, SP, T, KI>();
        slot_mov<K, T, T - 1, KI>();
        slot_mov<K, T - 1, T - 2, KI>();
        slot_mov<K, T - 2, SP, KI>();
    } else if constexpr (OP == OP_Dup2) {  // [a, b] -> [a, b, a, b]
        slot_mov<K, SP, T - 1, KI>();
        slot_mov<K, SP + 1, T, KI>();
    } else if constexpr (OP == OP_Swap) {
        slot_swap<K, T, T - 1, KI>();
    } else if constexpr (OP == OP_Select) {  // T > 0 ? S : U (predication.py:64-73)
        float c[4], x[4], y[4];
        slot_read<K, T, KI>(c);
        slot_read<K, T - 1, KI>(x);
        slot_read<K, T - 2, KI>(y);
#pragma unroll
        for (int w = 0; w < 4; w++) y[w] = c[w] > 0.0f ? x[w] : y[w];
        slot_write<K, T - 2, KI>(y);
    }
    /* ---- width-lane moves (move.py:69-135); operand indices pre-clamped to 0..3 ---- */
    else if constexpr (OP == OP_DupBroadcastW) {
        float t[4];
        slot_read<K, T, KI>(t);
        const float x = sel4(t, operand);
        r_set<LO(SP)>(x, x);
        r_set<HI(SP)>(x, x);
    } else if constexpr (OP == OP_FPermW) {
        float t[4];
        slot_read<K, T, KI>(t);
        const float o[4] = {sel4(t, operand), sel4(t, operand >> 8), sel4(t, operand >> 16), sel4(t, operand >> 24)};
        slot_write<K, T, KI>(o);
    } else if constexpr (OP == OP_FShuf2) {  // vec2 = T, vec1 = S -> (vec1[x], vec1[y], vec2[z], vec2[w])
        float v2[4], v1[4];
        slot_read<K, T, KI>(v2);
        slot_read<K, T - 1, KI>(v1);
        const float o[4] = {sel4(v1, operand), sel4(v1, operand >> 8), sel4(v2, operand >> 16), sel4(v2, operand >> 24)};
        slot_write<K, T - 1, KI>(o);
    }
    /* ---- DupBroadcastW with the lane index built into the opcode (see gint_opcodes.h) ---- */
    else if constexpr (OP >= OP_Bcast_0 && OP <= OP_Bcast_3) {
        r_pick<LO(SP), LO(T), HI(T), (OP - OP_Bcast_0), (OP - OP_Bcast_0)>();
        r_mov<HI(SP), LO(SP)>();
    }
    /* ---- virtual registers: reg n = pool[P-1-n] (state.py:38-41, reg.py:7-59) ---- */
    else if constexpr (OP >= OP_FLoadReg0 && OP <= OP_FLoadReg7) {
        slot_mov<K, SP, P - 1 - (OP - OP_FLoadReg0), KI>();
    } else if constexpr (OP >= OP_FStoreReg0 && OP <= OP_FStoreReg7) {
        slot_mov<K, P - 1 - (OP - OP_FStoreReg0), T, KI>();
    }
    /* ---- virtual registers in shared memory (kernels built with GINT_RF). Register n of tile k is the 512-byte block
     * (n * K + k) of the warp's register area, kept as four planes of 128 bytes: width value w of lane l at byte 128 w + 4 l.
     * %grf = address of block 0 plus 4 * lane. A load or store is four conflict-free 4-byte accesses, and a lane permutation
     * of a register costs nothing: it is the same four loads from other planes (RLoadP = RLoad, FPermW; RLoadS = RLoad a,
     * RLoad b, FShuf2 -- the host merges them, gint_capi.cu: rf_rewrite). Operands: RLoad / RStore 512 n; RLoadP 512 n in
     * bits 0..15 and the four 2-bit plane selectors in bits 16..23; RLoadS 512 a in bits 0..11, 512 b in bits 12..23, the
     * selectors in bits 24..31 (values 0, 1 from register a -- the deeper stack entry --, 2, 3 from b). ---- */
    else if constexpr (OP == OP_RLoad || OP == OP_RLoadP) {
        uint32_t o0 = 0, o1 = 128, o2 = 256, o3 = 384;
        if constexpr (OP == OP_RLoadP) {
            o0 = (operand >> 9) & 0x180u; o1 = (operand >> 11) & 0x180u; o2 = (operand >> 13) & 0x180u; o3 = (operand >> 15) & 0x180u;
        }
        const uint32_t at = rf_base() + (operand & 0xFFFFu) * (uint32_t)K;   // (not volatile: computed once for all K tiles)
        asm volatile("{\n\t.reg .b32 t<4>;\n\t"
                     "ld.shared.b32 t0, [%2+%6];\n\tld.shared.b32 t1, [%3+%6];\n\tld.shared.b32 t2, [%4+%6];\n\tld.shared.b32 t3, [%5+%6];\n\t"
                     "mov.b64 %%gs%0, {t0, t1};\n\tmov.b64 %%gs%1, {t2, t3};\n\t}"
                     ::"n"(LO(SP)), "n"(HI(SP)), "r"(at + o0), "r"(at + o1), "r"(at + o2), "r"(at + o3), "n"(KI * 512) : "memory");
    } else if constexpr (OP == OP_RLoadS) {
        const uint32_t a = rf_base() + (operand & 0xFFFu) * (uint32_t)K, b = rf_base() + ((operand >> 12) & 0xFFFu) * (uint32_t)K;
        const uint32_t o0 = (operand >> 17) & 0x180u, o1 = (operand >> 19) & 0x180u, o2 = (operand >> 21) & 0x180u, o3 = (operand >> 23) & 0x180u;
        asm volatile("{\n\t.reg .b32 t<4>;\n\t"
                     "ld.shared.b32 t0, [%2+%6];\n\tld.shared.b32 t1, [%3+%6];\n\tld.shared.b32 t2, [%4+%6];\n\tld.shared.b32 t3, [%5+%6];\n\t"
                     "mov.b64 %%gs%0, {t0, t1};\n\tmov.b64 %%gs%1, {t2, t3};\n\t}"
                     ::"n"(LO(SP)), "n"(HI(SP)), "r"(a + o0), "r"(a + o1), "r"(b + o2), "r"(b + o3), "n"(KI * 512) : "memory");
    } else if constexpr (OP == OP_RStore) {
        const uint32_t at = rf_base() + operand * (uint32_t)K;
        asm volatile("{\n\t.reg .b32 t<4>;\n\t"
                     "mov.b64 {t0, t1}, %%gs%0;\n\tmov.b64 {t2, t3}, %%gs%1;\n\t"
                     "st.shared.b32 [%2+%3], t0;\n\tst.shared.b32 [%2+%4], t1;\n\tst.shared.b32 [%2+%5], t2;\n\tst.shared.b32 [%2+%6], t3;\n\t}"
                     ::"n"(LO(T)), "n"(HI(T)), "r"(at), "n"(KI * 512), "n"(KI * 512 + 128), "n"(KI * 512 + 256), "n"(KI * 512 + 384) : "memory");
    }
    /* ---- warp all-reduce (reduction.py:7-30, nvptx.py:89-104): butterfly 16, 8, 4, 2, 1 per width lane ---- */
    else if constexpr (OP >= OP_WarpAllReduceSum && OP <= OP_WarpAllReduceProd) {
        float t[4];
        slot_read<K, T, KI>(t);
#pragma unroll
        for (int mask = 16; mask >= 1; mask >>= 1) {
#pragma unroll
            for (int w = 0; w < 4; w++) {
                const float o = __shfl_xor_sync(0xffffffffu, t[w], mask);
                if constexpr (OP == OP_WarpAllReduceSum) t[w] = __fadd_rn(t[w], o);
                else if constexpr (OP == OP_WarpAllReduceMax) t[w] = max_nan(t[w], o);
                else if constexpr (OP == OP_WarpAllReduceMin) t[w] = min_nan(t[w], o);
                else t[w] = __fmul_rn(t[w], o);
            }
        }
        slot_write<K, T, KI>(t);
    }
    /* ---- global memory (load_store.py) ---- */
    else if constexpr (OP == OP_LoadGlobal1DF32Fast) {  // full unit-stride tile (proved by the host): elem = off + lane + 32 w
#ifdef GINT_VEC
        {   // vector layout: lane l holds elements 4l..4l+3 of the tile
            const char *pv = fast_tile_address(cx.tiles + KI, operand) + cx.lane * 16;
            asm volatile("ld.global.v2.b64 {%%gs%0, %%gs%1}, [%2];" ::"n"(LO(SP)), "n"(HI(SP)), "l"(pv) : "memory");
            return;
        }
#endif
        const char *p = fast_tile_address(cx.tiles + KI, operand) + cx.lane * 4;
        asm volatile("{\n\t.reg .b32 t<4>;\n\t"
                     "ld.global.b32 t0, [%2];\n\tld.global.b32 t1, [%2+128];\n\tld.global.b32 t2, [%2+256];\n\tld.global.b32 t3, [%2+384];\n\t"
                     "mov.b64 %%gs%0, {t0, t1};\n\tmov.b64 %%gs%1, {t2, t3};\n\t}" ::"n"(LO(SP)), "n"(HI(SP)), "l"(p) : "memory");
    } else if constexpr (OP == OP_StoreGlobal1DF32Fast) {
#ifdef GINT_VEC
        {
            char *pv = fast_tile_address(cx.tiles + KI, operand) + cx.lane * 16;
            asm volatile("st.global.v2.b64 [%2], {%%gs%0, %%gs%1};" ::"n"(LO(T)), "n"(HI(T)), "l"(pv) : "memory");
            return;
        }
#endif
        char *p = fast_tile_address(cx.tiles + KI, operand) + cx.lane * 4;
        asm volatile("{\n\t.reg .b32 t<4>;\n\t"
                     "mov.b64 {t0, t1}, %%gs%0;\n\tmov.b64 {t2, t3}, %%gs%1;\n\t"
                     "st.global.b32 [%2], t0;\n\tst.global.b32 [%2+128], t1;\n\tst.global.b32 [%2+256], t2;\n\tst.global.b32 [%2+384], t3;\n\t}"
                     ::"n"(LO(T)), "n"(HI(T)), "l"(p) : "memory");
    } else if constexpr (OP == OP_LoadGlobal2DWF32Fast || OP == OP_StoreGlobal2DWF32Fast) {
        /* a 2DW row access that the host proved full, unmasked and 16-byte aligned for every logical program: lane = row,
         * four consecutive floats. Operand as for the 1-D fast accesses: {8 * slot in bits 26..31, byte offset of the column};
         * the row stride comes from the tile descriptor. */
        const TileInfo *ti = cx.tiles + KI;
        const int stride1 = *reinterpret_cast<const int *>(reinterpret_cast<const char *>(ti->s1) + (operand >> 26) + 4);
        char *p = fast_tile_address(ti, operand) + (long long)(cx.lane * stride1) * 4;
        if constexpr (OP == OP_LoadGlobal2DWF32Fast)
            asm volatile("ld.global.v2.b64 {%%gs%0, %%gs%1}, [%2];" ::"n"(LO(SP)), "n"(HI(SP)), "l"(p) : "memory");
        else
            asm volatile("st.global.v2.b64 [%2], {%%gs%0, %%gs%1};" ::"n"(LO(T)), "n"(HI(T)), "l"(p) : "memory");
    } else if constexpr (MemOp<OP>::is) {
        float v[4];
        if constexpr (MemOp<OP>::store) {
            slot_read<K, T, KI>(v);
            tile_rw<MemOp<OP>::layout, MemOp<OP>::dtype, true>(cx.tiles + KI, operand, cx.lane, v);
        } else {
            tile_rw<MemOp<OP>::layout, MemOp<OP>::dtype, false>(cx.tiles + KI, operand, cx.lane, v);
            slot_write<K, SP, KI>(v);
        }
    } else if constexpr (OP == OP_LoadGlobal1DF32Indirect) {  // pops indices, pushes values
        float idx[4], v[4];
        slot_read<K, T, KI>(idx);
        tile_indirect<false>(cx.tiles + KI, operand, idx, v);
        slot_write<K, T, KI>(v);
    } else if constexpr (OP == OP_StoreGlobal1DF32Indirect) {  // indices on top, values below
        float idx[4], v[4];
        slot_read<K, T, KI>(idx);
        slot_read<K, T - 1, KI>(v);
        tile_indirect<true>(cx.tiles + KI, operand, idx, v);
    } else if constexpr (OP == OP_AdvanceBlock2D || OP == OP_AdvanceBase) {  // load_store.py:291-321, operand >> 4 is arithmetic
        if (cx.lane == 0) {
            const int arg = operand & 15;
            const int delta = ((int)operand) >> 4;
            if constexpr (OP == OP_AdvanceBlock2D) cx.tiles[KI].adv[arg] += delta;
            else cx.tiles[KI].ptr[arg] += (u64)(long long)delta;  // bytes
        }
    }
#undef LO
#undef HI
}

template <int OP, int SP, int P, int K, int... KI>
__device__ __forceinline__ void exec_all(const uint32_t operand, const Ctx &cx, std::integer_sequence<int, KI...>)
{
    if constexpr (OP == OP_StageRows) {
        /* operand: tensor slot (bits 0..2), log2 of the 16-byte chunks per row (bits 3..4), byte offset of the block's copy
         * in the warp's row area (bits 8..23). The 32 rows of a tile are contiguous: chunk c = 32 i + lane of the block
         * goes to position swz(c); see staged_row_position. One commit for all tiles. */
        const uint32_t lq = (operand >> 3) & 3u, area = (operand >> 8) & 0xFFFFu;
        auto one = [&](int ki) {
            const char *src = reinterpret_cast<const char *>(cx.tiles[ki].ptr[operand & 7u]) + cx.lane * 16;
            const uint32_t dst = cx_rows<P, K>(cx) + (uint32_t)ki * cx_rows_stride<P, K>(cx) + area;
            for (uint32_t i = 0; i < (1u << lq); i++) {
                const uint32_t c = i * 32u + (uint32_t)cx.lane, m = c >> lq, r = c & ((1u << lq) - 1u);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + staged_row_position(m, r, lq) * 16u), "l"(src + i * 512u) : "memory");
            }
        };
        (one(KI), ...);
        asm volatile("cp.async.commit_group;" ::: "memory");
    } else if constexpr (OP == OP_RemapVN) {
        /* top of the stack from the vector layout (lane l: elements 4l..4l+3 of the tile) to the natural one (lane l: elements
         * l, l+32, l+64, l+96): through the warp's 512-byte-per-tile exchange area (aux_bytes; after the staged row blocks) */
        const uint32_t warp = threadIdx.x >> 5;
        const uint32_t area = cx_after_tiles<K>(cx, warp) + (uint32_t)(kWarpsPerBlock * K) * (cx.args->ring_bytes + cx.args->row_area_bytes) +
                              warp * (uint32_t)(K * 512);
        constexpr int T = SP - 1;
        (put_vector<K, T, KI>(area + (uint32_t)(KI * 512 + cx.lane * 16)), ...);
        __syncwarp();
        (take_natural<K, T, KI>(area + (uint32_t)(KI * 512 + cx.lane * 4)), ...);
        __syncwarp();
    } else if constexpr (OP == OP_LoadStagedRows) {
        /* operand: log2 chunks per row (bits 0..1), which chunk of the lane's row (bits 2..3), area offset (bits 8..23) */
        const uint32_t lq = operand & 3u, part = (operand >> 2) & 3u, area = (operand >> 8) & 0xFFFFu;
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncwarp();
        const uint32_t at = cx_rows<P, K>(cx) + area + staged_row_position((uint32_t)cx.lane, part, lq) * 16u;
        const uint32_t rows_stride = cx_rows_stride<P, K>(cx);
        (take_rows<K, SP, KI>(at + (uint32_t)KI * rows_stride), ...);
    } else if constexpr ((OP >= OP_PfTake && OP <= OP_PfSkip) || OP == OP_PfIssue1DFast || OP == OP_PfTakeIssue1DFast) {
        /* Early-issued loads. One cp.async group per load (all K tiles together). When load n is taken, the D-1 loads
         * after it are in flight, so "all but the newest D-1 groups have landed" is exactly "load n has landed"; a plain
         * PfTake belongs to the tail of the program, where fewer are in flight, and simply waits for everything. */
        constexpr bool take = OP == OP_PfTake || OP == OP_PfTakeIssue1D || OP == OP_PfTakeIssue1DFast;
        uint32_t ring;
        asm volatile("mov.b32 %0, %%gring;" : "=r"(ring));
        const uint32_t slot = cx_hidden<P, K>(cx) + ring;
        const uint32_t ring_mask = cx_ring_mask<P, K>(cx);
        /* the ring has D = 4 or 8 slots, chosen per program by the host (long rows gain from the deeper one); the wait
         * count is an immediate of the instruction, hence the (warp-uniform) branch */
        if constexpr (OP == OP_PfTake) asm volatile("cp.async.wait_group 0;" ::: "memory");
        else if constexpr (take) {
            if (ring_mask & (uint32_t)(K * 2048)) asm volatile("cp.async.wait_group 7;" ::: "memory");
            else asm volatile("cp.async.wait_group 3;" ::: "memory");
        }
        if constexpr (take) {
            __syncwarp();   // the group has landed for every lane: make the other lanes' copies visible to this one
            (take_hidden<K, SP, KI>(slot), ...);
        }
        if constexpr (OP == OP_PfIssue1D || OP == OP_PfTakeIssue1D) (tile_issue<K, KI>(cx.tiles + KI, operand, cx, slot), ...);
        if constexpr (OP == OP_PfIssue1DFast || OP == OP_PfTakeIssue1DFast) (tile_issue_fast<K, KI>(cx.tiles + KI, operand, cx, slot), ...);
        if constexpr (OP != OP_PfTake && OP != OP_PfSkip) asm volatile("cp.async.commit_group;" ::: "memory");
        if constexpr (OP == OP_PfSkip) asm volatile("mad.lo.u32 %%gring, %0, %1, %%gring;\n\tand.b32 %%gring, %%gring, %2;" ::"r"(operand), "n"(K * 512), "r"(ring_mask));
        else asm volatile("add.u32 %%gring, %%gring, %0;\n\tand.b32 %%gring, %%gring, %1;" ::"n"(K * 512), "r"(ring_mask));
    } else {
        if constexpr (OP == OP_AdvanceBlock2D || OP == OP_AdvanceBase) __syncwarp();
        (exec_tile<OP, SP, P, K, KI>(operand, cx), ...);
        if constexpr (OP == OP_AdvanceBlock2D || OP == OP_AdvanceBase) __syncwarp();
    }
}

template <typename S> struct SeqFirst;
template <int OP0, int... REST> struct SeqFirst<Seq<OP0, REST...>> { static constexpr int value = OP0; };
template <typename S> __host__ __device__ constexpr int seq_first() { return SeqFirst<S>::value; }

template <int A, int B> __device__ __forceinline__ void fma_barrier_one()
{
    asm volatile("xor.b64 %%gs%0, %%gs%0, %%gzero;\n\txor.b64 %%gs%1, %%gs%1, %%gzero;" ::"n"(A), "n"(B));
}
template <int K, int SLOT, int... KI> __device__ __forceinline__ void fma_barrier(std::integer_sequence<int, KI...>)
{
    (fma_barrier_one<gs<K>(SLOT, KI, 0), gs<K>(SLOT, KI, 1)>(), ...);
}

/* Run the members of a fused sequence back to back; member J takes its operand from ops[J] if it uses one. */
template <typename S, int SP, int P, int K, int J> struct SeqRun;
template <int SP, int P, int K, int J> struct SeqRun<Seq<>, SP, P, K, J> {
    static __device__ __forceinline__ void run(const Ctx &, const uint32_t *) {}
};
template <int OP0, int... REST, int SP, int P, int K, int J> struct SeqRun<Seq<OP0, REST...>, SP, P, K, J> {
    static __device__ __forceinline__ void run(const Ctx &cx, const uint32_t *ops)
    {
        exec_all<OP0, SP, P, K>(GINT_OP_USES_OPERAND(OP0) ? ops[J] : 0u, cx, std::make_integer_sequence<int, K>());
        if constexpr (sizeof...(REST) > 0 && (OP0 == OP_FMul || OP0 == OP_FMulImm)) {
            /* A product that the next member adds to or subtracts from: inside one handler ptxas contracts the packed
             * multiply and add into a fused multiply-add (observed, even with --fmad=false and explicit .rn), which would
             * change the rounding the bytecode asks for. XOR-ing the product with a zero that the assembler cannot see
             * through keeps the two operations apart. */
            constexpr int next = seq_first<Seq<REST...>>();
            if constexpr (next == OP_FAdd || next == OP_FSub || next == OP_FRSub || next == OP_FAddImm)
                fma_barrier<K, SP + OpInfo<OP0>::net_effect - 1>(std::make_integer_sequence<int, K>());
        }
        SeqRun<Seq<REST...>, SP + OpInfo<OP0>::net_effect, P, K, J + 1>::run(cx, ops);
    }
};
/* Operands of the members after the first: member J's operand is word 0 of the sequence's extra entry number
 * S::entry_of(J) (1-based), i.e. at [base + 8*(entry_of(J)-1)]; the last extra entry also carries, as word 1, the opcode to
 * dispatch on afterwards, so it is fetched as a pair. */
template <typename S, typename Rest, int J> struct SeqFetch;
template <typename S, int J> struct SeqFetch<S, Seq<>, J> {
    static __device__ __forceinline__ void run(uint32_t, uint32_t *, uint32_t &) {}
};
template <typename S, int OP0, int... REST, int J> struct SeqFetch<S, Seq<OP0, REST...>, J> {
    static __device__ __forceinline__ void run(uint32_t base, uint32_t *ops, uint32_t &next_opcode)
    {
        if constexpr (J >= 1 && GINT_OP_USES_OPERAND(OP0)) {
            constexpr int e = S::entry_of(J);
            if constexpr (e == S::entries() - 1) asm volatile("ld.shared.v2.u32 {%0, %1}, [%2+%3];" : "=r"(ops[J]), "=r"(next_opcode) : "r"(base), "n"(8 * (e - 1)));
            else asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(ops[J]) : "r"(base), "n"(8 * (e - 1)));
        }
        SeqFetch<S, Seq<REST...>, J + 1>::run(base, ops, next_opcode);
    }
};

/* ------------------------------------------------------------------------------------------------ */
/* fetch / dispatch loop for one group of K logical programs                                          */

template <int N> __device__ __forceinline__ void pool_clear()
{
    if constexpr (N > 0) {
        pool_clear<N - 1>();
        r_set64<N - 1>(0ull);
    }
}

/*
 * Interpreter state that is carried from one handler to the next lives, like the pool, in named PTX registers:
 *   %gc          address of the next stream entry to fetch (shared-memory address, or a global pointer in indirect mode)
 *   %ge0, %ge1   the current stream entry {operand of this instruction, opcode of the next one}
 *   %gkey        dispatch key for the C++ fallback switch (dead once the jump tables are in place)
 *   %gbudget     instructions left before the interpreter gives up (only with GINT_GUARD, a debugging aid)
 *   %gring       byte offset of the current slot in the warp's ring of early-issued loads
 *   %gzero       64 bits of zero that reach the kernel as a launch parameter (see fma_barrier)
 *   %grf         shared-memory address of the warp's virtual registers plus 4 * lane (kernels built with GINT_RF)
 * so no C++ value is live from handler to handler and a handler's basic block can be entered from any other handler.
 */
template <bool SMEM> __device__ __forceinline__ void state_declare()
{
#ifdef GINT_RF
    asm volatile(".reg .b32 %%grf; // %0" ::"n"(0));
#endif
    // (the unused "n" operand makes nvcc treat the string as a template, so that %% means %)
    if constexpr (SMEM) asm volatile(".reg .b32 %%gc; .reg .b32 %%ge<2>; .reg .b32 %%gkey; .reg .b32 %%gbudget; .reg .b32 %%gring; .reg .b64 %%gzero; // %0" ::"n"(0));
    else asm volatile(".reg .b64 %%gc; .reg .b32 %%ge<2>; .reg .b32 %%gkey; .reg .b32 %%gbudget; .reg .b32 %%gring; .reg .b64 %%gzero; // %0" ::"n"(0));
}

/* read the current entry, then start loading the following one */
template <bool SMEM> __device__ __forceinline__ void state_advance(uint32_t &operand, uint32_t &next_opcode)
{
    asm volatile("mov.b32 %0, %%ge0; mov.b32 %1, %%ge1;" : "=r"(operand), "=r"(next_opcode));
    if constexpr (SMEM) asm volatile("ld.shared.v2.u32 {%%ge0, %%ge1}, [%%gc]; add.u32 %%gc, %%gc, 8; // %0" ::"n"(0) : "memory");
    else asm volatile("ld.global.nc.v2.u32 {%%ge0, %%ge1}, [%%gc]; add.u64 %%gc, %%gc, 8; // %0" ::"n"(0) : "memory");
}

/*
 * Threaded dispatch. The pre-decoded stream is skewed: entry 0 = {-, opcode of insn 0}, entry i+1 = {operand of insn i,
 * opcode of insn i+1}. On entry to the handler of insn i, (%ge0, %ge1) hold entry i+1 -- everything this handler needs
 * (its own operand) and everything the NEXT dispatch needs (the next opcode; the next stack depth is a compile-time
 * property of the handler) -- and the handler's first act is to start the load of entry i+2. Each handler ends in its own
 * dispatch, so there is one indirect branch per interpreted instruction and the jump-table lookup for the next handler can
 * be issued before the current handler's payload.
 *
 * The marker comments survive into the PTX. nvcc lowers a C++ switch to a compare tree (about ten dependent branches for
 * this many cases) and never emits an indirect branch; the build step gint_b200/ptx_dispatch.py ends every handler with
 * one `brx.idx` jump-table branch, indexed by the opcode into the table of that handler's next stack depth and targeting
 * the blocks that carry TARGET markers. Without that step the code below is still a correct (slower) interpreter: every
 * handler loops back to the switch. With THREADED = false only the loop-top dispatch becomes a jump table (over all
 * (depth, opcode) keys) and handlers branch back to it: one more branch per instruction, but a control-flow graph that
 * ptxas digests in seconds whatever surrounds the interpreter.
 */
/* A fused handler covers n consecutive instructions but only m = S::entries() stream entries (see SeqFetch). On entry %ge
 * holds the first of them, {operand of the first member, opcode after the sequence if m == 1}, and %gc points at the
 * next entry. (Shared-memory streams only.) */
template <int NUM, int SP, int P, int K>
__device__ __forceinline__ void run_fused(const Ctx &cx, uint32_t &next_opcode)
{
    using S = typename FusedSeq<NUM>::type;
    constexpr int m = S::entries();
    uint32_t ops[GINT_MAX_FUSED_LEN];
    if constexpr (m == 1) {
        state_advance<true>(ops[0], next_opcode);
    } else {
        uint32_t base;
        asm volatile("mov.b32 %0, %%ge0; mov.b32 %1, %%gc;" : "=r"(ops[0]), "=r"(base));
        SeqFetch<S, S, 0>::run(base, ops, next_opcode);
        asm volatile("ld.shared.v2.u32 {%%ge0, %%ge1}, [%%gc+%0]; add.u32 %%gc, %%gc, %1;" ::"n"(8 * (m - 1)), "n"(8 * m) : "memory");
    }
#ifdef GINT_GUARD
    {
        uint32_t left;
        asm volatile("sub.u32 %%gbudget, %%gbudget, %1; mov.u32 %0, %%gbudget;" : "=r"(left) : "n"(S::n));
        if ((int)left < 0) { GINT_GUARD_TRIPPED; return; }
    }
#endif
    SeqRun<S, SP, P, K, 0>::run(cx, ops);
}

template <int P, int K, bool SMEM_CODE, bool THREADED>
__device__ __forceinline__ void interpret(const uint2 *code, uint32_t n_entries, const Ctx &cx)
{
    pool_clear<2 * P * K>();
    if constexpr (SMEM_CODE) {
        const uint32_t a = (uint32_t)__cvta_generic_to_shared(code);
        asm volatile("ld.shared.u32 %%gkey, [%0+4]; ld.shared.v2.u32 {%%ge0, %%ge1}, [%0+8]; add.u32 %%gc, %0, 16; mov.u32 %%gbudget, %1; mov.u32 %%gring, 0;"
                     ::"r"(a), "r"(n_entries) : "memory");
    } else {
        asm volatile("ld.global.nc.u32 %%gkey, [%0+4]; ld.global.nc.v2.u32 {%%ge0, %%ge1}, [%0+8]; add.u64 %%gc, %0, 16; mov.u32 %%gbudget, %1; mov.u32 %%gring, 0;"
                     ::"l"(code), "r"(n_entries) : "memory");
    }
    for (;;) {
        uint32_t key;
        asm volatile("mov.b32 %0, %%gkey;" : "=r"(key));
        if constexpr (THREADED) asm volatile("// GINT_DISPATCH %0 site entry depth 0;" ::"r"(key));
        else asm volatile("// GINT_DISPATCH %0 site entry depth all;" ::"r"(key));
        switch (key) {
#define GINT_CASE_SP(num, spv)                                                                          \
    case (spv) * GINT_N_DISPATCH + (num):                                                                \
        if constexpr (op_valid<num, spv, P, K>()) {                                                     \
            asm volatile("// GINT_TARGET %0;" ::"n"((spv) * GINT_N_DISPATCH + (num)));                   \
            if constexpr ((num) == OP_Halt) return;                                                     \
            else {                                                                                      \
                constexpr int next_depth = (spv) + OpInfo<num>::net_effect;                             \
                uint32_t operand, opc;                                                                  \
                if constexpr (GINT_IS_FUSED(num)) {                                                     \
                    run_fused<num, spv, P, K>(cx, opc);                                                 \
                } else {                                                                                \
                    state_advance<SMEM_CODE>(operand, opc);                                             \
                    GINT_GUARD_STEP                                                                     \
                    exec_all<num, spv, P, K>(operand, cx, std::make_integer_sequence<int, K>());        \
                }                                                                                       \
                asm volatile("add.u32 %%gkey, %0, %1;" ::"r"(opc), "n"(next_depth * GINT_N_DISPATCH));   \
                if constexpr (THREADED)                                                                 \
                    asm volatile("// GINT_DISPATCH %0 site %1 depth %2;" ::"r"(opc),                     \
                                 "n"((spv) * GINT_N_DISPATCH + (num)), "n"(next_depth));                 \
            }                                                                                           \
        }                                                                                               \
        continue;
#define GINT_X_CASES(name, num, md, net)                                                                           \
    GINT_CASE_SP(num, 0) GINT_CASE_SP(num, 1) GINT_CASE_SP(num, 2) GINT_CASE_SP(num, 3) GINT_CASE_SP(num, 4)       \
    GINT_CASE_SP(num, 5) GINT_CASE_SP(num, 6) GINT_CASE_SP(num, 7) GINT_CASE_SP(num, 8)
            GINT_OPCODE_LIST(GINT_X_CASES)
            GINT_INTERNAL_OPCODE_LIST(GINT_X_CASES)
#define GINT_X_FCASES(num, len, ...) GINT_X_CASES(fused, num, 0, 0)
            GINT_FUSED_LIST(GINT_X_FCASES)
#ifdef GINT_RF
            GINT_RF_OPCODE_LIST(GINT_X_CASES)
            GINT_RF_FUSED_LIST(GINT_X_FCASES)
#endif
#ifdef GINT_VEC
            GINT_VEC_OPCODE_LIST(GINT_X_CASES)
#endif
#undef GINT_X_FCASES
#undef GINT_X_CASES
#undef GINT_CASE_SP
        default:
            asm volatile("// GINT_TARGET default;");
#ifdef GINT_CHECKED
            chk_record(GINT_DEVICE_BAD_DISPATCH, -1, (u64)key);
#endif
            return;
        }
    }
}

/* ------------------------------------------------------------------------------------------------ */
/* kernels                                                                                           */

/*
 * The interpreter consumes every load right away (the value is needed by the next bytecode instruction), so by itself it
 * keeps only one tile per warp in flight and is bound by memory latency. The bytecode is straight-line, though, so what
 * each logical program will read is known before it starts: right after the descriptors of a group are decoded, the warp
 * asks for those bytes to be brought into L2 (prefetch.global.L2, one 128-byte line per lane and step). The loads that
 * follow then hit L2 while the DRAM transfers of the rest of the footprint overlap with interpretation.
 */
template <int K>
__device__ __forceinline__ void prefetch_footprints(const LaunchArgs &a, const TileInfo *tiles, int lane)
{
    for (uint32_t m = a.prefetch_mask; m; m &= m - 1) {
        const int t = __ffs(m) - 1;
        const Footprint f = a.fp[t];
#pragma unroll
        for (int k = 0; k < K; k++) {
            const TileInfo *ti = tiles + k;
            const char *base = reinterpret_cast<const char *>(ti->ptr[t]);
            const int2 s1 = ti->s1[t];
            if (f.kind == FP_1D) {
                if (s1.y != 1) continue;
                const int hi = min(f.hi, s1.x);
                const char *p = base + (long long)f.lo * 4;
                const char *end = base + (long long)hi * 4;
                for (p += lane * 128; p < end; p += 32 * 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
            } else {
                const int2 s2 = ti->s2[t];
                if (s2.y != 1 || lane >= s1.x) continue;
                const int hi = min(f.hi, s2.x);
                const char *p = base + ((long long)lane * s1.y + f.lo) * 4;
                const char *end = base + ((long long)lane * s1.y + hi) * 4;
                for (; p < end; p += 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
            }
        }
    }
}

/* Indirect mode: copy one program and its descriptor block from global memory into the warp's shared-memory slice. */
static __device__ __noinline__ void stage_for_warp(uint2 *code_s, const uint2 *code_g, uint32_t n_slots, gint_tensor_info *ti_s,
                                                   const gint_tensor_info *ti_g, int lane)
{
    for (uint32_t i = lane; i < n_slots; i += 32) code_s[i] = __ldg(code_g + i);
    const int *src = reinterpret_cast<const int *>(ti_g);
    int *dst = reinterpret_cast<int *>(ti_s);
    for (uint32_t i = lane; i < sizeof(gint_tensor_info) / 4; i += 32) dst[i] = __ldg(src + i);
    __syncwarp();
}

/* Direct mode: every logical program runs the same bytecode. Persistent blocks of kWarpsPerBlock warps;
 * shared memory = [program | descriptor block | kWarpsPerBlock x K TileInfo | kWarpsPerBlock x load staging]. */
template <int P, int K, bool THREADED = true>
__device__ __forceinline__ void geval_direct_body(const LaunchArgs &a)
{
    extern __shared__ __align__(16) unsigned char smem[];
    pool_declare<P, K>();
    state_declare<true>();
    asm volatile("mov.b64 %%gzero, %0;" ::"l"((u64)a.zero));
    uint2 *code_s = reinterpret_cast<uint2 *>(smem);
    gint_tensor_info *ti_s = reinterpret_cast<gint_tensor_info *>(smem + a.code_smem_bytes);
    TileInfo *tiles_s = reinterpret_cast<TileInfo *>(smem + a.code_smem_bytes + kTensorInfoSmemBytes);

    /* a short program travels inside the parameter block (a.code == nullptr): staging it costs no global-memory round trip,
     * which is most of what a launch of a few instructions per tile would otherwise wait for before its first load */
    if (a.code == nullptr) {
        if (threadIdx.x < a.n_slots) code_s[threadIdx.x] = a.inline_code[threadIdx.x];
    } else {
        for (uint32_t i = threadIdx.x; i < a.n_slots; i += kThreadsPerBlock) code_s[i] = a.code[i];
    }
    {
        const int *src = reinterpret_cast<const int *>(&a.ti);
        int *dst = reinterpret_cast<int *>(ti_s);
        for (uint32_t i = threadIdx.x; i < sizeof(gint_tensor_info) / 4; i += kThreadsPerBlock) dst[i] = src[i];
    }
#ifdef GINT_CHECKED
    if (threadIdx.x < GINT_MAX_TENSORS) {
        g_chk.lo[threadIdx.x] = a.chk_lo[threadIdx.x];
        g_chk.hi[threadIdx.x] = a.chk_hi[threadIdx.x];
    }
    if (threadIdx.x == 0) {
        g_chk.status = reinterpret_cast<gint_device_status *>(a.chk_status);
        g_chk.code_base = (uint32_t)__cvta_generic_to_shared(code_s);
    }
#endif
    __syncthreads();

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    Ctx cx;
    cx.tiles = tiles_s + warp * K;
    cx.lane = lane;
    cx.args = &a;
    if constexpr (!lean_ctx<P, K>()) {   // after the tile descriptors: the ring of early-issued loads (ring_bytes per tile), then the staged row blocks
        unsigned char *after = reinterpret_cast<unsigned char *>(tiles_s + kWarpsPerBlock * K);
#ifdef GINT_VEC
        cx.hidden = (uint32_t)__cvta_generic_to_shared(after + (size_t)(warp * K) * a.ring_bytes + lane * 16);   // lane l owns elements 4l..4l+3
#else
        cx.hidden = (uint32_t)__cvta_generic_to_shared(after + (size_t)(warp * K) * a.ring_bytes + lane * 4);
#endif
        cx.rows = (uint32_t)__cvta_generic_to_shared(after + (size_t)(kWarpsPerBlock * K) * a.ring_bytes + (size_t)(warp * K) * a.row_area_bytes);
        cx.rows_stride = a.row_area_bytes;
        cx.ring_mask = (uint32_t)K * a.ring_bytes - 1u;
    }
#ifdef GINT_RF
    {   /* after the staged row blocks: the virtual registers, rf_bytes (512 per register) per tile */
        unsigned char *after = reinterpret_cast<unsigned char *>(tiles_s + kWarpsPerBlock * K);
        const uint32_t rf = (uint32_t)__cvta_generic_to_shared(after + (size_t)(kWarpsPerBlock * K) * (a.ring_bytes + a.row_area_bytes) +
                                                               (size_t)(warp * K) * a.rf_bytes + lane * 4);
        asm volatile("mov.b32 %%grf, %0;" ::"r"(rf));
    }
#endif

    const uint32_t n_groups = (a.end - a.first + (uint32_t)K - 1u) / (uint32_t)K;
    for (uint32_t g = blockIdx.x * kWarpsPerBlock + warp; g < n_groups; g += gridDim.x * kWarpsPerBlock) {
        __syncwarp();  // every lane is done with the previous group's tile descriptors
        decode_tiles<K>(ti_s, (int)a.n_tensors, a.first + g * (uint32_t)K, a.end, cx.tiles, lane, a.gather_mask, a.gather_index, a.gather_rows);
        if (a.prefetch_mask) prefetch_footprints<K>(a, cx.tiles, lane);
#ifdef GINT_CHECKED
        if (lane == 0) g_chk.logical[warp] = a.first + g * (uint32_t)K;
        __syncwarp();
#endif
#ifdef GINT_CHECKED
        /* the instruction budget: a stream entry stands for at most GINT_MAX_FUSED_LEN instructions (a fused handler) */
        interpret<P, K, true, THREADED>(code_s, a.n_slots * (uint32_t)GINT_MAX_FUSED_LEN, cx);
#else
        interpret<P, K, true, THREADED>(code_s, a.n_slots, cx);
#endif
    }
}

/* Indirect mode (main.py:179-194, flag > 0): logical program i has its own bytecode and descriptors, listed in a
 * per-program table. Each warp copies them into its own slice of shared memory ([TileInfo | descriptor block | program],
 * `code_smem_bytes` for the program) and interprets from there. */
template <int P>
__device__ __forceinline__ void geval_indirect_body(const IndirectArgs &a)
{
    extern __shared__ __align__(16) unsigned char smem[];
    pool_declare<P, 1>();
    state_declare<true>();
    asm volatile("mov.b64 %%gzero, %0;" ::"l"((u64)a.reserved));
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned char *mine = smem + (size_t)warp * (sizeof(TileInfo) + kTensorInfoSmemBytes + a.code_smem_bytes);
    gint_tensor_info *ti_s = reinterpret_cast<gint_tensor_info *>(mine + sizeof(TileInfo));
    uint2 *code_s = reinterpret_cast<uint2 *>(mine + sizeof(TileInfo) + kTensorInfoSmemBytes);
    Ctx cx;
    cx.tiles = reinterpret_cast<TileInfo *>(mine);
    cx.lane = lane;
    cx.hidden = 0;   // indirect mode runs programs as written (no early-issued loads, no staged rows)
    cx.rows = 0;
    cx.rows_stride = 0;
    cx.ring_mask = 0;
    cx.args = nullptr;
    for (uint32_t g = blockIdx.x * kWarpsPerBlock + warp; g < a.grid_dim; g += gridDim.x * kWarpsPerBlock) {
        const IndirectEntry e = a.table[g];
        __syncwarp();  // every lane is done with the previous program's code and descriptors
        if (e.n_slots == 0) continue;   // warp-uniform: the entry belongs to the whole warp
        stage_for_warp(code_s, e.code, e.n_slots, ti_s, e.ti, lane);
        if (e.patch_slot) {
            if (lane == 0) ti_s->base_ptr[e.patch_slot - 1u] = (int64_t)e.patch_ptr;
            __syncwarp();
        }
        decode_tiles<1>(ti_s, (int)a.n_tensors, g, a.grid_dim, cx.tiles, lane);
        interpret<P, 1, true, false>(code_s, e.n_slots, cx);
    }
}

}  // namespace gint

/* Entry points have C names so the host can look them up in the loaded cubin by name. */
#define GINT_DEFINE_INDIRECT_KERNEL(P)                                                                          \
    extern "C" __global__ void __launch_bounds__(gint::kThreadsPerBlock, GINT_MIN_BLOCKS(P, 1))                  \
        gint_geval_indirect_##P(const __grid_constant__ gint::IndirectArgs a)                                   \
    {                                                                                                           \
        gint::geval_indirect_body<P>(a);                                                                        \
    }
/* The checked kernel: direct mode, one tile per warp, dispatch through a single jump table (compiles in seconds). */
#define GINT_DEFINE_CHECKED_KERNEL(P)                                                                           \
    extern "C" __global__ void __launch_bounds__(gint::kThreadsPerBlock, 4)                                      \
        gint_geval_checked_##P(const __grid_constant__ gint::LaunchArgs a)                                       \
    {                                                                                                           \
        gint::geval_direct_body<P, 1, false>(a);                                                                \
    }
#define GINT_DEFINE_RF_KERNEL(P, K)                                                                             \
    extern "C" __global__ void __launch_bounds__(gint::kThreadsPerBlock, GINT_MIN_BLOCKS(P, K))                  \
        gint_geval_rf_##P##_##K(const __grid_constant__ gint::LaunchArgs a)                                      \
    {                                                                                                           \
        gint::geval_direct_body<P, K>(a);                                                                       \
    }
#define GINT_DEFINE_VEC_KERNEL(P, K)                                                                            \
    extern "C" __global__ void __launch_bounds__(gint::kThreadsPerBlock, GINT_MIN_BLOCKS(P, K))                  \
        gint_geval_vec_##P##_##K(const __grid_constant__ gint::LaunchArgs a)                                     \
    {                                                                                                           \
        gint::geval_direct_body<P, K>(a);                                                                       \
    }
#define GINT_DEFINE_DIRECT_KERNEL(P, K)                                                                         \
    extern "C" __global__ void __launch_bounds__(gint::kThreadsPerBlock, GINT_MIN_BLOCKS(P, K))                  \
        gint_geval_direct_##P##_##K(const __grid_constant__ gint::LaunchArgs a)                                  \
    {                                                                                                           \
        gint::geval_direct_body<P, K>(a);                                                                       \
    }
