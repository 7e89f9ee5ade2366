/*
 * gint_variants.h -- the interpreter kernels shipped inside libgint_b200.so.
 *
 * Each (pool size P, tiles per warp K) pair is compiled separately (gint_b200/csrc/kernels/), its dispatch switch is
 * turned into a jump table at the PTX level (gint_b200/ptx_dispatch.py), and the resulting sm_100a cubin is embedded in
 * the library as a byte array. The host loads the arrays with cudaLibraryLoadData and looks the kernels up by name.
 */
#ifndef GINT_VARIANTS_H
#define GINT_VARIANTS_H

#ifdef __cplusplus
extern "C" {
#endif

#define GINT_DIRECT_VARIANTS(X) X(4, 1) X(4, 2) X(4, 4) X(7, 1) X(7, 2) X(12, 1) X(12, 2)
#define GINT_RF_VARIANTS(X) X(7, 2)       /* virtual registers in shared memory (GINT_RF): the pool is the operand stack alone */
#define GINT_VEC_VARIANTS(X) X(4, 1) X(4, 2)   /* 1-D tiles in the vector layout (GINT_VEC): lane l holds elements 4l..4l+3 */
#define GINT_INDIRECT_VARIANTS(X) X(12)
#define GINT_CHECKED_VARIANTS(X) X(12)

#define GINT_X_DECL(P, K)                                        \
    extern const unsigned char gint_cubin_direct_##P##_##K[];     \
    extern const unsigned char gint_cubin_direct_##P##_##K##_end[];
GINT_DIRECT_VARIANTS(GINT_X_DECL)
#undef GINT_X_DECL
#define GINT_X_DECL(P, K)                                    \
    extern const unsigned char gint_cubin_rf_##P##_##K[];     \
    extern const unsigned char gint_cubin_rf_##P##_##K##_end[];
GINT_RF_VARIANTS(GINT_X_DECL)
#undef GINT_X_DECL
#define GINT_X_DECL(P, K)                                     \
    extern const unsigned char gint_cubin_vec_##P##_##K[];     \
    extern const unsigned char gint_cubin_vec_##P##_##K##_end[];
GINT_VEC_VARIANTS(GINT_X_DECL)
#undef GINT_X_DECL
#define GINT_X_DECL(P)                                     \
    extern const unsigned char gint_cubin_indirect_##P[];   \
    extern const unsigned char gint_cubin_indirect_##P##_end[];
GINT_INDIRECT_VARIANTS(GINT_X_DECL)
#undef GINT_X_DECL
#define GINT_X_DECL(P)                                    \
    extern const unsigned char gint_cubin_checked_##P[];   \
    extern const unsigned char gint_cubin_checked_##P##_end[];
GINT_CHECKED_VARIANTS(GINT_X_DECL)
#undef GINT_X_DECL

#ifdef __cplusplus
}
#endif
#endif
