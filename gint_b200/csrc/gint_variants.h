/*
 * gint_variants.h -- the kernel instantiations compiled into libgint_b200.so.
 *
 * Each (pool size P, tiles per warp K) pair is compiled in its own translation unit so the build runs in
 * parallel; the host side only needs the kernel's address (for cudaLaunchKernel, cudaFuncGetAttributes and the
 * occupancy query).
 */
#ifndef GINT_VARIANTS_H
#define GINT_VARIANTS_H

#ifdef __cplusplus
extern "C" {
#endif

#define GINT_DIRECT_VARIANTS(X) X(4, 1) X(4, 2) X(4, 4) X(7, 1) X(7, 2) X(12, 1) X(12, 2)
#define GINT_INDIRECT_VARIANTS(X) X(12)

#define GINT_X_DECL(P, K) const void *gint_kernel_direct_##P##_##K(void);
GINT_DIRECT_VARIANTS(GINT_X_DECL)
#undef GINT_X_DECL
#define GINT_X_DECL(P) const void *gint_kernel_indirect_##P(void);
GINT_INDIRECT_VARIANTS(GINT_X_DECL)
#undef GINT_X_DECL

#ifdef __cplusplus
}
#endif
#endif
