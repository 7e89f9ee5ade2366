// Indirect-mode interpreter kernel (one program per warp, bytecode fetched from global memory), pool of 12 slots.
#include "gint_interp.cuh"
#include "gint_variants.h"
template __global__ void gint::geval_indirect<12>(const __grid_constant__ gint::IndirectArgs);
extern "C" const void *gint_kernel_indirect_12(void) { return reinterpret_cast<const void *>(&gint::geval_indirect<12>); }
