// Interpreter kernel for a pool of 4 slots, 1 logical program(s) per warp (see gint_interp.cuh).
#include "gint_interp.cuh"
#include "gint_variants.h"
template __global__ void gint::geval_direct<4, 1>(const __grid_constant__ gint::LaunchArgs);
extern "C" const void *gint_kernel_direct_4_1(void) { return reinterpret_cast<const void *>(&gint::geval_direct<4, 1>); }
