// Interpreter kernel for a pool of 7 slots, 1 logical program(s) per warp (see gint_interp.cuh).
#include "gint_interp.cuh"
#include "gint_variants.h"
template __global__ void gint::geval_direct<7, 1>(const __grid_constant__ gint::LaunchArgs);
extern "C" const void *gint_kernel_direct_7_1(void) { return reinterpret_cast<const void *>(&gint::geval_direct<7, 1>); }
