// Interpreter kernel for a pool of 12 slots, 1 logical program(s) per warp (see gint_interp.cuh).
#include "../gint_interp.cuh"
GINT_DEFINE_DIRECT_KERNEL(12, 1)
