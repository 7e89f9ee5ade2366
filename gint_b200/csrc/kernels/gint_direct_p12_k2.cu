// Interpreter kernel for a pool of 12 slots, 2 logical program(s) per warp (see gint_interp.cuh).
#include "../gint_interp.cuh"
GINT_DEFINE_DIRECT_KERNEL(12, 2)
