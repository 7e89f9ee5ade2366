// Interpreter kernel, pool of 4 slots, 1 logical program(s) per warp, 1-D tiles in the vector layout (lane l holds elements
// 4l..4l+3 of a tile: one 16-byte access per lane; see GINT_VEC in gint_interp.cuh).
#define GINT_VEC 1
#include "../gint_interp.cuh"
GINT_DEFINE_VEC_KERNEL(4, 1)
