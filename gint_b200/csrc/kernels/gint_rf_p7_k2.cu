// Interpreter kernel with the virtual registers in shared memory: the pool of 7 slots is the operand stack alone,
// 2 logical programs per warp (see GINT_RF in gint_interp.cuh).
#define GINT_RF 1
#include "../gint_interp.cuh"
GINT_DEFINE_RF_KERNEL(7, 2)
