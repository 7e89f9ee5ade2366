// Indirect-mode interpreter kernel (one program per warp, staged into the warp's shared-memory slice), pool of 12 slots.
#include "../gint_interp.cuh"
GINT_DEFINE_INDIRECT_KERNEL(12)
