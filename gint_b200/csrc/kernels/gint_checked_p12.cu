// Checked interpreter kernel: pool of 12 slots, one logical program per warp, every tensor access compared with the tensor's
// declared byte range (see GINT_CHECKED in gint_interp.cuh). Runs programs as written (no early-issued loads, no fused handlers).
#define GINT_CHECKED 1
#include "../gint_interp.cuh"
GINT_DEFINE_CHECKED_KERNEL(12)
