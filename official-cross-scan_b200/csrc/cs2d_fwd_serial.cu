// The forward kernels in the form that serves the reproducible direction merge: one CTA walks all groups
// (scan directions) of its channel tile, one after the other (see the note at the top of cs2d_fwd.cu).
#define CS2D_SERIAL_DIRS 1
#include "cs2d_fwd.cu"
