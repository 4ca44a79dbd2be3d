/*
 * TEST INFRASTRUCTURE - NOT PRODUCT CODE.  See cs2d_oracle_impl.h.
 * Builds the CPU restatement twice: float64 (the arbiter) and float32 (the
 * timed CPU baseline).  Only tests/, the smoke check and the benchmark's
 * cpu_baseline leg may load this library.
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <stddef.h>

typedef struct {
    int batch, dim, nrows, ncols, dstate, n_groups, delta_dim, delta_softplus;
} cs2d_oracle_shape;

#define REAL double
#define SUF _f64
#include "cs2d_oracle_impl.h"
#undef REAL
#undef SUF

#define REAL float
#define SUF _f32
#include "cs2d_oracle_impl.h"
#undef REAL
#undef SUF

int cs2d_oracle_max_threads(void) {
#ifdef _OPENMP
    extern int omp_get_max_threads(void);
    return omp_get_max_threads();
#else
    return 1;
#endif
}
