// The weight-streaming product of at most 16 rows (linear_rows.cuh), built for float32: the decode road of the
// 32-bit engine.
#include "linear_rows.cuh"

KVAD_LINEAR_ROWS_LIBRARY(float, KVAD_DTYPE_F32)
