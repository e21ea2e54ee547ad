// The weight-streaming product of at most 16 rows (linear_rows.cuh), built for bfloat16.
#include "linear_rows.cuh"

KVAD_LINEAR_ROWS_LIBRARY(__nv_bfloat16, KVAD_DTYPE_BF16)
