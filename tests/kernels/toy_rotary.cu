// A toy rotary position encoding with a kernel of its own, brought to the library from the tests
// folder through `kvad_b200.ops.register_kernels`: no file of the package knows it.  Pairs
// (2i, 2i+1) of every head of the rows' queries and keys are turned by position * theta^(-2i/head_dim).
// The angle is taken in double so that the test can hold it to the float64 plain implementation.
#include "common.cuh"

using namespace kvad;

template <typename T>
__global__ void toy_rotary_kernel(T* __restrict__ x, int64_t ld, const int* __restrict__ row_pos, int n_rows,
                                  int n_heads, int head_dim, double theta) {
  pdl_launch_dependents();
  pdl_wait();
  const int half = head_dim / 2;
  const int64_t total = (int64_t)n_rows * n_heads * half;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int p = (int)(i % half), h = (int)((i / half) % n_heads), r = (int)(i / ((int64_t)half * n_heads));
    double s, c;
    sincos((double)row_pos[r] * pow(theta, -2.0 * p / head_dim), &s, &c);
    T* at = x + r * ld + (int64_t)h * head_dim + 2 * p;
    const double a = (double)to_f32(at[0]), b = (double)to_f32(at[1]);
    at[0] = from_f32<T>((float)(a * c - b * s));
    at[1] = from_f32<T>((float)(a * s + b * c));
  }
}

KVAD_DEFINE_LAST_ERROR()

KVAD_EXPORT int toy_rotary(int dtype, void* x, int64_t ld, const int* row_pos, int n_rows, int n_heads, int head_dim,
                           double theta, cudaStream_t stream) {
  KVAD_REQUIRE(head_dim > 0 && head_dim % 2 == 0 && n_heads > 0 && n_rows >= 0, "toy_rotary: bad sizes");
  if (n_rows == 0) return KVAD_OK;
  const int64_t total = (int64_t)n_rows * n_heads * (head_dim / 2);
  const int blocks = (int)((total + 255) / 256 < 1184 ? (total + 255) / 256 : 1184);
  if (dtype == KVAD_DTYPE_F32)
    kvad_launch(toy_rotary_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)x, ld, row_pos, n_rows, n_heads, head_dim, theta);
  else if (dtype == KVAD_DTYPE_BF16)
    kvad_launch(toy_rotary_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16*)x, ld, row_pos, n_rows, n_heads, head_dim, theta);
  else
    KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "toy_rotary: unknown dtype %d", dtype);
  KVAD_CHECK_LAUNCH("toy_rotary");
  return KVAD_OK;
}
