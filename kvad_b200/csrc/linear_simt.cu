// out[M,N] = A[M,K] . W[N,K]^T + bias, on the CUDA cores in true 32-bit
// arithmetic: every product is an fmaf into a 32-bit accumulator and every
// output element sums k = 0..K-1 in that order, whatever M is and wherever the
// row sits in the batch.  This is the matrix kernel of the float32 engine, and
// the fallback of the bfloat16 engine for shapes its tensor-core kernel
// refuses.  bisand/kvad's counterpart is its CPU gemm_bt / matvec_bt
// (crates/llm/src/tensor.rs:56-193), bias added after the product
// (crates/llm/src/quant.rs:849-857).
#include "common.cuh"

using namespace kvad;

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;
constexpr int THREADS = (BM / TM) * (BN / TN);  // 256

template <typename T, int EPI>
__global__ void __launch_bounds__(THREADS)
linear_simt_kernel(const T* __restrict__ A, int64_t lda, const T* __restrict__ W,
                   const void* __restrict__ bias, int bias_f32, void* __restrict__ out,
                   int64_t ldo, int M, int N, int K) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tx = threadIdx.x % (BN / TN), ty = threadIdx.x / (BN / TN);
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;

  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  // each thread stages 4 elements of A and 4 of W per K tile
  const int lr = threadIdx.x / 4;          // 0..63: row of the tile
  const int lk = (threadIdx.x % 4) * 4;    // 0,4,8,12: first k of four

  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int k = k0 + lk + e;
      const int m = m0 + lr, n = n0 + lr;
      As[lk + e][lr] = (m < M && k < K) ? to_f32(A[(int64_t)m * lda + k]) : 0.f;
      Ws[lk + e][lr] = (n < N && k < K) ? to_f32(W[(int64_t)n * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Ws[k][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (bias != nullptr) v += load_param(bias, n, bias_f32);
      const int64_t o = (int64_t)m * ldo + n;
      if (EPI == EPI_STORE) {
        reinterpret_cast<T*>(out)[o] = from_f32<T>(v);
      } else if (EPI == EPI_GELU_TANH) {
        reinterpret_cast<T*>(out)[o] = from_f32<T>(gelu_tanh(v));
      } else if (EPI == EPI_GELU_ERF) {
        reinterpret_cast<T*>(out)[o] = from_f32<T>(gelu_erf(v));
      } else if (EPI == EPI_RESIDUAL) {
        reinterpret_cast<float*>(out)[o] += v;
      } else {
        reinterpret_cast<float*>(out)[o] = v;
      }
    }
  }
}

template <typename T>
int launch(const void* A, int64_t lda, const void* W, const void* bias, int bias_f32, void* out,
           int64_t ldo, int M, int N, int K, int epilogue, cudaStream_t stream) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
#define KVAD_LAUNCH_EPI(E)                                                                              \
  linear_simt_kernel<T, E><<<grid, THREADS, 0, stream>>>((const T*)A, lda, (const T*)W, bias, bias_f32, \
                                                         out, ldo, M, N, K)
  switch (epilogue) {
    case EPI_STORE: KVAD_LAUNCH_EPI(EPI_STORE); break;
    case EPI_GELU_TANH: KVAD_LAUNCH_EPI(EPI_GELU_TANH); break;
    case EPI_GELU_ERF: KVAD_LAUNCH_EPI(EPI_GELU_ERF); break;
    case EPI_RESIDUAL: KVAD_LAUNCH_EPI(EPI_RESIDUAL); break;
    case EPI_STORE_F32: KVAD_LAUNCH_EPI(EPI_STORE_F32); break;
    default: KVAD_FAIL(KVAD_ERR_ARGUMENT, "linear_simt: unknown epilogue %d", epilogue);
  }
#undef KVAD_LAUNCH_EPI
  KVAD_CHECK_LAUNCH("linear_simt");
  return KVAD_OK;
}

}  // namespace

KVAD_EXPORT int kvad_linear_simt(int dtype, const void* A, int64_t lda, const void* W, const void* bias,
                                 int bias_f32, void* out, int64_t ldo, int M, int N, int K,
                                 int epilogue, cudaStream_t stream) {
  KVAD_REQUIRE(M >= 0 && N > 0 && K > 0, "linear_simt: bad sizes M=%d N=%d K=%d", M, N, K);
  KVAD_REQUIRE(lda >= K && ldo >= N, "linear_simt: leading dimensions lda=%lld ldo=%lld too small for K=%d N=%d", (long long)lda, (long long)ldo, K, N);
  KVAD_REQUIRE((M + BM - 1) / BM <= 65535, "linear_simt: M=%d is more rows than one launch takes", M);
  if (M == 0) return KVAD_OK;
  if (dtype == KVAD_DTYPE_F32) return launch<float>(A, lda, W, bias, bias_f32, out, ldo, M, N, K, epilogue, stream);
  if (dtype == KVAD_DTYPE_BF16) return launch<__nv_bfloat16>(A, lda, W, bias, bias_f32, out, ldo, M, N, K, epilogue, stream);
  KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "linear_simt: unknown dtype %d", dtype);
}

KVAD_DEFINE_LAST_ERROR()
