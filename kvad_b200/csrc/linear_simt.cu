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

constexpr int BK = 16;
constexpr int THREADS = 256;

// Four consecutive elements of a row, k..k+3, as floats; one 16- or 8-byte load where the row allows it.
template <typename T>
__device__ __forceinline__ void load4(const T* __restrict__ row, int k, int K, bool vec_ok, float (&f)[4]) {
  if (vec_ok && k + 3 < K) {
    if (sizeof(T) == 4) {
      const float4 v = *reinterpret_cast<const float4*>(row + k);
      f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
    } else {
      const uint2 v = *reinterpret_cast<const uint2*>(row + k);
      const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
      const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
      f[0] = lo.x; f[1] = lo.y; f[2] = hi.x; f[3] = hi.y;
    }
  } else {
#pragma unroll
    for (int e = 0; e < 4; ++e) f[e] = (k + e < K) ? to_f32(row[k + e]) : 0.f;
  }
}

// A tile of B x B outputs per CTA, T x T of them per thread (B / T = 16 threads a side): 64 x 64 with 4 x 4 for
// few rows, 128 x 128 with 8 x 8 (twice the arithmetic per shared-memory read) for many.
template <typename T, int EPI, int B, int TT>
__global__ void __launch_bounds__(THREADS)
linear_simt_kernel(const T* __restrict__ A, int64_t lda, const T* __restrict__ W,
                   const void* __restrict__ bias, int bias_f32, void* __restrict__ out,
                   int64_t ldo, int M, int N, int K, int vec_a, int vec_w) {
  static_assert(B / TT == 16, "16 threads a side");
  __shared__ float As[BK][B + 4];
  __shared__ float Ws[BK][B + 4];
  pdl_launch_dependents();
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  const int m0 = blockIdx.y * B, n0 = blockIdx.x * B;

  float acc[TT][TT];
#pragma unroll
  for (int i = 0; i < TT; ++i)
#pragma unroll
    for (int j = 0; j < TT; ++j) acc[i][j] = 0.f;

  // per K tile a thread stages B * BK / THREADS elements of A and as many of W, four consecutive k at a time
  constexpr int QUADS = B * BK / 4 / THREADS;        // 1 (B = 64) or 2 (B = 128)
  pdl_wait();
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int q = 0; q < QUADS; ++q) {
      const int id = threadIdx.x + q * THREADS;
      const int lr = id / 4, lk = (id % 4) * 4;       // row of the tile, first k of four
      const int m = m0 + lr, n = n0 + lr;
      float fa[4] = {0.f, 0.f, 0.f, 0.f}, fw[4] = {0.f, 0.f, 0.f, 0.f};
      if (m < M) load4(A + (int64_t)m * lda, k0 + lk, K, vec_a != 0, fa);
      if (n < N) load4(W + (int64_t)n * K, k0 + lk, K, vec_w != 0, fw);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        As[lk + e][lr] = fa[e];
        Ws[lk + e][lr] = fw[e];
      }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[TT], b[TT];
#pragma unroll
      for (int i = 0; i < TT; ++i) a[i] = As[k][ty * TT + i];
#pragma unroll
      for (int j = 0; j < TT; ++j) b[j] = Ws[k][tx * TT + j];
#pragma unroll
      for (int i = 0; i < TT; ++i)
#pragma unroll
        for (int j = 0; j < TT; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < TT; ++i) {
    const int m = m0 + ty * TT + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TT; ++j) {
      const int n = n0 + tx * TT + j;
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

template <typename T, int B, int TT>
int launch_tile(const void* A, int64_t lda, const void* W, const void* bias, int bias_f32, void* out,
                int64_t ldo, int M, int N, int K, int epilogue, cudaStream_t stream) {
  dim3 grid((N + B - 1) / B, (M + B - 1) / B);
  // rows can be read four elements at a time where every row starts on a boundary of four elements' bytes
  const int bytes4 = 4 * (int)sizeof(T);
  const int vec_a = (reinterpret_cast<uintptr_t>(A) % bytes4 == 0 && lda % 4 == 0) ? 1 : 0;
  const int vec_w = (reinterpret_cast<uintptr_t>(W) % bytes4 == 0 && K % 4 == 0) ? 1 : 0;
#define KVAD_LAUNCH_EPI(E)                                                                                        \
  kvad_launch(linear_simt_kernel<T, E, B, TT>, grid, dim3(THREADS), 0, stream, (const T*)A, lda, (const T*)W, bias, \
              bias_f32, out, ldo, M, N, K, vec_a, vec_w)
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

template <typename T>
int launch(const void* A, int64_t lda, const void* W, const void* bias, int bias_f32, void* out,
           int64_t ldo, int M, int N, int K, int epilogue, cudaStream_t stream) {
  // the large tile where it fills the GPU; an output element's sum runs over k in order in both, so its bits do not depend on the choice
  if (M > 64 && (int64_t)((M + 127) / 128) * ((N + 127) / 128) >= 120)
    return launch_tile<T, 128, 8>(A, lda, W, bias, bias_f32, out, ldo, M, N, K, epilogue, stream);
  return launch_tile<T, 64, 4>(A, lda, W, bias, bias_f32, out, ldo, M, N, K, epilogue, stream);
}

}  // namespace

KVAD_EXPORT int kvad_linear_simt(int dtype, const void* A, int64_t lda, const void* W, const void* bias,
                                 int bias_f32, void* out, int64_t ldo, int M, int N, int K,
                                 int epilogue, cudaStream_t stream) {
  KVAD_REQUIRE(M >= 0 && N > 0 && K > 0, "linear_simt: bad sizes M=%d N=%d K=%d", M, N, K);
  KVAD_REQUIRE(lda >= K && ldo >= N, "linear_simt: leading dimensions lda=%lld ldo=%lld too small for K=%d N=%d", (long long)lda, (long long)ldo, K, N);
  KVAD_REQUIRE((M + 63) / 64 <= 65535, "linear_simt: M=%d is more rows than one launch takes", M);
  if (M == 0) return KVAD_OK;
  if (dtype == KVAD_DTYPE_F32) return launch<float>(A, lda, W, bias, bias_f32, out, ldo, M, N, K, epilogue, stream);
  if (dtype == KVAD_DTYPE_BF16) return launch<__nv_bfloat16>(A, lda, W, bias, bias_f32, out, ldo, M, N, K, epilogue, stream);
  KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "linear_simt: unknown dtype %d", dtype);
}

KVAD_DEFINE_LAST_ERROR()
