// out[M,N] = epilogue(A[M,K] . W[N,K]^T + bias) for at most 16 rows of bfloat16 (decoding at small
// batch), as a stream of weights over every SM.
//
// With so few rows the product is a read of W and nothing else: 2 M flops per weight.  What
// decides its time is not arithmetic but the length of the dependent chain after the previous
// kernel ends, and how many SMs pull on memory.  So: a warp owns output columns (rows of W), and all
// of a column's weights - K/256 16-byte loads per lane - are requested into registers BEFORE the
// dependent-launch wait (weights are parameters, not the previous kernel's work).  After the wait
// the block brings the few activation rows into shared memory (one trip to L2), each lane
// multiplies its weights with them in 32-bit, the warp adds up by shuffles, and the first lanes
// apply the epilogue and store.  No tensor memory, no barriers, no descriptors: the chain is two
// memory round trips long.  The tensor-core kernel (linear_tcgen05.cu) takes over above 16 rows.
//
// Sums are 32-bit; the order of additions for an output depends on K only.
#include "common.cuh"

using namespace kvad;

namespace {

constexpr int ROWS_THREADS = 256;
constexpr int ROWS_WARPS = ROWS_THREADS / 32;

__device__ __forceinline__ float gelu_tanh_hw(float t) {      // see linear_tcgen05.cu: the result is rounded to bfloat16
  float th;
  asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(0.79788456f * (t + 0.044715f * t * t * t)));
  return 0.5f * t * (1.0f + th);
}

// MR: activation rows handled (M <= MR); NI: 16-byte pieces of a weight row per lane (K <= NI * 256).
template <int MR, int NI, int EPI>
__global__ void __launch_bounds__(ROWS_THREADS)
linear_rows_kernel(const __nv_bfloat16* __restrict__ A, int64_t lda, const __nv_bfloat16* __restrict__ W,
                   const void* __restrict__ bias, int bias_f32, void* __restrict__ out, int64_t ldo,
                   int M, int N, int K, int cols_per_warp) {
  extern __shared__ __align__(16) unsigned char rows_smem[];
  __nv_bfloat16* As = reinterpret_cast<__nv_bfloat16*>(rows_smem);      // [MR][K]
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col0 = (blockIdx.x * ROWS_WARPS + warp) * cols_per_warp;

  // the first column's weights, before the wait
  uint4 w[NI];
  auto fetch = [&](int n) {
#pragma unroll
    for (int i = 0; i < NI; ++i) {
      const int k0 = (lane + 32 * i) * 8;
      w[i] = (n < N && k0 < K) ? *reinterpret_cast<const uint4*>(W + (int64_t)n * K + k0) : make_uint4(0u, 0u, 0u, 0u);
    }
  };
  fetch(col0);
  float b0 = (bias != nullptr && col0 < N) ? load_param(bias, col0, bias_f32) : 0.f;

  pdl_wait();
  // the activation rows -> shared memory (rows past M are zero)
  const int pieces = K / 8;
  for (int i = threadIdx.x; i < MR * pieces; i += ROWS_THREADS) {
    const int m = i / pieces, p = i % pieces;
    const uint4 v = m < M ? *reinterpret_cast<const uint4*>(A + (int64_t)m * lda + p * 8) : make_uint4(0u, 0u, 0u, 0u);
    *reinterpret_cast<uint4*>(As + (int64_t)m * K + p * 8) = v;
  }
  __syncthreads();

  for (int c = 0; c < cols_per_warp; ++c) {
    const int n = col0 + c;
    if (n >= N) break;
    float acc[MR];
#pragma unroll
    for (int m = 0; m < MR; ++m) acc[m] = 0.f;
#pragma unroll
    for (int i = 0; i < NI; ++i) {
      const int k0 = (lane + 32 * i) * 8;
      if (k0 < K) {
        const __nv_bfloat162* wh = reinterpret_cast<const __nv_bfloat162*>(&w[i]);
        float wf[8];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const float2 f = __bfloat1622float2(wh[t]);
          wf[2 * t] = f.x;
          wf[2 * t + 1] = f.y;
        }
#pragma unroll
        for (int m = 0; m < MR; ++m) {
          const uint4 av = *reinterpret_cast<const uint4*>(As + (int64_t)m * K + k0);
          const __nv_bfloat162* ah = reinterpret_cast<const __nv_bfloat162*>(&av);
          float s = acc[m];
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const float2 f = __bfloat1622float2(ah[t]);
            s = fmaf(wf[2 * t], f.x, s);
            s = fmaf(wf[2 * t + 1], f.y, s);
          }
          acc[m] = s;
        }
      }
    }
    const float b = b0;
    if (c + 1 < cols_per_warp) {             // the next column's weights are on their way during the reduction
      fetch(n + 1);
      b0 = (bias != nullptr && n + 1 < N) ? load_param(bias, n + 1, bias_f32) : 0.f;
    }
#pragma unroll
    for (int m = 0; m < MR; ++m) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], o);
    }
    // lane m stores row m
    float mine = 0.f;
#pragma unroll
    for (int m = 0; m < MR; ++m)
      if (lane == m) mine = acc[m];
    if (lane < M) {
      float t = mine + b;
      if (EPI == EPI_GELU_TANH) t = gelu_tanh_hw(t);
      if (EPI == EPI_GELU_ERF) t = gelu_erf(t);
      const int64_t o = (int64_t)lane * ldo + n;
      if (EPI == EPI_STORE || EPI == EPI_GELU_TANH || EPI == EPI_GELU_ERF) reinterpret_cast<__nv_bfloat16*>(out)[o] = __float2bfloat16_rn(t);
      else if (EPI == EPI_RESIDUAL) reinterpret_cast<float*>(out)[o] += t;
      else reinterpret_cast<float*>(out)[o] = t;
    }
  }
}

template <int MR, int NI>
int launch_epi(int epilogue, const void* A, int64_t lda, const void* W, const void* bias, int bias_f32, void* out,
               int64_t ldo, int M, int N, int K, cudaStream_t stream) {
  // columns per warp: enough CTAs to cover the SMs twice, not more
  int cpw = (N + ROWS_WARPS * 296 - 1) / (ROWS_WARPS * 296);
  if (cpw < 1) cpw = 1;
  const int grid = (N + ROWS_WARPS * cpw - 1) / (ROWS_WARPS * cpw);
  const size_t smem = (size_t)MR * K * 2;
#define KVAD_ROWS(E)                                                                                                \
  {                                                                                                                 \
    static size_t configured = 0;                                                                                   \
    if (smem > 48 * 1024 && smem > configured) {                                                                    \
      cudaError_t e = cudaFuncSetAttribute(linear_rows_kernel<MR, NI, E>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e != cudaSuccess) KVAD_FAIL(KVAD_ERR_CUDA, "linear_rows: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e)); \
      configured = smem;                                                                                            \
    }                                                                                                               \
    kvad_launch(linear_rows_kernel<MR, NI, E>, dim3(grid), dim3(ROWS_THREADS), smem, stream, (const __nv_bfloat16*)A, \
                lda, (const __nv_bfloat16*)W, bias, bias_f32, out, ldo, M, N, K, cpw);                              \
  }
  switch (epilogue) {
    case EPI_STORE: KVAD_ROWS(EPI_STORE) break;
    case EPI_GELU_TANH: KVAD_ROWS(EPI_GELU_TANH) break;
    case EPI_GELU_ERF: KVAD_ROWS(EPI_GELU_ERF) break;
    case EPI_RESIDUAL: KVAD_ROWS(EPI_RESIDUAL) break;
    case EPI_STORE_F32: KVAD_ROWS(EPI_STORE_F32) break;
    default: KVAD_FAIL(KVAD_ERR_ARGUMENT, "linear_rows: unknown epilogue %d", epilogue);
  }
#undef KVAD_ROWS
  KVAD_CHECK_LAUNCH("linear_rows");
  return KVAD_OK;
}

template <int MR>
int launch_ni(int epilogue, const void* A, int64_t lda, const void* W, const void* bias, int bias_f32, void* out,
              int64_t ldo, int M, int N, int K, cudaStream_t stream) {
  if (K <= 1024) return launch_epi<MR, 4>(epilogue, A, lda, W, bias, bias_f32, out, ldo, M, N, K, stream);
  if (K <= 2048) return launch_epi<MR, 8>(epilogue, A, lda, W, bias, bias_f32, out, ldo, M, N, K, stream);
  return launch_epi<MR, 16>(epilogue, A, lda, W, bias, bias_f32, out, ldo, M, N, K, stream);
}

}  // namespace

// Refuses (KVAD_ERR_UNSUPPORTED) more than 16 rows, K beyond 4096 or not a multiple of 8, or
// operands that are not 16-byte aligned; the caller then takes the tensor-core kernel.
KVAD_EXPORT int kvad_linear_rows(const void* A, int64_t lda, const void* W, const void* bias, int bias_f32, void* out,
                                 int64_t ldo, int M, int N, int K, int epilogue, cudaStream_t stream) {
  KVAD_REQUIRE(M >= 0 && N > 0 && K > 0, "linear_rows: bad sizes M=%d N=%d K=%d", M, N, K);
  if (M > 16 || K > 4096 || K % 8 != 0 || lda % 8 != 0 || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(W) & 15))
    KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "linear_rows: takes at most 16 rows, K a multiple of 8 up to 4096 and 16-byte aligned operands (M=%d K=%d)", M, K);
  KVAD_REQUIRE(lda >= K && ldo >= N, "linear_rows: leading dimensions lda=%lld ldo=%lld too small", (long long)lda, (long long)ldo);
  if (M == 0) return KVAD_OK;
  if (M <= 1) return launch_ni<1>(epilogue, A, lda, W, bias, bias_f32, out, ldo, M, N, K, stream);
  if (M <= 2) return launch_ni<2>(epilogue, A, lda, W, bias, bias_f32, out, ldo, M, N, K, stream);
  if (M <= 4) return launch_ni<4>(epilogue, A, lda, W, bias, bias_f32, out, ldo, M, N, K, stream);
  if (M <= 8) return launch_ni<8>(epilogue, A, lda, W, bias, bias_f32, out, ldo, M, N, K, stream);
  return launch_ni<16>(epilogue, A, lda, W, bias, bias_f32, out, ldo, M, N, K, stream);
}

KVAD_DEFINE_LAST_ERROR()
