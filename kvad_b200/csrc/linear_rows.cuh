// out[M,N] = epilogue(A[M,K] . W[N,K]^T + bias) for at most 16 rows (decoding at small batch), bfloat16
// or true 32-bit, as a stream of weights over every SM.
//
// With so few rows the product is a read of W and nothing else: 2 M flops per weight.  What
// decides its time is not arithmetic but the length of the dependent chain after the previous
// kernel ends, and how many SMs pull on memory.  So: a warp owns output columns (rows of W), and all
// of a column's weights - K/256 16-byte loads per lane - are requested into registers BEFORE the
// dependent-launch wait (weights are parameters, not the previous kernel's work).  After the wait
// the block brings the few activation rows into shared memory (one trip to L2), each lane
// multiplies its weights with them in 32-bit, the warp adds up by shuffles, and the first lanes
// apply the epilogue and store.  No tensor memory, no barriers, no descriptors: the chain is two
// memory round trips long.  In bfloat16 the tensor-core kernel (linear_tcgen05.cu) takes over above a
// few rows; in 32-bit this is the decode road of the float32 engine up to 16 rows (the tiled kernel
// of linear_simt.cu would run one row in a 64-row tile), every product an fmaf into a 32-bit sum.
//
// Two columns a warp on their way at a time (twice the registers for weights) were tried and lost: fewer
// warps fit an SM, and the warps in flight are what keeps memory busy (GPT-2 XL sizes, one row, an
// 8-layer model: 2 776 against 3 220 tokens a second; 32-bit GPT-2 small: 2 900 against 3 300).
//
// This header holds the kernel; linear_rows.cu builds it for bfloat16 and linear_rows_f32.cu for float32 - two
// libraries, compiled side by side, of which a model loads the one of its compute dtype.
//
// Sums are 32-bit; the order of additions for an output depends on K only, so a row's bits do not
// depend on its company.  (It is another order than the tiled kernel's: the two agree to rounding.)
#pragma once
#include "common.cuh"

using namespace kvad;

namespace {

#ifndef KVAD_ROWS_TARGET_CTAS
#define KVAD_ROWS_TARGET_CTAS 592      // CTAs a launch aims at, four an SM; one row, tokens a second at GPT-2 XL's sizes (8 layers) /
                                       // GPT-2 small: 148 -> 2650 / 3447, 296 -> 3119 / 3744, 592 -> 3222 / 3943, 1184 -> 3115 / 3948
#endif
constexpr int ROWS_THREADS = 256;
constexpr int ROWS_WARPS = ROWS_THREADS / 32;

__device__ __forceinline__ float gelu_tanh_hw(float t) {      // see linear_tcgen05.cu: the result is rounded to bfloat16
  float th;
  asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(0.79788456f * (t + 0.044715f * t * t * t)));
  return 0.5f * t * (1.0f + th);
}

template <typename T> struct Piece;            // a 16-byte piece of a row: VE elements
template <> struct Piece<__nv_bfloat16> {
  static constexpr int VE = 8;
  static __device__ __forceinline__ void unpack(const uint4& q, float* f) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float2 v = __bfloat1622float2(h[t]);
      f[2 * t] = v.x;
      f[2 * t + 1] = v.y;
    }
  }
};
template <> struct Piece<float> {
  static constexpr int VE = 4;
  static __device__ __forceinline__ void unpack(const uint4& q, float* f) {
    f[0] = __uint_as_float(q.x); f[1] = __uint_as_float(q.y); f[2] = __uint_as_float(q.z); f[3] = __uint_as_float(q.w);
  }
};

// MR: activation rows handled (M <= MR); NI: 16-byte pieces of a weight row per lane (K <= NI * 32 * VE).
template <typename T, int MR, int NI, int EPI>
__global__ void __launch_bounds__(ROWS_THREADS)
linear_rows_kernel(const T* __restrict__ A, int64_t lda, const T* __restrict__ W,
                   const void* __restrict__ bias, int bias_f32, void* __restrict__ out, int64_t ldo,
                   int M, int N, int K, int cols_per_warp) {
  constexpr int VE = Piece<T>::VE;
  extern __shared__ __align__(16) unsigned char rows_smem[];
  T* As = reinterpret_cast<T*>(rows_smem);      // [MR][K]
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col0 = (blockIdx.x * ROWS_WARPS + warp) * cols_per_warp;

  // the first column's weights, before the wait
  uint4 w[NI];
  auto fetch = [&](int n) {
#pragma unroll
    for (int i = 0; i < NI; ++i) {
      const int k0 = (lane + 32 * i) * VE;
      w[i] = (n < N && k0 < K) ? *reinterpret_cast<const uint4*>(W + (int64_t)n * K + k0) : make_uint4(0u, 0u, 0u, 0u);
    }
  };
  fetch(col0);
  float b0 = (bias != nullptr && col0 < N) ? load_param(bias, col0, bias_f32) : 0.f;

  pdl_wait();
  // the activation rows -> shared memory (rows past M are zero)
  const int pieces = K / VE;
  for (int i = threadIdx.x; i < MR * pieces; i += ROWS_THREADS) {
    const int m = i / pieces, p = i % pieces;
    const uint4 v = m < M ? *reinterpret_cast<const uint4*>(A + (int64_t)m * lda + p * VE) : make_uint4(0u, 0u, 0u, 0u);
    *reinterpret_cast<uint4*>(As + (int64_t)m * K + p * VE) = v;
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
      const int k0 = (lane + 32 * i) * VE;
      if (k0 < K) {
        float wf[VE];
        Piece<T>::unpack(w[i], wf);
#pragma unroll
        for (int m = 0; m < MR; ++m) {
          const uint4 av = *reinterpret_cast<const uint4*>(As + (int64_t)m * K + k0);
          float af[VE];
          Piece<T>::unpack(av, af);
          float s = acc[m];
#pragma unroll
          for (int t = 0; t < VE; ++t) s = fmaf(wf[t], af[t], s);
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
      if (EPI == EPI_GELU_TANH) t = sizeof(T) == 2 ? gelu_tanh_hw(t) : gelu_tanh(t);      // the fast form only where the result is rounded to bfloat16
      if (EPI == EPI_GELU_ERF) t = gelu_erf(t);
      const int64_t o = (int64_t)lane * ldo + n;
      if (EPI == EPI_STORE || EPI == EPI_GELU_TANH || EPI == EPI_GELU_ERF) reinterpret_cast<T*>(out)[o] = from_f32<T>(t);
      else if (EPI == EPI_RESIDUAL) reinterpret_cast<float*>(out)[o] += t;
      else reinterpret_cast<float*>(out)[o] = t;
    }
  }
}

template <typename T, int MR, int NI>
int launch_epi(int epilogue, const void* A, int64_t lda, const void* W, const void* bias, int bias_f32, void* out,
               int64_t ldo, int M, int N, int K, cudaStream_t stream) {
  // columns per warp: enough CTAs to fill every SM with four, not more
  int cpw = (N + ROWS_WARPS * KVAD_ROWS_TARGET_CTAS - 1) / (ROWS_WARPS * KVAD_ROWS_TARGET_CTAS);
  if (cpw < 1) cpw = 1;
  const int grid = (N + ROWS_WARPS * cpw - 1) / (ROWS_WARPS * cpw);
  const size_t smem = (size_t)MR * K * sizeof(T);
  if (smem > 200 * 1024)
    KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "linear_rows: %d rows of %d columns do not fit shared memory", MR, K);
#define KVAD_ROWS(E)                                                                                                \
  {                                                                                                                 \
    static size_t configured = 0;                                                                                   \
    if (smem > 48 * 1024 && smem > configured) {                                                                    \
      cudaError_t e = cudaFuncSetAttribute(linear_rows_kernel<T, MR, NI, E>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e != cudaSuccess) KVAD_FAIL(KVAD_ERR_CUDA, "linear_rows: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e)); \
      configured = smem;                                                                                            \
    }                                                                                                               \
    kvad_launch(linear_rows_kernel<T, MR, NI, E>, dim3(grid), dim3(ROWS_THREADS), smem, stream, (const T*)A,        \
                lda, (const T*)W, bias, bias_f32, out, ldo, M, N, K, cpw);                                          \
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

template <typename T, int MR>
int launch_ni(int epilogue, const void* A, int64_t lda, const void* W, const void* bias, int bias_f32, void* out,
              int64_t ldo, int M, int N, int K, cudaStream_t stream) {
  constexpr int PER = 32 * Piece<T>::VE;          // columns of K one piece per lane covers
  if (K <= 4 * PER) return launch_epi<T, MR, 4>(epilogue, A, lda, W, bias, bias_f32, out, ldo, M, N, K, stream);
  if (K <= 8 * PER) return launch_epi<T, MR, 8>(epilogue, A, lda, W, bias, bias_f32, out, ldo, M, N, K, stream);
  if (K <= 16 * PER) return launch_epi<T, MR, 16>(epilogue, A, lda, W, bias, bias_f32, out, ldo, M, N, K, stream);
  return launch_epi<T, MR, 32>(epilogue, A, lda, W, bias, bias_f32, out, ldo, M, N, K, stream);
}

template <typename T>
int launch_rows(int epilogue, const void* A, int64_t lda, const void* W, const void* bias, int bias_f32, void* out,
                int64_t ldo, int M, int N, int K, cudaStream_t stream) {
  if (M <= 1) return launch_ni<T, 1>(epilogue, A, lda, W, bias, bias_f32, out, ldo, M, N, K, stream);
  if (M <= 2) return launch_ni<T, 2>(epilogue, A, lda, W, bias, bias_f32, out, ldo, M, N, K, stream);
  if (M <= 4) return launch_ni<T, 4>(epilogue, A, lda, W, bias, bias_f32, out, ldo, M, N, K, stream);
  if (M <= 8) return launch_ni<T, 8>(epilogue, A, lda, W, bias, bias_f32, out, ldo, M, N, K, stream);
  return launch_ni<T, 16>(epilogue, A, lda, W, bias, bias_f32, out, ldo, M, N, K, stream);
}

}  // namespace

// The entry point of a library that holds the kernel for ONE element type.  Refuses (KVAD_ERR_UNSUPPORTED) the other
// dtype, more than 16 rows, K beyond 1024 16-byte pieces (8192 in bfloat16, 4096 in float32: 32 pieces a lane) or not
// a multiple of a piece, or operands that are not 16-byte aligned; the caller then takes another kernel.
#define KVAD_LINEAR_ROWS_LIBRARY(T, CODE)                                                                                          \
  KVAD_EXPORT int kvad_linear_rows(int dtype, const void* A, int64_t lda, const void* W, const void* bias, int bias_f32, void* out, \
                                   int64_t ldo, int M, int N, int K, int epilogue, cudaStream_t stream) {                          \
    KVAD_REQUIRE(M >= 0 && N > 0 && K > 0, "linear_rows: bad sizes M=%d N=%d K=%d", M, N, K);                                       \
    if (dtype != (CODE)) KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "linear_rows: this library holds dtype %d, not %d", (int)(CODE), dtype);    \
    const int ve = 16 / (int)sizeof(T);                                                                                             \
    if (M > 16 || K > 1024 * ve || K % ve != 0 || lda % ve != 0 || (reinterpret_cast<uintptr_t>(A) & 15) ||                         \
        (reinterpret_cast<uintptr_t>(W) & 15))                                                                                      \
      KVAD_FAIL(KVAD_ERR_UNSUPPORTED,                                                                                               \
                "linear_rows: takes at most 16 rows, K a multiple of %d up to %d and 16-byte aligned operands (M=%d K=%d)", ve,      \
                1024 * ve, M, K);                                                                                                   \
    KVAD_REQUIRE(lda >= K && ldo >= N, "linear_rows: leading dimensions lda=%lld ldo=%lld too small", (long long)lda,               \
                 (long long)ldo);                                                                                                   \
    if (M == 0) return KVAD_OK;                                                                                                     \
    return launch_rows<T>(epilogue, A, lda, W, bias, bias_f32, out, ldo, M, N, K, stream);                                          \
  }                                                                                                                                 \
  KVAD_DEFINE_LAST_ERROR()
