// Shared by every kernel file of kvad_b200: element types, loads that widen to
// 32-bit, block reductions, and the error convention of the exported C entry
// points (0 on success; otherwise a negative code and a message that
// kvad_last_error() returns).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define KVAD_DTYPE_F32 0
#define KVAD_DTYPE_BF16 1

#define KVAD_OK 0
#define KVAD_ERR_ARGUMENT (-1)
#define KVAD_ERR_UNSUPPORTED (-2)
#define KVAD_ERR_CUDA (-3)

static thread_local char kvad_err_text[768];

#define KVAD_EXPORT extern "C" __attribute__((visibility("default")))

#define KVAD_FAIL(code, ...)                                      \
  do {                                                            \
    snprintf(kvad_err_text, sizeof(kvad_err_text), __VA_ARGS__);  \
    return (code);                                                \
  } while (0)

#define KVAD_REQUIRE(cond, ...)                                   \
  do {                                                            \
    if (!(cond)) KVAD_FAIL(KVAD_ERR_ARGUMENT, __VA_ARGS__);       \
  } while (0)

#define KVAD_CHECK_LAUNCH(what)                                                    \
  do {                                                                             \
    cudaError_t e__ = cudaGetLastError();                                          \
    if (e__ != cudaSuccess)                                                        \
      KVAD_FAIL(KVAD_ERR_CUDA, "%s: launch failed: %s", what, cudaGetErrorString(e__)); \
  } while (0)

// Programmatic dependent launch: with it on, a kernel is launched so that it may start while the
// kernel before it in the stream is still running; it does what does not depend on that kernel
// (set-up, fetching weights) and then waits (pdl_wait) before it touches anything the stream's
// earlier work produced.  Every kernel of this library writes global memory only after pdl_wait.
static int kvad_pdl_enabled = 0;

#define KVAD_DEFINE_LAST_ERROR()                                                  \
  KVAD_EXPORT const char* kvad_last_error() { return kvad_err_text; }             \
  KVAD_EXPORT void kvad_set_pdl(int on) { kvad_pdl_enabled = on ? 1 : 0; }

template <typename... KArgs, typename... Args>
static inline cudaError_t kvad_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                      cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = kvad_pdl_enabled ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same with the grid cut into thread-block clusters of `cluster` CTAs (at most 8 in all): the CTAs
// of a cluster run together on one GPC and can read one another's shared memory.
template <typename... KArgs, typename... Args>
static inline cudaError_t kvad_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                              cudaStream_t stream, dim3 cluster, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster.x;
  attr[0].val.clusterDim.y = cluster.y;
  attr[0].val.clusterDim.z = cluster.z;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = kvad_pdl_enabled ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

namespace kvad {

// Waits until everything earlier in the stream has completed and is visible (a no-op unless the
// kernel was launched as a programmatic dependent); lets the next kernel in the stream start.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// All threads of all CTAs of the cluster meet; what they wrote to shared memory before is visible after.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The two halves of that meeting, for a CTA that has something else to do in between (every thread of the
// cluster arrives once; those that need the others' arrival wait).
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// A float into the shared memory of CTA `rank` of this cluster, at the place `local` has in this CTA's.
__device__ __forceinline__ void st_cluster_f32(float* local, unsigned rank, float v) {
  unsigned addr = (unsigned)__cvta_generic_to_shared(local), remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}
// Four floats (16-byte aligned) into the shared memory of CTA `rank`, at the place `local` has in this CTA's.
__device__ __forceinline__ void st_cluster_f32x4(float* local, unsigned rank, float4 v) {
  unsigned addr = (unsigned)__cvta_generic_to_shared(local), remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(remote), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
// Arrives on the mbarrier that CTA `rank` of this cluster has at the place `local_bar` has here; what this
// thread (and, after a __syncwarp, its warp) wrote to that CTA's shared memory before is visible to whoever
// sees the arrival.
__device__ __forceinline__ void mbar_arrive_cluster(uint64_t* local_bar, unsigned rank) {
  unsigned addr = (unsigned)__cvta_generic_to_shared(local_bar), remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote) : "memory");
}
// One poll of an mbarrier of this CTA on which other CTAs of the cluster arrive.
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"((unsigned)__cvta_generic_to_shared(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// A float from the shared memory of CTA `rank` of this cluster, at the place `local` has in this CTA's.
__device__ __forceinline__ float ld_cluster_f32(const float* local, unsigned rank) {
  unsigned addr = (unsigned)__cvta_generic_to_shared(local), remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// A parameter vector (bias, gain) may be stored in 32-bit even when the
// activations are bfloat16: `is_f32` says which.
__device__ __forceinline__ float load_param(const void* p, int64_t i, int is_f32) {
  return is_f32 ? reinterpret_cast<const float*>(p)[i]
                : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.
// `scratch` holds 33 floats.  The order of additions depends only on the block
// size, so a row's result does not depend on what else is in the batch.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n_warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < n_warps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n_warps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < n_warps ? scratch[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// tanh-form GELU with bisand/kvad's constants (crates/llm/src/tensor.rs:263-269).
__device__ __forceinline__ float gelu_tanh(float t) {
  const float c = 0.79788456f;
  return 0.5f * t * (1.0f + tanhf(c * (t + 0.044715f * t * t * t)));
}
// exact GELU, x * Phi(x), through erf.
__device__ __forceinline__ float gelu_erf(float t) {
  return 0.5f * t * (1.0f + erff(t * 0.70710678118654752440f));
}

// Epilogues of the linear kernels.
enum Epilogue : int {
  EPI_STORE = 0,       // out[T]   = acc + bias
  EPI_GELU_TANH = 1,   // out[T]   = gelu_tanh(acc + bias)
  EPI_GELU_ERF = 2,    // out[T]   = gelu_erf(acc + bias)
  EPI_RESIDUAL = 3,    // out[f32] += acc + bias   (the residual stream)
  EPI_STORE_F32 = 4,   // out[f32] = acc + bias    (logits)
};

}  // namespace kvad
