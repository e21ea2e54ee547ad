// Causal attention of a step's rows over the paged cache, on the CUDA cores in
// 32-bit arithmetic, for any head size and any grouping of heads.  Row r of
// sequence row_seq[r] at position row_pos[r] attends over that sequence's keys
// at positions max(0, pos-window+1) .. pos (window <= 0: all of them).  A block
// serves one (row, head); it walks the keys in tiles with a running maximum and
// sum, so the order of operations for a row depends on nothing but its own
// keys.  This is the attention of the float32 engine for prompts and decoding
// alike, and the bfloat16 engine's fallback for head sizes its tensor-core
// kernels refuse.
//
// bisand/kvad: attend(), crates/llm/src/model/mod.rs:769-819 - score =
// dot(q,k) * (1/sqrt(head_dim)), softmax with the maximum subtracted
// (crates/llm/src/tensor.rs:297-308), output = sum of weights times values;
// head h reads KV head h / (n_heads / n_kv_heads).
#include "common.cuh"

using namespace kvad;

namespace {

constexpr int ATT_THREADS = 128;
constexpr int MAX_DIMS_PER_THREAD = 4;   // head sizes up to 512

template <typename T>
__global__ void __launch_bounds__(ATT_THREADS)
attention_rows_kernel(const T* __restrict__ q, int64_t ld_q, T* __restrict__ out, int64_t ld_out,
                      const int* __restrict__ row_seq, const int* __restrict__ row_pos,
                      const int* __restrict__ page_table, int table_width,
                      const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                      int n_heads, int n_kv_heads, int head_dim, int page_size, float scale, int window) {
  extern __shared__ float smem[];
  float* qs = smem;                     // [head_dim]
  float* ps = smem + head_dim;          // [ATT_THREADS]
  __shared__ float scratch[33];

  const int r = blockIdx.x, h = blockIdx.y;
  const int kvh = h / (n_heads / n_kv_heads);
  const int pos = row_pos[r];
  const int* pages = page_table + (int64_t)row_seq[r] * table_width;
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;

  for (int d = threadIdx.x; d < head_dim; d += ATT_THREADS) qs[d] = to_f32(q[(int64_t)r * ld_q + (int64_t)h * head_dim + d]);
  __syncthreads();

  float acc[MAX_DIMS_PER_THREAD];
#pragma unroll
  for (int i = 0; i < MAX_DIMS_PER_THREAD; ++i) acc[i] = 0.f;
  float run_max = -INFINITY, run_sum = 0.f;

  for (int t0 = lo; t0 <= pos; t0 += ATT_THREADS) {
    const int t = t0 + threadIdx.x;
    float s = -INFINITY;
    if (t <= pos) {
      const int page = pages[t / page_size];
      const T* kr = k_pages + (((int64_t)page * n_kv_heads + kvh) * page_size + t % page_size) * head_dim;
      float dot = 0.f;
      for (int d = 0; d < head_dim; ++d) dot = fmaf(qs[d], to_f32(kr[d]), dot);
      s = dot * scale;
    }
    const float tile_max = block_max(s, scratch);
    const float new_max = fmaxf(run_max, tile_max);
    const float keep = (run_max == -INFINITY) ? 0.f : expf(run_max - new_max);
    const float p = (t <= pos) ? expf(s - new_max) : 0.f;
    ps[threadIdx.x] = p;
    const float tile_sum = block_sum(p, scratch);   // also orders the writes of ps before the reads below
    run_sum = run_sum * keep + tile_sum;
    run_max = new_max;

    const int n_here = (pos - t0 + 1) < ATT_THREADS ? (pos - t0 + 1) : ATT_THREADS;
#pragma unroll
    for (int i = 0; i < MAX_DIMS_PER_THREAD; ++i) {
      const int d = threadIdx.x + i * ATT_THREADS;
      if (d < head_dim) {
        float a = acc[i] * keep;
        for (int j = 0; j < n_here; ++j) {
          const int tj = t0 + j;
          const int page = pages[tj / page_size];
          const T* vr = v_pages + (((int64_t)page * n_kv_heads + kvh) * page_size + tj % page_size) * head_dim;
          a = fmaf(ps[j], to_f32(vr[d]), a);
        }
        acc[i] = a;
      }
    }
    __syncthreads();   // ps is rewritten by the next tile
  }

  const float inv = 1.0f / run_sum;
#pragma unroll
  for (int i = 0; i < MAX_DIMS_PER_THREAD; ++i) {
    const int d = threadIdx.x + i * ATT_THREADS;
    if (d < head_dim) out[(int64_t)r * ld_out + (int64_t)h * head_dim + d] = from_f32<T>(acc[i] * inv);
  }
}

}  // namespace

KVAD_EXPORT int kvad_attention_simt(int dtype, const void* q, int64_t ld_q, void* out, int64_t ld_out,
                                    const int* row_seq, const int* row_pos, const int* page_table,
                                    int table_width, const void* k_pages, const void* v_pages, int n_rows,
                                    int n_heads, int n_kv_heads, int head_dim, int page_size, float scale,
                                    int window, cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && n_heads > 0 && n_kv_heads > 0 && head_dim > 0 && page_size > 0 && table_width > 0,
               "attention: bad sizes rows=%d heads=%d kv_heads=%d head_dim=%d page=%d", n_rows, n_heads, n_kv_heads, head_dim, page_size);
  KVAD_REQUIRE(n_heads % n_kv_heads == 0, "attention: %d heads do not divide into %d key/value heads", n_heads, n_kv_heads);
  KVAD_REQUIRE(head_dim <= ATT_THREADS * MAX_DIMS_PER_THREAD, "attention: head size %d is above this kernel's limit of %d", head_dim, ATT_THREADS * MAX_DIMS_PER_THREAD);
  KVAD_REQUIRE(n_heads <= 65535, "attention: %d heads are more than one launch takes", n_heads);
  if (n_rows == 0) return KVAD_OK;
  dim3 grid(n_rows, n_heads);
  const size_t smem = (size_t)(head_dim + ATT_THREADS) * sizeof(float);
  if (dtype == KVAD_DTYPE_F32)
    attention_rows_kernel<float><<<grid, ATT_THREADS, smem, stream>>>((const float*)q, ld_q, (float*)out, ld_out, row_seq, row_pos, page_table, table_width, (const float*)k_pages, (const float*)v_pages, n_heads, n_kv_heads, head_dim, page_size, scale, window);
  else if (dtype == KVAD_DTYPE_BF16)
    attention_rows_kernel<__nv_bfloat16><<<grid, ATT_THREADS, smem, stream>>>((const __nv_bfloat16*)q, ld_q, (__nv_bfloat16*)out, ld_out, row_seq, row_pos, page_table, table_width, (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, n_heads, n_kv_heads, head_dim, page_size, scale, window);
  else
    KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "attention: unknown dtype %d", dtype);
  KVAD_CHECK_LAUNCH("attention_simt");
  return KVAD_OK;
}

KVAD_DEFINE_LAST_ERROR()
