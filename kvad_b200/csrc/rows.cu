// Row-wise kernels: token (+ position) embedding, LayerNorm, and writing a
// step's keys and values into the paged cache.  All arithmetic is 32-bit; the
// element type only says how tensors are stored.
#include "common.cuh"

using namespace kvad;

// ---------------------------------------------------------------------------
// x[r, :] = wte[token[r], :] + wpe[position[r], :]        (wpe may be absent)
// bisand/kvad: crates/llm/src/model/gpt2.rs:200-213.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void embed_kernel(const int* __restrict__ tokens, const int* __restrict__ positions,
                             const T* __restrict__ wte, const T* __restrict__ wpe,
                             float* __restrict__ x, int n_rows, int width, int vocab, int n_positions) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t total = (int64_t)n_rows * width;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / width), c = (int)(i % width);
    int tok = tokens[r];
    tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);   // ids are checked on the host; this only guards memory
    float v = to_f32(wte[(int64_t)tok * width + c]);
    if (wpe != nullptr) {
      int p = positions[r];
      p = p < 0 ? 0 : (p >= n_positions ? n_positions - 1 : p);
      v += to_f32(wpe[(int64_t)p * width + c]);
    }
    x[i] = v;
  }
}

KVAD_EXPORT int kvad_embed(int dtype, const int* tokens, const int* positions, const void* wte,
                           const void* wpe, float* x, int n_rows, int width, int vocab,
                           int n_positions, cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && width > 0 && vocab > 0, "embed: bad sizes rows=%d width=%d vocab=%d", n_rows, width, vocab);
  KVAD_REQUIRE(wpe == nullptr || n_positions > 0, "embed: a position table needs n_positions > 0");
  if (n_rows == 0) return KVAD_OK;
  const int64_t total = (int64_t)n_rows * width;
  const int threads = 256;
  const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
  if (dtype == KVAD_DTYPE_F32)
    kvad_launch(embed_kernel<float>, dim3(blocks), dim3(threads), 0, stream, tokens, positions, (const float*)wte, (const float*)wpe, x, n_rows, width, vocab, n_positions);
  else if (dtype == KVAD_DTYPE_BF16)
    kvad_launch(embed_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, tokens, positions, (const __nv_bfloat16*)wte, (const __nv_bfloat16*)wpe, x, n_rows, width, vocab, n_positions);
  else
    KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "embed: unknown dtype %d", dtype);
  KVAD_CHECK_LAUNCH("embed");
  return KVAD_OK;
}

// ---------------------------------------------------------------------------
// LayerNorm over rows of the 32-bit residual stream, optionally through a row
// list (the head only normalises the rows whose logits are wanted).
//   mean = sum(x)/n; var = sum((x-mean)^2)/n (biased, two passes);
//   y = (x-mean) * 1/sqrt(var+eps) * gain + bias
// bisand/kvad: crates/llm/src/tensor.rs:245-255.
// One block per row; the row is staged in shared memory.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void layernorm_kernel(const float* __restrict__ x, const int* __restrict__ row_index,
                                 const void* __restrict__ gain, const void* __restrict__ bias,
                                 int params_f32, T* __restrict__ out, int width, float eps) {
  extern __shared__ float row[];
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int64_t src = row_index ? (int64_t)row_index[r] : (int64_t)r;
  const float* xr = x + src * width;
  float s = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = xr[c];
    row[c] = v;
    s += v;
  }
  const float mean = block_sum(s, scratch) / (float)width;
  float q = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float d = row[c] - mean;
    q += d * d;
  }
  const float var = block_sum(q, scratch) / (float)width;
  const float inv = 1.0f / sqrtf(var + eps);
  T* o = out + (int64_t)r * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float g = load_param(gain, c, params_f32);
    const float b = bias ? load_param(bias, c, params_f32) : 0.f;
    o[c] = from_f32<T>((row[c] - mean) * inv * g + b);
  }
}

__device__ __forceinline__ void store8(float* o, const float* y) {
  *reinterpret_cast<float4*>(o) = make_float4(y[0], y[1], y[2], y[3]);
  *reinterpret_cast<float4*>(o + 4) = make_float4(y[4], y[5], y[6], y[7]);
}
__device__ __forceinline__ void store8(__nv_bfloat16* o, const float* y) {
  __nv_bfloat162 p0 = __floats2bfloat162_rn(y[0], y[1]), p1 = __floats2bfloat162_rn(y[2], y[3]);
  __nv_bfloat162 p2 = __floats2bfloat162_rn(y[4], y[5]), p3 = __floats2bfloat162_rn(y[6], y[7]);
  uint4 q;
  q.x = *reinterpret_cast<uint32_t*>(&p0); q.y = *reinterpret_cast<uint32_t*>(&p1);
  q.z = *reinterpret_cast<uint32_t*>(&p2); q.w = *reinterpret_cast<uint32_t*>(&p3);
  *reinterpret_cast<uint4*>(o) = q;
}

// Eight consecutive parameters (32-bit or bfloat16) in one or two 16-byte loads; zeros if `take` is false.
__device__ __forceinline__ void load_params8(const void* p, int k0, int is_f32, bool take, float* f) {
  if (!take) {
#pragma unroll
    for (int t = 0; t < 8; ++t) f[t] = 0.f;
  } else if (is_f32) {
    const float4 a = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + k0);
    const float4 c = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + k0 + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = c.x; f[5] = c.y; f[6] = c.z; f[7] = c.w;
  } else {
    const uint4 q = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p) + k0);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float2 v = __bfloat1622float2(h[t]);
      f[2 * t] = v.x;
      f[2 * t + 1] = v.y;
    }
  }
}

// The same with the row in registers: WPR warps per row (1: widths up to NI * 256, sums met by shuffles only;
// 8: a block of eight warps per row, widths up to NI * 2048, the warps' sums added in warp order through
// shared memory, the block walking rows blockIdx.x, blockIdx.x + gridDim.x, ...), NI chunks of 8 per thread.  Gain and bias are parameters, not the previous kernel's
// work: they are fetched before the dependent-launch wait.
template <typename T, int NI, int WPR>
__global__ void __launch_bounds__(WPR == 1 ? 128 : 32 * WPR)
layernorm_warp_kernel(const float* __restrict__ x, const int* __restrict__ row_index,
                      const void* __restrict__ gain, const void* __restrict__ bias, int params_f32,
                      T* __restrict__ out, int n_rows, int width, float eps) {
  constexpr int TPR = 32 * WPR;                     // threads per row
  __shared__ float met[2][WPR];
  pdl_launch_dependents();
  const int t = threadIdx.x % TPR, warp = threadIdx.x >> 5;
  const int r_first = WPR == 1 ? blockIdx.x * 4 + threadIdx.x / 32 : blockIdx.x;
  float g[NI][8], b[NI][8];
#pragma unroll
  for (int i = 0; i < NI; ++i) {
    const int k0 = (t + TPR * i) * 8;
    load_params8(gain, k0, params_f32, k0 < width, g[i]);
    load_params8(bias, k0, params_f32, k0 < width && bias != nullptr, b[i]);
  }
  pdl_wait();
  // (with four warps per row a block has one row at a time and walks rows blockIdx.x, blockIdx.x + gridDim.x, ...:
  // many rows share the parameters one block fetched)
  if (r_first >= n_rows) return;
  for (int r = r_first;;) {                         // (one trip with a warp per row: the loop is for the blocks that walk rows)
  const float* xr = x + (int64_t)(row_index ? row_index[r] : r) * width;
  float v[NI][8];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < NI; ++i) {
    const int k0 = (t + TPR * i) * 8;
    if (k0 < width) {
      const float4 a = *reinterpret_cast<const float4*>(xr + k0), c = *reinterpret_cast<const float4*>(xr + k0 + 4);
      v[i][0] = a.x; v[i][1] = a.y; v[i][2] = a.z; v[i][3] = a.w; v[i][4] = c.x; v[i][5] = c.y; v[i][6] = c.z; v[i][7] = c.w;
    } else {
#pragma unroll
      for (int u = 0; u < 8; ++u) v[i][u] = 0.f;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) sum += v[i][u];
  }
  sum = warp_sum(sum);
  if (WPR > 1) {
    __syncthreads();                                  // the sums of the row before have been read
    if ((threadIdx.x & 31) == 0) met[0][warp] = sum;
    __syncthreads();
    sum = met[0][0];
#pragma unroll
    for (int w = 1; w < WPR; ++w) sum += met[0][w];   // in warp order
  }
  const float mean = sum / (float)width;
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < NI; ++i) {
    if ((t + TPR * i) * 8 < width) {
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const float d = v[i][u] - mean;
        sq = fmaf(d, d, sq);
      }
    }
  }
  sq = warp_sum(sq);
  if (WPR > 1) {
    if ((threadIdx.x & 31) == 0) met[1][warp] = sq;
    __syncthreads();
    sq = met[1][0];
#pragma unroll
    for (int w = 1; w < WPR; ++w) sq += met[1][w];
  }
  const float inv = 1.0f / sqrtf(sq / (float)width + eps);
  T* o = out + (int64_t)r * width;
#pragma unroll
  for (int i = 0; i < NI; ++i) {
    const int k0 = (t + TPR * i) * 8;
    if (k0 < width) {
      float y[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) y[u] = (v[i][u] - mean) * inv * g[i][u] + b[i][u];
      store8(o + k0, y);
    }
  }
  if (WPR == 1) break;
  r += (int)gridDim.x;
  if (r >= n_rows) break;
  }
}

template <typename T>
void launch_layernorm_regs(const float* x, const int* row_index, const void* gain, const void* bias, int params_f32, T* out,
                           int n_rows, int width, float eps, cudaStream_t stream) {
  if (width <= 1024)       // narrow rows: a warp per row
    kvad_launch(layernorm_warp_kernel<T, 4, 1>, dim3((n_rows + 3) / 4), dim3(128), 0, stream, x, row_index, gain, bias, params_f32, out, n_rows, width, eps);
  else if (width <= 2048)  // eight warps per row, 8 values a thread: few registers, so many blocks fit an SM (2048 rows of 1600: 8.9 us with four warps a row and a row a block, 7.4 with such a block walking rows, 7.2 so)
    kvad_launch(layernorm_warp_kernel<T, 1, 8>, dim3(n_rows < 1184 ? n_rows : 1184), dim3(256), 0, stream, x, row_index, gain, bias, params_f32, out, n_rows, width, eps);
  else                     // up to 4096
    kvad_launch(layernorm_warp_kernel<T, 2, 8>, dim3(n_rows < 1184 ? n_rows : 1184), dim3(256), 0, stream, x, row_index, gain, bias, params_f32, out, n_rows, width, eps);
}

// Clears device memory in stream order (a memset node when the stream is being captured).
KVAD_EXPORT int kvad_zero_bytes(void* p, int64_t bytes, cudaStream_t stream) {
  KVAD_REQUIRE(p != nullptr && bytes >= 0, "zero_bytes: bad arguments");
  cudaError_t e = cudaMemsetAsync(p, 0, (size_t)bytes, stream);
  if (e != cudaSuccess) KVAD_FAIL(KVAD_ERR_CUDA, "zero_bytes: %s", cudaGetErrorString(e));
  return KVAD_OK;
}

KVAD_EXPORT int kvad_layernorm(int out_dtype, const float* x, const int* row_index, const void* gain,
                               const void* bias, int params_f32, void* out, int n_rows, int width,
                               float eps, cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && width > 0, "layernorm: bad sizes rows=%d width=%d", n_rows, width);
  KVAD_REQUIRE(gain != nullptr, "layernorm: no gain");
  if (n_rows == 0) return KVAD_OK;
  if (width % 8 == 0 && width <= 4096 &&
      ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(gain) | reinterpret_cast<uintptr_t>(bias) |
        reinterpret_cast<uintptr_t>(out)) & 15) == 0) {
    // the row in registers
    if (out_dtype == KVAD_DTYPE_F32)
      launch_layernorm_regs<float>(x, row_index, gain, bias, params_f32, (float*)out, n_rows, width, eps, stream);
    else if (out_dtype == KVAD_DTYPE_BF16)
      launch_layernorm_regs<__nv_bfloat16>(x, row_index, gain, bias, params_f32, (__nv_bfloat16*)out, n_rows, width, eps, stream);
    else
      KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "layernorm: unknown dtype %d", out_dtype);
    KVAD_CHECK_LAUNCH("layernorm");
    return KVAD_OK;
  }
  const size_t smem = (size_t)width * sizeof(float);
  KVAD_REQUIRE(smem <= 200 * 1024, "layernorm: width %d does not fit shared memory (limit %d)", width, 200 * 1024 / 4);
  const int threads = width >= 1024 ? 256 : 128;
  if (out_dtype == KVAD_DTYPE_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(layernorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    kvad_launch(layernorm_kernel<float>, dim3(n_rows), dim3(threads), smem, stream, x, row_index, gain, bias, params_f32, (float*)out, width, eps);
  } else if (out_dtype == KVAD_DTYPE_BF16) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(layernorm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    kvad_launch(layernorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), smem, stream, x, row_index, gain, bias, params_f32, (__nv_bfloat16*)out, width, eps);
  } else {
    KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "layernorm: unknown dtype %d", out_dtype);
  }
  KVAD_CHECK_LAUNCH("layernorm");
  return KVAD_OK;
}

// ---------------------------------------------------------------------------
// Keys and values of this step's rows go to their place in the paged cache
// before any row attends (crates/llm/src/model/gpt2.rs:237-242).
// Cache pages of one layer: [n_pages, n_kv_heads, page_size, head_dim].
// Row r belongs to sequence row_seq[r] and sits at position row_pos[r]; the
// sequence's pages are page_table[row_seq[r], :].
// ---------------------------------------------------------------------------
template <typename T>
__global__ void kv_store_kernel(const T* __restrict__ k_src, const T* __restrict__ v_src, int64_t ld_src,
                                const int* __restrict__ row_seq, const int* __restrict__ row_pos,
                                const int* __restrict__ page_table, int table_width,
                                T* __restrict__ k_pages, T* __restrict__ v_pages,
                                int n_rows, int n_kv_heads, int head_dim, int page_size) {
  pdl_launch_dependents();
  pdl_wait();
  const int kv_width = n_kv_heads * head_dim;
  const int64_t total = (int64_t)n_rows * kv_width;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / kv_width), c = (int)(i % kv_width);
    const int h = c / head_dim, d = c % head_dim;
    const int pos = row_pos[r];
    const int page = page_table[(int64_t)row_seq[r] * table_width + pos / page_size];
    const int64_t dst = (((int64_t)page * n_kv_heads + h) * page_size + pos % page_size) * head_dim + d;
    k_pages[dst] = k_src[(int64_t)r * ld_src + c];
    v_pages[dst] = v_src[(int64_t)r * ld_src + c];
  }
}

// The same in 16-byte pieces (head sizes are multiples of 8 elements of 2 bytes, or 4 of 4 bytes).
template <typename T>
__global__ void kv_store_vec_kernel(const T* __restrict__ k_src, const T* __restrict__ v_src, int64_t ld_src,
                                    const int* __restrict__ row_seq, const int* __restrict__ row_pos,
                                    const int* __restrict__ page_table, int table_width,
                                    T* __restrict__ k_pages, T* __restrict__ v_pages,
                                    int n_rows, int n_kv_heads, int head_dim, int page_size) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int E = 16 / (int)sizeof(T);                 // elements per piece
  const int pieces_per_head = head_dim / E, pieces_per_row = n_kv_heads * pieces_per_head;
  const int64_t total = (int64_t)n_rows * pieces_per_row;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / pieces_per_row), p = (int)(i % pieces_per_row);
    const int h = p / pieces_per_head, d = (p % pieces_per_head) * E;
    const int pos = row_pos[r];
    const int page = page_table[(int64_t)row_seq[r] * table_width + pos / page_size];
    const int64_t dst = (((int64_t)page * n_kv_heads + h) * page_size + pos % page_size) * head_dim + d;
    const int64_t src = (int64_t)r * ld_src + (int64_t)h * head_dim + d;
    *reinterpret_cast<uint4*>(k_pages + dst) = *reinterpret_cast<const uint4*>(k_src + src);
    *reinterpret_cast<uint4*>(v_pages + dst) = *reinterpret_cast<const uint4*>(v_src + src);
  }
}

KVAD_EXPORT int kvad_kv_store(int dtype, const void* k_src, const void* v_src, int64_t ld_src,
                              const int* row_seq, const int* row_pos, const int* page_table,
                              int table_width, void* k_pages, void* v_pages, int n_rows,
                              int n_kv_heads, int head_dim, int page_size, cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && n_kv_heads > 0 && head_dim > 0 && page_size > 0 && table_width > 0,
               "kv_store: bad sizes rows=%d kv_heads=%d head_dim=%d page=%d table=%d", n_rows, n_kv_heads, head_dim, page_size, table_width);
  if (n_rows == 0) return KVAD_OK;
  const int elem = dtype == KVAD_DTYPE_F32 ? 4 : 2;
  const int per = 16 / elem;
  const bool vec = head_dim % per == 0 && ld_src % per == 0 &&
                   ((reinterpret_cast<uintptr_t>(k_src) | reinterpret_cast<uintptr_t>(v_src) |
                     reinterpret_cast<uintptr_t>(k_pages) | reinterpret_cast<uintptr_t>(v_pages)) & 15) == 0;
  const int64_t total = (int64_t)n_rows * n_kv_heads * head_dim / (vec ? per : 1);
  const int threads = 256;
  const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
#define KVAD_KV(KERNEL, T)                                                                                            \
  kvad_launch(KERNEL<T>, dim3(blocks), dim3(threads), 0, stream, (const T*)k_src, (const T*)v_src, ld_src, row_seq,   \
              row_pos, page_table, table_width, (T*)k_pages, (T*)v_pages, n_rows, n_kv_heads, head_dim, page_size)
  if (dtype == KVAD_DTYPE_F32) {
    if (vec) KVAD_KV(kv_store_vec_kernel, float); else KVAD_KV(kv_store_kernel, float);
  } else if (dtype == KVAD_DTYPE_BF16) {
    if (vec) KVAD_KV(kv_store_vec_kernel, __nv_bfloat16); else KVAD_KV(kv_store_kernel, __nv_bfloat16);
  } else {
    KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "kv_store: unknown dtype %d", dtype);
  }
#undef KVAD_KV
  KVAD_CHECK_LAUNCH("kv_store");
  return KVAD_OK;
}

KVAD_DEFINE_LAST_ERROR()
