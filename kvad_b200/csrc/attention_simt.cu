// Causal attention of a step's rows over the paged cache, on the CUDA cores in
// 32-bit arithmetic, for any head size and any grouping of heads.  Row r of
// sequence row_seq[r] at position row_pos[r] attends over that sequence's keys
// at positions max(0, pos-window+1) .. pos (window <= 0: all of them).  A block
// serves one (row, head); it walks the keys in tiles with a running maximum and
// sum, so the order of operations for a row depends on nothing but its own
// keys.  It takes what the faster kernels do not: head sizes and page sizes
// that the decode kernel or the tiled kernel below refuse, in either dtype.
// The float32 engine's prompts (and the bfloat16 engine's, at head sizes its
// tensor-core kernel refuses) run the tiled kernel further down.
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

// ---------------------------------------------------------------------------------------------
// The same arithmetic for PROMPTS, tiled: a block takes 32 consecutive rows of one sequence and one head and
// walks the keys page by page (64 keys); a page's keys and values are brought into shared memory once for
// all 32 rows (the kernel above reads every key once per row).  Warp w owns rows 8w..8w+7: for the scores a
// lane takes two keys of the page for all eight rows (queries read as broadcasts, keys down padded rows, no
// bank conflicts), the rows' maxima and sums meet by shuffles, the weights go through shared memory, and for
// the output a lane owns dimensions lane, lane + 32, ... of all eight rows.  DPL = dimensions per lane.
// Rows of a step are the last positions of their sequences (seq_starts, kv_lens), as in the tensor-core kernel.
// ---------------------------------------------------------------------------------------------
constexpr int TR = 32, TK = 64, TILED_THREADS = 128, ROWS_PER_WARP = TR / (TILED_THREADS / 32);

template <typename T, int DPL>
__global__ void __launch_bounds__(TILED_THREADS)
attention_tiled_kernel(const T* __restrict__ q, int64_t ld_q, T* __restrict__ out, int64_t ld_out,
                       const int* __restrict__ seq_starts, const int* __restrict__ kv_lens,
                       const int* __restrict__ page_table, int table_width,
                       const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                       int n_heads, int n_kv_heads, int hd, float scale, int window) {
  extern __shared__ float tiled_smem[];
  float* Qs = tiled_smem;                         // [TR][hd]
  float* Ks = Qs + TR * hd;                       // [TK][hd + 1]
  float* Vs = Ks + TK * (hd + 1);                 // [TK][hd]
  float* Ps = Vs + TK * hd;                       // [TR][TK]
  const int s = blockIdx.y, h = blockIdx.z, row0 = blockIdx.x * TR;
  const int start = seq_starts[s], n_new = seq_starts[s + 1] - start;
  if (row0 >= n_new) return;
  const int n_rows = n_new - row0 < TR ? n_new - row0 : TR;
  const int pos0 = kv_lens[s] - n_new + row0;                     // position of the block's first row
  const int kvh = h / (n_heads / n_kv_heads);
  const int* pages = page_table + (int64_t)s * table_width;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  for (int i = tid; i < TR * hd; i += TILED_THREADS) {
    const int r = i / hd, d = i - r * hd;
    Qs[i] = r < n_rows ? to_f32(q[(int64_t)(start + row0 + r) * ld_q + (int64_t)h * hd + d]) : 0.f;
  }
  float acc[ROWS_PER_WARP][DPL], run_max[ROWS_PER_WARP], run_sum[ROWS_PER_WARP];
#pragma unroll
  for (int r = 0; r < ROWS_PER_WARP; ++r) {
    run_max[r] = -INFINITY;
    run_sum[r] = 0.f;
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[r][i] = 0.f;
  }
  const int last_pos = pos0 + n_rows - 1;
  const int first_key = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
  for (int j = first_key / TK; j <= last_pos / TK; ++j) {
    __syncthreads();                                              // the tile before has been used up (and Qs is written)
    const int page = pages[j];
    const T* kt = k_pages + ((int64_t)page * n_kv_heads + kvh) * TK * hd;
    const T* vt = v_pages + ((int64_t)page * n_kv_heads + kvh) * TK * hd;
    for (int i = tid; i < TK * hd; i += TILED_THREADS) {
      const int k = i / hd, d = i - k * hd;
      Ks[k * (hd + 1) + d] = to_f32(kt[i]);
      Vs[i] = j * TK + k <= last_pos ? to_f32(vt[i]) : 0.f;       // (a place no row sees yet may hold anything, and 0 x NaN is NaN)
    }
    __syncthreads();
    // scores of the warp's rows against keys lane and lane + 32 of the page
    float sc[ROWS_PER_WARP][2];
#pragma unroll
    for (int r = 0; r < ROWS_PER_WARP; ++r) sc[r][0] = sc[r][1] = 0.f;
    const float* k0 = Ks + lane * (hd + 1);
    const float* k1 = Ks + (lane + 32) * (hd + 1);
    const float* qw = Qs + warp * ROWS_PER_WARP * hd;
    for (int d = 0; d < hd; d += 4) {
      const float a0 = k0[d], a1 = k0[d + 1], a2 = k0[d + 2], a3 = k0[d + 3];
      const float b0 = k1[d], b1 = k1[d + 1], b2 = k1[d + 2], b3 = k1[d + 3];
#pragma unroll
      for (int r = 0; r < ROWS_PER_WARP; ++r) {
        const float4 qv = *reinterpret_cast<const float4*>(qw + r * hd + d);
        sc[r][0] = fmaf(qv.w, a3, fmaf(qv.z, a2, fmaf(qv.y, a1, fmaf(qv.x, a0, sc[r][0]))));
        sc[r][1] = fmaf(qv.w, b3, fmaf(qv.z, b2, fmaf(qv.y, b1, fmaf(qv.x, b0, sc[r][1]))));
      }
    }
    // running maximum and sum per row; the weights of the page go to shared memory
#pragma unroll
    for (int r = 0; r < ROWS_PER_WARP; ++r) {
      const int pos = pos0 + warp * ROWS_PER_WARP + r;            // (rows past the block's last one see nothing)
      const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
      const bool row_live = warp * ROWS_PER_WARP + r < n_rows;
      float v0 = -INFINITY, v1 = -INFINITY;
      const int t0 = j * TK + lane, t1 = t0 + 32;
      if (row_live && t0 >= lo && t0 <= pos) v0 = sc[r][0] * scale;
      if (row_live && t1 >= lo && t1 <= pos) v1 = sc[r][1] * scale;
      const float tile_max = warp_max(fmaxf(v0, v1));
      const float new_max = fmaxf(run_max[r], tile_max);
      const float base = new_max == -INFINITY ? 0.f : new_max;
      const float keep = run_max[r] == -INFINITY ? 0.f : expf(run_max[r] - base);
      const float p0 = v0 == -INFINITY ? 0.f : expf(v0 - base), p1 = v1 == -INFINITY ? 0.f : expf(v1 - base);
      run_sum[r] = run_sum[r] * keep + warp_sum(p0 + p1);
      run_max[r] = new_max;
#pragma unroll
      for (int i = 0; i < DPL; ++i) acc[r][i] *= keep;
      Ps[(warp * ROWS_PER_WARP + r) * TK + lane] = p0;
      Ps[(warp * ROWS_PER_WARP + r) * TK + lane + 32] = p1;
    }
    __syncwarp();
    // output: weights (broadcast) times values (a lane per dimension)
    const float* pw = Ps + warp * ROWS_PER_WARP * TK;
    for (int k = 0; k < TK; k += 4) {
      float4 pv[ROWS_PER_WARP];
#pragma unroll
      for (int r = 0; r < ROWS_PER_WARP; ++r) pv[r] = *reinterpret_cast<const float4*>(pw + r * TK + k);
#pragma unroll
      for (int i = 0; i < DPL; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) {
          const float x0 = Vs[k * hd + d], x1 = Vs[(k + 1) * hd + d], x2 = Vs[(k + 2) * hd + d], x3 = Vs[(k + 3) * hd + d];
#pragma unroll
          for (int r = 0; r < ROWS_PER_WARP; ++r)
            acc[r][i] = fmaf(pv[r].w, x3, fmaf(pv[r].z, x2, fmaf(pv[r].y, x1, fmaf(pv[r].x, x0, acc[r][i]))));
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < ROWS_PER_WARP; ++r) {
    const int row = warp * ROWS_PER_WARP + r;
    if (row < n_rows) {
      const float inv = 1.0f / run_sum[r];
#pragma unroll
      for (int i = 0; i < DPL; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) out[(int64_t)(start + row0 + row) * ld_out + (int64_t)h * hd + d] = from_f32<T>(acc[r][i] * inv);
      }
    }
  }
}

template <typename T, int DPL>
int launch_tiled(const void* q, int64_t ld_q, void* out, int64_t ld_out, const int* seq_starts, const int* kv_lens,
                 const int* page_table, int table_width, const void* k_pages, const void* v_pages, int n_seqs, int n_heads,
                 int n_kv_heads, int hd, int max_new, float scale, int window, cudaStream_t stream) {
  const size_t smem = ((size_t)TR * hd + (size_t)TK * (hd + 1) + (size_t)TK * hd + (size_t)TR * TK) * sizeof(float);
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_tiled_kernel<T, DPL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) KVAD_FAIL(KVAD_ERR_CUDA, "attention (tiled): cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = smem;
  }
  dim3 grid((max_new + TR - 1) / TR, n_seqs, n_heads);
  attention_tiled_kernel<T, DPL><<<grid, TILED_THREADS, smem, stream>>>((const T*)q, ld_q, (T*)out, ld_out, seq_starts, kv_lens, page_table,
                                                                         table_width, (const T*)k_pages, (const T*)v_pages, n_heads,
                                                                         n_kv_heads, hd, scale, window);
  KVAD_CHECK_LAUNCH("attention_tiled");
  return KVAD_OK;
}

}  // namespace

// Prompts (rows of sequences packed one after another, each sequence's rows being its last positions): head sizes that
// are multiples of 4 up to 256, pages of 64 positions; otherwise KVAD_ERR_UNSUPPORTED and the caller takes kvad_attention_simt.
KVAD_EXPORT int kvad_attention_tiled(int dtype, const void* q, int64_t ld_q, void* out, int64_t ld_out, const int* seq_starts,
                                     const int* kv_lens, const int* page_table, int table_width, const void* k_pages,
                                     const void* v_pages, int n_seqs, int n_heads, int n_kv_heads, int head_dim, int page_size,
                                     int max_new, float scale, int window, cudaStream_t stream) {
  KVAD_REQUIRE(n_seqs >= 0 && n_heads > 0 && n_kv_heads > 0 && head_dim > 0 && table_width > 0 && max_new >= 0,
               "attention (tiled): bad sizes seqs=%d heads=%d kv_heads=%d head_dim=%d", n_seqs, n_heads, n_kv_heads, head_dim);
  KVAD_REQUIRE(n_heads % n_kv_heads == 0, "attention (tiled): %d heads do not divide into %d key/value heads", n_heads, n_kv_heads);
  if (head_dim % 4 != 0 || head_dim > 256 || page_size != TK)
    KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "attention (tiled): takes head sizes that are multiples of 4 up to 256 and pages of %d positions (head size %d, page %d)", TK, head_dim, page_size);
  KVAD_REQUIRE(n_seqs <= 65535 && n_heads <= 65535, "attention (tiled): %d sequences x %d heads are more than one launch takes", n_seqs, n_heads);
  if (n_seqs == 0 || max_new == 0) return KVAD_OK;
  const int dpl = (head_dim + 31) / 32;
#define KVAD_TILED(D)                                                                                                           \
  case D:                                                                                                                       \
    if (dtype == KVAD_DTYPE_F32)                                                                                                \
      return launch_tiled<float, D>(q, ld_q, out, ld_out, seq_starts, kv_lens, page_table, table_width, k_pages, v_pages, n_seqs, \
                                    n_heads, n_kv_heads, head_dim, max_new, scale, window, stream);                             \
    if (dtype == KVAD_DTYPE_BF16)                                                                                               \
      return launch_tiled<__nv_bfloat16, D>(q, ld_q, out, ld_out, seq_starts, kv_lens, page_table, table_width, k_pages, v_pages, \
                                            n_seqs, n_heads, n_kv_heads, head_dim, max_new, scale, window, stream);             \
    break;
  switch (dpl) {
    KVAD_TILED(1) KVAD_TILED(2) KVAD_TILED(3) KVAD_TILED(4) KVAD_TILED(5) KVAD_TILED(6) KVAD_TILED(7) KVAD_TILED(8)
  }
#undef KVAD_TILED
  KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "attention (tiled): unknown dtype %d", dtype);
}

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
