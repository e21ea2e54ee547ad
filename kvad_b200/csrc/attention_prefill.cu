// Causal attention of a step's prompt rows over the paged cache, in bfloat16 on the tensor cores
// with a running (flash) softmax: nothing of size rows x keys ever reaches memory.
//
// A CTA of four warps serves 64 consecutive rows of one sequence and one head; it walks that
// sequence's cache pages (64 keys each) from the first page a row may see to the page of the last
// row, double-buffered through shared memory with cp.async.  Per page: S = Q.K^T on
// mma.sync.m16n8k16 (bfloat16 in, 32-bit out), scaled, masked by position (a row sees keys up to
// its own position and, with a window, not further back than the window), folded into each row's
// running maximum and sum in 32-bit, and P.V accumulated in 32-bit with P rounded to bfloat16 for
// the second product.  Rows of a cache page beyond the sequence's length are zero-filled on the
// way in, so that whatever a recycled page still holds cannot reach a result.
//
// The rows may continue a sequence that already has cached positions (a prompt in several steps):
// a row's position is its sequence's length before the step plus its offset.  Query head h reads
// key/value head h / (n_heads / n_kv_heads).  Head sizes: multiples of 16 up to 128; others are
// refused and the caller uses the general kernel.  Head sizes 64 and 128 run on the 5th-generation
// tensor cores instead (attention_prefill_tc.cuh); this kernel serves the other head sizes.
//
// bisand/kvad: attend() per row, crates/llm/src/model/mod.rs:769-819; its candle path builds the
// explicit mask instead (crates/gpu/src/gpt2.rs:249-276, crates/gpu/src/common.rs:1028-1042).
#include <cstdio>
#include <cstdlib>

#include "common.cuh"
#include "attention_prefill_tc.cuh"

using namespace kvad;

namespace {

constexpr int PF_THREADS = 128;
constexpr int PF_ROWS = 64;     // query rows per CTA (16 per warp)
constexpr int PF_KEYS = 64;     // keys per tile = one cache page

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async_16(void* dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&p);
}

template <int HD>
__global__ void __launch_bounds__(PF_THREADS)
attention_prefill_kernel(const __nv_bfloat16* __restrict__ q, int64_t ld_q, __nv_bfloat16* __restrict__ out, int64_t ld_out,
                         const int* __restrict__ seq_starts, const int* __restrict__ kv_lens,
                         const int* __restrict__ page_table, int table_width,
                         const __nv_bfloat16* __restrict__ k_pages, const __nv_bfloat16* __restrict__ v_pages,
                         int n_heads, int n_kv_heads, int n_q_tiles, float scale, int window) {
  constexpr int STRIDE = HD + 8;                 // bfloat16 per shared-memory row: 16 bytes of padding keep ldmatrix conflict-free
  constexpr int KSTEPS = HD / 16;                // k-steps of Q.K^T
  constexpr int DTILES = HD / 8;                 // 8-wide tiles of the output's head dimension
  constexpr int CHUNKS = HD / 8;                 // 16-byte chunks per row
  extern __shared__ __align__(16) unsigned char pf_smem[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(pf_smem);
  __nv_bfloat16* Ks = Qs + PF_ROWS * STRIDE;     // two buffers
  __nv_bfloat16* Vs = Ks + 2 * PF_KEYS * STRIDE; // two buffers

  const int s = blockIdx.z, h = blockIdx.y;
  const int qt = n_q_tiles - 1 - (int)blockIdx.x;        // long tiles first
  const int row0_seq = seq_starts[s];
  const int n_new = seq_starts[s + 1] - row0_seq;
  if (qt * PF_ROWS >= n_new) return;
  const int kv_len = kv_lens[s];
  const int first_pos = kv_len - n_new;
  const int kvh = h / (n_heads / n_kv_heads);
  const int* pages = page_table + (int64_t)s * table_width;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, tq = lane & 3;

  const int rows_here = (n_new - qt * PF_ROWS) < PF_ROWS ? (n_new - qt * PF_ROWS) : PF_ROWS;
  const int pos_first_row = first_pos + qt * PF_ROWS;
  const int pos_last_row = pos_first_row + rows_here - 1;
  const int j_hi = pos_last_row / PF_KEYS;
  int j_lo = 0;
  if (window > 0 && pos_first_row - window + 1 > 0) j_lo = (pos_first_row - window + 1) / PF_KEYS;

  // ---- Q tile -> shared memory (rows past the sequence's new rows are zero-filled)
  for (int i = tid; i < PF_ROWS * CHUNKS; i += PF_THREADS) {
    const int r = i / CHUNKS, c = i % CHUNKS;
    const bool ok = r < rows_here;
    const __nv_bfloat16* src = q + (int64_t)(row0_seq + qt * PF_ROWS + (ok ? r : 0)) * ld_q + (int64_t)h * HD + c * 8;
    cp_async_16(Qs + r * STRIDE + c * 8, src, ok ? 16 : 0);
  }
  auto load_kv = [&](int j, int buf) {
    const int page = pages[j];
    const __nv_bfloat16* kb = k_pages + ((int64_t)page * n_kv_heads + kvh) * PF_KEYS * HD;
    const __nv_bfloat16* vb = v_pages + ((int64_t)page * n_kv_heads + kvh) * PF_KEYS * HD;
    const int valid = kv_len - j * PF_KEYS;             // rows of this page that belong to the sequence
    for (int i = tid; i < PF_KEYS * CHUNKS; i += PF_THREADS) {
      const int r = i / CHUNKS, c = i % CHUNKS;
      const int bytes = r < valid ? 16 : 0;
      cp_async_16(Ks + (buf * PF_KEYS + r) * STRIDE + c * 8, kb + r * HD + c * 8, bytes);
      cp_async_16(Vs + (buf * PF_KEYS + r) * STRIDE + c * 8, vb + r * HD + c * 8, bytes);
    }
  };
  load_kv(j_lo, 0);
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();

  // ---- this warp's 16 rows of Q as A fragments, kept for the whole walk
  uint32_t qf[KSTEPS][4];
  {
    const int mi = lane >> 3;
    const int row = warp * 16 + (mi & 1) * 8 + (lane & 7);
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      const int col = ks * 16 + (mi >> 1) * 8;
      ldmatrix_x4(smem_addr(Qs + row * STRIDE + col), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
    }
  }

  float o[DTILES][4];
#pragma unroll
  for (int i = 0; i < DTILES; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float run_max[2] = {-INFINITY, -INFINITY}, run_sum[2] = {0.f, 0.f};
  const float sl2 = scale * 1.4426950408889634f;         // scores are folded into base-2 exponentials
  const int pos_r[2] = {pos_first_row + warp * 16 + g, pos_first_row + warp * 16 + g + 8};

  for (int j = j_lo; j <= j_hi; ++j) {
    const int buf = (j - j_lo) & 1;
    if (j < j_hi) load_kv(j + 1, buf ^ 1);               // the other buffer was last read before the barrier that ended the previous round
    cp_async_commit();

    // ---- S = Q . K^T for 16 rows x 64 keys
    float sc[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f;
    const __nv_bfloat16* Kb = Ks + buf * PF_KEYS * STRIDE;
    const __nv_bfloat16* Vb = Vs + buf * PF_KEYS * STRIDE;
    {
      const int mi = lane >> 3;
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
        for (int nt = 0; nt < 8; nt += 2) {
          const int row = (nt + (mi >> 1)) * 8 + (lane & 7);
          const int col = ks * 16 + (mi & 1) * 8;
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4(smem_addr(Kb + row * STRIDE + col), b0, b1, b2, b3);
          mma_bf16(sc[nt], qf[ks], b0, b1);
          mma_bf16(sc[nt + 1], qf[ks], b2, b3);
        }
      }
    }

    // ---- mask by position, fold into the running maximum and sum
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int t = j * PF_KEYS + nt * 8 + 2 * tq + (e & 1);
        const int p = pos_r[e >> 1];
        const bool seen = t <= p && (window <= 0 || t > p - window);
        const float v = seen ? sc[nt][e] * sl2 : -INFINITY;
        sc[nt][e] = v;
        tile_max[e >> 1] = fmaxf(tile_max[e >> 1], v);
      }
    }
    float keep[2], base[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float m = tile_max[r];
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
      const float new_max = fmaxf(run_max[r], m);
      base[r] = new_max == -INFINITY ? 0.f : new_max;    // a row that has seen nothing yet
      keep[r] = run_max[r] == -INFINITY ? 0.f : exp2f(run_max[r] - base[r]);
      run_max[r] = new_max;
    }
    float tile_sum[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float p = exp2f(sc[nt][e] - base[e >> 1]);  // exp2(-inf) = 0 for what is masked
        sc[nt][e] = p;
        tile_sum[e >> 1] += p;
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) run_sum[r] = run_sum[r] * keep[r] + tile_sum[r];
#pragma unroll
    for (int i = 0; i < DTILES; ++i) {
      o[i][0] *= keep[0]; o[i][1] *= keep[0];
      o[i][2] *= keep[1]; o[i][3] *= keep[1];
    }

    // ---- O += P . V, P rounded to bfloat16
    {
      const int mi = lane >> 3;
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {                   // 16 keys per step
        uint32_t pa[4];
        pa[0] = pack_bf16(sc[2 * kk][0], sc[2 * kk][1]);
        pa[1] = pack_bf16(sc[2 * kk][2], sc[2 * kk][3]);
        pa[2] = pack_bf16(sc[2 * kk + 1][0], sc[2 * kk + 1][1]);
        pa[3] = pack_bf16(sc[2 * kk + 1][2], sc[2 * kk + 1][3]);
#pragma unroll
        for (int dt = 0; dt < DTILES; dt += 2) {
          const int row = kk * 16 + (mi & 1) * 8 + (lane & 7);
          const int col = (dt + (mi >> 1)) * 8;
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4_trans(smem_addr(Vb + row * STRIDE + col), b0, b1, b2, b3);
          mma_bf16(o[dt], pa, b0, b1);
          mma_bf16(o[dt + 1], pa, b2, b3);
        }
      }
    }
    cp_async_wait<0>();
    __syncthreads();                                     // the next page has landed; this one may be overwritten
  }

  // ---- normalise and store
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float l = run_sum[r];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const int row = warp * 16 + g + r * 8;
    if (row < rows_here) {
      const float inv = 1.0f / l;
      __nv_bfloat16* dst = out + (int64_t)(row0_seq + qt * PF_ROWS + row) * ld_out + (int64_t)h * HD;
#pragma unroll
      for (int dt = 0; dt < DTILES; ++dt) {
        const uint32_t v = pack_bf16(o[dt][2 * r] * inv, o[dt][2 * r + 1] * inv);
        *reinterpret_cast<uint32_t*>(dst + dt * 8 + 2 * tq) = v;
      }
    }
  }
}

template <int HD>
int launch(const void* q, int64_t ld_q, void* out, int64_t ld_out, const int* seq_starts, const int* kv_lens,
           const int* page_table, int table_width, const void* k_pages, const void* v_pages, int n_seqs, int n_heads,
           int n_kv_heads, int max_new, float scale, int window, cudaStream_t stream) {
  constexpr size_t smem = (size_t)(PF_ROWS + 4 * PF_KEYS) * (HD + 8) * 2;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) KVAD_FAIL(KVAD_ERR_CUDA, "attention_prefill: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  const int n_q_tiles = (max_new + PF_ROWS - 1) / PF_ROWS;
  dim3 grid(n_q_tiles, n_heads, n_seqs);
  attention_prefill_kernel<HD><<<grid, PF_THREADS, smem, stream>>>(
      (const __nv_bfloat16*)q, ld_q, (__nv_bfloat16*)out, ld_out, seq_starts, kv_lens, page_table, table_width,
      (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, n_heads, n_kv_heads, n_q_tiles, scale, window);
  KVAD_CHECK_LAUNCH("attention_prefill");
  return KVAD_OK;
}

bool g_force_legacy = false;      // tests: keep every head size on the mma.sync kernel
int g_split_above = 0;            // tests: the tcgen05 kernel's page count above which a tile goes to both slots (0: its own)

// A [rows, cols] bfloat16 matrix with row stride ld, loaded in boxes of box_rows x 64 with the 128-byte swizzle.
int tile_map(const void* ptr, int64_t ld, int64_t rows, int cols, int box_rows, CUtensorMap* out) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) KVAD_FAIL(KVAD_ERR_CUDA, "attention_prefill: the driver does not offer cuTensorMapEncodeTiled");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    KVAD_FAIL(KVAD_ERR_CUDA, "attention_prefill: cuTensorMapEncodeTiled failed (%d) for a [%lld, %d] matrix with row stride %lld",
              (int)r, (long long)rows, cols, (long long)ld);
  return KVAD_OK;
}

template <int HD>
int launch_tc(const void* q, int64_t ld_q, int n_rows, void* out, int64_t ld_out, const int* seq_starts, const int* kv_lens,
              const int* page_table, int table_width, const void* k_pages, const void* v_pages, int64_t n_pages, int n_seqs,
              int n_heads, int n_kv_heads, int max_new, float scale, int window, cudaStream_t stream) {
  using L = pftc::Layout<HD>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(pftc::attention_prefill_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L::SMEM);
    if (e == cudaSuccess)       // all of the SM's shared memory, so that two CTAs of head size 64 fit
      e = cudaFuncSetAttribute(pftc::attention_prefill_tc_kernel<HD>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) KVAD_FAIL(KVAD_ERR_CUDA, "attention_prefill: cannot reserve %zu bytes of shared memory: %s", (size_t)L::SMEM, cudaGetErrorString(e));
    if (getenv("KVAD_DEBUG_OCCUPANCY")) {
      int n = 0;
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, pftc::attention_prefill_tc_kernel<HD>, pftc::THREADS, L::SMEM);
      cudaFuncAttributes fa;
      cudaFuncGetAttributes(&fa, pftc::attention_prefill_tc_kernel<HD>);
      size_t avail = 0;
      for (size_t sm : {(size_t)0, (size_t)49152, (size_t)81920, (size_t)99464, (size_t)110000}) {
        int k = 0;
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&k, pftc::attention_prefill_tc_kernel<HD>, pftc::THREADS, sm);
        fprintf(stderr, "  smem %zu -> %d CTAs\n", sm, k);
      }
      for (int th : {64, 128, 192, 256}) {
        int k = 0;
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&k, pftc::attention_prefill_tc_kernel<HD>, th, 0);
        fprintf(stderr, "  threads %d -> %d CTAs\n", th, k);
      }
      cudaGetLastError();
      fprintf(stderr, "attention_prefill_tc<%d>: %d CTAs per SM, %zu bytes of shared memory, %d registers, %zu static, %zu available for two\n",
              HD, n, (size_t)L::SMEM, fa.numRegs, fa.sharedSizeBytes, avail);
    }
    configured = true;
  }
  CUtensorMap mq, mk, mv;
  int rc = tile_map(q, ld_q, n_rows, n_heads * HD, pftc::ROWS, &mq);
  if (rc != KVAD_OK) return rc;
  rc = tile_map(k_pages, HD, n_pages * n_kv_heads * pftc::KEYS, HD, pftc::KEYS, &mk);
  if (rc != KVAD_OK) return rc;
  rc = tile_map(v_pages, HD, n_pages * n_kv_heads * pftc::KEYS, HD, pftc::KEYS, &mv);
  if (rc != KVAD_OK) return rc;
  // a CTA takes one long tile or two short ones, which it finds out from the sequence's length: at most a CTA a tile,
  // and the CTAs left over return at once
  const int n_q_tiles = (max_new + pftc::ROWS - 1) / pftc::ROWS;
  kvad_launch(pftc::attention_prefill_tc_kernel<HD>, dim3(n_q_tiles, n_heads, n_seqs), dim3(pftc::THREADS), L::SMEM, stream,
              mq, mk, mv, (__nv_bfloat16*)out, ld_out, seq_starts, kv_lens, page_table, table_width, n_heads, n_kv_heads,
              g_split_above > 0 ? g_split_above : pftc::SPLIT_ABOVE, scale, window);
  KVAD_CHECK_LAUNCH("attention_prefill_tc");
  return KVAD_OK;
}

}  // namespace

// Tests: 1 keeps head sizes 64 and 128 on the mma.sync kernel too.
KVAD_EXPORT void kvad_attention_prefill_force_legacy(int on) { g_force_legacy = on != 0; }

// Tests and measurements: from how many pages on (exclusive) the tcgen05 kernel gives a tile of rows to both of a
// CTA's slots, half of the pages each; 0: the kernel's own choice.
KVAD_EXPORT void kvad_attention_prefill_split_above(int pages) { g_split_above = pages; }

// How many bounded waits of the tcgen05 kernel have run out since the library was loaded (0 in a healthy run).
KVAD_EXPORT int kvad_attention_prefill_status() {
  int n = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&n, g_wait_timeouts, sizeof(int));
  if (e != cudaSuccess) {
    KVAD_FAIL(-1, "attention_prefill: cannot read the status word: %s", cudaGetErrorString(e));
  }
  return n;
}

// seq_starts[s]..seq_starts[s+1] are the packed rows of sequence s; kv_lens[s] its length after
// this step; max_new the largest number of rows any sequence brings (sizes the grid).
// n_rows: rows of q and out in all; n_pages: pages the cache tensors hold.
KVAD_EXPORT int kvad_attention_prefill(const void* q, int64_t ld_q, int n_rows, void* out, int64_t ld_out, const int* seq_starts,
                                       const int* kv_lens, const int* page_table, int table_width, const void* k_pages,
                                       const void* v_pages, int64_t n_pages, int n_seqs, int n_heads, int n_kv_heads,
                                       int head_dim, int page_size, int max_new, float scale, int window, cudaStream_t stream) {
  KVAD_REQUIRE(n_seqs >= 0 && n_heads > 0 && n_kv_heads > 0 && table_width > 0 && max_new >= 0,
               "attention_prefill: bad sizes seqs=%d heads=%d kv_heads=%d", n_seqs, n_heads, n_kv_heads);
  KVAD_REQUIRE(n_heads % n_kv_heads == 0, "attention_prefill: %d heads do not divide into %d key/value heads", n_heads, n_kv_heads);
  KVAD_REQUIRE(page_size == PF_KEYS, "attention_prefill: pages must hold %d positions, not %d", PF_KEYS, page_size);
  KVAD_REQUIRE(n_heads <= 65535 && n_seqs <= 65535, "attention_prefill: %d heads x %d sequences are more than one launch takes", n_heads, n_seqs);
  if (ld_q % 8 != 0 || ld_out % 2 != 0 || (reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(out) & 3) ||
      (reinterpret_cast<uintptr_t>(k_pages) & 15) || (reinterpret_cast<uintptr_t>(v_pages) & 15))
    KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "attention_prefill: queries and cache must be 16-byte aligned with row strides that are multiples of 8");
  if (n_seqs == 0 || max_new == 0) return KVAD_OK;
  if ((head_dim == 64 || head_dim == 128) && !g_force_legacy && scale > 0.f && ld_out % 8 == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
    if (head_dim == 64)
      return launch_tc<64>(q, ld_q, n_rows, out, ld_out, seq_starts, kv_lens, page_table, table_width, k_pages, v_pages, n_pages,
                           n_seqs, n_heads, n_kv_heads, max_new, scale, window, stream);
    return launch_tc<128>(q, ld_q, n_rows, out, ld_out, seq_starts, kv_lens, page_table, table_width, k_pages, v_pages, n_pages,
                          n_seqs, n_heads, n_kv_heads, max_new, scale, window, stream);
  }
#define KVAD_PF_CASE(HD)                                                                                           \
  case HD:                                                                                                         \
    return launch<HD>(q, ld_q, out, ld_out, seq_starts, kv_lens, page_table, table_width, k_pages, v_pages, n_seqs, \
                      n_heads, n_kv_heads, max_new, scale, window, stream);
  switch (head_dim) {
    KVAD_PF_CASE(16) KVAD_PF_CASE(32) KVAD_PF_CASE(48) KVAD_PF_CASE(64) KVAD_PF_CASE(80) KVAD_PF_CASE(96)
    KVAD_PF_CASE(112) KVAD_PF_CASE(128)
    default:
      KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "attention_prefill: head size %d is not a multiple of 16 up to 128", head_dim);
  }
#undef KVAD_PF_CASE
}

KVAD_DEFINE_LAST_ERROR()
