// out[M,N] = epilogue(A[M,K] . W[N,K]^T + bias) in bfloat16 on the 5th-generation
// tensor cores of sm_100a: operands come to shared memory by TMA
// (cp.async.bulk.tensor, 128-byte swizzle), one elected thread issues
// tcgen05.mma with the accumulator in tensor memory, and four warps read it
// back with tcgen05.ld for the fused epilogue (bias; GELU; the 32-bit residual
// sum; 32-bit logits).  Both operands are K-major, which is how activations
// lie in memory and how the weights are held ([out, in]); a tied output head
// is the embedding table as it is.
//
// One CTA computes one 128 x BN tile; BN (16..256) is chosen so that the grid
// fills the 148 SMs: wide tiles when there are many rows (prompts), narrow
// ones when there are few (decoding), where the kernel is a stream of weights
// and the rows beyond M are zero-filled by TMA at no memory traffic.  For the
// residual epilogue K may also be split over CTAs, the partial sums meeting in
// the 32-bit residual stream through atomic adds.
//
// With at most 64 rows (decoding) the roles are swapped: 128 rows of the WEIGHT
// matrix are the M side of the MMA and the few activation rows its N side, so
// that a stage of the pipeline is 16 KB of weights and 2-8 KB of activations
// instead of the other way round, every byte TMA brings is a byte the product
// needs, and a CTA can keep its whole share of the weights in flight at once.
//
// Sizes: any M and N (tails are predicated), K a multiple of 8 (a TMA row
// stride is a multiple of 16 bytes); the K tail of a 64-wide block is zero-
// filled.  Other shapes are refused with a message, and the caller falls back
// to the CUDA-core kernel.
//
// Every wait on an mbarrier is bounded; a wait that runs out raises a counter
// that kvad_linear_tcgen05_status() returns, and the CTA goes on to free its
// tensor memory and return.
//
// bisand/kvad's counterpart is its CPU gemm_bt (crates/llm/src/tensor.rs:102-193)
// and, on its Metal path, the tensor-op matmul behind Proj::Dense
// (crates/gpu/src/common.rs:67-73).
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "tcgen05.cuh"

using namespace kvad;

namespace {

constexpr int BM = 128;
constexpr int BK = 64;              // 64 bfloat16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;    // warp 0: TMA, warp 1: MMA + tensor memory, warps 2-5: epilogue
constexpr int NUM_THREADS_WIDE = 320;   // the wide form has eight epilogue warps: two per quarter of the tensor-memory lanes
constexpr int SMEM_BUDGET = 200 * 1024;
constexpr int SMEM_BUDGET_WIDE = 192 * 1024;     // the wide form keeps 33 KB for its output slabs

bool g_no_3d = false;               // tests: keep the swapped form on one TMA load per K block
bool g_test_skip_load = false;      // tests: the next launch of the swapped form (one load per K block) leaves out its first load
bool g_no_cluster_k = false;        // tests: never split K over a cluster under a storing epilogue
bool g_no_tma_out = false;          // tests: the wide form writes its output with plain stores
bool g_force_3d = false;            // tests: take the grouped three-dimensional loads at every row count

template <int BN> struct Tile {
  static constexpr uint32_t A_BYTES = BM * BK * 2;
  static constexpr uint32_t B_BYTES = BN * BK * 2;
  static constexpr int STAGES_RAW = SMEM_BUDGET_WIDE / (A_BYTES + B_BYTES);
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int TMEM_COLS = BN < 32 ? 32 : (BN <= 32 ? 32 : (BN <= 64 ? 64 : (BN <= 128 ? 128 : 256)));   // a power of two
  static constexpr int ACC_BUFS = 2;        // accumulators in tensor memory: the epilogue of one tile runs under the next one's products
  // after the stages: the barriers, the bias of a tile as floats, and one 4 KB slab per epilogue warp
  // from which TMA stores (or reduce-adds) 32 rows x 128 bytes of output at a time
  static constexpr size_t SLAB_OFFSET = (((size_t)STAGES * (A_BYTES + B_BYTES) + (2 * STAGES + 2 * ACC_BUFS) * 8 + 16 + BN * 4) + 1023) / 1024 * 1024;
  static constexpr size_t SMEM = SLAB_OFFSET + 8 * 4096 + 1024;
};

// bfloat16 x bfloat16 -> float32, both K-major, M = 128, N = BN.
template <int BN, int M_ROWS = BM> __device__ __forceinline__ constexpr uint32_t instr_desc() {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(M_ROWS >> 4) << 24);
}

// tanh-form GELU with the hardware tanh (tanh.approx.f32, relative error about 2^-11): the result is
// rounded to bfloat16 (8 bits of mantissa) right after, and the exact tanhf costs the epilogue of the
// up-projection several times what its whole product costs.
__device__ __forceinline__ float gelu_tanh_fast(float t) {
  const float c = 0.79788456f;
  float th;
  asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(c * (t + 0.044715f * t * t * t)));
  return 0.5f * t * (1.0f + th);
}

// One chunk of CH consecutive columns of one output row.
template <int EPI, int CH>
__device__ __forceinline__ void store_chunk(const float* v, void* out, int64_t ldo, int row, int col0, int N,
                                            const void* bias, int bias_f32, bool add_bias, bool atomic) {
  float x[CH];
#pragma unroll
  for (int j = 0; j < CH; ++j) {
    float t = v[j];
    if (add_bias && bias != nullptr && col0 + j < N) t += load_param(bias, col0 + j, bias_f32);
    if (EPI == EPI_GELU_TANH) t = gelu_tanh_fast(t);
    if (EPI == EPI_GELU_ERF) t = gelu_erf(t);
    x[j] = t;
  }
  const bool full = col0 + CH <= N;
  if (EPI == EPI_STORE || EPI == EPI_GELU_TANH || EPI == EPI_GELU_ERF) {
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out) + (int64_t)row * ldo + col0;
    if (full && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
#pragma unroll
      for (int j = 0; j < CH; j += 8) {
        __nv_bfloat162 p0 = __floats2bfloat162_rn(x[j], x[j + 1]), p1 = __floats2bfloat162_rn(x[j + 2], x[j + 3]);
        __nv_bfloat162 p2 = __floats2bfloat162_rn(x[j + 4], x[j + 5]), p3 = __floats2bfloat162_rn(x[j + 6], x[j + 7]);
        uint4 q;
        q.x = *reinterpret_cast<uint32_t*>(&p0); q.y = *reinterpret_cast<uint32_t*>(&p1);
        q.z = *reinterpret_cast<uint32_t*>(&p2); q.w = *reinterpret_cast<uint32_t*>(&p3);
        *reinterpret_cast<uint4*>(o + j) = q;
      }
    } else {
#pragma unroll
      for (int j = 0; j < CH; ++j)
        if (col0 + j < N) o[j] = __float2bfloat16_rn(x[j]);
    }
  } else {
    float* o = reinterpret_cast<float*>(out) + (int64_t)row * ldo + col0;
    if (EPI == EPI_RESIDUAL && atomic) {
#pragma unroll
      for (int j = 0; j < CH; ++j)
        if (col0 + j < N) atomicAdd(o + j, x[j]);
    } else if (full && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
#pragma unroll
      for (int j = 0; j < CH; j += 4) {
        float4 q = make_float4(x[j], x[j + 1], x[j + 2], x[j + 3]);
        if (EPI == EPI_RESIDUAL) {
          const float4 old = *reinterpret_cast<float4*>(o + j);
          q.x += old.x; q.y += old.y; q.z += old.z; q.w += old.w;
        }
        *reinterpret_cast<float4*>(o + j) = q;
      }
    } else {
#pragma unroll
      for (int j = 0; j < CH; ++j)
        if (col0 + j < N) o[j] = (EPI == EPI_RESIDUAL) ? o[j] + x[j] : x[j];
    }
  }
}

// One CTA per SM walks the tiles t = blockIdx.x, blockIdx.x + gridDim.x, ... (n fastest, then m, then the
// K split): the ring of stages runs on from one tile into the next, and with two accumulators in tensor
// memory the epilogue warps empty one while the MMAs fill the other.
template <int BN, int EPI>
__global__ void __launch_bounds__(NUM_THREADS_WIDE, 1)
linear_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                      const __grid_constant__ CUtensorMap map_out, int tma_out,
                      const void* __restrict__ bias, int bias_f32, void* __restrict__ out, int64_t ldo,
                      int M, int N, int K, int kb_per_split, int n_splits) {
  using T = Tile<BN>;
  constexpr int STAGES = T::STAGES, ACC_BUFS = T::ACC_BUFS;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* a_tiles = smem;
  uint8_t* b_tiles = smem + STAGES * T::A_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(b_tiles + STAGES * T::B_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full_bar = empty_bar + STAGES;           // [ACC_BUFS] the accumulator is complete
  uint64_t* tmem_empty_bar = tmem_full_bar + ACC_BUFS;    // [ACC_BUFS] the eight epilogue warps have read it
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + ACC_BUFS);
  float* bias_st = reinterpret_cast<float*>(tmem_slot + 4);   // [BN]

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 32) {
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_w);
    if (tma_out) prefetch_tensormap(&map_out);
  }
  const int n_tiles_n = (N + BN - 1) / BN, n_tiles_m = (M + BM - 1) / BM;
  const int n_tiles = n_tiles_n * n_tiles_m * n_splits;
  const int kb_total = (K + BK - 1) / BK;
  // tile t: its corner and its share of K
  auto tile_of = [&](int t, int* n0, int* m0, int* kb_begin, int* num_kb, int* z) {
    const int nt = t % n_tiles_n, rest = t / n_tiles_n;
    const int mt = rest % n_tiles_m;
    *z = rest / n_tiles_m;
    *n0 = nt * BN;
    *m0 = mt * BM;
    *kb_begin = *z * kb_per_split;
    const int kb_end = *kb_begin + kb_per_split < kb_total ? *kb_begin + kb_per_split : kb_total;
    *num_kb = kb_end - *kb_begin;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < ACC_BUFS; ++b) {
      mbar_init(&tmem_full_bar[b], 1);
      mbar_init(&tmem_empty_bar[b], 8);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, ACC_BUFS * T::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;                       // stages filled so far, over all tiles
      bool waited = false, ok = true;
      for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
        int n0, m0, kb_begin, num_kb, z;
        tile_of(t, &n0, &m0, &kb_begin, &num_kb, &z);
        int i = 0;
        if (!waited) {
          // weights do not depend on the kernel before: the first tile's first stages are on the way before the wait
          const int pre = num_kb < STAGES ? num_kb : STAGES;
          for (int j = 0; j < pre; ++j) {
            mbar_expect_tx(&full_bar[j], T::A_BYTES + T::B_BYTES);
            tma_load_2d(b_tiles + j * T::B_BYTES, &map_w, &full_bar[j], (kb_begin + j) * BK, n0);
          }
          pdl_wait();
          waited = true;
          for (int j = 0; j < pre; ++j)
            tma_load_2d(a_tiles + j * T::A_BYTES, &map_a, &full_bar[j], (kb_begin + j) * BK, m0);
          i = pre;
          it = pre;
        }
        for (; i < num_kb; ++i, ++it) {
          const int s = it % STAGES;
          if (it >= (uint32_t)STAGES && !mbar_wait(&empty_bar[s], ((it / STAGES) & 1) ^ 1)) { ok = false; break; }
          mbar_expect_tx(&full_bar[s], T::A_BYTES + T::B_BYTES);
          tma_load_2d(a_tiles + s * T::A_BYTES, &map_a, &full_bar[s], (kb_begin + i) * BK, m0);
          tma_load_2d(b_tiles + s * T::B_BYTES, &map_w, &full_bar[s], (kb_begin + i) * BK, n0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc<BN>();
      uint32_t it = 0;
      int lt = 0;                            // tiles of this CTA so far
      bool ok = true;
      for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, ++lt) {
        int n0, m0, kb_begin, num_kb, z;
        tile_of(t, &n0, &m0, &kb_begin, &num_kb, &z);
        const int buf = lt % ACC_BUFS;
        if (lt >= ACC_BUFS) {                // the epilogue has emptied this accumulator
          ok = mbar_wait(&tmem_empty_bar[buf], ((lt / ACC_BUFS) & 1) ^ 1);
          if (!ok) break;
          tc_fence_after();
        }
        const uint32_t acc = tmem_base + (uint32_t)(buf * T::TMEM_COLS);
        for (int i = 0; i < num_kb; ++i, ++it) {
          const int s = it % STAGES;
          ok = mbar_wait(&full_bar[s], (it / STAGES) & 1);
          if (!ok) break;
          tc_fence_after();
          const uint64_t a_desc = sw128_desc(smem_u32(a_tiles + s * T::A_BYTES));
          const uint64_t b_desc = sw128_desc(smem_u32(b_tiles + s * T::B_BYTES));
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // 16 elements further along K: 32 bytes inside the swizzled row, i.e. 2 in units of 16 bytes
            umma(acc, a_desc + (uint64_t)(k * 2), b_desc + (uint64_t)(k * 2), idesc, (i > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[s]);     // the stage is free again once these MMAs have read it
        }
        if (!ok) break;
        umma_commit(&tmem_full_bar[buf]); // the accumulator is complete once everything issued has run
      }
    }
  } else {
    const int quarter = warp & 3;       // the 32 tensor-memory lanes this warp may read
    bool waited = false, slab_used = false, dead = false;
    int lt = 0;
    for (int t = blockIdx.x; t < n_tiles; t += gridDim.x, ++lt) {
      int n0, m0, kb_begin, num_kb, z;
      tile_of(t, &n0, &m0, &kb_begin, &num_kb, &z);
      const int buf = lt % ACC_BUFS;
      const uint32_t acc = tmem_base + (uint32_t)(buf * T::TMEM_COLS) + ((uint32_t)(quarter * 32) << 16);
      const int row = m0 + quarter * 32 + lane;
      float* bias_sh = bias_st;
      if (tma_out) {                        // this tile's bias, as floats, while the product runs
        if (lt > 0) asm volatile("bar.sync 1, 256;" ::: "memory");   // all eight warps are done with the last tile's
        for (int j = threadIdx.x - 64; j < BN; j += NUM_THREADS_WIDE - 64)
          bias_sh[j] = (bias != nullptr && n0 + j < N) ? load_param(bias, n0 + j, bias_f32) : 0.f;
        asm volatile("bar.sync 1, 256;" ::: "memory");     // the eight epilogue warps
      }
      if (!waited) {
        pdl_wait();
        waited = true;
      }
      // (a warp whose wait ran out goes on through the loop without working, so that it still meets the
      // others at the barrier above)
      if (dead || !mbar_wait(&tmem_full_bar[buf], (lt / ACC_BUFS) & 1)) {
        dead = true;
        continue;
      }
      tc_fence_after();
      const bool add_bias = z == 0;
      const float bias_on = add_bias ? 1.f : 0.f;     // only the first share of K brings the bias (staged values are finite)
      const bool atomic = n_splits > 1;
      // two warps share a quarter of the lanes: the first takes the left half of the columns, the second the right
      constexpr int HALF = BN >= 32 ? BN / 2 : BN;
      const int c_begin = (BN >= 32 && warp >= 6) ? HALF : 0;
      const int c_end = (BN >= 32) ? c_begin + HALF : (warp >= 6 ? 0 : BN);
      if (tma_out) {
        // ---- through a slab in shared memory, out by TMA: whole 128-byte rows, no read-modify-write here
        constexpr bool F32_OUT = (EPI == EPI_RESIDUAL || EPI == EPI_STORE_F32);
        constexpr int SLAB_COLS = F32_OUT ? 32 : 64;              // 128 bytes of output per row
        uint8_t* slab = smem + T::SLAB_OFFSET + (size_t)(warp - 2) * 4096;
        // the two warps of a quarter take alternate slabs
        const int first = (warp >= 6 ? 1 : 0) * SLAB_COLS;
#pragma unroll 1
        for (int c0 = first; c0 < BN; c0 += 2 * SLAB_COLS) {
          if (slab_used) {                                          // the slab's last journey has been read
            if (lane == 0) bulk_wait_read();
            __syncwarp();
          }
          slab_used = true;
#pragma unroll
          for (int cc = 0; cc < SLAB_COLS; cc += 16) {
            float v[16];
            tmem_ld16(acc + (uint32_t)(c0 + cc), v);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              float x = fmaf(bias_sh[c0 + cc + j], bias_on, v[j]);     // (no test per element: see bias_on)
              if (EPI == EPI_GELU_TANH) x = gelu_tanh_fast(x);
              if (EPI == EPI_GELU_ERF) x = gelu_erf(x);
              v[j] = x;
            }
            if (F32_OUT) {
#pragma unroll
              for (int j = 0; j < 16; j += 4) {
                const int chunk = (cc + j) >> 2;                   // 16-byte piece of the 128-byte row
                *reinterpret_cast<float4*>(slab + lane * 128 + ((chunk ^ (lane & 7)) << 4)) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 16; j += 8) {
                const int chunk = (cc + j) >> 3;
                __nv_bfloat162 p0 = __floats2bfloat162_rn(v[j], v[j + 1]), p1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
                __nv_bfloat162 p2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]), p3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
                uint4 q;
                q.x = *reinterpret_cast<uint32_t*>(&p0); q.y = *reinterpret_cast<uint32_t*>(&p1);
                q.z = *reinterpret_cast<uint32_t*>(&p2); q.w = *reinterpret_cast<uint32_t*>(&p3);
                *reinterpret_cast<uint4*>(slab + lane * 128 + ((chunk ^ (lane & 7)) << 4)) = q;
              }
            }
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0 && n0 + c0 < N && m0 + quarter * 32 < M) {
            if (EPI == EPI_RESIDUAL) tma_reduce_add_2d(&map_out, slab, n0 + c0, m0 + quarter * 32);
            else tma_store_2d(&map_out, slab, n0 + c0, m0 + quarter * 32);
            bulk_commit();
          }
        }
      } else {
#pragma unroll 1
        for (int c = c_begin; c < c_end; c += 16) {
          float v[16];
          tmem_ld16(acc + (uint32_t)c, v);   // all lanes take part
          if (row < M && n0 + c < N)
            store_chunk<EPI, 16>(v, out, ldo, row, n0 + c, N, bias, bias_f32, add_bias, atomic);
        }
      }
      // this warp has read its share of the accumulator: the MMAs of the tile after next may overwrite it
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_one(&tmem_empty_bar[buf]);
    }
    if (lane == 0) bulk_wait_all();
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, ACC_BUFS * T::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------
// The swapped form for M <= MB <= 64 rows: D[n, m] = sum_k W[n, k] A[m, k].
// One CTA owns 128 rows of W (and, with split K, a range of K); the accumulator has the weight rows
// in the tensor-memory lanes and the activation rows in its columns, so a warp of the epilogue holds
// 32 consecutive outputs of one activation row and writes them side by side.
// ---------------------------------------------------------------------------------------------
template <int MB, int TM> struct SkinnyTile {
  static constexpr uint32_t W_BYTES = TM * BK * 2;
  static constexpr uint32_t A_BYTES = MB * BK * 2;
  static constexpr int STAGES_RAW = SMEM_BUDGET / (W_BYTES + A_BYTES);
  static constexpr int STAGES = STAGES_RAW > 12 ? 12 : STAGES_RAW;
  static constexpr int TMEM_COLS = MB < 32 ? 32 : MB;
  static constexpr size_t SMEM = (size_t)STAGES * (W_BYTES + A_BYTES) + (2 * STAGES + 1) * 8 + 16 + 1024;
};

// TM = 128 or 64 weight rows per CTA.  With 64 the accumulator sits in tensor-memory lanes
// (row % 16) + 32 * (row / 16): the first 16 lanes of each of the four warps' quarters.
template <int MB, int EPI, int TM>
__global__ void __launch_bounds__(NUM_THREADS, 1)
linear_tcgen05_skinny_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                             const void* __restrict__ bias, int bias_flags, void* __restrict__ out, int64_t ldo,
                             int M, int N, int K, int kb_per_split) {
  using T = SkinnyTile<MB, TM>;
  constexpr int STAGES = T::STAGES;
  const int bias_f32 = bias_flags & 1;
  const bool test_skip_first_load = (bias_flags & 2) != 0;     // a test's way to make a bounded wait run out: nothing ever fills stage 0
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* w_tiles = smem;
  uint8_t* a_tiles = smem + STAGES * T::W_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(a_tiles + STAGES * T::A_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full_bar = empty_bar + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_full_bar + 1);

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 32) {
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_w);
  }
  const int n0 = blockIdx.x * TM;
  const int kb_total = (K + BK - 1) / BK;
  const int kb_begin = blockIdx.y * kb_per_split;
  const int kb_end = kb_begin + kb_per_split < kb_total ? kb_begin + kb_per_split : kb_total;
  const int num_kb = kb_end - kb_begin;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(tmem_full_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, T::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      // this CTA's weights (often all of them) are requested before the kernel before has finished
      const int pre = num_kb < STAGES ? num_kb : STAGES;
      for (int i = test_skip_first_load ? 1 : 0; i < pre; ++i) {
        mbar_expect_tx(&full_bar[i], T::W_BYTES + T::A_BYTES);
        tma_load_2d(w_tiles + i * T::W_BYTES, &map_w, &full_bar[i], (kb_begin + i) * BK, n0);
      }
      pdl_wait();
      for (int i = test_skip_first_load ? 1 : 0; i < pre; ++i)
        tma_load_2d(a_tiles + i * T::A_BYTES, &map_a, &full_bar[i], (kb_begin + i) * BK, 0);
      for (int i = pre; i < num_kb; ++i) {
        const int s = i % STAGES;
        const uint32_t phase = (i / STAGES) & 1;
        if (!mbar_wait(&empty_bar[s], phase ^ 1)) break;
        mbar_expect_tx(&full_bar[s], T::W_BYTES + T::A_BYTES);
        tma_load_2d(w_tiles + s * T::W_BYTES, &map_w, &full_bar[s], (kb_begin + i) * BK, n0);
        tma_load_2d(a_tiles + s * T::A_BYTES, &map_a, &full_bar[s], (kb_begin + i) * BK, 0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc<MB, TM>();
      for (int i = 0; i < num_kb; ++i) {
        const int s = i % STAGES;
        const uint32_t phase = (i / STAGES) & 1;
        if (!mbar_wait(&full_bar[s], phase)) break;
        tc_fence_after();
        const uint64_t w_desc = sw128_desc(smem_u32(w_tiles + s * T::W_BYTES));
        const uint64_t a_desc = sw128_desc(smem_u32(a_tiles + s * T::A_BYTES));
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k)
          umma(tmem_base, w_desc + (uint64_t)(k * 2), a_desc + (uint64_t)(k * 2), idesc, (i > 0 || k > 0) ? 1u : 0u);
        umma_commit(&empty_bar[s]);
      }
      umma_commit(tmem_full_bar);
    }
  } else {
    const int quarter = warp & 3;
    const bool has_row = TM == 128 || lane < 16;
    const int n = has_row ? n0 + (TM == 128 ? quarter * 32 + lane : quarter * 16 + lane) : N;
    float b = 0.f;                                   // a parameter: fetched while the product is still running
    if (blockIdx.y == 0 && bias != nullptr && n < N) b = load_param(bias, n, bias_f32);
    pdl_wait();
    const bool ok = mbar_wait(tmem_full_bar, 0);
    tc_fence_after();
    if (ok) {
      const bool atomic = gridDim.y > 1;
#pragma unroll 1
      for (int c = 0; c < MB; c += 16) {
        float v[16];
        tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c, v);
        if (n < N && c < M) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = c + j;
            if (m < M) {
              float t = v[j] + b;
              if (EPI == EPI_GELU_TANH) t = gelu_tanh_fast(t);
              if (EPI == EPI_GELU_ERF) t = gelu_erf(t);
              const int64_t o = (int64_t)m * ldo + n;
              if (EPI == EPI_STORE || EPI == EPI_GELU_TANH || EPI == EPI_GELU_ERF) {
                reinterpret_cast<__nv_bfloat16*>(out)[o] = __float2bfloat16_rn(t);
              } else if (EPI == EPI_RESIDUAL) {
                if (atomic) atomicAdd(reinterpret_cast<float*>(out) + o, t);
                else reinterpret_cast<float*>(out)[o] += t;
              } else {
                reinterpret_cast<float*>(out)[o] = t;
              }
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, T::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------
// The swapped form with few, large TMA loads (K a multiple of 64).  Timing the form above showed its
// cost to grow with the NUMBER of 64-wide K blocks a CTA walks (about 0.3 us each), not with their
// bytes or their MMAs: every block costs two TMA instructions and a barrier round trip.  Here the
// matrices are described to TMA as three-dimensional, [K/64][rows][64], so that ONE instruction
// brings the CTA's whole share of the activations (all its K blocks) and one brings a group of G
// K blocks of 128 weight rows (64 KB for G = 4); a CTA of the qkv product issues 4 loads instead of 24.
// ---------------------------------------------------------------------------------------------
constexpr int W_GROUP = 4;          // K blocks of weights per TMA instruction and pipeline stage
#ifndef KVAD_MAX_SPLIT_CTAS
#define KVAD_MAX_SPLIT_CTAS 444     // CTAs of a launch whose K is split: three times the SMs
#endif

template <int MB, int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 1)
linear_tcgen05_skinny3d_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                               const void* __restrict__ bias, int bias_f32, void* __restrict__ out, int64_t ldo,
                               int M, int N, int K, int kb_per_split, int stages, int cluster_reduce) {
  constexpr uint32_t W_BYTES = BM * BK * 2;            // one K block of 128 weight rows
  constexpr uint32_t A_BYTES = MB * BK * 2;            // one K block of the activation rows
  constexpr int TMEM_COLS = MB < 32 ? 32 : MB;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* a_all = smem;                                               // kb_per_split blocks
  uint8_t* w_ring = smem + (size_t)kb_per_split * A_BYTES;             // stages x W_GROUP blocks
  uint64_t* w_full = reinterpret_cast<uint64_t*>(w_ring + (size_t)stages * W_GROUP * W_BYTES);
  uint64_t* w_empty = w_full + stages;
  uint64_t* a_full = w_empty + stages;
  uint64_t* tmem_full_bar = a_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_full_bar + 1);
  uint64_t* recv_bar = reinterpret_cast<uint64_t*>(tmem_slot + 4);     // credited with the partial sums the cluster's CTAs send here
  float* recv_sh = reinterpret_cast<float*>(recv_bar + 2);             // [ranks][rows of this CTA][128] received (cluster_reduce)
  float* part_sh = recv_sh + (size_t)(MB + 8) * BM;                    // [MB][128] this CTA's own partial sums, to be sent

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 32) {
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_w);
  }
  const int n0 = blockIdx.x * BM;
  const int kb_total = K / BK;
  const int kb_begin = blockIdx.y * kb_per_split;
  const int kb_end = kb_begin + kb_per_split < kb_total ? kb_begin + kb_per_split : kb_total;
  const int num_kb = kb_end - kb_begin;
  const int n_groups = (num_kb + W_GROUP - 1) / W_GROUP;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&w_full[s], 1);
      mbar_init(&w_empty[s], 1);
    }
    mbar_init(a_full, 1);
    mbar_init(tmem_full_bar, 1);
    mbar_init(recv_bar, 4 * gridDim.y);                    // the four epilogue warps of every CTA of the cluster
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      const int pre = n_groups < stages ? n_groups : stages;
      for (int g = 0; g < pre; ++g) {                      // weights: before the dependent-launch wait
        mbar_expect_tx(&w_full[g], W_GROUP * W_BYTES);
        tma_load_3d(w_ring + (size_t)g * W_GROUP * W_BYTES, &map_w, &w_full[g], 0, n0, kb_begin + g * W_GROUP);
      }
      pdl_wait();
      mbar_expect_tx(a_full, (uint32_t)kb_per_split * A_BYTES);
      tma_load_3d(a_all, &map_a, a_full, 0, 0, kb_begin);
    }
    // (every thread of the cluster arrives at its barrier once, early; the epilogue warps wait on it much later,
    // just before they write into the other CTAs' shared memory, whose barriers are then known to be initialised)
    __syncwarp();
    if (cluster_reduce) cluster_arrive();
    if (lane == 0) {
      const int pre = n_groups < stages ? n_groups : stages;
      for (int g = pre; g < n_groups; ++g) {
        const int s = g % stages;
        if (!mbar_wait(&w_empty[s], ((g / stages) & 1) ^ 1)) break;
        mbar_expect_tx(&w_full[s], W_GROUP * W_BYTES);
        tma_load_3d(w_ring + (size_t)s * W_GROUP * W_BYTES, &map_w, &w_full[s], 0, n0, kb_begin + g * W_GROUP);
      }
    }
  } else if (warp == 1) {
    if (cluster_reduce) cluster_arrive();
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc<MB>();
      bool ok = mbar_wait(a_full, 0);
      for (int g = 0; g < n_groups && ok; ++g) {
        const int s = g % stages;
        ok = mbar_wait(&w_full[s], (g / stages) & 1);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int j = 0; j < W_GROUP; ++j) {
          const int kb = g * W_GROUP + j;
          if (kb < num_kb) {
            const uint64_t w_desc = sw128_desc(smem_u32(w_ring + ((size_t)s * W_GROUP + j) * W_BYTES));
            const uint64_t a_desc = sw128_desc(smem_u32(a_all + (size_t)kb * A_BYTES));
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)
              umma(tmem_base, w_desc + (uint64_t)(k * 2), a_desc + (uint64_t)(k * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
        }
        umma_commit(&w_empty[s]);
      }
      umma_commit(tmem_full_bar);
    }
  } else {
    const int quarter = warp & 3;
    const int n = n0 + quarter * 32 + lane;
    float b = 0.f;
    if ((blockIdx.y == 0 || cluster_reduce) && bias != nullptr && n < N) b = load_param(bias, n, bias_f32);
    if (cluster_reduce) cluster_arrive();
    pdl_wait();
    const bool ok = mbar_wait(tmem_full_bar, 0);
    tc_fence_after();
    if (cluster_reduce) {
      // K is split over the CTAs of a thread-block cluster.  Row m is summed by CTA m % z: every CTA writes its
      // partial sums of that row into THAT CTA's shared memory and arrives on its barrier; the owner waits for
      // all of them, adds them in rank order, applies bias and activation and stores.  One one-way trip through
      // the cluster's network; no CTA reads another's memory, so none has to wait for the others before it exits.
      const int z = (int)gridDim.y, rank = (int)blockIdx.y;
      const int rows_max = (MB + z - 1) / z;
      const int n_local = quarter * 32 + lane;
      if (ok) {
#pragma unroll 1
        for (int c = 0; c < MB; c += 16) {
          float v[16];
          tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c, v);
#pragma unroll
          for (int j = 0; j < 16; ++j) part_sh[(c + j) * BM + n_local] = v[j];
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");          // the four epilogue warps: the rows are whole
      cluster_wait();
      for (int idx = (warp - 2) * 32 + lane; idx < M * (BM / 4); idx += 128) {
        const int m = idx / (BM / 4), col = (idx % (BM / 4)) * 4;
        const float4 v = *reinterpret_cast<const float4*>(&part_sh[m * BM + col]);
        st_cluster_f32x4(&recv_sh[((size_t)rank * rows_max + m / z) * BM + col], (unsigned)(m % z), v);
      }
      __syncwarp();
      if (lane < z) mbar_arrive_cluster(recv_bar, (unsigned)lane);
      bool got = false;
      for (uint32_t i = 0; i < WAIT_LIMIT && !got; ++i) got = mbar_try_wait_cluster(recv_bar, 0);
      if (!got && lane == 0) atomicAdd(&g_wait_timeouts, 1);
      if (got && n < N) {
        for (int m = rank; m < M; m += z) {
          float t = b;
          for (int src = 0; src < z; ++src) t += recv_sh[((size_t)src * rows_max + m / z) * BM + n_local];
          if (EPI == EPI_GELU_TANH) t = gelu_tanh_fast(t);
          if (EPI == EPI_GELU_ERF) t = gelu_erf(t);
          const int64_t o = (int64_t)m * ldo + n;
          if (EPI == EPI_STORE_F32) reinterpret_cast<float*>(out)[o] = t;
          else if (EPI == EPI_RESIDUAL) reinterpret_cast<float*>(out)[o] += t;
          else reinterpret_cast<__nv_bfloat16*>(out)[o] = __float2bfloat16_rn(t);
        }
      }
    } else if (ok) {
      const bool atomic = gridDim.y > 1;
#pragma unroll 1
      for (int c = 0; c < MB; c += 16) {
        float v[16];
        tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c, v);
        if (n < N && c < M) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = c + j;
            if (m < M) {
              float t = v[j] + b;
              if (EPI == EPI_GELU_TANH) t = gelu_tanh_fast(t);
              if (EPI == EPI_GELU_ERF) t = gelu_erf(t);
              const int64_t o = (int64_t)m * ldo + n;
              if (EPI == EPI_STORE || EPI == EPI_GELU_TANH || EPI == EPI_GELU_ERF) {
                reinterpret_cast<__nv_bfloat16*>(out)[o] = __float2bfloat16_rn(t);
              } else if (EPI == EPI_RESIDUAL) {
                if (atomic) atomicAdd(reinterpret_cast<float*>(out) + o, t);
                else reinterpret_cast<float*>(out)[o] += t;
              } else {
                reinterpret_cast<float*>(out)[o] = t;
              }
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------
// Host side: tensor maps (made once per tensor and shape, then reused) and the launch.
// ---------------------------------------------------------------------------------------------
struct MapKey {
  const void* ptr; int64_t ld; int rows, cols, box_rows;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && ld == o.ld && rows == o.rows && cols == o.cols && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    h = h * 1000003u ^ (size_t)k.ld;
    h = h * 1000003u ^ (size_t)k.rows;
    h = h * 1000003u ^ (size_t)k.cols;
    h = h * 1000003u ^ (size_t)k.box_rows;
    return h;
  }
};

std::mutex g_map_mutex;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;

// A [rows, cols] bfloat16 matrix with row stride ld, loaded in boxes of box_rows x 64.
int tensor_map(const void* ptr, int64_t ld, int rows, int cols, int box_rows, CUtensorMap* out) {
  MapKey key{ptr, ld, rows, cols, box_rows};
  std::lock_guard<std::mutex> lock(g_map_mutex);
  auto it = g_maps.find(key);
  if (it != g_maps.end()) {
    *out = it->second;
    return KVAD_OK;
  }
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) KVAD_FAIL(KVAD_ERR_CUDA, "linear_tcgen05: the driver does not offer cuTensorMapEncodeTiled");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  CUtensorMap m;
  CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    KVAD_FAIL(KVAD_ERR_CUDA, "linear_tcgen05: cuTensorMapEncodeTiled failed (%d) for a [%d, %d] matrix with row stride %lld", (int)r, rows, cols, (long long)ld);
  if (g_maps.size() > 8192) g_maps.clear();
  g_maps.emplace(key, m);
  *out = m;
  return KVAD_OK;
}

// An output matrix [rows, cols] with row stride ld, written in boxes of 32 rows x 128 bytes.
int tensor_map_out(const void* ptr, int64_t ld, int rows, int cols, bool f32, CUtensorMap* out) {
  MapKey key{ptr, ld, rows, cols, f32 ? -32 : -64};
  std::lock_guard<std::mutex> lock(g_map_mutex);
  auto it = g_maps.find(key);
  if (it != g_maps.end()) {
    *out = it->second;
    return KVAD_OK;
  }
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) KVAD_FAIL(KVAD_ERR_CUDA, "linear_tcgen05: the driver does not offer cuTensorMapEncodeTiled");
  const int elem_bytes = f32 ? 4 : 2;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * elem_bytes};
  cuuint32_t box[2] = {(cuuint32_t)(128 / elem_bytes), 32};
  cuuint32_t elem[2] = {1, 1};
  CUtensorMap m;
  CUresult r = fn(&m, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr),
                  dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    KVAD_FAIL(KVAD_ERR_CUDA, "linear_tcgen05: cuTensorMapEncodeTiled failed (%d) for an output of [%d, %d] with row stride %lld", (int)r, rows, cols, (long long)ld);
  if (g_maps.size() > 8192) g_maps.clear();
  g_maps.emplace(key, m);
  *out = m;
  return KVAD_OK;
}

// The same matrix seen as [cols / 64][rows][64], loaded in boxes of depth x box_rows x 64 (cols a multiple of 64).
int tensor_map_3d(const void* ptr, int64_t ld, int rows, int cols, int box_rows, int depth, CUtensorMap* out) {
  MapKey key{ptr, ld, rows, cols, box_rows + (depth << 16) + (1 << 30)};
  std::lock_guard<std::mutex> lock(g_map_mutex);
  auto it = g_maps.find(key);
  if (it != g_maps.end()) {
    *out = it->second;
    return KVAD_OK;
  }
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) KVAD_FAIL(KVAD_ERR_CUDA, "linear_tcgen05: the driver does not offer cuTensorMapEncodeTiled");
  cuuint64_t dims[3] = {(cuuint64_t)BK, (cuuint64_t)rows, (cuuint64_t)(cols / BK)};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)BK * 2};
  cuuint32_t box[3] = {(cuuint32_t)BK, (cuuint32_t)box_rows, (cuuint32_t)depth};
  cuuint32_t elem[3] = {1, 1, 1};
  CUtensorMap m;
  CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    KVAD_FAIL(KVAD_ERR_CUDA, "linear_tcgen05: cuTensorMapEncodeTiled (3-D) failed (%d) for a [%d, %d] matrix with row stride %lld", (int)r, rows, cols, (long long)ld);
  if (g_maps.size() > 8192) g_maps.clear();
  g_maps.emplace(key, m);
  *out = m;
  return KVAD_OK;
}

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0, v = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0) n = v;
    else n = 148;
  }
  return n;
}

template <int BN, int EPI>
int launch(const CUtensorMap& ma, const CUtensorMap& mw, const void* bias, int bias_f32, void* out, int64_t ldo,
           int M, int N, int K, int splits, cudaStream_t stream) {
  using T = Tile<BN>;
  // out by TMA where its rules hold: a 16-byte aligned base and row stride (not the 50257-wide logits)
  constexpr bool f32_out = (EPI == EPI_RESIDUAL || EPI == EPI_STORE_F32);
  const int elem_bytes = f32_out ? 4 : 2;
  CUtensorMap mo = ma;
  int tma_out = 0;
  if (BN >= 64 && !g_no_tma_out && (ldo * elem_bytes) % 16 == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
    int rc = tensor_map_out(out, ldo, M, N, f32_out, &mo);
    if (rc != KVAD_OK) return rc;
    tma_out = 1;
  }
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(linear_tcgen05_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)T::SMEM);
    if (e != cudaSuccess) KVAD_FAIL(KVAD_ERR_CUDA, "linear_tcgen05: cannot reserve %zu bytes of shared memory: %s", T::SMEM, cudaGetErrorString(e));
    configured = true;
  }
  const int kb_total = (K + BK - 1) / BK;
  const int kb_per_split = (kb_total + splits - 1) / splits;
  const int z = (kb_total + kb_per_split - 1) / kb_per_split;
  const int64_t n_tiles = (int64_t)((N + BN - 1) / BN) * ((M + BM - 1) / BM) * z;
  KVAD_REQUIRE(n_tiles < (1ll << 30), "linear_tcgen05: %lld tiles are more than one launch takes", (long long)n_tiles);
  const int ctas = n_tiles < sm_count() ? (int)n_tiles : sm_count();      // one CTA per SM walks the tiles
  kvad_launch(linear_tcgen05_kernel<BN, EPI>, dim3(ctas), dim3(NUM_THREADS_WIDE), T::SMEM, stream, ma, mw, mo, tma_out, bias,
              bias_f32, out, ldo, M, N, K, kb_per_split, z);
  KVAD_CHECK_LAUNCH("linear_tcgen05");
  return KVAD_OK;
}

template <int BN>
int launch_epi(int epilogue, const CUtensorMap& ma, const CUtensorMap& mw, const void* bias, int bias_f32, void* out,
               int64_t ldo, int M, int N, int K, int splits, cudaStream_t stream) {
  switch (epilogue) {
    case EPI_STORE: return launch<BN, EPI_STORE>(ma, mw, bias, bias_f32, out, ldo, M, N, K, 1, stream);
    case EPI_GELU_TANH: return launch<BN, EPI_GELU_TANH>(ma, mw, bias, bias_f32, out, ldo, M, N, K, 1, stream);
    case EPI_GELU_ERF: return launch<BN, EPI_GELU_ERF>(ma, mw, bias, bias_f32, out, ldo, M, N, K, 1, stream);
    case EPI_RESIDUAL: return launch<BN, EPI_RESIDUAL>(ma, mw, bias, bias_f32, out, ldo, M, N, K, splits, stream);
    case EPI_STORE_F32: return launch<BN, EPI_STORE_F32>(ma, mw, bias, bias_f32, out, ldo, M, N, K, 1, stream);
  }
  KVAD_FAIL(KVAD_ERR_ARGUMENT, "linear_tcgen05: unknown epilogue %d", epilogue);
}

template <int MB, int EPI, int TM>
int launch_skinny(const CUtensorMap& ma, const CUtensorMap& mw, const void* bias, int bias_f32, void* out, int64_t ldo,
                  int M, int N, int K, int splits, cudaStream_t stream) {
  using T = SkinnyTile<MB, TM>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(linear_tcgen05_skinny_kernel<MB, EPI, TM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)T::SMEM);
    if (e != cudaSuccess) KVAD_FAIL(KVAD_ERR_CUDA, "linear_tcgen05: cannot reserve %zu bytes of shared memory: %s", T::SMEM, cudaGetErrorString(e));
    configured = true;
  }
  const int kb_total = (K + BK - 1) / BK;
  const int kb_per_split = (kb_total + splits - 1) / splits;
  const int z = (kb_total + kb_per_split - 1) / kb_per_split;
  dim3 grid((N + TM - 1) / TM, z);
  const int test_skip = g_test_skip_load ? 2 : 0;       // rides in a free bit of bias_f32
  g_test_skip_load = false;
  kvad_launch(linear_tcgen05_skinny_kernel<MB, EPI, TM>, grid, dim3(NUM_THREADS), T::SMEM, stream, ma, mw, bias, bias_f32 | test_skip, out, ldo, M, N, K, kb_per_split);
  KVAD_CHECK_LAUNCH("linear_tcgen05_skinny");
  return KVAD_OK;
}

template <int MB, int TM>
int launch_skinny_epi(int epilogue, const CUtensorMap& ma, const CUtensorMap& mw, const void* bias, int bias_f32,
                      void* out, int64_t ldo, int M, int N, int K, int splits, cudaStream_t stream) {
  switch (epilogue) {
    case EPI_STORE: return launch_skinny<MB, EPI_STORE, TM>(ma, mw, bias, bias_f32, out, ldo, M, N, K, 1, stream);
    case EPI_GELU_TANH: return launch_skinny<MB, EPI_GELU_TANH, TM>(ma, mw, bias, bias_f32, out, ldo, M, N, K, 1, stream);
    case EPI_GELU_ERF: return launch_skinny<MB, EPI_GELU_ERF, TM>(ma, mw, bias, bias_f32, out, ldo, M, N, K, 1, stream);
    case EPI_RESIDUAL: return launch_skinny<MB, EPI_RESIDUAL, TM>(ma, mw, bias, bias_f32, out, ldo, M, N, K, splits, stream);
    case EPI_STORE_F32: return launch_skinny<MB, EPI_STORE_F32, TM>(ma, mw, bias, bias_f32, out, ldo, M, N, K, 1, stream);
  }
  KVAD_FAIL(KVAD_ERR_ARGUMENT, "linear_tcgen05: unknown epilogue %d", epilogue);
}

template <int MB, int EPI>
int launch_skinny3d(const CUtensorMap& ma, const CUtensorMap& mw, const void* bias, int bias_f32, void* out, int64_t ldo,
                    int M, int N, int K, int kb_per_split, int z, int stages, size_t smem, cudaStream_t stream) {
  // a split of K under a storing epilogue is reduced inside a thread-block cluster (the residual epilogue adds atomically)
  const int cluster_reduce = (EPI != EPI_RESIDUAL && z > 1) ? 1 : 0;
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(linear_tcgen05_skinny3d_kernel<MB, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) KVAD_FAIL(KVAD_ERR_CUDA, "linear_tcgen05: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = smem;
  }
  if (cluster_reduce)
    kvad_launch_cluster(linear_tcgen05_skinny3d_kernel<MB, EPI>, dim3((N + BM - 1) / BM, z), dim3(NUM_THREADS), smem, stream,
                        dim3(1, z, 1), ma, mw, bias, bias_f32, out, ldo, M, N, K, kb_per_split, stages, 1);
  else
    kvad_launch(linear_tcgen05_skinny3d_kernel<MB, EPI>, dim3((N + BM - 1) / BM, z), dim3(NUM_THREADS), smem, stream, ma, mw,
                bias, bias_f32, out, ldo, M, N, K, kb_per_split, stages, 0);
  KVAD_CHECK_LAUNCH("linear_tcgen05_skinny3d");
  return KVAD_OK;
}

template <int MB>
int launch_skinny3d_epi(int epilogue, const CUtensorMap& ma, const CUtensorMap& mw, const void* bias, int bias_f32, void* out,
                        int64_t ldo, int M, int N, int K, int kb_per_split, int z, int stages, size_t smem, cudaStream_t stream) {
  switch (epilogue) {
    case EPI_STORE: return launch_skinny3d<MB, EPI_STORE>(ma, mw, bias, bias_f32, out, ldo, M, N, K, kb_per_split, z, stages, smem, stream);
    case EPI_GELU_TANH: return launch_skinny3d<MB, EPI_GELU_TANH>(ma, mw, bias, bias_f32, out, ldo, M, N, K, kb_per_split, z, stages, smem, stream);
    case EPI_GELU_ERF: return launch_skinny3d<MB, EPI_GELU_ERF>(ma, mw, bias, bias_f32, out, ldo, M, N, K, kb_per_split, z, stages, smem, stream);
    case EPI_RESIDUAL: return launch_skinny3d<MB, EPI_RESIDUAL>(ma, mw, bias, bias_f32, out, ldo, M, N, K, kb_per_split, z, stages, smem, stream);
    case EPI_STORE_F32: return launch_skinny3d<MB, EPI_STORE_F32>(ma, mw, bias, bias_f32, out, ldo, M, N, K, kb_per_split, z, stages, smem, stream);
  }
  KVAD_FAIL(KVAD_ERR_ARGUMENT, "linear_tcgen05: unknown epilogue %d", epilogue);
}

}  // namespace

// `force` fixes what the kernel otherwise chooses (tests): bits 0-15 the tile width of the wide
// form (16, 32, 64, 128, 192 or 256); bits 16-23 how many CTAs share K (residual epilogue only);
// bits 24-25 the form: 1 wide (activation rows on the M side), 2 swapped (at most 64 rows; the
// tile width then means weight rows per CTA, 64 or 128).
KVAD_EXPORT int kvad_linear_tcgen05(const void* A, int64_t lda, const void* W, const void* bias, int bias_f32,
                                    void* out, int64_t ldo, int M, int N, int K, int epilogue, int force,
                                    cudaStream_t stream) {
  KVAD_REQUIRE(M >= 0 && N > 0 && K > 0, "linear_tcgen05: bad sizes M=%d N=%d K=%d", M, N, K);
  if (K % 8 != 0 || lda % 8 != 0)
    KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "linear_tcgen05: K=%d and the row stride %lld must be multiples of 8 (TMA strides are multiples of 16 bytes)", K, (long long)lda);
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(W) & 15))
    KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "linear_tcgen05: operands must start on 16-byte boundaries");
  KVAD_REQUIRE(lda >= K && ldo >= N, "linear_tcgen05: leading dimensions lda=%lld ldo=%lld too small", (long long)lda, (long long)ldo);
  KVAD_REQUIRE((M + BM - 1) / BM <= 65535, "linear_tcgen05: M=%d is more rows than one launch takes", M);
  if (M == 0) return KVAD_OK;

  const int force_bn = force & 0xffff, force_splits = (force >> 16) & 0xff, force_path = (force >> 24) & 3;
  KVAD_REQUIRE(force_path != 2 || M <= 64, "linear_tcgen05: the swapped form takes at most 64 rows, not %d", M);
  // Up to 16 rows the swapped form always; up to 64 rows too, except where its epilogue, which grows with the
  // rows (every thread stores a column of the transposed output, two bytes at a time), costs more than the wide
  // form's fixed tile: measured on a B200 at K = 768 and 3072, the wide form with 64-wide tiles takes the same
  // time from 17 to 64 rows (out-projection 2.9 us, up-projection 6.2 us, down-projection 4.4 us), the swapped
  // form 3.1 -> 4.7, 5.7 -> 7.5 and 4.0 -> 5.6 us from 24 to 64 rows.  The choice depends on the row count's
  // class and the epilogue only.
  bool swapped = (M <= 64 && force_path != 1 && force_bn == 0) || force_path == 2;
  if (swapped && force_path == 0 && M > 16) {
    const bool gelu = epilogue == EPI_GELU_TANH || epilogue == EPI_GELU_ERF;
    if ((epilogue == EPI_RESIDUAL && M >= 24) || (gelu && M >= 48)) swapped = false;
  }
  if (swapped) {
    // few rows: weights on the M side of the MMA, 64 rows a CTA unless that makes more CTAs than SMs
    const int mb = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    const int kb_all = (K + BK - 1) / BK;
    int tm = ((N + BM - 1) / BM < 74) ? 64 : 128;
    if (force_bn == 64 || force_bn == 128) tm = force_bn;
    const int tiles = (N + tm - 1) / tm;
    int sp = 1;
    if (epilogue == EPI_RESIDUAL) {
      sp = force_splits > 0 ? force_splits : (148 + tiles - 1) / tiles;
      if (sp > 16) sp = 16;
      if (sp > kb_all) sp = kb_all;
      if (sp < 1) sp = 1;
    }
    if (K % BK == 0 && force_bn == 0 && !g_no_3d && (mb == 16 || g_force_3d)) {
      // (with more activation rows their resident copy leaves room for one stage of weights only,
      // and the form above, which pipelines block by block, is the faster one: measured at 64 rows)
      // K in whole blocks of 64: few, large, three-dimensional TMA loads
      const int tiles128 = (N + BM - 1) / BM;
      // How many CTAs share K.  Measured at GPT-2 XL's sizes and 8 rows, launches back to back in one graph: with K
      // split until a CTA's share is ONE group of K blocks (W_GROUP of them, 64 KB of weights) a residual product
      // of 4800 x 1600 takes 4.2 us, with two groups a CTA (K in four, one wave of CTAs) 6.5 us; the q/k/v product,
      // whose splits are a cluster, 8.5 against 9.4 us.  Short CTAs, more of them than SMs: an SM takes up its next
      // CTA - of this launch or, under dependent launch, of the next - as soon as one leaves, so somewhere weights
      // are always on their way; a CTA with two or three groups in its ring holds its SM through two or three trips
      // to memory.  KVAD_MAX_SPLIT_CTAS bounds the grid.
      int sp3 = 1;
      const int one_group = (kb_all + W_GROUP - 1) / W_GROUP;     // the split that leaves every CTA one group
      if (epilogue == EPI_RESIDUAL) {
        sp3 = (148 + tiles128 - 1) / tiles128;
        if (sp3 < one_group) sp3 = one_group;
        if (sp3 > 32) sp3 = 32;
        while (sp3 > 1 && tiles128 * sp3 > KVAD_MAX_SPLIT_CTAS) --sp3;
        if (force_splits > 0) sp3 = force_splits > 32 ? 32 : force_splits;
        if (sp3 > kb_all) sp3 = kb_all;
        if (sp3 < 1) sp3 = 1;
      } else if (!g_no_cluster_k) {
        // storing epilogues: K over a cluster of CTAs (8 at most); measured at 8 rows and K = 768: 4.3 us whole,
        // 4.3 in two, 3.8 in four, 3.8..4.1 in six
        // (a cluster costs: at K = 512 and 118 tiles a split in three took 8.8 us against 4.8 whole - so K is split
        // in four while that stays one wave of CTAs, and further only to reach one group a CTA)
        sp3 = kb_all >= 8 ? 4 : 1;
        while (sp3 > 1 && tiles128 * sp3 > 160) --sp3;
        if (one_group > 4) {
          const int finer = one_group > 8 ? 8 : one_group;
          if (tiles128 * finer <= KVAD_MAX_SPLIT_CTAS) sp3 = finer;
        }
        if (force_splits > 0) sp3 = force_splits > 8 ? 8 : force_splits;
        if (sp3 > kb_all) sp3 = kb_all;
      }
      const int kb_per_split = (kb_all + sp3 - 1) / sp3;
      const int z = (kb_all + kb_per_split - 1) / kb_per_split;
      const size_t a_bytes = (size_t)kb_per_split * mb * BK * 2;
      const size_t stage_bytes = (size_t)W_GROUP * BM * BK * 2;
      const int groups = (kb_per_split + W_GROUP - 1) / W_GROUP;
      const size_t recv_bytes = (size_t)(2 * mb + 8) * BM * 4 + 16;  // partial sums received from the cluster's CTAs, and this CTA's own
      if (a_bytes + stage_bytes + 2048 + recv_bytes <= (size_t)SMEM_BUDGET && kb_per_split <= 256) {
        int stages3 = (int)(((size_t)SMEM_BUDGET - a_bytes - 2048 - recv_bytes) / stage_bytes);
        if (stages3 > groups) stages3 = groups;
        if (stages3 > 3) stages3 = 3;
        const size_t smem3 = a_bytes + (size_t)stages3 * stage_bytes + (2 * stages3 + 2) * 8 + 16 + 16 + recv_bytes + 1024;
        CUtensorMap ma3, mw3;
        int rc3 = tensor_map_3d(A, lda, M, K, mb, kb_per_split, &ma3);
        if (rc3 != KVAD_OK) return rc3;
        rc3 = tensor_map_3d(W, K, N, K, BM, W_GROUP, &mw3);
        if (rc3 != KVAD_OK) return rc3;
        switch (mb) {
          case 16: return launch_skinny3d_epi<16>(epilogue, ma3, mw3, bias, bias_f32, out, ldo, M, N, K, kb_per_split, z, stages3, smem3, stream);
          case 32: return launch_skinny3d_epi<32>(epilogue, ma3, mw3, bias, bias_f32, out, ldo, M, N, K, kb_per_split, z, stages3, smem3, stream);
          default: return launch_skinny3d_epi<64>(epilogue, ma3, mw3, bias, bias_f32, out, ldo, M, N, K, kb_per_split, z, stages3, smem3, stream);
        }
      }
    }
    CUtensorMap ma, mw;
    int rc = tensor_map(A, lda, M, K, mb, &ma);
    if (rc != KVAD_OK) return rc;
    rc = tensor_map(W, K, N, K, tm, &mw);
    if (rc != KVAD_OK) return rc;
#define KVAD_SKINNY(MBV, TMV) return launch_skinny_epi<MBV, TMV>(epilogue, ma, mw, bias, bias_f32, out, ldo, M, N, K, sp, stream)
    if (tm == 64) {
      switch (mb) {
        case 16: KVAD_SKINNY(16, 64);
        case 32: KVAD_SKINNY(32, 64);
        default: KVAD_SKINNY(64, 64);
      }
    }
    switch (mb) {
      case 16: KVAD_SKINNY(16, 128);
      case 32: KVAD_SKINNY(32, 128);
      default: KVAD_SKINNY(64, 128);
    }
#undef KVAD_SKINNY
  }
  // Tile width and K split by a small cost model fitted to measurements on a B200: a CTA pays a fixed
  // cost (set-up, filling the pipeline, the epilogue: larger for wider tiles) plus about 0.27 us per
  // 64-wide block of K whatever the tile's width (the ring of stages is bound by the latency of its
  // round trip, so a wide tile gets its extra work for free), and the grid runs in waves of 148 CTAs.
  const int m_tiles = (M + BM - 1) / BM;
  const int kb_total = (K + BK - 1) / BK;
  int bn = force_bn, splits = 1;
  {
    // (a kernel that allocates tensor memory has one CTA per SM, so a wave is 148 CTAs whatever their size)
    const int widths[6] = {256, 192, 128, 64, 32, 16};
    const float fixed_us[6] = {7.0f, 5.5f, 4.0f, 3.0f, 3.4f, 3.6f};      // (narrower than 64 buys nothing: measured)
    float best = 1e30f;
    for (int i = 0; i < 6; ++i) {
      if (force_bn != 0 && widths[i] != force_bn) continue;
      const int64_t tiles = (int64_t)m_tiles * ((N + widths[i] - 1) / widths[i]);
      for (int sp = 1; sp <= 8; ++sp) {
        if (sp > 1 && (epilogue != EPI_RESIDUAL || kb_total / sp < 2)) break;
        if (force_splits > 0 && sp != 1) break;
        const int64_t waves = (tiles * sp + 147) / 148;
        const float t = (float)waves * ((float)((kb_total + sp - 1) / sp) * 0.27f + fixed_us[i]);
        if (t < best) { best = t; bn = widths[i]; splits = sp; }
      }
    }
  }
  KVAD_REQUIRE(bn == 16 || bn == 32 || bn == 64 || bn == 128 || bn == 192 || bn == 256,
               "linear_tcgen05: tile width %d is not one of 16, 32, 64, 128, 192, 256", bn);
  if (epilogue == EPI_RESIDUAL && force_splits > 0) splits = force_splits;
  if (splits > kb_total) splits = kb_total;
  if (splits < 1) splits = 1;

  CUtensorMap ma, mw;
  int rc = tensor_map(A, lda, M, K, BM, &ma);
  if (rc != KVAD_OK) return rc;
  rc = tensor_map(W, K, N, K, bn, &mw);
  if (rc != KVAD_OK) return rc;

  switch (bn) {
    case 16: return launch_epi<16>(epilogue, ma, mw, bias, bias_f32, out, ldo, M, N, K, splits, stream);
    case 32: return launch_epi<32>(epilogue, ma, mw, bias, bias_f32, out, ldo, M, N, K, splits, stream);
    case 64: return launch_epi<64>(epilogue, ma, mw, bias, bias_f32, out, ldo, M, N, K, splits, stream);
    case 128: return launch_epi<128>(epilogue, ma, mw, bias, bias_f32, out, ldo, M, N, K, splits, stream);
    case 192: return launch_epi<192>(epilogue, ma, mw, bias, bias_f32, out, ldo, M, N, K, splits, stream);
    default: return launch_epi<256>(epilogue, ma, mw, bias, bias_f32, out, ldo, M, N, K, splits, stream);
  }
}

// Tests: 1 keeps the swapped form on two-dimensional loads (one per K block) for every K; 2 takes the
// grouped three-dimensional loads whenever K allows; 0 is the kernel's own choice (them, up to 16 rows).
KVAD_EXPORT void kvad_linear_tcgen05_no_3d(int on) { g_no_3d = on == 1; g_force_3d = on == 2; }

// Tests of the bounded waits: `wait_limit` > 0 sets how many polls a wait makes before it gives up (0: the
// library's own limit); `skip_first_load` makes the NEXT launch of the swapped form with one load per K block
// leave out its first load, so that the wait for it runs out: the launch raises the status counter, writes
// an output that means nothing, frees its tensor memory and returns; launches after it are ordinary.
KVAD_EXPORT int kvad_linear_tcgen05_test_hooks(unsigned wait_limit, int skip_first_load) {
  const uint32_t limit = wait_limit > 0 ? wait_limit : WAIT_LIMIT;
  cudaError_t e = cudaMemcpyToSymbol(g_wait_limit, &limit, sizeof(limit));
  if (e != cudaSuccess) KVAD_FAIL(KVAD_ERR_CUDA, "linear_tcgen05: cannot set the wait limit: %s", cudaGetErrorString(e));
  g_test_skip_load = skip_first_load != 0;
  return KVAD_OK;
}

// Tests: 1 makes the wide form write its output with plain stores instead of TMA stores / reduce-adds.
KVAD_EXPORT void kvad_linear_tcgen05_no_tma_out(int on) { g_no_tma_out = on != 0; }

// Tests: 1 keeps K whole under the storing epilogues of the swapped form (no cluster reduction).
KVAD_EXPORT void kvad_linear_tcgen05_no_cluster_k(int on) { g_no_cluster_k = on != 0; }

// How many bounded waits have run out since the library was loaded (0 in a healthy run).
// Synchronises the device.
KVAD_EXPORT int kvad_linear_tcgen05_status() {
  int n = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&n, g_wait_timeouts, sizeof(int));
  if (e != cudaSuccess) KVAD_FAIL(KVAD_ERR_CUDA, "linear_tcgen05_status: %s", cudaGetErrorString(e));
  return n;
}

KVAD_DEFINE_LAST_ERROR()
