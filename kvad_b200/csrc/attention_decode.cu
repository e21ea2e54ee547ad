// Attention of single-token rows over the paged cache (decoding), split over the keys.
//
// A decode step is a stream of cached keys and values: every (sequence, head)
// reads its whole history once and does two flops per element, so the kernel
// is built to keep many bytes in flight.  The keys of one (row, head) are cut
// into `n_splits` contiguous ranges; a CTA of four warps serves one (split,
// head, row), each warp walking chunks of 32 keys with a running maximum, sum
// and output of its own (a lane per key for the scores, 16-byte loads; HD/8
// lanes per key for the values) and the warps meeting once at the end.  With
// more than one split the CTA leaves an unnormalised partial result, its
// maximum and its sum in scratch memory; the CTA that finishes last merges
// them (or a second, tiny kernel does).  The step's own key and value can be
// taken straight from the projection's output and written to the cache here -
// or, in bfloat16, from 32-bit sums that a projection whose CTAs add their shares
// of K has left without bias (PreQkv below: bias, rounding and the cache write
// happen where the kernel reads them).
// All arithmetic is 32-bit; the order of operations for a row depends on the
// number of splits and on nothing else in the batch.
//
// Query head h reads key/value head h / (n_heads / n_kv_heads); `window` > 0
// limits a row to its latest positions.  Head sizes: multiples of 16 up to 128,
// and 256; others are refused (the caller falls back to the general kernel).
//
// bisand/kvad: attend(), crates/llm/src/model/mod.rs:769-819.
#include <type_traits>

#include "common.cuh"
#include "attention_decode_noalloc.h"

using namespace kvad;

namespace {

constexpr int DEC_THREADS = 128;
constexpr int DEC_WARPS = DEC_THREADS / 32;

template <typename T> struct Vec8;
template <> struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* f) {
    const uint4 q = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 v = __bfloat1622float2(h[i]);
      f[2 * i] = v.x;
      f[2 * i + 1] = v.y;
    }
  }
};
template <> struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float* f) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
};

// exp in the accuracy the element type deserves: the fast form for bfloat16 data, the exact one for 32-bit.
template <typename T> __device__ __forceinline__ float exp_for(float x);
template <> __device__ __forceinline__ float exp_for<__nv_bfloat16>(float x) { return __expf(x); }
template <> __device__ __forceinline__ float exp_for<float>(float x) { return expf(x); }

// Merges the partial results (unnormalised output, maximum, sum) of the splits of one (row, head).
template <typename T, int HD>
__device__ __forceinline__ void merge_partials(const float* part, T* dst, int n_splits,
                                               int tid, int n_threads) {
  // other CTAs of this launch may have written the partials: read them past the L1 cache
  float m = -INFINITY;
  for (int s = 0; s < n_splits; ++s) m = fmaxf(m, __ldcg(part + s * (HD + 2) + HD));
  float total = 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const float ms = __ldcg(part + s * (HD + 2) + HD);
    if (ms != -INFINITY) total += __ldcg(part + s * (HD + 2) + HD + 1) * exp_for<T>(ms - m);
  }
  for (int d = tid; d < HD; d += n_threads) {
    float o = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float ms = __ldcg(part + s * (HD + 2) + HD);
      if (ms != -INFINITY) o += __ldcg(part + s * (HD + 2) + d) * exp_for<T>(ms - m);
    }
    dst[d] = from_f32<T>(o / total);
  }
}

// One CTA = one (split, head, row).  Its four warps walk the split's keys in chunks of 32, each warp
// with a running maximum, sum and output of its own, and meet once at the end: no block-wide barrier
// stands inside the walk, so every lane has 16-byte loads of a whole chunk in flight.  Scoring: a lane
// per key.  Values: HD/8 lanes per key, 8 dimensions each, the key's weight handed round by shuffle.
//
// k_new / v_new (optional): this step's keys and values of the rows, [row, kv_head * HD], as the
// projection left them.  The key at the row's own position is then read from there, not from the
// cache, and the CTAs of split 0 write it to the cache - the step needs no separate store kernel.
// counters (optional, one int per (row, head), zero before the first launch): the CTA that finishes
// last merges the splits itself and puts the counter back to zero; without counters a second kernel merges.
template <typename T, int HD>
__global__ void __launch_bounds__(DEC_THREADS)
attention_decode_kernel(const T* __restrict__ q, int64_t ld_q, T* __restrict__ out, int64_t ld_out,
                        const int* __restrict__ row_seq, const int* __restrict__ row_pos,
                        const int* __restrict__ page_table, int table_width,
                        T* __restrict__ k_pages, T* __restrict__ v_pages,
                        const T* __restrict__ k_new, const T* __restrict__ v_new, int64_t ld_new,
                        float* __restrict__ scratch, int* __restrict__ counters,
                        int n_heads, int n_kv_heads, int page_size, int n_splits, float scale, int window) {
  constexpr int CH = HD / 8;                    // lanes that share one value row (8 dimensions each)
  constexpr int RPI = 32 / CH;                  // value rows a warp takes per pass
  constexpr int PASSES = (32 + RPI - 1) / RPI;
  __shared__ __align__(16) float qs[HD];
  __shared__ __align__(16) float acc_sh[DEC_WARPS][RPI][HD];
  __shared__ float ml_sh[DEC_WARPS][2];
  __shared__ int last_flag;

  pdl_launch_dependents();
  pdl_wait();
  const int split = blockIdx.x, h = blockIdx.y, r = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int group = n_heads / n_kv_heads;
  const int kvh = h / group;
  const int pos = row_pos[r];
  const int* pages = page_table + (int64_t)row_seq[r] * table_width;
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int n_keys = pos - lo + 1;
  int per = (n_keys + n_splits - 1) / n_splits;
  per = (per + 63) / 64 * 64;
  const int t_begin = lo + split * per;
  const int t_end = (t_begin + per < pos + 1) ? t_begin + per : pos + 1;
  const T* k_row_new = k_new ? k_new + (int64_t)r * ld_new + (int64_t)kvh * HD : nullptr;
  const T* v_row_new = v_new ? v_new + (int64_t)r * ld_new + (int64_t)kvh * HD : nullptr;

  for (int d = tid; d < HD; d += DEC_THREADS) qs[d] = to_f32(q[(int64_t)r * ld_q + (int64_t)h * HD + d]);
  if (k_row_new != nullptr && split == 0 && h % group == 0 && tid < 2 * CH) {
    // this step's key and value go to their place in the cache (nobody reads that place in this launch)
    const int page = pages[pos / page_size];
    const int64_t dst = (((int64_t)page * n_kv_heads + kvh) * page_size + pos % page_size) * HD;
    const int c = tid % CH;
    const T* src = (tid < CH ? k_row_new : v_row_new) + c * 8;
    T* to = (tid < CH ? k_pages : v_pages) + dst + c * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) to[i] = src[i];
  }
  __syncthreads();

  const int vrow = lane / CH, vc = lane % CH;   // this lane's place in the value passes
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  float run_max = -INFINITY, run_sum = 0.f;

  for (int t0 = t_begin + warp * 32; t0 < t_end; t0 += DEC_WARPS * 32) {
    // ---- a key per lane: score
    const int t = t0 + lane;
    float s = -INFINITY;
    if (t < t_end) {
      const T* kr;
      if (k_row_new != nullptr && t == pos) {
        kr = k_row_new;
      } else {
        const int page = pages[t / page_size];
        kr = k_pages + (((int64_t)page * n_kv_heads + kvh) * page_size + t % page_size) * HD;
      }
      float dot = 0.f;
#pragma unroll
      for (int j = 0; j < CH; ++j) {
        float f[8];
        Vec8<T>::load(kr + j * 8, f);
#pragma unroll
        for (int i = 0; i < 8; ++i) dot = fmaf(qs[j * 8 + i], f[i], dot);
      }
      s = dot * scale;
    }
    const float new_max = fmaxf(run_max, warp_max(s));          // the chunk has at least one key
    const float keep = (run_max == -INFINITY) ? 0.f : exp_for<T>(run_max - new_max);
    const float p = (t < t_end) ? exp_for<T>(s - new_max) : 0.f;
    run_sum = run_sum * keep + warp_sum(p);
    run_max = new_max;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] *= keep;

    // ---- values: CH lanes per key, RPI keys per pass
#pragma unroll
    for (int pass = 0; pass < PASSES; ++pass) {
      const int key = pass * RPI + vrow;                         // within the chunk
      const float w = __shfl_sync(0xffffffffu, p, key < 32 ? key : 0);
      const int tj = t0 + key;
      if (vrow < RPI && key < 32 && tj < t_end) {
        const T* vr;
        if (v_row_new != nullptr && tj == pos) {
          vr = v_row_new + vc * 8;
        } else {
          const int page = pages[tj / page_size];
          vr = v_pages + (((int64_t)page * n_kv_heads + kvh) * page_size + tj % page_size) * HD + vc * 8;
        }
        float f[8];
        Vec8<T>::load(vr, f);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = fmaf(w, f[i], acc[i]);
      }
    }
  }

  // ---- the warps meet
  if (vrow < RPI) {
#pragma unroll
    for (int i = 0; i < 8; ++i) acc_sh[warp][vrow][vc * 8 + i] = acc[i];
  }
  if (lane == 0) {
    ml_sh[warp][0] = run_max;
    ml_sh[warp][1] = run_sum;
  }
  __syncthreads();
  float m = -INFINITY;
#pragma unroll
  for (int w = 0; w < DEC_WARPS; ++w) m = fmaxf(m, ml_sh[w][0]);
  float total = 0.f, wscale[DEC_WARPS];
#pragma unroll
  for (int w = 0; w < DEC_WARPS; ++w) {
    wscale[w] = (ml_sh[w][0] == -INFINITY) ? 0.f : exp_for<T>(ml_sh[w][0] - m);
    total += ml_sh[w][1] * wscale[w];
  }
  float* part = n_splits > 1 ? scratch + (((int64_t)r * n_heads + h) * n_splits + split) * (HD + 2) : nullptr;
  for (int d = tid; d < HD; d += DEC_THREADS) {
    float o = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      float ow = 0.f;
#pragma unroll
      for (int g = 0; g < RPI; ++g) ow += acc_sh[w][g][d];
      o += ow * wscale[w];
    }
    if (n_splits == 1) {
      out[(int64_t)r * ld_out + (int64_t)h * HD + d] = from_f32<T>(o / total);
    } else {
      part[d] = o;
    }
  }
  if (n_splits > 1) {
    if (tid == 0) {
      part[HD] = m;
      part[HD + 1] = total;
    }
    if (counters != nullptr) {
      __threadfence();
      __syncthreads();
      if (tid == 0) {
        const int done = atomicAdd(&counters[r * n_heads + h], 1);
        last_flag = (done == n_splits - 1);
        if (last_flag) counters[r * n_heads + h] = 0;            // ready for the next launch
      }
      __syncthreads();
      if (last_flag) {
        __threadfence();
        merge_partials<T, HD>(scratch + ((int64_t)r * n_heads + h) * n_splits * (HD + 2),
                              out + (int64_t)r * ld_out + (int64_t)h * HD, n_splits, tid, DEC_THREADS);
      }
    }
  }
}

// The merge as a kernel of its own (when no counters are given).
template <typename T, int HD>
__global__ void attention_decode_merge_kernel(const float* __restrict__ scratch, T* __restrict__ out, int64_t ld_out,
                                              int n_heads, int n_splits) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, h = blockIdx.y;
  merge_partials<T, HD>(scratch + ((int64_t)r * n_heads + h) * n_splits * (HD + 2),
                        out + (int64_t)r * ld_out + (int64_t)h * HD, n_splits, threadIdx.x, blockDim.x);
}

// ---------------------------------------------------------------------------------------------
// The same work fed by the TMA engine (head sizes whose rows split evenly over a warp: 16, 32, 64,
// 128, 256).  One page of one head is one contiguous tile of keys and one of values; a producer warp
// streams them into a ring of shared-memory stages with cp.async.bulk, each stage signalling an
// mbarrier, so that the bytes in flight do not depend on registers or on how many warps are
// resident.  Four consumer warps take 16 keys of every tile each: HD/8 lanes per key both for the
// score (partial dots met by shuffles) and for the value sum, so a lane keeps the weight of its own
// key and nothing is handed round.  Pages of earlier steps do not depend on the kernel before this
// one, so their first stages are requested before the dependent-launch wait.
// Every wait is bounded; one that runs out raises g_decode_timeouts and the CTA runs on to its end.
// ---------------------------------------------------------------------------------------------
// The rows' queries, keys and values may come as 32-bit SUMS WITHOUT THEIR BIAS, [rows, q | k | v]: what a q/k/v
// product leaves that splits K over CTAs and adds the shares atomically into a zeroed buffer (no cluster, no second
// pass).  The kernel then adds the bias and rounds to the element type where it reads them, and every CTA also clears
// its share of another buffer (`zero`: the one the NEXT such product adds into; nothing reads it meanwhile).
struct PreQkv {
  const float* sums;        // null: queries, keys and values come in the element type (q, k_new, v_new)
  long long ld;
  const void* bias;         // [q | k | v] or null
  int bias_f32;
  int k_off, v_off;         // columns at which keys and values start
  float* zero;
  long long zero_floats;
};
PreQkv g_pre = {nullptr, 0, nullptr, 0, 0, 0, nullptr, 0};     // for the next launch (kvad_attention_decode_pre)
template <typename T>
__device__ __forceinline__ void pre_piece(const PreQkv& pre, int r, int col, float* f) {
  const float* p = pre.sums + (long long)r * pre.ld + col;
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    if (pre.bias != nullptr) f[i] += load_param(pre.bias, col + i, pre.bias_f32);
    f[i] = to_f32(from_f32<T>(f[i]));
  }
}

bool g_no_cluster = false;       // tests: merge the splits through global memory even where a cluster could
bool g_force_plain = false;      // tests: keep every head size on the kernel that loads through registers
constexpr int TMA_CONSUMER_WARPS = 4;
constexpr int TMA_THREADS = (TMA_CONSUMER_WARPS + 1) * 32;
constexpr int TILE_KEYS = 64;
constexpr uint32_t DEC_WAIT_LIMIT = 1u << 24;
__device__ int g_decode_timeouts = 0;

__device__ __forceinline__ uint32_t dec_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void dec_mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(dec_smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void dec_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(dec_smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void dec_mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(dec_smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool dec_mbar_wait(uint64_t* bar, uint32_t parity) {
  for (uint32_t i = 0; i < DEC_WAIT_LIMIT; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(dec_smem_u32(bar)), "r"(parity) : "memory");
    if (ok) return true;
  }
  atomicAdd(&g_decode_timeouts, 1);
  return false;
}
__device__ __forceinline__ void dec_bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dec_smem_u32(dst)), "l"(src), "r"(bytes), "r"(dec_smem_u32(bar)) : "memory");
}

template <typename T, int HD> struct DecTile {
  static constexpr int TILE_BYTES = TILE_KEYS * HD * (int)sizeof(T);     // keys (or values) of one page and head
  static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  static constexpr int STAGES_RAW = 65536 / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 4 ? 4 : (STAGES_RAW < 2 ? 2 : STAGES_RAW);     // the most a launch uses
  static constexpr size_t smem(int stages) { return (size_t)stages * STAGE_BYTES + 2 * stages * 8 + 128; }
  static constexpr size_t SMEM = smem(STAGES);
};

template <typename T, int HD, int STAGES, bool PRE>      // PRE: queries, keys and values come as PreQkv's sums
__global__ void __launch_bounds__(TMA_THREADS)
attention_decode_tma_kernel(const T* __restrict__ q, int64_t ld_q, T* __restrict__ out, int64_t ld_out,
                            const int* __restrict__ row_seq, const int* __restrict__ row_pos,
                            const int* __restrict__ page_table, int table_width,
                            T* __restrict__ k_pages, T* __restrict__ v_pages,
                            const T* __restrict__ k_new, const T* __restrict__ v_new, int64_t ld_new,
                            float* __restrict__ scratch, int* __restrict__ counters,
                            int n_heads, int n_kv_heads, int n_splits, float scale, int window, int cluster_merge,
                            const PreQkv pre) {
  using D = DecTile<T, HD>;
  constexpr int CH = HD / 8;                       // lanes per key
  constexpr int KPP = 32 / CH;                     // keys a warp takes per pass
  constexpr int WARP_KEYS = TILE_KEYS / TMA_CONSUMER_WARPS;
  constexpr int PASSES = (WARP_KEYS + KPP - 1) / KPP;
  extern __shared__ unsigned char dec_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(dec_raw) + 127) & ~(uintptr_t)127);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(base + (size_t)STAGES * D::STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  __shared__ __align__(16) float acc_sh[TMA_CONSUMER_WARPS][HD];
  __shared__ __align__(16) float recv_sh[8][HD + 4];         // cluster merge: the other splits' partial results arrive here
  __shared__ uint64_t merge_bar;
  __shared__ float ml_sh[TMA_CONSUMER_WARPS][2];
  __shared__ int last_flag;

  pdl_launch_dependents();
  const int split = blockIdx.x, h = blockIdx.y, r = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int group = n_heads / n_kv_heads;
  const int kvh = h / group;
  const int pos = row_pos[r];                      // uploaded by the host before the step's first kernel
  const int* pages = page_table + (int64_t)row_seq[r] * table_width;
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int n_keys = pos - lo + 1;
  int per = (n_keys + n_splits - 1) / n_splits;
  per = (per + 63) / 64 * 64;
  const int t_begin = lo + split * per;
  const int t_end = (t_begin + per < pos + 1) ? t_begin + per : pos + 1;
  const int j0 = t_begin / TILE_KEYS;
  const int n_tiles = t_end > t_begin ? (t_end - 1) / TILE_KEYS - j0 + 1 : 0;
  const T* k_row_new = k_new ? k_new + (int64_t)r * ld_new + (int64_t)kvh * HD : nullptr;
  const T* v_row_new = v_new ? v_new + (int64_t)r * ld_new + (int64_t)kvh * HD : nullptr;
  const bool has_new = PRE || k_row_new != nullptr;      // the step's own key and value are handed in

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      dec_mbar_init(&full_bar[s], 1);
      dec_mbar_init(&empty_bar[s], TMA_CONSUMER_WARPS);
    }
    dec_mbar_init(&merge_bar, n_splits > 1 ? n_splits - 1 : 1);     // the other splits' CTAs arrive here (cluster merge)
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();
  // (cluster merge: every thread of the cluster arrives at its barrier now; the CTAs that later write into the
  // first one's shared memory wait on it just before they do, by when its merge barrier is known to be initialised)
  if (n_splits > 1 && cluster_merge) cluster_arrive();

  const int c = lane % CH, kl = lane / CH;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  float run_max = -INFINITY, run_sum = 0.f;

  if (warp == TMA_CONSUMER_WARPS) {
    // ---- producer
    auto issue = [&](int i) {
      const int s = i % STAGES;
      const int page = pages[j0 + i];
      const T* kt = k_pages + ((int64_t)page * n_kv_heads + kvh) * TILE_KEYS * HD;
      const T* vt = v_pages + ((int64_t)page * n_kv_heads + kvh) * TILE_KEYS * HD;
      unsigned char* dst = base + (size_t)s * D::STAGE_BYTES;
      dec_mbar_expect_tx(&full_bar[s], D::STAGE_BYTES);
      dec_bulk_load(dst, kt, D::TILE_BYTES, &full_bar[s]);
      dec_bulk_load(dst + D::TILE_BYTES, vt, D::TILE_BYTES, &full_bar[s]);
    };
    // with the step's own key handed in, nothing read from the pages depends on the kernel before
    const int ahead = has_new ? (n_tiles < STAGES ? n_tiles : STAGES) : 0;
    if (lane == 0)
      for (int i = 0; i < ahead; ++i) issue(i);
    pdl_wait();
    if (has_new && split == 0 && h % group == 0) {
      // this step's key and value go to their place in the cache (no CTA of this launch reads that place)
      const int page = pages[pos / TILE_KEYS];
      const int64_t dst = (((int64_t)page * n_kv_heads + kvh) * TILE_KEYS + pos % TILE_KEYS) * HD;
      for (int idx = lane; idx < 2 * CH; idx += 32) {
        const int cc = idx % CH;
        T* to = (idx < CH ? k_pages : v_pages) + dst + cc * 8;
        if (PRE) {
          float f[8];
          pre_piece<T>(pre, r, (idx < CH ? pre.k_off : pre.v_off) + kvh * HD + cc * 8, f);
#pragma unroll
          for (int i = 0; i < 8; ++i) to[i] = from_f32<T>(f[i]);
        } else {
          const T* src = (idx < CH ? k_row_new : v_row_new) + cc * 8;
#pragma unroll
          for (int i = 0; i < 8; ++i) to[i] = src[i];
        }
      }
    }
    if (lane == 0) {
      for (int i = ahead; i < n_tiles; ++i) {
        const int s = i % STAGES;
        if (i >= STAGES && !dec_mbar_wait(&empty_bar[s], ((i / STAGES) & 1) ^ 1)) break;
        issue(i);
      }
    }
  } else {
    // ---- consumers
    pdl_wait();
    if (PRE && pre.zero != nullptr) {
      const long long n_ctas = (long long)gridDim.x * gridDim.y * gridDim.z;
      const long long cta = ((long long)blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
      for (long long i = cta * (TMA_CONSUMER_WARPS * 32) + tid; i < pre.zero_floats; i += n_ctas * (TMA_CONSUMER_WARPS * 32)) pre.zero[i] = 0.f;
    }
    float qreg[8];
    if (PRE) {
      pre_piece<T>(pre, r, h * HD + c * 8, qreg);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) qreg[i] = to_f32(q[(int64_t)r * ld_q + (int64_t)h * HD + c * 8 + i]);
    }
    // the step's own key and value, where they are handed in, replace what the page holds at the row's
    // position; they are fetched once, and chosen by a select where the loops below meet that position
    float k_own[8], v_own[8];
    const bool own = has_new && pos >= t_begin && pos < t_end;
    if (own && PRE) {
      pre_piece<T>(pre, r, pre.k_off + kvh * HD + c * 8, k_own);
      pre_piece<T>(pre, r, pre.v_off + kvh * HD + c * 8, v_own);
    } else if (own) {
      Vec8<T>::load(k_row_new + c * 8, k_own);
      Vec8<T>::load(v_row_new + c * 8, v_own);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) k_own[e] = v_own[e] = 0.f;
    }
    for (int i = 0; i < n_tiles; ++i) {
      const int s = i % STAGES;
      if (!dec_mbar_wait(&full_bar[s], (i / STAGES) & 1)) break;
      const T* Kt = reinterpret_cast<const T*>(base + (size_t)s * D::STAGE_BYTES);
      const T* Vt = reinterpret_cast<const T*>(base + (size_t)s * D::STAGE_BYTES + D::TILE_BYTES);
      const int tile_key0 = (j0 + i) * TILE_KEYS;
      // A page whose keys are all in this CTA's range and none of which is the step's own (all pages but the
      // first and last of a range, usually) takes the same code without the per-key tests and selects.
      float keep = 0.f, new_max = run_max, chunk_sum = 0.f;
      auto take_page = [&](auto whole_tag) {
        constexpr bool WHOLE = decltype(whole_tag)::value;
      // Passes are taken four at a time with each kind of work done for all four before the next kind: the
      // loads, then the dot products, then the shuffles that add a key's lanes up.  Written pass by pass the
      // shuffles of one pass stood between the loads of the next and the code ran as one long chain
      // (measured: 0.83 us per page and warp; this form: see the profile).
      constexpr int G = PASSES < 4 ? PASSES : 4;
      float sc[PASSES];
      float chunk_max = -INFINITY;
#pragma unroll
      for (int p0 = 0; p0 < PASSES; p0 += G) {
        float kf[G][8];
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const int key = warp * WARP_KEYS + (p0 + g) * KPP + kl;
          Vec8<T>::load(Kt + (key < TILE_KEYS ? key : 0) * HD + c * 8, kf[g]);
        }
        float dot[G];
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const int t = tile_key0 + warp * WARP_KEYS + (p0 + g) * KPP + kl;
          const bool mine = !WHOLE && own && t == pos;
          float d0 = 0.f, d1 = 0.f;
#pragma unroll
          for (int e = 0; e < 8; e += 2) {
            d0 = fmaf(qreg[e], mine ? k_own[e] : kf[g][e], d0);
            d1 = fmaf(qreg[e + 1], mine ? k_own[e + 1] : kf[g][e + 1], d1);
          }
          dot[g] = d0 + d1;
        }
#pragma unroll
        for (int o = 1; o < CH; o <<= 1) {
#pragma unroll
          for (int g = 0; g < G; ++g) dot[g] += __shfl_xor_sync(0xffffffffu, dot[g], o);
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const int pass = p0 + g;
          const int t = tile_key0 + warp * WARP_KEYS + pass * KPP + kl;
          const bool valid = (pass * KPP + kl < WARP_KEYS) && (WHOLE || (t >= t_begin && t < t_end));
          sc[pass] = valid ? dot[g] * scale : -INFINITY;
          chunk_max = fmaxf(chunk_max, sc[pass]);
        }
      }
#pragma unroll
      for (int o = CH; o < 32; o <<= 1) chunk_max = fmaxf(chunk_max, __shfl_xor_sync(0xffffffffu, chunk_max, o));
      new_max = fmaxf(run_max, chunk_max);
      const float base = new_max == -INFINITY ? 0.f : new_max;       // nothing seen yet: exp(-inf - 0) = 0 below
      keep = exp_for<T>(run_max - base);                 // (0 while the running maximum is -inf)
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] *= keep;
#pragma unroll
      for (int p0 = 0; p0 < PASSES; p0 += G) {
        float vf[G][8], pw[G];
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const int key = warp * WARP_KEYS + (p0 + g) * KPP + kl;
          Vec8<T>::load(Vt + (key < TILE_KEYS ? key : 0) * HD + c * 8, vf[g]);
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
          // a key outside the range adds nothing, whatever its page holds: its weight is 0 and its value is
          // replaced by 0 (a stale page may hold NaN)
          const bool in_range = (WHOLE && (p0 + g + 1) * KPP <= WARP_KEYS) || sc[p0 + g] != -INFINITY;
          pw[g] = exp_for<T>(sc[p0 + g] - base);                     // 0 for a key out of range, without a branch
          chunk_sum += pw[g];
          const int t = tile_key0 + warp * WARP_KEYS + (p0 + g) * KPP + kl;
          const bool mine = !WHOLE && own && t == pos;
#pragma unroll
          for (int e = 0; e < 8; ++e) vf[g][e] = mine ? v_own[e] : (in_range ? vf[g][e] : 0.f);
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[e] = fmaf(pw[g], vf[g][e], acc[e]);
        }
      }
      };
      const bool whole = tile_key0 >= t_begin && tile_key0 + TILE_KEYS <= t_end && !(own && pos >= tile_key0 && pos < tile_key0 + TILE_KEYS);
      if (whole) take_page(std::true_type{});
      else take_page(std::false_type{});
#pragma unroll
      for (int o = CH; o < 32; o <<= 1) chunk_sum += __shfl_xor_sync(0xffffffffu, chunk_sum, o);
      run_sum = run_sum * keep + chunk_sum;
      run_max = new_max;
      __syncwarp();
      if (lane == 0) dec_mbar_arrive(&empty_bar[s]);
    }
    // the warp's key groups meet
#pragma unroll
    for (int o = CH; o < 32; o <<= 1) {
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], o);
    }
    if (kl == 0) {
#pragma unroll
      for (int e = 0; e < 8; ++e) acc_sh[warp][c * 8 + e] = acc[e];
    }
    if (lane == 0) {
      ml_sh[warp][0] = run_max;
      ml_sh[warp][1] = run_sum;
    }
  }
  __syncthreads();

  // ---- the warps meet
  float m = -INFINITY;
#pragma unroll
  for (int w = 0; w < TMA_CONSUMER_WARPS; ++w) m = fmaxf(m, ml_sh[w][0]);
  float total = 0.f, wscale[TMA_CONSUMER_WARPS];
#pragma unroll
  for (int w = 0; w < TMA_CONSUMER_WARPS; ++w) {
    wscale[w] = (ml_sh[w][0] == -INFINITY) ? 0.f : exp_for<T>(ml_sh[w][0] - m);
    total += ml_sh[w][1] * wscale[w];
  }
  if (n_splits > 1 && cluster_merge) {
    // The splits of this (row, head) are the CTAs of one thread-block cluster.  Every CTA but the first writes
    // its partial result (unnormalised output, maximum, sum) into the FIRST one's shared memory and arrives on
    // its barrier, then is done; the first waits for them and merges.  One one-way trip through the cluster's
    // network: no trip to global memory, no CTA reads another's memory, nobody waits for a closing barrier.
    if (split != 0) {
      cluster_wait();
      for (int d = tid; d < HD; d += TMA_THREADS) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < TMA_CONSUMER_WARPS; ++w) o += acc_sh[w][d] * wscale[w];
        st_cluster_f32(&recv_sh[split][d], 0u, o);
      }
      if (tid == 0) {
        st_cluster_f32(&recv_sh[split][HD], 0u, m);
        st_cluster_f32(&recv_sh[split][HD + 1], 0u, total);
      }
      __syncthreads();                         // every thread's writes come before the one arrival
      if (tid == 0) mbar_arrive_cluster(&merge_bar, 0u);
      return;
    }
    bool got = false;
    for (uint32_t i = 0; i < DEC_WAIT_LIMIT && !got; ++i) got = mbar_try_wait_cluster(&merge_bar, 0);
    if (!got) {
      if (tid == 0) atomicAdd(&g_decode_timeouts, 1);
      return;
    }
    float ms[8], ws[8];
    ms[0] = m;
    ws[0] = total;
#pragma unroll
    for (int s2 = 1; s2 < 8; ++s2) {
      ms[s2] = s2 < n_splits ? recv_sh[s2][HD] : -INFINITY;
      ws[s2] = s2 < n_splits ? recv_sh[s2][HD + 1] : 0.f;
    }
    float gm = -INFINITY;
#pragma unroll
    for (int s2 = 0; s2 < 8; ++s2) gm = fmaxf(gm, ms[s2]);
    float gl = 0.f;
#pragma unroll
    for (int s2 = 0; s2 < 8; ++s2) {
      const float a = ms[s2] == -INFINITY ? 0.f : exp_for<T>(ms[s2] - gm);
      gl += ws[s2] * a;                   // (the sum in rank order)
      ws[s2] = a;
    }
    const float inv = 1.0f / gl;
    for (int d = tid; d < HD; d += TMA_THREADS) {
      float o = 0.f;
#pragma unroll
      for (int w = 0; w < TMA_CONSUMER_WARPS; ++w) o += acc_sh[w][d] * wscale[w];
      o *= ws[0];
#pragma unroll
      for (int s2 = 1; s2 < 8; ++s2) o += (s2 < n_splits ? recv_sh[s2][d] : 0.f) * ws[s2];
      out[(int64_t)r * ld_out + (int64_t)h * HD + d] = from_f32<T>(o * inv);
    }
    return;
  }
  float* part = n_splits > 1 ? scratch + (((int64_t)r * n_heads + h) * n_splits + split) * (HD + 2) : nullptr;
  for (int d = tid; d < HD; d += TMA_THREADS) {
    float o = 0.f;
#pragma unroll
    for (int w = 0; w < TMA_CONSUMER_WARPS; ++w) o += acc_sh[w][d] * wscale[w];
    if (n_splits == 1) out[(int64_t)r * ld_out + (int64_t)h * HD + d] = from_f32<T>(o / total);
    else part[d] = o;
  }
  if (n_splits > 1) {
    if (tid == 0) {
      part[HD] = m;
      part[HD + 1] = total;
    }
    if (counters != nullptr) {
      __threadfence();
      __syncthreads();
      if (tid == 0) {
        const int done = atomicAdd(&counters[r * n_heads + h], 1);
        last_flag = (done == n_splits - 1);
        if (last_flag) counters[r * n_heads + h] = 0;
      }
      __syncthreads();
      if (last_flag) {
        __threadfence();
        merge_partials<T, HD>(scratch + ((int64_t)r * n_heads + h) * n_splits * (HD + 2),
                              out + (int64_t)r * ld_out + (int64_t)h * HD, n_splits, tid, TMA_THREADS);
      }
    }
  }
}

template <typename T, int HD>
int launch(const void* q, int64_t ld_q, void* out, int64_t ld_out, const int* row_seq, const int* row_pos,
           const int* page_table, int table_width, const void* k_pages, const void* v_pages, const void* k_new,
           const void* v_new, int64_t ld_new, float* scratch, int* counters, int n_rows, int n_heads, int n_kv_heads,
           int page_size, int n_splits, float scale, int window, cudaStream_t stream) {
  dim3 grid(n_splits, n_heads, n_rows);
  constexpr bool tma_form = (HD == 16 || HD == 32 || HD == 64 || HD == 128 || HD == 256) &&
                            DecTile<T, HD>::SMEM <= 200 * 1024;      // two stages of 256-wide 32-bit rows do not fit
  if (tma_form && page_size == TILE_KEYS && !g_force_plain) {
    using D = DecTile<T, HD>;
    // with 2..8 splits and a merge asked for in the kernel, the splits form a cluster and merge on chip
    const bool cluster = counters != nullptr && n_splits > 1 && n_splits <= 8 && !g_no_cluster;
    // Four stages let three CTAs share an SM, three stages four.  A launch of more CTAs than three an SM but not more
    // than four an SM runs as ONE wave with three stages (40 rows x 12 heads, ~520 keys: 17.8 -> 12.9 us; 48 rows:
    // 18.8 -> 14.6); every other launch is faster with the deeper ring (32 rows: 10.3 against 11.5 us, 64: 21.2
    // against 23.6).  Decided by the grid's size alone.  (The depth is a template parameter: as a run-time value it
    // cost every launch 8 %.)
    int sms = 148, dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long long ctas = (long long)n_splits * n_heads * n_rows;
    const bool shallow = D::STAGES == 4 && ctas > 3ll * sms && ctas <= 4ll * sms;
    auto go = [&](auto kernel, size_t smem, bool& configured) -> int {
      if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) KVAD_FAIL(KVAD_ERR_CUDA, "attention_decode: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
      }
      if (cluster)
        kvad_launch_cluster(kernel, grid, dim3(TMA_THREADS), smem, stream, dim3(n_splits, 1, 1),
            (const T*)q, ld_q, (T*)out, ld_out, row_seq, row_pos, page_table, table_width, (T*)const_cast<void*>(k_pages),
            (T*)const_cast<void*>(v_pages), (const T*)k_new, (const T*)v_new, ld_new, scratch, counters, n_heads, n_kv_heads,
            n_splits, scale, window, 1, g_pre);
      else
        kvad_launch(kernel, grid, dim3(TMA_THREADS), smem, stream,
            (const T*)q, ld_q, (T*)out, ld_out, row_seq, row_pos, page_table, table_width, (T*)const_cast<void*>(k_pages),
            (T*)const_cast<void*>(v_pages), (const T*)k_new, (const T*)v_new, ld_new, scratch, counters, n_heads, n_kv_heads,
            n_splits, scale, window, 0, g_pre);
      return KVAD_OK;
    };
    static bool configured[4] = {false, false, false, false};
    constexpr int SHALLOW = D::STAGES == 4 ? 3 : D::STAGES;
    constexpr bool PRE_BUILT = sizeof(T) == 2;        // the sums form is built for bfloat16 only (its only user)
    int rc;
    if (g_pre.sums != nullptr) {
      if (!PRE_BUILT) KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "attention_decode: 32-bit sums for q/k/v are taken in bfloat16 only");
      rc = shallow ? go(attention_decode_tma_kernel<T, HD, SHALLOW, PRE_BUILT>, D::smem(SHALLOW), configured[0])
                   : go(attention_decode_tma_kernel<T, HD, D::STAGES, PRE_BUILT>, D::SMEM, configured[1]);
    } else {
      rc = shallow ? go(attention_decode_tma_kernel<T, HD, SHALLOW, false>, D::smem(SHALLOW), configured[2])
                   : go(attention_decode_tma_kernel<T, HD, D::STAGES, false>, D::SMEM, configured[3]);
    }
    if (rc != KVAD_OK) return rc;
  } else {
    if (g_pre.sums != nullptr)
      KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "attention_decode: 32-bit sums for q/k/v are taken by the TMA-fed kernel only (head size %d, page size %d)", HD, page_size);
    kvad_launch(attention_decode_kernel<T, HD>, grid, dim3(DEC_THREADS), 0, stream,
        (const T*)q, ld_q, (T*)out, ld_out, row_seq, row_pos, page_table, table_width, (T*)const_cast<void*>(k_pages),
        (T*)const_cast<void*>(v_pages), (const T*)k_new, (const T*)v_new, ld_new, scratch, counters, n_heads, n_kv_heads,
        page_size, n_splits, scale, window);
  }
  KVAD_CHECK_LAUNCH("attention_decode");
  if (n_splits > 1 && counters == nullptr) {
    kvad_launch(attention_decode_merge_kernel<T, HD>, dim3(n_rows, n_heads), dim3(HD < 64 ? 32 : 64), 0, stream, (const float*)scratch, (T*)out, ld_out, n_heads, n_splits);
    KVAD_CHECK_LAUNCH("attention_decode_merge");
  }
  return KVAD_OK;
}

}  // namespace

// Tests: 1 keeps every head size on the kernel that loads through registers; 2 keeps the TMA-fed kernel
// but merges its splits through global memory instead of a cluster's shared memory; 0: the kernel's own choice.
KVAD_EXPORT void kvad_attention_decode_force_plain(int on) { g_force_plain = on == 1; g_no_cluster = on == 2; }

// How many bounded waits of the TMA-fed kernel have run out (0 in a healthy run).  Synchronises the device.
KVAD_EXPORT int kvad_attention_decode_status() {
  int n = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&n, g_decode_timeouts, sizeof(int));
  if (e != cudaSuccess) KVAD_FAIL(KVAD_ERR_CUDA, "attention_decode_status: %s", cudaGetErrorString(e));
  return n;
}

// How many floats of scratch a call needs (0 with one split).
KVAD_EXPORT int64_t kvad_attention_decode_scratch(int n_rows, int n_heads, int head_dim, int n_splits) {
  return n_splits > 1 ? (int64_t)n_rows * n_heads * n_splits * (head_dim + 2) : 0;
}

// The full form.  k_new / v_new / ld_new: this step's keys and values of the rows (or null: every key
// is read from the cache, which then must already hold the rows' own positions).  counters: one
// zeroed int per (row, head), left zeroed (or null: a second kernel merges the splits).
KVAD_EXPORT int kvad_attention_decode_step(int dtype, const void* q, int64_t ld_q, void* out, int64_t ld_out,
                                           const int* row_seq, const int* row_pos, const int* page_table,
                                           int table_width, void* k_pages, void* v_pages, const void* k_new,
                                           const void* v_new, int64_t ld_new, float* scratch, int* counters, int n_rows,
                                           int n_heads, int n_kv_heads, int head_dim, int page_size, int n_splits,
                                           float scale, int window, cudaStream_t stream) {
  struct UseOnce {            // the hint of kvad_attention_decode_pre holds for this call only, however it ends
    ~UseOnce() { g_pre = {nullptr, 0, nullptr, 0, 0, 0, nullptr, 0}; }
  } use_once;
  KVAD_REQUIRE(n_rows >= 0 && n_heads > 0 && n_kv_heads > 0 && page_size > 0 && table_width > 0 && n_splits > 0,
               "attention_decode: bad sizes rows=%d heads=%d kv_heads=%d page=%d splits=%d", n_rows, n_heads, n_kv_heads, page_size, n_splits);
  KVAD_REQUIRE(g_pre.sums == nullptr || (g_pre.ld % 4 == 0 && (reinterpret_cast<uintptr_t>(g_pre.sums) & 15) == 0 && g_pre.k_off % 8 == 0 && g_pre.v_off % 8 == 0 && head_dim % 8 == 0),
               "attention_decode: the 32-bit q/k/v sums must be 16-byte aligned, with a row stride that is a multiple of 4");
  KVAD_REQUIRE(n_heads % n_kv_heads == 0, "attention_decode: %d heads do not divide into %d key/value heads", n_heads, n_kv_heads);
  KVAD_REQUIRE(n_heads <= 65535 && n_rows <= 65535, "attention_decode: %d heads x %d rows are more than one launch takes", n_heads, n_rows);
  KVAD_REQUIRE(n_splits == 1 || scratch != nullptr, "attention_decode: %d splits need scratch memory", n_splits);
  KVAD_REQUIRE((k_new == nullptr) == (v_new == nullptr), "attention_decode: new keys and new values come together");
  KVAD_REQUIRE((ld_q % 8 == 0) && ((reinterpret_cast<uintptr_t>(k_pages) & 15) == 0) && ((reinterpret_cast<uintptr_t>(v_pages) & 15) == 0) &&
                   (k_new == nullptr || (ld_new % 8 == 0 && (reinterpret_cast<uintptr_t>(k_new) & 15) == 0 && (reinterpret_cast<uintptr_t>(v_new) & 15) == 0)),
               "attention_decode: queries, new keys/values and the cache must be 16-byte aligned with row strides that are multiples of 8");
  if (n_rows == 0) return KVAD_OK;
#define KVAD_DEC_CASE(HD)                                                                                              \
  case HD:                                                                                                             \
    if (dtype == KVAD_DTYPE_BF16)                                                                                      \
      return launch<__nv_bfloat16, HD>(q, ld_q, out, ld_out, row_seq, row_pos, page_table, table_width, k_pages,       \
                                       v_pages, k_new, v_new, ld_new, scratch, counters, n_rows, n_heads, n_kv_heads,  \
                                       page_size, n_splits, scale, window, stream);                                    \
    if (dtype == KVAD_DTYPE_F32)                                                                                       \
      return launch<float, HD>(q, ld_q, out, ld_out, row_seq, row_pos, page_table, table_width, k_pages, v_pages,      \
                               k_new, v_new, ld_new, scratch, counters, n_rows, n_heads, n_kv_heads, page_size,        \
                               n_splits, scale, window, stream);                                                       \
    break;
  switch (head_dim) {
    KVAD_DEC_CASE(16) KVAD_DEC_CASE(32) KVAD_DEC_CASE(48) KVAD_DEC_CASE(64) KVAD_DEC_CASE(80) KVAD_DEC_CASE(96)
    KVAD_DEC_CASE(112) KVAD_DEC_CASE(128) KVAD_DEC_CASE(256)
    default:
      KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "attention_decode: head size %d is not one of 16..128 in steps of 16, or 256", head_dim);
  }
#undef KVAD_DEC_CASE
  KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "attention_decode: unknown dtype %d", dtype);
}

// The NEXT call of kvad_attention_decode_step takes the rows' queries, keys and values from `sums` (32-bit, [rows, ld],
// queries from column 0, keys from k_off, values from v_off, without their bias) instead of q / k_new / v_new, adds
// `bias` (as long as a row of sums; may be null) and rounds to the element type; it also clears `zero_floats` floats
// at `zero` (may be null).  Head sizes and page sizes that the TMA-fed kernel does not take are refused.
KVAD_EXPORT void kvad_attention_decode_pre(const float* sums, int64_t ld, const void* bias, int bias_f32, int k_off, int v_off,
                                           float* zero, int64_t zero_floats) {
  g_pre = {sums, (long long)ld, bias, bias_f32, k_off, v_off, zero, (long long)zero_floats};
}

// Whether kvad_attention_decode_pre's form is taken at this head size and page size (1) or not (0).
KVAD_EXPORT int kvad_attention_decode_takes_pre(int dtype, int head_dim, int page_size) {
  const bool hd_ok = head_dim == 16 || head_dim == 32 || head_dim == 64 || head_dim == 128 || head_dim == 256;
  return (dtype == KVAD_DTYPE_BF16 && hd_ok && page_size == TILE_KEYS && !g_force_plain) ? 1 : 0;
}

// The cache already holds every position; a second kernel merges the splits.
KVAD_EXPORT int kvad_attention_decode(int dtype, const void* q, int64_t ld_q, void* out, int64_t ld_out,
                                      const int* row_seq, const int* row_pos, const int* page_table, int table_width,
                                      const void* k_pages, const void* v_pages, float* scratch, int n_rows, int n_heads,
                                      int n_kv_heads, int head_dim, int page_size, int n_splits, float scale, int window,
                                      cudaStream_t stream) {
  return kvad_attention_decode_step(dtype, q, ld_q, out, ld_out, row_seq, row_pos, page_table, table_width,
                                    const_cast<void*>(k_pages), const_cast<void*>(v_pages), nullptr, nullptr, 0, scratch,
                                    nullptr, n_rows, n_heads, n_kv_heads, head_dim, page_size, n_splits, scale, window,
                                    stream);
}

// ---------------------------------------------------------------------------------------------
// The same kernel for callers that cannot allocate (see attention_decode_noalloc.h): the scratch is
// this file-scope device array.  In host code its name is only a stand-in for the symbol, not a
// device address, so the address is asked for once per device and that pointer is what the kernel
// gets.
// ---------------------------------------------------------------------------------------------
static __device__ __align__(256) float kvad_decode_noalloc_scratch[KVAD_DECODE_NOALLOC_SCRATCH_FLOATS];

namespace {
constexpr int NOALLOC_MAX_DEVICES = 64;
float* g_noalloc_scratch[NOALLOC_MAX_DEVICES] = {nullptr};
}  // namespace

KVAD_EXPORT int64_t kvad_attention_decode_noalloc_need(int n_rows, int n_heads, int head_dim, int n_splits) {
  return kvad_attention_decode_scratch(n_rows, n_heads, head_dim, n_splits);
}

KVAD_EXPORT int kvad_attention_decode_noalloc(int dtype, const void* q, int64_t ld_q, void* out, int64_t ld_out,
                                              const int* row_seq, const int* row_pos, const int* page_table,
                                              int table_width, const void* k_pages, const void* v_pages, int n_rows,
                                              int n_heads, int n_kv_heads, int head_dim, int page_size, int n_splits,
                                              float scale, int window, cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && n_heads > 0 && head_dim > 0 && n_splits > 0,
               "attention_decode_noalloc: bad sizes rows=%d heads=%d head_dim=%d splits=%d", n_rows, n_heads, head_dim, n_splits);
  const int64_t need = kvad_attention_decode_scratch(n_rows, n_heads, head_dim, n_splits);
  if (need > (int64_t)KVAD_DECODE_NOALLOC_SCRATCH_FLOATS)
    KVAD_FAIL(KVAD_ERR_ARGUMENT,
              "attention_decode_noalloc: %d rows x %d heads x %d splits x (%d + 2) = %lld floats of scratch exceed the built-in %d; "
              "use fewer splits or rows, or kvad_attention_decode with scratch of your own",
              n_rows, n_heads, n_splits, head_dim, (long long)need, (int)KVAD_DECODE_NOALLOC_SCRATCH_FLOATS);
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) KVAD_FAIL(KVAD_ERR_CUDA, "attention_decode_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
  KVAD_REQUIRE(device >= 0 && device < NOALLOC_MAX_DEVICES, "attention_decode_noalloc: device %d is beyond the %d this entry point keeps track of", device, NOALLOC_MAX_DEVICES);
  if (g_noalloc_scratch[device] == nullptr) {
    // set-up, once per device, with that device current
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), kvad_decode_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr)
      KVAD_FAIL(KVAD_ERR_CUDA, "attention_decode_noalloc: cudaGetSymbolAddress failed on device %d: %s", device, cudaGetErrorString(e));
    g_noalloc_scratch[device] = p;
  }
  return kvad_attention_decode(dtype, q, ld_q, out, ld_out, row_seq, row_pos, page_table, table_width, k_pages, v_pages,
                               g_noalloc_scratch[device], n_rows, n_heads, n_kv_heads, head_dim, page_size, n_splits,
                               scale, window, stream);
}

KVAD_DEFINE_LAST_ERROR()
