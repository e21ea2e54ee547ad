// Choosing the next token from 32-bit logits, one block per row.
//
// Greedy: the first index of the largest value; a NaN never wins
// (bisand/kvad: argmax, crates/llm/src/sampler.rs:217-227, 376-382).
//
// Otherwise, in bisand/kvad's order (crates/llm/src/sampler.rs:55-131):
// candidates are ranked best first, equal logits by lower id; top-k keeps the
// first k; probabilities are softmax(logit / temperature) over what is kept;
// top-p keeps the shortest prefix whose mass reaches p; one uniform number u
// from the request's own xorshift64* stream (crates/nervus/src/rng.rs:12-31)
// picks the first candidate at which the running mass reaches u times the kept
// mass.  The stream itself lives with the request on the host; a step brings
// one u per sampling row.
//
// Each of the three cuts is a selection: "walking the ranking from the top,
// where does the running weight reach this target?".  It is answered by a
// most-significant-digit-first radix search over the logits' bit patterns in
// digits of 11 bits: a histogram of weights by digit, a walk over its 2048
// bins to the one in which the target falls, and so on inside that bin.  As
// soon as the candidates of the bin are at most 1024 they are sorted in shared
// memory (by value, then by lower id), their weights are summed in rank
// order, and the place is read off the running sums.  More than 1024 exact
// ties on one value are searched by id in the same manner.
// Weights are fixed-point integers (probability relative to the best logit,
// scaled by 2^40), so sums do not depend on the order threads add them in and
// the same logits, options and seed give the same token on every run.
//
// The row is read from memory once: it stays in shared memory for all passes
// when it fits (up to about 50.8 thousand logits; a longer row is re-read from
// global memory, slower but the same).
//
// Top-k of at most 1024 takes a shorter way.  The k-th largest of the threads'
// own maxima is a lower bound of the k-th largest logit, so everything at or
// above it is a superset of what top-k keeps (for logits without many ties
// hardly more than k candidates).  If at most 1024 pass, they are sorted, the
// weights of the first k are summed in rank order, and top-p and the draw are
// read off the running sums: the same integers as the selections give,
// without walking the vocabulary again.
#include "common.cuh"

using namespace kvad;

namespace {

constexpr int SAMPLE_THREADS = 1024;
constexpr int SAMPLE_WARPS = SAMPLE_THREADS / 32;
constexpr int DIGIT_BITS = 11;
constexpr int BINS = 1 << DIGIT_BITS;          // two bins a thread when the histogram is walked
constexpr int LIST_MAX = SAMPLE_THREADS;       // the sorted list: one candidate a thread
constexpr double FIXED_ONE = 1099511627776.0;  // 2^40
static_assert(BINS == 2 * SAMPLE_THREADS && LIST_MAX <= BINS, "walk_bins and the list's running sums rely on this");

// Larger float -> larger key; NaN ranks lowest.
__device__ __forceinline__ uint32_t order_key(float v) {
  if (v != v) return 0u;
  const uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ float key_value(uint32_t key) {     // order_key's inverse; key 0 (any NaN) gives a NaN
  if (key == 0u) return __uint_as_float(0x7fc00000u);
  return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
}

struct Cut {          // a place in the ranking: everything ranked at or before (key, id) is kept
  uint32_t key;
  int id;
};

__device__ __forceinline__ bool kept(uint32_t key, int id, const Cut& c) {
  return key > c.key || (key == c.key && id <= c.id);
}

__device__ __forceinline__ unsigned long long weight_of(float logit, float best, float inv_temperature) {
  const float p = expf((logit - best) * inv_temperature);
  return (unsigned long long)((double)p * FIXED_ONE + 0.5);
}

// A candidate as one word: the logit's key above, the inverted id below, so that the larger word is ranked first.
__device__ __forceinline__ unsigned long long rank_word(uint32_t key, int id) {
  return ((unsigned long long)key << 32) | (unsigned long long)(0xffffffffu - (uint32_t)id);
}
__device__ __forceinline__ uint32_t word_key(unsigned long long w) { return (uint32_t)(w >> 32); }
__device__ __forceinline__ int word_id(unsigned long long w) { return (int)(0xffffffffu - (uint32_t)(w & 0xffffffffull)); }

struct Shared {
  unsigned long long hist[BINS];               // (the sorted list keeps its running sums in the first LIST_MAX words)
  unsigned long long list[LIST_MAX];
  unsigned long long bcast[4];
  unsigned long long red[SAMPLE_WARPS];
  float thread_max[SAMPLE_THREADS];
  float scratch[33];
  int ibcast[4];
  int list_n;
};

// The candidates a selection walks: logits val[0..n), the id of val[i] being i.
struct Items {
  const float* val;
  int n;
};

// Sum over the block; every thread gets it.
__device__ unsigned long long block_sum_u64(unsigned long long v, Shared& sh) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) sh.red[warp] = v;
  __syncthreads();
  unsigned long long t = sh.red[lane];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}

// Running sum over the block in thread order, this thread's own value included.
__device__ unsigned long long block_scan_u64(unsigned long long v, Shared& sh) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long t = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += t;
  }
  __syncthreads();
  if (lane == 31) sh.red[warp] = v;
  __syncthreads();
  unsigned long long t = sh.red[lane];
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long u = __shfl_up_sync(0xffffffffu, t, o);
    if (lane >= o) t += u;
  }
  const unsigned long long below = __shfl_sync(0xffffffffu, t, warp > 0 ? warp - 1 : 0);
  return warp > 0 ? v + below : v;
}

// bin += w in shared memory with the native 32-bit atomics (a 64-bit add there is a compare-and-swap
// loop, which queues badly when many threads meet on one bin): the low word wraps, and the one add
// that wrapped it carries into the high word, so the sum is exact in whatever order the adds land.
__device__ __forceinline__ void bin_add(unsigned long long* bin, unsigned long long w) {
  unsigned int* word = reinterpret_cast<unsigned int*>(bin);
  const unsigned int lo = (unsigned int)w;
  unsigned int hi = (unsigned int)(w >> 32);
  if (lo) {
    const unsigned int old = atomicAdd(word, lo);
    if (old + lo < old) hi += 1u;
  }
  if (hi) atomicAdd(word + 1, hi);
}

// Calls visit(value, id) for every candidate, four loads in flight a thread.
template <typename Visit>
__device__ __forceinline__ void for_each_item(const Items& items, Visit visit) {
  for (int i0 = threadIdx.x; i0 < items.n; i0 += 4 * SAMPLE_THREADS) {
    float v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = i0 + u * SAMPLE_THREADS;
      v[u] = i < items.n ? items.val[i] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = i0 + u * SAMPLE_THREADS;
      if (i < items.n) visit(v[u], i);
    }
  }
}

// Fills sh.hist[0..n_bins): for every candidate that passes `match`, its weight into the bin `digit`
// names.  A thread adds runs of equal digits up privately before it touches the bin.
template <typename Match>
__device__ void histogram(const Items& items, Shared& sh, int n_bins, Match match) {
  for (int i = threadIdx.x; i < n_bins; i += SAMPLE_THREADS) sh.hist[i] = 0ull;
  __syncthreads();
  int cur = -1;
  unsigned long long acc = 0;
  for_each_item(items, [&](float v, int id) {
    int digit;
    unsigned long long w;
    if (!match(v, id, &digit, &w) || w == 0ull) return;
    if (digit != cur) {
      if (acc) bin_add(&sh.hist[cur], acc);
      cur = digit;
      acc = 0ull;
    }
    acc += w;
  });
  if (acc) bin_add(&sh.hist[cur], acc);
  __syncthreads();
}

// Walking sh.hist's bins (from the last down when `down`, else from 0 up) and skipping empty ones: the
// first bin at which `start` plus the running sum reaches `target` (start < target), and through
// `before` the sum ahead of that bin.  If the whole sum stays below the target: the last bin that
// has anything.  -1 if all are empty.  Every thread calls it and gets the same answer.
__device__ int walk_bins(Shared& sh, int n_bins, bool down, unsigned long long start, unsigned long long target,
                         unsigned long long* before) {
  const int tid = threadIdx.x;
  const int p0 = 2 * tid, p1 = p0 + 1;            // places in walking order
  const unsigned long long h0 = p0 < n_bins ? sh.hist[down ? n_bins - 1 - p0 : p0] : 0ull;
  const unsigned long long h1 = p1 < n_bins ? sh.hist[down ? n_bins - 1 - p1 : p1] : 0ull;
  const unsigned long long sum = h0 + h1;
  const unsigned long long incl = block_scan_u64(sum, sh);
  if (tid == 0) { sh.ibcast[0] = -1; sh.ibcast[1] = -1; }
  __syncthreads();
  const unsigned long long ahead = start + incl - sum;
  if (sum > 0ull && ahead < target && ahead + sum >= target) {
    if (h0 > 0ull && ahead + h0 >= target) { sh.ibcast[0] = p0; sh.bcast[0] = ahead; }
    else { sh.ibcast[0] = p1; sh.bcast[0] = ahead + h0; }
  }
  if (sum > 0ull) atomicMax(&sh.ibcast[1], h1 > 0ull ? p1 : p0);
  __syncthreads();
  int place = sh.ibcast[0];
  if (place < 0) {                                 // the target lies beyond the whole sum
    place = sh.ibcast[1];
    if (place >= 0 && tid == place / 2) sh.bcast[0] = ahead + sum - (place == p1 ? h1 : h0);   // nothing follows it
    __syncthreads();
  }
  *before = place >= 0 ? sh.bcast[0] : start;
  __syncthreads();
  return place < 0 ? -1 : (down ? n_bins - 1 - place : place);
}

// Copies the rank words of the candidates that pass `take` to sh.list (at most LIST_MAX are stored) and
// returns how many passed.
template <typename Take>
__device__ int gather(const Items& items, Shared& sh, Take take) {
  if (threadIdx.x == 0) sh.list_n = 0;
  __syncthreads();
  for_each_item(items, [&](float v, int id) {
    const uint32_t key = order_key(v);
    if (!take(key, id)) return;
    const int at = atomicAdd(&sh.list_n, 1);
    if (at < LIST_MAX) sh.list[at] = rank_word(key, id);
  });
  __syncthreads();
  const int m = sh.list_n;
  __syncthreads();
  return m;
}

// sh.list[0..m), m <= LIST_MAX, into ranking order (bitonic, in shared memory); thread j gets rank j's
// word, threads from m on get 0.
__device__ unsigned long long sort_list(Shared& sh, int m) {
  const int tid = threadIdx.x;
  int n2 = 32;
  while (n2 < m) n2 <<= 1;
  if (tid >= m && tid < n2) sh.list[tid] = 0ull;
  __syncthreads();
  for (int size = 2; size <= n2; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      if (tid < n2 / 2) {
        const int i = 2 * tid - (tid & (stride - 1)), j = i + stride;
        const unsigned long long a = sh.list[i], b = sh.list[j];
        const bool down = (i & size) == 0;
        if (a != b && (a < b) == down) { sh.list[i] = b; sh.list[j] = a; }
      }
      __syncthreads();
    }
  }
  return tid < m ? sh.list[tid] : 0ull;
}

// The selection's last step on the sorted list of m candidates: the first rank at which `start` plus
// the running weight reaches `target`, else the last rank that has weight.
__device__ Cut list_cut(Shared& sh, int m, bool unit, float best, float inv_temperature, unsigned long long start,
                        unsigned long long target, unsigned long long* through) {
  const int tid = threadIdx.x;
  const unsigned long long mine = sort_list(sh, m);
  const unsigned long long w = tid < m ? (unit ? 1ull : weight_of(key_value(word_key(mine)), best, inv_temperature)) : 0ull;
  const unsigned long long run = start + block_scan_u64(w, sh);
  if (tid == 0) { sh.ibcast[0] = -1; sh.ibcast[1] = -1; }
  __syncthreads();
  if (w > 0ull && run >= target && run - w < target) sh.ibcast[0] = tid;
  if (w > 0ull) atomicMax(&sh.ibcast[1], tid);
  __syncthreads();
  const int at = sh.ibcast[0] >= 0 ? sh.ibcast[0] : sh.ibcast[1];
  if (tid == at) { sh.bcast[0] = run; sh.bcast[1] = mine; }
  __syncthreads();
  Cut c; c.key = 0xffffffffu; c.id = -1;
  if (at >= 0) { c.key = word_key(sh.bcast[1]); c.id = word_id(sh.bcast[1]); }
  if (through) *through = at >= 0 ? sh.bcast[0] : start;
  __syncthreads();
  return c;
}

// Where, walking down the ranking (restricted to `within`), does the running weight first reach the
// target?  Unit weights when `unit` (top-k counts), else softmax weights.  The target is `target`, or
// with share >= 0 that share of the whole weight within the cut (rounded up, at least 1); `total`
// receives that whole weight.  Returns the cut at that candidate and, through `through`, the running
// weight including it.  If the whole weight is below the target the cut is the last candidate that has
// any weight; if nothing has weight its id is -1.  With bound_levels > 0 the search stops after that
// many digits and returns their value with the digits below zero: a lower bound of the cut's key.
__device__ Cut select_cut(const Items& items, int id_limit, float best, float inv_temperature, bool unit, double share,
                          unsigned long long target, const Cut& within, Shared& sh, unsigned long long* through,
                          unsigned long long* total, int bound_levels = 0) {
  uint32_t prefix = 0, mask = 0;
  unsigned long long before = 0;   // weight ranked strictly above the current digit range
  Cut none; none.key = 0xffffffffu; none.id = -1;

  for (int level = 0; level < 3; ++level) {
    const int shift = level == 0 ? 21 : (level == 1 ? 10 : 0);
    const int n_bins = level == 2 ? 1024 : BINS;
    histogram(items, sh, n_bins, [&](float v, int id, int* digit, unsigned long long* w) {
      const uint32_t key = order_key(v);
      if ((key & mask) != prefix || !kept(key, id, within)) return false;
      *digit = (int)((key >> shift) & (uint32_t)(n_bins - 1));
      *w = unit ? 1ull : weight_of(v, best, inv_temperature);
      return true;
    });
    if (level == 0 && (share >= 0.0 || total != nullptr)) {
      const unsigned long long all = block_sum_u64(sh.hist[2 * threadIdx.x] + sh.hist[2 * threadIdx.x + 1], sh);
      if (total) *total = all;
      if (share >= 0.0) {
        target = (unsigned long long)(share * (double)all);
        if ((double)target < share * (double)all) target += 1;       // rounded up: running weight >= share * all
      }
    }
    if (target < 1) target = 1;
    const int chosen = walk_bins(sh, n_bins, true, before, target, &before);
    if (chosen < 0) {            // nothing has weight at all
      if (through) *through = 0;
      return none;
    }
    const unsigned long long in_bin = sh.hist[chosen];
    prefix |= ((uint32_t)chosen) << shift;
    mask |= ((uint32_t)(n_bins - 1)) << shift;
    __syncthreads();
    if (bound_levels > 0) {
      if (level + 1 < bound_levels) continue;
      Cut c; c.key = prefix; c.id = 0x7fffffff;
      return c;
    }
    if (unit && in_bin > (unsigned long long)LIST_MAX) continue;   // counts are known: too many for the list yet
    const int m = gather(items, sh, [&](uint32_t key, int id) { return (key & mask) == prefix && kept(key, id, within); });
    if (m <= LIST_MAX) return list_cut(sh, m, unit, best, inv_temperature, before, target, through);
  }

  // More than LIST_MAX exact ties on `prefix`, each with the same weight and ranked by ascending id:
  // the cut is the tie that brings the running weight to the target, found digit by digit over the ids.
  const unsigned long long w_tie = unit ? 1ull : weight_of(key_value(prefix), best, inv_temperature);
  int id_bits = DIGIT_BITS;
  while (id_bits < 33 && (((long long)id_limit - 1) >> id_bits)) id_bits += DIGIT_BITS;
  unsigned long long need = 1, ties_before = 0;
  uint32_t id_prefix = 0, id_mask = 0;
  for (int shift = id_bits - DIGIT_BITS; shift >= 0; shift -= DIGIT_BITS) {
    histogram(items, sh, BINS, [&](float v, int id, int* digit, unsigned long long* w) {
      if (order_key(v) != prefix || !kept(prefix, id, within) || ((uint32_t)id & id_mask) != id_prefix) return false;
      *digit = (int)(((uint32_t)id >> shift) & (uint32_t)(BINS - 1));
      *w = 1ull;
      return true;
    });
    if (shift == id_bits - DIGIT_BITS) {
      // how many ties it takes to reach the target from `before`: at least one, at most all
      const unsigned long long ties = block_sum_u64(sh.hist[2 * threadIdx.x] + sh.hist[2 * threadIdx.x + 1], sh);
      if (w_tie > 0ull && target > before) need = (target - before + w_tie - 1) / w_tie;
      if (need > ties) need = ties;
      if (need < 1) need = 1;
    }
    const int chosen = walk_bins(sh, BINS, false, ties_before, need, &ties_before);
    if (chosen < 0) {
      if (through) *through = before;
      return none;
    }
    id_prefix |= ((uint32_t)chosen) << shift;
    id_mask |= ((uint32_t)(BINS - 1)) << shift;
  }
  Cut c; c.key = prefix; c.id = (int)id_prefix;
  if (through) *through = before + need * w_tie;
  return c;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int64_t ld, int vocab, int row_in_shared, int force_general,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const float* __restrict__ uniform,
              int* __restrict__ out) {
  extern __shared__ __align__(16) unsigned char raw[];
  Shared& sh = *reinterpret_cast<Shared*>(raw);
  float* row_sh = reinterpret_cast<float*>(raw + ((sizeof(Shared) + 15) & ~(size_t)15));
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, tid = threadIdx.x;
  const float* row = logits + (int64_t)r * ld;
  const float temp = temperature[r];

  // the best logit and its first index; the row goes to shared memory on the way
  float best = -INFINITY;
  int best_id = 0x7fffffff;
  {
    const int head = (int)((4 - ((reinterpret_cast<uintptr_t>(row) >> 2) & 3)) & 3);   // up to a 16-byte boundary
    const int lead = head < vocab ? head : vocab;
    if (tid < lead) {
      const float v = row[tid];
      if (row_in_shared) row_sh[tid] = v;
      if (v > best) { best = v; best_id = tid; }
    }
    const int n4 = (vocab - lead) / 4;
    const float4* row4 = reinterpret_cast<const float4*>(row + lead);
    for (int i0 = tid; i0 < n4; i0 += 4 * SAMPLE_THREADS) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * SAMPLE_THREADS;
        if (i < n4) v[u] = row4[i];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * SAMPLE_THREADS;
        if (i >= n4) break;
        const int at = lead + 4 * i;
        const float e[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (row_in_shared) row_sh[at + j] = e[j];
          if (e[j] > best || (e[j] == best && at + j < best_id)) { best = e[j]; best_id = at + j; }   // NaN compares false
        }
      }
    }
    for (int i = lead + 4 * n4 + tid; i < vocab; i += SAMPLE_THREADS) {
      const float v = row[i];
      if (row_in_shared) row_sh[i] = v;
      if (v > best || (v == best && i < best_id)) { best = v; best_id = i; }
    }
  }
  const float block_best = block_max(best, sh.scratch);
  if (tid == 0) sh.ibcast[3] = 0x7fffffff;
  __syncthreads();
  if (best == block_best) atomicMin(&sh.ibcast[3], best_id);
  __syncthreads();
  const int arg = sh.ibcast[3] == 0x7fffffff ? 0 : sh.ibcast[3];
  if (temp <= 0.f || block_best == -INFINITY) {
    if (tid == 0) out[r] = arg;
    return;
  }

  const float inv_t = 1.0f / temp;
  Cut all; all.key = 0u; all.id = 0x7fffffff;      // keeps everything (key 0 is NaN, ranked last; no id is above this one)
  Cut within = all;
  Items items; items.val = row_in_shared ? row_sh : row; items.n = vocab;
  const float p = top_p[r];
  double u = (double)uniform[r];
  u = u < 0.0 ? 0.0 : (u > 1.0 ? 1.0 : u);

  const int k = top_k[r];
  if (k > 0 && k < vocab && k <= LIST_MAX && !force_general) {
    // the shorter way: a lower bound of the k-th largest logit from the threads' own maxima
    sh.thread_max[tid] = best;
    __syncthreads();
    Items maxima; maxima.val = sh.thread_max; maxima.n = SAMPLE_THREADS;
    const Cut bound = select_cut(maxima, SAMPLE_THREADS, 0.f, 0.f, true, -1.0, (unsigned long long)k, all, sh, nullptr, nullptr, 2);
    const int m = gather(items, sh, [&](uint32_t key, int) { return key >= bound.key; });
    if (bound.id >= 0 && m >= k && m <= LIST_MAX) {
      // thread j holds the candidate of rank j; the first k have weight
      const unsigned long long mine = sort_list(sh, m);
      const unsigned long long w = tid < k ? weight_of(key_value(word_key(mine)), block_best, inv_t) : 0ull;
      const unsigned long long run = block_scan_u64(w, sh);
      unsigned long long* sums = sh.hist;
      sums[tid] = run;
      if (tid == 0) sh.ibcast[0] = k - 1;
      __syncthreads();
      const unsigned long long below = run - w;
      unsigned long long kept_mass = sums[k - 1];
      if (p > 0.f && p < 1.f) {
        unsigned long long target = (unsigned long long)((double)p * (double)kept_mass);
        if ((double)target < (double)p * (double)kept_mass) target += 1;   // rounded up: running mass >= p * mass
        if (target < 1) target = 1;
        if (tid < k && run >= target && below < target) sh.ibcast[0] = tid;
        __syncthreads();
        kept_mass = sums[sh.ibcast[0]];
      }
      const int last = sh.ibcast[0];
      unsigned long long draw = (unsigned long long)(u * (double)kept_mass);
      if ((double)draw < u * (double)kept_mass) draw += 1;
      if (draw < 1) draw = 1;
      if (tid <= last && run >= draw && below < draw) out[r] = word_id(mine);
      return;
    }
  }
  if (k > 0 && k < vocab)
    within = select_cut(items, vocab, block_best, inv_t, true, -1.0, (unsigned long long)k, within, sh, nullptr, nullptr);

  Cut chosen;
  if (p > 0.f && p < 1.f) {
    // top-p: the shortest prefix of the ranking whose mass reaches p of what top-k kept
    unsigned long long kept_mass = 0;
    within = select_cut(items, vocab, block_best, inv_t, false, (double)p, 0ull, within, sh, &kept_mass, nullptr);
    unsigned long long draw = (unsigned long long)(u * (double)kept_mass);
    if ((double)draw < u * (double)kept_mass) draw += 1;
    chosen = select_cut(items, vocab, block_best, inv_t, false, -1.0, draw, within, sh, nullptr, nullptr);
  } else {
    chosen = select_cut(items, vocab, block_best, inv_t, false, u, 0ull, within, sh, nullptr, nullptr);
  }
  if (tid == 0) out[r] = chosen.id >= 0 ? chosen.id : arg;
}

bool g_force_general = false;     // tests: never take the shorter way of a small top-k

}  // namespace

// Tests: 1 sends every row the general way (selections over the whole vocabulary).
KVAD_EXPORT void kvad_sample_force_general(int on) { g_force_general = on != 0; }

// out[r] = token chosen for row r.  temperature[r] <= 0 means greedy; top_k[r]
// == 0 and top_p[r] outside (0,1) switch those cuts off.  uniform[r] in [0,1) is
// the row's draw (read only when it samples).
KVAD_EXPORT int kvad_sample(const float* logits, int64_t ld, int n_rows, int vocab, const float* temperature,
                            const int* top_k, const float* top_p, const float* uniform, int* out,
                            cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && vocab > 0 && ld >= vocab, "sample: bad sizes rows=%d vocab=%d ld=%lld", n_rows, vocab, (long long)ld);
  if (n_rows == 0) return KVAD_OK;
  static int smem_limit = -1;
  if (smem_limit < 0) {
    int dev = 0, limit = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&limit, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, limit);
    if (e != cudaSuccess) KVAD_FAIL(KVAD_ERR_CUDA, "sample: cannot reserve %d bytes of shared memory: %s", limit, cudaGetErrorString(e));
    smem_limit = limit;
  }
  const size_t fixed = ((sizeof(Shared) + 15) & ~(size_t)15) + 16;
  KVAD_REQUIRE(fixed <= (size_t)smem_limit, "sample: needs %zu bytes of shared memory, the device gives %d", fixed, smem_limit);
  const int row_in_shared = fixed + (size_t)vocab * 4 <= (size_t)smem_limit ? 1 : 0;
  const size_t smem = fixed + (row_in_shared ? (size_t)vocab * 4 : 0);
  kvad_launch(sample_kernel, dim3(n_rows), dim3(SAMPLE_THREADS), smem, stream, logits, ld, vocab, row_in_shared,
              g_force_general ? 1 : 0, temperature, top_k, top_p, uniform, out);
  KVAD_CHECK_LAUNCH("sample");
  return KVAD_OK;
}

// Greedy only: out[r] = first index of the largest logit of row r.
__global__ void __launch_bounds__(256)
argmax_kernel(const float* __restrict__ logits, int64_t ld, int vocab, int* __restrict__ out) {
  __shared__ float scratch[33];
  __shared__ int winner;
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, tid = threadIdx.x;
  const float* row = logits + (int64_t)r * ld;
  float best = -INFINITY;
  int best_id = 0x7fffffff;
  for (int i = tid; i < vocab; i += blockDim.x) {
    const float v = row[i];
    if (v > best) { best = v; best_id = i; }    // strided ascending: the first of equals stays
  }
  const float block_best = block_max(best, scratch);
  if (tid == 0) winner = 0x7fffffff;
  __syncthreads();
  if (best == block_best && best_id != 0x7fffffff) atomicMin(&winner, best_id);
  __syncthreads();
  if (tid == 0) out[r] = winner == 0x7fffffff ? 0 : winner;
}

// The same in two stages, for few rows of a large vocabulary: many blocks per row each reduce a
// chunk to one 64-bit key (value bits above, inverted index below, so that the larger key is the
// larger value and, among equals, the lower index), then one warp per row takes the largest key.
constexpr int ARGMAX_CHUNK = 2048;

__global__ void __launch_bounds__(256)
argmax_partial_kernel(const float* __restrict__ logits, int64_t ld, int vocab, unsigned long long* __restrict__ partial,
                      int n_chunks) {
  __shared__ unsigned long long keys[8];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.y, chunk = blockIdx.x, tid = threadIdx.x;
  const float* row = logits + (int64_t)r * ld;
  const int begin = chunk * ARGMAX_CHUNK;
  const int end = begin + ARGMAX_CHUNK < vocab ? begin + ARGMAX_CHUNK : vocab;
  unsigned long long best = 0ull;
  for (int i = begin + tid; i < end; i += 256) {
    const unsigned long long key = ((unsigned long long)order_key(row[i]) << 32) | (unsigned long long)(0xffffffffu - (uint32_t)i);
    best = key > best ? key : best;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
    best = other > best ? other : best;
  }
  if ((tid & 31) == 0) keys[tid >> 5] = best;
  __syncthreads();
  if (tid == 0) {
    for (int w = 1; w < 8; ++w) best = keys[w] > best ? keys[w] : best;
    partial[(int64_t)r * n_chunks + chunk] = best;
  }
}

__global__ void __launch_bounds__(32)
argmax_final_kernel(const unsigned long long* __restrict__ partial, int n_chunks, int* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  unsigned long long best = 0ull;
  for (int i = threadIdx.x; i < n_chunks; i += 32) {
    const unsigned long long key = partial[(int64_t)r * n_chunks + i];
    best = key > best ? key : best;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
    best = other > best ? other : best;
  }
  if (threadIdx.x == 0) out[r] = (int)(0xffffffffu - (uint32_t)(best & 0xffffffffull));
}

// How many 64-bit words of scratch the two-stage form needs.
KVAD_EXPORT int64_t kvad_argmax_scratch(int n_rows, int vocab) {
  return (int64_t)n_rows * ((vocab + ARGMAX_CHUNK - 1) / ARGMAX_CHUNK);
}

// scratch == nullptr: one block per row.  Otherwise two stages through `scratch`
// (kvad_argmax_scratch(n_rows, vocab) 64-bit words).
KVAD_EXPORT int kvad_argmax(const float* logits, int64_t ld, int n_rows, int vocab, int* out,
                            unsigned long long* scratch, cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && vocab > 0 && ld >= vocab, "argmax: bad sizes rows=%d vocab=%d ld=%lld", n_rows, vocab, (long long)ld);
  if (n_rows == 0) return KVAD_OK;
  if (scratch == nullptr) {
    kvad_launch(argmax_kernel, dim3(n_rows), dim3(256), 0, stream, logits, ld, vocab, out);
    KVAD_CHECK_LAUNCH("argmax");
    return KVAD_OK;
  }
  KVAD_REQUIRE(n_rows <= 65535, "argmax: %d rows are more than one launch takes", n_rows);
  const int n_chunks = (vocab + ARGMAX_CHUNK - 1) / ARGMAX_CHUNK;
  kvad_launch(argmax_partial_kernel, dim3(n_chunks, n_rows), dim3(256), 0, stream, logits, ld, vocab, scratch, n_chunks);
  KVAD_CHECK_LAUNCH("argmax_partial");
  kvad_launch(argmax_final_kernel, dim3(n_rows), dim3(32), 0, stream, (const unsigned long long*)scratch, n_chunks, out);
  KVAD_CHECK_LAUNCH("argmax_final");
  return KVAD_OK;
}

KVAD_DEFINE_LAST_ERROR()
