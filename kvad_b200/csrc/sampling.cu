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
// Nothing is sorted here.  Each of the three cuts is a selection: "walking the
// ranking from the top, where does the running weight reach this target?",
// answered by a most-significant-digit-first radix search over the logits'
// bit patterns (four passes of eight bits), then over ids among exact ties.
// Weights are fixed-point integers (probability relative to the best logit,
// scaled by 2^40), so sums do not depend on the order threads add them in and
// the same logits, options and seed give the same token on every run.
#include "common.cuh"

using namespace kvad;

namespace {

constexpr int SAMPLE_THREADS = 1024;
constexpr int SAMPLE_WARPS = SAMPLE_THREADS / 32;
constexpr double FIXED_ONE = 1099511627776.0;  // 2^40

// Larger float -> larger key; NaN ranks lowest.
__device__ __forceinline__ uint32_t order_key(float v) {
  if (v != v) return 0u;
  const uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
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

struct Shared {
  unsigned long long warp_hist[SAMPLE_WARPS][256];
  unsigned long long hist[256];
  unsigned long long scan[SAMPLE_THREADS];
  unsigned long long bcast[4];
  float scratch[33];
  int   ibcast[4];
};

// Where, walking down the ranking (restricted to `within`), does the running
// weight first reach `target`?  Unit weights when `unit` (top-k counts),
// else softmax weights.  Returns the cut at that candidate and, through
// `through`, the running weight including it.  If the whole weight is below
// the target the cut is the last candidate that has any weight.
__device__ Cut select_cut(const float* __restrict__ logits, int vocab, float best, float inv_temperature,
                          bool unit, unsigned long long target, const Cut& within, Shared& sh,
                          unsigned long long* through) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint32_t prefix = 0;
  unsigned long long before = 0;   // weight ranked strictly above the current prefix range

  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = lane; i < 256; i += 32) sh.warp_hist[warp][i] = 0ull;
    __syncwarp();
    const uint32_t high_mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
    for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
      const float v = logits[i];
      const uint32_t key = order_key(v);
      if ((key & high_mask) != (prefix & high_mask)) continue;
      if (!kept(key, i, within)) continue;
      const unsigned long long w = unit ? 1ull : weight_of(v, best, inv_temperature);
      if (w) atomicAdd(&sh.warp_hist[warp][(key >> shift) & 255u], w);
    }
    __syncthreads();
    if (tid < 256) {
      unsigned long long s = 0;
      for (int w = 0; w < SAMPLE_WARPS; ++w) s += sh.warp_hist[w][tid];
      sh.hist[tid] = s;
    }
    __syncthreads();
    if (tid == 0) {
      unsigned long long run = before;
      int chosen = -1, last_nonempty = -1;
      unsigned long long before_last = before;
      for (int d = 255; d >= 0; --d) {
        const unsigned long long h = sh.hist[d];
        if (h == 0) continue;
        last_nonempty = d;
        before_last = run;
        if (run + h >= target) { chosen = d; break; }
        run += h;
      }
      if (chosen < 0) { chosen = last_nonempty; run = before_last; }   // target beyond the total: the last one
      sh.ibcast[0] = chosen;
      sh.bcast[0] = run;
    }
    __syncthreads();
    const int chosen = sh.ibcast[0];
    before = sh.bcast[0];
    if (chosen < 0) {            // nothing has weight at all: keep the very first candidate
      if (through) *through = 0;
      Cut c; c.key = 0xffffffffu; c.id = -1;
      return c;
    }
    prefix |= ((uint32_t)chosen) << shift;
    __syncthreads();
  }

  // Exact ties on `prefix`: ranked by ascending id, each with the same weight.
  // Thread t owns a contiguous range of ids, counts its ties, and after a scan
  // the owner of the wanted tie walks its range.
  const int chunk = (vocab + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
  const int lo = tid * chunk, hi = min(vocab, lo + chunk);
  unsigned long long mine = 0, w_tie = 0;
  for (int i = lo; i < hi; ++i) {
    const float v = logits[i];
    if (order_key(v) == prefix && kept(prefix, i, within)) {
      w_tie = unit ? 1ull : weight_of(v, best, inv_temperature);
      mine += 1;
    }
  }
  sh.scan[tid] = mine;
  if (tid == 0) { sh.bcast[1] = 0; sh.ibcast[1] = -1; sh.bcast[2] = 0; }
  __syncthreads();
  if (w_tie) sh.bcast[1] = w_tie;     // every tie has the same weight; any writer will do
  __syncthreads();
  const unsigned long long w = sh.bcast[1];
  if (tid == 0) {
    // how many ties are needed to reach the target from `before`
    unsigned long long need = 1;
    if (w > 0 && target > before) need = (target - before + w - 1) / w;
    unsigned long long total = 0;
    for (int t = 0; t < SAMPLE_THREADS; ++t) total += sh.scan[t];
    if (need > total) need = total;
    if (need < 1) need = 1;
    unsigned long long run = 0;
    int owner = -1;
    for (int t = 0; t < SAMPLE_THREADS; ++t) {
      if (run + sh.scan[t] >= need) { owner = t; break; }
      run += sh.scan[t];
    }
    sh.ibcast[2] = owner;
    sh.bcast[2] = need - run;          // the owner's how-manieth tie
    sh.bcast[3] = before + need * w;   // running weight through the cut
  }
  __syncthreads();
  if (tid == sh.ibcast[2]) {
    unsigned long long left = sh.bcast[2];
    for (int i = lo; i < hi; ++i) {
      if (order_key(logits[i]) == prefix && kept(prefix, i, within)) {
        if (--left == 0) { sh.ibcast[1] = i; break; }
      }
    }
  }
  __syncthreads();
  Cut c; c.key = prefix; c.id = sh.ibcast[1];
  if (through) *through = sh.bcast[3];
  __syncthreads();
  return c;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int64_t ld, int vocab,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const float* __restrict__ uniform,
              int* __restrict__ out) {
  extern __shared__ unsigned char raw[];
  Shared& sh = *reinterpret_cast<Shared*>(raw);
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, tid = threadIdx.x;
  const float* row = logits + (int64_t)r * ld;
  const float temp = temperature[r];

  // the best logit and its first index
  float best = -INFINITY;
  int best_id = 0x7fffffff;
  for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
    const float v = row[i];
    if (v > best || (v == best && i < best_id)) { best = v; best_id = i; }   // NaN compares false
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
  Cut all; all.key = 0u; all.id = 0x7fffffff;   // keeps everything... (key 0 is NaN: ranked last, id below any cut)
  all.key = 0u; all.id = 0x7fffffff;
  Cut within = all;

  const int k = top_k[r];
  if (k > 0 && k < vocab) within = select_cut(row, vocab, block_best, inv_t, true, (unsigned long long)k, within, sh, nullptr);

  // mass of what top-k kept
  unsigned long long mass = 0;
  for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
    const float v = row[i];
    if (kept(order_key(v), i, within)) mass += weight_of(v, block_best, inv_t);
  }
  sh.scan[tid] = mass;
  __syncthreads();
  for (int s = SAMPLE_THREADS / 2; s > 0; s >>= 1) {
    if (tid < s) sh.scan[tid] += sh.scan[tid + s];
    __syncthreads();
  }
  unsigned long long kept_mass = sh.scan[0];
  __syncthreads();

  const float p = top_p[r];
  if (p > 0.f && p < 1.f) {
    unsigned long long target = (unsigned long long)((double)p * (double)kept_mass);
    if ((double)target < (double)p * (double)kept_mass) target += 1;   // ceil: running mass >= p * mass
    if (target < 1) target = 1;
    unsigned long long through = 0;
    within = select_cut(row, vocab, block_best, inv_t, false, target, within, sh, &through);
    kept_mass = through;
  }

  // this row's uniform number
  if (tid == 0) {
    double u = (double)uniform[r];
    u = u < 0.0 ? 0.0 : (u > 1.0 ? 1.0 : u);
    unsigned long long target = (unsigned long long)(u * (double)kept_mass);
    if ((double)target < u * (double)kept_mass) target += 1;
    sh.bcast[0] = target;
  }
  __syncthreads();
  const unsigned long long draw = sh.bcast[0];
  __syncthreads();
  const Cut chosen = select_cut(row, vocab, block_best, inv_t, false, draw, within, sh, nullptr);
  if (tid == 0) out[r] = chosen.id >= 0 ? chosen.id : arg;
}

}  // namespace

// out[r] = token chosen for row r.  temperature[r] <= 0 means greedy; top_k[r]
// == 0 and top_p[r] outside (0,1) switch those cuts off.  uniform[r] in [0,1) is
// the row's draw (read only when it samples).
KVAD_EXPORT int kvad_sample(const float* logits, int64_t ld, int n_rows, int vocab, const float* temperature,
                            const int* top_k, const float* top_p, const float* uniform, int* out,
                            cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && vocab > 0 && ld >= vocab, "sample: bad sizes rows=%d vocab=%d ld=%lld", n_rows, vocab, (long long)ld);
  if (n_rows == 0) return KVAD_OK;
  const size_t smem = sizeof(Shared);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) KVAD_FAIL(KVAD_ERR_CUDA, "sample: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  kvad_launch(sample_kernel, dim3(n_rows), dim3(SAMPLE_THREADS), smem, stream, logits, ld, vocab, temperature, top_k, top_p, uniform, out);
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
