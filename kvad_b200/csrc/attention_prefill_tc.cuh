// Causal attention of prompt rows on the 5th-generation tensor cores (head sizes 64 and 128).
//
// A CTA has two SLOTS, each a group of four softmax warps (a thread per row) with its own S, P and P.V
// buffers, that walk cache pages (64 keys each) side by side.  What limits the kernel is the chain
// through one softmax thread - ~0.9 us a page - so the work is cut to keep every chain short: a tile of
// 128 rows that sees more than 8 pages is given to BOTH slots, each walking half of its pages, and
// the halves (unnormalised output, maximum, sum) meet through shared memory at the end; shorter
// tiles go two to a CTA, a longer one paired with a shorter one.  Roles: warp 0 brings Q and a ring of
// K/V pages by TMA (128-byte swizzle), in the order the slots use them (a page both slots read at the
// same step is brought once); one thread of warp 1 issues tcgen05.mma; warps 2-5 are slot 0, warps 6-9
// slot 1.  (A kernel that allocates tensor memory gets one CTA per SM, whatever else it needs: the
// second slot is what keeps the tensor core busy while the first one's softmax runs.)
//
//   S_i = Q . K_i^T        128 x 64 in tensor memory, two buffers
//   softmax thread r       reads row r of S_i with tcgen05.ld, scales and masks it, keeps the row's running
//                          maximum and sum in 32-bit, writes P_i = exp2(S_i - max) as bfloat16 into shared
//                          memory in the layout the tensor core reads (K-major, 128-byte swizzle)
//   T_i = P_i . V_i        128 x head size in tensor memory, two buffers; V is read as it lies in the
//                          cache ([key][head size]: the MN-major operand form)
//   softmax thread r       O_r = O_r * exp2(old max - new max) + T_i, in registers
//
// so that the tensor core works on page i+1 while the softmax threads are on page i, and nothing of size
// rows x keys reaches memory.  Keys of a page beyond the sequence's length are masked by position (they
// lie after every row), and their V rows are zeroed in shared memory before the second product, so that
// whatever a recycled page still holds cannot reach a result.
//
// Every wait is bounded; one that runs out raises g_wait_timeouts and the CTA frees its tensor memory
// and returns.
#pragma once
#include "tcgen05.cuh"

namespace kvad {
namespace pftc {

constexpr int ROWS = 128;         // query rows per tile
constexpr int TILES = 2;          // slots of a CTA
constexpr int SPLIT_ABOVE = 8;    // a tile that sees more pages than this is walked by both slots, half each (the launch may say otherwise)
constexpr int KEYS = 64;          // keys per step = one cache page
constexpr int THREADS = 64 + TILES * 128;

template <int HD> struct Layout {
  static constexpr int KB = HD / 64;                          // 64-wide blocks of the head dimension
  static constexpr int STAGES = HD == 64 ? 6 : 3;             // pages in the ring; two slots on pages of their own use two a step
  static constexpr int T_BUFS = HD == 64 ? 2 : 1;             // buffers of P.V per tile in tensor memory
  static constexpr uint32_t Q_BYTES = ROWS * HD * 2;          // one tile's rows
  static constexpr uint32_t TILE_BYTES = KEYS * HD * 2;       // K or V of one page and head
  static constexpr uint32_t P_BYTES = ROWS * KEYS * 2;
  static constexpr uint32_t OFF_KV = TILES * Q_BYTES;
  static constexpr uint32_t OFF_P = OFF_KV + STAGES * 2 * TILE_BYTES;
  static constexpr uint32_t OFF_BAR = OFF_P + TILES * 2 * P_BYTES;
  static constexpr int N_BARS = 1 + 2 * STAGES + TILES * 8;
  static constexpr size_t SMEM = OFF_BAR + N_BARS * 8 + 16 + 1024;
  // tensor-memory columns of tile t: S buffers at t * 256 + b * 64, P.V buffers at t * 256 + 128 + b * HD
  static constexpr uint32_t TMEM_TILE = 256, TMEM_T = 2 * KEYS;
  static constexpr uint32_t TMEM_COLS = 512;
  static_assert(TMEM_T + T_BUFS * HD <= TMEM_TILE, "a tile's buffers must fit its 256 columns");
  static_assert(SMEM <= 227 * 1024, "the CTA's shared memory");
};

// V as the B operand of P.V: rows are keys (the product's K), 128 contiguous bytes are 64 of the
// head dimension (its N).  Groups of 8 keys are 1024 bytes apart; the next 64 of the head dimension
// lie one whole tile of 64 keys further on.
__device__ __forceinline__ uint64_t sw128_mn_desc(uint32_t smem_addr, uint32_t next_atom_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((next_atom_bytes >> 4) & 0x3FFFu) << 16;   // leading byte offset: between 64-wide blocks of N
  d |= (uint64_t)(1024 >> 4) << 32;                          // stride byte offset: between groups of 8 rows of K
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;                                    // SWIZZLE_128B
  return d;
}

__device__ __forceinline__ void tmem_ld32_issue(uint32_t addr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(addr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// tcgen05.alloc with the column count as an immediate, so that how much tensor memory a CTA takes is
// visible in the compiled kernel.
template <uint32_t COLS> __device__ __forceinline__ void tmem_alloc_fixed(uint32_t* slot) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "n"(COLS) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
template <uint32_t COLS> __device__ __forceinline__ void tmem_dealloc_fixed(uint32_t addr) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "n"(COLS) : "memory");
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Which pages slot `t` of a CTA walks, for which tile.
struct TileRange {
  int qt;            // index of the 128-row tile within the sequence's new rows; -1: none
  int rows;          // rows of it that exist
  int pos0;          // position of its first row
  int j_lo, j_hi;    // first and last page
};

template <int HD>
__global__ void __launch_bounds__(THREADS, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out, int64_t ld_out,
                            const int* __restrict__ seq_starts, const int* __restrict__ kv_lens,
                            const int* __restrict__ page_table, int table_width, int n_heads, int n_kv_heads,
                            int split_above, float scale, int window) {
  using L = Layout<HD>;
  constexpr int STAGES = L::STAGES, T_BUFS = L::T_BUFS;
  extern __shared__ uint8_t pftc_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(pftc_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* q_tiles = smem;
  uint8_t* kv_tiles = smem + L::OFF_KV;           // stage s: K at s * 2 * TILE_BYTES, V right after it
  uint8_t* p_tiles = smem + L::OFF_P;             // tile t, buffer b at (t * 2 + b) * P_BYTES
  uint64_t* q_full = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* kv_full = q_full + 1;
  uint64_t* kv_empty = kv_full + STAGES;
  uint64_t* s_full = kv_empty + STAGES;           // [tile][2] S is in tensor memory
  uint64_t* p_full = s_full + TILES * 2;          // [tile][2] P is in shared memory (and S has been read)
  uint64_t* t_full = p_full + TILES * 2;          // [tile][2] P.V is in tensor memory (and P, K, V have been read)
  uint64_t* t_empty = t_full + TILES * 2;         // [tile][2] P.V has been read
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(t_empty + TILES * 2);

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Which tiles this CTA serves is decided first, from the step's metadata (uploaded before the step's first
  // kernel, so readable before the dependent-launch wait): a CTA with nothing to do leaves before it has
  // set anything up.
  const int s = blockIdx.z, h = blockIdx.y;
  const int row0_seq = seq_starts[s];
  const int n_new = seq_starts[s + 1] - row0_seq;
  const int kv_len = kv_lens[s];
  const int first_pos = kv_len - n_new;
  const int kvh = h / (n_heads / n_kv_heads);
  const int* pages = page_table + (int64_t)s * table_width;
  const int n_tiles_seq = (n_new + ROWS - 1) / ROWS;
  auto tile_range = [&](int qt, TileRange& r) {
    r.qt = qt;
    r.rows = (n_new - qt * ROWS) < ROWS ? (n_new - qt * ROWS) : ROWS;
    r.pos0 = first_pos + qt * ROWS;
    r.j_hi = (r.pos0 + r.rows - 1) / KEYS;
    r.j_lo = 0;
    if (window > 0 && r.pos0 - window + 1 > 0) r.j_lo = (r.pos0 - window + 1) / KEYS;
  };
  TileRange tr[TILES];
  tr[0].qt = tr[1].qt = -1;
  tr[0].rows = tr[1].rows = 0;
  tr[0].pos0 = tr[1].pos0 = first_pos;
  tr[0].j_lo = tr[1].j_lo = 0x3fffffff;
  tr[0].j_hi = tr[1].j_hi = -1;
  bool split = false;
  {
    // CTAs 0 .. n_split-1 take the tiles that see more than `split_above` pages, latest first, both slots on one tile;
    // the CTAs after them pair the other tiles, the c-th latest with the c-th earliest.
    int n_split = 0;
    for (int qt = 0; qt < n_tiles_seq; ++qt) {
      TileRange r;
      tile_range(qt, r);
      n_split += (r.j_hi - r.j_lo + 1 > split_above) ? 1 : 0;
    }
    const int c = (int)blockIdx.x, n_rest = n_tiles_seq - n_split;
    const int want_a = c < n_split ? c : c - n_split;                      // how many tiles of its kind come before, latest first
    const int want_b = c < n_split ? -1 : n_rest - 1 - (c - n_split);
    int seen = 0;
    for (int qt = n_tiles_seq - 1; qt >= 0; --qt) {
      TileRange r;
      tile_range(qt, r);
      const bool is_split = r.j_hi - r.j_lo + 1 > split_above;
      if (is_split != (c < n_split)) continue;
      if (seen == want_a && (c < n_split || want_b >= want_a)) tr[0] = r;
      if (seen == want_b && want_b > want_a) tr[1] = r;
      ++seen;
    }
    if (c < n_split && tr[0].qt >= 0) {
      split = true;
      tr[1] = tr[0];
      const int mid = tr[0].j_lo + (tr[0].j_hi - tr[0].j_lo + 2) / 2;      // slot 0: the earlier pages; slot 1: the later ones, with the diagonal
      tr[0].j_hi = mid - 1;
      tr[1].j_lo = mid;
    }
  }
  const bool active = tr[0].qt >= 0;
  if (!active) return;
  const int n_steps0 = tr[0].j_hi - tr[0].j_lo + 1, n_steps1 = tr[1].qt >= 0 ? tr[1].j_hi - tr[1].j_lo + 1 : 0;
  const int n_steps_max = n_steps0 > n_steps1 ? n_steps0 : n_steps1;
  // The ring holds pages in the order of use: step by step, slot 0's page, then slot 1's unless it is the same one
  // (two tiles that start at the same page walk it together).  load_of(t, i): which load serves slot t at step i.
  const bool same_start = !split && tr[1].qt >= 0 && tr[0].j_lo == tr[1].j_lo;      // then slot 1 (the earlier tile) has no more steps than slot 0
  auto load_of = [&](int t, int i) -> int {
    if (same_start) return i;
    const int a = i < n_steps0 ? i : n_steps0, b = i < n_steps1 ? i : n_steps1;
    return a + b + ((t == 1 && i < n_steps0) ? 1 : 0);
  };

  if (threadIdx.x == 0) {
    prefetch_tensormap(&map_q);
    prefetch_tensormap(&map_k);
    prefetch_tensormap(&map_v);
    mbar_init(q_full, 1);
    for (int st = 0; st < STAGES; ++st) { mbar_init(&kv_full[st], 1); mbar_init(&kv_empty[st], 1); }
    for (int b = 0; b < TILES * 2; ++b) {
      mbar_init(&s_full[b], 1);
      mbar_init(&p_full[b], 128);
      mbar_init(&t_full[b], 1);
      mbar_init(&t_empty[b], 128);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_shared();
  }
  if (warp == 1) tmem_alloc_fixed<L::TMEM_COLS>(tmem_slot);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  pdl_wait();                                      // everything below reads what earlier kernels of the step wrote

  if (warp == 0) {
    if (lane == 0) {
      const int n_q = (tr[1].qt >= 0 && !split) ? 2 : 1;                   // both slots of a split tile read one copy of its rows
      mbar_expect_tx(q_full, n_q * L::Q_BYTES);
#pragma unroll
      for (int t = 0; t < TILES; ++t)
        if (t < n_q)
          for (int kb = 0; kb < L::KB; ++kb)
            tma_load_2d(q_tiles + t * L::Q_BYTES + kb * (ROWS * 128), &map_q, q_full, h * HD + kb * 64, row0_seq + tr[t].qt * ROWS);
      int li = 0;
      bool ok = true;
      for (int i = 0; i < n_steps_max && ok; ++i) {
#pragma unroll
        for (int t = 0; t < TILES; ++t) {
          if (i >= (t == 0 ? n_steps0 : n_steps1) || (t == 1 && same_start)) continue;
          const int st = li % STAGES;
          if (li >= STAGES && !mbar_wait(&kv_empty[st], ((li / STAGES) & 1) ^ 1)) { ok = false; break; }
          uint8_t* k_dst = kv_tiles + st * 2 * L::TILE_BYTES;
          uint8_t* v_dst = k_dst + L::TILE_BYTES;
          const int y = (pages[tr[t].j_lo + i] * n_kv_heads + kvh) * KEYS;
          mbar_expect_tx(&kv_full[st], 2 * L::TILE_BYTES);
#pragma unroll
          for (int kb = 0; kb < L::KB; ++kb) {
            tma_load_2d(k_dst + kb * (KEYS * 128), &map_k, &kv_full[st], kb * 64, y);
            tma_load_2d(v_dst + kb * (KEYS * 128), &map_v, &kv_full[st], kb * 64, y);
          }
          ++li;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_instr_desc(ROWS, KEYS);
      constexpr uint32_t idesc_pv = umma_instr_desc(ROWS, HD, false, true);
      bool ok = mbar_wait(q_full, 0);
      // Per step: S of both slots, then P.V of the step before for both, so that the first product of a step is
      // under way while the softmax threads are on the step before.  With a ring of fewer than four pages (head size
      // 128) and two slots on pages of their own that order would need a fourth page: there each slot's S is followed
      // at once by its P.V of the step before, which gives the page back.
      constexpr bool INTERLEAVE = STAGES < 4;
      auto product_s = [&](int t, int i) {
        const int ld = load_of(t, i), st = ld % STAGES, b = i & 1;
        if (!mbar_wait(&kv_full[st], (ld / STAGES) & 1)) { ok = false; return; }
        tc_fence_after();
        const uint32_t k_addr = smem_u32(kv_tiles + st * 2 * L::TILE_BYTES);
        const uint32_t q_addr = smem_u32(q_tiles + (split ? 0 : t) * L::Q_BYTES);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint64_t a_desc = sw128_desc(q_addr + (k / 4) * (ROWS * 128)) + (uint64_t)((k % 4) * 2);
          const uint64_t b_desc = sw128_desc(k_addr + (k / 4) * (KEYS * 128)) + (uint64_t)((k % 4) * 2);
          umma(tmem_base + t * L::TMEM_TILE + b * KEYS, a_desc, b_desc, idesc_qk, k > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[t * 2 + b]);
      };
      auto product_pv = [&](int t, int ip) {
        const int st = load_of(t, ip) % STAGES, b = ip & 1, tb = ip % T_BUFS;
        const uint32_t v_addr = smem_u32(kv_tiles + st * 2 * L::TILE_BYTES + L::TILE_BYTES);
        if (!(mbar_wait(&p_full[t * 2 + b], (ip >> 1) & 1) && mbar_wait(&t_empty[t * 2 + tb], ((ip / T_BUFS) & 1) ^ 1))) { ok = false; return; }
        tc_fence_after();
        const uint32_t p_addr = smem_u32(p_tiles + (t * 2 + b) * L::P_BYTES);
#pragma unroll
        for (int kk = 0; kk < KEYS / 16; ++kk) {
          const uint64_t a_desc = sw128_desc(p_addr) + (uint64_t)(kk * 2);
          const uint64_t b_desc = sw128_mn_desc(v_addr + kk * 2048, KEYS * 128);
          umma(tmem_base + t * L::TMEM_TILE + L::TMEM_T + tb * HD, a_desc, b_desc, idesc_pv, kk > 0 ? 1u : 0u);
        }
        umma_commit(&t_full[t * 2 + tb]);
      };
      const int n_steps_of[TILES] = {n_steps0, n_steps1};
      for (int i = 0; i <= n_steps_max && ok; ++i) {
        if (INTERLEAVE && !same_start) {
#pragma unroll
          for (int t = 0; t < TILES; ++t) {
            if (i < n_steps_of[t] && ok) product_s(t, i);
            if (i > 0 && i - 1 < n_steps_of[t] && ok) {
              product_pv(t, i - 1);
              if (ok) umma_commit(&kv_empty[load_of(t, i - 1) % STAGES]);      // the page has been read
            }
          }
        } else {
#pragma unroll
          for (int t = 0; t < TILES; ++t)
            if (i < n_steps_of[t] && ok) product_s(t, i);
          if (i > 0) {
#pragma unroll
            for (int t = 0; t < TILES; ++t)
              if (i - 1 < n_steps_of[t] && ok) product_pv(t, i - 1);
            // the step's pages have been read by all that use them
#pragma unroll
            for (int t = 0; t < TILES; ++t)
              if (ok && i - 1 < n_steps_of[t] && !(t == 1 && same_start)) umma_commit(&kv_empty[load_of(t, i - 1) % STAGES]);
          }
        }
      }
    }
  } else if (tr[(warp - 2) >> 2].qt >= 0) {
    // ---- softmax: warps 2-5 serve tile 0, warps 6-9 tile 1; thread -> row
    const int t = (warp - 2) >> 2;
    const TileRange me = tr[t];
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + t * L::TMEM_TILE;
    const int pos = me.pos0 + row;
    const int pos_last_row = me.pos0 + me.rows - 1;
    const int n_steps = me.j_hi - me.j_lo + 1;
    const float sl2 = scale * 1.4426950408889634f;
    float run_max = -INFINITY, run_sum = 0.f, keep_prev = 0.f;
    float o[HD];
#pragma unroll
    for (int c = 0; c < HD; ++c) o[c] = 0.f;
    bool ok = true;

    // O = O * keep + P.V of step k
    auto take_product = [&](int k, float keep) {
      const int tb = k % T_BUFS;
      if (!mbar_wait(&t_full[t * 2 + tb], (k / T_BUFS) & 1)) { ok = false; return; }
      tc_fence_after();
#pragma unroll
      for (int c0 = 0; c0 < HD; c0 += 32) {
        uint32_t r[32];
        tmem_ld32_issue(lane_addr + L::TMEM_T + tb * HD + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 32; ++c) o[c0 + c] = o[c0 + c] * keep + __uint_as_float(r[c]);
      }
      tc_fence_before();
      mbar_arrive(&t_empty[t * 2 + tb]);
    };

    for (int k = 0; k < n_steps && ok; ++k) {
      const int j = me.j_lo + k, b = k & 1;
      if (!mbar_wait(&s_full[t * 2 + b], (k >> 1) & 1)) { ok = false; break; }
      tc_fence_after();
      uint32_t sr[KEYS];
      tmem_ld32_issue(lane_addr + b * KEYS, sr);
      tmem_ld32_issue(lane_addr + b * KEYS + 32, sr + 32);
      tmem_ld_wait();
      const bool mask = (j * KEYS + KEYS - 1 > me.pos0) || (window > 0 && j * KEYS <= pos_last_row - window);
      // (two loops, so that the pages every row sees whole carry no per-element test; four running maxima
      // keep the chain of dependent instructions short.  The scale, which is positive, is applied to the
      // maximum here and to each score inside the exponent's multiply-add below.)
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (!mask) {
#pragma unroll
        for (int c = 0; c < KEYS; ++c) mx[c & 3] = fmaxf(mx[c & 3], __uint_as_float(sr[c]));
      } else {
        const int lo_key = window > 0 ? pos - window + 1 : 0;       // the row sees keys lo_key .. pos
#pragma unroll
        for (int c = 0; c < KEYS; ++c) {
          const int key = j * KEYS + c;
          const float v = (key <= pos && key >= lo_key) ? __uint_as_float(sr[c]) : -INFINITY;
          sr[c] = __float_as_uint(v);
          mx[c & 3] = fmaxf(mx[c & 3], v);
        }
      }
      const float tile_max = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * sl2;
      const float new_max = fmaxf(run_max, tile_max);
      const float base = new_max == -INFINITY ? 0.f : new_max;        // a row that has seen nothing yet
      const float keep = run_max == -INFINITY ? 0.f : fast_exp2(run_max - base);
      run_max = new_max;
      float sum2[2] = {0.f, 0.f};
      uint8_t* p_row = p_tiles + (t * 2 + b) * L::P_BYTES + row * 128;
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float p0 = fast_exp2(fmaf(__uint_as_float(sr[ch * 8 + 2 * e]), sl2, -base));
          const float p1 = fast_exp2(fmaf(__uint_as_float(sr[ch * 8 + 2 * e + 1]), sl2, -base));
          sum2[0] += p0;
          sum2[1] += p1;
          __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
          w[e] = *reinterpret_cast<uint32_t*>(&pk);
        }
        *reinterpret_cast<uint4*>(p_row + ((ch ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
      }
      run_sum = run_sum * keep + (sum2[0] + sum2[1]);
      // the last page may hold rows past the sequence's end: their V must not reach the product
      // (both tiles may clear the same rows; they write the same zeros)
      const int valid = kv_len - j * KEYS;
      if (valid < KEYS) {
        const int ld = load_of(t, k), st = ld % STAGES;
        if (!mbar_wait(&kv_full[st], (ld / STAGES) & 1)) { ok = false; break; }
        uint8_t* v_tile = kv_tiles + st * 2 * L::TILE_BYTES + L::TILE_BYTES;
        const int first = valid < 0 ? 0 : valid;
        const int n16 = (KEYS - first) * 8;                          // 16-byte pieces of the rows to clear, per 64-wide block
        for (int kb = 0; kb < L::KB; ++kb)
          for (int x = row; x < n16; x += 128)
            *reinterpret_cast<uint4*>(v_tile + kb * (KEYS * 128) + first * 128 + x * 16) = make_uint4(0u, 0u, 0u, 0u);
      }
      tc_fence_before();
      fence_async_shared();
      mbar_arrive(&p_full[t * 2 + b]);
      if (k >= 1) take_product(k - 1, keep_prev);
      keep_prev = keep;
    }
    if (ok && n_steps > 0) take_product(n_steps - 1, keep_prev);
    if (split) {
      // The two halves of the tile meet: all products of the CTA have been read (each slot has taken its last one),
      // so the page ring is free; slot 1 leaves its rows' sums, maxima and unnormalised outputs there, slot 0 adds.
      float* xch = reinterpret_cast<float*>(kv_tiles);                      // [ROWS][HD + 2]
      asm volatile("bar.sync 2, 256;" ::: "memory");
      if (t == 1) {
        float* mine = xch + row * (HD + 2);
#pragma unroll
        for (int c = 0; c < HD; ++c) mine[c] = o[c];
        mine[HD] = run_max;
        mine[HD + 1] = run_sum;
      }
      asm volatile("bar.sync 2, 256;" ::: "memory");
      if (t == 0) {
        const float* other = xch + row * (HD + 2);
        const float m1 = other[HD], l1 = other[HD + 1];
        const float m = fmaxf(run_max, m1);
        const float s0 = run_max == -INFINITY ? 0.f : fast_exp2(run_max - m), s1 = m1 == -INFINITY ? 0.f : fast_exp2(m1 - m);
        run_sum = run_sum * s0 + l1 * s1;
#pragma unroll
        for (int c = 0; c < HD; ++c) o[c] = o[c] * s0 + other[c] * s1;
      }
    }
    if (ok && row < me.rows && !(split && t == 1)) {
      const float inv = 1.0f / run_sum;
      __nv_bfloat16* dst = out + (int64_t)(row0_seq + me.qt * ROWS + row) * ld_out + (int64_t)h * HD;
#pragma unroll
      for (int c = 0; c < HD; c += 8) {
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          __nv_bfloat162 pk = __floats2bfloat162_rn(o[c + 2 * e] * inv, o[c + 2 * e + 1] * inv);
          w[e] = *reinterpret_cast<uint32_t*>(&pk);
        }
        *reinterpret_cast<uint4*>(dst + c) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc_fixed<L::TMEM_COLS>(tmem_base);
  }
}

}  // namespace pftc
}  // namespace kvad
