// Split-context paged attention for single decoded tokens, bfloat16 keys and values, float32
// scores, softmax and accumulation.
//
// The decode step is bound by reading the cache, so the kernel is built around the copy.  One
// persistent CTA per SM walks a list of work items, an item being one (request, key/value head,
// split of the context).  Inside the CTA the work is split by role:
//   * three producer warps, taking tiles in turn, run ahead through the items and stream their keys and values into a
//     ring of shared-memory tiles of 32 positions with bulk asynchronous copies (the TMA engine's
//     untiled form, cp.async.bulk), one instruction per page of keys or values (the cache stores
//     rows with permuted 16-byte chunks so that a page copied as it is can be read without bank
//     conflicts), completion counted on an mbarrier per tile; it waits only for a tile's slot to be
//     handed back, so the ring, nearly all of the SM's shared memory, stays full of copies in
//     flight, across item boundaries too;
//   * four consumer warps each take every fourth tile of the current item, whole: scores and
//     probabilities-times-values run on tensor cores (m16n8k16, the group's query heads padded to
//     the 16 rows), the softmax is online in float32; a consumer hands the slot back the moment
//     it has read it (rows it had to clear first are fenced towards the copy engine).  No barrier
//     spans the CTA inside an item.
// When an item's tiles are done the consumers merge their four states; the item's result is a
// partial one unless the item covers its row's whole context.  The last item of a (request,
// key/value head) to finish, found with an atomic counter, merges the splits' partial results, so
// no CTA ever waits for another and there is no second launch.
//
// The kernel is launched as a programmatic dependent of the kernel before it: its CTAs fill their
// rings with keys and values of old positions while that kernel is still running, and wait for it
// only before they touch what it wrote (the queries, a row's newest key and value).  Asked to, it
// also does that kernel's work (zb_paged_decode_fused): the first producer warp forms an item's
// queries from the raw projection (per-head RMS norm, rotation), and the producer whose turn it is
// to copy the tile of a row's newest position first writes that key and value into the cache.
//
// Math as in attention_simt.cu (reference: src/attention/paged_decode.cu:169-352 for the split
// scheme), except where that kernel is not exact: no epsilon is added to the denominator, and
// partial results stay float32.  Probabilities are rounded to bfloat16 for the second product, as
// the reference does (paged_decode.cu:289).  Every wait is bounded and reports instead of hanging.
#include <algorithm>

#include "common.cuh"
#include "mma.cuh"

namespace zb {

constexpr int DEC_CONSUMERS = 4;
constexpr int DEC_PRODUCERS = 3;         // producer warps take tiles in turn: one warp cannot issue copies fast enough to fill the memory pipe
constexpr int DEC_THREADS = (DEC_CONSUMERS + DEC_PRODUCERS) * 32;   // consumers are warps 0..3, producers the warps after them
constexpr int DEC_TILE = 32;             // positions per tile: one consumer warp's unit of work
constexpr int DEC_MAX_GROUP = 16;        // query heads per key/value head that fit one MMA tile
constexpr int DEC_WAIT_LIMIT = 1 << 24;  // polls of an mbarrier before a warp gives up and reports
constexpr int DEC_SMEM_BUDGET = 227 * 1024 - 1024;
constexpr int DEC_MAX_BALANCED_GRID = 256;  // CTAs of a launch with balanced items: the scratch holds two slots for each

struct DecodeArgs {
  const __nv_bfloat16* q;        // [T, nh*hd]
  __nv_bfloat16* out;            // [T, nh*hd]
  const __nv_bfloat16* kv_cache; // [num_pages][2][nkv][page_size][hd]
  const int* block_table;        // [R, max_blocks]
  const int* rows;               // [n_rows] request rows that decode one token
  const int* row_q_start;        // [R]
  const int* row_ctx;            // [R] tokens in the cache before this step (the new token's position)
  float* part_o;                 // [slots][g][hd]: partial outputs, one slot per item that is not its pair's only one
  float* part_ml;                // [slots][g][2]: their maxima and sums
  int* counters;                 // [n_rows, nkv] zero on entry, zero again on exit
  int max_blocks, page_shift, num_pages, num_rows, n_rows;
  int nh, nkv, window, split_size, max_splits, ring_slots, item_pages;
  float scale_log2;              // scale * log2(e)
  int* status;
  // Position encoding inside this kernel (`qkv` null: off; q then holds finished queries and the
  // cache the newest keys and values).  With it, q is not read: a request's new token lies raw in
  // qkv (query heads, key heads, value heads); every CTA norms and rotates the queries of its own
  // items, and the consumer warp that meets the tile of a row's newest position norms and rotates
  // that key, puts it and the value into the tile in shared memory and into the cache.
  const __nv_bfloat16* qkv;      // [T, qkv_stride]
  long long qkv_stride;
  const void* q_norm_w;          // [hd] or null
  const void* k_norm_w;
  int norm_w_dtype;
  float norm_eps;
  const float* cos_table;        // [max_positions, hd / 2] or null (no rotation)
  const float* sin_table;
  int max_positions;
  int* trace;                    // null, or [CTA][8] ints: the global timer (ns, low 32 bits) at the CTA's start, after
                                 // the wait for earlier kernels, when its first tile had landed, after its last tile,
                                 // at its end; then its items and its tiles, and when its last arrival among a
                                 // row's splits was counted
};

__device__ __forceinline__ int timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return static_cast<int>(t);
}

// How a (request, key/value head) pair's context is cut into work items.
//   Fixed splits (split_size > 0): item = (row, head, split of split_size positions); CTAs take items in
//     turn.  A pair's partial results lie in slots pair * max_splits + split.
//   Balanced (split_size == 0): the tiles of all pairs, laid end to end, are cut into ranges of equal
//     length, one range per CTA; an item is the part of a pair inside a range.  A CTA's range may
//     begin inside one pair and end inside another, so a range owns two slots: slot 0 for a pair that
//     began before the range, slot 1 for one that began inside it and goes on.  Every CTA streams
//     the same number of tiles whatever the batch and the context lengths are.
struct DecodeItem {
  int r, row, kvh, ctx_total, begin, end, first_tile, n_tiles;
  int n_parts;          // items the pair is cut into (1: this item's result is the pair's result)
  int my_slot;          // where this item's partial result goes
  int merge_first;      // fixed: slot of the pair's first item; balanced: the pair's first range
  long long pair_start; // balanced: the pair's first tile in the global order
};

struct ItemWalker {
  int next;             // fixed: the next item number; balanced: the next range
  int tile, range, range_end, r;
};

// Positions [begin, end) of split `s` of a row; empty if begin >= end.
__device__ __forceinline__ void split_range(int ctx_total, int window, int split_size, int s, int& begin, int& end) {
  const int lo = window > 0 ? max(0, ctx_total - window) : 0;   // the query sits at ctx_total - 1
  begin = max(s * split_size, lo);
  end = min((s + 1) * split_size, ctx_total);
}

__device__ __forceinline__ int balanced_slot(long long pair_start, int range, int per_range) {
  return range * 2 + (pair_start < static_cast<long long>(range) * per_range ? 0 : 1);
}

__device__ __forceinline__ void walker_init(ItemWalker& w) {
  w.next = blockIdx.x;
  w.tile = w.range_end = w.range = w.r = 0;
}

// The CTA's next item, the same sequence for every warp that asks.  `prefix` (balanced only): the
// first global tile of every row, n_rows + 1 entries; `per_range`: tiles per range.
__device__ __forceinline__ bool next_item(const DecodeArgs& a, const int* prefix, int per_range, ItemWalker& w,
                                          DecodeItem& it) {
  if (a.split_size > 0) {
    const int n_items = a.n_rows * a.nkv * a.max_splits;
    while (w.next < n_items) {
      const int id = w.next;
      w.next += gridDim.x;
      const int split = id % a.max_splits;
      it.kvh = (id / a.max_splits) % a.nkv;
      it.r = id / (a.max_splits * a.nkv);
      it.row = a.rows[it.r];
      if (it.row < 0 || it.row >= a.num_rows) continue;            // reported when the kernel starts
      it.ctx_total = a.row_ctx[it.row] + 1;
      split_range(it.ctx_total, a.window, a.split_size, split, it.begin, it.end);
      if (it.begin >= it.end) continue;
      it.first_tile = it.begin / DEC_TILE * DEC_TILE;
      it.n_tiles = (it.end - it.first_tile + DEC_TILE - 1) / DEC_TILE;
      const int lo = a.window > 0 ? max(0, it.ctx_total - a.window) : 0;
      const int first_split = lo / a.split_size, last_split = (it.ctx_total - 1) / a.split_size;
      it.n_parts = last_split - first_split + 1;
      it.merge_first = (it.r * a.nkv + it.kvh) * a.max_splits + first_split;
      it.my_slot = (it.r * a.nkv + it.kvh) * a.max_splits + split;
      it.pair_start = 0;
      return true;
    }
    return false;
  }
  const int total = prefix[a.n_rows];
  while (true) {
    if (w.tile >= w.range_end) {
      const long long begin = static_cast<long long>(w.next) * per_range;
      if (begin >= total) return false;
      w.range = w.next;
      w.next += gridDim.x;
      w.tile = static_cast<int>(begin);
      w.range_end = min(total, w.tile + per_range);
    }
    while (prefix[w.r + 1] <= w.tile) ++w.r;                        // ranges only move forward
    const int row_tiles = (prefix[w.r + 1] - prefix[w.r]) / a.nkv;
    it.r = w.r;
    it.row = a.rows[w.r];
    it.kvh = (w.tile - prefix[w.r]) / row_tiles;
    it.pair_start = prefix[w.r] + it.kvh * row_tiles;
    const int seg_end = min(w.range_end, static_cast<int>(it.pair_start) + row_tiles);
    it.ctx_total = a.row_ctx[it.row] + 1;
    const int lo = a.window > 0 ? max(0, it.ctx_total - a.window) : 0;
    const int first = lo / DEC_TILE + (w.tile - static_cast<int>(it.pair_start));   // the item's first tile of the row
    it.n_tiles = seg_end - w.tile;
    it.first_tile = first * DEC_TILE;
    it.begin = max(lo, it.first_tile);
    it.end = min(it.ctx_total, (first + it.n_tiles) * DEC_TILE);
    const int first_range = static_cast<int>(it.pair_start / per_range);
    const int last_range = static_cast<int>((it.pair_start + row_tiles - 1) / per_range);
    it.n_parts = last_range - first_range + 1;
    it.merge_first = first_range;
    it.my_slot = balanced_slot(it.pair_start, w.range, per_range);
    w.tile = seg_end;
    return true;
  }
}

// Slot of the k-th of the pair's partial results.
__device__ __forceinline__ int part_slot(const DecodeArgs& a, const DecodeItem& it, int k, int per_range) {
  return a.split_size > 0 ? it.merge_first + k : balanced_slot(it.pair_start, it.merge_first + k, per_range);
}

__device__ __forceinline__ void consumer_barrier() {      // the 128 consumer threads only
  asm volatile("bar.sync 1, %0;\n" ::"n"(DEC_CONSUMERS * 32) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}

// One head of a new token by one warp, as zb_qk_norm_rope_cache does it (rope_cache.cu: the same
// sums, factors and roundings): lane l owns the adjacent elements 2l, 2l + 1 of the head's first half
// and their partners in the second.  `norm_w` null: no norm; `rotate` false: no rotation (a value).
// Returns false for lanes that own nothing (head sizes below 128).
template <int HD>
__device__ __forceinline__ bool new_token_head(const __nv_bfloat16* src, const void* norm_w, int w_dtype, float eps,
                                               const float* cos_row, const float* sin_row, float (&x)[2], float (&y)[2]) {
  constexpr int HALF = HD / 2;
  const int lane = threadIdx.x & 31, i = 2 * lane;
  const bool mine = i < HALF;
  x[0] = x[1] = y[0] = y[1] = 0.0f;
  float ss = 0.0f;
  if (mine) {
    const float2 xv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + i));
    const float2 yv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + i + HALF));
    x[0] = xv.x; x[1] = xv.y; y[0] = yv.x; y[1] = yv.y;
    ss = x[0] * x[0] + x[1] * x[1] + y[0] * y[0] + y[1] * y[1];
  }
  if (norm_w != nullptr) {
    const float inv = rsqrtf(warp_sum(ss) / static_cast<float>(HD) + eps);
    if (mine) {
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        x[u] *= inv * load_scale(norm_w, w_dtype, i + u);
        y[u] *= inv * load_scale(norm_w, w_dtype, i + u + HALF);
      }
    }
  }
  if (cos_row != nullptr && mine) {
    const float2 cv = *reinterpret_cast<const float2*>(cos_row + i), sv = *reinterpret_cast<const float2*>(sin_row + i);
    const float cs[2] = {cv.x, cv.y}, sn[2] = {sv.x, sv.y};
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const float xr = x[u] * cs[u] - y[u] * sn[u];
      const float yr = y[u] * cs[u] + x[u] * sn[u];
      x[u] = xr;
      y[u] = yr;
    }
  }
  return mine;
}

// Whether merge_many_parts finds room for `n_parts` splits where the consumers' parts lay.
__device__ __forceinline__ bool merge_staging_fits(int n_parts, int g, int hd) {
  const int n_vec = g * hd / 4;
  return n_parts * g * 2 + g + 4 + (n_vec <= DEC_CONSUMERS * 16 ? n_vec * 4 : 0) <= DEC_CONSUMERS * g * hd;
}

// The last CTA of a (row, key/value head) pair to arrive merges the pair's more than a few splits;
// called by the 128 consumer threads together.  A function of its own: inlined, its registers
// changed the allocation of the kernel's main loop, which runs at the register limit.
// All loads of a round are issued before the first is used: a merge costs a few round trips to the
// L2, not one per split.  A thread takes whole vectors of four floats (16-byte loads), and where the
// vectors leave half of the threads idle, two halves of the threads share a vector's splits (even
// and odd ones) and add their sums at the end.  (Element by element the compiler strung a thread's
// loads one behind the other: 0.28 us a split.)
struct MergeJob {                        // what merge_many_parts needs of the launch and the item, by value
  const float* part_o;
  const float* part_ml;
  __nv_bfloat16* out;                    // the pair's first output element
  long long pair_start;
  int n_parts, merge_first, per_range, split_size, g;
  __device__ __forceinline__ int slot(int k) const {
    return split_size > 0 ? merge_first + k : balanced_slot(pair_start, merge_first + k, per_range);
  }
};

template <int HD>
__device__ __noinline__ void merge_many_parts(const MergeJob job, float* merge_o) {
  constexpr int BATCH = 8;
  const int g = job.g;
  const struct { int n_parts; } it = {job.n_parts};
  const int ctid = threadIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* ml_s = merge_o;                 // [n_parts][g][2], where the consumers' parts lay (they are merged by now)
  const int n_vec = g * HD / 4;          // the result as vectors of four floats
  const int groups = n_vec <= DEC_CONSUMERS * 16 ? 2 : 1, per_group = DEC_CONSUMERS * 32 / groups;
  const int grp = ctid / per_group, idx = ctid - grp * per_group;
  float4* sums_s = reinterpret_cast<float4*>(
      reinterpret_cast<uintptr_t>(merge_o + it.n_parts * g * 2 + g + 3) & ~static_cast<uintptr_t>(15));    // behind the weights
    // This thread's first vector's shares of its first BATCH splits are asked for before the maxima
    // are staged, so that both travel at the same time.
    float4 first[BATCH];
    {
      const int h = idx * 4 / HD, d = idx * 4 - h * HD;
#pragma unroll
      for (int u = 0; u < BATCH; ++u) {
        const int k = grp + u * groups;
        first[u] = idx < n_vec && k < it.n_parts
                       ? __ldcg(reinterpret_cast<const float4*>(&job.part_o[(static_cast<size_t>(job.slot(k)) * g + h) * HD + d]))
                       : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      }
    }
    for (int e = ctid; e < it.n_parts * g * 2; e += DEC_CONSUMERS * 32) {
      const int k = e / (g * 2), rest = e - k * g * 2;
      ml_s[e] = __ldcg(&job.part_ml[static_cast<size_t>(job.slot(k)) * g * 2 + rest]);
    }
    consumer_barrier();
    // One warp per head turns the maxima into the splits' weights, exp2(m_k - max), in place, and
    // leaves the head's weighted sum of the l_k behind the list: the vectors below then cost a
    // multiply-add per split and element.
    for (int h = warp; h < g; h += DEC_CONSUMERS) {
      float mx = -INFINITY;
      for (int k = lane; k < it.n_parts; k += 32) mx = fmaxf(mx, ml_s[(k * g + h) * 2]);
      mx = warp_max(mx);
      float lsum = 0.0f;
      for (int k = lane; k < it.n_parts; k += 32) {
        const float f = exp2f(ml_s[(k * g + h) * 2] - mx);
        lsum += ml_s[(k * g + h) * 2 + 1] * f;
        ml_s[(k * g + h) * 2] = f;
      }
      lsum = warp_sum(lsum);
      if (lane == 0) ml_s[it.n_parts * g * 2 + h] = lsum;
    }
    consumer_barrier();
    for (int v0 = 0; v0 < n_vec; v0 += per_group) {         // the same number of turns for every thread: barriers inside
      const int v = v0 + idx;
      const bool mine = v < n_vec;
      const int h = mine ? v * 4 / HD : 0, d = mine ? v * 4 - h * HD : 0;
      float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      for (int kb = grp; kb < it.n_parts; kb += groups * BATCH) {
        float4 po[BATCH];
#pragma unroll
        for (int u = 0; u < BATCH; ++u) {
          const int k = kb + u * groups;
          if (v0 == 0 && kb == grp) po[u] = first[u];
          else
            po[u] = mine && k < it.n_parts
                        ? __ldcg(reinterpret_cast<const float4*>(&job.part_o[(static_cast<size_t>(job.slot(k)) * g + h) * HD + d]))
                        : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
#pragma unroll
        for (int u = 0; u < BATCH; ++u) {                      // a fixed order: the group's splits in the order of the context
          const int k = kb + u * groups;
          if (k < it.n_parts) {
            const float f = ml_s[(k * g + h) * 2];
            acc.x += po[u].x * f; acc.y += po[u].y * f; acc.z += po[u].z * f; acc.w += po[u].w * f;
          }
        }
      }
      if (groups == 2) {
        if (grp == 1 && mine) sums_s[idx] = acc;
        consumer_barrier();
        if (grp == 0 && mine) {
          const float4 other = sums_s[idx];
          acc.x += other.x; acc.y += other.y; acc.z += other.z; acc.w += other.w;
        }
      }
      if (grp == 0 && mine) {
        const float l = ml_s[it.n_parts * g * 2 + h];
        const float inv = l > 0.0f ? 1.0f / l : 0.0f;
        uint2 packed;
        packed.x = pack_bf16(acc.x * inv, acc.y * inv);
        packed.y = pack_bf16(acc.z * inv, acc.w * inv);
        *reinterpret_cast<uint2*>(&job.out[v * 4]) = packed;
      }
      if (groups == 2 && v0 + per_group < n_vec) consumer_barrier();     // the sums' buffer is read before the next turn writes it
    }
}

template <int HD>
__global__ void __launch_bounds__(DEC_THREADS, 1)
paged_decode_kernel(const DecodeArgs a) {
  static_assert(HD % 32 == 0 && HD <= 128, "head sizes 32, 64, 96, 128");
  constexpr int KROW = HD + 8;                     // padded row of the query buffer
  constexpr int CHUNKS = HD / 8;                   // 16-byte chunks of a cache row
  // A ring slot holds 32 key rows and 32 value rows exactly as they lie in the cache pages: back to
  // back, chunks permuted (kv_swizzle), which is what makes unpadded rows conflict-free for ldmatrix.
  constexpr int SLOT = 2 * DEC_TILE * HD;
  constexpr unsigned ROW_BYTES = HD * sizeof(__nv_bfloat16);
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int g = a.nh / a.nkv, R = a.ring_slots;
  __nv_bfloat16* ring = reinterpret_cast<__nv_bfloat16*>(smem_raw);                 // [R][2][DEC_TILE][HD]
  __nv_bfloat16* qbuf = ring + static_cast<size_t>(R) * SLOT;                        // [2][16][KROW]
  float* merge_o = reinterpret_cast<float*>(qbuf + 2 * 16 * KROW);                   // [consumers][g][HD]
  float* merge_ml = merge_o + DEC_CONSUMERS * g * HD;                                // [consumers][g][2]
  unsigned long long* full = reinterpret_cast<unsigned long long*>(merge_ml + DEC_CONSUMERS * g * 2);
  unsigned long long* empty = full + R;
  unsigned long long* qfull = empty + R;
  unsigned long long* qempty = qfull + 2;
  int* page_ids_all = reinterpret_cast<int*>(qempty + 2);     // the current item's pages, one list per producer warp
  int* prefix = page_ids_all + DEC_PRODUCERS * a.item_pages;  // balanced items: every row's first global tile, n_rows + 1
  // How many fillings of each slot have been read to the end.  Several producers and consumers
  // run at their own pace, and an mbarrier's parity tells apart two successive phases only: nobody
  // waits for a slot's n-th filling, or for its release, before the count says the fillings before
  // it are done with.
  volatile int* consumed = prefix + a.n_rows + 2;
  __shared__ int is_last;
  __shared__ volatile int abort_flag;      // set by the first warp whose wait ran out; every later wait gives up at once

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) abort_flag = 0;
  int* const trace = a.trace != nullptr && threadIdx.x == 0 ? a.trace + 8 * blockIdx.x : nullptr;
  if (trace) trace[0] = timer_ns();
  // A bounded wait that also ends when another warp has given up.
  auto wait = [&](unsigned long long* bar, unsigned parity) -> bool {
    for (int i = 0; i < DEC_WAIT_LIMIT; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
      if ((i & 63) == 63 && abort_flag) return false;
    }
    return false;
  };
  for (int e = threadIdx.x; e < 2 * 16 * KROW / 8; e += DEC_THREADS)
    reinterpret_cast<uint4*>(qbuf)[e] = make_uint4(0, 0, 0, 0);      // rows past the group stay zero for good
  if (threadIdx.x == 0) {
    for (int s = 0; s < R; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); consumed[s] = 0; }
    for (int s = 0; s < 2; ++s) { mbar_init(&qfull[s], 1); mbar_init(&qempty[s], DEC_CONSUMERS); }
    fence_barrier_init();
  }
  // Rows that do not exist are reported once and own no tiles.
  for (int r = threadIdx.x; r < a.n_rows; r += DEC_THREADS) {
    // In a step of decoding requests only, row r is request r: its context is asked for together with
    // its number, which saves a round trip to memory at the head of every launch.
    const int guess = r < a.num_rows ? a.row_ctx[r] : 0;
    const int row = a.rows[r];
    if (a.split_size > 0 && r < a.num_rows)      // fixed splits: the producers ask for it next; let it be on its way
      asm volatile("prefetch.global.L1 [%0];\n" ::"l"(a.row_ctx + r));
    const bool ok = row >= 0 && row < a.num_rows;
    if (!ok) report(a.status, STATUS_ROW_OUT_OF_RANGE, row, r);
    if (a.split_size == 0) {
      int tiles = 0;
      if (ok) {
        const int ctx_total = (row == r ? guess : a.row_ctx[row]) + 1;
        const int lo = a.window > 0 ? max(0, ctx_total - a.window) : 0;
        tiles = (ctx_total + DEC_TILE - 1) / DEC_TILE - lo / DEC_TILE;
      }
      prefix[r + 1] = tiles * a.nkv;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && a.split_size == 0) {
    prefix[0] = 0;
    for (int r = 0; r < a.n_rows; ++r) prefix[r + 1] += prefix[r];
  }
  __syncthreads();
  fence_proxy_async();
  // Up to here nothing of an earlier kernel's output was read: the step's description is older than
  // any kernel of the step.  The queries and each row's newest key and value are an earlier kernel's
  // output; the rest of the cache is older than the step.  So the consumers wait for the earlier
  // kernels at once, and a producer only before the first copy that reads their output: the ring
  // fills with old keys and values while the kernel before this one is still running.
  let_dependents_launch();
  // Balanced items: as many tiles per range as spread all tiles evenly over the CTAs.
  const int per_range = a.split_size == 0 ? max(1, (prefix[a.n_rows] + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x)) : 0;
  const int page_size = 1 << a.page_shift;
  const long long page_stride = 2LL * a.nkv * page_size * HD;
  const bool fused = a.qkv != nullptr;       // the new tokens' position encoding happens in this kernel

  if (warp >= DEC_CONSUMERS) {
    // ------------------------------------------------------------------------ the producers
    // Both walk the same items and tiles; a tile belongs to the producer its number names, and
    // the first producer also fetches the queries.
    const int me = warp - DEC_CONSUMERS;
    int* page_ids = page_ids_all + me * a.item_pages;
    int tile_seq = 0, item_seq = 0;
    ItemWalker walker;
    walker_init(walker);
    DecodeItem it;
    bool waited = false;               // for the earlier kernels
    bool q_pending = false;            // the first producer: the item's queries are still to be fetched
    // With the position encoding inside the kernel the producers do its work, off the consumers'
    // path: the first producer forms an item's queries from the raw projection (the consumers find
    // them in the query buffer as if they had been copied there), and the producer whose turn it
    // is to copy the tile of a row's newest position first forms that key, writes it and the value
    // into the cache, and then copies the tile like any other.
    auto rotation_rows = [&](const float*& cos_row, const float*& sin_row) {
      const int pos = it.ctx_total - 1;
      const bool ok = a.cos_table != nullptr && pos >= 0 && pos < a.max_positions;
      if (a.cos_table != nullptr && !ok && lane == 0) report(a.status, STATUS_POSITION_OUT_OF_RANGE, pos, it.row);
      cos_row = ok ? a.cos_table + static_cast<size_t>(pos) * (HD / 2) : nullptr;
      sin_row = ok ? a.sin_table + static_cast<size_t>(pos) * (HD / 2) : nullptr;
    };
    auto fetch_queries = [&](int qb) {
      if (fused) {
        const __nv_bfloat16* token = a.qkv + static_cast<size_t>(a.row_q_start[it.row]) * a.qkv_stride;
        const float *cos_row, *sin_row;
        rotation_rows(cos_row, sin_row);
        for (int h = 0; h < g; ++h) {
          float x[2], y[2];
          if (new_token_head<HD>(token + static_cast<size_t>(it.kvh * g + h) * HD, a.q_norm_w, a.norm_w_dtype, a.norm_eps,
                                 cos_row, sin_row, x, y)) {
            __nv_bfloat16* dst = qbuf + (qb * 16 + h) * KROW + 2 * lane;
            *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(x[0], x[1]);
            *reinterpret_cast<__nv_bfloat162*>(dst + HD / 2) = __floats2bfloat162_rn(y[0], y[1]);
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&qfull[qb]);        // a release: the consumers' wait sees the stores
        return;
      }
      if (lane == 0) mbar_arrive_expect_tx(&qfull[qb], static_cast<unsigned>(g) * ROW_BYTES);
      if (lane < g)
        bulk_copy_g2s(qbuf + (qb * 16 + lane) * KROW,
                      a.q + (static_cast<size_t>(a.row_q_start[it.row]) * a.nh + static_cast<size_t>(it.kvh) * g + lane) * HD,
                      ROW_BYTES, &qfull[qb]);
    };
    // The new token's key and value into the cache (their row of the page, chunks permuted as
    // every cache row's are).
    auto write_newest = [&]() {
      const int pos = it.ctx_total - 1;
      const int block = pos >> a.page_shift;
      const int page = block < a.max_blocks ? a.block_table[static_cast<size_t>(it.row) * a.max_blocks + block] : -1;
      if (page <= 0 || page >= a.num_pages) {
        if (lane == 0) report(a.status, STATUS_PAGE_OUT_OF_RANGE, page, it.row);
        return;
      }
      const __nv_bfloat16* token = a.qkv + static_cast<size_t>(a.row_q_start[it.row]) * a.qkv_stride;
      const float *cos_row, *sin_row;
      rotation_rows(cos_row, sin_row);
      __nv_bfloat16* key_row = const_cast<__nv_bfloat16*>(a.kv_cache) + page * page_stride +
                               (static_cast<long long>(it.kvh) * page_size + (pos & (page_size - 1))) * HD;
      const int lo = kv_element_index(2 * lane, pos, HD, sizeof(__nv_bfloat16));
      const int hi = kv_element_index(2 * lane + HD / 2, pos, HD, sizeof(__nv_bfloat16));
#pragma unroll
      for (int kind = 0; kind < 2; ++kind) {              // the key, then the value
        float x[2], y[2];
        if (new_token_head<HD>(token + static_cast<size_t>(a.nh + kind * a.nkv + it.kvh) * HD, kind == 0 ? a.k_norm_w : nullptr,
                               a.norm_w_dtype, a.norm_eps, kind == 0 ? cos_row : nullptr, kind == 0 ? sin_row : nullptr, x, y)) {
          __nv_bfloat16* row = key_row + (kind == 0 ? 0 : static_cast<long long>(a.nkv) * page_size * HD);
          *reinterpret_cast<__nv_bfloat162*>(row + lo) = __floats2bfloat162_rn(x[0], x[1]);
          *reinterpret_cast<__nv_bfloat162*>(row + hi) = __floats2bfloat162_rn(y[0], y[1]);
        }
      }
      __syncwarp();
      fence_proxy_async();       // the tile's bulk copies, issued next by this warp, read these rows
    };
    while (next_item(a, prefix, per_range, walker, it)) {
      const int qb = item_seq & 1;
      if (me == 0) {
        if (!wait(&qempty[qb], ((item_seq >> 1) & 1) ^ 1)) {
          if (lane == 0) report(a.status, STATUS_COPY_TIMEOUT, -1, it.row);
          abort_flag = 1;
          return;
        }
        // The queries are an earlier kernel's output.  Before the wait for it, the ring's first
        // filling goes out (nothing can hold those copies up); then the wait, then the queries.
        if (waited) fetch_queries(qb);
        else q_pending = true;
      }
      ++item_seq;
      // The item's page ids in one go (one round trip to memory per item instead of one per tile).
      const int* table = a.block_table + static_cast<size_t>(it.row) * a.max_blocks;
      const int first_block = it.first_tile >> a.page_shift;
      const int n_blocks = ((it.first_tile + it.n_tiles * DEC_TILE - 1) >> a.page_shift) - first_block + 1;
      for (int i = lane; i < n_blocks; i += 32)
        page_ids[i] = first_block + i < a.max_blocks ? table[first_block + i] : -1;
      __syncwarp();
      const __nv_bfloat16* base = a.kv_cache + static_cast<long long>(it.kvh) * page_size * HD;
      const long long v_offset = static_cast<long long>(a.nkv) * page_size * HD;
      // A tile's rows are copied in runs that are contiguous in the cache: a whole page at a time for
      // pages of up to 32 positions, a 32-row piece of a page for larger ones.  One bulk copy for
      // the keys of a run and one for its values: a handful of instructions move 16 KB.
      const int run_rows = page_size < DEC_TILE ? page_size : DEC_TILE;
      const int n_runs = DEC_TILE / run_rows;
      for (int t = 0; t < it.n_tiles; ++t, ++tile_seq) {
        if (tile_seq % DEC_PRODUCERS != me) continue;
        const int slot = tile_seq % R, filling = tile_seq / R;
        // The tile that holds the row's newest position was written by an earlier kernel of this step,
        // or is written here from that kernel's projection.
        const bool newest = it.first_tile + (t + 1) * DEC_TILE >= it.ctx_total;
        if (!waited && (newest || (q_pending && filling > 0))) {
          wait_for_prior_grids();
          waited = true;
        }
        if (q_pending && waited) {
          fetch_queries(qb);
          q_pending = false;
        }
        if (fused && newest) write_newest();
        bool released = consumed[slot] >= filling;
        for (int i = 0; !released && i < DEC_WAIT_LIMIT && !abort_flag; ++i) released = consumed[slot] >= filling;
        if (!released || !wait(&empty[slot], (filling & 1) ^ 1)) {
          if (lane == 0) report(a.status, STATUS_COPY_TIMEOUT, -2, it.row);
          abort_flag = 1;
          return;
        }
        const int p0 = it.first_tile + t * DEC_TILE + lane * run_rows;     // first position of this lane's run
        const bool copies = lane < n_runs && (p0 >> a.page_shift) < a.max_blocks;
        if (copies) {
          int page = page_ids[(p0 >> a.page_shift) - first_block];
          if (page <= 0 || page >= a.num_pages) {
            // Fine for a run nobody wants (a page given back behind a window, the tail of the table);
            // an error if one of its positions is in the item.  Either way the bytes must arrive.
            if (p0 + run_rows > it.begin && p0 < it.end) report(a.status, STATUS_PAGE_OUT_OF_RANGE, page, it.row);
            page = 0;
          }
          const __nv_bfloat16* src = base + page * page_stride + (p0 & (page_size - 1)) * HD;
          __nv_bfloat16* dst = ring + static_cast<size_t>(slot) * SLOT + lane * run_rows * HD;
          // Self-check: both copies lie inside the cache.  One that does not is reported and replaced
          // by a copy from the null page.
          const long long src_off = src - a.kv_cache, cache_elems = static_cast<long long>(a.num_pages) * page_stride;
          if (src_off < 0 || src_off + v_offset + run_rows * HD > cache_elems) {
            report(a.status, STATUS_INTERNAL_CHECK, static_cast<int>(src_off >> 10), it.row);
            src = base;
          }
          bulk_copy_g2s(dst, src, run_rows * ROW_BYTES, &full[slot]);
          bulk_copy_g2s(dst + DEC_TILE * HD, src + v_offset, run_rows * ROW_BYTES, &full[slot]);
        }
        const unsigned copied_runs = __popc(__ballot_sync(0xffffffffu, copies));
        if (lane == 0) mbar_arrive_expect_tx(&full[slot], copied_runs * run_rows * 2u * ROW_BYTES);
      }
      if (q_pending) {         // an item with few tiles, none of them the newest
        wait_for_prior_grids();
        waited = true;
        fetch_queries(qb);
        q_pending = false;
      }
      __syncwarp();            // every lane is done with this item's page ids before the next item's overwrite them
    }
    return;
  }

  // ---------------------------------------------------------------------------- the consumers
  const int quad_row = lane >> 2, quad_col = (lane & 3) * 2;
  const int ctid = threadIdx.x;                       // 0..127 among the consumers
  int tile_base = 0, item_seq = 0;
  ItemWalker walker;
  walker_init(walker);
  DecodeItem it;
  wait_for_prior_grids();      // the consumers write results, and read queries: both wait for the kernels before
  if (trace) trace[1] = trace[2] = trace[3] = timer_ns();
  while (next_item(a, prefix, per_range, walker, it)) {
    const int qb = item_seq & 1;
    // A consumer whose wait runs out reports, raises the abort flag and keeps walking the items
    // without computing: the consumer barriers below need all four warps to the very end.
    if (!wait(&qfull[qb], (item_seq >> 1) & 1)) {
      if (lane == 0 && !abort_flag) report(a.status, STATUS_COPY_TIMEOUT, -3, it.row);
      abort_flag = 1;
    }
    ++item_seq;
    // The group's queries as the A operand (heads on the 16 rows; rows past the group are zero).
    unsigned qa[HD / 16][4];
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks)
      ldmatrix_x4(qa[ks], qbuf + (qb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * KROW + ks * 16 + (lane >> 4) * 8);
    __syncwarp();
    if (lane == 0) mbar_arrive(&qempty[qb]);

    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    float o[HD / 8][4];
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;

    for (int j = warp; j < it.n_tiles; j += DEC_CONSUMERS) {
      const int seq = tile_base + j, slot = seq % R, filling = seq / R;
      bool in_turn = consumed[slot] == filling;
      for (int i = 0; !in_turn && i < DEC_WAIT_LIMIT && !abort_flag; ++i) in_turn = consumed[slot] == filling;
      if (abort_flag || !in_turn || !wait(&full[slot], filling & 1)) {
        if (lane == 0 && !abort_flag) report(a.status, STATUS_COPY_TIMEOUT, j, it.row);
        abort_flag = 1;
        break;
      }
      if (trace && seq == 0) trace[2] = timer_ns();
      __nv_bfloat16* ks_tile = ring + static_cast<size_t>(slot) * SLOT;
      __nv_bfloat16* vs_tile = ks_tile + DEC_TILE * HD;
      const int key0 = it.first_tile + j * DEC_TILE;
      if (key0 < it.begin || key0 + DEC_TILE > it.end) {
        // The tile reaches past the item: those rows came along with their page and may hold
        // anything (another request's old values, NaN).  Their scores are masked below; their value
        // rows are cleared so that a probability of zero times such a row stays zero.
        const int pos = key0 + lane;
        if (lane < DEC_TILE && (pos < it.begin || pos >= it.end)) {
#pragma unroll
          for (int c = 0; c < CHUNKS; ++c) *reinterpret_cast<uint4*>(vs_tile + lane * HD + c * 8) = make_uint4(0, 0, 0, 0);
          fence_proxy_async();   // these ordinary stores come before the next bulk copy into the slot
        }
        __syncwarp();
      }
      const int swz = kv_swizzle(lane & 7, CHUNKS);      // a tile starts at a multiple of 32: row bits = lane bits

      // Scores of the tile's 32 keys: four n-tiles of 8, each its own accumulator chain.
      float s[DEC_TILE / 8][4];
#pragma unroll
      for (int nt = 0; nt < DEC_TILE / 8; ++nt) {
        s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f;
#pragma unroll
        for (int kk = 0; kk < HD / 32; ++kk) {
          unsigned b[4];
          ldmatrix_x4(b, ks_tile + (nt * 8 + (lane & 7)) * HD + (((kk * 4 + (lane >> 3)) ^ swz) << 3));
          mma_bf16_16816(s[nt], qa[2 * kk], b[0], b[1]);
          mma_bf16_16816(s[nt], qa[2 * kk + 1], b[2], b[3]);
        }
      }
      float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < DEC_TILE / 8; ++nt) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int pos = key0 + nt * 8 + quad_col + (c & 1);
          const bool valid = pos >= it.begin && pos < it.end;
          s[nt][c] = valid ? s[nt][c] * a.scale_log2 : -INFINITY;
          tile_max[c >> 1] = fmaxf(tile_max[c >> 1], s[nt][c]);
        }
      }
      float corr[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 1));
        tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 2));
        const float new_m = fmaxf(m_run[h], tile_max[h]);     // finite: every tile of an item holds a wanted key
        corr[h] = exp2f(m_run[h] - new_m);
        m_run[h] = new_m;
      }
      float row_sum[2] = {0.0f, 0.0f};
#pragma unroll
      for (int nt = 0; nt < DEC_TILE / 8; ++nt) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          s[nt][c] = exp2f(s[nt][c] - m_run[c >> 1]);          // exp2(-inf) = 0 for masked keys
          row_sum[c >> 1] += s[nt][c];
        }
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        row_sum[h] += __shfl_xor_sync(0xffffffffu, row_sum[h], 1);
        row_sum[h] += __shfl_xor_sync(0xffffffffu, row_sum[h], 2);
        l_run[h] = l_run[h] * corr[h] + row_sum[h];
      }
      // Once the running maximum has settled, corr is exactly 1 for every row and nothing is rescaled.
      if (!__all_sync(0xffffffffu, corr[0] == 1.0f && corr[1] == 1.0f)) {
#pragma unroll
        for (int n = 0; n < HD / 8; ++n) {
          o[n][0] *= corr[0]; o[n][1] *= corr[0]; o[n][2] *= corr[1]; o[n][3] *= corr[1];
        }
      }
#pragma unroll
      for (int ks = 0; ks < DEC_TILE / 16; ++ks) {
        unsigned pa[4];
        pa[0] = pack_bf16(s[2 * ks][0], s[2 * ks][1]);
        pa[1] = pack_bf16(s[2 * ks][2], s[2 * ks][3]);
        pa[2] = pack_bf16(s[2 * ks + 1][0], s[2 * ks + 1][1]);
        pa[3] = pack_bf16(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
        for (int n2 = 0; n2 < HD / 16; ++n2) {
          unsigned b[4];
          ldmatrix_x4_trans(b, vs_tile + (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * HD +
                                   (((n2 * 2 + (lane >> 4)) ^ swz) << 3));
          mma_bf16_16816(o[2 * n2], pa, b[0], b[1]);
          mma_bf16_16816(o[2 * n2 + 1], pa, b[2], b[3]);
        }
      }
      __syncwarp();            // every lane has read the tile
      if (lane == 0) {
        consumed[slot] = filling + 1;
        mbar_arrive(&empty[slot]);
      }
    }
    tile_base += it.n_tiles;
    if (trace) trace[3] = timer_ns();

    // Merge the four consumers (each saw its own tiles).  Only the group's rows are kept.
    consumer_barrier();        // the merge buffers of the previous item are no longer read
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int head = quad_row + 8 * h;
      if (head < g) {
        float* dst = merge_o + (warp * g + head) * HD + quad_col;
#pragma unroll
        for (int n = 0; n < HD / 8; ++n) {
          dst[n * 8] = o[n][2 * h];
          dst[n * 8 + 1] = o[n][2 * h + 1];
        }
        if ((lane & 3) == 0) {
          merge_ml[(warp * g + head) * 2] = m_run[h];
          merge_ml[(warp * g + head) * 2 + 1] = l_run[h];
        }
      }
    }
    consumer_barrier();

    const bool alone = it.n_parts == 1;
    const size_t out_base = (static_cast<size_t>(a.row_q_start[it.row]) * a.nh + static_cast<size_t>(it.kvh) * g) * HD;
    for (int e = ctid; e < g * HD; e += DEC_CONSUMERS * 32) {
      const int h = e / HD, d = e - h * HD;
      float mx = -INFINITY;
#pragma unroll
      for (int w = 0; w < DEC_CONSUMERS; ++w) mx = fmaxf(mx, merge_ml[(w * g + h) * 2]);
      float acc = 0.0f, l = 0.0f;
#pragma unroll
      for (int w = 0; w < DEC_CONSUMERS; ++w) {
        const float mw = merge_ml[(w * g + h) * 2];
        const float f = mw == -INFINITY ? 0.0f : exp2f(mw - mx);    // a consumer without a tile of this item
        acc += merge_o[(w * g + h) * HD + d] * f;
        l += merge_ml[(w * g + h) * 2 + 1] * f;
      }
      if (alone) {               // the only split of its row: this is the result
        a.out[out_base + e] = __float2bfloat16_rn(l > 0.0f ? acc / l : 0.0f);
      } else {
        const size_t slot = static_cast<size_t>(it.my_slot) * g + h;
        a.part_o[slot * HD + d] = acc;
        if (d == 0) {
          a.part_ml[slot * 2] = mx;
          a.part_ml[slot * 2 + 1] = l;
        }
      }
    }
    if (alone) continue;

    // Whoever arrives last finds every split's partial result written and merges them.  The barrier
    // orders the consumers' writes before the arrival, whose release makes them visible to whoever
    // reads the count with acquire; the barrier after it passes that on to the other consumers.
    consumer_barrier();
    if (ctid == 0) {
      int arrived;
      asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;"
                   : "=r"(arrived) : "l"(&a.counters[it.r * a.nkv + it.kvh]) : "memory");
      is_last = arrived == it.n_parts - 1;
    }
    consumer_barrier();
    if (trace) trace[7] = timer_ns();
    if (!is_last) continue;
    // All loads of a round are issued before the first is used: a merge costs a few round trips to
    // the L2, not one per split.
    constexpr int ROUND = 4;
    const bool staged = it.n_parts > ROUND && merge_staging_fits(it.n_parts, g, HD);
    if (staged) {
      MergeJob job;
      job.part_o = a.part_o; job.part_ml = a.part_ml; job.out = a.out + out_base;
      job.pair_start = it.pair_start;
      job.n_parts = it.n_parts; job.merge_first = it.merge_first; job.per_range = per_range; job.split_size = a.split_size; job.g = g;
      merge_many_parts<HD>(job, merge_o);
    } else {
      for (int e = ctid; e < g * HD; e += DEC_CONSUMERS * 32) {
        const int h = e / HD, d = e - h * HD;
        float acc = 0.0f, l = 0.0f;
        if (it.n_parts <= ROUND) {
          float pm[ROUND], pl[ROUND], po[ROUND];
#pragma unroll
          for (int k = 0; k < ROUND; ++k) {
            pm[k] = -INFINITY; pl[k] = 0.0f; po[k] = 0.0f;
            if (k < it.n_parts) {
              const size_t slot = static_cast<size_t>(part_slot(a, it, k, per_range)) * g + h;
              pm[k] = __ldcg(&a.part_ml[slot * 2]);
              pl[k] = __ldcg(&a.part_ml[slot * 2 + 1]);
              po[k] = __ldcg(&a.part_o[slot * HD + d]);
            }
          }
          float mx = pm[0];
#pragma unroll
          for (int k = 1; k < ROUND; ++k) mx = fmaxf(mx, pm[k]);
#pragma unroll
          for (int k = 0; k < ROUND; ++k) {                  // in the order of the context: a fixed order
            const float f = k < it.n_parts ? exp2f(pm[k] - mx) : 0.0f;
            acc += po[k] * f;
            l += pl[k] * f;
          }
        } else {
          float mx = -INFINITY;
          for (int k = 0; k < it.n_parts; ++k)
            mx = fmaxf(mx, __ldcg(&a.part_ml[(static_cast<size_t>(part_slot(a, it, k, per_range)) * g + h) * 2]));
          for (int k = 0; k < it.n_parts; ++k) {
            const size_t slot = static_cast<size_t>(part_slot(a, it, k, per_range)) * g + h;
            const float f = exp2f(__ldcg(&a.part_ml[slot * 2]) - mx);
            acc += __ldcg(&a.part_o[slot * HD + d]) * f;
            l += __ldcg(&a.part_ml[slot * 2 + 1]) * f;
          }
        }
        a.out[out_base + e] = __float2bfloat16_rn(l > 0.0f ? acc / l : 0.0f);
      }
    }
    if (ctid == 0) a.counters[it.r * a.nkv + it.kvh] = 0;    // left as it was found, for the next call
  }
  if (trace) { trace[4] = timer_ns(); trace[5] = item_seq; trace[6] = tile_base; }
  if (abort_flag) {
    // Something went wrong.  Give copies that are still in flight a bounded chance to land before
    // this CTA's shared memory is handed to another.
    for (int s = warp; s < R; s += DEC_CONSUMERS)
      for (int i = 0; i < (1 << 14) && !mbar_try_wait(&full[s], 0) && !mbar_try_wait(&full[s], 1); ++i) {}
  }
}

// Shared memory of one CTA with `slots` ring slots, and the most slots that fit.
template <int HD> size_t decode_smem_bytes(int slots, int g, int item_pages, int n_rows) {
  return static_cast<size_t>(item_pages) * DEC_PRODUCERS * sizeof(int)                     // the item's page ids, per producer
         + (static_cast<size_t>(n_rows) + 2 + slots) * sizeof(int)                         // rows' first tiles (balanced items), slots' counts
         + static_cast<size_t>(slots) * 2 * DEC_TILE * HD * sizeof(__nv_bfloat16)         // ring
         + 2 * 16 * (HD + 8) * sizeof(__nv_bfloat16)                                       // queries, two items
         + static_cast<size_t>(DEC_CONSUMERS) * g * (HD + 2) * sizeof(float)               // merge buffers
         + (2 * static_cast<size_t>(slots) + 4) * sizeof(unsigned long long);              // barriers
}

template <int HD>
int decode_launch(DecodeArgs& a, cudaStream_t stream) {
  const int g = a.nh / a.nkv;
  int device = 0, sms = 0;
  if (cudaGetDevice(&device) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess)
    return ERR_CUDA;
  sms = shared_sm_count(sms);
  // One persistent CTA per SM.  Fixed splits: max_splits items per pair.  Balanced: max_splits is the
  // most tiles a pair can have, and an item is at most a pair's tiles or a range's, whichever is less.
  const long long units = static_cast<long long>(a.n_rows) * a.nkv * a.max_splits;
  int grid = static_cast<int>(units < sms ? units : sms);
  if (a.split_size == 0 && grid > DEC_MAX_BALANCED_GRID) grid = DEC_MAX_BALANCED_GRID;
  const long long item_tiles = a.split_size > 0 ? a.split_size / DEC_TILE + 1
                                                : std::min<long long>(a.max_splits, (units + grid - 1) / grid) + 1;
  const int item_pages = static_cast<int>((item_tiles * DEC_TILE) >> a.page_shift) + 2;
  if (decode_smem_bytes<HD>(2, g, item_pages, a.n_rows) > static_cast<size_t>(DEC_SMEM_BUDGET)) return ERR_UNSUPPORTED;
  int slots = 2;
  while (decode_smem_bytes<HD>(slots + 1, g, item_pages, a.n_rows) <= static_cast<size_t>(DEC_SMEM_BUDGET)) ++slots;
  a.ring_slots = slots;
  a.item_pages = item_pages;
  const size_t smem = decode_smem_bytes<HD>(slots, g, item_pages, a.n_rows);
  auto kernel = paged_decode_kernel<HD>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
    return ERR_CUDA;
  return launch_dependent(kernel, dim3(grid), dim3(DEC_THREADS), smem, stream, false, a);
}

}  // namespace zb

using namespace zb;

// 1 if zb_paged_decode takes this shape, else 0 (the caller then uses the general kernel).
namespace zb {
inline int*& decode_trace() {
  static int* buffer = nullptr;
  return buffer;
}
}  // namespace zb

// Timelines for later launches of zb_paged_decode: `buffer` is null (off) or 8 ints per CTA on the
// device for up to 1024 CTAs (see DecodeArgs::trace).
ZB_API int zb_paged_decode_set_trace(int* buffer) {
  decode_trace() = buffer;
  return OK;
}

ZB_API int zb_paged_decode_supported(int nh, int nkv, int hd, int dtype) {
  if (dtype != DTYPE_BF16 || nkv <= 0 || nh % nkv != 0 || nh / nkv > DEC_MAX_GROUP) return 0;
  return hd == 32 || hd == 64 || hd == 96 || hd == 128 ? 1 : 0;
}

// Floats of scratch the kernel needs for the partial results of fixed splits.
ZB_API long long zb_paged_decode_scratch_floats(int n_rows, int nh, int hd, int max_splits) {
  return static_cast<long long>(n_rows) * nh * max_splits * (hd + 2);
}

// The same for balanced items (split_size 0): two slots per CTA, whatever the batch.
ZB_API long long zb_paged_decode_balanced_scratch_floats(int nh, int nkv, int hd) {
  return 2LL * DEC_MAX_BALANCED_GRID * (nh / nkv) * (hd + 2);
}

// Attention of `n_rows` single new tokens over their paged context.  `counters` holds n_rows * nkv
// ints that are zero on entry and are left zero; page_size is a power of two.
//   split_size > 0 (a multiple of 32): every row's context is cut into splits of that many positions;
//     max_splits >= ceil((longest context + 1) / split_size); `scratch` holds
//     zb_paged_decode_scratch_floats(...) floats (contents irrelevant).
//   split_size == 0: the tiles of all rows are spread evenly over the CTAs; max_splits >=
//     ceil((longest context + 1) / 32); `scratch` holds zb_paged_decode_balanced_scratch_floats(...).
namespace zb {
struct DecodeFusion {            // position encoding inside the kernel (see DecodeArgs)
  const void* qkv;
  long long qkv_stride;
  const void* q_norm_w;
  const void* k_norm_w;
  int norm_w_dtype;
  float norm_eps;
  const float* cos_table;
  const float* sin_table;
  int max_positions;
};
}  // namespace zb

static int paged_decode_entry(void* out, const void* q, const void* kv_cache, const int* block_table, int max_blocks,
                              int page_size, int num_pages, int num_rows, const int* rows, int n_rows,
                              const int* row_q_start, const int* row_ctx, int nh, int nkv, int hd, int window,
                              float scale, int split_size, int max_splits, float* scratch, int* counters, int* status,
                              const DecodeFusion* fusion, void* stream) {
  if (n_rows < 0 || max_splits <= 0 || split_size < 0 || split_size % DEC_TILE != 0 || page_size <= 0 || window < 0 ||
      counters == nullptr)
    return ERR_BAD_ARGUMENT;
  if (!zb_paged_decode_supported(nh, nkv, hd, DTYPE_BF16) || (page_size & (page_size - 1)) != 0) return ERR_UNSUPPORTED;
  if (n_rows == 0) return OK;
  if (static_cast<long long>(n_rows) * nkv * max_splits > 0x7fffffffLL) return ERR_UNSUPPORTED;
  int page_shift = 0;
  while ((1 << page_shift) < page_size) ++page_shift;
  DecodeArgs a;
  a.q = static_cast<const __nv_bfloat16*>(q);
  a.out = static_cast<__nv_bfloat16*>(out);
  a.kv_cache = static_cast<const __nv_bfloat16*>(kv_cache);
  a.block_table = block_table; a.rows = rows; a.row_q_start = row_q_start; a.row_ctx = row_ctx;
  a.part_o = scratch;
  a.part_ml = scratch + (split_size > 0 ? static_cast<size_t>(n_rows) * nh * max_splits * hd
                                        : static_cast<size_t>(2) * DEC_MAX_BALANCED_GRID * (nh / nkv) * hd);
  a.counters = counters;
  a.max_blocks = max_blocks; a.page_shift = page_shift; a.num_pages = num_pages; a.num_rows = num_rows;
  a.n_rows = n_rows;
  a.nh = nh; a.nkv = nkv; a.window = window; a.split_size = split_size; a.max_splits = max_splits;
  a.trace = decode_trace();
  a.qkv = nullptr;
  a.qkv_stride = 0;
  a.q_norm_w = a.k_norm_w = nullptr;
  a.norm_w_dtype = DTYPE_BF16;
  a.norm_eps = 0.0f;
  a.cos_table = a.sin_table = nullptr;
  a.max_positions = 0;
  if (fusion != nullptr) {
    if (fusion->qkv == nullptr || reinterpret_cast<uintptr_t>(fusion->qkv) % 4 != 0 || fusion->qkv_stride % 2 != 0 ||
        fusion->qkv_stride < static_cast<long long>(nh + 2 * nkv) * hd || (fusion->cos_table == nullptr) != (fusion->sin_table == nullptr) ||
        reinterpret_cast<uintptr_t>(fusion->cos_table) % 8 != 0 || reinterpret_cast<uintptr_t>(fusion->sin_table) % 8 != 0)
      return ERR_BAD_ARGUMENT;
    a.qkv = static_cast<const __nv_bfloat16*>(fusion->qkv);
    a.qkv_stride = fusion->qkv_stride;
    a.q_norm_w = fusion->q_norm_w;
    a.k_norm_w = fusion->k_norm_w;
    a.norm_w_dtype = fusion->norm_w_dtype;
    a.norm_eps = fusion->norm_eps;
    a.cos_table = fusion->cos_table;
    a.sin_table = fusion->sin_table;
    a.max_positions = fusion->max_positions;
  }
  a.ring_slots = 0;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.status = status;
  auto s = static_cast<cudaStream_t>(stream);
  switch (hd) {
    case 32: return decode_launch<32>(a, s);
    case 64: return decode_launch<64>(a, s);
    case 96: return decode_launch<96>(a, s);
    default: return decode_launch<128>(a, s);
  }
}

ZB_API int zb_paged_decode(void* out, const void* q, const void* kv_cache, const int* block_table, int max_blocks,
                           int page_size, int num_pages, int num_rows, const int* rows, int n_rows,
                           const int* row_q_start, const int* row_ctx, int nh, int nkv, int hd, int window,
                           float scale, int split_size, int max_splits, float* scratch, int* counters, int* status,
                           void* stream) {
  return paged_decode_entry(out, q, kv_cache, block_table, max_blocks, page_size, num_pages, num_rows, rows, n_rows,
                            row_q_start, row_ctx, nh, nkv, hd, window, scale, split_size, max_splits, scratch, counters,
                            status, nullptr, stream);
}

// The same with the new tokens' position encoding inside the kernel: `qkv` [T, qkv_stride] holds each
// request's new token raw (query heads, key heads, value heads); per-head RMS norms of q and k
// (scales may be null), the rotation by the tables (may be null) and the write of the new key and
// value into the cache (`kv_cache` is written) happen here, and no kernel has to run between the
// projection and this one.  For steps in which every request has exactly one new token.
ZB_API int zb_paged_decode_fused(void* out, void* kv_cache, const int* block_table, int max_blocks, int page_size,
                                 int num_pages, int num_rows, const int* rows, int n_rows, const int* row_q_start,
                                 const int* row_ctx, int nh, int nkv, int hd, int window, float scale, int split_size,
                                 int max_splits, float* scratch, int* counters, int* status, const void* qkv,
                                 long long qkv_stride, const void* q_norm_w, const void* k_norm_w, int norm_w_dtype,
                                 float norm_eps, const float* cos_table, const float* sin_table, int max_positions,
                                 void* stream) {
  const DecodeFusion fusion{qkv, qkv_stride, q_norm_w, k_norm_w, norm_w_dtype, norm_eps, cos_table, sin_table, max_positions};
  return paged_decode_entry(out, out, kv_cache, block_table, max_blocks, page_size, num_pages, num_rows, rows, n_rows,
                            row_q_start, row_ctx, nh, nkv, hd, window, scale, split_size, max_splits, scratch, counters,
                            status, &fusion, stream);
}

// ------------------------------------------------------------------------------------------
// The entry point that allocates nothing (declared and explained in no_alloc.h).  Its scratch
// is the array below, a part of the library image on every device that loads it.
#include <mutex>

#include "no_alloc.h"

static __device__ __align__(256) float zb_no_alloc_scratch[ZB_NO_ALLOC_SCRATCH_BYTES / sizeof(float)];

namespace {

constexpr int NO_ALLOC_MAX_DEVICES = 64;
std::mutex no_alloc_mutex;
float* no_alloc_address[NO_ALLOC_MAX_DEVICES] = {};   // device address of the array, per device ordinal

// In host code the array's name is only a handle for the runtime, not a device address, so the
// address the kernels get is looked up here: once per device, with that device current.
float* no_alloc_scratch_for_current_device() {
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= NO_ALLOC_MAX_DEVICES) return nullptr;
  std::lock_guard<std::mutex> lock(no_alloc_mutex);
  if (no_alloc_address[device] == nullptr) {
    float* address = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&address), zb_no_alloc_scratch) != cudaSuccess) {
      (void)cudaGetLastError();      // leave no sticky error behind for the caller's next call
      return nullptr;
    }
    no_alloc_address[device] = address;
  }
  return no_alloc_address[device];
}

}  // namespace

ZB_API long long zb_paged_decode_no_alloc_bytes_needed(int n_rows, int nh, int nkv, int hd, int split_size,
                                                       int max_splits) {
  if (n_rows < 0 || nh <= 0 || nkv <= 0 || nkv > nh || hd <= 0 || split_size < 0 || max_splits <= 0) return -1;
  // The arrival counters (one per row and key/value head, rounded up to 256 bytes), then the partial
  // results.  How many of those there are depends on how the work is cut: fixed splits keep one per
  // (row, head, split); balanced items (split_size 0) keep two per CTA and query head of a group,
  // whatever the rows and max_splits are.
  const long long counter_bytes = (static_cast<long long>(n_rows) * nkv * 4 + 255) / 256 * 256;
  const long long floats = split_size > 0 ? zb_paged_decode_scratch_floats(n_rows, nh, hd, max_splits)
                                          : zb_paged_decode_balanced_scratch_floats(nh, nkv, hd);
  return counter_bytes + floats * static_cast<long long>(sizeof(float));
}

ZB_API const char* zb_paged_decode_no_alloc_error(int code) {
  switch (code) {
    case OK: return "launched";
    case ERR_BAD_ARGUMENT: return "an argument lies outside the kernel's contract";
    case ERR_CUDA: return "the CUDA launch failed";
    case ERR_UNSUPPORTED: return "this head size, group size or type is not supported by the decode kernel";
    case ZB_ERR_SCRATCH_TOO_SMALL:
      return "the problem needs more than the 4 MiB of built-in scratch (zb_paged_decode_no_alloc_bytes_needed "
             "says how much: with fixed splits n_rows * heads * max_splits * (head_dim + 2) * 4 bytes, with balanced "
             "items 2 * 256 * (heads / kv_heads) * (head_dim + 2) * 4 bytes); use zb_paged_decode with a buffer of "
             "your own, or split the rows over several calls";
    case ZB_ERR_SCRATCH_ADDRESS: return "the device address of the built-in scratch array could not be looked up";
    default: return "unknown code";
  }
}

ZB_API int zb_paged_decode_no_alloc(void* out, const void* q, const void* kv_cache, const int* block_table,
                                    int max_blocks, int page_size, int num_pages, int num_rows, const int* rows,
                                    int n_rows, const int* row_q_start, const int* row_ctx, int nh, int nkv, int hd,
                                    int window, float scale, int split_size, int max_splits, int* status,
                                    void* stream) {
  // The bound depends on how the work is cut (split_size), exactly as the kernel lays its partial
  // results out; it is checked before anything is cleared or launched.
  const long long needed = zb_paged_decode_no_alloc_bytes_needed(n_rows, nh, nkv, hd, split_size, max_splits);
  if (needed < 0) return ERR_BAD_ARGUMENT;
  if (needed > static_cast<long long>(ZB_NO_ALLOC_SCRATCH_BYTES)) return ZB_ERR_SCRATCH_TOO_SMALL;
  float* scratch = no_alloc_scratch_for_current_device();
  if (scratch == nullptr) return ZB_ERR_SCRATCH_ADDRESS;
  // The array's head holds the arrival counters of the (row, key/value head) pairs, its rest the
  // partial results.  The counters must be zero when the kernel starts; the array keeps what the
  // last call left, so they are cleared here, on the caller's stream (a memset, no allocation).
  const size_t counter_bytes = (static_cast<size_t>(n_rows) * nkv * sizeof(int) + 255) / 256 * 256;
  if (cudaMemsetAsync(scratch, 0, counter_bytes, static_cast<cudaStream_t>(stream)) != cudaSuccess) return ERR_CUDA;
  return zb_paged_decode(out, q, kv_cache, block_table, max_blocks, page_size, num_pages, num_rows, rows, n_rows,
                         row_q_start, row_ctx, nh, nkv, hd, window, scale, split_size, max_splits,
                         scratch + counter_bytes / sizeof(float), reinterpret_cast<int*>(scratch), status, stream);
}
