// Paged causal attention for prompt portions on the fifth-generation tensor cores: tcgen05.mma
// with the A operands (queries, probabilities) and the accumulators in tensor memory (TMEM) and the
// B operands (keys, values) in shared memory.
//
// One CTA = up to 128 consecutive new tokens of one request x one query head, head size 128,
// bfloat16.  Keys and values stream through three stages each of 128-position tiles.  Roles:
//   * four loader warps, two for the keys and two for the values, copy a tile's rows from the cache
//     pages (TMA tiled copies per page for tiles inside the context, 16-byte asynchronous copies at
//     its edges, where rows have to be zero).  A cache row's 16-byte chunks are stored permuted
//     with the position (common.cuh: kv_swizzle); for rows of 256 bytes that permutation IS the
//     128-byte swizzle of the tensor core's canonical shared-memory layout, so a row is copied as
//     it lies, its first 128 bytes to the tile's first half (head dims 0..63), the rest to the
//     second half;
//   * one thread issues the products: S = Q K^T (M 128 queries, N 128 keys, eight steps of K = 16
//     over the head dims; Q from TMEM columns 384..447, two bfloat16 a column; the keys K-major)
//     into TMEM columns 0..127 or 128..255 by turns, and O += P V (A = the probabilities, which
//     the softmax leaves where their S lay; B = the values as they lie, MN-major) into columns
//     256..383; S of the next tile is issued before the wait for this tile's probabilities, so the
//     softmax runs beside the products; completion is reported to mbarriers by tcgen05.commit;
//   * eight softmax warps own the 128 query rows, two threads a row (TMEM lane = row; one thread
//     takes the first 64 columns of S and of O, the other the rest): they read their half of a row
//     of S with tcgen05.ld, keep the running sum in float32 in base 2, store the probabilities as
//     bfloat16 pairs with tcgen05.st, and rescale O in TMEM when the row's maximum has grown by
//     more than 2^8 since the value the row last rescaled to (the softmax does not care which
//     shift it is given as long as it is given everywhere; the bound keeps exp2 far from
//     overflow).  A row's two threads tell each other their largest score every tile, so both
//     take the same decisions.
// Math and masking as in attention_prefill.cu and attention_simt.cu (causal, lower-right aligned on
// the cached context, optional window; probabilities rounded to bfloat16 for the second product;
// reference: src/layer/paged_attention.cpp:118-296, deps/ttl/src/kernels/attention/attention.cu:58-170).
// Every wait is bounded and reports instead of hanging; TMEM is given back on every path.
#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"
#include "mma.cuh"
#include "tcgen05.cuh"
#include "tma.cuh"

namespace zb {

constexpr int TC_BM = 128;                 // query rows per CTA
constexpr int TC_BN = 128;                 // positions per key/value tile
constexpr int TC_HD = 128;
constexpr int TC_SOFTMAX_WARPS = 8;        // warps 0..7: TMEM lanes 32 (w % 4) .. + 31; warps 0..3 take a row's first 64 columns, 4..7 the rest
constexpr int TC_MMA_WARP = 8;
constexpr int TC_LOADER_WARPS = 4;         // warps 9, 10: keys; 11, 12: values
constexpr int TC_KIND_THREADS = TC_LOADER_WARPS * 32 / 2;
constexpr int TC_THREADS = (TC_SOFTMAX_WARPS + 1 + TC_LOADER_WARPS) * 32;
constexpr int TC_HALF_BYTES = TC_BN * 128;             // a tile's 128 rows of one 64-dim half
constexpr int TC_TILE_BYTES = 2 * TC_HALF_BYTES;       // 32 KB: both halves
constexpr int TC_WAIT_LIMIT = 1 << 18;
constexpr int TC_TMEM_COLUMNS = 512;        // S of even tiles, S of odd tiles, O, Q (a power of two is asked for)
constexpr int TC_O_COLUMN = 2 * TC_BN;      // O: 128 columns of float32
constexpr int TC_Q_COLUMN = 3 * TC_BN;      // Q: 64 columns, two bfloat16 each
constexpr int TC_STAGES = 3;                // key/value tiles in shared memory, each kind
constexpr float TC_RESCALE_THRESHOLD = 8.0f;

struct PrefillTcArgs {
  CUtensorMap cache_map;         // the cache as [rows of all pages, keys and values, heads][hd]; box: 64 dims x one page's rows (at most 128)
  int tiled;                     // 0: no map (every tile goes through 16-byte copies)
  const __nv_bfloat16* q;        // [T, nh*hd]
  __nv_bfloat16* out;            // [T, nh*hd]
  const __nv_bfloat16* kv_cache; // [num_pages][2][nkv][page_size][hd]
  const int* block_table;        // [R, max_blocks]
  const int* tile_row;           // [n_tiles]
  const int* tile_q0;            // [n_tiles]
  const int* row_q_start;        // [R]
  const int* row_q_len;          // [R]
  const int* row_ctx;            // [R]
  int max_blocks, page_shift, num_pages, num_rows;
  int nh, nkv, window;
  float scale_log2;
  int* status;
  int* trace;                    // null, or 4 ints per tile of the first CTA (the longest work of the launch): the global
                                 // timer (ns, low 32 bits) when S of the tile was issued, when its softmax began (S
                                 // complete), when its probabilities were written, when O += P V of it was issued
};

__device__ __forceinline__ int tc_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return static_cast<int>(t);
}

// The values (V) are MN-major in shared memory: a row is one position's 64 head dims; the stride
// offset of the descriptor steps over groups of 8 positions (K), the leading offset over the two
// 64-dim halves (N).  Fields as in desc_k_major.
__device__ __forceinline__ unsigned long long desc_mn_major(unsigned smem_address) {
  return static_cast<unsigned long long>((smem_address >> 4) & 0x3FFFu) |
         (static_cast<unsigned long long>(TC_HALF_BYTES >> 4) << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ float exp2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// One half (64 columns) of a row of S (this thread's TMEM lane) -> probabilities exp2(s * scale + neg_shift)
// as 32 words of two bfloat16 each, their sum, and the largest raw score.  MASKED: column i counts only if
// after < i <= last and i >= first (positions relative to the tile's first key).
template <bool MASKED>
__device__ __forceinline__ void softmax_pass(unsigned tmem_row, unsigned (&words)[TC_BN / 4], int half, float scale, float neg_shift,
                                             int last, int first, int after, float& raw_max, float& row_sum) {
  // Four running maxima and sums side by side: with one warp per scheduler a single chain of 128
  // dependent additions would cost its full latency 128 times.
  float max4[4] = {raw_max, -INFINITY, -INFINITY, -INFINITY}, sum4[4] = {row_sum, 0.0f, 0.0f, 0.0f};
#pragma unroll
  for (int cc = 0; cc < TC_BN / 64; ++cc) {
    const int c4 = half * (TC_BN / 64) + cc;
    unsigned v[32];
    tmem_ld32(tmem_row + c4 * 32, v);
    tc_wait_ld();
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      float p[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float raw = __uint_as_float(v[i + e]);
        const int column = c4 * 32 + i + e;
        const bool ok = !MASKED || (column <= last && column >= first && column > after);
        if (ok) max4[(i >> 1) & 3] = fmaxf(max4[(i >> 1) & 3], raw);
        p[e] = ok ? exp2_approx(fmaf(raw, scale, neg_shift)) : 0.0f;
        sum4[(i >> 1) & 3] += p[e];
      }
      words[16 * cc + (i >> 1)] = pack_bf16(p[0], p[1]);
    }
  }
  raw_max = fmaxf(fmaxf(max4[0], max4[1]), fmaxf(max4[2], max4[3]));
  row_sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
}

__global__ void __launch_bounds__(TC_THREADS, 1)
paged_prefill_tc_kernel(const __grid_constant__ PrefillTcArgs a) {
  // Shared memory holds keys and values only (three stages of each, tiles of 32 KB on 1024-byte
  // boundaries as the 128-byte swizzle wants them): the queries and the probabilities, the A
  // operands of the two products, live in tensor memory, so that a product reads 4 KB of shared
  // memory per step instead of 8 (with both operands there the products ran at the shared memory's
  // bandwidth, not at the tensor core's).
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* kv_s = smem;                              // [3 stages][keys, values][2 halves][128 rows][128 bytes]
  __shared__ unsigned long long bars[2 * 2 * TC_STAGES + 8];
  // Tile j uses stage j % 3 of the keys and of the values (phase j / 3 on their barriers) and entry
  // j % 2 of every other pair (phase j / 2); nobody ever waits for a phase that is more than one
  // behind the barrier's current one.
  // Keys and values have barriers of their own: a stage's keys are free again as soon as S of their
  // tile is complete, long before its values, so the keys of the tile after next are on their way
  // while this tile's softmax runs.  Index 0: keys, 1: values.
  unsigned long long* kv_full = bars;                          // [2 kinds][3 stages] the rows have landed (the kind's loader threads)
  unsigned long long* kv_empty = bars + 2 * TC_STAGES;         // [2 kinds][3 stages] the product that reads them is complete
  unsigned long long* s_full = bars + 4 * TC_STAGES;           // [2] S of the tile is complete
  unsigned long long* p_full = s_full + 2;     // [2] P is written, S has been read, O has been rescaled (all softmax threads)
  unsigned long long* o_done = s_full + 4;     // [2] O += P V of the tile is complete
  unsigned long long* halves_met = s_full + 6; // [2] both halves of every row have left their largest score (all softmax threads)
  __shared__ float half_note[2][2][TC_BM];     // [tile parity][half][row]: what a row's two threads tell each other
  __shared__ unsigned tmem_base_s;
  __shared__ volatile int abort_flag;

  // The host lists the tiles by the number of keys they see, fewest first: take the list back to
  // front, and all heads of a tile before the next tile, so that the longest work of the whole
  // launch starts first and the short tiles fill the gaps at the end.
  const int tile = gridDim.y - 1 - blockIdx.y, head = blockIdx.x;
  const int row = a.tile_row[tile], q0 = a.tile_q0[tile];
  if (row < 0 || row >= a.num_rows) {
    if (threadIdx.x == 0) report(a.status, STATUS_ROW_OUT_OF_RANGE, row, tile);
    return;
  }
  if ((smem_u32(smem) & 1023u) != 0) {          // the tiles must lie on 1024-byte boundaries
    if (threadIdx.x == 0) report(a.status, STATUS_INTERNAL_CHECK, static_cast<int>(smem_u32(smem) & 1023u), tile);
    return;
  }
  const int g = a.nh / a.nkv, kvh = head / g;
  const int q_len = a.row_q_len[row], ctx = a.row_ctx[row], tok0 = a.row_q_start[row] + q0;
  const int n_tok = min(TC_BM, q_len - q0);
  if (n_tok <= 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int page_size = 1 << a.page_shift;
  int* const trace = a.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 ? a.trace : nullptr;

  // Keys any query of this tile may see: [lo, hi).
  const int hi = ctx + q0 + n_tok;
  const int lo = a.window > 0 ? max(0, ctx + q0 - a.window + 1) : 0;
  const int first_tile = lo / TC_BN * TC_BN;
  const int n_tiles = (hi - first_tile + TC_BN - 1) / TC_BN;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int b = 0; b < 2 * TC_STAGES; ++b) {
      mbar_init(&kv_full[b], TC_KIND_THREADS);
      mbar_init(&kv_empty[b], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&s_full[b], 1);
      mbar_init(&p_full[b], TC_SOFTMAX_WARPS * 32);
      mbar_init(&o_done[b], 1);
      mbar_init(&halves_met[b], TC_SOFTMAX_WARPS * 32);
    }
    fence_barrier_init();
  }
  if (warp == TC_MMA_WARP) {
    tmem_alloc(&tmem_base_s, TC_TMEM_COLUMNS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const unsigned tmem_base = tmem_base_s;
  // The queries go to tensor memory, a row to its lane: a row's two threads store 64 elements each
  // as 32 columns of two.  Rows past the tile's tokens are zero.
  if (warp < TC_SOFTMAX_WARPS) {
    const int r = threadIdx.x & (TC_BM - 1), half = threadIdx.x / TC_BM;
    const uint4* src = reinterpret_cast<const uint4*>(a.q + (static_cast<size_t>(tok0 + (r < n_tok ? r : 0)) * a.nh + head) * TC_HD) + half * 8;
    unsigned words[32];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const uint4 v = r < n_tok ? src[c] : make_uint4(0, 0, 0, 0);
      words[4 * c] = v.x; words[4 * c + 1] = v.y; words[4 * c + 2] = v.z; words[4 * c + 3] = v.w;
    }
    tmem_st32(tmem_base + (static_cast<unsigned>((warp & 3) * 32) << 16) + TC_Q_COLUMN + 32 * half, words);
    tc_wait_st();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();

  auto wait = [&](unsigned long long* bar, unsigned parity) -> bool {
    if (mbar_try_wait(bar, parity)) return true;
    for (int i = 0; i < TC_WAIT_LIMIT; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
      if ((i & 63) == 63 && abort_flag) return false;
    }
    return false;
  };
  auto give_up = [&](int where) {
    if (!abort_flag) report(a.status, STATUS_COPY_TIMEOUT, where, tile);
    abort_flag = 1;
  };

  if (warp > TC_MMA_WARP) {
    // ------------------------------------------------------------------------- the loaders
    // Two warps fetch the keys and two the values, each pair at its own pace (the kernel's timeline
    // showed one group of loaders taking a microsecond per tile and kind, so that a tile's values
    // were asked for only when its probabilities were already written).
    const int lk = threadIdx.x - (TC_MMA_WARP + 1) * 32;          // 0..127
    const int kv = lk / TC_KIND_THREADS, lt = lk % TC_KIND_THREADS; // 0: keys, 1: values; 0..63 within the kind
    const int chunk = lt & 15, row_in_4 = lt >> 4;                // 16-byte copies: this thread's chunk of rows row_in_4 + 4 i
    const int* table = a.block_table + static_cast<size_t>(row) * a.max_blocks;
    const long long v_offset = static_cast<long long>(a.nkv) * page_size * TC_HD;
    const unsigned dst_base = (chunk >> 3) * TC_HALF_BYTES + ((chunk & 7) << 4);
    // A tile that lies wholly inside [lo, hi) comes by TMA: one tiled copy per page and 64-dim half
    // (the map's box is a page's rows by 64 dims, copied as they lie: the cache's own chunk
    // permutation is already the canonical swizzle), from eight lanes of each of the kind's warps,
    // the bytes counted on the stage's barrier.  A tile at an edge of [lo, hi) needs rows filled with
    // zeros (their scores are masked, and a zero probability times a zero value stays zero) and
    // goes through 16-byte copies that can do that.
    const int rows_per_copy = min(page_size, TC_BN), copies_per_half = TC_BN / rows_per_copy;
    // This lane's tiled copies: ids first_id and first_id + 16 of a tile's 2 * copies_per_half
    // (64-dim half, piece of the tile).  The page ids of the next tile are asked for as soon as this
    // tile's copies are out, so that the table's latency is not in front of them.
    const bool issues = (lt & 31) < 8;
    const int first_id = (lt >> 5) * 8 + (lt & 31);
    int ahead_tile = -1, ahead_page[2] = {0, 0};
    auto look_up = [&](int j, int (&page)[2]) {
      const int k0 = first_tile + j * TC_BN;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int id = first_id + 16 * u;
        const int block = (k0 + (id % copies_per_half) * rows_per_copy) >> a.page_shift;
        page[u] = id < 2 * copies_per_half && block < a.max_blocks ? table[block] : -1;
      }
    };
    auto issue_tiled = [&](int j) {
      const int stage = j % TC_STAGES, k0 = first_tile + j * TC_BN;
      unsigned char* dst = kv_s + stage * 2 * TC_TILE_BYTES + kv * TC_TILE_BYTES;
      unsigned long long* bar = &kv_full[kv * TC_STAGES + stage];
      if (lt == 0) mbar_arrive_expect_tx(bar, TC_TILE_BYTES);
      else tc_mbar_arrive(bar);
      if (!issues) return;
      int page[2];
      if (ahead_tile == j) { page[0] = ahead_page[0]; page[1] = ahead_page[1]; }
      else look_up(j, page);
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int id = first_id + 16 * u;
        if (id >= 2 * copies_per_half) break;
        const int half = id / copies_per_half, piece = id % copies_per_half;
        const int pos = k0 + piece * rows_per_copy;
        int pg = page[u];
        if (pg <= 0 || pg >= a.num_pages) {
          report(a.status, STATUS_PAGE_OUT_OF_RANGE, pg, tok0);
          pg = 0;                       // the bytes must arrive all the same
        }
        const int cache_row = ((pg * 2 + kv) * a.nkv + kvh) * page_size + (pos & (page_size - 1));
        tiled_copy_2d_g2s(dst + half * TC_HALF_BYTES + piece * rows_per_copy * 128, &a.cache_map, half * 64, cache_row, bar);
      }
      if (j + 1 < n_tiles) {
        look_up(j + 1, ahead_page);
        ahead_tile = j + 1;
      }
    };
    auto issue_plain = [&](int j) {
      const int stage = j % TC_STAGES;
      unsigned char* dst = kv_s + stage * 2 * TC_TILE_BYTES + kv * TC_TILE_BYTES + dst_base;
      const int k0 = first_tile + j * TC_BN;
#pragma unroll 1
      for (int part = 0; part < 2; ++part) {
        // The page ids of 16 of this thread's 32 rows first, all at once: a lookup per copy would put
        // the table's latency in front of every copy.
        int page[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int pos = k0 + row_in_4 + 4 * (16 * part + i), block = pos >> a.page_shift;
          page[i] = pos >= lo && pos < hi ? (block < a.max_blocks ? table[block] : -1) : 0;
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int r = row_in_4 + 4 * (16 * part + i), pos = k0 + r;
          bool ok = pos >= lo && pos < hi;
          const __nv_bfloat16* src = a.kv_cache;
          if (ok) {
            if (page[i] <= 0 || page[i] >= a.num_pages) {
              report(a.status, STATUS_PAGE_OUT_OF_RANGE, page[i], tok0);
              ok = false;
            } else {
              src += ((static_cast<long long>(page[i]) * 2 * a.nkv + kvh) * page_size + (pos & (page_size - 1))) * TC_HD +
                     chunk * 8 + (kv ? v_offset : 0);
            }
          }
          cp_async_16(dst + r * 128, src, ok);
        }
      }
      cp_async_commit();
      cp_async_wait<0>();
      fence_proxy_async();           // the tensor core reads what the copies wrote through the asynchronous proxy
      tc_mbar_arrive(&kv_full[kv * TC_STAGES + stage]);
    };
    for (int j = 0; j < n_tiles; ++j) {
      if (!wait(&kv_empty[kv * TC_STAGES + j % TC_STAGES], ((j / TC_STAGES) & 1) ^ 1)) {
        give_up(-1);
        break;
      }
      const int k0 = first_tile + j * TC_BN;
      if (trace && lt == 0 && j < 64) trace[256 + 4 * j + kv] = tc_timer_ns();
      if (a.tiled && k0 >= lo && k0 + TC_BN <= hi) issue_tiled(j); else issue_plain(j);
    }
  } else if (warp == TC_MMA_WARP) {
    // ------------------------------------------------------------- the thread that issues products
    if (lane == 0) {
      constexpr unsigned IDESC_QK = tc_idesc(false), IDESC_PV = tc_idesc(true);
      const unsigned tmem_o = tmem_base + TC_O_COLUMN, tmem_q = tmem_base + TC_Q_COLUMN;
      // S of tile j + 1 is issued before the wait for tile j's probabilities, so that the softmax of
      // one tile runs beside the products of its neighbours.
      auto issue_scores = [&](int j) {          // the tile's keys have landed
        const int stage = j % TC_STAGES;
        const unsigned k_addr = smem_u32(kv_s + stage * 2 * TC_TILE_BYTES);
        tc_fence_after_sync();
        const unsigned long long k_desc = desc_k_major(k_addr);       // the address field counts 16 bytes
        const unsigned tmem_s = tmem_base + (j & 1) * TC_BN;
        tc_mma_ts<false>(tmem_s, tmem_q, k_desc, IDESC_QK);
#pragma unroll
        for (int k = 1; k < TC_HD / 16; ++k)
          tc_mma_ts<true>(tmem_s, tmem_q + 8 * k, k_desc + (((k >> 2) * TC_HALF_BYTES + (k & 3) * 32) >> 4), IDESC_QK);
        tc_commit(&kv_empty[stage]);            // the keys' stage is free as soon as these products are complete
        tc_commit(&s_full[j & 1]);
        if (trace && j < 64) trace[4 * j] = tc_timer_ns();
      };
      // S of the next tile is issued as soon as its keys are there, before this tile's second
      // product if they come first.  S of tile j + 2 overwrites tile j's probabilities, which lie
      // where its S lay: it is issued after tile j's second product, and the tensor core takes its
      // work in the order of issue.  Neither product ever waits for something only the other can bring.
      int scores_issued = 0;
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int stage = j % TC_STAGES;
        const unsigned tmem_p = tmem_base + (j & 1) * TC_BN;      // a row's halves keep their words at columns 0.. and 64..
        const unsigned v_addr = smem_u32(kv_s + stage * 2 * TC_TILE_BYTES) + TC_TILE_BYTES;
        bool have_p = false;
        for (int polls = 0; !have_p; ++polls) {
          if (scores_issued <= j + 1 && scores_issued < n_tiles &&
              tc_mbar_test(&kv_full[scores_issued % TC_STAGES], (scores_issued / TC_STAGES) & 1)) {        // the tile's keys
            issue_scores(scores_issued++);
            continue;
          }
          if (scores_issued > j && tc_mbar_test(&p_full[j & 1], (j >> 1) & 1) &&
              tc_mbar_test(&kv_full[TC_STAGES + stage], (j / TC_STAGES) & 1))                          // P and the tile's values
            have_p = true;
          else if (polls > TC_WAIT_LIMIT || ((polls & 63) == 63 && abort_flag)) break;
          else __nanosleep(32);          // this warp shares its scheduler with softmax warps: leave them the issue slots
        }
        if (!have_p) { give_up(-3); ok = false; break; }
        tc_fence_after_sync();
        const unsigned long long v_desc = desc_mn_major(v_addr);
        if (j > 0) tc_mma_ts<true>(tmem_o, tmem_p, v_desc, IDESC_PV);
        else tc_mma_ts<false>(tmem_o, tmem_p, v_desc, IDESC_PV);
#pragma unroll
        for (int k = 1; k < TC_BN / 16; ++k)          // 16 positions: 8 columns of the half that wrote them
          tc_mma_ts<true>(tmem_o, tmem_p + (k >> 2) * 64 + (k & 3) * 8, v_desc + ((k * 2048) >> 4), IDESC_PV);
        tc_commit(&kv_empty[TC_STAGES + stage]);
        tc_commit(&o_done[j & 1]);
        if (trace && j < 64) trace[4 * j + 3] = tc_timer_ns();
      }
    }
  } else {
    // --------------------------------------------------------------------------- the softmax
    // A row (= TMEM lane) has two threads: warps 0..3 own the first 64 columns of S and of O, warps
    // 4..7 the other 64 (a warp reaches the lanes 32 (w % 4) .. + 31).  Eight warps because the row's
    // work is bound by latencies (tensor-memory reads, the special-function unit, conversions) that
    // one warp per scheduler cannot hide.  The halves share a row's shift: each tile they tell each
    // other their largest score (half_note, halves_met) and so take the same decisions.
    const int r = threadIdx.x & (TC_BM - 1), half = threadIdx.x / TC_BM;
    const unsigned lane_base = static_cast<unsigned>((warp & 3) * 32) << 16;
    const unsigned tmem_o = tmem_base + lane_base + 2 * TC_BN;
    const int qp = ctx + q0 + r;
    float m_used = -INFINITY, l_run = 0.0f;
    bool failed = false;
    for (int j = 0; j < n_tiles; ++j) {
      const int k0 = first_tile + j * TC_BN;
      // Whether to go on is decided by the warp as one: the tensor-memory instructions below are
      // for all of its lanes together.
      const int buffer = j & 1;
      const unsigned tmem_s = tmem_base + lane_base + buffer * TC_BN;
      if (!__all_sync(0xffffffffu, wait(&s_full[buffer], (j >> 1) & 1))) { give_up(-4); failed = true; break; }
      tc_fence_after_sync();
      if (trace && threadIdx.x == 0 && j < 64) trace[4 * j + 1] = tc_timer_ns();
      // Most tiles lie wholly in every row's past (and inside its window): no mask to evaluate.
      const bool open_tile = k0 + TC_BN - 1 <= ctx + q0 && k0 >= lo &&
                             (a.window == 0 || k0 > ctx + q0 + TC_BM - 1 - a.window);
      // One pass forms the probabilities with the shift the row already has and notes the row's
      // largest score; only if that has outgrown the shift by 2^8 (always for a row's first keys) is
      // the shift moved, O and the sum rescaled, and the pass repeated.  Per score the pass costs a
      // maximum, a fused multiply-add, an exp2 and an addition.  The probabilities stay in registers
      // until the shift is settled: they go where this thread's half of S lay, and a second pass
      // needs S once more.
      unsigned words[TC_BN / 4];
      for (int attempt = 0; attempt < 2; ++attempt) {
        const float neg_shift = m_used == -INFINITY ? 0.0f : -m_used;
        float raw_max = -INFINITY, row_sum = 0.0f;
        if (open_tile)
          softmax_pass<false>(tmem_s, words, half, a.scale_log2, neg_shift, 0, 0, 0, raw_max, row_sum);
        else
          softmax_pass<true>(tmem_s, words, half, a.scale_log2, neg_shift, qp - k0, lo - k0,
                             a.window > 0 ? qp - a.window - k0 : -(1 << 30), raw_max, row_sum);
        if (attempt == 0) {
          // The row's largest score is the larger of its halves'.
          half_note[j & 1][half][r] = raw_max;
          tc_mbar_arrive(&halves_met[j & 1]);
          if (!__all_sync(0xffffffffu, wait(&halves_met[j & 1], (j >> 1) & 1))) { give_up(-8); failed = true; break; }
          raw_max = fmaxf(raw_max, half_note[j & 1][half ^ 1][r]);
        }
        const float row_max = raw_max * a.scale_log2;       // the scale is positive
        const bool grow = attempt == 0 && (row_max > m_used + TC_RESCALE_THRESHOLD || (m_used == -INFINITY && row_max > -INFINITY));
        if (!__any_sync(0xffffffffu, grow)) {
          l_run += row_sum;
          break;
        }
        // Some row of the warp moves its shift: every lane takes part in the tensor-memory
        // instructions, rows that stay multiply by one.
        const float factor = grow ? exp2f(m_used - row_max) : 1.0f;       // 0 for a row's first keys
        if (grow) m_used = row_max;
        l_run *= factor;
        if (j > 0) {
          // O is touched only between the product of the tile before, which has to be complete, and
          // this tile's product, which waits for this warp's arrival below.
          if (!__all_sync(0xffffffffu, wait(&o_done[(j - 1) & 1], ((j - 1) >> 1) & 1))) { give_up(-7); failed = true; break; }
          tc_fence_after_sync();
#pragma unroll 1
          for (int c4 = half * (TC_HD / 64); c4 < (half + 1) * (TC_HD / 64); ++c4) {
            unsigned v[32];
            tmem_ld32(tmem_o + c4 * 32, v);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * factor);
            tmem_st32(tmem_o + c4 * 32, v);
          }
          tc_wait_st();
        }
      }
      if (failed) break;
      // Two probabilities a column, as the second product reads its A operand from tensor memory:
      // this half's 32 columns start where its 64 columns of S began.
      tmem_st32(tmem_s + 64 * half, words);
      tc_wait_st();
      tc_fence_before_sync();
      tc_mbar_arrive(&p_full[buffer]);
      if (trace && threadIdx.x == 0 && j < 64) trace[4 * j + 2] = tc_timer_ns();
    }
    if (!failed && !__all_sync(0xffffffffu, wait(&o_done[(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1))) { give_up(-6); failed = true; }
    if (!failed) {
      // The row's sum is the sum of its halves' (the exchange takes one more turn of the tiles' notes).
      half_note[n_tiles & 1][half][r] = l_run;
      tc_mbar_arrive(&halves_met[n_tiles & 1]);
      if (!__all_sync(0xffffffffu, wait(&halves_met[n_tiles & 1], (n_tiles >> 1) & 1))) { give_up(-9); failed = true; }
    }
    if (!failed) {
      tc_fence_after_sync();
      const float l_row = half_note[n_tiles & 1][0][r] + half_note[n_tiles & 1][1][r];
      const float inv = l_row > 0.0f ? 1.0f / l_row : 0.0f;
      // The keys' and values' stages are free by now (every product is complete): each warp puts its 32
      // rows x 64 columns there, 16-byte pieces permuted by the row so that neither the writes (a
      // thread a row) nor the reads (eight threads a row) meet in a bank, and then writes whole
      // 128-byte row pieces, four rows an instruction.  (A thread storing its own row's pieces
      // touches 32 rows with every instruction, which cost 1.4 us a CTA.)
      unsigned char* stage_out = kv_s + warp * 4096;
#pragma unroll
      for (int cc = 0; cc < TC_HD / 64; ++cc) {
        unsigned v[32];
        tmem_ld32(tmem_o + (half * (TC_HD / 64) + cc) * 32, v);
        tc_wait_ld();
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint4 o4;
          o4.x = pack_bf16(__uint_as_float(v[8 * q4]) * inv, __uint_as_float(v[8 * q4 + 1]) * inv);
          o4.y = pack_bf16(__uint_as_float(v[8 * q4 + 2]) * inv, __uint_as_float(v[8 * q4 + 3]) * inv);
          o4.z = pack_bf16(__uint_as_float(v[8 * q4 + 4]) * inv, __uint_as_float(v[8 * q4 + 5]) * inv);
          o4.w = pack_bf16(__uint_as_float(v[8 * q4 + 6]) * inv, __uint_as_float(v[8 * q4 + 7]) * inv);
          *reinterpret_cast<uint4*>(stage_out + lane * 128 + (((cc * 4 + q4) ^ (lane & 7)) << 4)) = o4;
        }
      }
      __syncwarp();
      const int row_base = (warp & 3) * 32, piece = lane & 7;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int rr = 4 * i + (lane >> 3);
        if (row_base + rr < n_tok) {
          const uint4 o4 = *reinterpret_cast<const uint4*>(stage_out + rr * 128 + ((piece ^ (rr & 7)) << 4));
          *reinterpret_cast<uint4*>(a.out + (static_cast<size_t>(tok0 + row_base + rr) * a.nh + head) * TC_HD + half * 64 + piece * 8) = o4;
        }
      }
    }
  }

  // Everybody meets here on every path, and the warp that took the tensor memory gives it back.
  tc_fence_before_sync();
  __syncthreads();
  if (warp == TC_MMA_WARP) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TC_TMEM_COLUMNS);
  }
}

// The cache [pages][2][nkv][page_size][hd] as rows of hd bfloat16; a box is 64 head dims by one
// page's rows (at most a tile's 128).  Maps are kept: the same caches come back every step.
bool cache_tensor_map(const __nv_bfloat16* cache, long long rows, int hd, int box_rows, CUtensorMap* out) {
  static std::mutex mutex;
  static std::map<std::tuple<const void*, long long, int, int>, CUtensorMap> kept;
  std::lock_guard<std::mutex> lock(mutex);
  const auto key = std::make_tuple(static_cast<const void*>(cache), rows, hd, box_rows);
  const auto found = kept.find(key);
  if (found != kept.end()) {
    *out = found->second;
    return true;
  }
  const EncodeTiled encode = tensor_map_encoder();
  if (encode == nullptr) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(hd), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(hd) * 2};
  const cuuint32_t box[2] = {64, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t element_strides[2] = {1, 1};
  if (encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<__nv_bfloat16*>(cache), dims, strides, box, element_strides,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (kept.size() > 4096) kept.clear();
  kept.emplace(key, *out);
  return true;
}

}  // namespace zb

using namespace zb;

// 1 if zb_paged_prefill_tc takes this shape.
namespace zb {
inline int*& prefill_tc_trace() {
  static int* buffer = nullptr;
  return buffer;
}
}  // namespace zb

// Timelines for later launches of zb_paged_prefill_tc: null (off) or 512 ints on the device (see
// PrefillTcArgs::trace; the second half: per tile, when the first loader thread began and ended
// the issue of its keys and of its values).
ZB_API int zb_paged_prefill_tc_set_trace(int* buffer) {
  prefill_tc_trace() = buffer;
  return OK;
}

ZB_API int zb_paged_prefill_tc_supported(int nh, int nkv, int hd, int dtype, int page_size) {
  if (dtype != DTYPE_BF16 || nkv <= 0 || nh <= 0 || nh % nkv != 0 || nh > 65535) return 0;
  if (hd != TC_HD || page_size < 8 || (page_size & (page_size - 1)) != 0) return 0;
  return 1;
}

// Attention of the tiles' tokens (tiles of 128 new tokens of one request) over their requests'
// pages; writes those tokens' rows of `out`.  Arguments as zb_paged_prefill.
ZB_API int zb_paged_prefill_tc(void* out, const void* q, const void* kv_cache, const int* block_table, int max_blocks,
                               int page_size, int num_pages, int num_rows, const int* tile_row, const int* tile_q0,
                               int n_tiles, const int* row_q_start, const int* row_q_len, const int* row_ctx, int nh,
                               int nkv, int hd, int window, float scale, int* status, void* stream) {
  if (n_tiles < 0 || page_size <= 0 || window < 0) return ERR_BAD_ARGUMENT;
  if (!zb_paged_prefill_tc_supported(nh, nkv, hd, DTYPE_BF16, page_size)) return ERR_UNSUPPORTED;
  if (reinterpret_cast<uintptr_t>(q) % 16 != 0 || reinterpret_cast<uintptr_t>(out) % 16 != 0 ||
      reinterpret_cast<uintptr_t>(kv_cache) % 16 != 0)
    return ERR_BAD_ARGUMENT;
  if (n_tiles == 0) return OK;
  if (n_tiles > 65535) return ERR_UNSUPPORTED;
  PrefillTcArgs a;
  const long long cache_rows = static_cast<long long>(num_pages) * 2 * nkv * page_size;
  a.tiled = cache_rows < (1LL << 31) &&
            cache_tensor_map(static_cast<const __nv_bfloat16*>(kv_cache), cache_rows, hd, page_size < TC_BN ? page_size : TC_BN,
                             &a.cache_map) ? 1 : 0;
  a.q = static_cast<const __nv_bfloat16*>(q);
  a.out = static_cast<__nv_bfloat16*>(out);
  a.kv_cache = static_cast<const __nv_bfloat16*>(kv_cache);
  a.block_table = block_table; a.tile_row = tile_row; a.tile_q0 = tile_q0;
  a.row_q_start = row_q_start; a.row_q_len = row_q_len; a.row_ctx = row_ctx;
  a.max_blocks = max_blocks; a.num_pages = num_pages; a.num_rows = num_rows;
  a.page_shift = 0;
  while ((1 << a.page_shift) < page_size) ++a.page_shift;
  a.nh = nh; a.nkv = nkv; a.window = window;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.status = status;
  a.trace = prefill_tc_trace();
  const size_t smem = 2 * TC_STAGES * TC_TILE_BYTES;
  if (cudaFuncSetAttribute(paged_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
    return ERR_CUDA;
  paged_prefill_tc_kernel<<<dim3(nh, n_tiles), TC_THREADS, smem, static_cast<cudaStream_t>(stream)>>>(a);
  return launch_result();
}
