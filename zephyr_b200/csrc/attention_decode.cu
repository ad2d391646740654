// Split-context paged attention for single decoded tokens, bfloat16 keys and values, float32
// scores, softmax and accumulation.
//
// The decode step is bound by reading the cache, so the kernel is built around the copy.  Each CTA
// owns one (request, key/value head, split of the context) and streams its keys and values
// through a ring of shared-memory tiles.  The copies are bulk asynchronous copies (the TMA engine's
// untiled form, cp.async.bulk): one instruction per key row, completion counted on an mbarrier, so
// the threads spend no time on address arithmetic and several tiles are in flight per SM.  All query
// heads of the group share each tile; the two small products (scores, and probabilities times
// values) run on tensor cores with the group's heads padded to the 16 rows of an m16n8k16 tile.
// The last CTA of a (request, key/value head) to finish merges the splits: an atomic counter tells
// it that it is last, so no CTA ever waits for another, and no second launch is needed.
//
// Math as in attention_simt.cu (reference: src/attention/paged_decode.cu:169-352 for the split
// scheme), except where that kernel is not exact: no epsilon is added to the denominator, and
// partial results stay float32.  Probabilities are rounded to bfloat16 for the second product, as
// the reference does (paged_decode.cu:289).
#include "common.cuh"
#include "mma.cuh"

namespace zb {

constexpr int DEC_WARPS = 4;
constexpr int DEC_TILE = 64;            // keys per shared-memory tile; 16 per warp
constexpr int DEC_STAGES = 3;
constexpr int DEC_MAX_GROUP = 16;       // query heads per key/value head that fit one MMA tile
constexpr int DEC_WAIT_LIMIT = 1 << 22; // polls of an mbarrier before the kernel gives up and reports
static_assert(DEC_WARPS * 32 == 2 * DEC_TILE, "one key row or one value row per thread and tile");

struct DecodeArgs {
  const __nv_bfloat16* q;        // [T, nh*hd]
  __nv_bfloat16* out;            // [T, nh*hd]
  const __nv_bfloat16* kv_cache; // [num_pages][2][nkv][page_size][hd]
  const int* block_table;        // [R, max_blocks]
  const int* rows;               // [n_rows] request rows that decode one token
  const int* row_q_start;        // [R]
  const int* row_ctx;            // [R] tokens in the cache before this step (the new token's position)
  float* part_o;                 // [n_rows, nh, max_splits, hd]
  float* part_ml;                // [n_rows, nh, max_splits, 2]
  int* counters;                 // [n_rows, nkv] zero on entry, zero again on exit
  int max_blocks, page_shift, num_pages, num_rows;
  int nh, nkv, window, split_size, max_splits;
  float scale_log2;              // scale * log2(e)
  int* status;
};

// Which positions split `s` of a row covers: [begin, end), empty if begin >= end.
__device__ __forceinline__ void split_range(int ctx_total, int window, int split_size, int s, int& begin, int& end) {
  const int lo = window > 0 ? max(0, ctx_total - window) : 0;   // the query sits at ctx_total - 1
  begin = max(s * split_size, lo);
  end = min((s + 1) * split_size, ctx_total);
}

template <int HD>
__global__ void __launch_bounds__(DEC_WARPS * 32)
paged_decode_split_kernel(const DecodeArgs a) {
  static_assert(HD % 32 == 0 && HD <= 128, "head sizes 32, 64, 96, 128");
  constexpr int KROW = HD + 8;                     // padded row: ldmatrix reads without bank conflicts
  constexpr int STAGE = 2 * DEC_TILE * KROW;       // elements of one stage (keys, then values)
  constexpr unsigned ROW_BYTES = HD * sizeof(__nv_bfloat16);
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* tiles = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(tiles + DEC_STAGES * STAGE);
  __shared__ int is_last;

  const int split = blockIdx.x, kvh = blockIdx.y, r = blockIdx.z;
  const int row = a.rows[r];
  if (row < 0 || row >= a.num_rows) {
    if (threadIdx.x == 0) report(a.status, STATUS_ROW_OUT_OF_RANGE, row, r);
    return;
  }
  const int ctx_total = a.row_ctx[row] + 1;
  int begin, end;
  split_range(ctx_total, a.window, a.split_size, split, begin, end);
  if (begin >= end) return;

  const int g = a.nh / a.nkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int quad_row = lane >> 2, quad_col = (lane & 3) * 2;
  const int* table = a.block_table + static_cast<size_t>(row) * a.max_blocks;
  const int page_size = 1 << a.page_shift;

  if (threadIdx.x == 0) {
#pragma unroll
    for (int st = 0; st < DEC_STAGES; ++st) mbar_init(&bars[st], 1);
    fence_barrier_init();
  }
  __syncthreads();

  const int first_tile = begin / DEC_TILE * DEC_TILE;
  const int n_tiles = (end - first_tile + DEC_TILE - 1) / DEC_TILE;

  // Thread (j, sel) brings key row j (sel 0) or value row j (sel 1) of every tile.
  const int my_key = threadIdx.x & (DEC_TILE - 1), my_sel = threadIdx.x >> 6;
  const long long page_stride = 2LL * a.nkv * page_size * HD;
  const __nv_bfloat16* my_base = a.kv_cache + (static_cast<long long>(my_sel) * a.nkv + kvh) * page_size * HD;
  __nv_bfloat16* my_dst = tiles + my_sel * DEC_TILE * KROW + my_key * KROW;
  // The page of this thread's row of tile t (-1 outside the split).  Looked up one iteration before it
  // is needed, so that the copy of a tile is issued the moment its stage is free.
  auto lookup = [&](int t) -> int {
    const int pos = first_tile + t * DEC_TILE + my_key;
    if (t >= n_tiles || pos < begin || pos >= end) return -1;
    const int block = pos >> a.page_shift;
    const int page = block < a.max_blocks ? table[block] : 0;
    return page < 0 ? 0 : page;
  };
  auto load_tile = [&](int t, int page) {
    const int stage = t % DEC_STAGES;
    __nv_bfloat16* dst = my_dst + stage * STAGE;
    const int k0 = first_tile + t * DEC_TILE;
    if (threadIdx.x == 0) {
      const int n_valid = max(0, min(end, k0 + DEC_TILE) - max(begin, k0));
      mbar_arrive_expect_tx(&bars[stage], static_cast<unsigned>(n_valid) * 2u * ROW_BYTES);
    }
    if (page >= 0) {
      if (page == 0 || page >= a.num_pages) {
        report(a.status, STATUS_PAGE_OUT_OF_RANGE, page, row);
        page = 0;            // the announced bytes must still arrive: read the null page instead
      }
      bulk_copy_g2s(dst, my_base + page * page_stride + ((k0 + my_key) & (page_size - 1)) * HD, ROW_BYTES,
                    &bars[stage]);
    } else {
      // Outside the split: zeros, so that a probability of zero times this row stays zero.
#pragma unroll
      for (int c = 0; c < HD / 8; ++c) *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(0, 0, 0, 0);
    }
  };

#pragma unroll
  for (int t = 0; t < DEC_STAGES - 1; ++t)
    if (t < n_tiles) load_tile(t, lookup(t));
  int next_page = lookup(DEC_STAGES - 1);

  // The group's queries as the A operand (heads on the 16 rows; rows past the group are zero).
  unsigned qa[HD / 16][4];
  {
    const __nv_bfloat16* qrow = a.q + (static_cast<size_t>(a.row_q_start[row]) * a.nh + static_cast<size_t>(kvh) * g) * HD;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
      const int c = ks * 16 + quad_col;
      const unsigned* lo_row = reinterpret_cast<const unsigned*>(qrow + static_cast<size_t>(quad_row) * HD + c);
      const unsigned* hi_row = reinterpret_cast<const unsigned*>(qrow + static_cast<size_t>(quad_row + 8) * HD + c);
      qa[ks][0] = quad_row < g ? lo_row[0] : 0u;
      qa[ks][1] = quad_row + 8 < g ? hi_row[0] : 0u;
      qa[ks][2] = quad_row < g ? lo_row[4] : 0u;       // columns + 8
      qa[ks][3] = quad_row + 8 < g ? hi_row[4] : 0u;
    }
  }

  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
  float o[HD / 8][4];
#pragma unroll
  for (int n = 0; n < HD / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;

  for (int t = 0; t < n_tiles; ++t) {
    const bool landed = mbar_wait(&bars[t % DEC_STAGES], (t / DEC_STAGES) & 1, DEC_WAIT_LIMIT);
    // All threads agree (and all are done with tile t-1, whose stage the next load reuses).
    if (!__syncthreads_and(landed)) {
      if (threadIdx.x == 0) report(a.status, STATUS_COPY_TIMEOUT, t, row);
      // Give copies still in flight one more bounded chance to land before this CTA's shared memory goes away.
      for (int st = 0; st < DEC_STAGES; ++st) mbar_wait(&bars[st], ((t + st) / DEC_STAGES) & 1, 1 << 16);
      return;
    }
    fence_proxy_async();
    if (t + DEC_STAGES - 1 < n_tiles) load_tile(t + DEC_STAGES - 1, next_page);
    next_page = lookup(t + DEC_STAGES);

    const __nv_bfloat16* ks = tiles + (t % DEC_STAGES) * STAGE;
    const __nv_bfloat16* vs = ks + DEC_TILE * KROW;
    const int key0 = first_tile + t * DEC_TILE + warp * 16;   // this warp's 16 keys
    if (key0 >= end || key0 + 16 <= begin) continue;          // uniform over the warp

    // Scores: two n-tiles of 8 keys.  Four independent accumulator chains (n-tile x k-step parity)
    // instead of two keep the tensor core busy while a product is in flight.
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    float s_odd[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int kk = 0; kk < HD / 32; ++kk) {
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        unsigned b[4];
        ldmatrix_x4(b, ks + (warp * 16 + nt * 8 + (lane & 7)) * KROW + kk * 32 + (lane >> 3) * 8);
        mma_bf16_16816(s[nt], qa[2 * kk], b[0], b[1]);
        mma_bf16_16816(s_odd[nt], qa[2 * kk + 1], b[2], b[3]);
      }
    }
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) s[nt][c] += s_odd[nt][c];

    // Mask, running maximum, probabilities.
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int pos = key0 + nt * 8 + quad_col + (c & 1);
        const bool valid = pos >= begin && pos < end;
        s[nt][c] = valid ? s[nt][c] * a.scale_log2 : -INFINITY;
        tile_max[c >> 1] = fmaxf(tile_max[c >> 1], s[nt][c]);
      }
    }
    float corr[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 1));
      tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 2));
      const float new_m = fmaxf(m_run[h], tile_max[h]);       // finite: the warp's keys hold a visible one
      corr[h] = exp2f(m_run[h] - new_m);
      m_run[h] = new_m;
    }
    float row_sum[2] = {0.0f, 0.0f};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
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
    unsigned pa[4];
    pa[0] = pack_bf16(s[0][0], s[0][1]);
    pa[1] = pack_bf16(s[0][2], s[0][3]);
    pa[2] = pack_bf16(s[1][0], s[1][1]);
    pa[3] = pack_bf16(s[1][2], s[1][3]);

    // O = O * corr + P V over this warp's 16 keys.  Once the running maximum has settled, corr is
    // exactly 1 for every row of the warp and the rescaling is skipped.
    if (!__all_sync(0xffffffffu, corr[0] == 1.0f && corr[1] == 1.0f)) {
#pragma unroll
      for (int n = 0; n < HD / 8; ++n) {
        o[n][0] *= corr[0]; o[n][1] *= corr[0]; o[n][2] *= corr[1]; o[n][3] *= corr[1];
      }
    }
#pragma unroll
    for (int n2 = 0; n2 < HD / 16; ++n2) {
      unsigned b[4];
      ldmatrix_x4_trans(b, vs + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * KROW + n2 * 16 + (lane >> 4) * 8);
      mma_bf16_16816(o[2 * n2], pa, b[0], b[1]);
      mma_bf16_16816(o[2 * n2 + 1], pa, b[2], b[3]);
    }
  }
  __syncthreads();              // every warp is done with the tiles (all copies have landed); reuse them

  // Merge the four warps (each saw its own keys).
  float* merge_o = reinterpret_cast<float*>(smem_raw);               // [DEC_WARPS][16][HD]
  float* merge_ml = merge_o + DEC_WARPS * 16 * HD;                   // [DEC_WARPS][16][2]
#pragma unroll
  for (int n = 0; n < HD / 8; ++n) {
    float* base = merge_o + (warp * 16 + quad_row) * HD + n * 8 + quad_col;
    base[0] = o[n][0]; base[1] = o[n][1];
    base[8 * HD] = o[n][2]; base[8 * HD + 1] = o[n][3];
  }
  if ((lane & 3) == 0) {
    merge_ml[(warp * 16 + quad_row) * 2] = m_run[0];
    merge_ml[(warp * 16 + quad_row) * 2 + 1] = l_run[0];
    merge_ml[(warp * 16 + quad_row + 8) * 2] = m_run[1];
    merge_ml[(warp * 16 + quad_row + 8) * 2 + 1] = l_run[1];
  }
  __syncthreads();

  // How many splits of this row hold keys (the others returned at the top).
  const int lo = a.window > 0 ? max(0, ctx_total - a.window) : 0;
  const int first_split = lo / a.split_size, last_split = (ctx_total - 1) / a.split_size;
  const bool alone = first_split == last_split;
  const size_t out_base = (static_cast<size_t>(a.row_q_start[row]) * a.nh + static_cast<size_t>(kvh) * g) * HD;

  for (int e = threadIdx.x; e < g * HD; e += DEC_WARPS * 32) {
    const int h = e / HD, d = e - h * HD;
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) mx = fmaxf(mx, merge_ml[(w * 16 + h) * 2]);
    float acc = 0.0f, l = 0.0f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float mw = merge_ml[(w * 16 + h) * 2];
      const float f = mw == -INFINITY ? 0.0f : exp2f(mw - mx);
      acc += merge_o[(w * 16 + h) * HD + d] * f;
      l += merge_ml[(w * 16 + h) * 2 + 1] * f;
    }
    if (alone) {                 // the only split of its row: this is the result
      a.out[out_base + e] = __float2bfloat16_rn(l > 0.0f ? acc / l : 0.0f);
    } else {
      const size_t slot = (static_cast<size_t>(r) * a.nh + static_cast<size_t>(kvh) * g + h) * a.max_splits + split;
      a.part_o[slot * HD + d] = acc;
      if (d == 0) {
        a.part_ml[slot * 2] = mx;
        a.part_ml[slot * 2 + 1] = l;
      }
    }
  }
  if (alone) return;

  // Whoever arrives last finds every split's partial result written and merges them.
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int arrived = atomicAdd(&a.counters[r * a.nkv + kvh], 1);
    is_last = arrived == last_split - first_split;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  for (int e = threadIdx.x; e < g * HD; e += DEC_WARPS * 32) {
    const int h = e / HD, d = e - h * HD;
    const size_t base = (static_cast<size_t>(r) * a.nh + static_cast<size_t>(kvh) * g + h) * a.max_splits;
    float mx = -INFINITY;
    for (int sp = first_split; sp <= last_split; ++sp) mx = fmaxf(mx, __ldcg(&a.part_ml[(base + sp) * 2]));
    float acc = 0.0f, l = 0.0f;
    for (int sp = first_split; sp <= last_split; ++sp) {
      const float f = exp2f(__ldcg(&a.part_ml[(base + sp) * 2]) - mx);
      acc += __ldcg(&a.part_o[(base + sp) * HD + d]) * f;
      l += __ldcg(&a.part_ml[(base + sp) * 2 + 1]) * f;
    }
    a.out[out_base + e] = __float2bfloat16_rn(l > 0.0f ? acc / l : 0.0f);
  }
  if (threadIdx.x == 0) a.counters[r * a.nkv + kvh] = 0;      // left as it was found, for the next call
}

template <int HD> size_t decode_smem_bytes() {
  const size_t ring = static_cast<size_t>(DEC_STAGES) * 2 * DEC_TILE * (HD + 8) * sizeof(__nv_bfloat16) +
                      DEC_STAGES * sizeof(unsigned long long);
  const size_t merge = static_cast<size_t>(DEC_WARPS) * 16 * (HD + 2) * sizeof(float);
  return ring > merge ? ring : merge;
}

template <int HD>
int decode_launch(const DecodeArgs& a, int n_rows, cudaStream_t stream) {
  const size_t smem = decode_smem_bytes<HD>();
  auto kernel = paged_decode_split_kernel<HD>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
    return ERR_CUDA;
  kernel<<<dim3(a.max_splits, a.nkv, n_rows), DEC_WARPS * 32, smem, stream>>>(a);
  return launch_result();
}

}  // namespace zb

using namespace zb;

// 1 if zb_paged_decode takes this shape, else 0 (the caller then uses the general kernel).
ZB_API int zb_paged_decode_supported(int nh, int nkv, int hd, int dtype) {
  if (dtype != DTYPE_BF16 || nkv <= 0 || nh % nkv != 0 || nh / nkv > DEC_MAX_GROUP) return 0;
  return hd == 32 || hd == 64 || hd == 96 || hd == 128 ? 1 : 0;
}

// Floats of scratch the kernel needs for the partial results of the splits.
ZB_API long long zb_paged_decode_scratch_floats(int n_rows, int nh, int hd, int max_splits) {
  return static_cast<long long>(n_rows) * nh * max_splits * (hd + 2);
}

// Attention of `n_rows` single new tokens over their paged context.  `scratch` holds
// zb_paged_decode_scratch_floats(...) floats (contents irrelevant); `counters` holds n_rows * nkv
// ints that are zero on entry and are left zero.  max_splits >= ceil((longest context + 1) /
// split_size); split_size is a multiple of 64; page_size is a power of two.
ZB_API int zb_paged_decode(void* out, const void* q, const void* kv_cache, const int* block_table, int max_blocks,
                           int page_size, int num_pages, int num_rows, const int* rows, int n_rows,
                           const int* row_q_start, const int* row_ctx, int nh, int nkv, int hd, int window,
                           float scale, int split_size, int max_splits, float* scratch, int* counters, int* status,
                           void* stream) {
  if (n_rows < 0 || max_splits <= 0 || split_size <= 0 || split_size % DEC_TILE != 0 || page_size <= 0 || window < 0 ||
      counters == nullptr)
    return ERR_BAD_ARGUMENT;
  if (!zb_paged_decode_supported(nh, nkv, hd, DTYPE_BF16) || (page_size & (page_size - 1)) != 0) return ERR_UNSUPPORTED;
  if (n_rows == 0) return OK;
  if (n_rows > 65535 || nkv > 65535) return ERR_UNSUPPORTED;
  int page_shift = 0;
  while ((1 << page_shift) < page_size) ++page_shift;
  DecodeArgs a;
  a.q = static_cast<const __nv_bfloat16*>(q);
  a.out = static_cast<__nv_bfloat16*>(out);
  a.kv_cache = static_cast<const __nv_bfloat16*>(kv_cache);
  a.block_table = block_table; a.rows = rows; a.row_q_start = row_q_start; a.row_ctx = row_ctx;
  a.part_o = scratch;
  a.part_ml = scratch + static_cast<size_t>(n_rows) * nh * max_splits * hd;
  a.counters = counters;
  a.max_blocks = max_blocks; a.page_shift = page_shift; a.num_pages = num_pages; a.num_rows = num_rows;
  a.nh = nh; a.nkv = nkv; a.window = window; a.split_size = split_size; a.max_splits = max_splits;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.status = status;
  auto s = static_cast<cudaStream_t>(stream);
  switch (hd) {
    case 32: return decode_launch<32>(a, n_rows, s);
    case 64: return decode_launch<64>(a, n_rows, s);
    case 96: return decode_launch<96>(a, n_rows, s);
    default: return decode_launch<128>(a, n_rows, s);
  }
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

ZB_API long long zb_paged_decode_no_alloc_bytes_needed(int n_rows, int nh, int hd, int max_splits) {
  // Partial results, plus the arrival counters (at most one per row and head) rounded up to 256 bytes.
  return zb_paged_decode_scratch_floats(n_rows, nh, hd, max_splits) * static_cast<long long>(sizeof(float)) +
         (static_cast<long long>(n_rows) * nh * 4 + 255) / 256 * 256;
}

ZB_API const char* zb_paged_decode_no_alloc_error(int code) {
  switch (code) {
    case OK: return "launched";
    case ERR_BAD_ARGUMENT: return "an argument lies outside the kernel's contract";
    case ERR_CUDA: return "the CUDA launch failed";
    case ERR_UNSUPPORTED: return "this head size, group size or type is not supported by the decode kernel";
    case ZB_ERR_SCRATCH_TOO_SMALL:
      return "the problem needs more than the 4 MiB of built-in scratch: n_rows * heads * max_splits * "
             "(head_dim + 2) * 4 bytes must not exceed ZB_NO_ALLOC_SCRATCH_BYTES; use zb_paged_decode with a buffer "
             "of your own, or split the rows over several calls";
    case ZB_ERR_SCRATCH_ADDRESS: return "the device address of the built-in scratch array could not be looked up";
    default: return "unknown code";
  }
}

ZB_API int zb_paged_decode_no_alloc(void* out, const void* q, const void* kv_cache, const int* block_table,
                                    int max_blocks, int page_size, int num_pages, int num_rows, const int* rows,
                                    int n_rows, const int* row_q_start, const int* row_ctx, int nh, int nkv, int hd,
                                    int window, float scale, int split_size, int max_splits, int* status,
                                    void* stream) {
  if (n_rows < 0 || nh <= 0 || nkv <= 0 || nkv > nh || hd <= 0 || max_splits <= 0) return ERR_BAD_ARGUMENT;
  if (zb_paged_decode_no_alloc_bytes_needed(n_rows, nh, hd, max_splits) > static_cast<long long>(ZB_NO_ALLOC_SCRATCH_BYTES))
    return ZB_ERR_SCRATCH_TOO_SMALL;
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
