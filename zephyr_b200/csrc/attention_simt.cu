// Paged causal attention on CUDA cores, float32 arithmetic throughout: the kernel of the true
// 32-bit path, and the general one (any head size in steps of 16 up to 256, any head and group
// counts, any page size, with or without a window, any mixture of prompt portions and single
// decoded tokens).
//
// Math (reference: deps/ttl/src/kernels/attention/attention.cu:46-56,76-77,90-166): query head j
// uses key/value head j / g; s = scale * (q . k) with scale = 1/sqrt(hd); a query at absolute
// position p sees the keys of its own sequence at positions <= p (and > p - window when the
// layer has a window); softmax with a running maximum; o = sum softmax * v.  There is no epsilon
// in the denominator and exp is expf.  A position encoding that is a bias on the scores, linear
// in the distance (a slope per query head), is added here; the one architecture has none, and
// the faster kernels do not take one.
//
// One CTA serves one tile: a run of consecutive new tokens of one request, one key/value head,
// and a chunk of that head's query heads.  The (token, head) pairs of the tile are dealt to the
// warps; key/value tiles of 32 positions are staged in shared memory once and used by all pairs.
#include "common.cuh"

namespace zb {

constexpr int ATT_WARPS = 4;
constexpr int ATT_PAIRS_PER_WARP = 4;
constexpr int ATT_MAX_PAIRS = ATT_WARPS * ATT_PAIRS_PER_WARP;   // 16 (token, head) pairs per CTA
constexpr int ATT_TILE = 32;                                    // keys per shared-memory tile

struct AttentionArgs {
  const void* q;            // [T, nh*hd]
  void* out;                // [T, nh*hd]
  const void* kv_cache;     // [num_pages][2][nkv][page_size][hd]
  const int* block_table;   // [R, max_blocks]
  const int* tile_row;      // [n_tiles] request row of the tile
  const int* tile_q0;       // [n_tiles] offset of the tile's first token within the row's new tokens
  const int* row_q_start;   // [R] index of the row's first new token in the flattened stream
  const int* row_q_len;     // [R]
  const int* row_ctx;       // [R] tokens already in the cache before this step
  int max_blocks, page_size, num_pages, num_rows;
  int nh, nkv, hd, window, tile_tokens, heads_per_chunk;
  float scale;
  const float* head_slopes;  // null, or [nh]: query head h adds head_slopes[h] * (key position - query position) to its scores
  int* status;
};

template <typename T> struct KPad;
template <> struct KPad<float> { static constexpr int N = 1; };
template <> struct KPad<__nv_bfloat16> { static constexpr int N = 2; };

template <typename T, int ACC>
__global__ void __launch_bounds__(ATT_WARPS * 32)
paged_attention_simt_kernel(const AttentionArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int hd = a.hd, g = a.nh / a.nkv;
  const int kstride = hd + KPad<T>::N;
  float* q_s = reinterpret_cast<float*>(smem_raw);                       // [ATT_MAX_PAIRS][hd]
  T* k_s = reinterpret_cast<T*>(q_s + ATT_MAX_PAIRS * hd);               // [ATT_TILE][kstride]
  T* v_s = k_s + ATT_TILE * kstride;                                      // [ATT_TILE][hd]

  const int tile = blockIdx.x, kvh = blockIdx.y, chunk = blockIdx.z;
  const int row = a.tile_row[tile], q0 = a.tile_q0[tile];
  if (row < 0 || row >= a.num_rows) {
    if (threadIdx.x == 0) report(a.status, STATUS_ROW_OUT_OF_RANGE, row, tile);
    return;
  }
  const int q_len = a.row_q_len[row], ctx = a.row_ctx[row], tok0 = a.row_q_start[row] + q0;
  const int n_tok = min(a.tile_tokens, q_len - q0);
  const int n_heads = min(a.heads_per_chunk, g - chunk * a.heads_per_chunk);
  if (n_tok <= 0 || n_heads <= 0) return;
  const int n_pairs = n_tok * n_heads;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* q = static_cast<const T*>(a.q);
  const T* cache = static_cast<const T*>(a.kv_cache);

  // Queries of all pairs, as float32.
  for (int e = threadIdx.x; e < n_pairs * hd; e += blockDim.x) {
    const int p = e / hd, d = e - p * hd;
    const int qi = p / n_heads, hj = p - qi * n_heads;
    const int head = kvh * g + chunk * a.heads_per_chunk + hj;
    q_s[p * hd + d] = to_float(q[(static_cast<size_t>(tok0 + qi) * a.nh + head) * hd + d]);
  }

  float m[ATT_PAIRS_PER_WARP], l[ATT_PAIRS_PER_WARP], acc[ATT_PAIRS_PER_WARP][ACC];
#pragma unroll
  for (int i = 0; i < ATT_PAIRS_PER_WARP; ++i) {
    m[i] = -INFINITY;
    l[i] = 0.0f;
#pragma unroll
    for (int c = 0; c < ACC; ++c) acc[i][c] = 0.0f;
  }

  // Keys any pair of this tile may see: [lo, hi).
  const int hi = ctx + q0 + n_tok;
  const int lo = a.window > 0 ? max(0, ctx + q0 - a.window + 1) : 0;
  const int vec = 16 / static_cast<int>(sizeof(T));
  const int chunks_per_row = hd / vec;

  for (int k0 = lo / ATT_TILE * ATT_TILE; k0 < hi; k0 += ATT_TILE) {
    __syncthreads();     // the previous tile is no longer read (and q_s is complete on the first pass)
    for (int e = threadIdx.x; e < ATT_TILE * chunks_per_row; e += blockDim.x) {
      const int j = e / chunks_per_row, d = (e - j * chunks_per_row) * vec;
      const int pos = k0 + j;
      bool ok = pos >= lo && pos < hi;
      long long base = 0;
      if (ok) {
        const int block = pos / a.page_size;
        const int page = block < a.max_blocks ? a.block_table[static_cast<size_t>(row) * a.max_blocks + block] : -1;
        if (page <= 0 || page >= a.num_pages) {
          report(a.status, STATUS_PAGE_OUT_OF_RANGE, page, tok0);
          ok = false;
        } else {
          // logical chunk d / vec of the row sits at the permuted chunk (common.cuh: kv_swizzle)
          base = ((static_cast<long long>(page) * 2 * a.nkv + kvh) * a.page_size + pos % a.page_size) * hd +
                 (((d / vec) ^ kv_swizzle(pos, chunks_per_row)) * vec);
        }
      }
      // Positions outside [lo, hi) hold zeros: a page that was given back, or one that another
      // request used before, is never read.
      uint4 kr = make_uint4(0, 0, 0, 0), vr = make_uint4(0, 0, 0, 0);
      if (ok) {
        kr = *reinterpret_cast<const uint4*>(cache + base);
        vr = *reinterpret_cast<const uint4*>(cache + base + static_cast<long long>(a.nkv) * a.page_size * hd);
      }
      const T* ke = reinterpret_cast<const T*>(&kr);
      const T* ve = reinterpret_cast<const T*>(&vr);
#pragma unroll
      for (int u = 0; u < 16 / static_cast<int>(sizeof(T)); ++u) {
        k_s[j * kstride + d + u] = ke[u];
        v_s[j * hd + d + u] = ve[u];
      }
    }
    __syncthreads();

    const int kp = k0 + lane;
#pragma unroll
    for (int i = 0; i < ATT_PAIRS_PER_WARP; ++i) {
      const int p = warp + i * ATT_WARPS;
      if (p >= n_pairs) continue;                       // uniform over the warp
      const int qpos = ctx + q0 + p / n_heads;
      const float slope = a.head_slopes != nullptr
                              ? a.head_slopes[kvh * g + chunk * a.heads_per_chunk + (p - p / n_heads * n_heads)] : 0.0f;
      const int first = a.window > 0 ? max(0, qpos - a.window + 1) : 0;
      if (k0 > qpos || k0 + ATT_TILE <= first) continue;  // no key of this tile is visible
      const bool valid = kp <= qpos && kp >= first;
      float s = 0.0f;
      const float* qp = q_s + p * hd;
      const T* kr = k_s + lane * kstride;
      for (int d = 0; d < hd; d += 2) {
        s = fmaf(qp[d], to_float(kr[d]), s);
        s = fmaf(qp[d + 1], to_float(kr[d + 1]), s);
      }
      s = valid ? fmaf(slope, static_cast<float>(kp - qpos), s * a.scale) : -INFINITY;
      const float new_m = fmaxf(m[i], warp_max(s));      // finite: the tile holds a visible key
      const float pr = valid ? expf(s - new_m) : 0.0f;
      const float corr = expf(m[i] - new_m);             // exp(-inf) = 0 on the first tile
      l[i] = l[i] * corr + warp_sum(pr);
      m[i] = new_m;
#pragma unroll
      for (int c = 0; c < ACC; ++c) acc[i][c] *= corr;
      for (int j = 0; j < ATT_TILE; ++j) {
        const float pj = __shfl_sync(0xffffffffu, pr, j);
        if (pj == 0.0f) continue;                         // uniform over the warp
#pragma unroll
        for (int c = 0; c < ACC; ++c) {
          const int d = lane + 32 * c;
          if (d < hd) acc[i][c] = fmaf(pj, to_float(v_s[j * hd + d]), acc[i][c]);
        }
      }
    }
  }

  T* out = static_cast<T*>(a.out);
#pragma unroll
  for (int i = 0; i < ATT_PAIRS_PER_WARP; ++i) {
    const int p = warp + i * ATT_WARPS;
    if (p >= n_pairs) continue;
    const int qi = p / n_heads, hj = p - qi * n_heads;
    const int head = kvh * g + chunk * a.heads_per_chunk + hj;
    const float inv = l[i] > 0.0f ? 1.0f / l[i] : 0.0f;   // a fully masked row gives zeros
#pragma unroll
    for (int c = 0; c < ACC; ++c) {
      const int d = lane + 32 * c;
      if (d < hd) out[(static_cast<size_t>(tok0 + qi) * a.nh + head) * hd + d] = from_float<T>(acc[i][c] * inv);
    }
  }
}

template <typename T, int ACC>
int attention_simt_launch(const AttentionArgs& a, int n_tiles, int head_chunks, cudaStream_t stream) {
  const size_t smem = static_cast<size_t>(ATT_MAX_PAIRS) * a.hd * sizeof(float) +
                      static_cast<size_t>(ATT_TILE) * (2 * a.hd + KPad<T>::N) * sizeof(T);
  auto kernel = paged_attention_simt_kernel<T, ACC>;
  if (smem > 48 * 1024 &&
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
    return ERR_CUDA;
  kernel<<<dim3(n_tiles, a.nkv, head_chunks), ATT_WARPS * 32, smem, stream>>>(a);
  return launch_result();
}

template <typename T>
int attention_simt_dispatch(const AttentionArgs& a, int n_tiles, int head_chunks, cudaStream_t stream) {
  switch ((a.hd + 31) / 32) {
    case 1: return attention_simt_launch<T, 1>(a, n_tiles, head_chunks, stream);
    case 2: return attention_simt_launch<T, 2>(a, n_tiles, head_chunks, stream);
    case 3: return attention_simt_launch<T, 3>(a, n_tiles, head_chunks, stream);
    case 4: return attention_simt_launch<T, 4>(a, n_tiles, head_chunks, stream);
    case 5: return attention_simt_launch<T, 5>(a, n_tiles, head_chunks, stream);
    case 6: return attention_simt_launch<T, 6>(a, n_tiles, head_chunks, stream);
    case 7: return attention_simt_launch<T, 7>(a, n_tiles, head_chunks, stream);
    case 8: return attention_simt_launch<T, 8>(a, n_tiles, head_chunks, stream);
    default: return ERR_UNSUPPORTED;
  }
}

}  // namespace zb

using namespace zb;

// How many consecutive new tokens of one request a tile of the general kernel covers, for a
// model with `group` query heads per key/value head.  The host cuts each row's new tokens into
// tiles of this many tokens.
ZB_API int zb_attention_simt_tile_tokens(int group) {
  const int heads_per_chunk = group < ATT_MAX_PAIRS ? group : ATT_MAX_PAIRS;
  const int t = ATT_MAX_PAIRS / heads_per_chunk;
  return t < 1 ? 1 : t;
}

ZB_API int zb_paged_attention_simt(void* out, const void* q, const void* kv_cache, const int* block_table,
                                   int max_blocks, int page_size, int num_pages, int num_rows, const int* tile_row,
                                   const int* tile_q0, int n_tiles, int tile_tokens, const int* row_q_start,
                                   const int* row_q_len, const int* row_ctx, int nh, int nkv, int hd, int window,
                                   float scale, const float* head_slopes, int dtype, int* status, void* stream) {
  if (nh <= 0 || nkv <= 0 || nh % nkv != 0 || hd <= 0 || page_size <= 0 || n_tiles < 0 || window < 0)
    return ERR_BAD_ARGUMENT;
  if (hd % 16 != 0 || hd > 256) return ERR_UNSUPPORTED;
  if (n_tiles == 0) return OK;
  const int g = nh / nkv;
  const int heads_per_chunk = g < ATT_MAX_PAIRS ? g : ATT_MAX_PAIRS;
  if (tile_tokens <= 0 || tile_tokens * heads_per_chunk > ATT_MAX_PAIRS) return ERR_BAD_ARGUMENT;
  const int head_chunks = (g + heads_per_chunk - 1) / heads_per_chunk;
  AttentionArgs a;
  a.q = q; a.out = out; a.kv_cache = kv_cache; a.block_table = block_table;
  a.tile_row = tile_row; a.tile_q0 = tile_q0;
  a.row_q_start = row_q_start; a.row_q_len = row_q_len; a.row_ctx = row_ctx;
  a.max_blocks = max_blocks; a.page_size = page_size; a.num_pages = num_pages; a.num_rows = num_rows;
  a.nh = nh; a.nkv = nkv; a.hd = hd; a.window = window; a.tile_tokens = tile_tokens;
  a.heads_per_chunk = heads_per_chunk; a.scale = scale; a.head_slopes = head_slopes; a.status = status;
  auto s = static_cast<cudaStream_t>(stream);
  return dtype == DTYPE_F32 ? attention_simt_dispatch<float>(a, n_tiles, head_chunks, s)
                            : attention_simt_dispatch<__nv_bfloat16>(a, n_tiles, head_chunks, s);
}
