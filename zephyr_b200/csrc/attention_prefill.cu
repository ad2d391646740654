// Paged causal attention for prompt portions (rows with several new tokens), bfloat16, on tensor
// cores: a flash-attention loop that reads keys and values straight from the cache pages, so a
// portion attends to everything its request has cached without any gather copy (the reference
// gathers the whole context of every row into packed tensors for each portion,
// src/layer/paged_attention.cpp:118-296, and then runs one scalar kernel per query row,
// deps/ttl/src/kernels/attention/attention.cu:58-170).
//
// One CTA = up to 128 consecutive new tokens of one request x one query head; 8 warps of 16 query
// rows.  Key/value tiles of 64 positions stream through a two-stage shared-memory ring filled by
// 16-byte asynchronous copies; S = Q K^T and O += P V run as m16n8k16 tensor-core products with
// float32 accumulators; the softmax is online, in float32, in base 2 with scale*log2(e) folded
// in; probabilities are rounded to bfloat16 for the second product.  Math and masking as in
// attention_simt.cu (causal, lower-right aligned on the cached context, optional window).
#include "common.cuh"
#include "mma.cuh"

namespace zb {

constexpr int PRE_BM = 128;     // query rows per CTA
constexpr int PRE_BN = 64;      // keys per tile
constexpr int PRE_WARPS = 8;

struct PrefillArgs {
  const __nv_bfloat16* q;        // [T, nh*hd]
  __nv_bfloat16* out;            // [T, nh*hd]
  const __nv_bfloat16* kv_cache; // [num_pages][2][nkv][page_size][hd]
  const int* block_table;        // [R, max_blocks]
  const int* tile_row;           // [n_tiles]
  const int* tile_q0;            // [n_tiles]
  const int* row_q_start;        // [R]
  const int* row_q_len;          // [R]
  const int* row_ctx;            // [R]
  int max_blocks, page_size, num_pages, num_rows;
  int nh, nkv, window;
  float scale_log2;
  int* status;
};

template <int HD>
__global__ void __launch_bounds__(PRE_WARPS * 32, 1)
paged_prefill_kernel(const PrefillArgs a) {
  static_assert(HD % 32 == 0 && HD <= 128, "head sizes 32, 64, 96, 128");
  constexpr int KROW = HD + 8;                      // padded rows: conflict-free ldmatrix
  constexpr int CHUNKS = HD / 8;
  constexpr int STAGE = 2 * PRE_BN * KROW;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);     // [PRE_BM][KROW]
  __nv_bfloat16* ring = q_s + PRE_BM * KROW;                             // [2][keys, values][PRE_BN][KROW]

  // The host lists the tiles by the number of keys they see, fewest first: take the list back to
  // front, and all heads of a tile before the next tile, so that the longest work of the whole
  // launch starts first and the short tiles fill the gaps at the end.
  const int tile = gridDim.y - 1 - blockIdx.y, head = blockIdx.x;
  const int row = a.tile_row[tile], q0 = a.tile_q0[tile];
  if (row < 0 || row >= a.num_rows) {
    if (threadIdx.x == 0) report(a.status, STATUS_ROW_OUT_OF_RANGE, row, tile);
    return;
  }
  const int g = a.nh / a.nkv, kvh = head / g;
  const int q_len = a.row_q_len[row], ctx = a.row_ctx[row], tok0 = a.row_q_start[row] + q0;
  const int n_tok = min(PRE_BM, q_len - q0);
  if (n_tok <= 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int quad_row = lane >> 2, quad_col = (lane & 3) * 2;
  const int* table = a.block_table + static_cast<size_t>(row) * a.max_blocks;

  // Keys any query of this tile may see: [lo, hi).
  const int hi = ctx + q0 + n_tok;
  const int lo = a.window > 0 ? max(0, ctx + q0 - a.window + 1) : 0;
  const int first_tile = lo / PRE_BN * PRE_BN;
  const int n_tiles = (hi - first_tile + PRE_BN - 1) / PRE_BN;

  for (int e = threadIdx.x; e < PRE_BM * CHUNKS; e += PRE_WARPS * 32) {
    const int j = e / CHUNKS, c = (e - j * CHUNKS) * 8;
    const bool ok = j < n_tok;
    cp_async_16(q_s + j * KROW + c, a.q + (static_cast<size_t>(tok0 + (ok ? j : 0)) * a.nh + head) * HD + c, ok);
  }
  auto load_tile = [&](int t) {
    __nv_bfloat16* ks = ring + (t & 1) * STAGE;
    __nv_bfloat16* vs = ks + PRE_BN * KROW;
    const int k0 = first_tile + t * PRE_BN;
    for (int e = threadIdx.x; e < PRE_BN * CHUNKS; e += PRE_WARPS * 32) {
      const int j = e / CHUNKS, c = (e - j * CHUNKS) * 8;
      const int pos = k0 + j;
      bool ok = pos >= lo && pos < hi;
      const __nv_bfloat16* src = a.kv_cache;
      if (ok) {
        const int block = pos / a.page_size;
        const int page = block < a.max_blocks ? table[block] : -1;
        if (page <= 0 || page >= a.num_pages) {
          report(a.status, STATUS_PAGE_OUT_OF_RANGE, page, tok0);
          ok = false;
        } else {
          // logical chunk c / 8 of the row sits at the permuted chunk (common.cuh: kv_swizzle)
          src += ((static_cast<long long>(page) * 2 * a.nkv + kvh) * a.page_size + pos % a.page_size) * HD +
                 (((c >> 3) ^ kv_swizzle(pos, CHUNKS)) << 3);
        }
      }
      cp_async_16(ks + j * KROW + c, src, ok);
      cp_async_16(vs + j * KROW + c, ok ? src + static_cast<long long>(a.nkv) * a.page_size * HD : src, ok);
    }
  };
  load_tile(0);
  cp_async_commit();

  // This warp's 16 query rows; this lane's two rows sit at positions qpos[0] and qpos[1].
  const int warp_row0 = warp * 16;
  const bool warp_active = warp_row0 < n_tok;
  const int qpos[2] = {ctx + q0 + warp_row0 + quad_row, ctx + q0 + warp_row0 + quad_row + 8};
  const int warp_last_pos = ctx + q0 + min(warp_row0 + 15, n_tok - 1);
  const int warp_first_visible = a.window > 0 ? max(0, ctx + q0 + warp_row0 - a.window + 1) : 0;

  unsigned qa[HD / 16][4];
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
  float o[HD / 8][4];
#pragma unroll
  for (int n = 0; n < HD / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;

  for (int t = 0; t < n_tiles; ++t) {
    cp_async_wait<0>();
    __syncthreads();                 // tile t (and, the first time, Q) has landed; tile t-1 is no longer read
    if (t + 1 < n_tiles) load_tile(t + 1);
    cp_async_commit();
    if (t == 0) {
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks)
        ldmatrix_x4(qa[ks], q_s + (warp_row0 + (lane & 7) + ((lane >> 3) & 1) * 8) * KROW + ks * 16 + (lane >> 4) * 8);
    }
    const int k0 = first_tile + t * PRE_BN;
    if (!warp_active || k0 > warp_last_pos || k0 + PRE_BN <= warp_first_visible) continue;   // uniform over the warp
    const __nv_bfloat16* ks_tile = ring + (t & 1) * STAGE;
    const __nv_bfloat16* vs_tile = ks_tile + PRE_BN * KROW;

    float s[PRE_BN / 8][4];
#pragma unroll
    for (int nt = 0; nt < PRE_BN / 8; ++nt) {
      s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f;
#pragma unroll
      for (int kk = 0; kk < HD / 32; ++kk) {
        unsigned b[4];
        ldmatrix_x4(b, ks_tile + (nt * 8 + (lane & 7)) * KROW + kk * 32 + (lane >> 3) * 8);
        mma_bf16_16816(s[nt], qa[2 * kk], b[0], b[1]);
        mma_bf16_16816(s[nt], qa[2 * kk + 1], b[2], b[3]);
      }
    }

    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < PRE_BN / 8; ++nt) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int pos = k0 + nt * 8 + quad_col + (c & 1);
        const int qp = qpos[c >> 1];
        const bool valid = pos <= qp && pos >= lo && (a.window == 0 || pos > qp - a.window);
        s[nt][c] = valid ? s[nt][c] * a.scale_log2 : -INFINITY;
        tile_max[c >> 1] = fmaxf(tile_max[c >> 1], s[nt][c]);
      }
    }
    float corr[2], m_use[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 1));
      tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 2));
      const float new_m = fmaxf(m_run[h], tile_max[h]);
      m_use[h] = new_m == -INFINITY ? 0.0f : new_m;      // a row that has seen no key yet: keep exp2 finite
      corr[h] = exp2f(m_run[h] - m_use[h]);              // 0 while the running maximum is -inf
      m_run[h] = new_m;
    }
    float row_sum[2] = {0.0f, 0.0f};
#pragma unroll
    for (int nt = 0; nt < PRE_BN / 8; ++nt) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        s[nt][c] = exp2f(s[nt][c] - m_use[c >> 1]);
        row_sum[c >> 1] += s[nt][c];
      }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      row_sum[h] += __shfl_xor_sync(0xffffffffu, row_sum[h], 1);
      row_sum[h] += __shfl_xor_sync(0xffffffffu, row_sum[h], 2);
      l_run[h] = l_run[h] * corr[h] + row_sum[h];
    }
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) {
      o[n][0] *= corr[0]; o[n][1] *= corr[0]; o[n][2] *= corr[1]; o[n][3] *= corr[1];
    }
#pragma unroll
    for (int ks = 0; ks < PRE_BN / 16; ++ks) {
      unsigned pa[4];
      pa[0] = pack_bf16(s[2 * ks][0], s[2 * ks][1]);
      pa[1] = pack_bf16(s[2 * ks][2], s[2 * ks][3]);
      pa[2] = pack_bf16(s[2 * ks + 1][0], s[2 * ks + 1][1]);
      pa[3] = pack_bf16(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
      for (int n2 = 0; n2 < HD / 16; ++n2) {
        unsigned b[4];
        ldmatrix_x4_trans(b, vs_tile + (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * KROW + n2 * 16 + (lane >> 4) * 8);
        mma_bf16_16816(o[2 * n2], pa, b[0], b[1]);
        mma_bf16_16816(o[2 * n2 + 1], pa, b[2], b[3]);
      }
    }
  }
  cp_async_wait<0>();

  if (!warp_active) return;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = warp_row0 + quad_row + 8 * h;
    if (r >= n_tok) continue;
    const float inv = l_run[h] > 0.0f ? 1.0f / l_run[h] : 0.0f;
    __nv_bfloat16* dst = a.out + (static_cast<size_t>(tok0 + r) * a.nh + head) * HD + quad_col;
#pragma unroll
    for (int n = 0; n < HD / 8; ++n)
      *reinterpret_cast<unsigned*>(dst + n * 8) = pack_bf16(o[n][2 * h] * inv, o[n][2 * h + 1] * inv);
  }
}

template <int HD>
int prefill_launch(const PrefillArgs& a, int n_tiles, cudaStream_t stream) {
  const size_t smem = (static_cast<size_t>(PRE_BM) + 4 * PRE_BN) * (HD + 8) * sizeof(__nv_bfloat16);
  auto kernel = paged_prefill_kernel<HD>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
    return ERR_CUDA;
  kernel<<<dim3(a.nh, n_tiles), PRE_WARPS * 32, smem, stream>>>(a);
  return launch_result();
}

}  // namespace zb

using namespace zb;

// Tokens of one request that a tile of this kernel covers (the host cuts rows into such tiles).
ZB_API int zb_paged_prefill_tile_tokens() { return PRE_BM; }

ZB_API int zb_paged_prefill_supported(int nh, int nkv, int hd, int dtype) {
  if (dtype != DTYPE_BF16 || nkv <= 0 || nh <= 0 || nh % nkv != 0 || nh > 65535) return 0;
  return hd == 32 || hd == 64 || hd == 96 || hd == 128 ? 1 : 0;
}

// Attention of the tiles' tokens over their requests' pages; writes those tokens' rows of `out`.
ZB_API int zb_paged_prefill(void* out, const void* q, const void* kv_cache, const int* block_table, int max_blocks,
                            int page_size, int num_pages, int num_rows, const int* tile_row, const int* tile_q0,
                            int n_tiles, const int* row_q_start, const int* row_q_len, const int* row_ctx, int nh,
                            int nkv, int hd, int window, float scale, int* status, void* stream) {
  if (n_tiles < 0 || page_size <= 0 || window < 0) return ERR_BAD_ARGUMENT;
  if (!zb_paged_prefill_supported(nh, nkv, hd, DTYPE_BF16)) return ERR_UNSUPPORTED;
  if (n_tiles == 0) return OK;
  if (n_tiles > 65535) return ERR_UNSUPPORTED;
  PrefillArgs a;
  a.q = static_cast<const __nv_bfloat16*>(q);
  a.out = static_cast<__nv_bfloat16*>(out);
  a.kv_cache = static_cast<const __nv_bfloat16*>(kv_cache);
  a.block_table = block_table; a.tile_row = tile_row; a.tile_q0 = tile_q0;
  a.row_q_start = row_q_start; a.row_q_len = row_q_len; a.row_ctx = row_ctx;
  a.max_blocks = max_blocks; a.page_size = page_size; a.num_pages = num_pages; a.num_rows = num_rows;
  a.nh = nh; a.nkv = nkv; a.window = window;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.status = status;
  auto s = static_cast<cudaStream_t>(stream);
  switch (hd) {
    case 32: return prefill_launch<32>(a, n_tiles, s);
    case 64: return prefill_launch<64>(a, n_tiles, s);
    case 96: return prefill_launch<96>(a, n_tiles, s);
    default: return prefill_launch<128>(a, n_tiles, s);
  }
}
