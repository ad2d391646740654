// Per-head RMSNorm of q and k, NeoX rotary embedding, and the write of k and v into cache pages:
// fused in one pass over the projection output, and as separate kernels for mixers that combine
// other parts.
//
// Formulas (reference): q and k are normalised per head over the head size with one shared
// scale vector each and the layer's eps, before the rotation (src/model/causal_lm/qwen3.cpp:53-56);
// rotation pairs are (i, i + hd/2): x' = x*c - y*s, y' = y*c + x*s with c, s from the table row of
// the token's position (src/layer/rotary_embedding.cu:24-47); k and v rows go to the page slot
// page*page_size + pos % page_size (src/attention/cache.cu:17-56).  Unlike the reference, which
// rounds to the storage type after the norm and after each product of the rotation, everything
// here is float32 until the single store.
//
// Cache layout of one cache: [num_pages][2 (k, v)][num_kv_heads][page_size][head_dim], each row with
// its 16-byte chunks permuted by kv_swizzle(position) (common.cuh).
#include "common.cuh"

namespace zb {

constexpr int ROPE_WARPS = 4;
constexpr int MAX_PAIRS_PER_LANE = 4;   // head sizes up to 256

struct CacheView {
  void* base;            // null: nothing is written
  const int* block_table;
  int max_blocks;        // row length of block_table
  int page_size;
  int num_pages;
  int num_rows;
};

__device__ __forceinline__ long long cache_row_offset(const CacheView& c, int row, int pos, int kv_sel, int kvh,
                                                      int nkv, int hd, int* status, int t) {
  const int block = pos / c.page_size;
  if (row < 0 || row >= c.num_rows || block >= c.max_blocks) {
    report(status, STATUS_ROW_OUT_OF_RANGE, row, t);
    return -1;
  }
  const int page = c.block_table[static_cast<size_t>(row) * c.max_blocks + block];
  if (page <= 0 || page >= c.num_pages) {      // page 0 is the null page and is never written
    report(status, STATUS_PAGE_OUT_OF_RANGE, page, t);
    return -1;
  }
  return (((static_cast<long long>(page) * 2 + kv_sel) * nkv + kvh) * c.page_size + pos % c.page_size) * hd;
}

// Two adjacent elements as one load or store.
template <typename T> struct Pair;
template <> struct Pair<float> {
  using type = float2;
  static __device__ __forceinline__ void load(const float* p, float& a, float& b) {
    const float2 v = *reinterpret_cast<const float2*>(p);
    a = v.x; b = v.y;
  }
  static __device__ __forceinline__ void store(float* p, float a, float b) {
    *reinterpret_cast<float2*>(p) = make_float2(a, b);
  }
};
template <> struct Pair<__nv_bfloat16> {
  using type = __nv_bfloat162;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float& a, float& b) {
    const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
    a = v.x; b = v.y;
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
  }
};

// One warp per (token, head).  Lane l of pass k owns the adjacent elements 2(l + 32k), +1 of the
// first half of the head and their partners in the second half (the rotation pairs i, i + hd/2).
template <typename T>
__global__ void qk_norm_rope_cache_kernel(T* __restrict__ q_out, const T* __restrict__ qkv, long long qkv_stride,
                                          const void* __restrict__ q_norm_w, const void* __restrict__ k_norm_w,
                                          int w_dtype, float eps, const float* __restrict__ cos_table,
                                          const float* __restrict__ sin_table, int max_positions,
                                          const int* __restrict__ positions, const int* __restrict__ token_row,
                                          CacheView cache, int nh, int nkv, int hd, int* status) {
  constexpr int PASSES = MAX_PAIRS_PER_LANE / 2;      // 64 elements of a half per pass: head sizes up to 256
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31;
  const int head = blockIdx.y * ROPE_WARPS + (threadIdx.x >> 5);
  const int total_heads = cache.base != nullptr ? nh + 2 * nkv : nh;
  if (head >= total_heads) return;
  const int half = hd / 2;
  const int pos = positions[t];
  const bool is_q = head < nh, is_k = !is_q && head < nh + nkv;
  const T* src = qkv + static_cast<size_t>(t) * qkv_stride + static_cast<size_t>(head) * hd;

  float x[PASSES][2], y[PASSES][2];
  float ss = 0.0f;
#pragma unroll
  for (int k = 0; k < PASSES; ++k) {
    const int i = 2 * (lane + 32 * k);
    x[k][0] = x[k][1] = y[k][0] = y[k][1] = 0.0f;
    if (i < half) {
      Pair<T>::load(src + i, x[k][0], x[k][1]);
      Pair<T>::load(src + i + half, y[k][0], y[k][1]);
      ss += x[k][0] * x[k][0] + x[k][1] * x[k][1] + y[k][0] * y[k][0] + y[k][1] * y[k][1];
    }
  }

  T* dst;
  if (is_q) {
    dst = q_out + (static_cast<size_t>(t) * nh + head) * hd;
  } else {
    const int kvh = is_k ? head - nh : head - nh - nkv;
    const long long off = cache_row_offset(cache, token_row[t], pos, is_k ? 0 : 1, kvh, nkv, hd, status, t);
    if (off < 0) return;
    dst = static_cast<T*>(cache.base) + off;
  }

  if (is_q || is_k) {
    const void* w = is_q ? q_norm_w : k_norm_w;
    if (w != nullptr) {
      const float inv = rsqrtf(warp_sum(ss) / static_cast<float>(hd) + eps);
#pragma unroll
      for (int k = 0; k < PASSES; ++k) {
        const int i = 2 * (lane + 32 * k);
        if (i < half) {
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            x[k][u] *= inv * load_scale(w, w_dtype, i + u);
            y[k][u] *= inv * load_scale(w, w_dtype, i + u + half);
          }
        }
      }
    }
    if (cos_table != nullptr) {
      if (pos < 0 || pos >= max_positions) {
        if (lane == 0) report(status, STATUS_POSITION_OUT_OF_RANGE, pos, t);
        return;
      }
      const float* c = cos_table + static_cast<size_t>(pos) * half;
      const float* s = sin_table + static_cast<size_t>(pos) * half;
#pragma unroll
      for (int k = 0; k < PASSES; ++k) {
        const int i = 2 * (lane + 32 * k);
        if (i < half) {
          const float2 cv = *reinterpret_cast<const float2*>(c + i), sv = *reinterpret_cast<const float2*>(s + i);
          const float cs[2] = {cv.x, cv.y}, sn[2] = {sv.x, sv.y};
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const float xr = x[k][u] * cs[u] - y[k][u] * sn[u];
            const float yr = y[k][u] * cs[u] + x[k][u] * sn[u];
            x[k][u] = xr;
            y[k][u] = yr;
          }
        }
      }
    }
  }
  // q goes out as it is; cache rows are stored with their 16-byte chunks permuted (kv_swizzle); two
  // adjacent elements never straddle a chunk.
#pragma unroll
  for (int k = 0; k < PASSES; ++k) {
    const int i = 2 * (lane + 32 * k);
    if (i < half) {
      const int lo = is_q ? i : kv_element_index(i, pos, hd, sizeof(T));
      const int hi = is_q ? i + half : kv_element_index(i + half, pos, hd, sizeof(T));
      Pair<T>::store(dst + lo, x[k][0], x[k][1]);
      Pair<T>::store(dst + hi, y[k][0], y[k][1]);
    }
  }
}

// The same for bfloat16 and head sizes 64 and 128, E = 4 or 8 elements of each half a lane: a head is
// HD / (2 E) lanes (lane j owns elements E j .. E j + E - 1 of the first half and their partners in
// the second), so a warp takes several heads of a token at once and every load and store is a
// vector.  The math and the cache layout are those of the kernel above; the sum of squares runs
// in another order.  Everything a lane needs is asked for in two rounds (the token's position and
// row and the lane's elements and scales; then the page id and the angles), and with E = 8 a
// prompt's tokens make half as many warps: the kernel is bound by those rounds, not by bytes.
template <int HD, int E>
__global__ void __launch_bounds__(ROPE_WARPS * 32)
qk_norm_rope_cache_wide_kernel(__nv_bfloat16* __restrict__ q_out, const __nv_bfloat16* __restrict__ qkv,
                               long long qkv_stride, const void* __restrict__ q_norm_w,
                               const void* __restrict__ k_norm_w, int w_dtype, float eps,
                               const float* __restrict__ cos_table, const float* __restrict__ sin_table,
                               int max_positions, const int* __restrict__ positions,
                               const int* __restrict__ token_row, CacheView cache, int nh, int nkv, int* status) {
  constexpr int LANES = HD / (2 * E), HEADS_PER_WARP = 32 / LANES, HALF = HD / 2, WORDS = E / 2;
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, sub = lane % LANES;
  const int head = (blockIdx.y * ROPE_WARPS + (threadIdx.x >> 5)) * HEADS_PER_WARP + lane / LANES;
  const int total_heads = cache.base != nullptr ? nh + 2 * nkv : nh;
  const bool active = head < total_heads;
  const bool is_q = head < nh, is_k = !is_q && head < nh + nkv;
  const int i = E * sub;                                        // this lane's elements i .. i + E - 1 and i + HALF ..
  const int pos = positions[t], row = token_row[t];             // the step's description: older than any kernel of the step
  // The scales do not depend on the step either.
  float scale_x[E], scale_y[E];
  const void* w = is_q ? q_norm_w : (is_k ? k_norm_w : nullptr);
  if (active && w != nullptr) {
#pragma unroll
    for (int u = 0; u < E; ++u) {
      scale_x[u] = load_scale(w, w_dtype, i + u);
      scale_y[u] = load_scale(w, w_dtype, i + u + HALF);
    }
  }
  wait_for_prior_grids();           // the projections are an earlier kernel's output
  let_dependents_launch();
  unsigned xw[WORDS], yw[WORDS];
#pragma unroll
  for (int u = 0; u < WORDS; ++u) xw[u] = yw[u] = 0u;
  if (active) {
    const __nv_bfloat16* src = qkv + static_cast<size_t>(t) * qkv_stride + static_cast<size_t>(head) * HD;
    if (E == 8) {
      const uint4 xv = *reinterpret_cast<const uint4*>(src + i), yv = *reinterpret_cast<const uint4*>(src + i + HALF);
      xw[0] = xv.x; xw[1] = xv.y; xw[WORDS - 2] = xv.z; xw[WORDS - 1] = xv.w;
      yw[0] = yv.x; yw[1] = yv.y; yw[WORDS - 2] = yv.z; yw[WORDS - 1] = yv.w;
    } else {
      const uint2 xv = *reinterpret_cast<const uint2*>(src + i), yv = *reinterpret_cast<const uint2*>(src + i + HALF);
      xw[0] = xv.x; xw[1] = xv.y;
      yw[0] = yv.x; yw[1] = yv.y;
    }
  }
  // The second round: where the row goes, and its angles.
  long long off = 0;
  if (active && !is_q) {
    const int kvh = is_k ? head - nh : head - nh - nkv;
    off = cache_row_offset(cache, row, pos, is_k ? 0 : 1, kvh, nkv, HD, status, t);
  }
  const bool rotates = active && (is_q || is_k) && cos_table != nullptr;
  const bool pos_ok = pos >= 0 && pos < max_positions;
  float cs[E], si[E];
  if (rotates && pos_ok) {
#pragma unroll
    for (int u = 0; u < E; u += 4) {
      const float4 c = *reinterpret_cast<const float4*>(cos_table + static_cast<size_t>(pos) * HALF + i + u);
      const float4 sn = *reinterpret_cast<const float4*>(sin_table + static_cast<size_t>(pos) * HALF + i + u);
      cs[u] = c.x; cs[u + 1] = c.y; cs[u + 2] = c.z; cs[u + 3] = c.w;
      si[u] = sn.x; si[u + 1] = sn.y; si[u + 2] = sn.z; si[u + 3] = sn.w;
    }
  }
  float x[E], y[E];
#pragma unroll
  for (int u = 0; u < WORDS; ++u) {
    const float2 xf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xw[u]));
    const float2 yf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&yw[u]));
    x[2 * u] = xf.x; x[2 * u + 1] = xf.y;
    y[2 * u] = yf.x; y[2 * u + 1] = yf.y;
  }
  float ss = 0.0f;
#pragma unroll
  for (int u = 0; u < E; ++u) ss += x[u] * x[u] + y[u] * y[u];
#pragma unroll
  for (int o = LANES / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);     // over the head's lanes
  if (!active || off < 0) return;

  __nv_bfloat16* dst = is_q ? q_out + (static_cast<size_t>(t) * nh + head) * HD
                            : static_cast<__nv_bfloat16*>(cache.base) + off;
  if (is_q || is_k) {
    if (w != nullptr) {
      const float inv = rsqrtf(ss / static_cast<float>(HD) + eps);
#pragma unroll
      for (int u = 0; u < E; ++u) {
        x[u] *= inv * scale_x[u];
        y[u] *= inv * scale_y[u];
      }
    }
    if (cos_table != nullptr) {
      if (!pos_ok) {
        if (sub == 0) report(status, STATUS_POSITION_OUT_OF_RANGE, pos, t);
        return;
      }
#pragma unroll
      for (int u = 0; u < E; ++u) {
        const float xr = x[u] * cs[u] - y[u] * si[u];
        const float yr = y[u] * cs[u] + x[u] * si[u];
        x[u] = xr;
        y[u] = yr;
      }
    }
  }
  // E adjacent elements never straddle a 16-byte chunk of a cache row.
  const int lo = is_q ? i : kv_element_index(i, pos, HD, sizeof(__nv_bfloat16));
  const int hi = is_q ? i + HALF : kv_element_index(i + HALF, pos, HD, sizeof(__nv_bfloat16));
  unsigned xo[WORDS], yo[WORDS];
#pragma unroll
  for (int u = 0; u < WORDS; ++u) {
    *reinterpret_cast<__nv_bfloat162*>(&xo[u]) = __floats2bfloat162_rn(x[2 * u], x[2 * u + 1]);
    *reinterpret_cast<__nv_bfloat162*>(&yo[u]) = __floats2bfloat162_rn(y[2 * u], y[2 * u + 1]);
  }
  if (E == 8) {
    *reinterpret_cast<uint4*>(dst + lo) = make_uint4(xo[0], xo[1], xo[WORDS - 2], xo[WORDS - 1]);
    *reinterpret_cast<uint4*>(dst + hi) = make_uint4(yo[0], yo[1], yo[WORDS - 2], yo[WORDS - 1]);
  } else {
    *reinterpret_cast<uint2*>(dst + lo) = make_uint2(xo[0], xo[1]);
    *reinterpret_cast<uint2*>(dst + hi) = make_uint2(yo[0], yo[1]);
  }
}

// In-place rotation of x [T, heads, hd] (rows `stride` elements apart).
template <typename T>
__global__ void rope_kernel(T* __restrict__ x, long long stride, int heads, int hd,
                            const float* __restrict__ cos_table, const float* __restrict__ sin_table,
                            int max_positions, const int* __restrict__ positions, int* status) {
  const int t = blockIdx.x;
  const int pos = positions[t];
  if (pos < 0 || pos >= max_positions) {
    if (threadIdx.x == 0) report(status, STATUS_POSITION_OUT_OF_RANGE, pos, t);
    return;
  }
  const int half = hd / 2;
  const float* c = cos_table + static_cast<size_t>(pos) * half;
  const float* s = sin_table + static_cast<size_t>(pos) * half;
  for (int e = threadIdx.x; e < heads * half; e += blockDim.x) {
    const int h = e / half, i = e - h * half;
    T* row = x + static_cast<size_t>(t) * stride + static_cast<size_t>(h) * hd;
    const float a = to_float(row[i]), b = to_float(row[i + half]);
    row[i] = from_float<T>(a * c[i] - b * s[i]);
    row[i + half] = from_float<T>(b * c[i] + a * s[i]);
  }
}

// k and v [T, nkv, hd] (rows `stride` elements apart) into their page slots.
template <typename T>
__global__ void kv_write_kernel(const T* __restrict__ k, const T* __restrict__ v, long long k_stride,
                                long long v_stride, const int* __restrict__ positions,
                                const int* __restrict__ token_row, CacheView cache, int nkv, int hd, int* status) {
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int row = token_row[t];
  for (int kvh = 0; kvh < nkv; ++kvh) {
    for (int sel = 0; sel < 2; ++sel) {
      const long long off = cache_row_offset(cache, row, pos, sel, kvh, nkv, hd, status, t);
      if (off < 0) return;
      const T* src = (sel == 0 ? k + static_cast<size_t>(t) * k_stride : v + static_cast<size_t>(t) * v_stride) +
                     static_cast<size_t>(kvh) * hd;
      T* dst = static_cast<T*>(cache.base) + off;
      for (int i = threadIdx.x; i < hd; i += blockDim.x) dst[kv_element_index(i, pos, hd, sizeof(T))] = src[i];
    }
  }
}

}  // namespace zb

using namespace zb;

// Fused: per-head RMSNorm of q and k (scales may be null: no norm), NeoX rotation by the tables
// (may be null: no rotation), q to q_out [T, nh*hd], k and v into the cache (kv_cache may be null:
// only q is produced, for a layer that reads another layer's cache).
// qkv: [T, >= (nh + 2*nkv)*hd], q heads first, then k heads, then v heads.
ZB_API int zb_qk_norm_rope_cache(void* q_out, const void* qkv, long long qkv_stride, const void* q_norm_w,
                                 const void* k_norm_w, int w_dtype, float eps, const float* cos_table,
                                 const float* sin_table, int max_positions, const int* positions,
                                 const int* token_row, void* kv_cache, const int* block_table, int max_blocks,
                                 int page_size, int num_pages, int num_rows, int T, int nh, int nkv, int hd,
                                 int dtype, int* status, void* stream) {
  if (T < 0 || nh <= 0 || nkv <= 0 || hd <= 0 || hd % 2 != 0 || page_size <= 0) return ERR_BAD_ARGUMENT;
  if (hd > 64 * MAX_PAIRS_PER_LANE) return ERR_UNSUPPORTED;
  if ((cos_table == nullptr) != (sin_table == nullptr)) return ERR_BAD_ARGUMENT;
  if (T == 0) return OK;
  const CacheView cache{kv_cache, block_table, max_blocks, page_size, num_pages, num_rows};
  const int heads = kv_cache != nullptr ? nh + 2 * nkv : nh;
  const dim3 grid(T, (heads + ROPE_WARPS - 1) / ROPE_WARPS);
  auto s = static_cast<cudaStream_t>(stream);
  if (dtype == DTYPE_F32)
    qk_norm_rope_cache_kernel<float><<<grid, ROPE_WARPS * 32, 0, s>>>(
        (float*)q_out, (const float*)qkv, qkv_stride, q_norm_w, k_norm_w, w_dtype, eps, cos_table, sin_table,
        max_positions, positions, token_row, cache, nh, nkv, hd, status);
  else if ((hd == 64 || hd == 128) && qkv_stride % 4 == 0 && reinterpret_cast<uintptr_t>(qkv) % 8 == 0 &&
           reinterpret_cast<uintptr_t>(q_out) % 8 == 0 && reinterpret_cast<uintptr_t>(kv_cache) % 8 == 0 &&
           reinterpret_cast<uintptr_t>(cos_table) % 16 == 0 && reinterpret_cast<uintptr_t>(sin_table) % 16 == 0) {
    // Sixteen bytes a lane where everything is aligned for it and there are tokens enough to fill
    // the GPU with half as many warps; eight bytes a lane otherwise.
    const bool sixteen = T >= 64 && qkv_stride % 8 == 0 && reinterpret_cast<uintptr_t>(qkv) % 16 == 0 &&
                         reinterpret_cast<uintptr_t>(q_out) % 16 == 0 && reinterpret_cast<uintptr_t>(kv_cache) % 16 == 0;
    const int per_warp = 32 / (hd / (sixteen ? 16 : 8));
    const dim3 wide(T, (heads + ROPE_WARPS * per_warp - 1) / (ROPE_WARPS * per_warp));
#define ZB_WIDE(HD_, E_)                                                                                            \
  return launch_dependent(qk_norm_rope_cache_wide_kernel<HD_, E_>, wide, dim3(ROPE_WARPS * 32), 0, s, false,        \
                          (__nv_bfloat16*)q_out, (const __nv_bfloat16*)qkv, qkv_stride, q_norm_w, k_norm_w, w_dtype, eps, \
                          cos_table, sin_table, max_positions, positions, token_row, cache, nh, nkv, status)
    if (hd == 64 && sixteen) ZB_WIDE(64, 8);
    else if (hd == 64) ZB_WIDE(64, 4);
    else if (sixteen) ZB_WIDE(128, 8);
    else ZB_WIDE(128, 4);
#undef ZB_WIDE
  } else
    qk_norm_rope_cache_kernel<__nv_bfloat16><<<grid, ROPE_WARPS * 32, 0, s>>>(
        (__nv_bfloat16*)q_out, (const __nv_bfloat16*)qkv, qkv_stride, q_norm_w, k_norm_w, w_dtype, eps, cos_table,
        sin_table, max_positions, positions, token_row, cache, nh, nkv, hd, status);
  return launch_result();
}

ZB_API int zb_rope(void* x, long long stride, int T, int heads, int hd, const float* cos_table,
                   const float* sin_table, int max_positions, const int* positions, int dtype, int* status,
                   void* stream) {
  if (T < 0 || heads <= 0 || hd <= 0 || hd % 2 != 0 || cos_table == nullptr || sin_table == nullptr)
    return ERR_BAD_ARGUMENT;
  if (T == 0) return OK;
  auto s = static_cast<cudaStream_t>(stream);
  if (dtype == DTYPE_F32)
    rope_kernel<float><<<T, 128, 0, s>>>((float*)x, stride, heads, hd, cos_table, sin_table, max_positions,
                                         positions, status);
  else
    rope_kernel<__nv_bfloat16><<<T, 128, 0, s>>>((__nv_bfloat16*)x, stride, heads, hd, cos_table, sin_table,
                                                 max_positions, positions, status);
  return launch_result();
}

ZB_API int zb_kv_write(const void* k, const void* v, long long k_stride, long long v_stride, const int* positions,
                       const int* token_row, void* kv_cache, const int* block_table, int max_blocks, int page_size,
                       int num_pages, int num_rows, int T, int nkv, int hd, int dtype, int* status, void* stream) {
  if (T < 0 || nkv <= 0 || hd <= 0 || page_size <= 0 || kv_cache == nullptr) return ERR_BAD_ARGUMENT;
  if (T == 0) return OK;
  const CacheView cache{kv_cache, block_table, max_blocks, page_size, num_pages, num_rows};
  auto s = static_cast<cudaStream_t>(stream);
  if (dtype == DTYPE_F32)
    kv_write_kernel<float><<<T, 128, 0, s>>>((const float*)k, (const float*)v, k_stride, v_stride, positions,
                                             token_row, cache, nkv, hd, status);
  else
    kv_write_kernel<__nv_bfloat16><<<T, 128, 0, s>>>((const __nv_bfloat16*)k, (const __nv_bfloat16*)v, k_stride,
                                                     v_stride, positions, token_row, cache, nkv, hd, status);
  return launch_result();
}
