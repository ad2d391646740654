// Memory-bound kernels around the matrix products: embedding gather, RMSNorm (alone and fused
// with the residual sum), SiLU(gate)*up, row gather.  All arithmetic is float32; one rounding at
// each store.  Formulas: the reference computes y = x * rsqrt(mean(x^2) + eps) * w
// (deps/ttl/src/kernels/normalization/normalization.cu:76-139), silu(z) = z / (1 + exp(-z))
// (src/layer/activation.cu:31-33) and r = a + x in float32 (src/model/causal_lm/qwen3.cpp:85-87).
#include <algorithm>

#include <type_traits>

#include "common.cuh"

namespace zb {

// Elements per 16-byte vector.
template <typename T> struct Vec;
template <> struct Vec<float> { static constexpr int N = 4; };
template <> struct Vec<__nv_bfloat16> { static constexpr int N = 8; };

template <typename T> __device__ __forceinline__ void load_vec(const T* p, float (&v)[Vec<T>::N]);
template <> __device__ __forceinline__ void load_vec<float>(const float* p, float (&v)[4]) {
  const float4 r = *reinterpret_cast<const float4*>(p);
  v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
}
template <> __device__ __forceinline__ void load_vec<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 r = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
template <typename T> __device__ __forceinline__ void store_vec(T* p, const float (&v)[Vec<T>::N]);
template <> __device__ __forceinline__ void store_vec<float>(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <> __device__ __forceinline__ void store_vec<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}

// ----------------------------------------------------------------------------- embedding
template <typename T, bool VECTOR>
__global__ void embedding_kernel(T* __restrict__ out, const T* __restrict__ table, const int* __restrict__ ids,
                                 int H, int V, int* status) {
  const int t = blockIdx.x;
  const int id = ids[t];
  if (id < 0 || id >= V) {
    if (threadIdx.x == 0) report(status, STATUS_TOKEN_OUT_OF_RANGE, id, t);
    return;
  }
  const T* src = table + static_cast<size_t>(id) * H;
  T* dst = out + static_cast<size_t>(t) * H;
  if (VECTOR) {
    constexpr int N = Vec<T>::N;
    for (int i = threadIdx.x * N; i < H; i += blockDim.x * N)
      *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>(src + i);
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = src[i];
  }
}

// Rows of x picked by index (the hidden states whose logits are wanted).
template <typename T>
__global__ void gather_rows_kernel(T* __restrict__ out, const T* __restrict__ x, const int* __restrict__ rows,
                                   int H, int num_src_rows, int* status) {
  const int r = blockIdx.x;
  const int src_row = rows[r];
  if (src_row < 0 || src_row >= num_src_rows) {
    if (threadIdx.x == 0) report(status, STATUS_ROW_OUT_OF_RANGE, src_row, r);
    return;
  }
  const T* src = x + static_cast<size_t>(src_row) * H;
  T* dst = out + static_cast<size_t>(r) * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = src[i];
}

// ------------------------------------------------------------------------------- RMSNorm
// One block per row.  With ADD the row of `residual` first takes `delta` (float32 sum, one
// rounding, stored back) and the norm is taken of the stored value, so that the fused and the
// separate form give the same bits.
template <typename T, bool ADD, bool VECTOR>
__global__ void rmsnorm_kernel(T* __restrict__ out, T* __restrict__ x, const T* __restrict__ delta,
                               const void* __restrict__ w, int w_dtype, float eps, int H,
                               long long x_stride, long long out_stride) {
  __shared__ float scratch[33];
  T* xr = x + static_cast<size_t>(blockIdx.x) * x_stride;
  const T* dr = ADD ? delta + static_cast<size_t>(blockIdx.x) * x_stride : nullptr;
  T* orow = out + static_cast<size_t>(blockIdx.x) * out_stride;
  float ss = 0.0f;
  if (VECTOR) {
    constexpr int N = Vec<T>::N;
    for (int i = threadIdx.x * N; i < H; i += blockDim.x * N) {
      float v[N];
      load_vec<T>(xr + i, v);
      if (ADD) {
        float d[N];
        load_vec<T>(dr + i, d);
#pragma unroll
        for (int k = 0; k < N; ++k) v[k] = to_float(from_float<T>(v[k] + d[k]));
        store_vec<T>(xr + i, v);
      }
#pragma unroll
      for (int k = 0; k < N; ++k) ss += v[k] * v[k];
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float v = to_float(xr[i]);
      if (ADD) {
        const T r = from_float<T>(v + to_float(dr[i]));
        xr[i] = r;
        v = to_float(r);
      }
      ss += v * v;
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / static_cast<float>(H) + eps);
  // Each thread re-reads exactly the elements it wrote above, so no fence is needed.
  if (VECTOR) {
    constexpr int N = Vec<T>::N;
    for (int i = threadIdx.x * N; i < H; i += blockDim.x * N) {
      float v[N];
      load_vec<T>(xr + i, v);
#pragma unroll
      for (int k = 0; k < N; ++k) v[k] = v[k] * inv * load_scale(w, w_dtype, i + k);
      store_vec<T>(orow + i, v);
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x)
      orow[i] = from_float<T>(to_float(xr[i]) * inv * load_scale(w, w_dtype, i));
  }
}

// The same for bfloat16 rows of up to 32 * 8 * V elements (V up to 8: 2048), one warp a row, four rows a block: all of a
// row's loads (the row, what is added to it, the scale) are in flight together, the values stay
// in registers between the sum of squares and the scaling, and nothing waits at a block's barrier.
// A prompt's 2048 rows of 1024 took 5.7 us with the kernel above (a second trip to memory for the
// row, the scale element by element).
constexpr int NORM_ROWS_PER_BLOCK = 4;

template <int V, bool ADD>
__global__ void __launch_bounds__(NORM_ROWS_PER_BLOCK * 32)
rmsnorm_warp_rows_kernel(__nv_bfloat16* __restrict__ out, __nv_bfloat16* __restrict__ x,
                         const __nv_bfloat16* __restrict__ delta, const void* __restrict__ w, int w_dtype, float eps,
                         int rows, int H, long long x_stride, long long out_stride) {
  const int lane = threadIdx.x & 31, row = blockIdx.x * NORM_ROWS_PER_BLOCK + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int n_vec = H / 8;
  __nv_bfloat16* xr = x + static_cast<size_t>(row) * x_stride;
  const __nv_bfloat16* dr = ADD ? delta + static_cast<size_t>(row) * x_stride : nullptr;
  __nv_bfloat16* orow = out + static_cast<size_t>(row) * out_stride;
  uint4 xv[V], dv[V], sv[V][2];
#pragma unroll
  for (int j = 0; j < V; ++j) {
    const int i = lane + 32 * j;
    if (i < n_vec) {
      xv[j] = *reinterpret_cast<const uint4*>(xr + i * 8);
      if (ADD) dv[j] = *reinterpret_cast<const uint4*>(dr + i * 8);
      if (w_dtype == DTYPE_F32) {
        sv[j][0] = *reinterpret_cast<const uint4*>(static_cast<const float*>(w) + i * 8);
        sv[j][1] = *reinterpret_cast<const uint4*>(static_cast<const float*>(w) + i * 8 + 4);
      } else {
        sv[j][0] = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(w) + i * 8);
      }
    }
  }
  float ss = 0.0f;
#pragma unroll
  for (int j = 0; j < V; ++j) {
    if (lane + 32 * j >= n_vec) break;
    __nv_bfloat162* x2 = reinterpret_cast<__nv_bfloat162*>(&xv[j]);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float2 v = __bfloat1622float2(x2[e]);
      if (ADD) {
        const float2 d = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(&dv[j])[e]);
        x2[e] = __floats2bfloat162_rn(v.x + d.x, v.y + d.y);       // the stream keeps the rounded sum ...
        v = __bfloat1622float2(x2[e]);                             // ... and the norm is taken of what it keeps
      }
      ss += v.x * v.x + v.y * v.y;
    }
    if (ADD) *reinterpret_cast<uint4*>(xr + (lane + 32 * j) * 8) = xv[j];
  }
  ss = warp_sum(ss);
  const float inv = rsqrtf(ss / static_cast<float>(H) + eps);
#pragma unroll
  for (int j = 0; j < V; ++j) {
    const int i = lane + 32 * j;
    if (i >= n_vec) break;
    const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&xv[j]);
    uint4 o;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 v = __bfloat1622float2(x2[e]);
      float2 scale;
      if (w_dtype == DTYPE_F32) {
        const float* s32 = reinterpret_cast<const float*>(&sv[j][0]);       // eight floats in the two vectors
        scale = make_float2(s32[2 * e], s32[2 * e + 1]);
      } else {
        scale = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(&sv[j][0])[e]);
      }
      o2[e] = __floats2bfloat162_rn(v.x * inv * scale.x, v.y * inv * scale.y);
    }
    *reinterpret_cast<uint4*>(orow + i * 8) = o;
  }
}

// ----------------------------------------------------------------------------- SiLU * up
// gu is [T, 2I]: columns [0, I) hold the gate, [I, 2I) the up projection.
template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gu, long long total, int I) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; e < total; e += stride) {
    const long long t = e / I;
    const int i = static_cast<int>(e - t * I);
    const float g = to_float(gu[t * 2 * I + i]);
    const float u = to_float(gu[t * 2 * I + I + i]);
    out[e] = from_float<T>(g / (1.0f + expf(-g)) * u);
  }
}

template <typename T>
__global__ void silu_mul_vec_kernel(T* __restrict__ out, const T* __restrict__ gu, long long total_vec, int I) {
  constexpr int N = Vec<T>::N;
  const int per_row = I / N;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; e < total_vec; e += stride) {
    const long long t = e / per_row;
    const int i = static_cast<int>(e - t * per_row) * N;
    float g[N], u[N];
    load_vec<T>(gu + t * 2 * I + i, g);
    load_vec<T>(gu + t * 2 * I + I + i, u);
#pragma unroll
    for (int k = 0; k < N; ++k) g[k] = g[k] / (1.0f + expf(-g[k])) * u[k];
    store_vec<T>(out + t * I + i, g);
  }
}

// The same for gate and up columns interleaved in blocks of 8: columns [16j, 16j+8) are gate
// values, [16j+8, 16j+16) the matching up values; out[t, 8j + r] = silu(gate) * up.
template <typename T>
__global__ void silu_mul_blocked_kernel(T* __restrict__ out, const T* __restrict__ gu, long long total, int I) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; e < total; e += stride) {
    const long long t = e / I;
    const int i = static_cast<int>(e - t * I);
    const long long base = t * 2 * I + (i / 8) * 16 + (i % 8);
    const float g = to_float(gu[base]);
    const float u = to_float(gu[base + 8]);
    out[e] = from_float<T>(g / (1.0f + expf(-g)) * u);
  }
}

// One thread per block of 8 outputs: the gate block and the up block are one 16-byte (bfloat16) or
// two 16-byte (float32) loads each.
template <typename T>
__global__ void silu_mul_blocked_vec_kernel(T* __restrict__ out, const T* __restrict__ gu, long long blocks8, int I) {
  constexpr int N = Vec<T>::N, PARTS = 8 / N;
  const int per_row = I / 8;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; e < blocks8; e += stride) {
    const long long t = e / per_row;
    const int j = static_cast<int>(e - t * per_row);
    const T* src = gu + t * 2 * I + j * 16;
    T* dst = out + t * I + j * 8;
#pragma unroll
    for (int p = 0; p < PARTS; ++p) {
      float g[N], u[N];
      load_vec<T>(src + p * N, g);
      load_vec<T>(src + 8 + p * N, u);
#pragma unroll
      for (int k = 0; k < N; ++k) g[k] = g[k] / (1.0f + expf(-g[k])) * u[k];
      store_vec<T>(dst + p * N, g);
    }
  }
}

// The same with one block per token row: no division to find the row, and a thread's loads (two
// blocks of eight outputs where the row has them) are all asked for before the first is used.
template <typename T>
__global__ void silu_mul_blocked_rows_kernel(T* __restrict__ out, const T* __restrict__ gu, int I) {
  constexpr int N = Vec<T>::N, PARTS = 8 / N;
  const int per_row = I / 8;
  const T* src = gu + static_cast<size_t>(blockIdx.x) * 2 * I;
  T* dst = out + static_cast<size_t>(blockIdx.x) * I;
  for (int j0 = threadIdx.x; j0 < per_row; j0 += 2 * blockDim.x) {
    const int j1 = j0 + blockDim.x;
    const bool second = j1 < per_row;
    float g[2][PARTS][N], u[2][PARTS][N];
#pragma unroll
    for (int p = 0; p < PARTS; ++p) {
      load_vec<T>(src + j0 * 16 + p * N, g[0][p]);
      load_vec<T>(src + j0 * 16 + 8 + p * N, u[0][p]);
      if (second) {
        load_vec<T>(src + j1 * 16 + p * N, g[1][p]);
        load_vec<T>(src + j1 * 16 + 8 + p * N, u[1][p]);
      }
    }
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      if (b == 1 && !second) break;
#pragma unroll
      for (int p = 0; p < PARTS; ++p) {
#pragma unroll
        for (int k = 0; k < N; ++k) g[b][p][k] = g[b][p][k] / (1.0f + expf(-g[b][p][k])) * u[b][p][k];
        store_vec<T>(dst + (b ? j1 : j0) * 8 + p * N, g[b][p]);
      }
    }
  }
}

// y[t, i] += b[i]: the bias of a projection, added in float32 and rounded once (no part of the one
// architecture has a bias; a mixer or feed-forward of another one may).
template <typename T>
__global__ void add_bias_kernel(T* __restrict__ y, long long ldy, const void* __restrict__ bias, int b_dtype, int T_, int N) {
  const long long total = static_cast<long long>(T_) * N;
  for (long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; e < total;
       e += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = e / N;
    const int i = static_cast<int>(e - t * N);
    T* at = y + t * ldy + i;
    *at = from_float<T>(to_float(*at) + load_scale(bias, b_dtype, i));
  }
}

template <typename T> bool aligned16(const void* p, long long elems) {
  return reinterpret_cast<uintptr_t>(p) % 16 == 0 && elems % Vec<T>::N == 0;
}

template <typename T>
int embedding_launch(void* out, const void* table, const int* ids, int T_, int H, int V, int* status,
                     cudaStream_t stream) {
  if (T_ == 0) return OK;
  const bool vec = aligned16<T>(out, H) && aligned16<T>(table, H);
  const int threads = 128;
  if (vec) embedding_kernel<T, true><<<T_, threads, 0, stream>>>((T*)out, (const T*)table, ids, H, V, status);
  else embedding_kernel<T, false><<<T_, threads, 0, stream>>>((T*)out, (const T*)table, ids, H, V, status);
  return launch_result();
}

template <typename T>
int rmsnorm_launch(void* out, void* x, const void* delta, const void* w, int w_dtype, float eps, int rows, int H,
                   long long x_stride, long long out_stride, cudaStream_t stream) {
  if (rows == 0) return OK;
  const bool vec = aligned16<T>(out, H) && aligned16<T>(x, H) && x_stride % Vec<T>::N == 0 &&
                   out_stride % Vec<T>::N == 0 && (delta == nullptr || aligned16<T>(delta, H));
  if (std::is_same<T, __nv_bfloat16>::value && vec && H % 8 == 0 && H <= 32 * 8 * 8 && rows >= 64 &&
      reinterpret_cast<uintptr_t>(w) % 16 == 0) {
    const int vectors = (H / 8 + 31) / 32;          // per lane
    const int blocks = (rows + NORM_ROWS_PER_BLOCK - 1) / NORM_ROWS_PER_BLOCK;
    const bool add = delta != nullptr;
#define ZB_ROWS(V_)                                                                                                  \
  do {                                                                                                               \
    if (add) rmsnorm_warp_rows_kernel<V_, true><<<blocks, NORM_ROWS_PER_BLOCK * 32, 0, stream>>>(                    \
        (__nv_bfloat16*)out, (__nv_bfloat16*)x, (const __nv_bfloat16*)delta, w, w_dtype, eps, rows, H, x_stride, out_stride); \
    else rmsnorm_warp_rows_kernel<V_, false><<<blocks, NORM_ROWS_PER_BLOCK * 32, 0, stream>>>(                       \
        (__nv_bfloat16*)out, (__nv_bfloat16*)x, nullptr, w, w_dtype, eps, rows, H, x_stride, out_stride);           \
  } while (0)
    if (vectors <= 1) ZB_ROWS(1);
    else if (vectors <= 2) ZB_ROWS(2);
    else if (vectors <= 4) ZB_ROWS(4);
    else ZB_ROWS(8);
#undef ZB_ROWS
    return launch_result();
  }
  const int per = vec ? Vec<T>::N : 1;
  int threads = ((H + per - 1) / per + 31) / 32 * 32;
  threads = threads < 32 ? 32 : (threads > 512 ? 512 : threads);
  const bool add = delta != nullptr;
#define ZB_NORM(ADD_, VEC_)                                                                            \
  rmsnorm_kernel<T, ADD_, VEC_><<<rows, threads, 0, stream>>>((T*)out, (T*)x, (const T*)delta, w, w_dtype, \
                                                               eps, H, x_stride, out_stride)
  if (add && vec) ZB_NORM(true, true);
  else if (add) ZB_NORM(true, false);
  else if (vec) ZB_NORM(false, true);
  else ZB_NORM(false, false);
#undef ZB_NORM
  return launch_result();
}

template <typename T>
int silu_mul_launch(void* out, const void* gu, int T_, int I, cudaStream_t stream) {
  if (T_ == 0 || I == 0) return OK;
  const int threads = 256;
  if (aligned16<T>(out, I) && aligned16<T>(gu, I)) {
    const long long total = static_cast<long long>(T_) * (I / Vec<T>::N);
    const int blocks = static_cast<int>(std::min<long long>((total + threads - 1) / threads, 148LL * 16));
    silu_mul_vec_kernel<T><<<blocks, threads, 0, stream>>>((T*)out, (const T*)gu, total, I);
  } else {
    const long long total = static_cast<long long>(T_) * I;
    const int blocks = static_cast<int>(std::min<long long>((total + threads - 1) / threads, 148LL * 16));
    silu_mul_kernel<T><<<blocks, threads, 0, stream>>>((T*)out, (const T*)gu, total, I);
  }
  return launch_result();
}

}  // namespace zb

using namespace zb;

// out[t, :] = table[ids[t], :]; an id outside [0, V) is reported in `status` and its row left as it was.
ZB_API int zb_embedding(void* out, const void* table, const int* ids, int T, int H, int V, int dtype, int* status,
                        void* stream) {
  if (T < 0 || H <= 0 || V <= 0) return ERR_BAD_ARGUMENT;
  auto s = static_cast<cudaStream_t>(stream);
  return dtype == DTYPE_F32 ? embedding_launch<float>(out, table, ids, T, H, V, status, s)
                            : embedding_launch<__nv_bfloat16>(out, table, ids, T, H, V, status, s);
}

ZB_API int zb_gather_rows(void* out, const void* x, const int* rows, int num_rows, int H, int num_src_rows,
                          int dtype, int* status, void* stream) {
  if (num_rows < 0 || H <= 0) return ERR_BAD_ARGUMENT;
  if (num_rows == 0) return OK;
  auto s = static_cast<cudaStream_t>(stream);
  if (dtype == DTYPE_F32)
    gather_rows_kernel<float><<<num_rows, 128, 0, s>>>((float*)out, (const float*)x, rows, H, num_src_rows, status);
  else
    gather_rows_kernel<__nv_bfloat16><<<num_rows, 128, 0, s>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)x, rows,
                                                               H, num_src_rows, status);
  return launch_result();
}

// out[r, :] = rmsnorm(x[r, :]) * w.  Rows are `x_stride` / `out_stride` elements apart (a per-head
// norm passes rows = tokens * heads, H = head size).  `out` may equal `x`.
ZB_API int zb_rmsnorm(void* out, const void* x, const void* w, int w_dtype, float eps, int rows, int H,
                      long long x_stride, long long out_stride, int dtype, void* stream) {
  if (rows < 0 || H <= 0 || x_stride < H || out_stride < H) return ERR_BAD_ARGUMENT;
  auto s = static_cast<cudaStream_t>(stream);
  return dtype == DTYPE_F32
             ? rmsnorm_launch<float>(out, const_cast<void*>(x), nullptr, w, w_dtype, eps, rows, H, x_stride, out_stride, s)
             : rmsnorm_launch<__nv_bfloat16>(out, const_cast<void*>(x), nullptr, w, w_dtype, eps, rows, H, x_stride,
                                             out_stride, s);
}

// residual[r, :] += delta[r, :] (stored), then out[r, :] = rmsnorm(residual[r, :]) * w.
ZB_API int zb_add_rmsnorm(void* out, void* residual, const void* delta, const void* w, int w_dtype, float eps,
                          int rows, int H, int dtype, void* stream) {
  if (rows < 0 || H <= 0 || delta == nullptr) return ERR_BAD_ARGUMENT;
  auto s = static_cast<cudaStream_t>(stream);
  return dtype == DTYPE_F32
             ? rmsnorm_launch<float>(out, residual, delta, w, w_dtype, eps, rows, H, H, H, s)
             : rmsnorm_launch<__nv_bfloat16>(out, residual, delta, w, w_dtype, eps, rows, H, H, H, s);
}

// out[t, i] = silu(gu[t, i]) * gu[t, I + i]; with blocked != 0 gate and up columns alternate in
// blocks of 8 (I a multiple of 8): out[t, 8j + r] = silu(gu[t, 16j + r]) * gu[t, 16j + 8 + r].
ZB_API int zb_silu_mul(void* out, const void* gu, int T, int I, int dtype, int blocked, void* stream) {
  if (T < 0 || I < 0 || (blocked && I % 8 != 0)) return ERR_BAD_ARGUMENT;
  auto s = static_cast<cudaStream_t>(stream);
  if (blocked) {
    if (T == 0 || I == 0) return OK;
    const bool vec = reinterpret_cast<uintptr_t>(out) % 16 == 0 && reinterpret_cast<uintptr_t>(gu) % 16 == 0;
    if (vec && T >= 64 && T <= 65535 * 1024) {
      const int per_row = I / 8;
      int threads = ((per_row + 1) / 2 + 31) / 32 * 32;
      threads = threads < 32 ? 32 : (threads > 256 ? 256 : threads);
      if (dtype == DTYPE_F32) silu_mul_blocked_rows_kernel<float><<<T, threads, 0, s>>>((float*)out, (const float*)gu, I);
      else silu_mul_blocked_rows_kernel<__nv_bfloat16><<<T, threads, 0, s>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)gu, I);
      return launch_result();
    }
    const long long total = vec ? static_cast<long long>(T) * (I / 8) : static_cast<long long>(T) * I;
    const int blocks = static_cast<int>(std::min<long long>((total + 255) / 256, 148LL * 16));
    if (dtype == DTYPE_F32) {
      if (vec) silu_mul_blocked_vec_kernel<float><<<blocks, 256, 0, s>>>((float*)out, (const float*)gu, total, I);
      else silu_mul_blocked_kernel<float><<<blocks, 256, 0, s>>>((float*)out, (const float*)gu, total, I);
    } else {
      if (vec) silu_mul_blocked_vec_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)gu, total, I);
      else silu_mul_blocked_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)gu, total, I);
    }
    return launch_result();
  }
  return dtype == DTYPE_F32 ? silu_mul_launch<float>(out, gu, T, I, s)
                            : silu_mul_launch<__nv_bfloat16>(out, gu, T, I, s);
}

// y [T, N] (rows ldy apart) += bias [N], the bias bfloat16 or float32.
ZB_API int zb_add_bias(void* y, long long ldy, const void* bias, int b_dtype, int T, int N, int dtype, void* stream) {
  if (T < 0 || N < 0 || ldy < N) return ERR_BAD_ARGUMENT;
  if (T == 0 || N == 0) return OK;
  const long long total = static_cast<long long>(T) * N;
  const int blocks = static_cast<int>(std::min<long long>((total + 255) / 256, 148LL * 16));
  auto s = static_cast<cudaStream_t>(stream);
  if (dtype == DTYPE_F32) add_bias_kernel<float><<<blocks, 256, 0, s>>>((float*)y, ldy, bias, b_dtype, T, N);
  else add_bias_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((__nv_bfloat16*)y, ldy, bias, b_dtype, T, N);
  return launch_result();
}

// The CUDA runtime's words for the last call of this library that failed (return code 2).
ZB_API const char* zb_last_cuda_error() { return last_cuda_error_text(); }
