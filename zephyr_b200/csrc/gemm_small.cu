// Y[M, N] = X[M, K] * W[N, K]^T for the few rows of a decode step (M <= 64), bfloat16 with float32
// accumulation: a weight streamer.  Every weight is read once, straight from global memory into
// tensor-core fragments by 16-byte loads (no shared-memory staging), so many loads are in flight
// per warp; the activations, a few KB, come from L2 the same way.
//
// The weight rows sit on the 16-row side of m16n8k16 and the tokens on the 8-column side (the
// product is computed as W X^T).  Inside a block of 32 consecutive k, lane t of a quad owns the 8
// consecutive values k = 8t .. 8t+7 of its row: one 16-byte load feeds two tensor-core products.
// The products see k in a permuted order, the same for both operands, so the sum is unchanged.
//
// One CTA owns 16 rows of W; its four warps split K, and for matrices with few rows a cluster of
// up to 8 CTAs splits K further.  Partial sums meet in (distributed) shared memory and are added in
// a fixed order, so the result does not depend on timing.  With SWIGLU the 16 rows are 8 gate
// rows followed by their 8 up rows, and the epilogue writes silu(gate) * up: the activation costs
// no extra pass over memory (reference: src/layer/mlp.cpp:29-36, src/layer/activation.cu:31-33).
#include <cooperative_groups.h>

#include "common.cuh"
#include "mma.cuh"

namespace zb {

namespace cg = cooperative_groups;

constexpr int GS_ROWS = 16;       // weight rows per CTA
constexpr int GS_WARPS = 4;
constexpr int GS_MAX_MT = 8;      // token tiles of 8: M <= 64
constexpr int GS_MAX_KSPLIT = 8;

struct SmallGemmArgs {
  void* y;
  const __nv_bfloat16* x;
  const __nv_bfloat16* w;
  int M, N, K;
  long long ldx, ldw, ldy;
};

__device__ __forceinline__ uint4 load16_or_zero(const __nv_bfloat16* p, bool ok) {
  return ok ? *reinterpret_cast<const uint4*>(p) : make_uint4(0, 0, 0, 0);
}

template <typename T> __device__ __forceinline__ void store_out(T* p, float v);
template <> __device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16* p, float v) {
  *p = __float2bfloat16_rn(v);
}

template <int MT, typename TOut, bool SWIGLU>
__global__ void __launch_bounds__(GS_WARPS * 32)
gemm_small_kernel(const SmallGemmArgs a) {
  // Partial sums of this CTA's warps: [warp][mt][row][token].
  __shared__ float red[GS_WARPS][MT][GS_ROWS][8];
  cg::cluster_group cluster = cg::this_cluster();
  const int ksplit = gridDim.y, krank = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * GS_ROWS;

  const int total_blocks = (a.K + 31) / 32;
  const int slices = GS_WARPS * ksplit, slice = krank * GS_WARPS + warp;
  const int b_begin = static_cast<int>(static_cast<long long>(total_blocks) * slice / slices);
  const int b_end = static_cast<int>(static_cast<long long>(total_blocks) * (slice + 1) / slices);

  const bool lo_ok = n0 + g < a.N, hi_ok = n0 + g + 8 < a.N;
  const __nv_bfloat16* w_lo = a.w + static_cast<size_t>(lo_ok ? n0 + g : 0) * a.ldw + 8 * t;
  const __nv_bfloat16* w_hi = a.w + static_cast<size_t>(hi_ok ? n0 + g + 8 : 0) * a.ldw + 8 * t;
  const __nv_bfloat16* x_row[MT];
  bool x_ok[MT];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    x_ok[mt] = mt * 8 + g < a.M;
    x_row[mt] = a.x + static_cast<size_t>(x_ok[mt] ? mt * 8 + g : 0) * a.ldx + 8 * t;
  }

  float acc[MT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.0f;

#pragma unroll 8
  for (int b = b_begin; b < b_end; ++b) {
    const int k = b * 32;
    const bool k_ok = k + 8 * t + 8 <= a.K;          // K is a multiple of 8: a chunk is whole or absent
    const uint4 wl = load16_or_zero(w_lo + k, lo_ok && k_ok);
    const uint4 wh = load16_or_zero(w_hi + k, hi_ok && k_ok);
    const unsigned a0[4] = {wl.x, wh.x, wl.y, wh.y};
    const unsigned a1[4] = {wl.z, wh.z, wl.w, wh.w};
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const uint4 xv = load16_or_zero(x_row[mt] + k, x_ok[mt] && k_ok);
      mma_bf16_16816(acc[mt], a0, xv.x, xv.y);
      mma_bf16_16816(acc[mt], a1, xv.z, xv.w);
    }
  }

#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    red[warp][mt][g][2 * t] = acc[mt][0];
    red[warp][mt][g][2 * t + 1] = acc[mt][1];
    red[warp][mt][g + 8][2 * t] = acc[mt][2];
    red[warp][mt][g + 8][2 * t + 1] = acc[mt][3];
  }
  // Every CTA of the cluster has its partial sums in its shared memory; a cluster of one needs only
  // its own barrier (the cluster's costs a fence that the language-model head paid 9496 times).
  if (ksplit == 1) __syncthreads();
  else cluster.sync();

  if (krank == 0) {
    // The first CTA of the cluster adds all partial sums, warp by warp and CTA by CTA, and writes.
    const float* parts[GS_MAX_KSPLIT];
    for (int r = 0; r < ksplit; ++r) parts[r] = cluster.map_shared_rank(&red[0][0][0][0], r);
    constexpr int PER_WARP = MT * GS_ROWS * 8;
    TOut* y = static_cast<TOut*>(a.y);
    if (SWIGLU) {
      // rows 0..7 are gate rows, rows 8..15 the matching up rows
      for (int e = threadIdx.x; e < MT * 8 * 8; e += GS_WARPS * 32) {
        const int mt = e / 64, r = (e / 8) % 8, tok = e % 8;
        float gate = 0.0f, up = 0.0f;
        for (int c = 0; c < ksplit; ++c)
#pragma unroll
          for (int w = 0; w < GS_WARPS; ++w) {
            gate += parts[c][w * PER_WARP + (mt * GS_ROWS + r) * 8 + tok];
            up += parts[c][w * PER_WARP + (mt * GS_ROWS + r + 8) * 8 + tok];
          }
        const int token = mt * 8 + tok, col = blockIdx.x * 8 + r;
        if (token < a.M && n0 + r + 8 < a.N)
          store_out<TOut>(y + static_cast<size_t>(token) * a.ldy + col, gate / (1.0f + expf(-gate)) * up);
      }
    } else {
      for (int e = threadIdx.x; e < PER_WARP; e += GS_WARPS * 32) {
        const int mt = e / (GS_ROWS * 8), r = (e / 8) % GS_ROWS, tok = e % 8;
        float sum = 0.0f;
        for (int c = 0; c < ksplit; ++c)
#pragma unroll
          for (int w = 0; w < GS_WARPS; ++w) sum += parts[c][w * PER_WARP + e];
        const int token = mt * 8 + tok;
        if (token < a.M && n0 + r < a.N) store_out<TOut>(y + static_cast<size_t>(token) * a.ldy + n0 + r, sum);
      }
    }
  }
  if (ksplit > 1) cluster.sync();           // nobody leaves while its shared memory may still be read
}

template <int MT, typename TOut, bool SWIGLU>
int small_gemm_launch(const SmallGemmArgs& a, int ksplit, cudaStream_t stream) {
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3((a.N + GS_ROWS - 1) / GS_ROWS, ksplit, 1);
  config.blockDim = dim3(GS_WARPS * 32, 1, 1);
  config.dynamicSmemBytes = 0;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeClusterDimension;
  attribute[0].val.clusterDim.x = 1;
  attribute[0].val.clusterDim.y = ksplit;
  attribute[0].val.clusterDim.z = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  if (cudaLaunchKernelEx(&config, gemm_small_kernel<MT, TOut, SWIGLU>, a) != cudaSuccess) return ERR_CUDA;
  return launch_result();
}

template <typename TOut, bool SWIGLU>
int small_gemm_dispatch(const SmallGemmArgs& a, int ksplit, cudaStream_t stream) {
  switch ((a.M + 7) / 8) {
    case 1: return small_gemm_launch<1, TOut, SWIGLU>(a, ksplit, stream);
    case 2: return small_gemm_launch<2, TOut, SWIGLU>(a, ksplit, stream);
    case 3: case 4: return small_gemm_launch<4, TOut, SWIGLU>(a, ksplit, stream);
    default: return small_gemm_launch<8, TOut, SWIGLU>(a, ksplit, stream);
  }
}

}  // namespace zb

using namespace zb;

// 1 if zb_gemm_small takes this problem.
ZB_API int zb_gemm_small_supported(int M, int N, int K) {
  return M >= 1 && M <= 8 * GS_MAX_MT && N >= 1 && K >= 8 && K % 8 == 0 ? 1 : 0;
}

// How many CTAs share the K dimension of one 16-row tile: enough for the grid to fill the GPU, a
// power of two up to 8, and no finer than one 32-wide block of k per warp.
ZB_API int zb_gemm_small_ksplit(int N, int K) {
  const int tiles = (N + GS_ROWS - 1) / GS_ROWS;
  const int blocks = (K + 31) / 32;
  int ksplit = 1;
  while (ksplit < GS_MAX_KSPLIT && tiles * ksplit < 592 && blocks >= GS_WARPS * ksplit * 2) ksplit *= 2;
  return ksplit;
}

// y = x w^T (swiglu = 0), or y[:, 8j + r] = silu(x w[16j + r]^T) * (x w[16j + 8 + r]^T) (swiglu = 1;
// w holds gate and up rows interleaved in blocks of 8, y has N / 2 columns).
// x: [M, K] bfloat16 rows ldx apart (ldx, ldw multiples of 8, pointers 16-byte aligned);
// out_dtype: bfloat16 or float32.
ZB_API int zb_gemm_small(void* y, const void* x, const void* w, int M, int N, int K, long long ldx, long long ldw,
                         long long ldy, int out_dtype, int swiglu, void* stream) {
  if (!zb_gemm_small_supported(M, N, K)) return ERR_UNSUPPORTED;
  if (ldx < K || ldw < K || ldx % 8 != 0 || ldw % 8 != 0 || reinterpret_cast<uintptr_t>(x) % 16 != 0 ||
      reinterpret_cast<uintptr_t>(w) % 16 != 0 || (swiglu && N % 16 != 0))
    return ERR_BAD_ARGUMENT;
  SmallGemmArgs a;
  a.y = y;
  a.x = static_cast<const __nv_bfloat16*>(x);
  a.w = static_cast<const __nv_bfloat16*>(w);
  a.M = M; a.N = N; a.K = K; a.ldx = ldx; a.ldw = ldw; a.ldy = ldy;
  const int ksplit = zb_gemm_small_ksplit(N, K);
  auto s = static_cast<cudaStream_t>(stream);
  if (swiglu)
    return out_dtype == DTYPE_F32 ? small_gemm_dispatch<float, true>(a, ksplit, s)
                                  : small_gemm_dispatch<__nv_bfloat16, true>(a, ksplit, s);
  return out_dtype == DTYPE_F32 ? small_gemm_dispatch<float, false>(a, ksplit, s)
                                : small_gemm_dispatch<__nv_bfloat16, false>(a, ksplit, s);
}
