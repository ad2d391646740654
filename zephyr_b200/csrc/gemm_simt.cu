// Y[M, N] = X[M, K] * W[N, K]^T on CUDA cores with float32 multiply-adds: the matrix product of
// the true 32-bit path.  No tensor cores, hence no TF32 or other reduced-precision mode: the
// reference's "float32" linear layers run in TF32 (deps/ttl/src/ops/matmul.cpp:269-271), which is
// exactly what this path exists to avoid.  Each output sums its K products in ascending order of
// 16-wide slices, independent of M and N, so a row's result does not depend on the batch around it.
// Inputs may be float32 or bfloat16 (read exactly); the output is float32 or the input type.
#include "common.cuh"

namespace zb {

constexpr int GT = 64;      // output tile edge
constexpr int GK = 16;      // K slice
constexpr int GPAD = 4;

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(256)
gemm_nt_simt_kernel(TOut* __restrict__ y, const TIn* __restrict__ x, const TIn* __restrict__ w, int M, int N, int K,
                    long long ldx, long long ldw, long long ldy) {
  __shared__ __align__(16) float xs[GK][GT + GPAD];
  __shared__ __align__(16) float ws[GK][GT + GPAD];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * GT, n0 = blockIdx.x * GT;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  const int lr = threadIdx.x >> 2;          // row of the tile this thread loads (0..63)
  const int lc = (threadIdx.x & 3) * 4;     // first of its 4 columns of the K slice
  for (int k0 = 0; k0 < K; k0 += GK) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int k = k0 + lc + u;
      const int m = m0 + lr, n = n0 + lr;
      xs[lc + u][lr] = (m < M && k < K) ? to_float(x[static_cast<size_t>(m) * ldx + k]) : 0.0f;
      ws[lc + u][lr] = (n < N && k < K) ? to_float(w[static_cast<size_t>(n) * ldw + k]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < GK; ++k) {
      const float4 a = *reinterpret_cast<const float4*>(&xs[k][ty * 4]);
      const float4 b = *reinterpret_cast<const float4*>(&ws[k][tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) y[static_cast<size_t>(m) * ldy + n] = from_float<TOut>(acc[i][j]);
    }
  }
}

template <typename TIn, typename TOut>
int gemm_launch(void* y, const void* x, const void* w, int M, int N, int K, long long ldx, long long ldw,
                long long ldy, cudaStream_t stream) {
  const dim3 grid((N + GT - 1) / GT, (M + GT - 1) / GT);
  if (grid.y > 65535) return ERR_UNSUPPORTED;
  gemm_nt_simt_kernel<TIn, TOut><<<grid, 256, 0, stream>>>((TOut*)y, (const TIn*)x, (const TIn*)w, M, N, K, ldx,
                                                           ldw, ldy);
  return launch_result();
}

}  // namespace zb

using namespace zb;

// y = x * w^T.  x: [M, K] rows ldx apart; w: [N, K] rows ldw apart; y: [M, N] rows ldy apart.
ZB_API int zb_gemm_nt_simt(void* y, const void* x, const void* w, int M, int N, int K, long long ldx, long long ldw,
                           long long ldy, int in_dtype, int out_dtype, void* stream) {
  if (M < 0 || N < 0 || K <= 0 || ldx < K || ldw < K || ldy < N) return ERR_BAD_ARGUMENT;
  if (M == 0 || N == 0) return OK;
  auto s = static_cast<cudaStream_t>(stream);
  if (in_dtype == DTYPE_F32 && out_dtype == DTYPE_F32)
    return gemm_launch<float, float>(y, x, w, M, N, K, ldx, ldw, ldy, s);
  if (in_dtype == DTYPE_BF16 && out_dtype == DTYPE_F32)
    return gemm_launch<__nv_bfloat16, float>(y, x, w, M, N, K, ldx, ldw, ldy, s);
  if (in_dtype == DTYPE_BF16 && out_dtype == DTYPE_BF16)
    return gemm_launch<__nv_bfloat16, __nv_bfloat16>(y, x, w, M, N, K, ldx, ldw, ldy, s);
  return ERR_BAD_ARGUMENT;
}
