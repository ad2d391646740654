// Seeded normal values written straight into a tensor of the engine's type: the random-weights mode
// fills a model's tensors where they will be read, without a float32 copy of each (the largest
// benchmarked shape holds 65 GB of weights).
//
// The generator is counter-based (Philox 4x32 with 10 rounds; Salmon, Moraes, Dror, Shaw: "Parallel
// random numbers: as easy as 1, 2, 3", 2011): the four 32-bit words for elements 4 i .. 4 i + 3 are a
// function of the tensor's 64-bit key and the counter i alone, so a value does not depend on the
// grid, on the other tensors or on the order in which tensors are made.  Two words make two normal
// values by the Box-Muller transform: u1 in (0, 1] from the upper 24 bits (so the logarithm is
// finite), u2 in [0, 1).  The reference fills its random models the same way
// (deps/ttl/src/kernels/random/random.cu:83-125); keys, counters and the order of the values are this
// package's own.
#include "common.cuh"

namespace zb {

struct PhiloxWords {
  unsigned v[4];
};

__device__ __forceinline__ PhiloxWords philox_4x32_10(unsigned long long counter, unsigned long long key) {
  constexpr unsigned M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
  unsigned c0 = static_cast<unsigned>(counter), c1 = static_cast<unsigned>(counter >> 32), c2 = 0u, c3 = 0u;
  unsigned k0 = static_cast<unsigned>(key), k1 = static_cast<unsigned>(key >> 32);
#pragma unroll
  for (int round = 0; round < 10; ++round) {
    const unsigned hi0 = __umulhi(M0, c0), lo0 = M0 * c0;
    const unsigned hi1 = __umulhi(M1, c2), lo1 = M1 * c2;
    const unsigned n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += W0; k1 += W1;
  }
  return PhiloxWords{{c0, c1, c2, c3}};
}

__device__ __forceinline__ void box_muller(unsigned a, unsigned b, float& z0, float& z1) {
  const float u1 = static_cast<float>((a >> 8) + 1u) * (1.0f / 16777216.0f);      // (0, 1]
  const float u2 = static_cast<float>(b >> 8) * (1.0f / 16777216.0f);             // [0, 1)
  const float radius = sqrtf(-2.0f * logf(u1));
  float s, c;
  sincosf(6.2831853071795864769f * u2, &s, &c);
  z0 = radius * c;
  z1 = radius * s;
}

template <typename T>
__global__ void fill_normal_kernel(T* __restrict__ out, long long n, unsigned long long key, float mean, float std) {
  const long long quads = (n + 3) / 4;
  const long long step = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < quads; i += step) {
    const PhiloxWords w = philox_4x32_10(static_cast<unsigned long long>(i), key);
    float z[4];
    box_muller(w.v[0], w.v[1], z[0], z[1]);
    box_muller(w.v[2], w.v[3], z[2], z[3]);
#pragma unroll
    for (int e = 0; e < 4; ++e)
      if (4 * i + e < n) out[4 * i + e] = from_float<T>(fmaf(z[e], std, mean));
  }
}

}  // namespace zb

using namespace zb;

// out[i] = mean + std * z_i for i < n, z standard normal, a function of (key, i) only.
ZB_API int zb_fill_normal(void* out, long long n, unsigned long long key, float mean, float std, int dtype, void* stream) {
  if (n < 0 || (dtype != DTYPE_F32 && dtype != DTYPE_BF16)) return ERR_BAD_ARGUMENT;
  if (n == 0) return OK;
  const long long quads = (n + 3) / 4;
  const int blocks = static_cast<int>(quads + 255 < 256LL * 148 * 16 ? (quads + 255) / 256 : 148 * 16);
  const cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == DTYPE_F32) fill_normal_kernel<float><<<blocks, 256, 0, s>>>(static_cast<float*>(out), n, key, mean, std);
  else fill_normal_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(static_cast<__nv_bfloat16*>(out), n, key, mean, std);
  return launch_result();
}
