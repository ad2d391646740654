// Token selection from float32 logits: greedy (lowest index among equal maxima) and temperature
// sampling over the whole vocabulary.
//
// Definitions (reference): a temperature below 1e-7 means greedy (src/sampler/sampler.cpp:36,
// 316-324); argmax ties go to the lowest index (deps/ttl reduction_operations.cuh:108-131);
// z = (x - max) / T is formed in double and stored as float (src/sampler/sampler.cu:82-83);
// p = exp(z) (softmax with maximum 0); the inclusive prefix sums run in index order and the token is
// the first index with positive weight whose prefix sum exceeds min(u * total, the float below
// total), else the last index with positive weight (sampler.cu:150-167).  NaN or +inf in a row is
// reported in the status word (sampler.cu:77-80).
#include "common.cuh"

namespace zb {

constexpr int SAMPLE_THREADS = 1024;
constexpr float GREEDY_TEMPERATURE = 1e-7f;

struct MaxIdx { float v; int i; };

__device__ __forceinline__ MaxIdx better(MaxIdx a, MaxIdx b) {
  if (b.i >= 0 && (a.i < 0 || b.v > a.v || (b.v == a.v && b.i < a.i))) return b;
  return a;
}

__device__ MaxIdx block_argmax(MaxIdx mine, MaxIdx* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxIdx other{__shfl_xor_sync(0xffffffffu, mine.v, o), __shfl_xor_sync(0xffffffffu, mine.i, o)};
    mine = better(mine, other);
  }
  __syncthreads();
  if (lane == 0) scratch[warp] = mine;
  __syncthreads();
  if (warp == 0) {
    MaxIdx t = lane < nwarps ? scratch[lane] : MaxIdx{0.0f, -1};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      MaxIdx other{__shfl_xor_sync(0xffffffffu, t.v, o), __shfl_xor_sync(0xffffffffu, t.i, o)};
      t = better(t, other);
    }
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// One block per row.  temperature[r] < 1e-7: out[r] = argmax.  Otherwise sample with uniform[r] in [0, 1).
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(int* __restrict__ out, const float* __restrict__ logits, long long row_stride, int V,
              const float* __restrict__ temperature, const float* __restrict__ uniform, int* status) {
  __shared__ MaxIdx mscratch[33];
  __shared__ float fscratch[33];
  __shared__ float chunk_sum[SAMPLE_THREADS];
  __shared__ int found, last_positive;
  const int r = blockIdx.x;
  const float* x = logits + static_cast<size_t>(r) * row_stride;

  // Each thread owns a contiguous chunk, so that prefix sums follow index order.
  const int per = (V + blockDim.x - 1) / blockDim.x;
  const int begin = min(V, static_cast<int>(threadIdx.x) * per), end = min(V, begin + per);

  // The maximum does not care in which order the row is visited (equal maxima go to the lowest
  // index whatever the order), so this pass strides through the row with coalesced loads.
  MaxIdx mine{0.0f, -1};
  bool bad = false;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = x[i];
    if (isnan(v) || (isinf(v) && v > 0.0f)) bad = true;
    mine = better(mine, MaxIdx{v, i});
  }
  if (bad) report(status, STATUS_BAD_LOGIT, r, begin);
  const MaxIdx top = block_argmax(mine, mscratch);
  const float T = temperature != nullptr ? temperature[r] : 0.0f;
  if (T < GREEDY_TEMPERATURE || top.i < 0 || !isfinite(top.v)) {
    if (threadIdx.x == 0) out[r] = top.i < 0 ? 0 : top.i;
    return;
  }

  const double dmax = static_cast<double>(top.v), dT = static_cast<double>(T);
  float sum = 0.0f;
  for (int i = begin; i < end; ++i)
    sum += expf(static_cast<float>((static_cast<double>(x[i]) - dmax) / dT));
  chunk_sum[threadIdx.x] = sum;
  if (threadIdx.x == 0) { found = V; last_positive = -1; }
  __syncthreads();
  // Prefix of this thread's chunk: the chunk sums before it, added in index order by one warp in
  // a fixed pattern (each lane sums 32 consecutive chunks, then a serial pass over the 32 lanes).
  __shared__ float lane_prefix[33];
  if (threadIdx.x < 32) {
    float s = 0.0f;
    for (int k = 0; k < 32; ++k) s += chunk_sum[threadIdx.x * 32 + k];
    fscratch[threadIdx.x] = s;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.0f;
    for (int k = 0; k < 32; ++k) { lane_prefix[k] = s; s += fscratch[k]; }
    lane_prefix[32] = s;
  }
  __syncthreads();
  const float total = lane_prefix[32];
  float prefix = lane_prefix[threadIdx.x >> 5];
  for (int k = (threadIdx.x >> 5) * 32; k < static_cast<int>(threadIdx.x); ++k) prefix += chunk_sum[k];

  const float target = fminf(uniform[r] * total, nextafterf(total, 0.0f));
  float run = prefix;
  int my_found = V, my_last = -1;
  for (int i = begin; i < end; ++i) {
    const float p = expf(static_cast<float>((static_cast<double>(x[i]) - dmax) / dT));
    run += p;
    if (p > 0.0f) {
      my_last = i;
      if (my_found == V && run > target) my_found = i;
    }
  }
  if (my_found < V) atomicMin(&found, my_found);
  if (my_last >= 0) atomicMax(&last_positive, my_last);
  __syncthreads();
  if (threadIdx.x == 0) out[r] = found < V ? found : (last_positive >= 0 ? last_positive : top.i);
}

}  // namespace zb

using namespace zb;

// out[r] = selected token of row r.  `temperature` may be null (all rows greedy); `uniform` is read
// only for rows with temperature >= 1e-7.
ZB_API int zb_sample(int* out, const float* logits, long long row_stride, int rows, int V, const float* temperature,
                     const float* uniform, int* status, void* stream) {
  if (rows < 0 || V <= 0 || row_stride < V) return ERR_BAD_ARGUMENT;
  if (temperature != nullptr && uniform == nullptr) return ERR_BAD_ARGUMENT;
  if (rows == 0) return OK;
  sample_kernel<<<rows, SAMPLE_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(out, logits, row_stride, V,
                                                                                temperature, uniform, status);
  return launch_result();
}
