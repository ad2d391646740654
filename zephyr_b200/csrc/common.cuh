// Shared helpers of the hand-written kernels: element types, conversions, reductions and the
// device status word.  Everything is compiled for sm_100a only.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace zb {

// dtype codes of the C interface.
constexpr int DTYPE_F32 = 0;
constexpr int DTYPE_BF16 = 1;

// Return codes of the C interface (0 = launched).
constexpr int OK = 0;
constexpr int ERR_BAD_ARGUMENT = 1;     // a size or flag outside what the kernel takes
constexpr int ERR_CUDA = 2;             // the launch itself failed; see zb_last_cuda_error
constexpr int ERR_UNSUPPORTED = 3;      // a valid configuration that this kernel refuses

// Codes a kernel leaves in the status word (status[0]); status[1] holds a detail value and
// status[2] the index of the offending element.  The first error wins; nothing traps.
constexpr int STATUS_OK = 0;
constexpr int STATUS_TOKEN_OUT_OF_RANGE = 1;
constexpr int STATUS_POSITION_OUT_OF_RANGE = 2;
constexpr int STATUS_PAGE_OUT_OF_RANGE = 3;
constexpr int STATUS_ROW_OUT_OF_RANGE = 4;
constexpr int STATUS_BAD_LOGIT = 5;
constexpr int STATUS_COPY_TIMEOUT = 6;    // an asynchronous copy did not complete within the wait limit
constexpr int STATUS_INTERNAL_CHECK = 7;  // a kernel's own check of an address or size failed
constexpr int STATUS_BARRIER_TIMEOUT = 8; // a barrier across the grid did not complete within the wait limit

__device__ __forceinline__ void report(int* status, int code, int detail, int index) {
  if (status != nullptr && atomicCAS(status, STATUS_OK, code) == STATUS_OK) {
    status[1] = detail;
    status[2] = index;
  }
}

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// A norm scale may be stored in either type, whatever the activations are.
__device__ __forceinline__ float load_scale(const void* w, int w_dtype, int i) {
  return w_dtype == DTYPE_F32 ? static_cast<const float*>(w)[i]
                              : __bfloat162float(static_cast<const __nv_bfloat16*>(w)[i]);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();                       // scratch may still be read from an earlier call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.0f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// ---- The cache's row layout ------------------------------------------------------------------------
// A cache row (the head_dim values of one position and head) is stored with its 16-byte chunks
// permuted: logical chunk c of the row at position `pos` lives at chunk c ^ kv_swizzle(pos, chunks).
// The permutation is chosen so that a page copied to shared memory as it is, rows back to back
// with no padding (one bulk copy), can be read by ldmatrix without bank conflicts: eight
// consecutive rows at the same logical chunk then fall into eight different 16-byte bank groups.
// `chunks` = row bytes / 16.  The permutation only swaps chunks inside aligned groups of 8, 4 or 2,
// so it stays inside the row for every head size that is a multiple of 16 bytes.
__host__ __device__ __forceinline__ int kv_swizzle(int pos, int chunks) {
  const int step = chunks & 7;                 // bank-group stride between consecutive rows
  if (step == 0) return pos & 7;
  if (step == 4) return (pos >> 1) & 3;
  if (step == 2 || step == 6) return (pos >> 2) & 1;
  return 0;                                    // odd strides are conflict-free as they are
}
// Index of logical element `i` of a row inside the stored row, for elements of `elem_bytes` bytes.
__host__ __device__ __forceinline__ int kv_element_index(int i, int pos, int head_dim, int elem_bytes) {
  const int per_chunk = 16 / elem_bytes;
  const int chunk = i / per_chunk;
  return ((chunk ^ kv_swizzle(pos, head_dim * elem_bytes / 16)) * per_chunk) + (i - chunk * per_chunk);
}

// What the CUDA runtime said when a call of this library last failed (zb_last_cuda_error hands it out).
inline const char*& last_cuda_error_text() {
  static const char* text = "no CUDA call of this library has failed";
  return text;
}
// True, with the runtime's words kept, if `e` is an error.
inline bool cuda_failed(cudaError_t e) {
  if (e == cudaSuccess) return false;
  last_cuda_error_text() = cudaGetErrorString(e);
  return true;
}

inline int launch_result() {
  return cuda_failed(cudaPeekAtLastError()) ? ERR_CUDA : OK;
}

// Programmatic dependent launch.  A kernel launched with `launch_dependent` may start while the
// kernel before it in the stream is still running: its CTAs take the SMs as they become free and
// do whatever does not read the earlier kernel's results (shared memory set-up, barriers, plans from
// the step's description, weights).  `wait_for_prior_grids` then blocks until every earlier kernel
// has completed and its writes are visible; nothing an earlier kernel wrote is read, and nothing it
// reads is written, before that.  `let_dependents_launch`, called after the wait, lets the next
// kernel start in the same way (called before the wait, the order of completion would no longer be
// a chain).  In a kernel launched the ordinary way both are no-ops.
__device__ __forceinline__ void wait_for_prior_grids() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void let_dependents_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// How many CTAs a persistent kernel of this library (the decode attention, the chain of small
// products) takes at most: 0 means one per SM.  Two halves of a batch that run side by side on two
// streams are given half the SMs each.
inline int& sm_share() {
  static int ctas = 0;
  return ctas;
}
inline int shared_sm_count(int sms) { return sm_share() > 0 && sm_share() < sms ? sm_share() : sms; }

inline bool& dependent_launch_enabled() {
  static bool enabled = true;
  return enabled;
}

template <typename... Params, typename... Args>
inline int launch_dependent(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                            bool cooperative, Args&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attributes[2];
  int n = 0;
  if (dependent_launch_enabled()) {
    attributes[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cooperative) {
    attributes[n].id = cudaLaunchAttributeCooperative;
    attributes[n].val.cooperative = 1;
    ++n;
  }
  config.attrs = attributes;
  config.numAttrs = n;
  return cuda_failed(cudaLaunchKernelEx(&config, kernel, Params(args)...)) ? ERR_CUDA : launch_result();
}

}  // namespace zb

#define ZB_API extern "C" __attribute__((visibility("default")))
