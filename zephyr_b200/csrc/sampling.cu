// Token selection from float32 logits: greedy, temperature, top-k, top-p and min-p sampling,
// penalties and biases from the request's history, and log-probability reports.
//
// Definitions (reference, src/sampler/sampler.cpp and src/sampler/sampler.cu):
//   * adjustments (sampler.cu:28-56): for a token of the history, score -= frequency_penalty * (times
//     generated) + presence_penalty if it was generated; score = score > 0 ? score / repetition_penalty
//     : score * repetition_penalty if it occurs anywhere in the history; then score += bias;
//   * a temperature below 1e-7 means greedy (sampler.cpp:36, 300-309): argmax, the lowest index among
//     equal maxima (deps/ttl reduction_operations.cuh:108-131);
//   * z = (x - max) / T in double, stored as float (sampler.cu:82-83), T = 1 for greedy rows;
//     p = softmax(z), here kept unnormalised as exp(z) (max z = 0): every rule below is a ratio;
//   * top-k or top-p rows rank the vocabulary by p, descending, equal values by ascending index
//     (deps/ttl/include/ttl/ops/topk.hpp:27-29); rank r stays if r < k, if the mass before r is
//     below top_p times the mass of the first k (the candidate that reaches the threshold stays; rank
//     0 always stays), and if p > min_p * max p (sampler.cu:99-118); the draw runs over the ranks;
//   * other rows draw over the vocabulary in index order (min-p applied in place);
//   * the draw (sampler.cu:150-167): inclusive prefix sums of the kept weights, the first candidate
//     with positive weight whose prefix sum exceeds min(u * total, the float below total), else the
//     last candidate with positive weight;
//   * reports (sampler.cu:178-194): log-softmax of z over the whole vocabulary, before any filter:
//     the chosen token's value and the top-n tokens ranked by z, descending, ties by index.
// NaN or +inf in a row, or a row without a finite maximum, is reported in the status word
// (sampler.cu:71-80).
//
// How it runs: passes over a row are spread over many CTAs (chunks of 4096 logits) and meet through
// small per-chunk partial results, merged in chunk order so that a row's result does not depend on
// the batch around it; the chunk that arrives last finishes the row's maximum.  Ranking runs in two
// steps.  The first ranks only the head of the order: a histogram of a sample of the row over the
// keys' leading 12 bits says which leading bins hold about 2048 tokens (one CTA per row), the pass
// that forms the weights (many CTAs per row) lists all tokens of those bins, and one CTA per row
// sorts the list in shared memory (if it has at most 4096 entries) and decides the row if the
// draw (or the report) can be decided within it, which it can whenever the distribution has a
// peak.  Rows that are not done go through a
// stable least-significant-digit radix sort of the whole vocabulary.  Both steps produce the same
// order and feed the same draw, whose sums run in blocks of 4096 ranks, so a rank's prefix sum does
// not depend on how many ranks were sorted.
#include "common.cuh"

namespace zb {

constexpr int SAMPLE_CHUNK = 4096;          // logits per CTA of the chunked passes
constexpr int CHUNK_THREADS = 256;
constexpr int ROW_THREADS = 1024;           // CTAs that own a whole row
constexpr double GREEDY_TEMPERATURE = 1e-7;
constexpr int SAMPLE_MAX_VOCAB = 1 << 22;
constexpr int SORT_UNROLL = 8;              // loads in flight per lane of the ranking kernel
constexpr int HEAD_BINS = 4096;             // the keys' leading 12 bits
constexpr int HEAD_MAX = 4096;              // tokens of the order's head, sorted in shared memory
constexpr int HEAD_AIM = 2048;              // tokens the head is meant to have when the vocabulary is larger

// One row's parameters, as the host packs them (64 bytes).
struct SampleRow {
  double temperature;          // below 1e-7: greedy
  double top_p;                // 0: off
  double min_p;                // 0: off
  float uniform;               // the row's draw in [0, 1)
  float frequency_penalty, presence_penalty, repetition_penalty;
  int top_k;                   // 0: off
  int num_logprobs;            // -1: no report; n >= 0: the chosen token's log-probability and the top n
  int result_offset;           // where the row's results start in the outputs
  int sort_slot;               // sort job that ranks this row by weight, or -1
  int report_slot;             // sort job that ranks this row by z, or -1
  int reserved;
};
static_assert(sizeof(SampleRow) == 64, "the host packs 64 bytes per row");

struct TokenAdjustment {       // 20 bytes
  int row, token, generated_count, seen;
  float bias;
};

struct SortJob {               // 8 bytes
  int row;
  int by_z;                    // 0: by weight, descending; 1: by z, descending
};

struct MaxIdx { float v; int i; };

__device__ __forceinline__ MaxIdx better(MaxIdx a, MaxIdx b) {
  if (b.i >= 0 && (a.i < 0 || b.v > a.v || (b.v == a.v && b.i < a.i))) return b;
  return a;
}

__device__ __forceinline__ MaxIdx warp_argmax(MaxIdx mine) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxIdx other{__shfl_xor_sync(0xffffffffu, mine.v, o), __shfl_xor_sync(0xffffffffu, mine.i, o)};
    mine = better(mine, other);
  }
  return mine;
}

__device__ MaxIdx block_argmax(MaxIdx mine, MaxIdx* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  mine = warp_argmax(mine);
  __syncthreads();
  if (lane == 0) scratch[warp] = mine;
  __syncthreads();
  if (warp == 0) {
    MaxIdx t = warp_argmax(lane < nwarps ? scratch[lane] : MaxIdx{0.0f, -1});
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// Exclusive prefix of `v` over the block's threads in thread order; `total` gets the block's sum.
// `scratch` holds 33 values.
template <typename T>
__device__ T block_exclusive_scan(T v, T* scratch, T& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  T inclusive = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const T below = __shfl_up_sync(0xffffffffu, inclusive, o);
    if (lane >= o) inclusive += below;
  }
  __syncthreads();
  if (lane == 31) scratch[warp] = inclusive;
  __syncthreads();
  if (warp == 0) {
    const T mine = lane < nwarps ? scratch[lane] : T(0);
    T run = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const T below = __shfl_up_sync(0xffffffffu, run, o);
      if (lane >= o) run += below;
    }
    scratch[lane] = run - mine;
    if (lane == 31) scratch[32] = run;
  }
  __syncthreads();
  total = scratch[32];
  return scratch[warp] + inclusive - v;
}

__device__ __forceinline__ bool is_greedy(const SampleRow* rows, int r) {
  return rows == nullptr || rows[r].temperature < GREEDY_TEMPERATURE;
}
__device__ __forceinline__ bool is_ranked(const SampleRow& p) {
  return p.temperature >= GREEDY_TEMPERATURE && (p.top_k > 0 || p.top_p > 0.0);
}
__device__ __forceinline__ float scaled(float x, float maximum, double temperature) {
  return static_cast<float>((static_cast<double>(x) - static_cast<double>(maximum)) / temperature);
}
__device__ __forceinline__ double scaling_temperature(const SampleRow& p) {
  return p.temperature < GREEDY_TEMPERATURE ? 1.0 : p.temperature;
}

// ---------------------------------------------------------------------------------- adjustments
__global__ void sample_adjust_kernel(float* __restrict__ logits, long long row_stride, int rows_n, int V,
                                     const SampleRow* __restrict__ rows, const TokenAdjustment* __restrict__ adjustments,
                                     int count, int* status) {
  for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < count; e += gridDim.x * blockDim.x) {
    const TokenAdjustment a = adjustments[e];
    if (a.row < 0 || a.row >= rows_n || a.token < 0 || a.token >= V) {
      report(status, STATUS_TOKEN_OUT_OF_RANGE, a.token, a.row);
      continue;
    }
    const SampleRow& row = rows[a.row];
    float* cell = logits + static_cast<size_t>(a.row) * row_stride + a.token;
    float score = *cell;
    if (a.generated_count > 0) {
      score -= row.frequency_penalty * static_cast<float>(a.generated_count);
      score -= row.presence_penalty;
    }
    if (a.seen && row.repetition_penalty != 1.0f)
      score = score > 0.0f ? score / row.repetition_penalty : score * row.repetition_penalty;
    score += a.bias;
    *cell = score;       // a NaN or +inf made here is found by the pass over the row that follows
  }
}

// ----------------------------------------------------------------------- maximum and argmax
// Grid (chunks, rows).  The last chunk of a row to finish merges the row's partial maxima.
__global__ void __launch_bounds__(CHUNK_THREADS)
sample_max_kernel(const float* __restrict__ logits, long long row_stride, int V, int chunks,
                  const SampleRow* __restrict__ rows, float* part_max, int* part_idx, int* counters,
                  float* row_max, int* row_arg, int* out_ids, int* status) {
  __shared__ MaxIdx scratch[33];
  __shared__ int last;
  const int c = blockIdx.x, r = blockIdx.y;
  const float* x = logits + static_cast<size_t>(r) * row_stride;
  const int begin = c * SAMPLE_CHUNK, end = min(V, begin + SAMPLE_CHUNK);
  MaxIdx mine{0.0f, -1};
  int bad = -1;
  for (int i = begin + threadIdx.x; i < end; i += CHUNK_THREADS) {
    const float v = x[i];
    if (isnan(v) || (isinf(v) && v > 0.0f)) bad = i;
    mine = better(mine, MaxIdx{v, i});
  }
  if (bad >= 0) report(status, STATUS_BAD_LOGIT, r, bad);
  const MaxIdx top = block_argmax(mine, scratch);
  if (threadIdx.x == 0) {
    part_max[r * chunks + c] = top.v;
    part_idx[r * chunks + c] = top.i;
    __threadfence();
    last = atomicAdd(&counters[r], 1) == chunks - 1;
  }
  __syncthreads();
  if (!last || threadIdx.x >= 32) return;
  __threadfence();
  MaxIdx t{0.0f, -1};
  for (int k = threadIdx.x; k < chunks; k += 32)
    t = better(t, MaxIdx{__ldcg(&part_max[r * chunks + k]), __ldcg(&part_idx[r * chunks + k])});
  t = warp_argmax(t);
  if (threadIdx.x == 0) {
    const bool usable = t.i >= 0 && isfinite(t.v);
    if (!usable) report(status, STATUS_BAD_LOGIT, r, t.i);
    row_max[r] = usable ? t.v : -INFINITY;        // -inf tells the later passes to leave the row alone
    row_arg[r] = t.i >= 0 ? t.i : 0;
    if (is_greedy(rows, r)) out_ids[rows != nullptr ? rows[r].result_offset : r] = t.i >= 0 ? t.i : 0;
    counters[r] = 0;                               // left as it was found, for the next call
  }
}

// ------------------------------------------------------------------------ weights and their sums
// Grid (chunks, rows).  weights[r][i] = exp(z_i), zero where min-p removes the token from a row
// that draws in index order.  part_all: the chunk's sum of exp(z); part_kept: of the weights.
// A warp's lanes that `take` get consecutive places in a job's list of candidates (one addition to
// the job's count for all of them) and leave their key and token there if the list has room.
__device__ __forceinline__ void add_candidates(bool take, unsigned key, int token, int* count, unsigned* keys, int* tokens,
                                               int room) {
  const unsigned takers = __ballot_sync(0xffffffffu, take);
  if (takers == 0) return;
  const int lane = threadIdx.x & 31, leader = __ffs(takers) - 1;
  int base = 0;
  if (lane == leader) base = atomicAdd(count, __popc(takers));
  base = __shfl_sync(0xffffffffu, base, leader);
  const int at = base + __popc(takers & ((1u << lane) - 1u));
  if (take && at < room) {
    keys[at] = key;
    tokens[at] = token;
  }
}

__global__ void __launch_bounds__(CHUNK_THREADS)
sample_exp_kernel(const float* __restrict__ logits, long long row_stride, int V, int chunks,
                  const SampleRow* __restrict__ rows, const float* __restrict__ row_max, float* __restrict__ weights,
                  float* part_all, float* part_kept, unsigned* sort_keys, int* sort_idx, int* job_state) {
  __shared__ float scratch_a[33], scratch_b[33];
  const int c = blockIdx.x, r = blockIdx.y;
  const SampleRow p = rows[r];
  const bool greedy = p.temperature < GREEDY_TEMPERATURE;
  if (greedy && p.num_logprobs < 0) return;
  const float maximum = row_max[r];
  if (!isfinite(maximum)) return;
  const double T = scaling_temperature(p);
  const bool filter = !greedy && !is_ranked(p) && p.min_p > 0.0;
  const float* x = logits + static_cast<size_t>(r) * row_stride;
  float* w = weights + static_cast<size_t>(r) * V;
  // Rows that are ranked (by weight for a draw, by z for a report) leave the tokens of the order's
  // head in their job's first buffers on the way: those whose key lies in the leading bins that
  // sample_head_bins_kernel chose.  The list is the head kernel's input.
  const int draw_job = !greedy && is_ranked(p) ? p.sort_slot : -1;
  const int report_job = p.num_logprobs > 0 ? p.report_slot : -1;
  const int room = min(HEAD_MAX, V);
  const unsigned draw_bins = draw_job >= 0 ? job_state[4 * draw_job + 2] : 0u;
  const unsigned report_bins = report_job >= 0 ? job_state[4 * report_job + 2] : 0u;
  const int begin = c * SAMPLE_CHUNK, end = min(V, begin + SAMPLE_CHUNK);
  float all = 0.0f, kept = 0.0f;
  for (int i0 = begin; i0 < end; i0 += CHUNK_THREADS) {          // whole warps stay in the loop
    const int i = i0 + threadIdx.x;
    const bool valid = i < end;
    const float z = valid ? scaled(x[i], maximum, T) : 0.0f;
    const float e = valid ? expf(z) : 0.0f;
    // The largest probability is exp(0) = 1 before normalisation.
    const float k = filter && !(static_cast<double>(e) > p.min_p) ? 0.0f : e;
    all += e;
    kept += k;
    if (valid && !greedy) w[i] = k;
    if (draw_bins)
      add_candidates(valid && (~__float_as_uint(k) >> 20) < draw_bins, ~__float_as_uint(k), i, &job_state[4 * draw_job + 3],
                     sort_keys + static_cast<size_t>(draw_job) * 2 * V, sort_idx + static_cast<size_t>(draw_job) * 2 * V, room);
    if (report_bins)
      add_candidates(valid && (__float_as_uint(fabsf(z)) >> 20) < report_bins, __float_as_uint(fabsf(z)), i,
                     &job_state[4 * report_job + 3], sort_keys + static_cast<size_t>(report_job) * 2 * V,
                     sort_idx + static_cast<size_t>(report_job) * 2 * V, room);
  }
  all = block_sum(all, scratch_a);
  kept = block_sum(kept, scratch_b);
  if (threadIdx.x == 0) {
    part_all[r * chunks + c] = all;
    part_kept[r * chunks + c] = kept;
  }
}

// ------------------------------------------------------------------- the draw in index order
// One CTA per row.  The chunk sums locate the chunk in which the prefix sum crosses the target; the
// CTA then scans that chunk.
__global__ void __launch_bounds__(ROW_THREADS)
sample_select_kernel(const float* __restrict__ weights, int V, int chunks, const SampleRow* __restrict__ rows,
                     const float* __restrict__ part_kept, const float* __restrict__ row_max,
                     const int* __restrict__ row_arg, int* out_ids) {
  __shared__ float scratch[33];
  __shared__ float s_base, s_target;
  __shared__ int s_chunk, s_exact, s_first, s_last;
  const int r = blockIdx.x;
  const SampleRow p = rows[r];
  if (p.temperature < GREEDY_TEMPERATURE || is_ranked(p)) return;
  if (!isfinite(row_max[r])) {
    if (threadIdx.x == 0) out_ids[p.result_offset] = row_arg[r];
    return;
  }
  if (threadIdx.x == 0) {
    const float* sums = part_kept + r * chunks;
    float total = 0.0f;
    for (int c = 0; c < chunks; ++c) total += sums[c];
    const float target = fminf(p.uniform * total, nextafterf(total, 0.0f));
    float run = 0.0f, base = 0.0f;
    int chosen = -1, last_positive = -1;
    for (int c = 0; c < chunks; ++c) {
      const float s = sums[c];
      if (s > 0.0f) {
        last_positive = c;
        if (chosen < 0 && run + s > target) { chosen = c; base = run; }
      }
      run += s;
    }
    s_exact = chosen >= 0;
    s_chunk = chosen >= 0 ? chosen : last_positive;
    s_base = base;
    s_target = target;
    s_first = V;
    s_last = -1;
  }
  __syncthreads();
  if (s_chunk < 0) {            // no weight at all: cannot happen for a finite maximum; stay defined
    if (threadIdx.x == 0) out_ids[p.result_offset] = row_arg[r];
    return;
  }
  constexpr int PER = SAMPLE_CHUNK / ROW_THREADS;
  const float* w = weights + static_cast<size_t>(r) * V;
  const int begin = s_chunk * SAMPLE_CHUNK + threadIdx.x * PER;
  float mine[PER], local = 0.0f;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    mine[j] = begin + j < V ? w[begin + j] : 0.0f;
    local += mine[j];
  }
  float total;
  float run = s_base + block_exclusive_scan(local, scratch, total);
  int first = V, last = -1;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    run += mine[j];
    if (mine[j] > 0.0f) {
      last = begin + j;
      if (first == V && s_exact && run > s_target) first = begin + j;
    }
  }
  if (first < V) atomicMin(&s_first, first);
  if (last >= 0) atomicMax(&s_last, last);
  __syncthreads();
  if (threadIdx.x == 0) out_ids[p.result_offset] = s_first < V ? s_first : (s_last >= 0 ? s_last : row_arg[r]);
}

// ------------------------------------------------------------------------------------- ranking
// One CTA per job: a stable radix sort of a row's keys, 8 bits a pass, between the job's two
// buffers; the result lies in the second buffer.  Each warp owns a contiguous stretch of the input,
// counts its digits, and after a scan over (digit, warp) scatters its stretch in order, so equal
// keys keep their index order.
__device__ __forceinline__ unsigned sort_key(const SortJob& job, int i, const float* x, const float* w, float maximum,
                                             double T) {
  // Ascending keys: weights descending (the bit pattern of a non-negative float grows with it),
  // or |z| ascending, which is z descending because z <= 0.
  return job.by_z ? __float_as_uint(fabsf(scaled(x[i], maximum, T))) : ~__float_as_uint(w[i]);
}

// Lanes of the warp whose 8-bit digit equals this lane's (lanes with `valid` false match nobody):
// eight ballots, one per bit, where a single match instruction walks the distinct values one by one.
__device__ __forceinline__ unsigned lanes_with_same_digit(unsigned digit, bool valid) {
  unsigned peers = __ballot_sync(0xffffffffu, valid);
#pragma unroll
  for (int bit = 0; bit < 8; ++bit) {
    const unsigned set = __ballot_sync(0xffffffffu, (digit >> bit) & 1u);
    peers &= (digit >> bit) & 1u ? set : ~set;
  }
  return valid ? peers : 0u;
}

__global__ void __launch_bounds__(ROW_THREADS)
sample_sort_kernel(const SortJob* __restrict__ jobs, const float* __restrict__ logits, long long row_stride, int V,
                   const SampleRow* __restrict__ rows, const float* __restrict__ row_max,
                   const float* __restrict__ weights, unsigned* keys, int* idx, int* job_state) {
  __shared__ int hist[256 * 32];
  __shared__ int scratch[33];
  const SortJob job = jobs[blockIdx.x];
  const int r = job.row;
  const float maximum = row_max[r];
  if (!isfinite(maximum)) return;
  if (job_state[4 * blockIdx.x + 1]) return;        // decided within the head of the order
  const double T = scaling_temperature(rows[r]);
  const float* x = logits + static_cast<size_t>(r) * row_stride;
  const float* w = weights + static_cast<size_t>(r) * V;
  unsigned* key_buf[2] = {keys + static_cast<size_t>(blockIdx.x) * 2 * V, keys + (static_cast<size_t>(blockIdx.x) * 2 + 1) * V};
  int* idx_buf[2] = {idx + static_cast<size_t>(blockIdx.x) * 2 * V, idx + (static_cast<size_t>(blockIdx.x) * 2 + 1) * V};
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per_warp = ((V + 31) / 32 + 31) / 32 * 32;
  const int w_begin = min(V, warp * per_warp), w_end = min(V, w_begin + per_warp);
  const unsigned lanes_below = (1u << lane) - 1u;

  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 8 * pass;
    const unsigned* src_key = pass == 0 ? nullptr : key_buf[(pass - 1) & 1];
    const int* src_idx = pass == 0 ? nullptr : idx_buf[(pass - 1) & 1];
    unsigned* dst_key = key_buf[pass & 1];
    int* dst_idx = idx_buf[pass & 1];
    for (int e = threadIdx.x; e < 256 * 32; e += ROW_THREADS) hist[e] = 0;
    __syncthreads();
    // Loads run SORT_UNROLL steps ahead of their use: a step's work is short, a load's latency is not.
    for (int i = w_begin; i < w_end; i += 32 * SORT_UNROLL) {
      unsigned key[SORT_UNROLL];
#pragma unroll
      for (int u = 0; u < SORT_UNROLL; ++u) {
        const int e = i + u * 32 + lane;
        key[u] = e >= w_end ? 0u : (pass == 0 ? sort_key(job, e, x, w, maximum, T) : src_key[e]);
      }
#pragma unroll
      for (int u = 0; u < SORT_UNROLL; ++u) {
        const bool valid = i + u * 32 + lane < w_end;
        const unsigned digit = (key[u] >> shift) & 255u;
        const unsigned peers = lanes_with_same_digit(digit, valid);
        if (valid && (peers & lanes_below) == 0) hist[digit * 32 + warp] += __popc(peers);
        __syncwarp();
      }
    }
    __syncthreads();
    {   // exclusive scan over the 8192 counters in (digit, warp) order
      constexpr int PER = 256 * 32 / ROW_THREADS;
      int mine[PER], local = 0;
#pragma unroll
      for (int j = 0; j < PER; ++j) { mine[j] = hist[threadIdx.x * PER + j]; local += mine[j]; }
      int total;
      int run = block_exclusive_scan(local, scratch, total);
#pragma unroll
      for (int j = 0; j < PER; ++j) { hist[threadIdx.x * PER + j] = run; run += mine[j]; }
    }
    __syncthreads();
    for (int i = w_begin; i < w_end; i += 32 * SORT_UNROLL) {
      unsigned key[SORT_UNROLL];
      int source[SORT_UNROLL];
#pragma unroll
      for (int u = 0; u < SORT_UNROLL; ++u) {
        const int e = i + u * 32 + lane;
        key[u] = e >= w_end ? 0u : (pass == 0 ? sort_key(job, e, x, w, maximum, T) : src_key[e]);
        source[u] = e >= w_end ? 0 : (pass == 0 ? e : src_idx[e]);
      }
#pragma unroll
      for (int u = 0; u < SORT_UNROLL; ++u) {
        const bool valid = i + u * 32 + lane < w_end;
        const unsigned digit = (key[u] >> shift) & 255u;
        const unsigned peers = lanes_with_same_digit(digit, valid);
        if (valid) {
          const int at = hist[digit * 32 + warp] + __popc(peers & lanes_below);
          dst_key[at] = key[u];
          dst_idx[at] = source[u];
        }
        __syncwarp();
        if (valid && (peers & lanes_below) == 0) hist[digit * 32 + warp] += __popc(peers);
        __syncwarp();
      }
    }
    __syncthreads();            // this pass's stores are visible to the whole CTA before the next reads them
  }
  if (threadIdx.x == 0) job_state[4 * blockIdx.x] = V;
}

// ---------------------------------------------------------------------- the draw over the ranks
constexpr int RANK_BLOCK = 4096;            // ranks per round of the draw's sums: four per thread
constexpr int RANK_PER = RANK_BLOCK / ROW_THREADS;

struct RankScratch {
  float scan[33];
  float carry, total;
  int cut, first, last;
};

// The draw of one ranked row by the whole CTA.  `sorted`/`source`: the first `n_sorted` ranks (keys
// are the inverted bit patterns of the weights).  Returns the chosen token, or -1 if the decision
// needs ranks beyond `n_sorted`.  The ranks that stay form a prefix of the order: the limits on the
// rank, on the mass before a rank and on the weight all cut a tail off.  Prefix sums run in rounds of
// RANK_BLOCK ranks (a block scan plus the carry of the rounds before), so the sum at a rank is the
// same whatever `n_sorted` is.
__device__ int ranked_draw(const SampleRow& p, const unsigned* sorted, const int* source, int n_sorted, int V,
                           float total_all, RankScratch& sh) {
  const int k = p.top_k > 0 ? min(p.top_k, V) : V;
  const int seen = min(k, n_sorted);
  if (seen <= 0) return -1;
  auto weight = [&](int i) { return __uint_as_float(~sorted[i]); };
  const int mine = static_cast<int>(threadIdx.x) * RANK_PER;

  // Inclusive prefix sums of the round starting at `begin`, over ranks below `limit`; `start` is the
  // sum before this thread's first rank.
  auto round_sums = [&](int begin, int limit, float (&w)[RANK_PER], float (&prefix)[RANK_PER], float& start) {
    float local = 0.0f;
#pragma unroll
    for (int j = 0; j < RANK_PER; ++j) {
      const int i = begin + mine + j;
      w[j] = i < limit ? weight(i) : 0.0f;
      local += w[j];
    }
    float total;
    start = sh.carry + block_exclusive_scan(local, sh.scan, total);
    float run = start;
#pragma unroll
    for (int j = 0; j < RANK_PER; ++j) { run += w[j]; prefix[j] = run; }
    return total;
  };
  // Between rounds: the carry moves on after every thread has used it.
  auto next_round = [&](float total) {
    __syncthreads();
    if (threadIdx.x == 0) sh.carry += total;
    __syncthreads();
  };

  // The mass of the first k ranks, which the top-p threshold is a share of.
  float mass = total_all;
  if (p.top_p > 0.0 && k < V) {
    if (k > n_sorted) return -1;
    __syncthreads();
    if (threadIdx.x == 0) sh.carry = 0.0f;
    __syncthreads();
    for (int begin = 0; begin < k; begin += RANK_BLOCK) {
      float w[RANK_PER], prefix[RANK_PER], start;
      const float total = round_sums(begin, k, w, prefix, start);
#pragma unroll
      for (int j = 0; j < RANK_PER; ++j)
        if (begin + mine + j == k - 1) sh.total = prefix[j];
      next_round(total);
    }
    mass = sh.total;
  }
  const float largest = weight(0);
  const double threshold = p.top_p * static_cast<double>(mass);

  // How many ranks stay, and their mass.
  __syncthreads();
  if (threadIdx.x == 0) { sh.carry = 0.0f; sh.cut = seen; sh.total = 0.0f; }
  __syncthreads();
  for (int begin = 0; begin < seen; begin += RANK_BLOCK) {
    float w[RANK_PER], prefix[RANK_PER], start;
    const float total = round_sums(begin, seen, w, prefix, start);
    int cut = seen;
#pragma unroll
    for (int j = RANK_PER - 1; j >= 0; --j) {
      const int i = begin + mine + j;
      if (i >= seen) continue;
      const float before = j == 0 ? start : prefix[j - 1];
      bool stays = true;
      if (p.top_p > 0.0 && i > 0 && !(static_cast<double>(before) < threshold)) stays = false;
      if (p.min_p > 0.0 && !(static_cast<double>(w[j]) > p.min_p * static_cast<double>(largest))) stays = false;
      if (!stays) cut = i;
    }
    if (cut < seen) atomicMin(&sh.cut, cut);
    __syncthreads();
    const int end = min(seen, begin + RANK_BLOCK);
    const int keep_here = min(sh.cut, end);          // the ranks of this round that stay end here
#pragma unroll
    for (int j = 0; j < RANK_PER; ++j)
      if (begin + mine + j == keep_here - 1) sh.total = prefix[j];
    next_round(total);
    if (sh.cut < end) break;
  }
  const int kept = sh.cut;
  if (kept == seen && seen < k) return -1;           // the ranks that stay may go on beyond the sorted ones
  if (kept == 0) return source[0];                   // cannot happen: rank 0 always stays
  const float total_kept = sh.total;
  const float target = fminf(p.uniform * total_kept, nextafterf(total_kept, 0.0f));

  // The first rank with positive weight whose prefix sum exceeds the target, else the last positive one.
  __syncthreads();
  if (threadIdx.x == 0) { sh.carry = 0.0f; sh.first = kept; sh.last = -1; }
  __syncthreads();
  for (int begin = 0; begin < kept; begin += RANK_BLOCK) {
    float w[RANK_PER], prefix[RANK_PER], start;
    const float total = round_sums(begin, kept, w, prefix, start);
    int first = kept, last = -1;
#pragma unroll
    for (int j = 0; j < RANK_PER; ++j) {
      const int i = begin + mine + j;
      if (i < kept && w[j] > 0.0f) {
        last = i;
        if (first == kept && prefix[j] > target) first = i;
      }
    }
    if (first < kept) atomicMin(&sh.first, first);
    if (last >= 0) atomicMax(&sh.last, last);
    next_round(total);
    if (sh.first < kept) break;
  }
  const int rank = sh.first < kept ? sh.first : sh.last;
  return rank >= 0 ? source[rank] : -2;
}

__device__ float chunk_total(const float* part, int r, int chunks) {
  float total = 0.0f;
  for (int c = 0; c < chunks; ++c) total += part[r * chunks + c];
  return total;
}

// ------------------------------------------------------------------- ranking the head of the order

// A job's four words of state: [0] how many ranks lie sorted in the job's second buffer, [1] 1 if the
// row needs no more than those, [2] the leading bins of the keys' first 12 bits that make the head of
// the order (0: no head), [3] how many tokens lie in those bins.
//
// One CTA per job, before the weights are formed.  Where the head ends is guessed from every
// `stride`-th token: the leading bins that hold HEAD_AIM / stride of them hold about HEAD_AIM tokens
// of the whole row.  The guess only decides how many ranks the head has (none, if more than
// HEAD_MAX tokens lie in those bins after all); the head is always every token of the leading
// bins, so it is the true start of the order.  The pass over the whole row that finds those tokens
// is the one that forms the weights (sample_exp_kernel, many CTAs a row): a single CTA walking the
// row twice took 100 us.
__global__ void __launch_bounds__(ROW_THREADS)
sample_head_bins_kernel(const SortJob* __restrict__ jobs, const float* __restrict__ logits, long long row_stride, int V,
                        const SampleRow* __restrict__ rows, const float* __restrict__ row_max, int* job_state) {
  __shared__ int hist[HEAD_BINS];
  __shared__ int scratch[33];
  __shared__ int s_bins;
  const SortJob job = jobs[blockIdx.x];
  const int r = job.row;
  const float maximum = row_max[r];
  int* state = job_state + 4 * blockIdx.x;
  if (threadIdx.x == 0) state[0] = state[1] = state[2] = state[3] = 0;
  if (!isfinite(maximum)) return;
  const int stride = (V + HEAD_MAX - 1) / HEAD_MAX;
  if (stride == 1) {                 // the whole row fits into the head
    if (threadIdx.x == 0) state[2] = HEAD_BINS;
    return;
  }
  const double T = scaling_temperature(rows[r]);
  const float* x = logits + static_cast<size_t>(r) * row_stride;
  // A row that needs few ranks (a small top-k, a report of a few tokens) aims at a shorter head:
  // half as many keys to sort, and still four times what it needs with room for the guess's error.
  const int needs = job.by_z ? rows[r].num_logprobs : rows[r].top_k;
  const int aim = needs > 0 && needs <= HEAD_AIM / 8 ? HEAD_AIM / 2 : HEAD_AIM;
  for (int e = threadIdx.x; e < HEAD_BINS; e += ROW_THREADS) hist[e] = 0;
  if (threadIdx.x == 0) s_bins = 0;
  __syncthreads();
  for (int i = threadIdx.x * stride; i < V; i += ROW_THREADS * stride) {
    const float z = scaled(x[i], maximum, T);
    const unsigned key = job.by_z ? __float_as_uint(fabsf(z)) : ~__float_as_uint(expf(z));
    atomicAdd(&hist[key >> 20], 1);
  }
  __syncthreads();
  constexpr int PER = HEAD_BINS / ROW_THREADS;
  int counts[PER], local = 0;
#pragma unroll
  for (int j = 0; j < PER; ++j) { counts[j] = hist[threadIdx.x * PER + j]; local += counts[j]; }
  int total;
  int run = block_exclusive_scan(local, scratch, total);
  int leading = 0;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    run += counts[j];
    if (run * stride <= aim) leading = threadIdx.x * PER + j + 1;
  }
  if (leading > 0) atomicMax(&s_bins, leading);
  __syncthreads();
  if (threadIdx.x == 0) state[2] = s_bins;
}

// One CTA per job, after the weights: sorts the head's tokens and decides the row if they are enough.
__global__ void __launch_bounds__(ROW_THREADS)
sample_rank_head_kernel(const SortJob* __restrict__ jobs, int V, int chunks, const SampleRow* __restrict__ rows,
                        const float* __restrict__ row_max, const float* __restrict__ part_all, unsigned* keys, int* idx,
                        const int* __restrict__ row_arg, int* job_state, int* out_ids) {
  __shared__ unsigned long long candidates[HEAD_MAX];
  __shared__ RankScratch sh;
  const SortJob job = jobs[blockIdx.x];
  const int r = job.row;
  const SampleRow p = rows[r];
  int* state = job_state + 4 * blockIdx.x;
  const int n = state[3];
  if (!isfinite(row_max[r]) || state[2] == 0 || n == 0 || n > min(HEAD_MAX, V)) return;      // no head, or more than fits
  int padded = 1;
  while (padded < n) padded <<= 1;
  const unsigned* found_keys = keys + static_cast<size_t>(blockIdx.x) * 2 * V;
  const int* found_tokens = idx + static_cast<size_t>(blockIdx.x) * 2 * V;
  for (int e = threadIdx.x; e < padded; e += ROW_THREADS)
    candidates[e] = e < n ? (static_cast<unsigned long long>(found_keys[e]) << 32) | static_cast<unsigned>(found_tokens[e]) : ~0ull;
  __syncthreads();
  // Bitonic sort, ascending: by key, equal keys by index.
  for (int size = 2; size <= padded; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = threadIdx.x; t < padded / 2; t += ROW_THREADS) {
        const int low = 2 * t - (t & (stride - 1)), high = low + stride;
        const bool ascending = (low & size) == 0;
        const unsigned long long a = candidates[low], b = candidates[high];
        if ((a > b) == ascending) { candidates[low] = b; candidates[high] = a; }
      }
      __syncthreads();
    }
  }
  unsigned* sorted = keys + (static_cast<size_t>(blockIdx.x) * 2 + 1) * V;
  int* source = idx + (static_cast<size_t>(blockIdx.x) * 2 + 1) * V;
  for (int e = threadIdx.x; e < n; e += ROW_THREADS) {
    sorted[e] = static_cast<unsigned>(candidates[e] >> 32);
    source[e] = static_cast<int>(candidates[e] & 0xffffffffu);
  }
  __syncthreads();
  if (threadIdx.x == 0) state[0] = n;
  if (job.by_z) {
    if (threadIdx.x == 0) state[1] = n >= min(p.num_logprobs, V);
    return;
  }
  const int token = ranked_draw(p, sorted, source, n, V, chunk_total(part_all, r, chunks), sh);
  if (threadIdx.x == 0 && token != -1) {
    out_ids[p.result_offset] = token >= 0 ? token : row_arg[r];
    state[1] = 1;
  }
}

// One CTA per row: the draw of the rows whose whole vocabulary had to be ranked.
__global__ void __launch_bounds__(ROW_THREADS)
sample_select_sorted_kernel(int V, int chunks, const SampleRow* __restrict__ rows, const unsigned* __restrict__ keys,
                            const int* __restrict__ idx, const float* __restrict__ row_max,
                            const int* __restrict__ row_arg, const float* __restrict__ part_all,
                            const int* __restrict__ job_state, int* out_ids) {
  __shared__ RankScratch sh;
  const int r = blockIdx.x;
  const SampleRow p = rows[r];
  if (!is_ranked(p) || p.sort_slot < 0) return;
  if (!isfinite(row_max[r])) {
    if (threadIdx.x == 0) out_ids[p.result_offset] = row_arg[r];
    return;
  }
  if (job_state[4 * p.sort_slot + 1]) return;
  const unsigned* sorted = keys + (static_cast<size_t>(p.sort_slot) * 2 + 1) * V;
  const int* source = idx + (static_cast<size_t>(p.sort_slot) * 2 + 1) * V;
  const int token = ranked_draw(p, sorted, source, job_state[4 * p.sort_slot], V, chunk_total(part_all, r, chunks), sh);
  if (threadIdx.x == 0) out_ids[p.result_offset] = token >= 0 ? token : row_arg[r];
}

// ---------------------------------------------------------------------------------- reports
// One CTA per row: log-probabilities of the chosen token and of the row's top tokens.
__global__ void __launch_bounds__(CHUNK_THREADS)
sample_report_kernel(const float* __restrict__ logits, long long row_stride, int V, int chunks,
                     const SampleRow* __restrict__ rows, const float* __restrict__ row_max,
                     const float* __restrict__ part_all, const int* __restrict__ idx, int* out_ids,
                     float* out_logprobs) {
  __shared__ float s_log_total;
  const int r = blockIdx.x;
  const SampleRow p = rows[r];
  if (p.num_logprobs < 0) return;
  const float maximum = row_max[r];
  const bool usable = isfinite(maximum);
  if (threadIdx.x == 0) {
    float total = 0.0f;
    for (int c = 0; c < chunks && usable; ++c) total += part_all[r * chunks + c];
    s_log_total = usable ? logf(total) : 0.0f;
  }
  __syncthreads();
  const double T = scaling_temperature(p);
  const float* x = logits + static_cast<size_t>(r) * row_stride;
  if (threadIdx.x == 0) {
    const int token = out_ids[p.result_offset];
    out_logprobs[p.result_offset] = usable && token >= 0 && token < V ? scaled(x[token], maximum, T) - s_log_total : 0.0f;
  }
  if (p.num_logprobs == 0 || p.report_slot < 0) return;
  const int* ranked = idx + (static_cast<size_t>(p.report_slot) * 2 + 1) * V;
  for (int rank = threadIdx.x; rank < p.num_logprobs && rank < V; rank += CHUNK_THREADS) {
    const int token = usable ? ranked[rank] : rank;
    out_ids[p.result_offset + 1 + rank] = token;
    out_logprobs[p.result_offset + 1 + rank] = usable ? scaled(x[token], maximum, T) - s_log_total : 0.0f;
  }
}

}  // namespace zb

using namespace zb;

// Chunks a row of V logits is cut into; the partial-result buffers hold rows * chunks entries.
ZB_API int zb_sample_chunks(int V) { return (V + SAMPLE_CHUNK - 1) / SAMPLE_CHUNK; }

// Phases of zb_sample beyond adjustments, maximum and sorting, which follow from the arguments.
constexpr int PHASE_WEIGHTS = 1;        // some row draws or reports
constexpr int PHASE_DRAW_INDEXED = 2;   // some row draws in index order
constexpr int PHASE_DRAW_RANKED = 4;    // some row draws over ranks
constexpr int PHASE_REPORT = 8;         // some row reports log-probabilities

// Selects one token per row of `logits` [rows, V] (float32, rows `row_stride` apart; adjusted in
// place when there are adjustments).
//   row_params   null: every row greedy, out_ids[r] = argmax of row r.  Else one SampleRow per row; a row's
//                results start at its result_offset: the chosen token, then its top tokens if it reports.
//   out_logprobs parallel to out_ids, written for reporting rows only; may be null without PHASE_REPORT.
//   jobs         the rows to rank, by weight (draws with top-k or top-p) or by z (reports with n > 0);
//                sort_keys and sort_idx hold 2 * n_jobs * V entries each, job_state 4 * n_jobs ints.
//   part_f       3 * rows * chunks floats; part_i rows * chunks ints; counters: rows ints, zero on entry and
//                on exit; row_max, row_arg: rows entries; weights: rows * V floats (unused without PHASE_WEIGHTS).
ZB_API int zb_sample(int* out_ids, float* out_logprobs, float* logits, long long row_stride, int rows, int V,
                     const void* row_params, const void* adjustments, int n_adjustments, const void* jobs, int n_jobs,
                     int phases, float* part_f, int* part_i, int* counters, float* row_max, int* row_arg,
                     float* weights, unsigned* sort_keys, int* sort_idx, int* job_state, int* status, void* stream) {
  if (rows < 0 || V <= 0 || row_stride < V || n_adjustments < 0 || n_jobs < 0) return ERR_BAD_ARGUMENT;
  if (V > SAMPLE_MAX_VOCAB || rows > 65535) return ERR_UNSUPPORTED;
  if (rows == 0) return OK;
  if (row_params == nullptr && (phases != 0 || n_adjustments > 0 || n_jobs > 0)) return ERR_BAD_ARGUMENT;
  if ((phases & PHASE_REPORT) && out_logprobs == nullptr) return ERR_BAD_ARGUMENT;
  if (phases != 0 && weights == nullptr) return ERR_BAD_ARGUMENT;
  if (n_jobs > 0 && (sort_keys == nullptr || sort_idx == nullptr || jobs == nullptr || job_state == nullptr))
    return ERR_BAD_ARGUMENT;
  auto s = static_cast<cudaStream_t>(stream);
  const auto* params = static_cast<const SampleRow*>(row_params);
  const int chunks = zb_sample_chunks(V);
  float* part_max = part_f;
  float* part_all = part_f + static_cast<size_t>(rows) * chunks;
  float* part_kept = part_all + static_cast<size_t>(rows) * chunks;
  const dim3 chunk_grid(chunks, rows);
  if (n_adjustments > 0)
    sample_adjust_kernel<<<(n_adjustments + 255) / 256, 256, 0, s>>>(
        logits, row_stride, rows, V, params, static_cast<const TokenAdjustment*>(adjustments), n_adjustments, status);
  sample_max_kernel<<<chunk_grid, CHUNK_THREADS, 0, s>>>(logits, row_stride, V, chunks, params, part_max, part_i,
                                                        counters, row_max, row_arg, out_ids, status);
  if (n_jobs > 0)
    sample_head_bins_kernel<<<n_jobs, ROW_THREADS, 0, s>>>(static_cast<const SortJob*>(jobs), logits, row_stride, V, params,
                                                          row_max, job_state);
  if (phases & PHASE_WEIGHTS)
    sample_exp_kernel<<<chunk_grid, CHUNK_THREADS, 0, s>>>(logits, row_stride, V, chunks, params, row_max, weights,
                                                          part_all, part_kept, sort_keys, sort_idx, job_state);
  if (n_jobs > 0) {
    sample_rank_head_kernel<<<n_jobs, ROW_THREADS, 0, s>>>(static_cast<const SortJob*>(jobs), V, chunks, params, row_max,
                                                          part_all, sort_keys, sort_idx, row_arg, job_state, out_ids);
    sample_sort_kernel<<<n_jobs, ROW_THREADS, 0, s>>>(static_cast<const SortJob*>(jobs), logits, row_stride, V, params,
                                                     row_max, weights, sort_keys, sort_idx, job_state);
  }
  if (phases & PHASE_DRAW_INDEXED)
    sample_select_kernel<<<rows, ROW_THREADS, 0, s>>>(weights, V, chunks, params, part_kept, row_max, row_arg, out_ids);
  if (phases & PHASE_DRAW_RANKED)
    sample_select_sorted_kernel<<<rows, ROW_THREADS, 0, s>>>(V, chunks, params, sort_keys, sort_idx, row_max, row_arg,
                                                            part_all, job_state, out_ids);
  if (phases & PHASE_REPORT)
    sample_report_kernel<<<rows, CHUNK_THREADS, 0, s>>>(logits, row_stride, V, chunks, params, row_max, part_all,
                                                       sort_idx, out_ids, out_logprobs);
  return launch_result();
}
