// A chain of small matrix products in one launch, for steps with few tokens (M <= 16).
//
// A decode step of a few tokens spends most of a layer's time between its kernels: each small
// product waits for the one before, starts cold, and reads its weights at a fraction of what the
// memory system gives.  Here one cooperative launch runs a whole list of stages
//
//     y_s = epilogue_s( prologue_s(...) W_s^T ),        s = 0 .. n - 1,
//
// over all SMs, one persistent CTA per SM:
//   * a producer warp streams the CTA's share of every stage's weights, in stage order, through a
//     ring of shared-memory slots with the TMA engine: one tiled copy (cp.async.bulk.tensor over a
//     three-dimensional view of the matrix, 128-byte swizzle) brings 8 rows by 1024 columns, 16 KB,
//     per instruction; matrices whose width is no multiple of 64 go row by row with the untiled
//     form (cp.async.bulk).  Completion is counted on an mbarrier per slot.  Weights depend on nothing, so the copies of later stages are in
//     flight while earlier stages compute and while the CTAs wait for each other: the launch reads
//     the chain's weights as one stream;
//   * eight consumer warps form the products on tensor cores (m16n8k16, float32 accumulators; for
//     up to 8 tokens two tiles of 8 weight rows on the 16-row side and the tokens on the other, for
//     more the tokens on the 16-row side and one tile on the other: warp-level products run at a
//     fraction of the tensor cores' rate on this GPU, and a stage of a wide model spends as long on
//     them as on its weights' way from memory, so none should be spent on rows that do not exist).  The stage's input, a few rows, lies
//     in shared memory.  A CTA owns whole rows of W_s over the full K, so no sum crosses CTAs; its
//     warps split K and add their parts in warp order, so every result is a fixed-order sum;
//   * stages are separated by a barrier across the grid (an arrival counter in global memory; the
//     launch is cooperative, so all CTAs are resident).  Every wait is bounded and reports instead
//     of hanging.
// Prologues: the input as given; or rmsnorm(residual) * w; or residual + delta (rounded and
// written to a second residual buffer), then rmsnorm of it.  Each CTA forms the few normalised
// rows for itself.  Epilogues: none, or silu(gate) * up over weight rows laid out as blocks of 8
// gate rows followed by their 8 up rows.
// Math: as the separate kernels (rmsnorm_kernel, gemm_small_kernel): sums, norms and the
// activation in float32, one rounding to bfloat16 where a tensor is stored
// (reference: src/model/causal_lm/qwen3.cpp:17-88, src/layer/mlp.cpp:16-36,
// src/layer/normalization.cpp:10-18).
#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"
#include "mma.cuh"
#include "tma.cuh"

namespace zb {

constexpr int CH_CONSUMERS = 8;
constexpr int CH_THREADS = (CH_CONSUMERS + 1) * 32;    // the last warp is the producer
constexpr int CH_KC = 1024;                            // k per ring slot
constexpr int CH_PAD = 64;        // row strides of 64 mod 128 bytes keep the 16-byte fragment loads free of bank conflicts
constexpr int CH_ROW_BYTES = CH_KC * 2 + CH_PAD;
constexpr int CH_TILED_BYTES = 8 * CH_KC * 2;          // a slot filled by one tiled copy: 8 rows of 16 segments of 128 bytes
constexpr int CH_SLOT_BYTES = (8 * CH_ROW_BYTES + 1023) / 1024 * 1024;   // room for either form, 1024-byte aligned
constexpr int CH_MAX_STAGES = 8;
constexpr int CH_MAX_TOKENS = 16;
constexpr int CH_WAIT_LIMIT = 1 << 22;
constexpr int CH_SMEM_BUDGET = 227 * 1024 - 1024;
constexpr int CH_MIN_SLOTS = 4;
constexpr int CH_GROUP_TILES = 8;                     // tiles whose sums a warp keeps in registers at a time

constexpr int PROLOGUE_NONE = 0, PROLOGUE_NORM = 1, PROLOGUE_ADD_NORM = 2;
constexpr int EPILOGUE_NONE = 0, EPILOGUE_SWIGLU = 1;

struct ChainStage {
  const __nv_bfloat16* w;            // [N, K], rows ldw apart
  long long ldw;
  int N, K;
  int prologue, epilogue;
  const __nv_bfloat16* x;            // PROLOGUE_NONE: [M, K], rows ldx apart
  long long ldx;
  const __nv_bfloat16* residual_in;  // PROLOGUE_NORM, PROLOGUE_ADD_NORM: [M, K] contiguous
  __nv_bfloat16* residual_out;       // PROLOGUE_ADD_NORM: [M, K] contiguous, not residual_in
  const __nv_bfloat16* delta;        // PROLOGUE_ADD_NORM: [M, K], rows ldd apart
  long long ldd;
  const void* norm_w;                // [K]
  int norm_w_dtype;
  float eps;
  __nv_bfloat16* y;                  // [M, N], or [M, N / 2] after EPILOGUE_SWIGLU; rows ldy apart
  long long ldy;
};

struct ChainArgs {
  CUtensorMap map[CH_MAX_STAGES];    // the stage's weights as [N][K / 64][64], for stages with tiled != 0
  int tiled[CH_MAX_STAGES];
  ChainStage stage[CH_MAX_STAGES];
  int n_stages, M, ring_shift, xs_row_bytes;      // the ring holds 1 << ring_shift slots
  __nv_bfloat16* xn;                 // null, or room for 16 rows of the longest normalised input: where long rows are
                                     // normalised once for all CTAs
  int* sync;                         // [0] barrier arrivals, [1] CTAs done; zero on entry and on exit
  int* status;
  int* trace;                        // null, or [CTA][stage][4] ints: the global timer (ns, low 32 bits) at the stage's
                                     // start, after its input is in place, after its products, after the barrier
};

struct StagePlan { int tiles_per_block, b0, b1, chunks; };

__device__ __forceinline__ StagePlan plan_stage(const ChainStage& st, int cta, int ctas) {
  StagePlan p;
  p.tiles_per_block = st.epilogue == EPILOGUE_SWIGLU ? 2 : 1;
  const long long blocks = st.N / (8 * p.tiles_per_block);
  p.b0 = static_cast<int>(blocks * cta / ctas);
  p.b1 = static_cast<int>(blocks * (cta + 1) / ctas);
  p.chunks = (st.K + CH_KC - 1) / CH_KC;
  return p;
}

__device__ __forceinline__ void chain_consumer_barrier() {
  asm volatile("bar.sync 1, %0;\n" ::"n"(CH_CONSUMERS * 32) : "memory");
}
__device__ __forceinline__ void chain_mbar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ uint4 lds128(unsigned address) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(address));
  return v;
}
__device__ __forceinline__ int load_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// One tiled copy: the box [8 rows][16 segments][64 columns] at (row, segment) into a slot.
__device__ __forceinline__ void tiled_copy_g2s(void* smem_dst, const CUtensorMap* map, int row, int segment,
                                               unsigned long long* bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n"
               ::"r"(smem_u32(smem_dst)), "l"(map), "r"(0), "r"(segment), "r"(row), "r"(smem_u32(bar)) : "memory");
}

// HI: more than 8 tokens, so the second half of the 16 token rows is in use.  FLIP (up to 8 tokens
// only): the weights take the tensor cores' 16-row side, two tiles at a time.
template <bool HI, bool FLIP>
__global__ void __launch_bounds__(CH_THREADS, 1)
fused_chain_kernel(const __grid_constant__ ChainArgs a) {
  static_assert(!(HI && FLIP), "the tokens fit the 8-column side only up to 8");
  extern __shared__ unsigned char smem_unaligned[];
  // Swizzled tiles want 1024-byte alignment.
  unsigned char* smem_raw = smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u);
  const int R = 1 << a.ring_shift;
  unsigned char* ring = smem_raw;                                              // [R][CH_SLOT_BYTES]
  unsigned char* xs = ring + static_cast<size_t>(R) * CH_SLOT_BYTES;            // [8 or 16][xs_row_bytes]: the stage's input
  unsigned long long* full = reinterpret_cast<unsigned long long*>(xs + static_cast<size_t>(HI ? 16 : 8) * a.xs_row_bytes);
  unsigned long long* empty = full + R;
  unsigned long long* xfull = empty + R;
  float* red = reinterpret_cast<float*>(xfull + 1);     // [warps][CH_GROUP_TILES][8 or 16][8]: the warps' parts of the sums
  __shared__ volatile int abort_flag;
  __shared__ StagePlan plans[CH_MAX_STAGES];      // divisions are slow where every instruction's latency shows

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x, ctas = gridDim.x;
  if (threadIdx.x >= 32 && threadIdx.x < 32 + a.n_stages) plans[threadIdx.x - 32] = plan_stage(a.stage[threadIdx.x - 32], cta, ctas);
  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < R; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], CH_CONSUMERS); }
    mbar_init(xfull, 1);
    fence_barrier_init();
  }
  __syncthreads();
  fence_proxy_async();
  auto wait = [&](unsigned long long* bar, unsigned parity) -> bool {
    if (mbar_try_wait(bar, parity)) return true;
    for (int i = 0; i < CH_WAIT_LIMIT; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
      if ((i & 63) == 63 && abort_flag) return false;
    }
    return false;
  };

  if (warp == CH_CONSUMERS) {
    // ------------------------------------------------------------------------- the producer
    // Units in the order group of blocks, chunk of K, block, tile; unit number `seq` lives in slot seq mod R.
    if (lane != 0) return;
    int seq = 0;
    for (int s = 0; s < a.n_stages; ++s) {
      const ChainStage& st = a.stage[s];
      const StagePlan p = plans[s];
      const bool tiled = a.tiled[s] != 0;
      const int group_blocks = CH_GROUP_TILES / p.tiles_per_block;
      for (int gb = p.b0; gb < p.b1; gb += group_blocks)
        for (int c = 0; c < p.chunks; ++c)
          for (int u = 0; u < CH_GROUP_TILES; ++u) {
            const int b = gb + u / p.tiles_per_block, t = u % p.tiles_per_block;
            if (b >= p.b1 || b >= gb + group_blocks) break;
            const int slot = seq & (R - 1);
            if (!wait(&empty[slot], ((seq >> a.ring_shift) & 1) ^ 1)) {
              report(a.status, STATUS_COPY_TIMEOUT, -10 - s, cta);
              abort_flag = 1;
              return;
            }
            ++seq;
            unsigned char* dst = ring + static_cast<size_t>(slot) * CH_SLOT_BYTES;
            const int row0 = (b * p.tiles_per_block + t) * 8;
            if (tiled) {
              // One instruction for the whole slot; columns past K are filled with zeros.
              mbar_arrive_expect_tx(&full[slot], CH_TILED_BYTES);
              tiled_copy_g2s(dst, &a.map[s], row0, c * (CH_KC / 64), &full[slot]);
            } else {
              const unsigned bytes = static_cast<unsigned>(min(CH_KC, st.K - c * CH_KC)) * 2u;
              mbar_arrive_expect_tx(&full[slot], 8u * bytes);
              for (int r = 0; r < 8; ++r)
                bulk_copy_g2s(dst + r * CH_ROW_BYTES, st.w + static_cast<long long>(row0 + r) * st.ldw + static_cast<long long>(c) * CH_KC,
                              bytes, &full[slot]);
            }
          }
    }
    return;
  }

  // ---------------------------------------------------------------------------- the consumers
  const int ctid = threadIdx.x;                   // 0 .. 32 * CH_CONSUMERS - 1
  const int g = lane >> 2, t4 = lane & 3;
  const int M = a.M;
  const unsigned ring_s = smem_u32(ring);
  const unsigned xs_lo = smem_u32(xs) + g * a.xs_row_bytes + t4 * 16, xs_hi = xs_lo + 8 * a.xs_row_bytes;
  const bool lo_ok = g < M, hi_ok = HI && g + 8 < M;
  constexpr int RM = HI ? 16 : 8;     // token rows kept
  int seq = 0, barriers = 0, x_uses = 0;
  const bool tracing = a.trace != nullptr && ctid == 0;
  int* const trace = a.trace + static_cast<size_t>(cta) * 4 * a.n_stages;
  auto now = [] {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return static_cast<int>(t);
  };
  // A warp whose wait runs out reports, raises the abort flag and walks on without waiting or
  // computing: the barriers among the consumers need every warp to the very end.
  bool failed = false;
  // The producer is already streaming weights, which no kernel writes; the inputs, the residual and
  // the barrier's counters are earlier kernels' business until this returns.
  wait_for_prior_grids();
  let_dependents_launch();
  // The barrier across the grid.  The CTA's barrier orders its threads' stores before thread 0,
  // whose arrival is a release at device scope; its polls are acquires, and the CTA's second
  // barrier hands what they saw on to the other threads.
  auto grid_barrier = [&](int where) {
    ++barriers;
    chain_consumer_barrier();
    if (ctid == 0) {
      asm volatile("red.release.gpu.global.add.s32 [%0], 1;\n" ::"l"(&a.sync[0]) : "memory");
      const int target = barriers * ctas;
      bool ok = !abort_flag;
      for (int polls = 0; ok && load_acquire(&a.sync[0]) < target; ++polls)
        if (polls > CH_WAIT_LIMIT || ((polls & 63) == 63 && (abort_flag || *reinterpret_cast<volatile int*>(a.status) != 0)))
          ok = false;
      if (!ok) {
        report(a.status, STATUS_BARRIER_TIMEOUT, where, cta);
        abort_flag = 1;
      }
    }
    chain_consumer_barrier();
    failed = failed || abort_flag != 0;
  };
  // The stage's input as it lies in global memory: one bulk copy per token row.
  auto fetch_rows = [&](const __nv_bfloat16* src, long long ld, int K, int s) {
    if (ctid < M) {
      fence_proxy_async();
      bulk_copy_g2s(xs + static_cast<size_t>(ctid) * a.xs_row_bytes, src + static_cast<size_t>(ctid) * ld,
                    static_cast<unsigned>(K) * 2u, xfull);
    }
    if (ctid == 0) mbar_arrive_expect_tx(xfull, static_cast<unsigned>(M) * static_cast<unsigned>(K) * 2u);
    if (!failed && !wait(xfull, x_uses & 1)) {
      if (lane == 0 && !abort_flag) report(a.status, STATUS_COPY_TIMEOUT, -20 - s, cta);
      abort_flag = 1;
      failed = true;
    }
    ++x_uses;
  };
  for (int s = 0; s < a.n_stages; ++s) {
    const ChainStage& st = a.stage[s];
    const StagePlan p = plans[s];
    const int K = st.K;
    if (tracing) trace[4 * s] = now();

    // ---- the stage's input, [M, K] bfloat16 in shared memory
    if (st.prologue == PROLOGUE_NONE) {
      fetch_rows(st.x, st.ldx, K, s);
    } else if (K > 4 * 256 && a.xn != nullptr) {
      // A long row is normalised once, by the CTA of its number with all its warps, and fetched
      // by everybody after one more barrier across the grid: 148 CTAs each normalising all rows of
      // 4096 took 10 us a stage (the same 128 KB asked of the L2 by every SM, four rounds of it).
      if (cta < M) {
        const int m = cta;
        const __nv_bfloat16* res = st.residual_in + static_cast<size_t>(m) * K;
        const __nv_bfloat16* del = st.prologue == PROLOGUE_ADD_NORM ? st.delta + static_cast<size_t>(m) * st.ldd : nullptr;
        __nv_bfloat16* staged = reinterpret_cast<__nv_bfloat16*>(xs + static_cast<size_t>(m) * a.xs_row_bytes);
        float ss = 0.0f;
        for (int i = ctid * 8; i < K; i += CH_CONSUMERS * 32 * 8) {
          uint4 rv = __ldcg(reinterpret_cast<const uint4*>(res + i));
          __nv_bfloat162* r2 = reinterpret_cast<__nv_bfloat162*>(&rv);
          if (del != nullptr) {
            const uint4 dv = __ldcg(reinterpret_cast<const uint4*>(del + i));
            const __nv_bfloat162* d2 = reinterpret_cast<const __nv_bfloat162*>(&dv);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 rf = __bfloat1622float2(r2[e]), df = __bfloat1622float2(d2[e]);
              r2[e] = __floats2bfloat162_rn(rf.x + df.x, rf.y + df.y);
            }
            *reinterpret_cast<uint4*>(st.residual_out + static_cast<size_t>(m) * K + i) = rv;
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 rf = __bfloat1622float2(r2[e]);
            ss += rf.x * rf.x + rf.y * rf.y;
          }
          *reinterpret_cast<uint4*>(staged + i) = rv;
        }
        ss = warp_sum(ss);
        if (lane == 0) red[warp] = ss;
        chain_consumer_barrier();
        float total = 0.0f;
#pragma unroll
        for (int w = 0; w < CH_CONSUMERS; ++w) total += red[w];
        const float inv = rsqrtf(total / static_cast<float>(K) + st.eps);
        for (int i = ctid * 8; i < K; i += CH_CONSUMERS * 32 * 8) {       // each thread meets its own elements again
          uint4 rv = *reinterpret_cast<const uint4*>(staged + i);
          __nv_bfloat162* r2 = reinterpret_cast<__nv_bfloat162*>(&rv);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 rf = __bfloat1622float2(r2[e]);
            r2[e] = __floats2bfloat162_rn(rf.x * inv * load_scale(st.norm_w, st.norm_w_dtype, i + 2 * e),
                                          rf.y * inv * load_scale(st.norm_w, st.norm_w_dtype, i + 2 * e + 1));
          }
          *reinterpret_cast<uint4*>(a.xn + static_cast<size_t>(m) * K + i) = rv;
        }
        fence_proxy_async();        // the row's place in shared memory is about to be filled by a bulk copy
      }
      grid_barrier(-30 - s);
      fetch_rows(a.xn, K, K, s);
    } else {
      // Normalised rows, each warp its own: the (new) residual goes to shared memory as it is and is
      // scaled in place once the row's sum of squares is known.  All of a row's loads are in flight
      // together, four 16-byte pieces of each operand per lane and round.
      for (int m = warp; m < M; m += CH_CONSUMERS) {
        const __nv_bfloat16* res = st.residual_in + static_cast<size_t>(m) * K;
        const __nv_bfloat16* del = st.prologue == PROLOGUE_ADD_NORM ? st.delta + static_cast<size_t>(m) * st.ldd : nullptr;
        __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(xs + static_cast<size_t>(m) * a.xs_row_bytes);
        float ss = 0.0f;
        const bool wide = st.norm_w_dtype == DTYPE_F32;
        const float* w32 = static_cast<const float*>(st.norm_w);
        const __nv_bfloat16* w16 = static_cast<const __nv_bfloat16*>(st.norm_w);
        if (K <= 4 * 256 && !wide) {
          // The usual case (a bfloat16 scale, a row of at most four pieces per lane): everything the
          // row needs, the scale included, is asked for at once.
          uint4 rv[4], dv[4], sv[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int i = lane * 8 + j * 256;
            if (i < K) {
              rv[j] = __ldcg(reinterpret_cast<const uint4*>(res + i));
              if (del != nullptr) dv[j] = __ldcg(reinterpret_cast<const uint4*>(del + i));
              sv[j] = *reinterpret_cast<const uint4*>(w16 + i);
            }
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int i = lane * 8 + j * 256;
            if (i >= K) break;
            __nv_bfloat162* r2 = reinterpret_cast<__nv_bfloat162*>(&rv[j]);
            if (del != nullptr) {
              const __nv_bfloat162* d2 = reinterpret_cast<const __nv_bfloat162*>(&dv[j]);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 rf = __bfloat1622float2(r2[e]), df = __bfloat1622float2(d2[e]);
                r2[e] = __floats2bfloat162_rn(rf.x + df.x, rf.y + df.y);
              }
              if (cta == 0) *reinterpret_cast<uint4*>(st.residual_out + static_cast<size_t>(m) * K + i) = rv[j];
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 rf = __bfloat1622float2(r2[e]);
              ss += rf.x * rf.x + rf.y * rf.y;
            }
          }
          ss = warp_sum(ss);
          const float inv = rsqrtf(ss / static_cast<float>(K) + st.eps);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int i = lane * 8 + j * 256;
            if (i >= K) break;
            __nv_bfloat162* r2 = reinterpret_cast<__nv_bfloat162*>(&rv[j]);
            const __nv_bfloat162* s16 = reinterpret_cast<const __nv_bfloat162*>(&sv[j]);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 rf = __bfloat1622float2(r2[e]);
              const float2 sf = __bfloat1622float2(s16[e]);
              r2[e] = __floats2bfloat162_rn(rf.x * inv * sf.x, rf.y * inv * sf.y);
            }
            *reinterpret_cast<uint4*>(out + i) = rv[j];
          }
          continue;
        }
        for (int i0 = lane * 8; i0 < K; i0 += 4 * 256) {
          uint4 rv[4], dv[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int i = i0 + j * 256;
            if (i < K) {
              rv[j] = __ldcg(reinterpret_cast<const uint4*>(res + i));
              if (del != nullptr) dv[j] = __ldcg(reinterpret_cast<const uint4*>(del + i));
            }
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int i = i0 + j * 256;
            if (i >= K) break;
            __nv_bfloat162* r2 = reinterpret_cast<__nv_bfloat162*>(&rv[j]);
            if (del != nullptr) {
              const __nv_bfloat162* d2 = reinterpret_cast<const __nv_bfloat162*>(&dv[j]);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 rf = __bfloat1622float2(r2[e]), df = __bfloat1622float2(d2[e]);
                r2[e] = __floats2bfloat162_rn(rf.x + df.x, rf.y + df.y);
              }
              if (cta == 0) *reinterpret_cast<uint4*>(st.residual_out + static_cast<size_t>(m) * K + i) = rv[j];
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 rf = __bfloat1622float2(r2[e]);
              ss += rf.x * rf.x + rf.y * rf.y;
            }
            *reinterpret_cast<uint4*>(out + i) = rv[j];
          }
        }
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / static_cast<float>(K) + st.eps);
        __syncwarp();
        for (int i = lane * 8; i < K; i += 32 * 8) {
          float scale[8];
          if (wide) {
            const float4 lo = *reinterpret_cast<const float4*>(w32 + i);
            const float4 hi = *reinterpret_cast<const float4*>(w32 + i + 4);
            scale[0] = lo.x; scale[1] = lo.y; scale[2] = lo.z; scale[3] = lo.w;
            scale[4] = hi.x; scale[5] = hi.y; scale[6] = hi.z; scale[7] = hi.w;
          } else {
            const uint4 wv = *reinterpret_cast<const uint4*>(w16 + i);
            const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 wf = __bfloat1622float2(w2[e]);
              scale[2 * e] = wf.x;
              scale[2 * e + 1] = wf.y;
            }
          }
          uint4 rv = *reinterpret_cast<const uint4*>(out + i);
          __nv_bfloat162* r2 = reinterpret_cast<__nv_bfloat162*>(&rv);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 rf = __bfloat1622float2(r2[e]);
            r2[e] = __floats2bfloat162_rn(rf.x * inv * scale[2 * e], rf.y * inv * scale[2 * e + 1]);
          }
          *reinterpret_cast<uint4*>(out + i) = rv;
        }
      }
    }
    chain_consumer_barrier();
    if (tracing) trace[4 * s + 1] = now();

    // ---- the products.  The CTA's blocks are taken in groups of up to 8 tiles.  Every warp works
    // on every slot: of a slot's 32 k-blocks it takes four (warp, warp + 8, ...), so the input's
    // fragments are read once per chunk of K and serve all tiles of the group.  Each warp keeps its
    // part of every tile's sum in registers; the parts meet once per group, in warp order.
    const bool tiled = a.tiled[s] != 0;
    const int T = p.tiles_per_block, group_blocks = CH_GROUP_TILES / T;
    unsigned w_at[4], x_at[4];           // byte offsets of this lane's four pieces in a slot and in an input row
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int kb = warp + j * CH_CONSUMERS;
      // Tiled: rows of 2048 bytes in segments of 128 whose 16-byte chunks are permuted with the
      // segment's number (the 128-byte swizzle works on address bits 7..9).
      w_at[j] = tiled ? g * (CH_KC * 2) + (kb >> 1) * 128 + (((((kb & 1) << 2) + t4) ^ ((kb >> 1) & 7)) << 4)
                      : g * CH_ROW_BYTES + kb * 64 + t4 * 16;
      x_at[j] = kb * 64;
    }
    for (int gb = p.b0; gb < p.b1; gb += group_blocks) {
      const int n_tiles = min(group_blocks, p.b1 - gb) * T;
      float acc[CH_GROUP_TILES][4];           // [tile][fragment]
#pragma unroll
      for (int u = 0; u < CH_GROUP_TILES; ++u) acc[u][0] = acc[u][1] = acc[u][2] = acc[u][3] = 0.0f;
      for (int c = 0; c < p.chunks; ++c) {
        const int klen = min(CH_KC, K - c * CH_KC);
        const unsigned x_chunk = static_cast<unsigned>(c) * CH_KC * 2;
        bool ok[4];
        uint4 xl[4], xh[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          ok[j] = (warp + j * CH_CONSUMERS) * 32 + 8 * t4 + 8 <= klen;
          xl[j] = ok[j] && lo_ok ? lds128(xs_lo + x_chunk + x_at[j]) : make_uint4(0, 0, 0, 0);
          xh[j] = ok[j] && hi_ok ? lds128(xs_hi + x_chunk + x_at[j]) : make_uint4(0, 0, 0, 0);
        }
        if (!FLIP) {
#pragma unroll
          for (int u = 0; u < CH_GROUP_TILES; ++u) {
            if (u >= n_tiles) break;
            const int slot = seq & (R - 1);
            const unsigned parity = (seq >> a.ring_shift) & 1;
            ++seq;
            if (failed) continue;
            if (!wait(&full[slot], parity)) {
              if (lane == 0 && !abort_flag) report(a.status, STATUS_COPY_TIMEOUT, s, cta);
              abort_flag = 1;
              failed = true;
              continue;
            }
            const unsigned wslot = ring_s + static_cast<unsigned>(slot) * CH_SLOT_BYTES;
            uint4 wv[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[j] = ok[j] ? lds128(wslot + w_at[j]) : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const unsigned a0[4] = {xl[j].x, xh[j].x, xl[j].y, xh[j].y};
              const unsigned a1[4] = {xl[j].z, xh[j].z, xl[j].w, xh[j].w};
              mma_bf16_16816(acc[u], a0, wv[j].x, wv[j].y);
              mma_bf16_16816(acc[u], a1, wv[j].z, wv[j].w);
            }
            __syncwarp();
            if (lane == 0) chain_mbar_arrive(&empty[slot]);
          }
        } else {
          // Up to 8 tokens: the weights take the 16-row side, two tiles at a time (the lane's row of
          // either), and the tokens the 8-column side, so no half of a product is wasted on rows of
          // tokens that do not exist.  acc[u / 2] then holds, for lane (g, t4), weight row g of tile u
          // (elements 0, 1) and of tile u + 1 (elements 2, 3) at tokens 2 t4 and 2 t4 + 1.
#pragma unroll
          for (int u = 0; u < CH_GROUP_TILES; u += 2) {
            if (u >= n_tiles) break;
            const bool pair = u + 1 < n_tiles;
            const int slot0 = seq & (R - 1), slot1 = (seq + 1) & (R - 1);
            const unsigned parity0 = (seq >> a.ring_shift) & 1, parity1 = ((seq + 1) >> a.ring_shift) & 1;
            seq += pair ? 2 : 1;
            if (failed) continue;
            if (!wait(&full[slot0], parity0) || (pair && !wait(&full[slot1], parity1))) {
              if (lane == 0 && !abort_flag) report(a.status, STATUS_COPY_TIMEOUT, s, cta);
              abort_flag = 1;
              failed = true;
              continue;
            }
            const unsigned w0 = ring_s + static_cast<unsigned>(slot0) * CH_SLOT_BYTES;
            const unsigned w1 = ring_s + static_cast<unsigned>(slot1) * CH_SLOT_BYTES;
            uint4 wl[4], wh[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              wl[j] = ok[j] ? lds128(w0 + w_at[j]) : make_uint4(0, 0, 0, 0);
              wh[j] = ok[j] && pair ? lds128(w1 + w_at[j]) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const unsigned a0[4] = {wl[j].x, wh[j].x, wl[j].y, wh[j].y};
              const unsigned a1[4] = {wl[j].z, wh[j].z, wl[j].w, wh[j].w};
              mma_bf16_16816(acc[u >> 1], a0, xl[j].x, xl[j].y);
              mma_bf16_16816(acc[u >> 1], a1, xl[j].z, xl[j].w);
            }
            __syncwarp();
            if (lane == 0) {
              chain_mbar_arrive(&empty[slot0]);
              if (pair) chain_mbar_arrive(&empty[slot1]);
            }
          }
        }
      }
      // The warps' parts go to shared memory as [tile][token][weight row].  More than 8 tokens: lane
      // (g, t4) holds tokens g and g + 8 at weight rows 2 t4 and 2 t4 + 1 of each tile.
#pragma unroll
      for (int u = 0; u < CH_GROUP_TILES; ++u) {
        if (u >= n_tiles) break;
        float* dst = red + ((warp * CH_GROUP_TILES + u) * RM) * 8;
        if (!FLIP) {
          *reinterpret_cast<float2*>(dst + g * 8 + 2 * t4) = make_float2(acc[u][0], acc[u][1]);
          if (HI) *reinterpret_cast<float2*>(dst + (g + 8) * 8 + 2 * t4) = make_float2(acc[u][2], acc[u][3]);
        } else {
          dst[(2 * t4) * 8 + g] = acc[u >> 1][(u & 1) * 2];
          dst[(2 * t4 + 1) * 8 + g] = acc[u >> 1][(u & 1) * 2 + 1];
        }
      }
      chain_consumer_barrier();
      const int n_out = (n_tiles / T) * RM * 8;          // outputs of the group: [block][token][row]
      for (int e = ctid; e < n_out; e += CH_CONSUMERS * 32) {
        const int blk = e / (RM * 8), m = (e / 8) % RM, r = e % 8;
        float first = 0.0f, second = 0.0f;
#pragma unroll
        for (int w = 0; w < CH_CONSUMERS; ++w) {
          first += red[((w * CH_GROUP_TILES + blk * T) * RM + m) * 8 + r];
          if (T == 2) second += red[((w * CH_GROUP_TILES + blk * T + 1) * RM + m) * 8 + r];
        }
        if (m < M && !failed) {
          const float v = st.epilogue == EPILOGUE_SWIGLU ? first / (1.0f + expf(-first)) * second : first;
          st.y[static_cast<size_t>(m) * st.ldy + static_cast<size_t>(gb + blk) * 8 + r] = __float2bfloat16_rn(v);
        }
      }
      chain_consumer_barrier();
    }
    if (tracing) trace[4 * s + 2] = now();

    if (s + 1 < a.n_stages) grid_barrier(s);
    if (tracing) trace[4 * s + 3] = now();
  }

  chain_consumer_barrier();           // nobody raises the flag after this point
  if (abort_flag) {
    // Give copies that are still in flight a bounded chance to land before the CTA's shared memory
    // goes to someone else.
    for (int s = warp; s < R; s += CH_CONSUMERS)
      for (int i = 0; i < (1 << 14) && !mbar_try_wait(&full[s], 0) && !mbar_try_wait(&full[s], 1); ++i) {}
    return;
  }
  // Whoever is done last leaves the counters at zero for the next launch.
  if (ctid == 0) {
    __threadfence();
    if (atomicAdd(&a.sync[1], 1) == ctas - 1) {
      a.sync[0] = 0;
      a.sync[1] = 0;
      __threadfence();
    }
  }
}

// Chains whose weights come to at most this many bytes a CTA put the weights on the tensor cores'
// 16-row side when there are at most 8 tokens (half as many products).  Measured on three shapes at
// batch 8 and 1: a chain of 32 MB (0.2 MB a CTA) takes 4.7 % off a decode step, one of 50 MB (0.34 MB)
// 1 to 2 %; chains of 105 MB (0.7 MB a CTA) and more, whose stream from memory is what counts, lose
// up to 5 % (a pair of tiles is waited for together).
inline long long& chain_flip_max_bytes() {
  static long long bytes = 640ll << 10;
  return bytes;
}

size_t chain_smem_bytes(int slots, int xs_rows, int xs_row_bytes) {
  return 1024 + static_cast<size_t>(slots) * CH_SLOT_BYTES + static_cast<size_t>(xs_rows) * xs_row_bytes +
         (2 * static_cast<size_t>(slots) + 1) * sizeof(unsigned long long) +
         static_cast<size_t>(CH_CONSUMERS) * CH_GROUP_TILES * xs_rows * 8 * sizeof(float);
}

// ---- tensor maps -------------------------------------------------------------------------------
// W [N, K] (K a multiple of 64, rows ldw apart) seen as [N][K / 64][64]: a box of 8 x 16 x 64 is
// 8 rows by 1024 columns.  Maps are kept: the same weights come back every step.
bool weight_tensor_map(const __nv_bfloat16* w, int N, int K, long long ldw, CUtensorMap* out) {
  static std::mutex mutex;
  static std::map<std::tuple<const void*, int, int, long long>, CUtensorMap> cache;
  std::lock_guard<std::mutex> lock(mutex);
  const auto key = std::make_tuple(static_cast<const void*>(w), N, K, ldw);
  const auto found = cache.find(key);
  if (found != cache.end()) {
    *out = found->second;
    return true;
  }
  const EncodeTiled encode = tensor_map_encoder();
  if (encode == nullptr) return false;
  const cuuint64_t dims[3] = {64, static_cast<cuuint64_t>(K / 64), static_cast<cuuint64_t>(N)};
  const cuuint64_t strides[2] = {128, static_cast<cuuint64_t>(ldw) * 2};
  const cuuint32_t box[3] = {64, CH_KC / 64, 8};
  const cuuint32_t element_strides[3] = {1, 1, 1};
  if (encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<__nv_bfloat16*>(w), dims, strides, box, element_strides,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (cache.size() > 65536) cache.clear();
  cache.emplace(key, *out);
  return true;
}

}  // namespace zb

using namespace zb;

// 1 if a stage of this shape can be part of a chain for M tokens.
ZB_API int zb_fused_chain_stage_supported(int M, int N, int K, int prologue, int epilogue) {
  if (M < 1 || M > CH_MAX_TOKENS || N < 8 || K < 8 || K % 8 != 0) return 0;
  if (N % (epilogue == EPILOGUE_SWIGLU ? 16 : 8) != 0) return 0;
  // The stage's whole input, M rows of K, sits in shared memory beside the ring.
  if (chain_smem_bytes(CH_MIN_SLOTS, M <= 8 ? 8 : 16, K * 2 + CH_PAD) > static_cast<size_t>(CH_SMEM_BUDGET)) return 0;
  (void)prologue;
  return 1;
}

ZB_API int zb_fused_chain_max_stages() { return CH_MAX_STAGES; }

// CTAs that the persistent kernels of later launches take at most (0: one per SM); returns the old setting.
ZB_API int zb_set_sm_share(int ctas) {
  const int before = sm_share();
  sm_share() = ctas < 0 ? 0 : ctas;
  return before;
}

// The limit described at chain_flip_max_bytes (bytes of weights per CTA and launch); returns the old one.
ZB_API long long zb_fused_chain_set_flip_bytes(long long bytes) {
  const long long before = chain_flip_max_bytes();
  chain_flip_max_bytes() = bytes;
  return before;
}

// Whether the kernels of a decode step (position encoding with cache write, decode attention, chain)
// are launched as programmatic dependents of the kernel before them (on by default).  Returns the
// setting that was in force.
ZB_API int zb_set_dependent_launch(int enabled) {
  const int before = dependent_launch_enabled() ? 1 : 0;
  dependent_launch_enabled() = enabled != 0;
  return before;
}

// CTAs of a launch: one per SM of the current device (0 if the device cannot be asked).
ZB_API int zb_fused_chain_grid() {
  int device = 0, sms = 0;
  if (cudaGetDevice(&device) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess)
    return 0;
  return shared_sm_count(sms);
}

// `trace`: null, or zb_fused_chain_grid() * n_stages * 4 ints on the device that receive every CTA's
// timeline (see ChainArgs).
// `xn`: null, or 16-byte aligned room on the device for 16 rows of the longest K among the stages with
// a norm (long rows are normalised there once for all CTAs; without it every CTA normalises them).
// Runs `n_stages` stages (an array of ChainStage on the host) for M tokens.  `sync`: two ints on the
// device, zero on entry, left zero.  The launch is cooperative: one CTA per SM.
ZB_API int zb_fused_chain(const void* stages, int n_stages, int M, int* sync, int* status, int* trace, void* xn,
                          void* stream) {
  if (stages == nullptr || n_stages < 1 || n_stages > CH_MAX_STAGES || sync == nullptr) return ERR_BAD_ARGUMENT;
  static ChainArgs a;         // large; every field that a launch reads is set below
  static std::mutex launch_mutex;
  std::lock_guard<std::mutex> launch_lock(launch_mutex);
  a = ChainArgs{};
  const auto* in = static_cast<const ChainStage*>(stages);
  int xs_k = 0;
  for (int s = 0; s < n_stages; ++s) {
    const ChainStage& st = in[s];
    if (!zb_fused_chain_stage_supported(M, st.N, st.K, st.prologue, st.epilogue)) return ERR_UNSUPPORTED;
    const auto aligned = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    if (st.w == nullptr || st.y == nullptr || !aligned(st.w) || st.ldw < st.K || st.ldw % 8 != 0 || st.ldy % 2 != 0 ||
        reinterpret_cast<uintptr_t>(st.y) % 4 != 0)
      return ERR_BAD_ARGUMENT;
    if (st.prologue == PROLOGUE_NONE) {
      if (st.x == nullptr || !aligned(st.x) || st.ldx < st.K || st.ldx % 8 != 0) return ERR_BAD_ARGUMENT;
    } else {
      if (st.residual_in == nullptr || !aligned(st.residual_in) || st.norm_w == nullptr) return ERR_BAD_ARGUMENT;
      if (st.prologue == PROLOGUE_ADD_NORM &&
          (st.delta == nullptr || !aligned(st.delta) || st.ldd < st.K || st.ldd % 8 != 0 || st.residual_out == nullptr ||
           !aligned(st.residual_out) || st.residual_out == st.residual_in))
        return ERR_BAD_ARGUMENT;
    }
    xs_k = st.K > xs_k ? st.K : xs_k;
    a.stage[s] = st;
    a.tiled[s] = st.K % 64 == 0 && weight_tensor_map(st.w, st.N, st.K, st.ldw, &a.map[s]) ? 1 : 0;
  }
  a.n_stages = n_stages;
  a.M = M;
  a.sync = sync;
  a.status = status;
  a.trace = trace;
  a.xn = reinterpret_cast<uintptr_t>(xn) % 16 == 0 ? static_cast<__nv_bfloat16*>(xn) : nullptr;
  const int xs_rows = M <= 8 ? 8 : 16;
  a.xs_row_bytes = xs_k * 2 + CH_PAD;
  int slots = CH_MIN_SLOTS;
  if (chain_smem_bytes(slots, xs_rows, a.xs_row_bytes) > static_cast<size_t>(CH_SMEM_BUDGET)) return ERR_UNSUPPORTED;
  while (slots < 64 && chain_smem_bytes(slots * 2, xs_rows, a.xs_row_bytes) <= static_cast<size_t>(CH_SMEM_BUDGET)) slots *= 2;
  a.ring_shift = 0;
  while ((1 << a.ring_shift) < slots) ++a.ring_shift;
  const size_t smem = chain_smem_bytes(slots, xs_rows, a.xs_row_bytes);
  long long weight_bytes = 0;
  for (int s = 0; s < n_stages; ++s) weight_bytes += static_cast<long long>(in[s].N) * in[s].K * 2;
  int device = 0, sms = 0, per_sm = 0;
  if (cuda_failed(cudaGetDevice(&device)) ||
      cuda_failed(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device)))
    return ERR_CUDA;
  const bool flip = M <= 8 && weight_bytes / (sms > 0 ? sms : 1) <= chain_flip_max_bytes();
  sms = shared_sm_count(sms);
  const auto launch = [&](auto kernel) -> int {
    if (cuda_failed(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem))) ||
        cuda_failed(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, CH_THREADS, smem)))
      return ERR_CUDA;
    if (per_sm < 1) return ERR_UNSUPPORTED;
    return launch_dependent(kernel, dim3(sms), dim3(CH_THREADS), smem, static_cast<cudaStream_t>(stream), true, a);
  };
  if (M > 8) return launch(fused_chain_kernel<true, false>);
  return flip ? launch(fused_chain_kernel<false, true>) : launch(fused_chain_kernel<false, false>);
}
