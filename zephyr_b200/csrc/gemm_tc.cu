// y = x w^T for a prompt's many rows on the fifth-generation tensor cores (tcgen05.mma, accumulators
// in tensor memory, operands by TMA), with what follows the product done where the sums are read
// out: nothing, or silu(gate) * up for a packed gate/up weight whose rows alternate in blocks of 8.
//
// x [M, K] and w [N, K] are bfloat16 with K contiguous.  The kernel is persistent: one CTA per SM
// takes output tiles of 128 rows x BN columns (BN = 256 or 128) in turn, the tiles that share
// weight rows next to each other in time so that they meet in the L2.  Roles of its six warps:
//   * warp 0, one thread: for every 64 elements of K one tiled copy of the tile's 128 rows of x and
//     one of its BN rows of w into the next of the stages of a ring in shared memory (128-byte
//     swizzle, the tensor core's K-major layout); rows and columns beyond M, N and K are filled
//     with zeros by the copy engine, so every size is taken;
//   * warp 1, one thread: four products 128 x BN x 16 per stage into one of two accumulators in
//     tensor memory (2 x BN columns of float32); tcgen05.commit frees the stage for the copies and,
//     after a tile's last product, hands the accumulator to the epilogue;
//   * warps 2..5: a thread owns one output row (its TMEM lane), reads 32 columns at a time, applies
//     the epilogue in float32, rounds once and puts its pieces into the warp's staging buffer in
//     shared memory, from where tiled TMA stores of 64 columns x 32 rows write them (rows and columns
//     beyond the matrix are left out by the copy engine).  While they work on one accumulator the
//     products of the next tile fill the other.
// A second form of the kernel runs a tile of 256 x 256 on a pair of SMs (further down).
// The activation reads the sums in float32, as the decode kernels do (one rounding; the
// reference rounds gate and up to bfloat16 first, src/layer/mlp.cpp:16-36, src/layer/activation.cu:31-33).
// Every wait is bounded and reports instead of hanging; tensor memory is given back on every path.
#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"
#include "mma.cuh"
#include "tcgen05.cuh"
#include "tma.cuh"

namespace zb {

constexpr int GT_BM = 128;
constexpr int GT_BK = 64;                  // elements of K per stage: one 128-byte swizzled row
constexpr int GT_THREADS = 192;
constexpr int GT_WAIT_LIMIT = 1 << 18;
constexpr int GT_PAIR = 2;                 // as block_n: tiles of 256 x 256 on pairs of SMs
constexpr int GT_EPI_PLAIN = 0;
constexpr int GT_EPI_SWIGLU = 1;           // columns 16 j .. 16 j + 7 are gates, 16 j + 8 .. 16 j + 15 their ups
constexpr int GT_EPI_FLOAT = 2;            // the sums as they are, float32 (logits)
constexpr int GT_A_BYTES = GT_BM * GT_BK * 2;
constexpr int GT_STAGING_BYTES = 32 * 128;  // an epilogue warp's 32 rows x 64 output columns on their way out; two a warp

template <int BN> struct GemmTcShape {
  static constexpr int B_BYTES = BN * GT_BK * 2;
  static constexpr int STAGE_BYTES = GT_A_BYTES + B_BYTES;
  static constexpr int STAGES = BN == 256 ? 4 : 6;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 8 * GT_STAGING_BYTES + 1024;   // the ring begins on a multiple of 1024
  static constexpr int TMEM_COLUMNS = 2 * BN;
};

struct GemmTcArgs {
  CUtensorMap x_map;             // x as [M][K]; box 64 x 128
  CUtensorMap w_map;             // w as [N][K]; box 64 x BN
  CUtensorMap y_map;             // y as [M][N, or N / 2 with the activation]; box 64 x 32; rows and columns beyond are not written
  int M, N, K;
  int tiles_m, tiles;
  int* status;
};

struct GemmTcShared {
  unsigned long long full[6], empty[6], acc_full[2], acc_empty[2];
  unsigned tmem_base;
  volatile int failed;
};

// A bounded wait that also gives up when another role of the CTA has.
__device__ __forceinline__ bool gt_wait(GemmTcShared& sh, unsigned long long* bar, unsigned parity) {
  for (int i = 0; i < GT_WAIT_LIMIT; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255) == 255 && sh.failed) return false;
  }
  return false;
}

// x / (1 + e^-x) with the special-function unit's exp2 and reciprocal (relative error about 2^-21,
// far inside the rounding to bfloat16 that follows): a thread has 128 of these to do per tile beside
// the products of the next tile, and the exact forms take some fifty dependent instructions each.
__device__ __forceinline__ float silu_fast(float x) {
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(e) : "f"(-1.4426950408889634f * x));
  asm("rcp.approx.ftz.f32 %0, %1;\n" : "=f"(r) : "f"(1.0f + e));
  return x * r;
}

// One box from shared memory to the matrix behind `map` at (x, y); x * element size is a multiple of 16
// bytes.  Part of the thread's current bulk group.
__device__ __forceinline__ void tiled_store_2d_s2g(const CUtensorMap* map, int x, int y, const void* smem_src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];\n"
               ::"l"(map), "r"(x), "r"(y), "r"(smem_u32(smem_src)) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;\n" ::: "memory"); }
// Until at most N of this thread's bulk groups have still to read their shared memory.
template <int N> __device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;\n" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory"); }

// An epilogue warp's 32 rows of a tile (its TMEM lanes, accumulator columns tmem_row .. + BN) -> y:
// the sums are read 32 columns at a time, the epilogue applied in float32, and groups of 64 output
// columns go through one of the warp's two staging buffers to a tiled store, which leaves out
// what lies beyond the matrix.
template <int BN, int EPI>
__device__ __forceinline__ void write_out_rows(const CUtensorMap& y_map, unsigned tmem_row, int row0, int n0, int width,
                                               unsigned char* staging, int& stores, int lane) {
  // A group = 128 bytes of a row's output: 64 bfloat16 columns from two reads of 32 sums (four reads with
  // the activation, which halves them), or 32 float32 columns from one read.
  constexpr int READS = EPI == GT_EPI_SWIGLU ? 4 : EPI == GT_EPI_FLOAT ? 1 : 2;
  constexpr int PIECES = 8 / READS;                                  // 16-byte pieces a read leaves
  constexpr int GROUP_COLUMNS = EPI == GT_EPI_FLOAT ? 32 : 64;       // output columns of a group
#pragma unroll 1
  for (int group = 0; group < BN / (32 * READS); ++group) {
    const int out_col = (EPI == GT_EPI_SWIGLU ? n0 / 2 : n0) + group * GROUP_COLUMNS;
    if (out_col >= width) break;                // the same for the whole warp
    unsigned char* buffer = staging + (stores & 1) * GT_STAGING_BYTES;
    if (stores >= 2) {                          // the store before last has read this buffer
      if (lane == 0) bulk_wait_read<1>();
      __syncwarp();
    }
#pragma unroll
    for (int r = 0; r < READS; ++r) {
      unsigned v[32];
      tmem_ld32(tmem_row + (group * READS + r) * 32, v);
      tc_wait_ld();
#pragma unroll
      for (int j = 0; j < PIECES; ++j) {
        // piece q of row `lane` lies where the 128-byte swizzle of the store's map expects it
        const int q = r * PIECES + j;
        uint4 w;
        if (EPI == GT_EPI_FLOAT) {
          w = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        } else {
          float o[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            if (EPI == GT_EPI_SWIGLU) {
              const float gate = __uint_as_float(v[16 * j + i]), up = __uint_as_float(v[16 * j + 8 + i]);
              o[i] = silu_fast(gate) * up;
            } else {
              o[i] = __uint_as_float(v[8 * j + i]);
            }
          }
          w.x = pack_bf16(o[0], o[1]);
          w.y = pack_bf16(o[2], o[3]);
          w.z = pack_bf16(o[4], o[5]);
          w.w = pack_bf16(o[6], o[7]);
        }
        *reinterpret_cast<uint4*>(buffer + lane * 128 + ((q ^ (lane & 7)) << 4)) = w;
      }
    }
    fence_proxy_async();
    __syncwarp();
    if (lane == 0) {
      tiled_store_2d_s2g(&y_map, out_col, row0, buffer);
      bulk_commit();
    }
    ++stores;
  }
}

template <int BN, int EPI>
__global__ void __launch_bounds__(GT_THREADS, 1) gemm_tc_kernel(const __grid_constant__ GemmTcArgs a) {
  using Shape = GemmTcShape<BN>;
  extern __shared__ unsigned char gt_smem_raw[];
  __shared__ GemmTcShared sh;
  unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(gt_smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_blocks = (a.K + GT_BK - 1) / GT_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Shape::STAGES; ++s) {
      mbar_init(&sh.full[s], 1);
      mbar_init(&sh.empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sh.acc_full[b], 1);
      mbar_init(&sh.acc_empty[b], 4);
    }
    sh.failed = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&sh.tmem_base, Shape::TMEM_COLUMNS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const unsigned tmem_base = sh.tmem_base;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      unsigned phase = 0;
      for (int tile = blockIdx.x; tile < a.tiles && !sh.failed; tile += gridDim.x) {
        const int m0 = (tile % a.tiles_m) * GT_BM, n0 = (tile / a.tiles_m) * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!gt_wait(sh, &sh.empty[stage], phase ^ 1)) {
            if (!sh.failed) report(a.status, STATUS_COPY_TIMEOUT, tile, kb);
            sh.failed = 1;
            break;
          }
          unsigned char* slot = ring + stage * Shape::STAGE_BYTES;
          mbar_arrive_expect_tx(&sh.full[stage], Shape::STAGE_BYTES);
          tiled_copy_2d_g2s(slot, &a.x_map, kb * GT_BK, m0, &sh.full[stage]);
          tiled_copy_2d_g2s(slot + GT_A_BYTES, &a.w_map, kb * GT_BK, n0, &sh.full[stage]);
          if (++stage == Shape::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr unsigned IDESC = tc_idesc(false, BN);
      int stage = 0, acc = 0;
      unsigned phase = 0, acc_phase = 0;
      for (int tile = blockIdx.x; tile < a.tiles && !sh.failed; tile += gridDim.x) {
        if (!gt_wait(sh, &sh.acc_empty[acc], acc_phase ^ 1)) {
          if (!sh.failed) report(a.status, STATUS_BARRIER_TIMEOUT, tile, -1);
          sh.failed = 1;
          break;
        }
        tc_fence_after_sync();
        const unsigned d = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!gt_wait(sh, &sh.full[stage], phase)) {
            if (!sh.failed) report(a.status, STATUS_COPY_TIMEOUT, tile, -2 - kb);
            sh.failed = 1;
            break;
          }
          tc_fence_after_sync();
          const unsigned slot = smem_u32(ring + stage * Shape::STAGE_BYTES);
          const unsigned long long x_desc = desc_k_major(slot), w_desc = desc_k_major(slot + GT_A_BYTES);
#pragma unroll
          for (int k = 0; k < GT_BK / 16; ++k) tc_mma(d, x_desc + 2 * k, w_desc + 2 * k, IDESC, (kb | k) != 0 ? 1u : 0u);
          tc_commit(&sh.empty[stage]);
          if (++stage == Shape::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (sh.failed) break;
        tc_commit(&sh.acc_full[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    const int quarter = warp & 3;                   // the TMEM lanes this warp may read: 32 quarter .. + 31
    unsigned char* staging = ring + Shape::STAGES * Shape::STAGE_BYTES + (warp - 2) * 2 * GT_STAGING_BYTES;
    const int width = EPI == GT_EPI_SWIGLU ? a.N / 2 : a.N;
    int acc = 0, stores = 0;
    unsigned acc_phase = 0;
    for (int tile = blockIdx.x; tile < a.tiles && !sh.failed; tile += gridDim.x) {
      const int m0 = (tile % a.tiles_m) * GT_BM, n0 = (tile / a.tiles_m) * BN;
      if (!gt_wait(sh, &sh.acc_full[acc], acc_phase)) {
        if (!sh.failed) report(a.status, STATUS_BARRIER_TIMEOUT, tile, -3);
        sh.failed = 1;
        break;
      }
      tc_fence_after_sync();
      write_out_rows<BN, EPI>(a.y_map, tmem_base + (static_cast<unsigned>(32 * quarter) << 16) + acc * BN,
                              m0 + 32 * quarter, n0, width, staging, stores, lane);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) tc_mbar_arrive(&sh.acc_empty[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
    if (lane == 0) bulk_wait_all();                 // the staging buffers are read, the rows written
  }

  // Everybody meets here on every path, and the warp that took the tensor memory gives it back.
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Shape::TMEM_COLUMNS);
  }
}

// ---- The same on pairs of SMs ------------------------------------------------------------------
// Two CTAs of a cluster on neighbouring SMs share an output tile of 256 rows x 256 columns
// (tcgen05.mma.cta_group::2): each copies its 128 rows of x and its 128 of the tile's 256 rows of w,
// the products read the halves of w from both CTAs' shared memory, and each CTA's tensor memory
// receives the sums of its own 128 rows.  A product then reads 8 KB of a CTA's shared memory per
// 128 cycles of tensor work instead of 12 KB, which leaves the copies the bandwidth they need; alone,
// an SM's shared memory holds the tensor cores at two thirds of their rate.
//   * The first CTA of a pair (rank 0) owns the barriers of the stages' arrival: both CTAs' copies
//     count their bytes there.  Its one thread issues the products for both and reports their
//     completion to the barriers of both CTAs (stage free again; accumulator ready).
//   * Each CTA's copy thread waits for its own stage to be free, each CTA's epilogue warps for their
//     own accumulator, and they hand an accumulator back by arriving on rank 0's barrier.
// No copy is multicast: every CTA fetches its own operands.
constexpr int GP_BN = 256;
constexpr int GP_HALF_BYTES = 128 * GT_BK * 2;               // 128 rows of x, or of w, of one stage
constexpr int GP_STAGE_BYTES = 2 * GP_HALF_BYTES;
constexpr int GP_STAGES = 6;
constexpr int GP_SMEM_BYTES = GP_STAGES * GP_STAGE_BYTES + 8 * GT_STAGING_BYTES + 1024;
constexpr int GP_TMEM_COLUMNS = 2 * GP_BN;

__device__ __forceinline__ unsigned cluster_rank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// The address, in the cluster's window, of this CTA's shared-memory address `smem_address` in the CTA of rank `rank`.
__device__ __forceinline__ unsigned in_cta_of_rank(unsigned smem_address, unsigned rank) {
  unsigned r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(smem_address), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_in_cluster(unsigned cluster_address) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_address) : "memory");
}
// A tiled copy into this CTA's shared memory whose bytes are counted on a barrier of the pair's first CTA.
__device__ __forceinline__ void tiled_copy_2d_g2s_pair(void* smem_dst, const CUtensorMap* map, int x, int y, unsigned bar_cluster_address) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
               ::"r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(bar_cluster_address) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(unsigned* smem_result, unsigned columns) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(smem_result)), "r"(columns) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(unsigned address, unsigned columns) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(address), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_mma_pair(unsigned d_tmem, unsigned long long a_desc, unsigned long long b_desc,
                                            unsigned idesc, unsigned accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
               ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// One arrival on the barrier at this address in BOTH CTAs of the pair when every product issued so far is complete.
__device__ __forceinline__ void tc_commit_pair(unsigned long long* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n"
               ::"r"(smem_u32(bar)), "h"(static_cast<unsigned short>(3)) : "memory");
}
// Instruction descriptor of the pair's product: as tc_idesc with M = 256.
__host__ __device__ constexpr unsigned tc_idesc_pair(unsigned n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((256u >> 4) << 24);
}

template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GT_THREADS, 1) gemm_tc_pair_kernel(const __grid_constant__ GemmTcArgs a) {
  extern __shared__ unsigned char gt_smem_raw[];
  __shared__ GemmTcShared sh;
  unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(gt_smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned rank = cluster_rank();
  const int k_blocks = (a.K + GT_BK - 1) / GT_BK;
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < GP_STAGES; ++s) {
      mbar_init(&sh.full[s], 1);
      mbar_init(&sh.empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sh.acc_full[b], 1);
      mbar_init(&sh.acc_empty[b], 8);               // four epilogue warps in each CTA
    }
    sh.failed = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(&sh.tmem_base, GP_TMEM_COLUMNS);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();                               // both CTAs' barriers and tensor memory are there
  tc_fence_after_sync();
  const unsigned tmem_base = sh.tmem_base;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      unsigned phase = 0;
      for (int tile = pair; tile < a.tiles && !sh.failed; tile += pairs) {
        const int m0 = (tile % a.tiles_m) * 256 + 128 * rank, n0 = (tile / a.tiles_m) * GP_BN + 128 * rank;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!gt_wait(sh, &sh.empty[stage], phase ^ 1)) {
            if (!sh.failed) report(a.status, STATUS_COPY_TIMEOUT, tile, kb);
            sh.failed = 1;
            break;
          }
          unsigned char* slot = ring + stage * GP_STAGE_BYTES;
          if (rank == 0) mbar_arrive_expect_tx(&sh.full[stage], 2 * GP_STAGE_BYTES);
          const unsigned full = in_cta_of_rank(smem_u32(&sh.full[stage]), 0);
          tiled_copy_2d_g2s_pair(slot, &a.x_map, kb * GT_BK, m0, full);
          tiled_copy_2d_g2s_pair(slot + GP_HALF_BYTES, &a.w_map, kb * GT_BK, n0, full);
          if (++stage == GP_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      constexpr unsigned IDESC = tc_idesc_pair(GP_BN);
      int stage = 0, acc = 0;
      unsigned phase = 0, acc_phase = 0;
      for (int tile = pair; tile < a.tiles && !sh.failed; tile += pairs) {
        if (!gt_wait(sh, &sh.acc_empty[acc], acc_phase ^ 1)) {
          if (!sh.failed) report(a.status, STATUS_BARRIER_TIMEOUT, tile, -1);
          sh.failed = 1;
          break;
        }
        tc_fence_after_sync();
        const unsigned d = tmem_base + acc * GP_BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!gt_wait(sh, &sh.full[stage], phase)) {
            if (!sh.failed) report(a.status, STATUS_COPY_TIMEOUT, tile, -2 - kb);
            sh.failed = 1;
            break;
          }
          tc_fence_after_sync();
          const unsigned slot = smem_u32(ring + stage * GP_STAGE_BYTES);
          const unsigned long long x_desc = desc_k_major(slot), w_desc = desc_k_major(slot + GP_HALF_BYTES);
#pragma unroll
          for (int k = 0; k < GT_BK / 16; ++k) tc_mma_pair(d, x_desc + 2 * k, w_desc + 2 * k, IDESC, (kb | k) != 0 ? 1u : 0u);
          tc_commit_pair(&sh.empty[stage]);
          if (++stage == GP_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (sh.failed) break;
        tc_commit_pair(&sh.acc_full[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    const int quarter = warp & 3;
    unsigned char* staging = ring + GP_STAGES * GP_STAGE_BYTES + (warp - 2) * 2 * GT_STAGING_BYTES;
    const int width = EPI == GT_EPI_SWIGLU ? a.N / 2 : a.N;
    int acc = 0, stores = 0;
    unsigned acc_phase = 0;
    for (int tile = pair; tile < a.tiles && !sh.failed; tile += pairs) {
      const int m0 = (tile % a.tiles_m) * 256 + 128 * rank, n0 = (tile / a.tiles_m) * GP_BN;
      if (!gt_wait(sh, &sh.acc_full[acc], acc_phase)) {
        if (!sh.failed) report(a.status, STATUS_BARRIER_TIMEOUT, tile, -3);
        sh.failed = 1;
        break;
      }
      tc_fence_after_sync();
      write_out_rows<GP_BN, EPI>(a.y_map, tmem_base + (static_cast<unsigned>(32 * quarter) << 16) + acc * GP_BN,
                                 m0 + 32 * quarter, n0, width, staging, stores, lane);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_in_cluster(in_cta_of_rank(smem_u32(&sh.acc_empty[acc]), 0));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
    if (lane == 0) bulk_wait_all();
  }

  // Both CTAs meet here on every path (the other's barriers and tensor memory are used until
  // then), and the warps that took the tensor memory give it back.
  tc_fence_before_sync();
  __syncthreads();
  __syncwarp();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, GP_TMEM_COLUMNS);
  }
}

// A row-major matrix [rows][cols] of bfloat16 (or float32) with `ld` elements between rows, copied in
// boxes of 128 bytes (64 or 32 columns) x box_rows rows with the 128-byte swizzle.  Maps are kept: weights come back every step,
// and so do the activations of a captured step.
bool matrix_tensor_map(const void* base, long long rows, int cols, long long ld, int box_rows, CUtensorMap* out,
                       int element_bytes = 2) {
  static std::mutex mutex;
  static std::map<std::tuple<const void*, long long, int, long long, int, int>, CUtensorMap> kept;
  std::lock_guard<std::mutex> lock(mutex);
  const auto key = std::make_tuple(base, rows, cols, ld, box_rows, element_bytes);
  const auto found = kept.find(key);
  if (found != kept.end()) {
    *out = found->second;
    return true;
  }
  const EncodeTiled encode = tensor_map_encoder();
  if (encode == nullptr) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * element_bytes};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / element_bytes), static_cast<cuuint32_t>(box_rows)};     // 128 bytes a row
  const cuuint32_t element_strides[2] = {1, 1};
  if (encode(out, element_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
             const_cast<void*>(base), dims, strides, box, element_strides,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (kept.size() > 4096) kept.clear();
  kept.emplace(key, *out);
  return true;
}

template <int BN, int EPI>
int gemm_tc_launch(GemmTcArgs& a, const void* w, int sms, cudaStream_t stream) {
  using Shape = GemmTcShape<BN>;
  if (!matrix_tensor_map(w, a.N, a.K, a.K, BN, &a.w_map)) return ERR_CUDA;
  a.tiles_m = (a.M + GT_BM - 1) / GT_BM;
  a.tiles = a.tiles_m * ((a.N + BN - 1) / BN);
  if (cuda_failed(cudaFuncSetAttribute(gemm_tc_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, Shape::SMEM_BYTES)))
    return ERR_CUDA;
  const int grid = a.tiles < sms ? a.tiles : sms;
  gemm_tc_kernel<BN, EPI><<<grid, GT_THREADS, Shape::SMEM_BYTES, stream>>>(a);
  return launch_result();
}

template <int EPI>
int gemm_tc_pair_launch(GemmTcArgs& a, const void* w, int sms, cudaStream_t stream) {
  if (!matrix_tensor_map(w, a.N, a.K, a.K, 128, &a.w_map)) return ERR_CUDA;
  a.tiles_m = (a.M + 255) / 256;
  a.tiles = a.tiles_m * ((a.N + GP_BN - 1) / GP_BN);
  if (cuda_failed(cudaFuncSetAttribute(gemm_tc_pair_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, GP_SMEM_BYTES)))
    return ERR_CUDA;
  cudaLaunchConfig_t config = {};
  config.blockDim = dim3(GT_THREADS);
  config.dynamicSmemBytes = GP_SMEM_BYTES;
  config.stream = stream;
  config.gridDim = dim3(2 * (sms / 2));
  int clusters = 0;                                 // how many pairs the device holds at once
  if (cuda_failed(cudaOccupancyMaxActiveClusters(&clusters, gemm_tc_pair_kernel<EPI>, &config)) || clusters <= 0) return ERR_CUDA;
  const int pairs = a.tiles < clusters ? a.tiles : clusters;
  config.gridDim = dim3(2 * pairs);
  return cuda_failed(cudaLaunchKernelEx(&config, gemm_tc_pair_kernel<EPI>, a)) ? ERR_CUDA : launch_result();
}

}  // namespace zb

using namespace zb;

// 1 if zb_gemm_tc takes these sizes (x [M, K] with ldx elements between rows, w [N, K], y with ldy).
ZB_API int zb_gemm_tc_supported(int M, int N, int K, long long ldx, int ldy, int epilogue) {
  if (M <= 0 || N <= 0 || K <= 0 || K % 8 != 0 || ldx % 8 != 0 || ldx < K || (epilogue != GT_EPI_FLOAT && ldy % 8 != 0)) return 0;
  if (epilogue == GT_EPI_SWIGLU) return N % 16 == 0 && ldy >= N / 2;
  if (epilogue == GT_EPI_FLOAT) return ldy % 4 == 0 && ldy >= N;          // ldy counts float32 elements then
  return epilogue == GT_EPI_PLAIN && ldy >= N;
}

// y = epilogue(x w^T), x and w bfloat16.  epilogue 0: y [M, N] bfloat16; 2: the same in float32;
// 1: y [M, N / 2] = silu(gate) * up for w's rows in
// blocks of 8 gate rows and their 8 up rows.  block_n is 256 or 128, or 2 for tiles of 256 x 256 on pairs of
// SMs (0: chosen from the sizes).
ZB_API int zb_gemm_tc(void* y, const void* x, const void* w, int M, int N, int K, long long ldx, int ldy, int epilogue,
                      int block_n, int* status, void* stream) {
  if (!zb_gemm_tc_supported(M, N, K, ldx, ldy, epilogue)) return ERR_UNSUPPORTED;
  if (reinterpret_cast<uintptr_t>(y) % 16 != 0 || reinterpret_cast<uintptr_t>(x) % 16 != 0 ||
      reinterpret_cast<uintptr_t>(w) % 16 != 0)
    return ERR_BAD_ARGUMENT;
  int device = 0, sms = 0;
  if (cuda_failed(cudaGetDevice(&device)) ||
      cuda_failed(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device)))
    return ERR_CUDA;
  if (block_n == 0) {
    // From three tiles of rows on, pairs of SMs on tiles of 256 x 256: their products do not wait for
    // shared memory.  Below, one SM a tile: 256 columns halve the traffic of x through shared memory;
    // where that would leave SMs without a tile, tiles of 128 columns fill them.
    const long long tiles256 = static_cast<long long>((M + GT_BM - 1) / GT_BM) * ((N + 255) / 256);
    block_n = M > 2 * GT_BM ? GT_PAIR : tiles256 >= sms ? 256 : 128;
  }
  if (block_n != 256 && block_n != 128 && block_n != GT_PAIR) return ERR_BAD_ARGUMENT;
  GemmTcArgs a;
  a.M = M; a.N = N; a.K = K;
  a.status = status;
  if (!matrix_tensor_map(x, M, K, ldx, GT_BM, &a.x_map)) return ERR_CUDA;
  if (!matrix_tensor_map(y, M, epilogue == GT_EPI_SWIGLU ? N / 2 : N, ldy, 32, &a.y_map, epilogue == GT_EPI_FLOAT ? 4 : 2)) return ERR_CUDA;
  const cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (block_n == GT_PAIR)
    return epilogue == GT_EPI_SWIGLU ? gemm_tc_pair_launch<GT_EPI_SWIGLU>(a, w, sms, s)
           : epilogue == GT_EPI_FLOAT ? gemm_tc_pair_launch<GT_EPI_FLOAT>(a, w, sms, s) : gemm_tc_pair_launch<GT_EPI_PLAIN>(a, w, sms, s);
  if (epilogue == GT_EPI_FLOAT)
    return block_n == 256 ? gemm_tc_launch<256, GT_EPI_FLOAT>(a, w, sms, s) : gemm_tc_launch<128, GT_EPI_FLOAT>(a, w, sms, s);
  if (epilogue == GT_EPI_SWIGLU)
    return block_n == 256 ? gemm_tc_launch<256, GT_EPI_SWIGLU>(a, w, sms, s) : gemm_tc_launch<128, GT_EPI_SWIGLU>(a, w, sms, s);
  return block_n == 256 ? gemm_tc_launch<256, GT_EPI_PLAIN>(a, w, sms, s) : gemm_tc_launch<128, GT_EPI_PLAIN>(a, w, sms, s);
}
