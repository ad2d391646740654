// The fifth-generation tensor cores in PTX: tensor memory (TMEM) allocation, tcgen05.mma with the
// operands in shared or tensor memory, completion reported to mbarriers, loads and stores of TMEM
// rows, and the descriptors of operands that lie in shared memory with the 128-byte swizzle.
#pragma once

#include "common.cuh"
#include "mma.cuh"

namespace zb {

__device__ __forceinline__ void tmem_alloc(unsigned* smem_result, unsigned columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(smem_result)), "r"(columns) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(unsigned address, unsigned columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(address), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
// D[tmem] (+)= A[smem] * B[smem]; `accumulate` 0 overwrites D.
__device__ __forceinline__ void tc_mma(unsigned d_tmem, unsigned long long a_desc, unsigned long long b_desc,
                                       unsigned idesc, unsigned accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
               ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]: A's 128 rows lie in the 128 lanes, 16 bfloat16 along K as 8 columns
// of two (the lower index in the lower half).
// The thread that issues the products shares its scheduler with softmax warps, and a product of
// this size is done sooner than a dozen instructions get issued there: everything but the
// instruction itself is taken out of the way (descriptors advance by a constant, the predicate is
// set once).
template <bool ACCUMULATE>
__device__ __forceinline__ void tc_mma_ts(unsigned d_tmem, unsigned a_tmem, unsigned long long b_desc, unsigned idesc) {
  if (ACCUMULATE)
    asm volatile("{\n.reg .pred p;\nsetp.eq.b32 p, 0, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc) : "memory");
  else
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, 0, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc) : "memory");
}
// The mbarrier gets one arrival when every product issued so far by this thread is complete.
__device__ __forceinline__ void tc_commit(unsigned long long* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
// 32 consecutive columns of this thread's TMEM lane (the warp's 32 lanes start at `address`'s lane).
__device__ __forceinline__ void tmem_ld32(unsigned address, unsigned (&r)[32]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
               "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                 "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                 "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
               : "r"(address) : "memory");
}
__device__ __forceinline__ void tmem_st32(unsigned address, const unsigned (&r)[32]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
               "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
               ::"r"(address), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                 "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                 "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                 "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
               : "memory");
}
// Has the phase with this parity completed?  Never suspends the thread (try_wait may, for a while).
__device__ __forceinline__ bool tc_mbar_test(unsigned long long* bar, unsigned parity) {
  unsigned done;
  asm volatile("{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return done != 0;
}
__device__ __forceinline__ void tc_mbar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}

// Shared-memory matrix descriptor (64 bits): start address >> 4 in bits 0..13, leading byte
// offset >> 4 in 16..29, stride byte offset >> 4 in 32..45, version 1 in 46..47, layout type 2
// (128-byte swizzle) in 61..63.  K-major operand with rows of 128 bytes (64 bfloat16 of K); groups of
// 8 rows are 1024 bytes apart (the stride offset); 16 elements of K are 32 bytes further along the row.
__device__ __forceinline__ unsigned long long desc_k_major(unsigned smem_address) {
  return static_cast<unsigned long long>((smem_address >> 4) & 0x3FFFu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: float32 accumulator (bits 4..5 = 1), bfloat16 A and B (7..9 = 1, 10..12 = 1),
// B MN-major if asked (bit 16), N >> 3 in 17..22, M >> 4 in 24..28.  M is 128.
__host__ __device__ constexpr unsigned tc_idesc(bool b_mn_major, unsigned n = 128) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn_major ? (1u << 16) : 0u) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}

}  // namespace zb
