// Fifth-generation tensor-core (tcgen05) helpers for the sm_100a token kernels: tensor-memory
// allocation, shared-memory matrix descriptors, the instruction descriptor of the BF16 x BF16 -> FP32
// product, MMA issue with the row operand in shared memory or in tensor memory, completion through an
// mbarrier, and tensor-memory loads / stores of one row per thread.  Everything is for one CTA per
// MMA (cta_group::1); nothing here touches another GPU's memory or uses cluster multicast.
#pragma once

#include "ms_tma.cuh"

namespace ms {
namespace tc {

// ---------------------------------------------------------------------------------------
// tensor memory (512 columns of 128 lanes x 32 bits per SM)
// ---------------------------------------------------------------------------------------
// Executed by one whole warp: reserves `cols` columns (a power of two >= 32) and writes the base
// address to the shared-memory word at `dst`.  The same warp frees them with tmem_free.
__device__ __forceinline__ void tmem_alloc(uint32_t dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(dst), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_free(uint32_t base, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(base), "r"(cols) : "memory");
}

__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

// ---------------------------------------------------------------------------------------
// descriptors
// ---------------------------------------------------------------------------------------
// Shared-memory matrix descriptor (64 bits): start address / 16 in bits [0,14), "leading" byte offset / 16
// in [16,30), "stride" byte offset / 16 in [32,46), descriptor version 1 in [46,48), swizzle mode in
// [61,64) (2 = 128-byte, 4 = 64-byte, 6 = 32-byte).  The tiles here are what TMA writes with the
// matching swizzle: rows of ROW_BYTES bytes, tile base 1024-byte aligned.
//
//  * contraction-major operand (rows = M or N index, the contraction index runs along a row): groups of
//    eight rows are `8 * ROW_BYTES` apart (stride offset); one MMA consumes 16 elements = 32 bytes of
//    each row, so the k-th step starts 32*k bytes further.
//  * row-major-in-N operand (rows = contraction index, 64 N-elements = 128 bytes along a row, 128-byte
//    swizzle): groups of eight contraction rows are 1024 bytes apart (stride offset); one MMA
//    consumes 16 rows = 2048 bytes.
template <int ROW_BYTES>
__device__ __forceinline__ uint64_t smem_desc_k_major(uint32_t addr) {
  static_assert(ROW_BYTES == 32 || ROW_BYTES == 64 || ROW_BYTES == 128, "row bytes");
  constexpr uint64_t layout = ROW_BYTES == 128 ? 2 : (ROW_BYTES == 64 ? 4 : 6);
  constexpr uint64_t sbo = (8 * ROW_BYTES) >> 4;
  return (uint64_t)((addr & 0x3ffffu) >> 4) | (uint64_t(1) << 16) | (sbo << 32) | (uint64_t(1) << 46) | (layout << 61);
}
__device__ __forceinline__ uint64_t smem_desc_n_major_128(uint32_t addr) {
  constexpr uint64_t sbo = 1024 >> 4, lbo = 1024 >> 4;
  return (uint64_t)((addr & 0x3ffffu) >> 4) | (lbo << 16) | (sbo << 32) | (uint64_t(1) << 46) | (uint64_t(2) << 61);
}

// Instruction descriptor of kind::f16 with BF16 operands and an FP32 accumulator: accumulator format
// in bits [4,6) (1 = F32), operand formats in [7,10) and [10,13) (1 = BF16), operand-major bits 15 (A)
// and 16 (B) (0 = contraction-major), N/8 in [17,23), M/16 in [24,29).
__host__ __device__ constexpr uint32_t idesc_bf16(int m, int n, bool b_n_major, bool a_m_major = false) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((a_m_major ? 1u : 0u) << 15) | ((b_n_major ? 1u : 0u) << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// ---------------------------------------------------------------------------------------
// MMA issue and completion
// ---------------------------------------------------------------------------------------
// The three functions below are called by a whole, converged warp with warp-uniform arguments; one elected
// lane (always the same one) executes the instruction.  Keeping the surrounding code warp-uniform lets the
// compiler hold descriptors in uniform registers, which is where the MMA instruction wants them: issued
// from a divergent `if (lane == 0)` region the same loop took about 80 cycles per MMA.
__device__ __forceinline__ bool elect_one() {
  uint32_t chosen;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "elect.sync _|p, 0xffffffff;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(chosen));
  return chosen != 0;
}
// D[128 x N] (+)= A[128 x 16] B[N x 16]^T; `accumulate` == 0 overwrites D.
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  if (elect_one()) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
// the same with the row operand A in tensor memory: lane = row, 8 columns per 16 BF16 values
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  if (elect_one()) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
        "}\n" ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
// the mbarrier at `bar` receives one arrival when every MMA issued so far by the elected lane has completed
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  if (elect_one())
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}

// ---------------------------------------------------------------------------------------
// the same instructions for a batch issued from inside ONE elected region: no election per MMA, the
// constant upper descriptor word and the instruction descriptor are immediates, the lower word (start
// address / 16 and leading offset) is the only run-time part.  With the election, the 64-bit descriptor
// arithmetic and the conversions to uniform registers done per MMA, the issuing warp (which shares its
// scheduler with compute warps) needed ~200 cycles per MMA against the 22-50 the tensor core takes.
// ---------------------------------------------------------------------------------------
constexpr uint32_t desc_hi_k_major(int row_bytes) {
  return (uint32_t)((8 * row_bytes) >> 4) | (1u << 14) | ((row_bytes == 128 ? 2u : (row_bytes == 64 ? 4u : 6u)) << 29);
}
constexpr uint32_t desc_hi_n_major_128() { return (uint32_t)(1024 >> 4) | (1u << 14) | (2u << 29); }
__device__ __forceinline__ uint32_t desc_lo_k_major(uint32_t addr) { return ((addr & 0x3ffffu) >> 4) | (1u << 16); }
__device__ __forceinline__ uint32_t desc_lo_n_major_128(uint32_t addr) { return ((addr & 0x3ffffu) >> 4) | ((1024u >> 4) << 16); }

template <uint32_t HI_A, uint32_t HI_B, uint32_t IDESC>
__device__ __forceinline__ void mma_ss_raw(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      ".reg .b64 da, db;\n"
      "mov.b64 da, {%1, %4};\n"
      "mov.b64 db, {%2, %5};\n"
      "setp.ne.b32 p, %3, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %6, p;\n"
      "}\n" ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(accumulate), "n"(HI_A), "n"(HI_B), "n"(IDESC)
      : "memory");
}
template <uint32_t HI_B, uint32_t IDESC>
__device__ __forceinline__ void mma_ts_raw(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      ".reg .b64 db;\n"
      "mov.b64 db, {%2, %4};\n"
      "setp.ne.b32 p, %3, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %5, p;\n"
      "}\n" ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(accumulate), "n"(HI_B), "n"(IDESC)
      : "memory");
}
__device__ __forceinline__ void mma_commit_raw(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}

// ---------------------------------------------------------------------------------------
// tensor-memory loads and stores, shape 32x32b: thread i of a warp owns lane 32*(warp%4) + i and moves
// N consecutive 32-bit columns starting at the column of `addr` (whose lane field is 32*(warp%4))
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_ld16(uint32_t addr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(addr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t addr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(addr)
               : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t addr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n" ::"r"(addr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

constexpr int kErrTensorMemory = 0x400;   // tensor-memory allocation returned nothing usable

}  // namespace tc
}  // namespace ms
