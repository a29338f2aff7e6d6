// TMA (cp.async.bulk.tensor) and mbarrier helpers for the sm_100a streaming kernels, plus the
// host-side tensor-map encoder.  All loads are local (this GPU's memory) and never use cluster
// multicast.  Every wait on an mbarrier is bounded: after kWaitLimit polls the caller records
// an error word and leaves, it never spins forever.
#pragma once

#include <cuda.h>

#include "ms_common.cuh"

namespace ms {

// ---------------------------------------------------------------------------------------
// host: tensor maps
// ---------------------------------------------------------------------------------------
enum class Swizzle : int { None = 0, B32 = 1, B64 = 2, B128 = 3 };

// Rank-2 or rank-3 row-major tensor of 2-byte or 4-byte elements.  dims[0] is the innermost
// (contiguous) extent; strides_bytes[i] is the byte stride of dims[i+1].  Returns MS_OK or
// MS_ERR_LAUNCH (driver entry point missing / encode rejected).
int encode_tensor_map(CUtensorMap* out, void* base, int elem_bytes, int rank, const uint64_t* dims,
                      const uint64_t* strides_bytes, const uint32_t* box, Swizzle swizzle);

// Address of the library's device error word (0 = no error) on the current device.
int* device_error_word();

constexpr int kErrBarrierTimeout = 0x100;  // an mbarrier wait ran out of polls

// ---------------------------------------------------------------------------------------
// device: shared-memory swizzles that match the TMA swizzle modes (tile base 1024-byte aligned)
// ---------------------------------------------------------------------------------------
template <int ROW_BYTES>
__device__ __forceinline__ uint32_t swz_rows(uint32_t off) {
  static_assert(ROW_BYTES == 32 || ROW_BYTES == 64 || ROW_BYTES == 128, "row bytes");
  constexpr uint32_t mask = ROW_BYTES == 128 ? 7u : (ROW_BYTES == 64 ? 3u : 1u);
  return off ^ (((off >> 7) & mask) << 4);
}
template <int ROW_BYTES>
constexpr Swizzle swizzle_for_rows() {
  return ROW_BYTES == 128 ? Swizzle::B128 : (ROW_BYTES == 64 ? Swizzle::B64 : Swizzle::B32);
}

// ---------------------------------------------------------------------------------------
// device: mbarrier
// ---------------------------------------------------------------------------------------
constexpr int kWaitLimit = 1 << 22;

__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::);
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
// true when the phase with the given parity has completed; false after kWaitLimit polls
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (int i = 0; i < kWaitLimit; ++i) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}

// one non-blocking look at the phase with the given parity
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}

// ---------------------------------------------------------------------------------------
// device: bulk tensor copies
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, int c0, int c1, int c2, uint32_t src) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];\n"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(src)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;\n" ::: "memory"); }
// wait until at most N of this thread's committed store groups still READ shared memory
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;\n" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;\n" ::"n"(N) : "memory");
}
// make generic-proxy writes to shared memory visible to the async proxy (before a TMA store)
// Make the warp wait until `bits` is in its registers.  ld.shared only ISSUES a read; an mbarrier arrive that follows
// it in the program can be performed -- and the buffer it releases be overwritten by the producer's next bulk copy --
// before the data has come back.  (Measured: rotary rows released right after their loads were replaced by the next
// tile's rows for single threads in about every second launch of 32768 tokens.)  A warp issues in order, so one
// instruction that consumes a value derived from every load holds back everything after it until the loads have
// returned.  The store is never taken for real data, and would only touch the scratch word if it were.
__device__ __forceinline__ void wait_for_loaded(uint32_t bits, uint32_t scratch) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.eq.u32 p, %0, 0x9e3779b9;\n"
      "@p st.shared.u32 [%1], %0;\n"
      "}\n" ::"r"(bits),
      "r"(scratch)
      : "memory");
}

__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

}  // namespace ms
