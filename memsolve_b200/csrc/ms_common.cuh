// Shared device helpers for the MemSolve sm_100a kernels: swizzled shared-memory tiles,
// asynchronous global->shared copies, ldmatrix / mma.sync wrappers, BF16 split words.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <utility>

#include "../../include/memsolve_b200.h"

namespace ms {

constexpr int kTileTokens = 64;   // token rows per shared-memory tile
constexpr int kChanBlock = 64;    // content channels handled per pass (one 128-byte row)

// ---------------------------------------------------------------------------------------
// launch bookkeeping shared by the host-side launchers
// ---------------------------------------------------------------------------------------
struct Plan {
  int systems;       // B*H
  int dblocks;       // ceil(d / 64)
  int de_slots;      // <dY,C> partial entries per (system, chunk): two per 64-channel block
  int dpad;          // d rounded up to a multiple of 8 (pitch of split coefficient tensors)
  int chunks;        // token chunks per system in the reductions
  int chunk_tokens;  // tokens per chunk (multiple of 64)
  int chunks_bwd;        // the same for the adjoint reduction, whose grid has no per-head CTAs riding along
  int chunk_tokens_bwd;  // (see backward_plan)
  bool aligned;      // 16-byte vector path usable for projected / dy / tables
  bool tma;          // TMA kernels allowed (off when the environment sets MEMSOLVE_NO_TMA=1)
  bool tc;           // tcgen05 kernels allowed (off with MEMSOLVE_NO_TMA=1 or MEMSOLVE_NO_TCGEN05=1)
  bool stats_tc;     // the token chunks were sized for the tcgen05 statistics kernel (head groups, 128-token tiles)
  bool pack;         // ms_mix_forward / ms_mix_backward add the partials in a launch of their own (many chunks)
  size_t fwd_partial_floats;  // per (system, chunk): r*r + r*d
  size_t bwd_partial_floats;  // per (system, chunk): r*d
  size_t ws_partials;         // floats
  size_t ws_de;               // floats: systems * chunks * de_slots
  size_t ws_hmat;             // floats: systems * r * r
  size_t ws_de_sys;           // floats: systems
  size_t ws_packed;           // floats: reduced statistics of all systems (+ the <dY, C> sums)
  size_t ws_total_bytes;
};

// arguments of the per-head core adjoint when it rides along with the token-backward launch
struct CoreAdjoint {
  const float* base_raw;
  const float* hmat;
  const float* de_sys;
  float* d_base;
  float* d_eta_raw;
  float grad_scale;
};

// ---------------------------------------------------------------------------------------
// chained launches (programmatic dependent launch)
// ---------------------------------------------------------------------------------------
// While this flag is set on the calling thread, launch_kernel() lets the new grid start as soon as
// every block of the previous kernel in the stream has passed grid_launch_dependents(): its blocks
// become resident and set up their shared memory while the previous grid drains.  Every kernel of this
// library calls grid_dependency_wait() before its first access to global memory; that call returns
// once the previous grid has completed and its writes are visible (at once for a normal launch).
// The statistics and compact kernels signal after their main loop: signalling at the start of the
// kernel parks the next grid's blocks on the SMs for the whole kernel and measured slower than no
// chaining at all (189 us against 179 us for the six launches at 32768 tokens; 174 us signalling late).
// Only the second and third launch of ms_mix_forward / ms_mix_backward are chained, so the kernel
// ahead of a chained launch is always one of this library's (chaining the first launch to the
// caller's kernel ahead of it measured no gain).
extern thread_local bool g_chain_launches;
struct ChainScope {
  bool before;
  explicit ChainScope(bool on) : before(g_chain_launches) { g_chain_launches = on; }
  ~ChainScope() { g_chain_launches = before; }
};
bool chaining_allowed();   // false when the environment sets MEMSOLVE_NO_CHAIN=1

template <typename... Expected, typename... Actual>
inline void launch_kernel(void (*kernel)(Expected...), dim3 grid, dim3 block, size_t smem_bytes, cudaStream_t st,
                          Actual&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem_bytes;
  config.stream = st;
  cudaLaunchAttribute chain;
  chain.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  chain.val.programmaticStreamSerializationAllowed = 1;
  if (g_chain_launches) {
    config.attrs = &chain;
    config.numAttrs = 1;
  }
  cudaLaunchKernelEx(&config, kernel, std::forward<Actual>(args)...);
}

Plan make_plan(const ms_shape& s);
// the plan with the chunking of the adjoint reduction in `chunks` / `chunk_tokens`: what the adjoint
// statistics, their pack / exchange and the compact backward take
inline Plan backward_plan(Plan p) {
  p.chunks = p.chunks_bwd;
  p.chunk_tokens = p.chunk_tokens_bwd;
  return p;
}
int check_shape(const ms_shape* s);
int sm_count();
int ensure_dynamic_smem(const void* kernel, int bytes);

// ---------------------------------------------------------------------------------------
// shared-memory addressing
// ---------------------------------------------------------------------------------------
// XOR the 16-byte-chunk bits [4,7) of a byte offset with bits [7,10): conflict-free ldmatrix
// for densely packed rows of 32/64/128 bytes.
// see launch_kernel(): both are no-ops for a grid that was launched the normal way
__device__ __forceinline__ void grid_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ uint32_t swz(uint32_t off) { return off ^ (((off >> 7) & 7u) << 4); }

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void st_shared_u16(uint32_t addr, unsigned short v) {
  asm volatile("st.shared.u16 [%0], %1;\n" ::"r"(addr), "h"(v));
}
__device__ __forceinline__ void st_shared_u32(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(addr), "r"(v));
}
__device__ __forceinline__ void st_shared_f32(uint32_t addr, float v) {
  asm volatile("st.shared.f32 [%0], %1;\n" ::"r"(addr), "f"(v));
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w));
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t ld_shared_u32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ float4 ld_shared_f4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];\n"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(addr));
  return v;
}

// Copy a [tile_rows x tile_cols] BF16 tile (tile_cols a multiple of 8, row pitch tile_cols*2
// bytes, swizzled) from global rows `src + row*stride`.  Rows >= rows_valid and columns >= cols_valid
// become zero.  ALIGNED: 16-byte cp.async (caller commits); otherwise synchronous 2-byte loads.
template <bool ALIGNED>
__device__ __forceinline__ void load_tile_bf16(uint32_t tile, int tile_rows, int tile_cols,
                                               const __nv_bfloat16* __restrict__ src, long stride,
                                               int rows_valid, int cols_valid, int tid,
                                               int nthreads) {
  const int pitch = tile_cols * 2;
  if (ALIGNED) {
    const int cpr = tile_cols >> 3;  // 16-byte chunks per row
    for (int i = tid; i < tile_rows * cpr; i += nthreads) {
      int row = i / cpr, c = i - row * cpr;
      bool ok = row < rows_valid && c * 8 < cols_valid;
      const __nv_bfloat16* g = ok ? src + (long)row * stride + c * 8 : src;
      cp_async16(tile + swz(row * pitch + c * 16), g, ok);
    }
  } else {
    const unsigned short* s16 = reinterpret_cast<const unsigned short*>(src);
    for (int i = tid; i < tile_rows * tile_cols; i += nthreads) {
      int row = i / tile_cols, c = i - row * tile_cols;
      unsigned short v = 0;
      if (row < rows_valid && c < cols_valid) v = __ldg(s16 + (long)row * stride + c);
      st_shared_u16(tile + swz(row * pitch + c * 2), v);
    }
  }
}

// Copy a [64 x 32] FP32 table tile (row pitch 128 bytes, not swizzled).
template <bool ALIGNED>
__device__ __forceinline__ void load_tile_f32(uint32_t tile, const float* __restrict__ src,
                                              long stride, int rows_valid, int cols_valid, int tid,
                                              int nthreads) {
  if (ALIGNED) {
    for (int i = tid; i < kTileTokens * 8; i += nthreads) {
      int row = i >> 3, c = i & 7;
      bool ok = row < rows_valid && c * 4 < cols_valid;
      const float* g = ok ? src + (long)row * stride + c * 4 : src;
      cp_async16(tile + row * 128 + c * 16, g, ok);
    }
  } else {
    for (int i = tid; i < kTileTokens * 32; i += nthreads) {
      int row = i >> 5, c = i & 31;
      float v = 0.f;
      if (row < rows_valid && c < cols_valid) v = __ldg(src + (long)row * stride + c);
      st_shared_f32(tile + row * 128 + c * 4, v);
    }
  }
}

// ---------------------------------------------------------------------------------------
// tensor-core fragments (mma.sync.m16n8k16, BF16 x BF16 -> FP32)
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// ---------------------------------------------------------------------------------------
// BF16 words
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float2 bf2_to_f2(uint32_t w) {
  // a BF16 is the upper half of an FP32
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
__device__ __forceinline__ uint32_t f2_to_bf2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// x = hi + lo with hi = bf16(x), lo = bf16(x - hi)  (two-word split of an FP32 value)
__device__ __forceinline__ void split2(float x0, float x1, uint32_t& hi, uint32_t& lo) {
  hi = f2_to_bf2(x0, x1);
  float2 h = bf2_to_f2(hi);
  lo = f2_to_bf2(x0 - h.x, x1 - h.y);
}

// planar rotation of one adjacent channel pair; inverse flips the sine
__device__ __forceinline__ float2 rot_pair(float ev, float od, float c, float s) {
  return make_float2(fmaf(ev, c, -(od * s)), fmaf(ev, s, od * c));
}

// 1/sqrt(n) and 1/n with IEEE rounding
__device__ __forceinline__ float inv_sqrt_rn(float n) { return __fdiv_rn(1.0f, __fsqrt_rn(n)); }
__device__ __forceinline__ float inv_rn(float n) { return __fdiv_rn(1.0f, n); }

}  // namespace ms
