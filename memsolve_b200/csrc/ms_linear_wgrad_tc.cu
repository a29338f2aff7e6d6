// Weight and bias gradients of a projection on the fifth-generation tensor cores:
//
//   dW[o, i] = sum_m dy[m, o] x[m, i]        db[o] = sum_m dy[m, o]        (BF16 operands, FP32 sums, FP32 results)
//
// the reference's fused dW + db GEMM (csrc/ball/binding.cpp:114-196, memsolve/ball/cuda.py:959-1041).  The
// contraction runs over the rows (tokens), so both operands are read with the contraction index strided: 64-row boxes
// of dy and x land in shared memory by TMA (128-byte swizzle) and enter tcgen05.mma as M-major / N-major operands.
// The result is small (out x in) and the contraction long, so the rows are split over `splits` CTAs per 128 x BN tile:
//
//   warp 4 (one thread)  TMA producer: per 64-row block one stage = dy [64 x 128] + x [64 x BN]
//   warp 5               MMA issue: accumulator [128 x BN] FP32 in tensor memory
//   warps 0-3            while the MMAs run: column sums of the dy boxes (db) in the CTAs of the first column tile;
//                        afterwards: accumulator -> partial tile in global memory; the CTA that finishes a tile last
//                        adds the partial tiles in split order (so the sum does not depend on which CTA that is) and
//                        writes dW / db
//
// No CTA waits for another one; every wait inside a CTA is bounded.  Row masks are not handled here (the caller
// falls back to separate passes when a projection has them).
#include "ms_tc.cuh"

namespace ms {

constexpr int kWgThreads = 192;

template <int BN>
struct WgradTcCfg {
  static constexpr int A_TILE = 2 * 8192;             // 64 rows x 128 dy columns
  static constexpr int B_TILE = (BN / 64) * 8192;     // 64 rows x BN x columns
  static constexpr int STAGE = A_TILE + B_TILE;
  static constexpr int STAGES = BN == 256 ? 4 : 6;
  static constexpr int BAR_BYTES = (2 * STAGES + 1) * 8 + 16;
  static constexpr int TOTAL = 1024 + STAGES * STAGE + 4 * 128 * 4 + BAR_BYTES;
  static constexpr int TMEM_COLS = BN;
  static_assert(TOTAL <= 227 * 1024, "shared memory");
};

struct WgradTcParams {
  float* dw;            // [out, in]
  float* db;            // [out] or null
  float* partial;       // [tiles][splits][BN / 4][128][4]
  float* db_partial;    // [o_tiles][splits][128]
  unsigned int* counters;   // [tiles], zero on entry
  int* error;
  int rows, in_features, out_features, i_tiles, splits, k_blocks;
};

__device__ __forceinline__ void wg_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ float wg_ld_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ bool wg_wait(uint32_t bar, uint32_t parity) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity));
}

template <int BN>
__global__ void __launch_bounds__(kWgThreads, 1)
linear_wgrad_tc_kernel(const __grid_constant__ CUtensorMap map_dy, const __grid_constant__ CUtensorMap map_x,
                       const WgradTcParams p) {
  using Cfg = WgradTcCfg<BN>;
  constexpr int S = Cfg::STAGES;
  extern __shared__ unsigned char smem_raw[];
  __shared__ int s_last;
  const uint32_t smem = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t ring = smem;
  const uint32_t db_red = ring + S * Cfg::STAGE;       // [4 warps][128] floats
  const uint32_t bar_full = db_red + 4 * 128 * 4;
  const uint32_t bar_empty = bar_full + 8 * S;
  const uint32_t bar_acc = bar_empty + 8 * S;
  const uint32_t tslot = bar_acc + 8;

  const int tile = blockIdx.x / p.splits, split = blockIdx.x - tile * p.splits;
  const int o_tile = tile / p.i_tiles, i_tile = tile - o_tile * p.i_tiles;
  const bool do_db = p.db != nullptr && i_tile == 0;
  const int per = (p.k_blocks + p.splits - 1) / p.splits;
  const int kb0 = min(p.k_blocks, split * per), kb1 = min(p.k_blocks, kb0 + per);
  const int n_kb = kb1 - kb0;

  if (tid == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(bar_full + 8 * i, 1);
      mbar_init(bar_empty + 8 * i, do_db ? 5 : 1);
    }
    mbar_init(bar_acc, 1);
    mbar_fence_init();
  }
  __syncthreads();
  if (warp == 5) tc::tmem_alloc(tslot, Cfg::TMEM_COLS);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = ld_shared_u32(tslot);
  grid_dependency_wait();
  bool ok = true;

  if (warp == 4) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      for (int it = 0; it < n_kb; ++it) {
        const int s = it % S;
        if (it >= S) {
          ok = mbar_wait(bar_empty + 8 * s, ((it / S) - 1) & 1);
          if (!ok) break;
        }
        const uint32_t st = ring + s * Cfg::STAGE, bar = bar_full + 8 * s;
        const int row0 = (kb0 + it) * 64;
        mbar_expect_tx(bar, Cfg::STAGE);
#pragma unroll
        for (int j = 0; j < 2; ++j) tma_load_2d(st + j * 8192, &map_dy, o_tile * 128 + j * 64, row0, bar);
#pragma unroll
        for (int j = 0; j < BN / 64; ++j)
          tma_load_2d(st + Cfg::A_TILE + j * 8192, &map_x, i_tile * BN + j * 64, row0, bar);
      }
      if (!ok) atomicExch(p.error, kErrBarrierTimeout);
    }
  } else if (warp == 5) {
    // ---------------------------------------------------------------- MMA issuer
    constexpr uint32_t IDESC = tc::idesc_bf16(128, BN, true, true);
    constexpr uint32_t HI = tc::desc_hi_n_major_128();
    // both tiles: 64-column blocks 8192 bytes apart, 16 rows (2048 bytes) per MMA
    const uint32_t ring_lo = ((ring & 0x3ffffu) >> 4) | ((8192u >> 4) << 16);
    for (int it = 0; it < n_kb && ok; ++it) {
      const int s = it % S;
      ok = wg_wait(bar_full + 8 * s, (it / S) & 1);
      if (!ok) break;
      tc::fence_after_sync();
      const uint32_t a_lo = ring_lo + (uint32_t)(s * (Cfg::STAGE >> 4)), b_lo = a_lo + (Cfg::A_TILE >> 4);
      if (tc::elect_one()) {
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) tc::mma_ss_raw<HI, HI, IDESC>(tmem, a_lo + ks * 128, b_lo + ks * 128, (it | ks) != 0);
        tc::mma_commit_raw(bar_empty + 8 * s);
      }
      __syncwarp();
    }
    if (ok) {
      if (tc::elect_one()) tc::mma_commit_raw(bar_acc);
      __syncwarp();
    }
    if (!ok && lane == 0) atomicExch(p.error, kErrBarrierTimeout);
  } else {
    // ---------------------------------------------------------------- column sums, then the accumulator
    if (do_db) {
      // warp w: rows 16 w .. 16 w + 15 of every 64-row box; lane l: dy columns 4 l .. 4 l + 3 of the tile
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      const uint32_t col_off = (uint32_t)(lane >> 4) * 8192u;
      const int chunk = (lane & 15) >> 1;
      const uint32_t within = (uint32_t)(lane & 1) * 8u;
      for (int it = 0; it < n_kb && ok; ++it) {
        const int s = it % S;
        ok = wg_wait(bar_full + 8 * s, (it / S) & 1);
        if (!ok) break;
        const uint32_t base = ring + s * Cfg::STAGE + col_off;
#pragma unroll
        for (int rr = 0; rr < 16; ++rr) {
          const int r = warp * 16 + rr;
          uint32_t w0, w1;
          asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];\n"
                       : "=r"(w0), "=r"(w1)
                       : "r"(base + r * 128 + ((uint32_t)(chunk ^ (r & 7)) << 4) + within));
          const float2 f0 = bf2_to_f2(w0), f1 = bf2_to_f2(w1);
          acc[0] += f0.x; acc[1] += f0.y; acc[2] += f1.x; acc[3] += f1.y;
        }
        __syncwarp();
        if (lane == 0) wg_arrive(bar_empty + 8 * s);
      }
      asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};\n" ::"r"(db_red + (uint32_t)(warp * 128 + 4 * lane) * 4u),
                   "f"(acc[0]), "f"(acc[1]), "f"(acc[2]), "f"(acc[3])
                   : "memory");
    }
    asm volatile("bar.sync 1, 128;\n" ::: "memory");
    const int o_local = warp * 32 + lane;
    const size_t pidx = (size_t)tile * p.splits + split;
    float* part = p.partial + pidx * (size_t)(128 * BN);
    const bool single = p.splits == 1;
    if (do_db) {
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) v += wg_ld_f32(db_red + (uint32_t)(w * 128 + o_local) * 4u);
      if (single) p.db[o_tile * 128 + o_local] = v;
      else p.db_partial[((size_t)o_tile * p.splits + split) * 128 + o_local] = v;
    }
    if (n_kb > 0 && ok) ok = wg_wait(bar_acc, 0);
    tc::fence_after_sync();
    const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
#pragma unroll 1
    for (int c16 = 0; c16 < BN / 16; ++c16) {
      uint32_t v[16];
      if (n_kb > 0 && ok) {
        tc::tmem_ld16(lane_base + c16 * 16, v);
        tc::wait_ld();
      } else {
#pragma unroll
        for (int e = 0; e < 16; ++e) v[e] = 0u;
      }
      if (single) {
        float* dst = p.dw + (size_t)(o_tile * 128 + o_local) * p.in_features + i_tile * BN + c16 * 16;
#pragma unroll
        for (int q = 0; q < 4; ++q)
          *reinterpret_cast<uint4*>(dst + 4 * q) = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
      } else {
        // partial tile as [column / 4][row][4]: the threads of a warp write 512 contiguous bytes
#pragma unroll
        for (int q = 0; q < 4; ++q)
          *reinterpret_cast<uint4*>(part + ((size_t)(c16 * 4 + q) * 128 + o_local) * 4) =
              make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
      }
    }
    if (!single) {
      __threadfence();
      asm volatile("bar.sync 1, 128;\n" ::: "memory");
      if (tid == 0) s_last = atomicAdd(p.counters + tile, 1u) == (unsigned)(p.splits - 1);
      asm volatile("bar.sync 1, 128;\n" ::: "memory");
      if (s_last) {
        __threadfence();
        const float* first = p.partial + (size_t)tile * p.splits * (size_t)(128 * BN);
#pragma unroll 1
        for (int c4 = 0; c4 < BN / 4; ++c4) {
          float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int sp = 0; sp < p.splits; ++sp) {
            const float4 t = __ldcg(reinterpret_cast<const float4*>(first + (size_t)sp * (128 * BN) +
                                                                    ((size_t)c4 * 128 + o_local) * 4));
            sum.x += t.x; sum.y += t.y; sum.z += t.z; sum.w += t.w;
          }
          *reinterpret_cast<float4*>(p.dw + (size_t)(o_tile * 128 + o_local) * p.in_features + i_tile * BN + c4 * 4) = sum;
        }
        if (do_db) {
          float v = 0.f;
          for (int sp = 0; sp < p.splits; ++sp) v += __ldcg(p.db_partial + ((size_t)o_tile * p.splits + sp) * 128 + o_local);
          p.db[o_tile * 128 + o_local] = v;
        }
      }
    }
    if (!ok && lane == 0) atomicExch(p.error, kErrBarrierTimeout);
  }

  tc::fence_before_sync();
  __syncthreads();
  if (warp == 5) tc::tmem_free(tmem, Cfg::TMEM_COLS);
}

static int wgrad_splits(int tiles, int k_blocks) {
  int splits = sm_count() / tiles;
  if (splits < 1) splits = 1;
  if (splits > k_blocks) splits = k_blocks > 0 ? k_blocks : 1;
  return splits;
}

// bytes of scratch ms_linear_weight_grad needs for this shape (0 outside the kernel's envelope)
size_t linear_wgrad_workspace_bytes(long rows, int in_features, int out_features) {
  if (rows <= 0 || (out_features % 128) != 0 || (in_features % 128) != 0) return 0;
  const int bn = in_features % 256 == 0 ? 256 : 128;
  const int tiles = (out_features / 128) * (in_features / bn);
  const int k_blocks = (int)((rows + 63) / 64);
  const int splits = wgrad_splits(tiles, k_blocks);
  const size_t counters = ((size_t)tiles * 4 + 255) & ~size_t(255);
  return counters + (size_t)tiles * splits * 128 * bn * 4 + (size_t)(out_features / 128) * splits * 128 * 4;
}

template <int BN>
static int launch_wgrad_bn(long rows, int in_features, int out_features, const void* x, const void* dy, float* dw, float* db,
                           void* workspace, cudaStream_t st) {
  using Cfg = WgradTcCfg<BN>;
  CUtensorMap map_dy, map_x;
  {
    const uint64_t dims[2] = {(uint64_t)out_features, (uint64_t)rows};
    const uint64_t str[1] = {(uint64_t)out_features * 2};
    const uint32_t box[2] = {64, 64};
    if (encode_tensor_map(&map_dy, const_cast<void*>(dy), 2, 2, dims, str, box, Swizzle::B128)) return MS_ERR_LAUNCH;
  }
  {
    const uint64_t dims[2] = {(uint64_t)in_features, (uint64_t)rows};
    const uint64_t str[1] = {(uint64_t)in_features * 2};
    const uint32_t box[2] = {64, 64};
    if (encode_tensor_map(&map_x, const_cast<void*>(x), 2, 2, dims, str, box, Swizzle::B128)) return MS_ERR_LAUNCH;
  }
  WgradTcParams p;
  p.dw = dw; p.db = db;
  p.rows = (int)rows; p.in_features = in_features; p.out_features = out_features;
  p.i_tiles = in_features / BN;
  const int tiles = (out_features / 128) * p.i_tiles;
  p.k_blocks = (int)((rows + 63) / 64);
  p.splits = wgrad_splits(tiles, p.k_blocks);
  const size_t counters = ((size_t)tiles * 4 + 255) & ~size_t(255);
  p.counters = static_cast<unsigned int*>(workspace);
  p.partial = reinterpret_cast<float*>(static_cast<unsigned char*>(workspace) + counters);
  p.db_partial = p.partial + (size_t)tiles * p.splits * 128 * BN;
  p.error = device_error_word();
  if (!p.error) return MS_ERR_LAUNCH;
  if (cudaMemsetAsync(workspace, 0, counters, st) != cudaSuccess) return MS_ERR_LAUNCH;
  auto kern = linear_wgrad_tc_kernel<BN>;
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(kern), Cfg::TOTAL)) return MS_ERR_LAUNCH;
  launch_kernel(kern, dim3((unsigned)(tiles * p.splits)), dim3(kWgThreads), Cfg::TOTAL, st, map_dy, map_x, p);
  return cudaGetLastError() == cudaSuccess ? MS_OK : MS_ERR_LAUNCH;
}

// MS_OK / error, or -1 when the shape is outside this kernel's envelope.
int launch_linear_wgrad_tc(long rows, int in_features, int out_features, const void* x, const void* dy, float* dw, float* db,
                           void* workspace, size_t workspace_bytes, cudaStream_t st) {
  if (rows <= 0 || rows > 0x7fffff00L || (out_features % 128) != 0 || (in_features % 128) != 0) return -1;
  if (((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(dw) |
        reinterpret_cast<uintptr_t>(workspace)) & 15u) != 0)
    return -1;
  if (!workspace || workspace_bytes < linear_wgrad_workspace_bytes(rows, in_features, out_features)) return MS_ERR_WORKSPACE;
  if (in_features % 256 == 0) return launch_wgrad_bn<256>(rows, in_features, out_features, x, dy, dw, db, workspace, st);
  return launch_wgrad_bn<128>(rows, in_features, out_features, x, dy, dw, db, workspace, st);
}

}  // namespace ms
