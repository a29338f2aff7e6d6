// Projection GEMM on the fifth-generation tensor cores with the reference's epilogue fused:
//
//   out[m, n] = output_mask[m] ? (input_mask[m] ? sum_k x[m, k] w[n, k] : 0) + bias[n] : 0        (one BF16 rounding)
//
// BF16 x BF16 products accumulated in FP32, FP32 bias, masked input rows contribute nothing (whatever they
// hold, NaN included), masked output rows are exactly zero: the contract of the reference's `_biased_gemm` /
// `_wide_gemm` (memsolve/ball/cuda.py:418-708), which builds it from a Triton GEMM.  Here: one persistent
// CTA per SM walks over 128 x BN output tiles;
//
//   warp 4 (one thread)  TMA: x tile [128 x 64] and weight tile [BN x 64] per k-block into a ring of stages
//                        (128-byte swizzle; both operands have the contraction index contiguous)
//   warp 5               tcgen05.mma issue, accumulator [128 x BN] FP32 in tensor memory, two accumulators so
//                        that the epilogue of a tile overlaps the MMAs of the next; stages go back to the TMA
//                        warp by tcgen05.commit
//   warps 0-3            epilogue: one output row per thread; tcgen05.ld, mask / bias, BF16, 64-column chunks
//                        through two staging tiles and a TMA store
//
// Shapes: in_features a multiple of 64, out_features a multiple of 128; any number of rows.  Every wait is
// bounded; a timeout sets the device error word and the CTA drains.
#include "ms_tc.cuh"

namespace ms {

constexpr int kLinThreads = 192;

template <int BN>
struct LinearTcCfg {
  static constexpr int A_TILE = 128 * 128;            // 128 rows x 64 BF16
  static constexpr int B_TILE = BN * 128;
  static constexpr int STAGE = A_TILE + B_TILE;
  static constexpr int STAGES = BN == 256 ? 4 : (BN == 192 ? 4 : 6);
  static constexpr int OUT_TILE = 128 * 128;          // 128 rows x 64 BF16 of output
  static constexpr int BAR_BYTES = (2 * STAGES + 4) * 8 + 16;
  static constexpr int TOTAL = 1024 + STAGES * STAGE + 2 * OUT_TILE + BN * 4 + BAR_BYTES;
  static constexpr int TMEM_COLS = BN <= 128 ? 256 : 512;
  static_assert(TOTAL <= 227 * 1024, "shared memory");
};

struct LinearTcParams {
  const float* bias;
  const unsigned char* input_mask;
  const unsigned char* output_mask;
  int* error;
  int rows, k_blocks, m_tiles, n_tiles;
};

__device__ __forceinline__ void lin_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool lin_wait(uint32_t bar, uint32_t parity) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity));
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int c0, int c1, uint32_t src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];\n" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(c0), "r"(c1), "r"(src)
               : "memory");
}

// BNM: the second operand is stored [k][n] with n contiguous (the input-gradient product dY W, W = [out, in]):
// its tile is BN / 64 boxes of 64 k-rows x 64 columns, read by the MMA as an N-major operand.
template <int BN, bool BNM>
__global__ void __launch_bounds__(kLinThreads, 1)
linear_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                 const __grid_constant__ CUtensorMap map_out, const LinearTcParams p) {
  using Cfg = LinearTcCfg<BN>;
  constexpr int S = Cfg::STAGES;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t smem = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t ring = smem;
  const uint32_t out_buf = ring + S * Cfg::STAGE;
  const uint32_t bias_buf = out_buf + 2 * Cfg::OUT_TILE;
  const uint32_t bar_full = bias_buf + BN * 4;
  const uint32_t bar_empty = bar_full + 8 * S;
  const uint32_t bar_acc_full = bar_empty + 8 * S;    // two
  const uint32_t bar_acc_empty = bar_acc_full + 16;   // two
  const uint32_t tslot = bar_acc_empty + 16;

  if (tid == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(bar_full + 8 * i, 1);
      mbar_init(bar_empty + 8 * i, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_acc_full + 8 * i, 1);
      mbar_init(bar_acc_empty + 8 * i, 128);
    }
    mbar_fence_init();
  }
  __syncthreads();
  if (warp == 5) tc::tmem_alloc(tslot, Cfg::TMEM_COLS);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = ld_shared_u32(tslot);
  grid_dependency_wait();

  const int total = p.m_tiles * p.n_tiles;
  bool ok = true;

  if (warp == 4) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int it = 0;
      for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
        const int m = t / p.n_tiles, n = t - m * p.n_tiles;
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const int s = it % S;
          if (it >= S) {
            ok = mbar_wait(bar_empty + 8 * s, ((it / S) - 1) & 1);
            if (!ok) break;
          }
          const uint32_t st = ring + s * Cfg::STAGE, bar = bar_full + 8 * s;
          mbar_expect_tx(bar, Cfg::STAGE);
          tma_load_2d(st, &map_x, kb * 64, m * 128, bar);
          if (BNM) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(st + Cfg::A_TILE + j * 8192, &map_w, n * BN + j * 64, kb * 64, bar);
          } else {
            tma_load_2d(st + Cfg::A_TILE, &map_w, kb * 64, n * BN, bar);
          }
        }
      }
      if (!ok) atomicExch(p.error, kErrBarrierTimeout);
    }
  } else if (warp == 5) {
    // ---------------------------------------------------------------- MMA issuer
    constexpr uint32_t IDESC = tc::idesc_bf16(128, BN, BNM);
    constexpr uint32_t HI = tc::desc_hi_k_major(128);
    constexpr uint32_t HI_B = BNM ? tc::desc_hi_n_major_128() : HI;
    // N-major tile: 8192 bytes between its 64-column blocks, 16 k-rows (2048 bytes) per MMA
    constexpr uint32_t B_FIX = BNM ? (((8192u >> 4) << 16) - (1u << 16)) : 0u;
    constexpr uint32_t B_STEP = BNM ? 128u : 2u;
    const uint32_t ring_lo = tc::desc_lo_k_major(ring);
    int it = 0, local = 0;
    for (int t = blockIdx.x; t < total && ok; t += gridDim.x, ++local) {
      const int buf = local & 1;
      if (local >= 2) {
        ok = lin_wait(bar_acc_empty + 8 * buf, ((local >> 1) - 1) & 1);
        if (!ok) break;
      }
      const uint32_t d = tmem + buf * (Cfg::TMEM_COLS / 2);
      for (int kb = 0; kb < p.k_blocks && ok; ++kb, ++it) {
        const int s = it % S;
        ok = lin_wait(bar_full + 8 * s, (it / S) & 1);
        if (!ok) break;
        tc::fence_after_sync();
        const uint32_t a_lo = ring_lo + (uint32_t)(s * (Cfg::STAGE >> 4)), b_lo = a_lo + (Cfg::A_TILE >> 4) + B_FIX;
        if (tc::elect_one()) {
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            tc::mma_ss_raw<HI, HI_B, IDESC>(d, a_lo + ks * 2, b_lo + ks * B_STEP, (kb | ks) != 0);
          tc::mma_commit_raw(bar_empty + 8 * s);
          if (kb == p.k_blocks - 1) tc::mma_commit_raw(bar_acc_full + 8 * buf);
        }
        __syncwarp();
      }
    }
    if (!ok && lane == 0) atomicExch(p.error, kErrBarrierTimeout);
  } else {
    // ---------------------------------------------------------------- epilogue: one output row per thread
    const int row = warp * 32 + lane;
    const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
    int local = 0, chunk_no = 0;
    for (int t = blockIdx.x; t < total && ok; t += gridDim.x, ++local) {
      const int m = t / p.n_tiles, n = t - m * p.n_tiles, buf = local & 1;
      const int grow = m * 128 + row;
      const bool in_range = grow < p.rows;
      const bool keep_in = !p.input_mask || (in_range && p.input_mask[grow] != 0);
      const bool keep_out = !p.output_mask || (in_range && p.output_mask[grow] != 0);
      // this tile's bias columns (all four warps read them below)
      asm volatile("bar.sync 1, 128;\n" ::: "memory");
      for (int c = tid; c < BN; c += 128) st_shared_f32(bias_buf + 4 * c, p.bias ? __ldg(p.bias + n * BN + c) : 0.f);
      asm volatile("bar.sync 1, 128;\n" ::: "memory");
      ok = lin_wait(bar_acc_full + 8 * buf, (local >> 1) & 1);
      if (!ok) break;
      tc::fence_after_sync();
#pragma unroll 1
      for (int c64 = 0; c64 < BN / 64; ++c64, ++chunk_no) {
        const uint32_t stage_tile = out_buf + (chunk_no & 1) * Cfg::OUT_TILE;
        uint32_t acc[64];
#pragma unroll
        for (int q = 0; q < 4; ++q)
          tc::tmem_ld16(lane_base + buf * (Cfg::TMEM_COLS / 2) + c64 * 64 + q * 16, *reinterpret_cast<uint32_t(*)[16]>(&acc[q * 16]));
        tc::wait_ld();
        if (c64 == BN / 64 - 1) {
          tc::fence_before_sync();
          lin_arrive(bar_acc_empty + 8 * buf);   // the accumulator is in registers
        }
        // the staging tile was handed to a TMA store two chunks ago: its reads must have completed
        if (tid == 0) tma_store_wait_read<1>();
        asm volatile("bar.sync 1, 128;\n" ::: "memory");
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          uint32_t ow[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int col = ch * 8 + 2 * k;
            float v0 = keep_in ? __uint_as_float(acc[col]) : 0.f, v1 = keep_in ? __uint_as_float(acc[col + 1]) : 0.f;
            float b0, b1;
            asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];\n" : "=f"(b0), "=f"(b1) : "r"(bias_buf + 4 * (c64 * 64 + col)));
            v0 = keep_out ? v0 + b0 : 0.f;
            v1 = keep_out ? v1 + b1 : 0.f;
            ow[k] = f2_to_bf2(v0, v1);
          }
          st_shared_v4(stage_tile + row * 128 + ((ch ^ (row & 7)) << 4), make_uint4(ow[0], ow[1], ow[2], ow[3]));
        }
        fence_async_shared();
        asm volatile("bar.sync 1, 128;\n" ::: "memory");
        if (tid == 0) {
          tma_store_2d(&map_out, n * BN + c64 * 64, m * 128, stage_tile);
          tma_store_commit();
        }
      }
    }
    if (tid == 0) tma_store_wait_all<0>();
    if (!ok && lane == 0) atomicExch(p.error, kErrBarrierTimeout);
  }

  tc::fence_before_sync();
  __syncthreads();
  if (warp == 5) tc::tmem_free(tmem, Cfg::TMEM_COLS);
}

// BNM false: out[rows, out_features] = x[rows, in_features] weight[out_features, in_features]^T
// BNM true:  out[rows, out_features] = x[rows, in_features] weight[in_features, out_features]
template <int BN, bool BNM>
static int launch_linear_tc_bn(long rows, int in_features, int out_features, const void* x, const void* weight,
                               const float* bias, const unsigned char* input_mask, const unsigned char* output_mask,
                               void* out, cudaStream_t st) {
  using Cfg = LinearTcCfg<BN>;
  CUtensorMap map_x, map_w, map_out;
  {
    const uint64_t dims[2] = {(uint64_t)in_features, (uint64_t)rows};
    const uint64_t str[1] = {(uint64_t)in_features * 2};
    const uint32_t box[2] = {64, 128};
    if (encode_tensor_map(&map_x, const_cast<void*>(x), 2, 2, dims, str, box, Swizzle::B128)) return MS_ERR_LAUNCH;
  }
  if (BNM) {
    const uint64_t dims[2] = {(uint64_t)out_features, (uint64_t)in_features};
    const uint64_t str[1] = {(uint64_t)out_features * 2};
    const uint32_t box[2] = {64, 64};
    if (encode_tensor_map(&map_w, const_cast<void*>(weight), 2, 2, dims, str, box, Swizzle::B128)) return MS_ERR_LAUNCH;
  } else {
    const uint64_t dims[2] = {(uint64_t)in_features, (uint64_t)out_features};
    const uint64_t str[1] = {(uint64_t)in_features * 2};
    const uint32_t box[2] = {64, (uint32_t)BN};
    if (encode_tensor_map(&map_w, const_cast<void*>(weight), 2, 2, dims, str, box, Swizzle::B128)) return MS_ERR_LAUNCH;
  }
  {
    const uint64_t dims[2] = {(uint64_t)out_features, (uint64_t)rows};
    const uint64_t str[1] = {(uint64_t)out_features * 2};
    const uint32_t box[2] = {64, 128};
    if (encode_tensor_map(&map_out, out, 2, 2, dims, str, box, Swizzle::B128)) return MS_ERR_LAUNCH;
  }
  LinearTcParams p;
  p.bias = bias; p.input_mask = input_mask; p.output_mask = output_mask;
  p.error = device_error_word();
  if (!p.error) return MS_ERR_LAUNCH;
  p.rows = (int)rows; p.k_blocks = in_features / 64;
  p.m_tiles = (int)((rows + 127) / 128); p.n_tiles = out_features / BN;
  const long total = (long)p.m_tiles * p.n_tiles;
  long ctas = sm_count();
  if (ctas > total) ctas = total;
  auto kern = linear_tc_kernel<BN, BNM>;
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(kern), Cfg::TOTAL)) return MS_ERR_LAUNCH;
  launch_kernel(kern, dim3((unsigned)ctas), dim3(kLinThreads), Cfg::TOTAL, st, map_x, map_w, map_out, p);
  return cudaGetLastError() == cudaSuccess ? MS_OK : MS_ERR_LAUNCH;
}

// MS_OK / error, or -1 when the shape is outside this kernel's envelope.
int launch_linear_tc(long rows, int in_features, int out_features, const void* x, const void* weight, const float* bias,
                     const unsigned char* input_mask, const unsigned char* output_mask, void* out, cudaStream_t st) {
  if (rows <= 0 || rows > 0x7fffff00L || in_features <= 0 || (in_features % 64) != 0 || (out_features % 128) != 0) return -1;
  if (((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(out)) & 15u) != 0)
    return -1;
  if (out_features % 256 == 0)
    return launch_linear_tc_bn<256, false>(rows, in_features, out_features, x, weight, bias, input_mask, output_mask, out, st);
  if (out_features % 192 == 0)
    return launch_linear_tc_bn<192, false>(rows, in_features, out_features, x, weight, bias, input_mask, output_mask, out, st);
  return launch_linear_tc_bn<128, false>(rows, in_features, out_features, x, weight, bias, input_mask, output_mask, out, st);
}

// dx[rows, in_features] = row masks * (dy[rows, out_features] weight[out_features, in_features]), one BF16 rounding: the
// input gradient of the projection (memsolve/ball/cuda.py:959-1041).  A row is zero when either mask clears it (a
// cleared output row had no influence on the loss, a cleared input row was not read).  MS_OK / error, or -1 outside
// the envelope (out_features a multiple of 64, in_features a multiple of 128, 16-byte aligned pointers).
int launch_linear_input_grad_tc(long rows, int in_features, int out_features, const void* dy, const void* weight,
                                const unsigned char* input_mask, const unsigned char* output_mask, void* dx,
                                cudaStream_t st) {
  if (rows <= 0 || rows > 0x7fffff00L || out_features <= 0 || (out_features % 64) != 0 || (in_features % 128) != 0) return -1;
  if (((reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(dx)) & 15u) != 0)
    return -1;
  // the contraction runs over out_features, the result has in_features columns
  if (in_features % 256 == 0)
    return launch_linear_tc_bn<256, true>(rows, out_features, in_features, dy, weight, nullptr, input_mask, output_mask, dx, st);
  if (in_features % 192 == 0)
    return launch_linear_tc_bn<192, true>(rows, out_features, in_features, dy, weight, nullptr, input_mask, output_mask, dx, st);
  return launch_linear_tc_bn<128, true>(rows, out_features, in_features, dy, weight, nullptr, input_mask, output_mask, dx, st);
}

}  // namespace ms
