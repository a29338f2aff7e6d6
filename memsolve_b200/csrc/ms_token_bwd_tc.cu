// Token backward on the fifth-generation tensor cores (tcgen05), for long sequences: head dimension 64,
// rank 16/32/64, aligned pointers, at least kTcMinTokens tokens per sample (other shapes take the
// mma.sync kernels in ms_token_bwd_tma.cu / ms_token.cu).
//
//   dA = s*( A_raw S' + rot(dY) W^T + rot(C) dQ^T ),   S' = s (dG + dG^T),   dC = eta*dY + s*rot^-1(A_raw dQ)
//
// Same arithmetic as the reference's `_token_backward` (memsolve/ball/cuda.py:1767-1922): FP32 rotation,
// rotated operands and the compact matrices W, dQ, S' carried as two BF16 words each, products of the
// words accumulated in FP32 (high*high + low*high + high*low).
//
// Work item = (128-token tile, head).  A CTA serves one sample and one group of heads whose compact
// matrices stay in shared memory, and walks over its items with a ring of shared-memory stages:
//
//   warp 16 (one thread)  TMA: loads the relation and upstream-gradient boxes of an item into a stage;
//                         stores dA and dC, which the compute warps wrote over those boxes, back to
//                         `dprojected`.
//   warp 19 (one thread)  TMA: content boxes, in a ring of their own (a box is free again as soon as its rows
//                         have been rotated into tensor memory, long before the item's outputs are stored).
//   warp 17               issues the tcgen05 MMAs (warp-uniform control flow, one elected lane issues each
//                         batch); the accumulators of an item (dC: 128 x 64, dA: 128 x r, FP32) live in
//                         tensor memory, two items in flight (slots).
//   warps 0-7 / 8-15      one group per slot, half a token row per thread: rotate dY and C in FP32, split them
//                         into two BF16 words and write those straight into tensor memory, from where the
//                         MMAs take them as the row operand (no rotated copy in shared memory); later read
//                         the accumulators, apply the inverse rotation / eta / scale and write BF16 rows.
//
//   warp 18 (one thread)  TMA: brings the cos / sin rows of the next token tile (128 x 32 FP32 each) into a
//                         shared-memory buffer; every compute thread copies its 16 + 16 entries to registers
//                         once per tile.  (Read straight from global memory, one row per thread, the tables
//                         cost 16 us of a 60 us launch: 32 cache lines per load instruction.)
//
// Every wait is bounded (mbar_wait); after a timeout the error word is set and the CTA drains.  Spare
// CTAs (blockIdx.x >= work CTAs) compute the per-head parameter gradients as in the mma.sync kernel.
#include "ms_core.cuh"
#include "ms_tc.cuh"

namespace ms {

constexpr int kTcComputeWarps = 16;                  // two groups of eight
constexpr int kTcThreads = (kTcComputeWarps + 4) * 32;
constexpr int kTcGroupThreads = 256;
constexpr int kTcTile = 128;       // tokens per item
constexpr int kTcMinTokens = 512;  // shorter samples leave most of a tile empty: mma.sync kernels

template <int R>
struct TokenBwdTcCfg {
  static constexpr int A_ROW = R * 2;                   // bytes of one relation row
  static constexpr int A_TILE = kTcTile * A_ROW;
  static constexpr int STAGE = 16384 + A_TILE;          // gradient and relation boxes (outputs are written over them)
  static constexpr int STAGES = R == 64 ? 3 : 4;
  static constexpr int C_STAGES = 3;                    // content boxes have a ring of their own: they are free
  static constexpr int C_STAGE = 16384;                 // again as soon as the rows have been rotated
  static constexpr int TABLE_BYTES = 32768;             // cos and sin rows of one token tile
  static constexpr int W_BYTES = R * 128;
  static constexpr int S_BYTES = R * R * 2;
  static constexpr int HEAD_BYTES = 4 * W_BYTES + 2 * S_BYTES;   // W hi/lo, dQ hi/lo, S' hi/lo
  static constexpr int BAR_BYTES = (2 * STAGES + 2 * C_STAGES + 11) * 8 + 16;
  static constexpr int RING_BYTES = STAGES * STAGE + C_STAGES * C_STAGE;
  static constexpr int MAX_SMEM = 227 * 1024;
  static constexpr int RESIDENT_BUDGET = MAX_SMEM - 1024 - RING_BYTES - TABLE_BYTES - BAR_BYTES;
  // tensor-memory columns of one slot
  static constexpr int COL_DC = 0, COL_DA = 64, COL_YH = 128, COL_YL = 160, COL_CH = 192, COL_CL = 224, SLOT_COLS = 256;
  static_assert(64 + R <= 128, "accumulators of a slot");
};

struct TokenBwdTcParams {
  const float* cos;
  const float* sin;
  const float* counts;
  const float* eta;
  float* debug;      // optional FP32 copy of dprojected before the BF16 rounding ([B, N, H*(r+64)]), or null
  int* error;
  int tokens, heads, rotary_rows, group_heads, tiles, work_ctas, batch;
  int core_ctas;
  const float* base_raw;
  const float* hmat;
  const float* de_sys;
  const float* eta_slope;
  const float* core_map;
  float* d_base;
  float* d_eta_raw;
  float grad_scale;
  int complement;
};

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}

// one warp-uniform bounded wait
__device__ __forceinline__ bool wait_uniform(uint32_t bar, uint32_t parity) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity));
}

// Rotate 32 channels (64 bytes: 16-byte chunks 4*half .. 4*half + 3) of one row of a 128-byte-swizzled tile and
// write their two BF16 words to 16 tensor-memory columns each, starting at t_hi / t_lo, of this thread's lane.
__device__ __forceinline__ void rotate_half_row_to_tmem(uint32_t tile, int row, int half, const float (&cs)[16],
                                                        const float (&sn)[16], uint32_t t_hi, uint32_t t_lo) {
  uint32_t hi[16], lo[16];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int chunk = half * 4 + c;
    const uint4 v = ld_shared_v4(tile + row * 128 + ((chunk ^ (row & 7)) << 4));
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = bf2_to_f2(w[k]);
      const float2 r = rot_pair(f.x, f.y, cs[c * 4 + k], sn[c * 4 + k]);
      split2(r.x, r.y, hi[c * 4 + k], lo[c * 4 + k]);
    }
  }
  tc::tmem_st16(t_hi, hi);
  tc::tmem_st16(t_lo, lo);
}

template <int R, bool ROT, bool DEBUG>
__global__ void __launch_bounds__(kTcThreads, 1)
token_backward_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_c,
                         const __grid_constant__ CUtensorMap map_y, const __grid_constant__ CUtensorMap map_w,
                         const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_s,
                         const __grid_constant__ CUtensorMap map_oa, const __grid_constant__ CUtensorMap map_oc,
                         const __grid_constant__ CUtensorMap map_cos, const __grid_constant__ CUtensorMap map_sin,
                         const TokenBwdTcParams p) {
  using Cfg = TokenBwdTcCfg<R>;
  constexpr int S = Cfg::STAGES;
  constexpr int SC = Cfg::C_STAGES;
  constexpr int kProducerWarp = kTcComputeWarps, kMmaWarp = kTcComputeWarps + 1, kTableWarp = kTcComputeWarps + 2,
                kContentWarp = kTcComputeWarps + 3;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t smem = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  grid_launch_dependents();

  if ((int)blockIdx.x >= p.work_ctas) {
    grid_dependency_wait();
    if (blockIdx.y == 0 && blockIdx.z == 0) {
      for (int head = (int)blockIdx.x - p.work_ctas; head < p.heads; head += p.core_ctas) {
        core_backward_device(p.base_raw, p.hmat, p.de_sys, p.eta_slope, p.core_map, R, head, p.heads, p.batch,
                             p.complement, p.grad_scale, p.d_base, p.d_eta_raw,
                             smem_raw + (smem - smem_u32(smem_raw)), tid, kTcThreads);
        __syncthreads();
      }
    }
    return;
  }

  const int b = blockIdx.y;
  const int h0 = blockIdx.z * p.group_heads;
  const int gh = min(p.group_heads, p.heads - h0);
  const uint32_t res_base = smem;
  const uint32_t ring = smem + p.group_heads * Cfg::HEAD_BYTES;
  const uint32_t c_ring = ring + S * Cfg::STAGE;
  const uint32_t tab_buf = c_ring + SC * Cfg::C_STAGE;
  const uint32_t bar_full = tab_buf + Cfg::TABLE_BYTES;
  const uint32_t bar_out = bar_full + 8 * S;
  const uint32_t bar_cfull = bar_out + 8 * S;
  const uint32_t bar_cfree = bar_cfull + 8 * SC;
  const uint32_t bar_xf = bar_cfree + 8 * SC;
  const uint32_t bar_m1 = bar_xf + 16, bar_m2 = bar_m1 + 16, bar_free = bar_m2 + 16, bar_res = bar_free + 16;
  const uint32_t bar_tab_full = bar_res + 8, bar_tab_free = bar_tab_full + 8;
  const uint32_t tslot = bar_tab_free + 8;

  if (tid == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(bar_full + 8 * i, 1);
      mbar_init(bar_out + 8 * i, kTcGroupThreads);
    }
    for (int i = 0; i < SC; ++i) {
      mbar_init(bar_cfull + 8 * i, 1);
      mbar_init(bar_cfree + 8 * i, kTcGroupThreads);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_xf + 8 * i, kTcGroupThreads);
      mbar_init(bar_m1 + 8 * i, 1);
      mbar_init(bar_m2 + 8 * i, 1);
      mbar_init(bar_free + 8 * i, kTcGroupThreads);
    }
    mbar_init(bar_res, 1);
    mbar_init(bar_tab_full, 1);
    mbar_init(bar_tab_free, 2 * kTcGroupThreads);
    mbar_fence_init();
  }
  __syncthreads();
  if (warp == kMmaWarp) tc::tmem_alloc(tslot, 512);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = ld_shared_u32(tslot);

  const int total = p.tiles * gh;
  const int per = (total + p.work_ctas - 1) / p.work_ctas;
  const int it0 = min(total, (int)blockIdx.x * per);
  const int n_items = min(total, it0 + per) - it0;
  // token tiles this CTA touches: ordinal k = tile - tile0
  const int tile0 = it0 / gh;
  const int n_tiles = n_items > 0 ? (it0 + n_items - 1) / gh - tile0 + 1 : 0;
  bool ok = true;

  if (warp == kProducerWarp) {
    // ---------------------------------------------------------------- TMA producer / store issuer
    if (lane == 0) {
      auto issue_load = [&](int i) {
        const int idx = it0 + i, tile = idx / gh, h = h0 + (idx - tile * gh);
        const uint32_t st = ring + (i % S) * Cfg::STAGE, bar = bar_full + 8 * (i % S);
        mbar_expect_tx(bar, Cfg::STAGE);
        tma_load_3d(st + 16384, &map_a, h * R, tile * kTcTile, b, bar);
        tma_load_3d(st, &map_y, h * 64, tile * kTcTile, b, bar);
      };
      // `projected` and the upstream gradient were complete before the kernel ahead of this one started, so
      // a chained launch may fetch them while that kernel (which produces dQ and S') is still draining
      for (int k = 0; k < S && k < n_items; ++k) issue_load(k);
      grid_dependency_wait();
      mbar_expect_tx(bar_res, (uint32_t)(gh * Cfg::HEAD_BYTES));
      for (int hl = 0; hl < gh; ++hl) {
        const int sys = b * p.heads + h0 + hl;
        const uint32_t hb = res_base + hl * Cfg::HEAD_BYTES;
        tma_load_2d(hb, &map_w, 0, (sys * 2) * R, bar_res);
        tma_load_2d(hb + Cfg::W_BYTES, &map_w, 0, (sys * 2 + 1) * R, bar_res);
        tma_load_2d(hb + 2 * Cfg::W_BYTES, &map_q, 0, (sys * 2) * R, bar_res);
        tma_load_2d(hb + 3 * Cfg::W_BYTES, &map_q, 0, (sys * 2 + 1) * R, bar_res);
        tma_load_2d(hb + 4 * Cfg::W_BYTES, &map_s, 0, (sys * 2) * R, bar_res);
        tma_load_2d(hb + 4 * Cfg::W_BYTES + Cfg::S_BYTES, &map_s, 0, (sys * 2 + 1) * R, bar_res);
      }
      for (int i = 0; i < n_items; ++i) {
        ok = mbar_wait(bar_out + 8 * (i % S), (i / S) & 1);
        if (!ok) break;
        const int idx = it0 + i, tile = idx / gh, h = h0 + (idx - tile * gh);
        const uint32_t st = ring + (i % S) * Cfg::STAGE;
        tma_store_3d(&map_oc, p.heads * R + h * 64, tile * kTcTile, b, st);
        tma_store_3d(&map_oa, h * R, tile * kTcTile, b, st + 16384);
        tma_store_commit();
        if (i + S < n_items) {
          tma_store_wait_read<0>();   // the stage is read by the stores just issued
          issue_load(i + S);
        }
      }
      tma_store_wait_all<0>();
      if (!ok) atomicExch(p.error, kErrBarrierTimeout);
    }
  } else if (warp == kContentWarp) {
    // ---------------------------------------------------------------- content boxes, a ring of their own
    if (lane == 0) {
      for (int j = 0; j < n_items; ++j) {
        if (j >= SC) {
          ok = mbar_wait(bar_cfree + 8 * (j % SC), ((j / SC) - 1) & 1);   // item j - SC no longer reads the box
          if (!ok) break;
        }
        const int idx = it0 + j, tile = idx / gh, h = h0 + (idx - tile * gh);
        mbar_expect_tx(bar_cfull + 8 * (j % SC), Cfg::C_STAGE);
        tma_load_3d(c_ring + (j % SC) * Cfg::C_STAGE, &map_c, p.heads * R + h * 64, tile * kTcTile, b, bar_cfull + 8 * (j % SC));
      }
      if (!ok) atomicExch(p.error, kErrBarrierTimeout);
    }
  } else if (warp == kTableWarp) {
    // ---------------------------------------------------------------- table producer
    if (ROT && lane == 0) {
      const int tab_b = p.rotary_rows > 1 ? b : 0;
      for (int k = 0; k < n_tiles; ++k) {
        if (k > 0) {
          ok = mbar_wait(bar_tab_free, (k - 1) & 1);   // every compute thread has copied the rows of tile k - 1
          if (!ok) break;
        }
        mbar_expect_tx(bar_tab_full, Cfg::TABLE_BYTES);
        tma_load_3d(tab_buf, &map_cos, 0, (tile0 + k) * kTcTile, tab_b, bar_tab_full);
        tma_load_3d(tab_buf + 16384, &map_sin, 0, (tile0 + k) * kTcTile, tab_b, bar_tab_full);
      }
      if (!ok) atomicExch(p.error, kErrBarrierTimeout);
    }
  } else if (warp == kMmaWarp) {
    // ---------------------------------------------------------------- MMA issuer: the whole warp runs the control
    // flow (uniform), one elected lane issues each batch of MMAs and its commit
    constexpr uint32_t IDESC_C = tc::idesc_bf16(128, 64, true);    // dC: B = dQ stored [r][64]
    constexpr uint32_t IDESC_A = tc::idesc_bf16(128, R, false);    // dA: B stored [r output columns][k]
    constexpr uint32_t HI_A = tc::desc_hi_k_major(Cfg::A_ROW), HI_K = tc::desc_hi_k_major(128), HI_N = tc::desc_hi_n_major_128();
    grid_dependency_wait();
    ok = wait_uniform(bar_res, 0);
    const uint32_t res_lo = tc::desc_lo_k_major(res_base);   // leading-offset field of the contraction-major form
    const uint32_t ring_lo = tc::desc_lo_k_major(ring);
    const uint32_t cring_lo = tc::desc_lo_k_major(c_ring);
    constexpr uint32_t N_MAJOR_LBO = ((1024u >> 4) - 1u) << 16;   // added to a contraction-major low word
    auto item_words = [&](int i, uint32_t& st_lo, uint32_t& hb_lo) {
      const int idx = it0 + i, tile = idx / gh;
      st_lo = ring_lo + (uint32_t)((i % S) * (Cfg::STAGE >> 4));
      hb_lo = res_lo + (uint32_t)((idx - tile * gh) * (Cfg::HEAD_BYTES >> 4));
    };
    // products that need only the raw relation rows: dC = A dQ, dA = A S'
    auto ready_a = [&](int i) {
      return mbar_test(bar_full + 8 * (i % S), (i / S) & 1) &&
             (i < 2 || mbar_test(bar_free + 8 * (i & 1), ((i >> 1) - 1) & 1));
    };
    auto phase_a = [&](int i) {
      const int slot = i & 1;
      tc::fence_after_sync();
      uint32_t st_lo, hb_lo;
      item_words(i, st_lo, hb_lo);
      const uint32_t a_lo = st_lo + (16384 >> 4), tb = tmem + slot * Cfg::SLOT_COLS;
      const uint32_t qh = hb_lo + ((2 * Cfg::W_BYTES) >> 4) + N_MAJOR_LBO, ql = qh + (Cfg::W_BYTES >> 4);
      const uint32_t sh = hb_lo + ((4 * Cfg::W_BYTES) >> 4), sl = sh + (Cfg::S_BYTES >> 4);
      if (tc::elect_one()) {
#pragma unroll
        for (int word = 0; word < 2; ++word) {
#pragma unroll
          for (int ks = 0; ks < R / 16; ++ks)
            tc::mma_ss_raw<HI_A, HI_N, IDESC_C>(tb + Cfg::COL_DC, a_lo + ks * 2, (word == 0 ? ql : qh) + ks * 128,
                                                (word | ks) != 0);
        }
#pragma unroll
        for (int word = 0; word < 2; ++word) {
#pragma unroll
          for (int ks = 0; ks < R / 16; ++ks)
            tc::mma_ss_raw<HI_A, HI_A, IDESC_A>(tb + Cfg::COL_DA, a_lo + ks * 2, (word == 0 ? sl : sh) + ks * 2,
                                                (word | ks) != 0);
        }
        tc::mma_commit_raw(bar_m1 + 8 * slot);
      }
      __syncwarp();
    };
    // products with the (rotated) content and gradient rows: dA += rot(dY) W^T + rot(C) dQ^T
    auto ready_b = [&](int i) {
      return ROT ? mbar_test(bar_xf + 8 * (i & 1), (i >> 1) & 1) : mbar_test(bar_cfull + 8 * (i % SC), (i / SC) & 1);
    };
    auto phase_b = [&](int i) {
      const int slot = i & 1;
      tc::fence_after_sync();
      uint32_t st_lo, hb_lo;
      item_words(i, st_lo, hb_lo);
      const uint32_t tb = tmem + slot * Cfg::SLOT_COLS;
      const uint32_t wh = hb_lo, wl = wh + (Cfg::W_BYTES >> 4), qh = wl + (Cfg::W_BYTES >> 4), ql = qh + (Cfg::W_BYTES >> 4);
      if (tc::elect_one()) {
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          if (ROT) {
            tc::mma_ts_raw<HI_K, IDESC_A>(tb + Cfg::COL_DA, tb + Cfg::COL_YL + ks * 8, wh + ks * 2, 1);
            tc::mma_ts_raw<HI_K, IDESC_A>(tb + Cfg::COL_DA, tb + Cfg::COL_YH + ks * 8, wl + ks * 2, 1);
            tc::mma_ts_raw<HI_K, IDESC_A>(tb + Cfg::COL_DA, tb + Cfg::COL_YH + ks * 8, wh + ks * 2, 1);
            tc::mma_ts_raw<HI_K, IDESC_A>(tb + Cfg::COL_DA, tb + Cfg::COL_CL + ks * 8, qh + ks * 2, 1);
            tc::mma_ts_raw<HI_K, IDESC_A>(tb + Cfg::COL_DA, tb + Cfg::COL_CH + ks * 8, ql + ks * 2, 1);
            tc::mma_ts_raw<HI_K, IDESC_A>(tb + Cfg::COL_DA, tb + Cfg::COL_CH + ks * 8, qh + ks * 2, 1);
          } else {
            const uint32_t y_lo = st_lo + ks * 2, c_lo = cring_lo + (uint32_t)((i % SC) * (Cfg::C_STAGE >> 4)) + ks * 2;
            tc::mma_ss_raw<HI_K, HI_K, IDESC_A>(tb + Cfg::COL_DA, y_lo, wl + ks * 2, 1);
            tc::mma_ss_raw<HI_K, HI_K, IDESC_A>(tb + Cfg::COL_DA, y_lo, wh + ks * 2, 1);
            tc::mma_ss_raw<HI_K, HI_K, IDESC_A>(tb + Cfg::COL_DA, c_lo, ql + ks * 2, 1);
            tc::mma_ss_raw<HI_K, HI_K, IDESC_A>(tb + Cfg::COL_DA, c_lo, qh + ks * 2, 1);
          }
        }
        tc::mma_commit_raw(bar_m2 + 8 * slot);
      }
      __syncwarp();
    };
    // Event loop: the first phase of the next item and the second phase of the oldest open item are issued
    // in whichever order their inputs become ready (an item's second phase follows its first; both advance
    // in item order).  Waiting for them in a fixed order made the two compute groups take turns.  The loop is
    // bounded like every other wait: after kWaitLimit rounds without progress it gives up.
    int next_a = 0, next_b = 0, idle = 0;
    while (ok && next_b < n_items) {
      bool progressed = false;
      if (next_a < n_items && next_a < next_b + 2 && __all_sync(0xffffffffu, ready_a(next_a))) {
        phase_a(next_a++);
        progressed = true;
      }
      if (next_b < next_a && __all_sync(0xffffffffu, ready_b(next_b))) {
        phase_b(next_b++);
        progressed = true;
      }
      if (progressed) {
        idle = 0;
      } else {
        __nanosleep(40);   // leave the issue slots to the compute warps of this scheduler
        if (++idle > kWaitLimit) ok = false;
      }
    }
    if (!ok && lane == 0) atomicExch(p.error, kErrBarrierTimeout);
  } else {
    // ---------------------------------------------------------------- compute warps: eight per slot; a thread owns
    // one token row (the lanes its warp may touch in tensor memory: 32 * (warp % 4) ...) and half of its channels
    const int g = warp >> 3, q = warp & 3, half = (warp >> 2) & 1, row = q * 32 + lane;
    const uint32_t lane_base = tmem + ((uint32_t)(q * 32) << 16) + g * Cfg::SLOT_COLS;
    grid_dependency_wait();
    const float n = p.counts ? p.counts[b] : (float)p.tokens;
    const float inv_s = inv_sqrt_rn(n);
    const long tab_row_b = p.rotary_rows > 1 ? (long)b * p.tokens : 0;
    const int width = p.heads * (R + 64);
    float cs[16], sn[16];
    int tab_next = 0;   // ordinal of the next tile whose table rows this thread has not yet passed
    bool owe_table = false;   // this thread holds the rows of a tile and has not yet released the buffer
    // Copy this thread's 16 cos / sin entries of tile ordinal k from the shared-memory buffer; tiles in between
    // (this group had no item in them) are passed without copying, so that the buffer can be refilled.
    auto take_tables = [&](int k) {
      bool good = true;
      while (tab_next <= k && good) {
        good = wait_uniform(bar_tab_full, tab_next & 1);
        if (good && tab_next == k) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const uint32_t off = row * 128 + (((half * 4 + v) ^ (row & 7)) << 4);
            const float4 cv = ld_shared_f4(tab_buf + off), sv = ld_shared_f4(tab_buf + 16384 + off);
            cs[4 * v] = cv.x; cs[4 * v + 1] = cv.y; cs[4 * v + 2] = cv.z; cs[4 * v + 3] = cv.w;
            sn[4 * v] = sv.x; sn[4 * v + 1] = sv.y; sn[4 * v + 2] = sv.z; sn[4 * v + 3] = sv.w;
          }
        }
        if (good) {
          // A tile whose rows were copied is handed back only after they have been USED (below): ld.shared merely
          // issues the reads, and an arrive right behind it can let the table warp's next bulk copy land first.
          if (tab_next == k) owe_table = true;
          else mbar_arrive(bar_tab_free);
        }
        ++tab_next;
      }
      return good;
    };

    for (int i = g; i < n_items && ok; i += 2) {
      const int stage = i % S;
      const int idx = it0 + i, tile = idx / gh, h = h0 + (idx - tile * gh);
      const uint32_t st = ring + stage * Cfg::STAGE;
      const uint32_t y_tile = st, a_tile = st + 16384, c_tile = c_ring + (i % SC) * Cfg::C_STAGE;
      const int tok = tile * kTcTile + row;
      const bool valid = tok < p.tokens;
      const float eta = __ldg(p.eta + h);
      const uint32_t par = (i >> 1) & 1;

      if (ROT && tile - tile0 >= tab_next) {
        // rows past the end of the sample come back as zeros from the TMA load: rotation by cos = sin = 0 of
        // zero content, harmless
        ok = take_tables(tile - tile0);
        if (!ok) break;
      }
      ok = wait_uniform(bar_full + 8 * stage, (i / S) & 1);
      if (!ok) break;
      if (ROT) {
        rotate_half_row_to_tmem(y_tile, row, half, cs, sn, lane_base + Cfg::COL_YH + half * 16,
                                lane_base + Cfg::COL_YL + half * 16);
        if (owe_table) {   // every cos / sin register has been consumed by an instruction issued above
          mbar_arrive(bar_tab_free);
          owe_table = false;
        }
        ok = wait_uniform(bar_cfull + 8 * (i % SC), (i / SC) & 1);
        if (!ok) break;
        rotate_half_row_to_tmem(c_tile, row, half, cs, sn, lane_base + Cfg::COL_CH + half * 16,
                                lane_base + Cfg::COL_CL + half * 16);
        mbar_arrive(bar_cfree + 8 * (i % SC));   // the content box is in registers / tensor memory now
        tc::wait_st();
        tc::fence_before_sync();
        mbar_arrive(bar_xf + 8 * g);
      }

      // dC = eta*dY + s * rot^-1(A dQ), written over the upstream-gradient row.  Without rotation the MMAs
      // read that row from shared memory, so all of them must have completed first.
      ok = wait_uniform((ROT ? bar_m1 : bar_m2) + 8 * g, par);
      if (!ok) break;
      tc::fence_after_sync();
      if (!ROT) mbar_arrive(bar_cfree + 8 * (i % SC));   // the MMAs that read the content box have completed
      float* dbg = (DEBUG && valid) ? p.debug + ((size_t)b * p.tokens + tok) * width : nullptr;
      {
        uint32_t acc[32];
        tc::tmem_ld16(lane_base + Cfg::COL_DC + half * 32, *reinterpret_cast<uint32_t(*)[16]>(&acc[0]));
        tc::tmem_ld16(lane_base + Cfg::COL_DC + half * 32 + 16, *reinterpret_cast<uint32_t(*)[16]>(&acc[16]));
        tc::wait_ld();
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int chunk = half * 4 + c;
          const uint32_t addr = y_tile + row * 128 + ((chunk ^ (row & 7)) << 4);
          const uint4 yv = ld_shared_v4(addr);
          const uint32_t yw[4] = {yv.x, yv.y, yv.z, yv.w};
          uint32_t ow[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int j = c * 4 + k;
            float2 corr = make_float2(__uint_as_float(acc[2 * j]), __uint_as_float(acc[2 * j + 1]));
            if (ROT) corr = rot_pair(corr.x, corr.y, cs[j], -sn[j]);
            const float2 yy = bf2_to_f2(yw[k]);
            const float o0 = fmaf(corr.x, inv_s, eta * yy.x), o1 = fmaf(corr.y, inv_s, eta * yy.y);
            ow[k] = f2_to_bf2(o0, o1);
            if (DEBUG && dbg) {
              dbg[p.heads * R + h * 64 + half * 32 + 2 * j] = o0;
              dbg[p.heads * R + h * 64 + half * 32 + 2 * j + 1] = o1;
            }
          }
          st_shared_v4(addr, make_uint4(ow[0], ow[1], ow[2], ow[3]));
        }
      }

      // dA = s * (A S' + rot(dY) W^T + rot(C) dQ^T), written over the relation row: this thread's R/2 columns
      if (ROT) {
        ok = wait_uniform(bar_m2 + 8 * g, par);
        if (!ok) break;
        tc::fence_after_sync();
      }
      {
        constexpr int COLS = R / 2;   // 8, 16 or 32
        uint32_t acc[COLS];
        if constexpr (COLS >= 16) {
#pragma unroll
          for (int c0 = 0; c0 < COLS; c0 += 16)
            tc::tmem_ld16(lane_base + Cfg::COL_DA + half * COLS + c0, *reinterpret_cast<uint32_t(*)[16]>(&acc[c0]));
        } else {
          tc::tmem_ld8(lane_base + Cfg::COL_DA + half * COLS, *reinterpret_cast<uint32_t(*)[8]>(&acc[0]));
        }
        tc::wait_ld();
#pragma unroll
        for (int c = 0; c < COLS / 8; ++c) {
          const int src = 8 * c;
          uint32_t ow[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float o0 = __uint_as_float(acc[src + 2 * k]) * inv_s, o1 = __uint_as_float(acc[src + 2 * k + 1]) * inv_s;
            ow[k] = f2_to_bf2(o0, o1);
            if (DEBUG && dbg) {
              dbg[h * R + half * COLS + 8 * c + 2 * k] = o0;
              dbg[h * R + half * COLS + 8 * c + 2 * k + 1] = o1;
            }
          }
          st_shared_v4(a_tile + swz_rows<Cfg::A_ROW>(row * Cfg::A_ROW + (half * (COLS / 8) + c) * 16),
                       make_uint4(ow[0], ow[1], ow[2], ow[3]));
        }
      }
      tc::fence_before_sync();
      mbar_arrive(bar_free + 8 * g);
      fence_async_shared();
      mbar_arrive(bar_out + 8 * stage);
    }
    // tiles after this group's last item: pass them, the other group may still need the buffer refilled
    while (ROT && ok && tab_next < n_tiles) {
      ok = wait_uniform(bar_tab_full, tab_next & 1);
      if (ok) mbar_arrive(bar_tab_free);
      ++tab_next;
    }
    if (!ok && lane == 0) atomicExch(p.error, kErrBarrierTimeout);
  }

  // all roles meet here; the tensor memory goes back before the CTA exits
  tc::fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarp) tc::tmem_free(tmem, 512);
}

template <int R>
static int launch_token_bwd_tc_r(const ms_shape& s, const Plan& plan, const void* projected, const void* dy,
                                 const float* cos, const float* sin, const float* counts, const ms_tape& t,
                                 const void* gram_grad, const void* cross_grad, void* dprojected,
                                 const CoreAdjoint* core, float* debug, cudaStream_t st) {
  using Cfg = TokenBwdTcCfg<R>;
  const int heads = s.heads, width = heads * (R + 64), dmodel = heads * 64;
  int group = Cfg::RESIDENT_BUDGET / Cfg::HEAD_BYTES;
  if (group < 1) return -1;
  if (group > heads) group = heads;
  const int groups = (heads + group - 1) / group;
  group = (heads + groups - 1) / groups;   // even out the groups

  CUtensorMap map_a, map_c, map_y, map_w, map_q, map_s, map_oa, map_oc;
  {
    const uint64_t dims[3] = {(uint64_t)width, (uint64_t)s.tokens, (uint64_t)s.batch};
    const uint64_t str[2] = {(uint64_t)width * 2, (uint64_t)s.tokens * width * 2};
    const uint32_t box_a[3] = {(uint32_t)R, kTcTile, 1};
    const uint32_t box_c[3] = {64, kTcTile, 1};
    const Swizzle sa = swizzle_for_rows<R * 2>();
    if (encode_tensor_map(&map_a, const_cast<void*>(projected), 2, 3, dims, str, box_a, sa)) return MS_ERR_LAUNCH;
    if (encode_tensor_map(&map_c, const_cast<void*>(projected), 2, 3, dims, str, box_c, Swizzle::B128)) return MS_ERR_LAUNCH;
    if (encode_tensor_map(&map_oa, dprojected, 2, 3, dims, str, box_a, sa)) return MS_ERR_LAUNCH;
    if (encode_tensor_map(&map_oc, dprojected, 2, 3, dims, str, box_c, Swizzle::B128)) return MS_ERR_LAUNCH;
  }
  {
    const uint64_t dims[3] = {(uint64_t)dmodel, (uint64_t)s.tokens, (uint64_t)s.batch};
    const uint64_t str[2] = {(uint64_t)dmodel * 2, (uint64_t)s.tokens * dmodel * 2};
    const uint32_t box[3] = {64, kTcTile, 1};
    if (encode_tensor_map(&map_y, const_cast<void*>(dy), 2, 3, dims, str, box, Swizzle::B128)) return MS_ERR_LAUNCH;
  }
  {
    const uint64_t dims[2] = {64, (uint64_t)plan.systems * 2 * R};
    const uint64_t str[1] = {128};
    const uint32_t box[2] = {64, (uint32_t)R};
    if (encode_tensor_map(&map_w, t.coeff, 2, 2, dims, str, box, Swizzle::B128)) return MS_ERR_LAUNCH;
    if (encode_tensor_map(&map_q, const_cast<void*>(cross_grad), 2, 2, dims, str, box, Swizzle::B128)) return MS_ERR_LAUNCH;
    const uint64_t sdims[2] = {(uint64_t)R, (uint64_t)plan.systems * 2 * R};
    const uint64_t sstr[1] = {(uint64_t)R * 2};
    const uint32_t sbox[2] = {(uint32_t)R, (uint32_t)R};
    if (encode_tensor_map(&map_s, const_cast<void*>(gram_grad), 2, 2, sdims, sstr, sbox, swizzle_for_rows<R * 2>()))
      return MS_ERR_LAUNCH;
  }

  CUtensorMap map_cos = map_a, map_sin = map_a;   // placeholders when there is no rotation
  if (s.rotary_rows > 0) {
    const uint64_t dims[3] = {32, (uint64_t)s.tokens, (uint64_t)s.rotary_rows};
    const uint64_t str[2] = {128, (uint64_t)s.tokens * 128};
    const uint32_t box[3] = {32, kTcTile, 1};
    if (encode_tensor_map(&map_cos, const_cast<float*>(cos), 4, 3, dims, str, box, Swizzle::B128)) return MS_ERR_LAUNCH;
    if (encode_tensor_map(&map_sin, const_cast<float*>(sin), 4, 3, dims, str, box, Swizzle::B128)) return MS_ERR_LAUNCH;
  }

  TokenBwdTcParams p;
  p.cos = cos; p.sin = sin; p.counts = counts; p.eta = t.eta; p.debug = debug;
  p.error = device_error_word();
  if (!p.error) return MS_ERR_LAUNCH;
  p.tokens = s.tokens; p.heads = heads; p.rotary_rows = s.rotary_rows; p.group_heads = group;
  p.tiles = (s.tokens + kTcTile - 1) / kTcTile; p.batch = s.batch;
  p.base_raw = nullptr; p.hmat = nullptr; p.de_sys = nullptr; p.eta_slope = t.eta_slope; p.core_map = t.core_map;
  p.d_base = nullptr; p.d_eta_raw = nullptr; p.grad_scale = 1.f; p.complement = s.complement;
  if (core) {
    p.base_raw = core->base_raw; p.hmat = core->hmat; p.de_sys = core->de_sys;
    p.d_base = core->d_base; p.d_eta_raw = core->d_eta_raw; p.grad_scale = core->grad_scale;
  }
  const long total = (long)p.tiles * group;
  // one CTA per SM; SMs are left for the per-head CTAs that ride along so that the whole grid is resident
  const int core_ctas = core ? (s.batch <= 4 ? (heads + 1) / 2 : heads) : 0;
  long ctas = (sm_count() - core_ctas) / ((long)s.batch * groups);
  if (ctas < 1) ctas = 1;
  const long need = (total + 3) / 4;   // at least four items per CTA pay for its resident matrices
  if (ctas > need) ctas = need < 1 ? 1 : need;
  p.work_ctas = (int)ctas;
  p.core_ctas = core_ctas > 0 ? core_ctas : 1;
  dim3 grid((unsigned)ctas + core_ctas, s.batch, groups);
  int smem_bytes = 1024 + group * Cfg::HEAD_BYTES + Cfg::RING_BYTES + Cfg::TABLE_BYTES + Cfg::BAR_BYTES;
  const int core_bytes = (int)core_backward_smem_bytes(R) + 1024;
  if (core && smem_bytes < core_bytes) smem_bytes = core_bytes;
  void (*kern)(CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap,
               CUtensorMap, CUtensorMap, TokenBwdTcParams);
  if (s.rotary_rows > 0) kern = debug ? token_backward_tc_kernel<R, true, true> : token_backward_tc_kernel<R, true, false>;
  else kern = debug ? token_backward_tc_kernel<R, false, true> : token_backward_tc_kernel<R, false, false>;
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem_bytes)) return MS_ERR_LAUNCH;
  launch_kernel(kern, grid, dim3(kTcThreads), smem_bytes, st, map_a, map_c, map_y, map_w, map_q, map_s, map_oa, map_oc,
                map_cos, map_sin, p);
  return cudaGetLastError() == cudaSuccess ? MS_OK : MS_ERR_LAUNCH;
}

// MS_OK / error, or -1 when the shape is outside this kernel's envelope.  `debug` (FP32 [B, N, H*(r+64)], or
// null) receives the values before the BF16 rounding; with `debug` set shapes below kTcMinTokens are taken too.
int launch_token_backward_tc(const ms_shape& s, const Plan& plan, const void* projected, const void* dy,
                             const float* cos, const float* sin, const float* counts, const ms_tape& t,
                             const void* gram_grad, const void* cross_grad, void* dprojected,
                             const CoreAdjoint* core, float* debug, cudaStream_t st) {
  if (!plan.aligned || s.head_dim != 64) return -1;
  if (s.tokens < kTcMinTokens && !debug) return -1;
  if (s.batch > 65535) return -1;
  if (((reinterpret_cast<uintptr_t>(t.coeff) | reinterpret_cast<uintptr_t>(gram_grad) |
        reinterpret_cast<uintptr_t>(cross_grad)) & 15u) != 0)
    return -1;
#define MS_TC_ARGS s, plan, projected, dy, cos, sin, counts, t, gram_grad, cross_grad, dprojected, core, debug, st
  switch (s.rank) {
    case 16: return launch_token_bwd_tc_r<16>(MS_TC_ARGS);
    case 32: return launch_token_bwd_tc_r<32>(MS_TC_ARGS);
    case 64: return launch_token_bwd_tc_r<64>(MS_TC_ARGS);
  }
#undef MS_TC_ARGS
  return -1;
}

}  // namespace ms
