// Token reductions on the fifth-generation tensor cores (tcgen05), for long sequences: head dimension 64,
// rank 16/32/64, aligned pointers, at least kStMinTokens tokens per sample (other shapes take the mma.sync
// kernels in ms_stats_tma.cu / ms_stats.cu).
//
//   forward:  G = A^T A,  Q = A^T rot(C)          adjoint:  E = A^T rot(dY),  de = <dY, C>
//
// (unscaled sums over the tokens of one chunk; the compact kernels add the chunks and scale).  Same arithmetic
// as the reference's `_chunk_statistics` (memsolve/ball/cuda.py:1925-2046): FP32 rotation, the rotated operand
// carried as two BF16 words, both products accumulated in FP32.
//
// The contraction runs over tokens, so the accumulators stay in tensor memory for the whole launch and are
// written once.  A CTA takes ONE head and one chunk of tokens.  Both MMA operands are token-major tiles exactly
// as TMA delivers them (rows = tokens): the "M-major" / "N-major" shared-memory operand forms.  The rotated
// content (or gradient) tile is the M operand -- its high BF16 word is written over the raw tile, its low word
// to a second tile, and one descriptor addresses the two as the two 64-row blocks of a 128-row operand -- and the
// head's r relation columns are the N operand, so that per 128-token tile and k-step of 16 tokens
//
//   D_Q [high 64 | low 64 channels][r]  +=  [X_high ; X_low]^T A_h        (moment = high rows + low rows)
//   D_G [64][r]                         +=  A_box^T A_h                   (rows 0 .. r-1 are the head's Gram)
//
// where A_box is the 64-column box of `projected` that starts at the head's relations.  Shared-memory traffic,
// which is what bounds this kernel (an MMA costs the time its operands take to read at 128 B/clk), is 5 KB per
// k-step for the moment instead of 4 KB per word and head pair, no accumulator rows are spent on other heads,
// and a system gets one partial per CTA: 11-12 per system at 32768 tokens and twelve heads, which the compact
// kernels stage in shared memory.
//
//   warp 16 (one thread)  TMA: content / gradient tiles (and, for the adjoint, the content tile of <dY, C>)
//   warp 19 (one thread)  TMA: relation boxes
//   warp 18 (one thread)  TMA: cos / sin rows of the next token tile
//   warp 17               MMA issue (warp-uniform control flow, an elected lane issues each batch); shared
//                         memory is handed back to the TMA warps by tcgen05.commit on their "free" barriers
//   warps 0-7 / 8-15      two groups that alternate tiles: rotate + split (half a token row per thread); at the
//                         end all sixteen read the accumulators and write the chunk's partial
//
// Spare CTAs of the forward grid compute the per-head core (eta, F) as in the mma.sync kernel.  Every wait
// is bounded; after a timeout the error word is set and the CTA drains.
#include "ms_core.cuh"
#include "ms_tc.cuh"

namespace ms {

constexpr int kStComputeWarps = 16;
constexpr int kStThreads = (kStComputeWarps + 4) * 32;
constexpr int kStGroupThreads = 256;
constexpr int kStTile = 128;

template <int R, bool GRAD, bool ROT>
struct StatsTcCfg {
  static constexpr int A_TILE = 16384;                    // 128 tokens x the 64-column box at the head's relations
  static constexpr int A_STAGES = (GRAD && ROT) ? 2 : 3;
  static constexpr int X_TILE = GRAD ? 32768 : 16384;     // gradient (+ content for <dY, C>) or content
  // an odd ring is shared by the two compute groups, which is only safe together with the low-word ring (see the
  // waits of the compute warps); without rotation there is none, and room for four stages
  static constexpr int X_STAGES = ROT ? 3 : 4;
  // low-word tiles: a deep ring lets a compute group rotate its next tile while the MMAs of its last one run
  static constexpr int LO_STAGES = ROT ? 2 : 0;
  static constexpr int LO_TILE = 16384;
  // cos / sin rows of a tile: 32 KB for 24 KB of tokens.  The copy takes about 2 us under load, so the rows of
  // several tiles ahead must be in flight (with one buffer the kernel ran at one tile per copy latency)
  static constexpr int TABLE_TILE = 32768;
  static constexpr int TAB_STAGES = !ROT ? 0 : (GRAD ? 2 : 3);
  static constexpr int TABLE_BYTES = TAB_STAGES * TABLE_TILE;
  static constexpr int BAR_BYTES = (2 * A_STAGES + 3 * X_STAGES + 4 + 8) * 8 + 16 + 16 * 4;
  static constexpr int TOTAL = 1024 + A_STAGES * A_TILE + X_STAGES * X_TILE + LO_STAGES * LO_TILE + TABLE_BYTES + BAR_BYTES;
  static constexpr int MQ = ROT ? 128 : 64;               // accumulator rows of the moment: [high ; low] or raw channels
  static constexpr int COL_Q = 0, COL_G = R;              // tensor-memory columns
  static constexpr int COLS = GRAD ? R : 2 * R;
  static constexpr int TMEM_COLS = COLS <= 32 ? 32 : (COLS <= 64 ? 64 : 128);
  static_assert(TOTAL <= 227 * 1024, "shared memory");
  static_assert(64 * R * 4 <= X_STAGES * X_TILE, "the low rows of the moment pass through the idle X ring");
};

struct StatsTcParams {
  float* partials;
  float* de_partials;
  int* error;
  int tokens, heads, rotary_rows, chunks, chunk_tokens, de_slots, partial_floats;
  const float* base_raw;
  const float* eta_raw;
  float* eta;
  float* eta_slope;
  float* core_map;
  int* core_info;
  int complement;
};

__device__ __forceinline__ void st_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool st_wait(uint32_t bar, uint32_t parity) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity));
}

template <int R, bool GRAD, bool ROT>
__global__ void __launch_bounds__(kStThreads, 1)
stats_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_c,
                const __grid_constant__ CUtensorMap map_y, const __grid_constant__ CUtensorMap map_cos,
                const __grid_constant__ CUtensorMap map_sin, const StatsTcParams p) {
  using Cfg = StatsTcCfg<R, GRAD, ROT>;
  constexpr int SA = Cfg::A_STAGES, SX = Cfg::X_STAGES, SL = ROT ? Cfg::LO_STAGES : 1, MQ = Cfg::MQ;
  constexpr int ST = ROT ? Cfg::TAB_STAGES : 1;
  constexpr bool TRANSFORM = ROT || GRAD;   // the compute warps touch every tile
  constexpr int kXWarp = kStComputeWarps, kMmaWarp = kStComputeWarps + 1, kTableWarp = kStComputeWarps + 2,
                kAWarp = kStComputeWarps + 3;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t smem = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  const int chunk = blockIdx.x;
  if (chunk >= p.chunks) {
    // spare CTAs of the forward grid: the per-head core runs beside the token reduction
    grid_launch_dependents();
    grid_dependency_wait();
    const int head = (chunk - p.chunks) * (int)gridDim.y * (int)gridDim.z + (int)blockIdx.z * (int)gridDim.y + (int)blockIdx.y;
    if (!GRAD && head < p.heads)
      core_forward_device<R, kStThreads>(p.base_raw, p.eta_raw, head, p.complement, p.eta, p.eta_slope, p.core_map,
                                         p.core_info, smem_raw + (smem - smem_u32(smem_raw)), tid);
    return;
  }

  const int b = blockIdx.z;
  const int h = blockIdx.y;
  const uint32_t a_ring = smem;
  const uint32_t x_ring = a_ring + SA * Cfg::A_TILE;
  const uint32_t lo_ring = x_ring + SX * Cfg::X_TILE;
  const uint32_t tab_buf = lo_ring + Cfg::LO_STAGES * Cfg::LO_TILE;
  const uint32_t bar_afull = tab_buf + Cfg::TABLE_BYTES;
  const uint32_t bar_afree = bar_afull + 8 * SA;
  const uint32_t bar_xfull = bar_afree + 8 * SA;
  const uint32_t bar_xfree = bar_xfull + 8 * SX;
  const uint32_t bar_xf = bar_xfree + 8 * SX;          // tile rotated / inspected by the compute warps
  const uint32_t bar_lofree = bar_xf + 8 * SX;         // up to four
  const uint32_t bar_tab_full = bar_lofree + 32, bar_tab_free = bar_tab_full + 8 * 3;   // up to three each
  const uint32_t bar_done = bar_tab_free + 8 * 3;
  const uint32_t tslot = bar_done + 8;
  const uint32_t de_red = tslot + 16;                  // [16 warps] floats

  if (tid == 0) {
    for (int i = 0; i < SA; ++i) {
      mbar_init(bar_afull + 8 * i, 1);
      mbar_init(bar_afree + 8 * i, 1);
    }
    for (int i = 0; i < SX; ++i) {
      mbar_init(bar_xfull + 8 * i, 1);
      mbar_init(bar_xfree + 8 * i, 1);
      mbar_init(bar_xf + 8 * i, kStGroupThreads);
    }
    for (int i = 0; i < 4; ++i) mbar_init(bar_lofree + 8 * i, 1);
    for (int i = 0; i < 3; ++i) {
      mbar_init(bar_tab_full + 8 * i, 1);
      mbar_init(bar_tab_free + 8 * i, 2 * kStGroupThreads);
    }
    mbar_init(bar_done, 1);
    mbar_fence_init();
  }
  __syncthreads();
  if (warp == kMmaWarp) tc::tmem_alloc(tslot, Cfg::TMEM_COLS);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = ld_shared_u32(tslot);

  const int tok0 = chunk * p.chunk_tokens;
  const int tok1 = min(p.tokens, tok0 + p.chunk_tokens);
  const int n_tiles = (tok1 - tok0 + kStTile - 1) / kStTile;   // chunk_tokens is a multiple of the tile
  bool ok = true;

  if (warp == kXWarp) {
    // ---------------------------------------------------------------- content / gradient tiles
    if (lane == 0) {
      grid_dependency_wait();
      for (int j = 0; j < n_tiles; ++j) {
        if (j >= SX) {
          ok = mbar_wait(bar_xfree + 8 * (j % SX), ((j / SX) - 1) & 1);   // the MMAs that read the slot have completed
          if (!ok) break;
        }
        const uint32_t dst = x_ring + (j % SX) * Cfg::X_TILE, bar = bar_xfull + 8 * (j % SX);
        mbar_expect_tx(bar, Cfg::X_TILE);
        if (GRAD) {
          tma_load_3d(dst, &map_y, h * 64, tok0 + j * kStTile, b, bar);
          tma_load_3d(dst + 16384, &map_c, p.heads * R + h * 64, tok0 + j * kStTile, b, bar);
        } else {
          tma_load_3d(dst, &map_c, p.heads * R + h * 64, tok0 + j * kStTile, b, bar);
        }
      }
      if (!ok) atomicExch(p.error, kErrBarrierTimeout);
    }
  } else if (warp == kAWarp) {
    // ---------------------------------------------------------------- relation boxes: 64 columns from the head's first
    if (lane == 0) {
      grid_dependency_wait();
      for (int t = 0; t < n_tiles; ++t) {
        if (t >= SA) {
          ok = mbar_wait(bar_afree + 8 * (t % SA), ((t / SA) - 1) & 1);
          if (!ok) break;
        }
        const uint32_t dst = a_ring + (t % SA) * Cfg::A_TILE, bar = bar_afull + 8 * (t % SA);
        mbar_expect_tx(bar, Cfg::A_TILE);
        tma_load_3d(dst, &map_a, h * R, tok0 + t * kStTile, b, bar);
      }
      if (!ok) atomicExch(p.error, kErrBarrierTimeout);
    }
  } else if (warp == kTableWarp) {
    // ---------------------------------------------------------------- cos / sin rows
    if (ROT && lane == 0) {
      grid_dependency_wait();
      const int tab_b = p.rotary_rows > 1 ? b : 0;
      for (int k = 0; k < n_tiles; ++k) {
        if (k >= ST) {
          ok = mbar_wait(bar_tab_free + 8 * (k % ST), ((k / ST) - 1) & 1);   // every compute thread has passed tile k - ST
          if (!ok) break;
        }
        const uint32_t dst = tab_buf + (k % ST) * Cfg::TABLE_TILE, bar = bar_tab_full + 8 * (k % ST);
        mbar_expect_tx(bar, 32768);
        tma_load_3d(dst, &map_cos, 0, tok0 + k * kStTile, tab_b, bar);
        tma_load_3d(dst + 16384, &map_sin, 0, tok0 + k * kStTile, tab_b, bar);
      }
      if (!ok) atomicExch(p.error, kErrBarrierTimeout);
    }
  } else if (warp == kMmaWarp) {
    // ---------------------------------------------------------------- MMA issuer
    // Gram: M = the 64 columns of the relation box, N = the head's r columns of the same box.
    // Moment: M = 128 rows [high ; low] (64 without rotation: the raw tile), N as above.
    constexpr uint32_t IDESC_G = tc::idesc_bf16(64, R, true, true);
    constexpr uint32_t IDESC_Q = tc::idesc_bf16(MQ, R, true, true);
    constexpr uint32_t HI = tc::desc_hi_n_major_128();
    const uint32_t a_lo0 = ((a_ring & 0x3ffffu) >> 4) | ((1024u >> 4) << 16);
    for (int t = 0; t < n_tiles && ok; ++t) {
      ok = st_wait(bar_afull + 8 * (t % SA), (t / SA) & 1);
      if (!ok) break;
      tc::fence_after_sync();
      const uint32_t a_lo = a_lo0 + (uint32_t)((t % SA) * (Cfg::A_TILE >> 4));
      if (!GRAD) {
        if (tc::elect_one()) {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            tc::mma_ss_raw<HI, HI, IDESC_G>(tmem + Cfg::COL_G, a_lo + ks * 128, a_lo + ks * 128, (t | ks) != 0);
        }
        __syncwarp();
      }
      ok = st_wait((TRANSFORM ? bar_xf : bar_xfull) + 8 * (t % SX), (t / SX) & 1);
      if (!ok) break;
      tc::fence_after_sync();
      // the tile's two words as ONE operand: 64-row blocks `lo - x` bytes apart (leading-dimension field)
      const uint32_t x_addr = x_ring + (uint32_t)((t % SX) * Cfg::X_TILE);
      const uint32_t l_addr = ROT ? lo_ring + (uint32_t)((t % SL) * Cfg::LO_TILE) : x_addr + 1024u;
      const uint32_t x_lo = ((x_addr & 0x3ffffu) >> 4) | (((l_addr - x_addr) >> 4) << 16);
      if (tc::elect_one()) {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          tc::mma_ss_raw<HI, HI, IDESC_Q>(tmem + Cfg::COL_Q, x_lo + ks * 128, a_lo + ks * 128, (t | ks) != 0);
        tc::mma_commit_raw(bar_xfree + 8 * (t % SX));
        if (ROT) tc::mma_commit_raw(bar_lofree + 8 * (t % SL));
        tc::mma_commit_raw(bar_afree + 8 * (t % SA));
      }
      __syncwarp();
    }
    if (ok) {
      if (tc::elect_one()) tc::mma_commit_raw(bar_done);
      __syncwarp();
    }
    if (!ok && lane == 0) atomicExch(p.error, kErrBarrierTimeout);
  }

  // The next kernel of a chained launch may become resident once this CTA's streaming part is over (signalling at
  // the start of the kernel parks its blocks on the SMs for the whole launch: measured slower).
  if (warp >= kStComputeWarps) grid_launch_dependents();

  // ------------------------------------------------------------------ compute warps
  float de_acc = 0.f;
  if (warp < kStComputeWarps) {
    const int g = warp >> 3, q = warp & 3, half = (warp >> 2) & 1, row = q * 32 + lane;
    grid_dependency_wait();
    if (TRANSFORM) {
      float cs[16], sn[16];
      int tab_next = 0;
      auto take_tables = [&](int k) {
        bool good = true;
        while (tab_next <= k && good) {
          uint32_t seen = 0;   // one word of every load below
          good = st_wait(bar_tab_full + 8 * (tab_next % ST), (tab_next / ST) & 1);
          if (good && tab_next == k) {
            const uint32_t tab = tab_buf + (tab_next % ST) * Cfg::TABLE_TILE;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              const uint32_t off = row * 128 + (((half * 4 + v) ^ (row & 7)) << 4);
              const float4 cv = ld_shared_f4(tab + off), sv = ld_shared_f4(tab + 16384 + off);
              cs[4 * v] = cv.x; cs[4 * v + 1] = cv.y; cs[4 * v + 2] = cv.z; cs[4 * v + 3] = cv.w;
              sn[4 * v] = sv.x; sn[4 * v + 1] = sv.y; sn[4 * v + 2] = sv.z; sn[4 * v + 3] = sv.w;
              seen ^= __float_as_uint(cv.w) ^ __float_as_uint(sv.w);
            }
          }
          if (good) {
            // the rows must be in registers before the buffer goes back to the table warp's next bulk copy
            wait_for_loaded(seen, tslot + 8);
            st_arrive(bar_tab_free + 8 * (tab_next % ST));
          }
          ++tab_next;
        }
        return good;
      };
      for (int j = g; j < n_tiles && ok; j += 2) {
        const uint32_t x_tile = x_ring + (j % SX) * Cfg::X_TILE;
        const uint32_t lo_tile = lo_ring + (j % SL) * Cfg::LO_TILE;
        if (ROT) {
          ok = take_tables(j);   // also passes the tiles of the other group
          if (!ok) break;
        }
        // Order matters.  A parity wait is only meaningful while the waiter is at most one phase behind the
        // barrier.  With an odd ring the last user of this X slot (tile j - SX) belonged to the OTHER group, so
        // this group has not observed that phase: were it to test the "full" barrier before that load had landed
        // (loads complete out of order), the test for tile j would pass at once on the phase before it and the
        // stale tile would be rotated.  The low-word slot comes back by tcgen05.commit after the MMAs of tile
        // j - SL, which (MMAs complete in order, SL <= SX) follow the other group's arrival for tile j - SX and
        // hence its genuine wait for that load: after this wait the barrier cannot be behind.  (Rings whose
        // length is even are used by one group only and need no such argument.)
        static_assert(!TRANSFORM || (SX % 2) == 0 || (ROT && SL <= SX), "X ring shared by the two groups");
        if (ROT && j >= SL) ok = st_wait(bar_lofree + 8 * (j % SL), ((j / SL) - 1) & 1);
        if (ok) ok = st_wait(bar_xfull + 8 * (j % SX), (j / SX) & 1);
        if (!ok) break;
        float dot = 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint32_t off = row * 128 + (((half * 4 + c) ^ (row & 7)) << 4);
          const uint4 v = ld_shared_v4(x_tile + off);
          const uint32_t w[4] = {v.x, v.y, v.z, v.w};
          if (GRAD) {
            const uint4 cv = ld_shared_v4(x_tile + 16384 + off);
            const uint32_t cw[4] = {cv.x, cv.y, cv.z, cv.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const float2 a = bf2_to_f2(w[k]), bb = bf2_to_f2(cw[k]);
              dot = fmaf(a.x, bb.x, dot);
              dot = fmaf(a.y, bb.y, dot);
            }
          }
          if (ROT) {
            uint32_t hi[4], lo[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const float2 f = bf2_to_f2(w[k]);
              const float2 r = rot_pair(f.x, f.y, cs[c * 4 + k], sn[c * 4 + k]);
              split2(r.x, r.y, hi[k], lo[k]);
            }
            st_shared_v4(x_tile + off, make_uint4(hi[0], hi[1], hi[2], hi[3]));
            st_shared_v4(lo_tile + off, make_uint4(lo[0], lo[1], lo[2], lo[3]));
          }
        }
        de_acc += dot;
        if (ROT) fence_async_shared();   // the MMAs read the tiles through the asynchronous proxy
        st_arrive(bar_xf + 8 * (j % SX));
      }
      while (ROT && ok && tab_next < n_tiles) {
        ok = st_wait(bar_tab_full + 8 * (tab_next % ST), (tab_next / ST) & 1);
        if (ok) st_arrive(bar_tab_free + 8 * (tab_next % ST));
        ++tab_next;
      }
    }

    // ---- the chunk's partial sums
    grid_launch_dependents();
    if (ok) ok = st_wait(bar_done, 0);
    tc::fence_after_sync();
    float* out = p.partials + ((size_t)(b * p.heads + h) * p.chunks + chunk) * p.partial_floats;
    const int sub = warp >> 2;   // the four warps of a lane quarter split the column blocks of 16
    const uint32_t lane_base = tmem + ((uint32_t)(q * 32) << 16);
    const uint32_t scratch = x_ring;   // [64 channels][r] floats: the low rows of the moment (the ring is idle now)
    if (ok && ROT && q >= 2) {
      // accumulator rows 64 .. 127 hold the products with the low word: hand them to the owners of rows 0 .. 63
      const int ch = (q - 2) * 32 + lane;
      for (int blk = sub; blk < R / 16; blk += 4) {
        uint32_t v[16];
        tc::tmem_ld16(lane_base + Cfg::COL_Q + blk * 16, v);
        tc::wait_ld();
#pragma unroll
        for (int e = 0; e < 16; e += 4)
          st_shared_v4(scratch + (uint32_t)(ch * R + blk * 16 + e) * 4u, make_uint4(v[e], v[e + 1], v[e + 2], v[e + 3]));
      }
    }
    asm volatile("bar.sync 2, %0;\n" ::"n"(kStComputeWarps * 32) : "memory");
    if (ok) {
      // moment: thread = channel (rows 0 .. 63 of the accumulator: lanes 0 .. 63 with rotation; without, the 64-row
      // form keeps rows 16k .. 16k + 15 in lanes 32k .. 32k + 15), written as Q[relation][channel]
      const bool has_q = ROT ? q < 2 : lane < 16;
      const int ch = ROT ? q * 32 + lane : q * 16 + lane;
      float* qout = out + (GRAD ? 0 : R * R);
      for (int blk = sub; blk < R / 16; blk += 4) {
        uint32_t v[16];
        tc::tmem_ld16(lane_base + Cfg::COL_Q + blk * 16, v);
        tc::wait_ld();
        if (has_q) {
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            float val = __uint_as_float(v[e]);
            if (ROT) {
              float low;
              asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(low) : "r"(scratch + (uint32_t)(ch * R + blk * 16 + e) * 4u));
              val += low;
            }
            qout[(blk * 16 + e) * 64 + ch] = val;
          }
        }
      }
      if (!GRAD) {
        // Gram: accumulator row m = column m of the relation box (64-row form); rows below r are this head's
        const int m = q * 16 + lane;
        const bool has_g = lane < 16 && m < R;
        for (int blk = sub; blk < R / 16; blk += 4) {
          uint32_t v[16];
          tc::tmem_ld16(lane_base + Cfg::COL_G + blk * 16, v);
          tc::wait_ld();
          if (has_g) {
            float* dst = out + m * R + blk * 16;
#pragma unroll
            for (int e = 0; e < 16; e += 4)
              *reinterpret_cast<float4*>(dst + e) = make_float4(__uint_as_float(v[e]), __uint_as_float(v[e + 1]),
                                                                __uint_as_float(v[e + 2]), __uint_as_float(v[e + 3]));
          }
        }
      }
    }
    if (GRAD) {
      // <dY, C> of the chunk: fixed shuffle tree, then the sixteen warps in order
      float v = de_acc;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0) st_shared_f32(de_red + warp * 4, v);
    }
    if (!ok && lane == 0) atomicExch(p.error, kErrBarrierTimeout);
  }

  tc::fence_before_sync();
  __syncthreads();
  if (GRAD && tid == 0) {
    float v = 0.f;
    for (int w = 0; w < kStComputeWarps; ++w) {
      float part;
      asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(part) : "r"(de_red + w * 4));
      v += part;
    }
    float* de = p.de_partials + ((size_t)(b * p.heads + h) * p.chunks + chunk) * p.de_slots;
    de[0] = v;
    for (int sidx = 1; sidx < p.de_slots; ++sidx) de[sidx] = 0.f;
  }
  if (warp == kMmaWarp) tc::tmem_free(tmem, Cfg::TMEM_COLS);
}

template <int R, bool GRAD, bool ROT>
static int launch_stats_tc_one(const ms_shape& s, const Plan& plan, const void* projected, const void* dy,
                               const float* cos, const float* sin, StatsTcParams& p, bool fuse_core, cudaStream_t st) {
  using Cfg = StatsTcCfg<R, GRAD, ROT>;
  const int heads = s.heads, width = heads * (R + 64), dmodel = heads * 64;
  CUtensorMap map_a, map_c, map_y, map_cos, map_sin;
  {
    const uint64_t dims[3] = {(uint64_t)width, (uint64_t)s.tokens, (uint64_t)s.batch};
    const uint64_t str[2] = {(uint64_t)width * 2, (uint64_t)s.tokens * width * 2};
    const uint32_t box[3] = {64, kStTile, 1};
    if (encode_tensor_map(&map_a, const_cast<void*>(projected), 2, 3, dims, str, box, Swizzle::B128)) return MS_ERR_LAUNCH;
    map_c = map_a;
  }
  map_y = map_c;
  if (GRAD) {
    const uint64_t dims[3] = {(uint64_t)dmodel, (uint64_t)s.tokens, (uint64_t)s.batch};
    const uint64_t str[2] = {(uint64_t)dmodel * 2, (uint64_t)s.tokens * dmodel * 2};
    const uint32_t box[3] = {64, kStTile, 1};
    if (encode_tensor_map(&map_y, const_cast<void*>(dy), 2, 3, dims, str, box, Swizzle::B128)) return MS_ERR_LAUNCH;
  }
  map_cos = map_c;
  map_sin = map_c;
  if (ROT) {
    const uint64_t dims[3] = {32, (uint64_t)s.tokens, (uint64_t)s.rotary_rows};
    const uint64_t str[2] = {128, (uint64_t)s.tokens * 128};
    const uint32_t box[3] = {32, kStTile, 1};
    if (encode_tensor_map(&map_cos, const_cast<float*>(cos), 4, 3, dims, str, box, Swizzle::B128)) return MS_ERR_LAUNCH;
    if (encode_tensor_map(&map_sin, const_cast<float*>(sin), 4, 3, dims, str, box, Swizzle::B128)) return MS_ERR_LAUNCH;
  }
  int smem_bytes = Cfg::TOTAL;
  int spare = 0;
  if (fuse_core) {
    const int core_bytes = (int)core_forward_smem_bytes(R) + 1024;
    if (smem_bytes < core_bytes) smem_bytes = core_bytes;
    spare = 1;   // one slab of gridDim.y * gridDim.z CTAs holds a CTA per head
  }
  auto kern = stats_tc_kernel<R, GRAD, ROT>;
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem_bytes)) return MS_ERR_LAUNCH;
  dim3 grid(plan.chunks + spare, heads, s.batch);
  launch_kernel(kern, grid, dim3(kStThreads), smem_bytes, st, map_a, map_c, map_y, map_cos, map_sin, p);
  return cudaGetLastError() == cudaSuccess ? MS_OK : MS_ERR_LAUNCH;
}

template <int R>
static int launch_stats_tc_r(const ms_shape& s, const Plan& plan, bool grad, const void* projected, const void* dy,
                             const float* cos, const float* sin, StatsTcParams& p, bool fuse_core, cudaStream_t st) {
  const bool rot = s.rotary_rows > 0;
  if (grad) return rot ? launch_stats_tc_one<R, true, true>(s, plan, projected, dy, cos, sin, p, false, st)
                       : launch_stats_tc_one<R, true, false>(s, plan, projected, dy, cos, sin, p, false, st);
  return rot ? launch_stats_tc_one<R, false, true>(s, plan, projected, dy, cos, sin, p, fuse_core, st)
             : launch_stats_tc_one<R, false, false>(s, plan, projected, dy, cos, sin, p, fuse_core, st);
}

// Heads per CTA of this kernel (the launch planner sizes the token chunks with it): one.
int stats_tc_group_heads(int) { return 1; }

// MS_OK / error, or -1 when the shape is outside this kernel's envelope (the plan must have been made for it:
// plan.stats_tc).
int launch_stats_tc(const ms_shape& s, const Plan& plan, bool grad, const void* projected, const void* dy,
                    const float* cos, const float* sin, float* partials, float* de_partials, const float* base_raw,
                    const float* eta_raw, const ms_tape* core_tape, cudaStream_t st) {
  if (!plan.stats_tc || !plan.aligned || s.head_dim != 64) return -1;
  if ((plan.chunk_tokens % kStTile) != 0 || s.batch > 65535) return -1;
  StatsTcParams p;
  p.partials = partials; p.de_partials = de_partials;
  p.error = device_error_word();
  if (!p.error) return MS_ERR_LAUNCH;
  p.tokens = s.tokens; p.heads = s.heads; p.rotary_rows = s.rotary_rows;
  p.chunks = plan.chunks; p.chunk_tokens = plan.chunk_tokens; p.de_slots = plan.de_slots;
  p.partial_floats = (int)(grad ? plan.bwd_partial_floats : plan.fwd_partial_floats);
  const bool fuse_core = !grad && core_tape != nullptr;
  p.base_raw = base_raw; p.eta_raw = eta_raw;
  p.eta = fuse_core ? core_tape->eta : nullptr;
  p.eta_slope = fuse_core ? core_tape->eta_slope : nullptr;
  p.core_map = fuse_core ? core_tape->core_map : nullptr;
  p.core_info = fuse_core ? core_tape->core_info : nullptr;
  p.complement = s.complement;
  switch (s.rank) {
    case 16: return launch_stats_tc_r<16>(s, plan, grad, projected, dy, cos, sin, p, fuse_core, st);
    case 32: return launch_stats_tc_r<32>(s, plan, grad, projected, dy, cos, sin, p, fuse_core, st);
    case 64: return launch_stats_tc_r<64>(s, plan, grad, projected, dy, cos, sin, p, fuse_core, st);
  }
  return -1;
}

}  // namespace ms
