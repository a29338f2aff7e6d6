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
// written once.  tcgen05 wants at least 64 accumulator rows: a CTA therefore takes a GROUP of heads whose
// relation columns are adjacent in `projected` (2 heads at rank 32 or 64, 4 at rank 16 -> 64 or 128 columns
// = accumulator rows) and one chunk of tokens.  Per 128-token tile and k-step of 16 tokens:
//
//   G block   D_G [rows x rows]  += A_grp^T A_grp        (the diagonal r x r blocks are the heads' Grams)
//   per head  D_Q[h] [rows x 64] += A_grp^T X_h(high) + A_grp^T X_h(low)     (rows of head h are its moment)
//
// Both MMA operands are token-major tiles exactly as TMA delivers them (rows = tokens): the "M-major" /
// "N-major" shared-memory operand forms.  With rotation, compute warps rotate each content (or gradient)
// tile in FP32, write the high BF16 word over the raw tile and the low word to a second tile; the MMAs read
// both.  Without rotation the raw tile is the operand.
//
//   warp 16 (one thread)  TMA: content / gradient tiles (and, for the adjoint, the content tile of <dY, C>)
//   warp 19 (one thread)  TMA: relation tiles of the head group
//   warp 18 (one thread)  TMA: cos / sin rows of the next token tile
//   warp 17               MMA issue (warp-uniform control flow, an elected lane issues each batch); shared
//                         memory is handed back to the TMA warps by tcgen05.commit on their "free" barriers
//   warps 0-7 / 8-15      two groups that alternate (tile, head) units: rotate + split (half a token row per
//                         thread); at the end all sixteen read the accumulators and write the chunk's partial
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
  static constexpr int G = R == 16 ? 4 : 2;              // heads per CTA
  static constexpr int ROWS = G * R;                      // accumulator rows: 64 or 128
  static constexpr int A_TILE = kStTile * ROWS * 2;       // 16 or 32 KB (one or two 64-column tiles)
  static constexpr int A_STAGES = R == 64 ? 2 : 3;
  static constexpr int X_TILE = GRAD ? 32768 : 16384;     // gradient (+ content for <dY, C>) or content
  // an odd ring is shared by the two compute groups, which is only safe together with the low-word ring (see the
  // waits of the compute warps); without rotation there is none, and room for four stages
  static constexpr int X_STAGES = (GRAD && ROT) ? 3 : 4;
  // low-word tiles: a deep ring lets a compute group rotate its next unit while the MMAs of its last one run
  static constexpr int LO_STAGES = !ROT ? 0 : (!GRAD ? 4 : (R == 64 ? 2 : 3));
  static constexpr int LO_TILE = 16384;
  static constexpr int TABLE_BYTES = ROT ? 32768 : 0;
  static constexpr int BAR_BYTES = (2 * A_STAGES + 3 * X_STAGES + 4 + 4) * 8 + 16 + 16 * 4 * 4;
  static constexpr int TOTAL = 1024 + A_STAGES * A_TILE + X_STAGES * X_TILE + LO_STAGES * LO_TILE + TABLE_BYTES + BAR_BYTES;
  static constexpr int COL_Q = GRAD ? 0 : ROWS;           // first column of the per-head accumulators
  static constexpr int COLS = COL_Q + G * 64;
  static constexpr int TMEM_COLS = COLS <= 128 ? 128 : (COLS <= 256 ? 256 : 512);
  static_assert(TOTAL <= 227 * 1024, "shared memory");
};

struct StatsTcParams {
  float* partials;
  float* de_partials;
  int* error;
  int tokens, heads, rotary_rows, chunks, chunk_tokens, de_slots, partial_floats, groups;
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
  constexpr int G = Cfg::G, ROWS = Cfg::ROWS, SA = Cfg::A_STAGES, SX = Cfg::X_STAGES, SL = ROT ? Cfg::LO_STAGES : 1;
  constexpr bool TRANSFORM = ROT || GRAD;   // the compute warps touch every (tile, head) unit
  constexpr int kXWarp = kStComputeWarps, kMmaWarp = kStComputeWarps + 1, kTableWarp = kStComputeWarps + 2,
                kAWarp = kStComputeWarps + 3;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t smem = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  grid_launch_dependents();

  const int chunk = blockIdx.x;
  if (chunk >= p.chunks) {
    // spare CTAs of the forward grid: the per-head core runs beside the token reduction
    grid_dependency_wait();
    const int head = (chunk - p.chunks) * (int)gridDim.y * (int)gridDim.z + (int)blockIdx.z * (int)gridDim.y + (int)blockIdx.y;
    if (!GRAD && head < p.heads)
      core_forward_device<R, kStThreads>(p.base_raw, p.eta_raw, head, p.complement, p.eta, p.eta_slope, p.core_map,
                                         p.core_info, smem_raw + (smem - smem_u32(smem_raw)), tid);
    return;
  }

  const int b = blockIdx.z;
  const int h0 = blockIdx.y * G;
  const int gh = min(G, p.heads - h0);
  const uint32_t a_ring = smem;
  const uint32_t x_ring = a_ring + SA * Cfg::A_TILE;
  const uint32_t lo_ring = x_ring + SX * Cfg::X_TILE;
  const uint32_t tab_buf = lo_ring + Cfg::LO_STAGES * Cfg::LO_TILE;
  const uint32_t bar_afull = tab_buf + Cfg::TABLE_BYTES;
  const uint32_t bar_afree = bar_afull + 8 * SA;
  const uint32_t bar_xfull = bar_afree + 8 * SA;
  const uint32_t bar_xfree = bar_xfull + 8 * SX;
  const uint32_t bar_xf = bar_xfree + 8 * SX;          // unit rotated / inspected by the compute warps
  const uint32_t bar_lofree = bar_xf + 8 * SX;         // up to four
  const uint32_t bar_tab_full = bar_lofree + 32, bar_tab_free = bar_tab_full + 8;
  const uint32_t bar_done = bar_tab_free + 8;
  const uint32_t tslot = bar_done + 8;
  const uint32_t de_red = tslot + 16;                  // [16 warps][4 heads] floats

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
    mbar_init(bar_tab_full, 1);
    mbar_init(bar_tab_free, 2 * kStGroupThreads);
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
  const int n_units = n_tiles * gh;                            // (tile, head) units, tile-major
  bool ok = true;

  if (warp == kXWarp) {
    // ---------------------------------------------------------------- content / gradient tiles
    if (lane == 0) {
      grid_dependency_wait();
      for (int j = 0; j < n_units; ++j) {
        if (j >= SX) {
          ok = mbar_wait(bar_xfree + 8 * (j % SX), ((j / SX) - 1) & 1);   // the MMAs that read the slot have completed
          if (!ok) break;
        }
        const int t = j / gh, h = h0 + (j - t * gh);
        const uint32_t dst = x_ring + (j % SX) * Cfg::X_TILE, bar = bar_xfull + 8 * (j % SX);
        mbar_expect_tx(bar, Cfg::X_TILE);
        if (GRAD) {
          tma_load_3d(dst, &map_y, h * 64, tok0 + t * kStTile, b, bar);
          tma_load_3d(dst + 16384, &map_c, p.heads * R + h * 64, tok0 + t * kStTile, b, bar);
        } else {
          tma_load_3d(dst, &map_c, p.heads * R + h * 64, tok0 + t * kStTile, b, bar);
        }
      }
      if (!ok) atomicExch(p.error, kErrBarrierTimeout);
    }
  } else if (warp == kAWarp) {
    // ---------------------------------------------------------------- relation tiles of the head group
    if (lane == 0) {
      grid_dependency_wait();
      for (int t = 0; t < n_tiles; ++t) {
        if (t >= SA) {
          ok = mbar_wait(bar_afree + 8 * (t % SA), ((t / SA) - 1) & 1);
          if (!ok) break;
        }
        const uint32_t dst = a_ring + (t % SA) * Cfg::A_TILE, bar = bar_afull + 8 * (t % SA);
        mbar_expect_tx(bar, Cfg::A_TILE);
#pragma unroll
        for (int part = 0; part < ROWS / 64; ++part)
          tma_load_3d(dst + part * 16384, &map_a, h0 * R + part * 64, tok0 + t * kStTile, b, bar);
      }
      if (!ok) atomicExch(p.error, kErrBarrierTimeout);
    }
  } else if (warp == kTableWarp) {
    // ---------------------------------------------------------------- cos / sin rows
    if (ROT && lane == 0) {
      grid_dependency_wait();
      const int tab_b = p.rotary_rows > 1 ? b : 0;
      for (int k = 0; k < n_tiles; ++k) {
        if (k > 0) {
          ok = mbar_wait(bar_tab_free, (k - 1) & 1);
          if (!ok) break;
        }
        mbar_expect_tx(bar_tab_full, 32768);
        tma_load_3d(tab_buf, &map_cos, 0, tok0 + k * kStTile, tab_b, bar_tab_full);
        tma_load_3d(tab_buf + 16384, &map_sin, 0, tok0 + k * kStTile, tab_b, bar_tab_full);
      }
      if (!ok) atomicExch(p.error, kErrBarrierTimeout);
    }
  } else if (warp == kMmaWarp) {
    // ---------------------------------------------------------------- MMA issuer
    constexpr uint32_t IDESC_G = tc::idesc_bf16(ROWS, ROWS, true, true);
    constexpr uint32_t IDESC_Q = tc::idesc_bf16(ROWS, 64, true, true);
    constexpr uint32_t HI = tc::desc_hi_n_major_128();
    // low descriptor word of a token-major tile: start address / 16, and 16384 bytes between its 64-column halves
    const uint32_t lbo = (16384u >> 4) << 16;
    const uint32_t a_lo0 = ((a_ring & 0x3ffffu) >> 4) | lbo, x_lo0 = ((x_ring & 0x3ffffu) >> 4) | lbo,
                   l_lo0 = ((lo_ring & 0x3ffffu) >> 4) | lbo;
    for (int t = 0; t < n_tiles && ok; ++t) {
      ok = st_wait(bar_afull + 8 * (t % SA), (t / SA) & 1);
      if (!ok) break;
      tc::fence_after_sync();
      const uint32_t a_lo = a_lo0 + (uint32_t)((t % SA) * (Cfg::A_TILE >> 4));
      if (!GRAD) {
        if (tc::elect_one()) {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            tc::mma_ss_raw<HI, HI, IDESC_G>(tmem, a_lo + ks * 128, a_lo + ks * 128, (t | ks) != 0);
        }
        __syncwarp();
      }
      for (int hl = 0; hl < gh && ok; ++hl) {
        const int j = t * gh + hl;
        ok = st_wait((TRANSFORM ? bar_xf : bar_xfull) + 8 * (j % SX), (j / SX) & 1);
        if (!ok) break;
        tc::fence_after_sync();
        const uint32_t x_lo = x_lo0 + (uint32_t)((j % SX) * (Cfg::X_TILE >> 4));
        const uint32_t l_lo = l_lo0 + (uint32_t)((j % SL) * (Cfg::LO_TILE >> 4));
        const uint32_t d = tmem + Cfg::COL_Q + hl * 64;
        if (tc::elect_one()) {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            if (ROT) tc::mma_ss_raw<HI, HI, IDESC_Q>(d, a_lo + ks * 128, l_lo + ks * 128, (t | ks) != 0);
            tc::mma_ss_raw<HI, HI, IDESC_Q>(d, a_lo + ks * 128, x_lo + ks * 128, ROT || (t | ks) != 0);
          }
          tc::mma_commit_raw(bar_xfree + 8 * (j % SX));
          if (ROT) tc::mma_commit_raw(bar_lofree + 8 * (j % SL));
          if (hl == gh - 1) tc::mma_commit_raw(bar_afree + 8 * (t % SA));
        }
        __syncwarp();
      }
    }
    if (ok) {
      if (tc::elect_one()) tc::mma_commit_raw(bar_done);
      __syncwarp();
    }
    if (!ok && lane == 0) atomicExch(p.error, kErrBarrierTimeout);
  }

  // ------------------------------------------------------------------ compute warps
  float de_acc[G];
#pragma unroll
  for (int e = 0; e < G; ++e) de_acc[e] = 0.f;
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
          good = st_wait(bar_tab_full, tab_next & 1);
          if (good && tab_next == k) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              const uint32_t off = row * 128 + (((half * 4 + v) ^ (row & 7)) << 4);
              const float4 cv = ld_shared_f4(tab_buf + off), sv = ld_shared_f4(tab_buf + 16384 + off);
              cs[4 * v] = cv.x; cs[4 * v + 1] = cv.y; cs[4 * v + 2] = cv.z; cs[4 * v + 3] = cv.w;
              sn[4 * v] = sv.x; sn[4 * v + 1] = sv.y; sn[4 * v + 2] = sv.z; sn[4 * v + 3] = sv.w;
              seen ^= __float_as_uint(cv.w) ^ __float_as_uint(sv.w);
            }
          }
          if (good) {
            // the rows must be in registers before the buffer goes back to the table warp's next bulk copy
            wait_for_loaded(seen, tslot + 8);
            st_arrive(bar_tab_free);
          }
          ++tab_next;
        }
        return good;
      };
      for (int j = g; j < n_units && ok; j += 2) {
        const int t = j / gh, hl = j - t * gh;
        const uint32_t x_tile = x_ring + (j % SX) * Cfg::X_TILE;
        const uint32_t lo_tile = lo_ring + (j % SL) * Cfg::LO_TILE;
        if (ROT && t >= tab_next) {
          ok = take_tables(t);
          if (!ok) break;
        }
        // Order matters.  A parity wait is only meaningful while the waiter is at most one phase behind the
        // barrier.  With an odd ring the last user of this X slot (unit j - SX) belonged to the OTHER group, so
        // this group has not observed that phase: were it to test the "full" barrier before that load had landed
        // (loads complete out of order), the test for unit j would pass at once on the phase before it and the
        // stale tile would be rotated.  The low-word slot comes back by tcgen05.commit after the MMAs of unit
        // j - SL, which (MMAs complete in order, SL <= SX) follow the other group's arrival for unit j - SX and
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
        if (GRAD) {
#pragma unroll
          for (int e = 0; e < G; ++e)
            if (e == hl) de_acc[e] += dot;
        }
        if (ROT) fence_async_shared();   // the MMAs read the tiles through the asynchronous proxy
        st_arrive(bar_xf + 8 * (j % SX));
      }
      while (ROT && ok && tab_next < n_tiles) {
        ok = st_wait(bar_tab_full, tab_next & 1);
        if (ok) st_arrive(bar_tab_free);
        ++tab_next;
      }
    }

    // ---- the chunk's partial sums: accumulator row m = relation column m of the group
    if (ok) ok = st_wait(bar_done, 0);
    tc::fence_after_sync();
    if (ok) {
      // ROWS = 128: lane of tensor memory = row; ROWS = 64: rows 16k .. 16k + 15 sit in lanes 32k .. 32k + 15
      const int m = ROWS == 128 ? q * 32 + lane : q * 16 + lane;
      const bool has_row = ROWS == 128 || lane < 16;
      const int hl = m / R, i = m - hl * R;
      const bool live = has_row && hl < gh;
      const int sub = warp >> 2;   // the four warps of a lane quarter split the columns
      const uint32_t lane_base = tmem + ((uint32_t)(q * 32) << 16);
      float* out = p.partials + ((size_t)(b * p.heads + h0 + (live ? hl : 0)) * p.chunks + chunk) * p.partial_floats;
      // column blocks of 16: the Gram block of this row's head (R / 16 blocks), then its 64 moment columns
      constexpr int GB = GRAD ? 0 : R / 16, NB = GB + 4;
      for (int blk = sub; blk < NB; blk += 4) {
        uint32_t v[16];
        const bool gram = blk < GB;
        const int col = gram ? hl * R + blk * 16 : Cfg::COL_Q + hl * 64 + (blk - GB) * 16;
        tc::tmem_ld16(lane_base + (live ? col : 0), v);
        tc::wait_ld();
        if (live) {
          float* dst = gram ? out + i * R + blk * 16 : out + (GRAD ? 0 : R * R) + i * 64 + (blk - GB) * 16;
#pragma unroll
          for (int e = 0; e < 16; e += 4)
            *reinterpret_cast<float4*>(dst + e) = make_float4(__uint_as_float(v[e]), __uint_as_float(v[e + 1]),
                                                              __uint_as_float(v[e + 2]), __uint_as_float(v[e + 3]));
        }
      }
    }
    if (GRAD) {
      // <dY, C> of the chunk per head: fixed shuffle tree, then the sixteen warps in order
#pragma unroll
      for (int e = 0; e < G; ++e) {
        float v = de_acc[e];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0) st_shared_f32(de_red + (warp * 4 + e) * 4, v);
      }
    }
    if (!ok && lane == 0) atomicExch(p.error, kErrBarrierTimeout);
  }

  tc::fence_before_sync();
  __syncthreads();
  if (GRAD && tid < gh) {
    float v = 0.f;
    for (int w = 0; w < kStComputeWarps; ++w) {
      float part;
      asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(part) : "r"(de_red + (w * 4 + tid) * 4));
      v += part;
    }
    float* de = p.de_partials + ((size_t)(b * p.heads + h0 + tid) * p.chunks + chunk) * p.de_slots;
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
  p.groups = (heads + Cfg::G - 1) / Cfg::G;
  int smem_bytes = Cfg::TOTAL;
  int spare = 0;
  if (fuse_core) {
    const int core_bytes = (int)core_forward_smem_bytes(R) + 1024;
    if (smem_bytes < core_bytes) smem_bytes = core_bytes;
    const int per_x = p.groups * s.batch;            // spare CTAs come in slabs of gridDim.y * gridDim.z
    spare = (heads + per_x - 1) / per_x;
  }
  auto kern = stats_tc_kernel<R, GRAD, ROT>;
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem_bytes)) return MS_ERR_LAUNCH;
  dim3 grid(plan.chunks + spare, p.groups, s.batch);
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

// Heads per CTA of this kernel (the launch planner sizes the token chunks with it).
int stats_tc_group_heads(int rank) { return rank == 16 ? 4 : 2; }

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
