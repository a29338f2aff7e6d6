// Token-parallel passes of the MemSolve mixer.
//
//   readout         Y  = eta*C + rot^-1(A_raw W) / sqrt(n)
//   token backward  dA = s*( A_raw S' + rot(dY) W^T + rot(C) dQ^T ),   S' = s (dG+dG^T),   s = 1/sqrt(n)
//                   dC = eta*dY + s * rot^-1(A_raw dQ)
//
// Replaces the reference's `_readout` and `_token_backward` (memsolve/ball/cuda.py:1670-1922).
// One CTA owns a tile of 64 tokens of one sample and walks over all heads (and 64-channel
// blocks), so the rotary table entries of its tokens are fetched once and stay in registers.
// Per head the relation/content/gradient tiles and the head's compact matrices (two BF16
// words each) arrive through a cp.async pipeline in swizzled shared memory; each warp owns 16
// token rows, products are mma.sync.m16n8k16 with FP32 accumulation, results are written back
// into the tile in shared memory and leave with 16-byte coalesced stores.
#include "ms_core.cuh"
#include "ms_frag.cuh"

namespace ms {

constexpr int kTokenThreads = 128;

struct TokenParams {
  const __nv_bfloat16* projected;
  const __nv_bfloat16* dy;          // backward only
  const float* cos;
  const float* sin;
  const float* counts;
  const float* eta;
  const __nv_bfloat16* coeff;       // [systems][2][r][dpad]
  const __nv_bfloat16* gram_grad;   // [systems][2][r][r]      backward only
  const __nv_bfloat16* cross_grad;  // [systems][2][r][dpad]   backward only
  __nv_bfloat16* out;               // mixed [B,N,D] or dprojected [B,N,W]
  int batch, tokens, heads, head_dim, width, rotary_rows, dblocks, dpad;
  // per-head core adjoint, computed by spare CTAs blockIdx.x >= tiles (backward only, optional)
  const float* base_raw;
  const float* hmat;
  const float* de_sys;
  const float* eta_slope;
  const float* core_map;
  float* d_base;
  float* d_eta_raw;
  float grad_scale;
  int complement, tiles;
};

// coalesced store of a [64 x cols] BF16 tile from swizzled shared memory
template <bool ALIGNED>
__device__ __forceinline__ void store_tile_bf16(uint32_t tile, int tile_cols, __nv_bfloat16* dst, long stride,
                                                int rows_valid, int cols_valid, int tid) {
  const int pitch = tile_cols * 2;
  if (ALIGNED) {
    const int cpr = tile_cols >> 3;
    for (int i = tid; i < kTileTokens * cpr; i += kTokenThreads) {
      const int row = i / cpr, c = i - row * cpr;
      if (row < rows_valid && c * 8 < cols_valid) {
        uint4 v = ld_shared_v4(tile + swz(row * pitch + c * 16));
        *reinterpret_cast<uint4*>(dst + (long)row * stride + c * 8) = v;
      }
    }
  } else {
    unsigned short* d16 = reinterpret_cast<unsigned short*>(dst);
    for (int i = tid; i < kTileTokens * tile_cols; i += kTokenThreads) {
      const int row = i / tile_cols, c = i - row * tile_cols;
      if (row < rows_valid && c < cols_valid) {
        unsigned short v;
        asm volatile("ld.shared.u16 %0, [%1];\n" : "=h"(v) : "r"(tile + swz(row * pitch + c * 2)));
        d16[(long)row * stride + c] = v;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// readout
// ---------------------------------------------------------------------------------------
template <int R>
struct ReadoutSmem {
  static constexpr int A_BYTES = kTileTokens * R * 2;
  static constexpr int C_BYTES = kTileTokens * 128;
  static constexpr int W_BYTES = R * 128;  // one word (high or residual), 64 channels
  static constexpr int STAGE = A_BYTES + C_BYTES + 2 * W_BYTES;
  static constexpr int STAGES = 3;
  static constexpr int TOTAL = STAGE * STAGES + 128;
};

template <int R, bool ROT, bool ALIGNED>
__global__ void __launch_bounds__(kTokenThreads)
readout_kernel(const TokenParams p) {
  using Sm = ReadoutSmem<R>;
  constexpr int STAGES = Sm::STAGES;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t smem = (smem_u32(smem_raw) + 127u) & ~127u;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  grid_launch_dependents();
  grid_dependency_wait();
  const int b = blockIdx.y;
  const int tk = blockIdx.x * kTileTokens;
  const int rows = min(kTileTokens, p.tokens - tk);
  const int d = p.head_dim, dmodel = p.heads * d, half = d >> 1;
  const int items = p.heads * p.dblocks;
  const float n = p.counts ? p.counts[b] : (float)p.tokens;
  const float inv_s = inv_sqrt_rn(n);

  const __nv_bfloat16* rowbase = p.projected + ((long)b * p.tokens + tk) * p.width;
  __nv_bfloat16* outbase = p.out + ((long)b * p.tokens + tk) * dmodel;
  const long tab_row0 = (p.rotary_rows > 1 ? (long)b * p.tokens : 0) + tk + warp * 16;

  auto issue = [&](int it, int s) {
    const int h = it / p.dblocks, jb = it - h * p.dblocks;
    const int d0 = jb * 64, dv = min(64, d - d0);
    uint32_t base = smem + s * Sm::STAGE;
    load_tile_bf16<ALIGNED>(base, kTileTokens, R, rowbase + h * R, p.width, rows, R, tid, kTokenThreads);
    base += Sm::A_BYTES;
    load_tile_bf16<ALIGNED>(base, kTileTokens, 64, rowbase + p.heads * R + h * d + d0, p.width, rows, dv, tid, kTokenThreads);
    base += Sm::C_BYTES;
    const __nv_bfloat16* w = p.coeff + ((size_t)(b * p.heads + h) * 2) * R * p.dpad + d0;
    const int wv = min(64, p.dpad - d0);
    load_tile_bf16<true>(base, R, 64, w, p.dpad, R, wv, tid, kTokenThreads);
    load_tile_bf16<true>(base + Sm::W_BYTES, R, 64, w + (size_t)R * p.dpad, p.dpad, R, wv, tid, kTokenThreads);
  };

#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < items) issue(s, s);
    cp_async_commit();
  }

  TableFrag tab;
  int tab_jb = -1;
  const int g = lane >> 2, tq = lane & 3;
  const int mi = lane >> 3, mr = lane & 7;

  for (int it = 0; it < items; ++it) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();
    {
      const int nx = it + STAGES - 1;
      if (nx < items) issue(nx, nx % STAGES);
      cp_async_commit();
    }
    const int h = it / p.dblocks, jb = it - h * p.dblocks;
    const int d0 = jb * 64, dv = min(64, d - d0);
    const uint32_t a_tile = smem + (it % STAGES) * Sm::STAGE;
    const uint32_t c_tile = a_tile + Sm::A_BYTES;
    const uint32_t wh_tile = c_tile + Sm::C_BYTES;
    const uint32_t wl_tile = wh_tile + Sm::W_BYTES;
    if (ROT && jb != tab_jb) {
      load_table_frag(tab, p.cos, p.sin, tab_row0, rows - warp * 16, half, d0 >> 1, dv >> 1, lane);
      tab_jb = jb;
    }
    const float eta = p.eta[h];

    float acc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int k = 0; k < 4; ++k) acc[j][k] = 0.f;

#pragma unroll
    for (int ks = 0; ks < R / 16; ++ks) {
      uint32_t af[4];
      ldsm_x4(af, a_tile + swz((warp * 16 + mr + 8 * (mi & 1)) * (R * 2) + (ks * 16 + 8 * (mi >> 1)) * 2));
#pragma unroll
      for (int n2 = 0; n2 < 4; ++n2) {
        const uint32_t off = swz((ks * 16 + mr + 8 * (mi & 1)) * 128 + (n2 * 16 + 8 * (mi >> 1)) * 2);
        uint32_t bf[4];
        ldsm_x4_t(bf, wl_tile + off);
        mma_bf16(acc[2 * n2], af, bf[0], bf[1]);
        mma_bf16(acc[2 * n2 + 1], af, bf[2], bf[3]);
        ldsm_x4_t(bf, wh_tile + off);
        mma_bf16(acc[2 * n2], af, bf[0], bf[1]);
        mma_bf16(acc[2 * n2 + 1], af, bf[2], bf[3]);
      }
    }
    // epilogue in place on the content tile (each warp touches only its own 16 rows)
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int row = warp * 16 + g + 8 * k;
        const uint32_t addr = c_tile + swz(row * 128 + (8 * j + 2 * tq) * 2);
        float2 corr = make_float2(acc[j][2 * k], acc[j][2 * k + 1]);
        if (ROT) corr = rot_pair(corr.x, corr.y, tab.c[j][k], -tab.s[j][k]);
        const float2 cv = bf2_to_f2(ld_shared_u32(addr));
        st_shared_u32(addr, f2_to_bf2(fmaf(corr.x, inv_s, eta * cv.x), fmaf(corr.y, inv_s, eta * cv.y)));
      }
    }
    __syncthreads();
    store_tile_bf16<ALIGNED>(c_tile, 64, outbase + h * d + d0, dmodel, rows, dv, tid);
  }
  cp_async_wait<0>();
}

// ---------------------------------------------------------------------------------------
// token backward
// ---------------------------------------------------------------------------------------
template <int R>
struct TokenBwdSmem {
  static constexpr int A_BYTES = kTileTokens * R * 2;
  static constexpr int C_BYTES = kTileTokens * 128;
  static constexpr int W_BYTES = R * 128;
  static constexpr int S_BYTES = R * R * 2;
  // A, C, dY, W hi/lo, dQ hi/lo, S hi/lo
  static constexpr int STAGE = A_BYTES + 2 * C_BYTES + 4 * W_BYTES + 2 * S_BYTES;
  static constexpr int STAGES = 2;
  static constexpr int CORE = (int)core_backward_smem_bytes(R);
  static constexpr int TOTAL = (STAGE * STAGES > CORE ? STAGE * STAGES : CORE) + 128;
};

template <int R, bool ROT, bool ALIGNED>
__global__ void __launch_bounds__(kTokenThreads)
token_backward_kernel(const TokenParams p) {
  using Sm = TokenBwdSmem<R>;
  constexpr int STAGES = Sm::STAGES;
  constexpr int NR = R / 8;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t smem = (smem_u32(smem_raw) + 127u) & ~127u;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  grid_launch_dependents();
  grid_dependency_wait();
  const int b = blockIdx.y;
  if ((int)blockIdx.x >= p.tiles) {
    // spare CTAs: parameter gradients of one head each, beside the token pass
    if (b == 0)
      core_backward_device(p.base_raw, p.hmat, p.de_sys, p.eta_slope, p.core_map, R, blockIdx.x - p.tiles,
                           p.heads, p.batch, p.complement, p.grad_scale, p.d_base, p.d_eta_raw,
                           smem_raw + (smem - smem_u32(smem_raw)), tid, kTokenThreads);
    return;
  }
  const int tk = blockIdx.x * kTileTokens;
  const int rows = min(kTileTokens, p.tokens - tk);
  const int d = p.head_dim, dmodel = p.heads * d, half = d >> 1;
  const int items = p.heads * p.dblocks;
  const float n = p.counts ? p.counts[b] : (float)p.tokens;
  const float inv_s = inv_sqrt_rn(n);

  const __nv_bfloat16* rowbase = p.projected + ((long)b * p.tokens + tk) * p.width;
  const __nv_bfloat16* dybase = p.dy + ((long)b * p.tokens + tk) * dmodel;
  __nv_bfloat16* outbase = p.out + ((long)b * p.tokens + tk) * p.width;
  const long tab_row0 = (p.rotary_rows > 1 ? (long)b * p.tokens : 0) + tk + warp * 16;

  auto issue = [&](int it, int s) {
    const int h = it / p.dblocks, jb = it - h * p.dblocks;
    const int d0 = jb * 64, dv = min(64, d - d0);
    const size_t sys = (size_t)b * p.heads + h;
    uint32_t base = smem + s * Sm::STAGE;
    load_tile_bf16<ALIGNED>(base, kTileTokens, R, rowbase + h * R, p.width, rows, R, tid, kTokenThreads);
    base += Sm::A_BYTES;
    load_tile_bf16<ALIGNED>(base, kTileTokens, 64, rowbase + p.heads * R + h * d + d0, p.width, rows, dv, tid, kTokenThreads);
    base += Sm::C_BYTES;
    load_tile_bf16<ALIGNED>(base, kTileTokens, 64, dybase + h * d + d0, dmodel, rows, dv, tid, kTokenThreads);
    base += Sm::C_BYTES;
    const int wv = min(64, p.dpad - d0);
    const __nv_bfloat16* w = p.coeff + sys * 2 * R * p.dpad + d0;
    load_tile_bf16<true>(base, R, 64, w, p.dpad, R, wv, tid, kTokenThreads);
    load_tile_bf16<true>(base + Sm::W_BYTES, R, 64, w + (size_t)R * p.dpad, p.dpad, R, wv, tid, kTokenThreads);
    base += 2 * Sm::W_BYTES;
    const __nv_bfloat16* q = p.cross_grad + sys * 2 * R * p.dpad + d0;
    load_tile_bf16<true>(base, R, 64, q, p.dpad, R, wv, tid, kTokenThreads);
    load_tile_bf16<true>(base + Sm::W_BYTES, R, 64, q + (size_t)R * p.dpad, p.dpad, R, wv, tid, kTokenThreads);
    base += 2 * Sm::W_BYTES;
    const __nv_bfloat16* sg = p.gram_grad + sys * 2 * R * R;
    load_tile_bf16<true>(base, R, R, sg, R, R, R, tid, kTokenThreads);
    load_tile_bf16<true>(base + Sm::S_BYTES, R, R, sg + R * R, R, R, R, tid, kTokenThreads);
  };

#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < items) issue(s, s);
    cp_async_commit();
  }

  TableFrag tab;
  int tab_jb = -1;
  const int g = lane >> 2, tq = lane & 3;
  const int mi = lane >> 3, mr = lane & 7;
  float acc_a[NR][4];

  for (int it = 0; it < items; ++it) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();
    {
      const int nx = it + STAGES - 1;
      if (nx < items) issue(nx, nx % STAGES);
      cp_async_commit();
    }
    const int h = it / p.dblocks, jb = it - h * p.dblocks;
    const int d0 = jb * 64, dv = min(64, d - d0);
    const uint32_t a_tile = smem + (it % STAGES) * Sm::STAGE;
    const uint32_t c_tile = a_tile + Sm::A_BYTES;
    const uint32_t y_tile = c_tile + Sm::C_BYTES;
    const uint32_t wh_tile = y_tile + Sm::C_BYTES;
    const uint32_t wl_tile = wh_tile + Sm::W_BYTES;
    const uint32_t qh_tile = wl_tile + Sm::W_BYTES;
    const uint32_t ql_tile = qh_tile + Sm::W_BYTES;
    const uint32_t sh_tile = ql_tile + Sm::W_BYTES;
    const uint32_t sl_tile = sh_tile + Sm::S_BYTES;
    if (ROT && jb != tab_jb) {
      load_table_frag(tab, p.cos, p.sin, tab_row0, rows - warp * 16, half, d0 >> 1, dv >> 1, lane);
      tab_jb = jb;
    }
    const float eta = p.eta[h];

    // relation rows of this warp as the row operand (K = rank)
    uint32_t af[R / 16][4];
#pragma unroll
    for (int ks = 0; ks < R / 16; ++ks)
      ldsm_x4(af[ks], a_tile + swz((warp * 16 + mr + 8 * (mi & 1)) * (R * 2) + (ks * 16 + 8 * (mi >> 1)) * 2));

    if (jb == 0) {
      // A S' with S' = s (dG + dG^T): the symmetric matrix is stored [n][k], residual word first
#pragma unroll
      for (int j = 0; j < NR; ++j)
#pragma unroll
        for (int k = 0; k < 4; ++k) acc_a[j][k] = 0.f;
#pragma unroll
      for (int word = 0; word < 2; ++word) {
        const uint32_t st = word == 0 ? sl_tile : sh_tile;
#pragma unroll
        for (int ks = 0; ks < R / 16; ++ks) {
#pragma unroll
          for (int n2 = 0; n2 < R / 16; ++n2) {
            uint32_t bf[4];
            ldsm_x4(bf, st + swz((n2 * 16 + mr + 8 * (mi >> 1)) * (R * 2) + (ks * 16 + 8 * (mi & 1)) * 2));
            mma_bf16(acc_a[2 * n2], af[ks], bf[0], bf[1]);
            mma_bf16(acc_a[2 * n2 + 1], af[ks], bf[2], bf[3]);
          }
        }
      }
    }

    // rot(dY) W^T and rot(C) dQ^T
    uint32_t yraw[4][4];
    load_row_frags(yraw, y_tile, warp, lane);
    {
      uint32_t xh[4][4], xl[4][4];
      if (ROT) {
        rotate_split(yraw, tab, xh, xl);
        mma_rows_by_stored_nk<R>(acc_a, xl, wh_tile, lane);
        mma_rows_by_stored_nk<R>(acc_a, xh, wl_tile, lane);
        mma_rows_by_stored_nk<R>(acc_a, xh, wh_tile, lane);
      } else {
        mma_rows_by_stored_nk<R>(acc_a, yraw, wl_tile, lane);
        mma_rows_by_stored_nk<R>(acc_a, yraw, wh_tile, lane);
      }
      uint32_t craw[4][4];
      load_row_frags(craw, c_tile, warp, lane);
      if (ROT) {
        rotate_split(craw, tab, xh, xl);
        mma_rows_by_stored_nk<R>(acc_a, xl, qh_tile, lane);
        mma_rows_by_stored_nk<R>(acc_a, xh, ql_tile, lane);
        mma_rows_by_stored_nk<R>(acc_a, xh, qh_tile, lane);
      } else {
        mma_rows_by_stored_nk<R>(acc_a, craw, ql_tile, lane);
        mma_rows_by_stored_nk<R>(acc_a, craw, qh_tile, lane);
      }
    }

    // dC = eta*dY + s * rot^-1(A dQ)
    {
      float acc[8][4];
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int k = 0; k < 4; ++k) acc[j][k] = 0.f;
#pragma unroll
      for (int word = 0; word < 2; ++word) {
        const uint32_t qt = word == 0 ? ql_tile : qh_tile;
#pragma unroll
        for (int ks = 0; ks < R / 16; ++ks) {
#pragma unroll
          for (int n2 = 0; n2 < 4; ++n2) {
            uint32_t bf[4];
            ldsm_x4_t(bf, qt + swz((ks * 16 + mr + 8 * (mi & 1)) * 128 + (n2 * 16 + 8 * (mi >> 1)) * 2));
            mma_bf16(acc[2 * n2], af[ks], bf[0], bf[1]);
            mma_bf16(acc[2 * n2 + 1], af[ks], bf[2], bf[3]);
          }
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const int row = warp * 16 + g + 8 * k;
          float2 corr = make_float2(acc[j][2 * k], acc[j][2 * k + 1]);
          if (ROT) corr = rot_pair(corr.x, corr.y, tab.c[j][k], -tab.s[j][k]);
          // dY of the same (row, channel pair): fragment q = (j odd ? 2 : 0) + k of k-step j/2
          const float2 yv = bf2_to_f2(yraw[j >> 1][2 * (j & 1) + k]);
          st_shared_u32(c_tile + swz(row * 128 + (8 * j + 2 * tq) * 2),
                        f2_to_bf2(fmaf(corr.x, inv_s, eta * yv.x), fmaf(corr.y, inv_s, eta * yv.y)));
        }
      }
    }
    const bool last_block = jb == p.dblocks - 1;
    if (last_block) {
#pragma unroll
      for (int j = 0; j < NR; ++j) {
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const int row = warp * 16 + g + 8 * k;
          st_shared_u32(a_tile + swz(row * (R * 2) + (8 * j + 2 * tq) * 2),
                        f2_to_bf2(acc_a[j][2 * k] * inv_s, acc_a[j][2 * k + 1] * inv_s));
        }
      }
    }
    __syncthreads();
    store_tile_bf16<ALIGNED>(c_tile, 64, outbase + p.heads * R + h * d + d0, p.width, rows, dv, tid);
    if (last_block) store_tile_bf16<ALIGNED>(a_tile, R, outbase + h * R, p.width, rows, R, tid);
  }
  cp_async_wait<0>();
}

// ---------------------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------------------
template <class K>
static int launch_token(K kern, int smem_bytes, const TokenParams& p, cudaStream_t st) {
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem_bytes) != MS_OK) return MS_ERR_LAUNCH;
  dim3 grid(p.tiles + (p.d_eta_raw ? p.heads : 0), p.batch);
  launch_kernel(kern, grid, dim3(kTokenThreads), smem_bytes, st, p);
  return cudaGetLastError() == cudaSuccess ? MS_OK : MS_ERR_LAUNCH;
}

template <int R>
static int launch_readout_r(const TokenParams& p, bool rot, bool aligned, cudaStream_t st) {
  const int bytes = ReadoutSmem<R>::TOTAL;
  if (rot) return aligned ? launch_token(readout_kernel<R, true, true>, bytes, p, st)
                          : launch_token(readout_kernel<R, true, false>, bytes, p, st);
  return aligned ? launch_token(readout_kernel<R, false, true>, bytes, p, st)
                 : launch_token(readout_kernel<R, false, false>, bytes, p, st);
}

template <int R>
static int launch_token_bwd_r(const TokenParams& p, bool rot, bool aligned, cudaStream_t st) {
  const int bytes = TokenBwdSmem<R>::TOTAL;
  if (rot) return aligned ? launch_token(token_backward_kernel<R, true, true>, bytes, p, st)
                          : launch_token(token_backward_kernel<R, true, false>, bytes, p, st);
  return aligned ? launch_token(token_backward_kernel<R, false, true>, bytes, p, st)
                 : launch_token(token_backward_kernel<R, false, false>, bytes, p, st);
}

int launch_readout_tma(const ms_shape& s, const Plan& plan, const void* projected, const float* cos,
                       const float* sin, const float* counts, const ms_tape& t, void* mixed, cudaStream_t st);

int launch_token_backward_tma(const ms_shape& s, const Plan& plan, const void* projected, const void* dy,
                              const float* cos, const float* sin, const float* counts, const ms_tape& t,
                              const void* gram_grad, const void* cross_grad, void* dprojected,
                              const CoreAdjoint* core, cudaStream_t st);

int launch_token_backward_tc(const ms_shape& s, const Plan& plan, const void* projected, const void* dy,
                             const float* cos, const float* sin, const float* counts, const ms_tape& t,
                             const void* gram_grad, const void* cross_grad, void* dprojected,
                             const CoreAdjoint* core, float* debug, cudaStream_t st);

int launch_readout_tc(const ms_shape& s, const Plan& plan, const void* projected, const float* cos, const float* sin,
                      const float* counts, const ms_tape& t, void* mixed, float* debug, cudaStream_t st);

static TokenParams token_params(const ms_shape& s, const Plan& plan, const void* projected, const void* dy,
                                const float* cos, const float* sin, const float* counts, const ms_tape& t,
                                const void* gram_grad, const void* cross_grad, void* out) {
  TokenParams p;
  p.projected = static_cast<const __nv_bfloat16*>(projected);
  p.dy = static_cast<const __nv_bfloat16*>(dy);
  p.cos = cos; p.sin = sin; p.counts = counts; p.eta = t.eta;
  p.coeff = static_cast<const __nv_bfloat16*>(t.coeff);
  p.gram_grad = static_cast<const __nv_bfloat16*>(gram_grad);
  p.cross_grad = static_cast<const __nv_bfloat16*>(cross_grad);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.batch = s.batch; p.tokens = s.tokens; p.heads = s.heads; p.head_dim = s.head_dim;
  p.width = s.heads * (s.rank + s.head_dim);
  p.rotary_rows = s.rotary_rows; p.dblocks = plan.dblocks; p.dpad = plan.dpad;
  p.base_raw = nullptr; p.hmat = nullptr; p.de_sys = nullptr; p.eta_slope = t.eta_slope; p.core_map = t.core_map;
  p.d_base = nullptr; p.d_eta_raw = nullptr; p.grad_scale = 1.f; p.complement = s.complement;
  p.tiles = (s.tokens + kTileTokens - 1) / kTileTokens;
  return p;
}

int launch_readout(const ms_shape& s, const Plan& plan, const void* projected, const float* cos,
                   const float* sin, const float* counts, const ms_tape& t, void* mixed, cudaStream_t st) {
  if (plan.tc) {
    const int r = launch_readout_tc(s, plan, projected, cos, sin, counts, t, mixed, nullptr, st);
    if (r != -1) return r;
  }
  if (plan.tma) {
    const int r = launch_readout_tma(s, plan, projected, cos, sin, counts, t, mixed, st);
    if (r != -1) return r;
  }
  const TokenParams p = token_params(s, plan, projected, nullptr, cos, sin, counts, t, nullptr, nullptr, mixed);
  const bool rot = s.rotary_rows > 0;
  switch (s.rank) {
    case 16: return launch_readout_r<16>(p, rot, plan.aligned, st);
    case 32: return launch_readout_r<32>(p, rot, plan.aligned, st);
    case 48: return launch_readout_r<48>(p, rot, plan.aligned, st);
    case 64: return launch_readout_r<64>(p, rot, plan.aligned, st);
  }
  return MS_ERR_UNSUPPORTED_RANK;
}

int launch_token_backward(const ms_shape& s, const Plan& plan, const void* projected, const void* dy,
                          const float* cos, const float* sin, const float* counts, const ms_tape& t,
                          const void* gram_grad, const void* cross_grad, void* dprojected,
                          const CoreAdjoint* core, cudaStream_t st) {
  if (plan.tc) {
    const int r = launch_token_backward_tc(s, plan, projected, dy, cos, sin, counts, t, gram_grad, cross_grad,
                                           dprojected, core, nullptr, st);
    if (r != -1) return r;
  }
  if (plan.tma) {
    const int r = launch_token_backward_tma(s, plan, projected, dy, cos, sin, counts, t, gram_grad, cross_grad,
                                            dprojected, core, st);
    if (r != -1) return r;
  }
  TokenParams p = token_params(s, plan, projected, dy, cos, sin, counts, t, gram_grad, cross_grad, dprojected);
  if (core) {
    p.base_raw = core->base_raw; p.hmat = core->hmat; p.de_sys = core->de_sys;
    p.d_base = core->d_base; p.d_eta_raw = core->d_eta_raw; p.grad_scale = core->grad_scale;
  }
  const bool rot = s.rotary_rows > 0;
  switch (s.rank) {
    case 16: return launch_token_bwd_r<16>(p, rot, plan.aligned, st);
    case 32: return launch_token_bwd_r<32>(p, rot, plan.aligned, st);
    case 48: return launch_token_bwd_r<48>(p, rot, plan.aligned, st);
    case 64: return launch_token_bwd_r<64>(p, rot, plan.aligned, st);
  }
  return MS_ERR_UNSUPPORTED_RANK;
}

}  // namespace ms
