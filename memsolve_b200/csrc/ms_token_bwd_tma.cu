// Token backward -- TMA / persistent-warp version (head dimension 64, rank 16/32/64, aligned
// pointers; other shapes take token_backward_kernel in ms_token.cu).
//
//   dA = s*( A_raw S' + rot(dY) W^T + rot(C) dQ^T ),  S' = s (dG+dG^T),   dC = eta*dY + s*rot^-1(A_raw dQ)
//
// Same arithmetic as the generic kernel (the reference's `_token_backward`,
// memsolve/ball/cuda.py:1767-1922).  A CTA serves one sample and one group of heads whose
// compact matrices (W, dQ and dG+dG^T, two BF16 words each) are loaded once with TMA and stay in
// shared memory.  Each warp walks over its own (16-token slice, head) items: lane 0 issues the
// TMA loads of the relation, content and upstream-gradient boxes into the warp's private ring
// (one mbarrier per stage), the warp runs the tensor-core products, writes dA and dC over the
// relation and content boxes and lane 0 stores both with TMA.  No CTA-wide barrier after the
// prologue; the 3-D tensor maps clip tokens past the end of a sample.  Spare CTAs
// (blockIdx.x >= work CTAs) compute the per-head parameter gradients.
#include "ms_core.cuh"
#include "ms_frag.cuh"
#include "ms_tma.cuh"

namespace ms {

// WARPS independent warps per CTA, each with a ring of STAGES buffers of which PRE are in flight
// ahead of the one being computed (STAGES - PRE - 1 buffers may still be read by earlier stores).
template <int R, int WARPS_, int STAGES_, int PRE_>
struct TokenBwdTmaCfg {
  static constexpr int WARPS = WARPS_;
  static constexpr int STAGES = STAGES_;
  static constexpr int PRE = PRE_;
  static constexpr int A_SLICE = 16 * R * 2;
  static constexpr int STAGE = ((4096 + A_SLICE + 1023) / 1024) * 1024;   // C, dY, A
  static constexpr int RING = WARPS * STAGES * STAGE;
  static constexpr int W_BYTES = R * 128;
  static constexpr int S_BYTES = R * R * 2;
  static constexpr int HEAD_BYTES = 4 * W_BYTES + 2 * S_BYTES;   // W hi/lo, dQ hi/lo, S hi/lo
  static constexpr int BAR_BYTES = (WARPS * STAGES + 1) * 8;
  static constexpr int MAX_SMEM = 227 * 1024;
  static constexpr int RESIDENT_BUDGET = MAX_SMEM - 1024 - RING - BAR_BYTES - 64;
  static_assert(PRE >= 1 && PRE < STAGES, "prefetch depth");
};

struct TokenBwdTmaParams {
  const float* cos;
  const float* sin;
  const float* counts;
  const float* eta;
  int* error;
  int tokens, heads, rotary_rows, group_heads, slices, work_ctas, batch;
  int core_ctas;   // spare CTAs of the grid; spare CTA c takes the heads c, c + core_ctas, ...
  // per-head core adjoint (spare CTAs); d_eta_raw == nullptr disables it
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

// acc += rot(X) M^T for the 16 x 64 row operand `raw` (BF16 fragments of one warp) and a matrix
// stored [R output columns][64 channels] as two BF16 words (128-byte pitch, 128-byte swizzle).
// One 16-channel step at a time: rotate and split the step's fragment, then the two residual
// products and the dominant one, so that only one step of split fragments is live.
template <int R, bool ROT>
__device__ __forceinline__ void mma_rotated_rows(float (&acc)[R / 8][4], const uint32_t (&raw)[4][4],
                                                 const TableFrag& tab, uint32_t hi_tile, uint32_t lo_tile,
                                                 int lane) {
  const int mi = lane >> 3, mr = lane & 7;
#pragma unroll
  for (int ks = 0; ks < 4; ++ks) {
    uint32_t xh[4], xl[4];
    if (ROT) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int j = 2 * ks + (q >> 1), k = q & 1;   // q: (row g|g+8) x (cols 0-7 | 8-15)
        const float2 v = bf2_to_f2(raw[ks][q]);
        const float2 r = rot_pair(v.x, v.y, tab.c[j][k], tab.s[j][k]);
        split2(r.x, r.y, xh[q], xl[q]);
      }
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q) xh[q] = raw[ks][q];
    }
#pragma unroll
    for (int n2 = 0; n2 < R / 16; ++n2) {
      const uint32_t off = swz((n2 * 16 + mr + 8 * (mi >> 1)) * 128 + (ks * 16 + 8 * (mi & 1)) * 2);
      uint32_t bh[4], bl[4];
      ldsm_x4(bh, hi_tile + off);
      ldsm_x4(bl, lo_tile + off);
      if (ROT) {
        mma_bf16(acc[2 * n2], xl, bh[0], bh[1]);
        mma_bf16(acc[2 * n2 + 1], xl, bh[2], bh[3]);
      }
      mma_bf16(acc[2 * n2], xh, bl[0], bl[1]);
      mma_bf16(acc[2 * n2 + 1], xh, bl[2], bl[3]);
      mma_bf16(acc[2 * n2], xh, bh[0], bh[1]);
      mma_bf16(acc[2 * n2 + 1], xh, bh[2], bh[3]);
    }
  }
}

template <int R, bool ROT, class Cfg>
__global__ void __launch_bounds__(Cfg::WARPS * 32)
token_backward_tma_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_c,
                          const __grid_constant__ CUtensorMap map_y, const __grid_constant__ CUtensorMap map_w,
                          const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_s,
                          const __grid_constant__ CUtensorMap map_oa, const __grid_constant__ CUtensorMap map_oc,
                          const TokenBwdTmaParams p) {
  constexpr int STAGES = Cfg::STAGES;
  constexpr int PRE = Cfg::PRE;
  constexpr int WARPS = Cfg::WARPS;
  constexpr int NR = R / 8;
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
                             smem_raw + (smem - smem_u32(smem_raw)), tid, WARPS * 32);
        __syncthreads();
      }
    }
    return;
  }

  const int b = blockIdx.y;
  const int h0 = blockIdx.z * p.group_heads;
  const int gh = min(p.group_heads, p.heads - h0);
  const uint32_t res_base = smem;
  const uint32_t ring = smem + p.group_heads * Cfg::HEAD_BYTES + warp * STAGES * Cfg::STAGE;
  const uint32_t bars = smem + p.group_heads * Cfg::HEAD_BYTES + Cfg::RING;
  const uint32_t rbar = bars + WARPS * STAGES * 8;
  const uint32_t mybar = bars + warp * STAGES * 8;

  if (tid == 0) {
    for (int i = 0; i < WARPS * STAGES + 1; ++i) mbar_init(bars + i * 8, 1);
    mbar_fence_init();
  }
  __syncthreads();
  const int total = p.slices * gh;
  const int nwarps = p.work_ctas * WARPS;
  const int per = (total + nwarps - 1) / nwarps;
  const int it0 = min(total, (blockIdx.x * WARPS + warp) * per);
  const int n_items = min(total, it0 + per) - it0;

  const float n = p.counts ? p.counts[b] : (float)p.tokens;
  const float inv_s = inv_sqrt_rn(n);
  const long tab_row_b = p.rotary_rows > 1 ? (long)b * p.tokens : 0;
  const int g = lane >> 2, tq = lane & 3;
  const int mi = lane >> 3, mr = lane & 7;

  // position of an item: (slice, head in group) and its ring stage; advanced without divisions
  struct Cursor {
    int slice, hl, stage;
  };
  auto advance = [&](Cursor& c) {
    if (++c.hl == gh) {
      c.hl = 0;
      ++c.slice;
    }
    c.stage = c.stage + 1 == STAGES ? 0 : c.stage + 1;
  };
  Cursor ahead;   // next item to load
  ahead.slice = it0 / gh;
  ahead.hl = it0 - ahead.slice * gh;
  ahead.stage = 0;
  Cursor cur = ahead;   // item being computed
  uint32_t parity = 0;

  auto issue = [&](const Cursor& c) {
    const int h = h0 + c.hl;
    const uint32_t st = ring + c.stage * Cfg::STAGE;
    const uint32_t bar = mybar + c.stage * 8;
    mbar_expect_tx(bar, 4096 + Cfg::A_SLICE);
    tma_load_3d(st, &map_c, p.heads * R + h * 64, c.slice * 16, b, bar);
    tma_load_3d(st + 2048, &map_y, h * 64, c.slice * 16, b, bar);
    tma_load_3d(st + 4096, &map_a, h * R, c.slice * 16, b, bar);
  };

  for (int k = 0; k < PRE && k < n_items; ++k) {
    if (lane == 0) issue(ahead);
    advance(ahead);
  }
  // The token boxes above were requested before this point on purpose: `projected`, the gradient and the counts were
  // complete before the kernel ahead of the previous one started, so a chained launch may fetch them while
  // the previous kernel (which produces the resident matrices) is still draining.
  grid_dependency_wait();
  if (tid == 0) {
    mbar_expect_tx(rbar, (uint32_t)(gh * Cfg::HEAD_BYTES));
    for (int hl = 0; hl < gh; ++hl) {
      const int sys = b * p.heads + h0 + hl;
      const uint32_t hb = res_base + hl * Cfg::HEAD_BYTES;
      tma_load_2d(hb, &map_w, 0, (sys * 2) * R, rbar);
      tma_load_2d(hb + Cfg::W_BYTES, &map_w, 0, (sys * 2 + 1) * R, rbar);
      tma_load_2d(hb + 2 * Cfg::W_BYTES, &map_q, 0, (sys * 2) * R, rbar);
      tma_load_2d(hb + 3 * Cfg::W_BYTES, &map_q, 0, (sys * 2 + 1) * R, rbar);
      tma_load_2d(hb + 4 * Cfg::W_BYTES, &map_s, 0, (sys * 2) * R, rbar);
      tma_load_2d(hb + 4 * Cfg::W_BYTES + Cfg::S_BYTES, &map_s, 0, (sys * 2 + 1) * R, rbar);
    }
  }
  bool ok = mbar_wait(rbar, 0);
  ok = __all_sync(0xffffffffu, ok);

  TableFrag tab;
  int tab_slice = -1;

  for (int k = 0; k < n_items && ok; ++k) {
    if (k + PRE < n_items) {
      if (lane == 0) {
        // the buffer being refilled was the source of the stores of item k + PRE - STAGES
        tma_store_wait_read<STAGES - PRE - 1>();
        issue(ahead);
      }
      advance(ahead);
    }
    const int slice = cur.slice, hl = cur.hl;
    const int h = h0 + hl;
    const uint32_t c_tile = ring + cur.stage * Cfg::STAGE;
    const uint32_t y_tile = c_tile + 2048;
    const uint32_t a_tile = c_tile + 4096;
    const uint32_t wh_tile = res_base + hl * Cfg::HEAD_BYTES;
    const uint32_t wl_tile = wh_tile + Cfg::W_BYTES;
    const uint32_t qh_tile = wl_tile + Cfg::W_BYTES;
    const uint32_t ql_tile = qh_tile + Cfg::W_BYTES;
    const uint32_t sh_tile = ql_tile + Cfg::W_BYTES;
    const uint32_t sl_tile = sh_tile + Cfg::S_BYTES;

    if (ROT && slice != tab_slice) {
      load_table_frag(tab, p.cos, p.sin, tab_row_b + slice * 16, p.tokens - slice * 16, 32, 0, 32, lane);
      tab_slice = slice;
    }
    const float eta = __ldg(p.eta + h);

    ok = mbar_wait(mybar + cur.stage * 8, parity);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) break;
    uint32_t af[R / 16][4];
#pragma unroll
    for (int ks = 0; ks < R / 16; ++ks)
      ldsm_x4(af[ks], a_tile + swz_rows<R * 2>((mr + 8 * (mi & 1)) * (R * 2) + (ks * 16 + 8 * (mi >> 1)) * 2));
    uint32_t xraw[4][4];
    load_row_frags(xraw, y_tile, 0, lane);
    __syncwarp();   // every lane has read the gradient box before dC is written over it

    // dC = eta*dY + s * rot^-1(A dQ), written over the upstream-gradient box
    {
      float acc[8][4];
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[j][q] = 0.f;
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
        for (int kk = 0; kk < 2; ++kk) {
          float2 corr = make_float2(acc[j][2 * kk], acc[j][2 * kk + 1]);
          if (ROT) corr = rot_pair(corr.x, corr.y, tab.c[j][kk], -tab.s[j][kk]);
          const float2 yv = bf2_to_f2(xraw[j >> 1][2 * (j & 1) + kk]);
          st_shared_u32(y_tile + swz((g + 8 * kk) * 128 + (8 * j + 2 * tq) * 2),
                        f2_to_bf2(fmaf(corr.x, inv_s, eta * yv.x), fmaf(corr.y, inv_s, eta * yv.y)));
        }
      }
    }

    // dA = s*( A S' + rot(dY) W^T + rot(C) dQ^T ): the symmetric matrix S' = s (dG + dG^T) is stored [n][k],
    // residual word first
    float acc_a[NR][4];
#pragma unroll
    for (int j = 0; j < NR; ++j)
#pragma unroll
      for (int q = 0; q < 4; ++q) acc_a[j][q] = 0.f;
#pragma unroll
    for (int word = 0; word < 2; ++word) {
      const uint32_t st = word == 0 ? sl_tile : sh_tile;
#pragma unroll
      for (int ks = 0; ks < R / 16; ++ks) {
#pragma unroll
        for (int n2 = 0; n2 < R / 16; ++n2) {
          uint32_t bf[4];
          ldsm_x4(bf, st + swz_rows<R * 2>((n2 * 16 + mr + 8 * (mi >> 1)) * (R * 2) + (ks * 16 + 8 * (mi & 1)) * 2));
          mma_bf16(acc_a[2 * n2], af[ks], bf[0], bf[1]);
          mma_bf16(acc_a[2 * n2 + 1], af[ks], bf[2], bf[3]);
        }
      }
    }
    mma_rotated_rows<R, ROT>(acc_a, xraw, tab, wh_tile, wl_tile, lane);
    load_row_frags(xraw, c_tile, 0, lane);
    mma_rotated_rows<R, ROT>(acc_a, xraw, tab, qh_tile, ql_tile, lane);
    // dA over the relation box
#pragma unroll
    for (int j = 0; j < NR; ++j) {
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {
        st_shared_u32(a_tile + swz_rows<R * 2>((g + 8 * kk) * (R * 2) + (8 * j + 2 * tq) * 2),
                      f2_to_bf2(acc_a[j][2 * kk] * inv_s, acc_a[j][2 * kk + 1] * inv_s));
      }
    }
    fence_async_shared();
    __syncwarp();
    if (lane == 0) {
      tma_store_3d(&map_oc, p.heads * R + h * 64, slice * 16, b, y_tile);
      tma_store_3d(&map_oa, h * R, slice * 16, b, a_tile);
      tma_store_commit();
    }
    advance(cur);
    if (cur.stage == 0) parity ^= 1u;
  }
  if (lane == 0) {
    tma_store_wait_all<0>();
    if (!ok) atomicExch(p.error, kErrBarrierTimeout);
  }
}

template <int R, class Cfg>
static int launch_token_bwd_tma_cfg(const ms_shape& s, const Plan& plan, const void* projected, const void* dy,
                                    const float* cos, const float* sin, const float* counts, const ms_tape& t,
                                    const void* gram_grad, const void* cross_grad, void* dprojected,
                                    const CoreAdjoint* core, cudaStream_t st) {
  constexpr int kTbWarps = Cfg::WARPS;
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
    const uint32_t box_a[3] = {(uint32_t)R, 16, 1};
    const uint32_t box_c[3] = {64, 16, 1};
    const Swizzle sa = swizzle_for_rows<R * 2>();
    if (encode_tensor_map(&map_a, const_cast<void*>(projected), 2, 3, dims, str, box_a, sa)) return MS_ERR_LAUNCH;
    if (encode_tensor_map(&map_c, const_cast<void*>(projected), 2, 3, dims, str, box_c, Swizzle::B128)) return MS_ERR_LAUNCH;
    if (encode_tensor_map(&map_oa, dprojected, 2, 3, dims, str, box_a, sa)) return MS_ERR_LAUNCH;
    if (encode_tensor_map(&map_oc, dprojected, 2, 3, dims, str, box_c, Swizzle::B128)) return MS_ERR_LAUNCH;
  }
  {
    const uint64_t dims[3] = {(uint64_t)dmodel, (uint64_t)s.tokens, (uint64_t)s.batch};
    const uint64_t str[2] = {(uint64_t)dmodel * 2, (uint64_t)s.tokens * dmodel * 2};
    const uint32_t box[3] = {64, 16, 1};
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

  TokenBwdTmaParams p;
  p.cos = cos; p.sin = sin; p.counts = counts; p.eta = t.eta;
  p.error = device_error_word();
  if (!p.error) return MS_ERR_LAUNCH;
  p.tokens = s.tokens; p.heads = heads; p.rotary_rows = s.rotary_rows; p.group_heads = group;
  p.slices = (s.tokens + 15) / 16; p.batch = s.batch;
  p.base_raw = nullptr; p.hmat = nullptr; p.de_sys = nullptr; p.eta_slope = t.eta_slope; p.core_map = t.core_map;
  p.d_base = nullptr; p.d_eta_raw = nullptr; p.grad_scale = 1.f; p.complement = s.complement;
  if (core) {
    p.base_raw = core->base_raw; p.hmat = core->hmat; p.de_sys = core->de_sys;
    p.d_base = core->d_base; p.d_eta_raw = core->d_eta_raw; p.grad_scale = core->grad_scale;
  }
  const long total = (long)p.slices * group;
  // one CTA per SM: leave SMs for the per-head CTAs that ride along, so that the whole grid is
  // resident at once (a CTA that has to wait for a free SM would run after all the others)
  // With few samples the adjoint of one head takes a small part of the launch: one spare CTA then takes two
  // heads, which frees SMs for the token pass (at 32768 tokens and 12 heads: 15 instead of 16 items per warp).
  const int core_ctas = core ? (s.batch <= 4 ? (heads + 1) / 2 : heads) : 0;
  long ctas = (sm_count() - core_ctas) / ((long)s.batch * groups);
  if (ctas < 1) ctas = 1;
  const long need = (total + kTbWarps * 6 - 1) / (kTbWarps * 6);
  if (ctas > need) ctas = need < 1 ? 1 : need;
  p.work_ctas = (int)ctas;
  p.core_ctas = core_ctas > 0 ? core_ctas : 1;
  dim3 grid((unsigned)ctas + core_ctas, s.batch, groups);
  int smem_bytes = 1024 + group * Cfg::HEAD_BYTES + Cfg::RING + Cfg::BAR_BYTES;
  const int core_bytes = (int)core_backward_smem_bytes(R) + 1024;
  if (core && smem_bytes < core_bytes) smem_bytes = core_bytes;
  if (s.rotary_rows > 0) {
    auto kern = token_backward_tma_kernel<R, true, Cfg>;
    if (ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem_bytes)) return MS_ERR_LAUNCH;
    launch_kernel(kern, grid, dim3(kTbWarps * 32), smem_bytes, st, map_a, map_c, map_y, map_w, map_q, map_s, map_oa,
                  map_oc, p);
  } else {
    auto kern = token_backward_tma_kernel<R, false, Cfg>;
    if (ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem_bytes)) return MS_ERR_LAUNCH;
    launch_kernel(kern, grid, dim3(kTbWarps * 32), smem_bytes, st, map_a, map_c, map_y, map_w, map_q, map_s, map_oa,
                  map_oc, p);
  }
  return cudaGetLastError() == cudaSuccess ? MS_OK : MS_ERR_LAUNCH;
}

template <int R>
static int launch_token_bwd_tma_r(const ms_shape& s, const Plan& plan, const void* projected, const void* dy,
                                  const float* cos, const float* sin, const float* counts, const ms_tape& t,
                                  const void* gram_grad, const void* cross_grad, void* dprojected,
                                  const CoreAdjoint* core, cudaStream_t st) {
#define MS_TB_ARGS s, plan, projected, dy, cos, sin, counts, t, gram_grad, cross_grad, dprojected, core, st
  // rank 64: the resident matrices of one head take 48 KB, eight warps leave room for them
  if (R == 64) return launch_token_bwd_tma_cfg<R, TokenBwdTmaCfg<R, 8, 3, 1>>(MS_TB_ARGS);
  return launch_token_bwd_tma_cfg<R, TokenBwdTmaCfg<R, 12, 2, 1>>(MS_TB_ARGS);
#undef MS_TB_ARGS
}

// MS_OK / error, or -1 when the shape is outside this kernel's envelope.
int launch_token_backward_tma(const ms_shape& s, const Plan& plan, const void* projected, const void* dy,
                              const float* cos, const float* sin, const float* counts, const ms_tape& t,
                              const void* gram_grad, const void* cross_grad, void* dprojected,
                              const CoreAdjoint* core, cudaStream_t st) {
  if (!plan.aligned || s.head_dim != 64) return -1;
  if (((reinterpret_cast<uintptr_t>(t.coeff) | reinterpret_cast<uintptr_t>(gram_grad) |
        reinterpret_cast<uintptr_t>(cross_grad)) & 15u) != 0)
    return -1;
  switch (s.rank) {
    case 16: return launch_token_bwd_tma_r<16>(s, plan, projected, dy, cos, sin, counts, t, gram_grad, cross_grad, dprojected, core, st);
    case 32: return launch_token_bwd_tma_r<32>(s, plan, projected, dy, cos, sin, counts, t, gram_grad, cross_grad, dprojected, core, st);
    case 64: return launch_token_bwd_tma_r<64>(s, plan, projected, dy, cos, sin, counts, t, gram_grad, cross_grad, dprojected, core, st);
  }
  return -1;
}

}  // namespace ms
