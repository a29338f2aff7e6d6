// Token reductions of the MemSolve mixer.
//
// Forward:  per (sample b, head h)  G += A^T A  (r x r),  Q += A^T rot(C)  (r x d)
// Adjoint:  per (b, h)              E += A^T rot(dY) (r x d),  de += <dY, C>
//
// A and C are the relation / content columns of the packed BF16 projection; the sums run
// over tokens.  Replaces the reference's `_statistics`, `_chunk_statistics`, `reduce_fwd`
// and `reduce_bwd` (memsolve/ball/cuda.py:1542-1667, 1925-2046, 2058-2112).
//
// One CTA owns one (system, token chunk, 64-channel block).  Tiles of 64 tokens stream
// through a multi-stage cp.async pipeline into swizzled shared memory; the rotary rotation
// is applied in FP32 in shared memory and the result is kept as two BF16 words (value and
// residual) so that the tensor-core product keeps about 16 mantissa bits; the contractions
// are mma.sync.m16n8k16 with FP32 accumulators held in registers for the whole chunk.
// Each CTA writes one partial; partials are summed later in fixed order, so the result does
// not depend on scheduling.
#include "ms_core.cuh"

namespace ms {

template <int R>
struct StatsCfg;
template <>
struct StatsCfg<16> { static constexpr int MT = 1, MS = 1, KS = 4; };
template <>
struct StatsCfg<32> { static constexpr int MT = 2, MS = 1, KS = 4; };
template <>
struct StatsCfg<48> { static constexpr int MT = 1, MS = 3, KS = 2; };
template <>
struct StatsCfg<64> { static constexpr int MT = 2, MS = 2, KS = 2; };

struct StatsParams {
  const __nv_bfloat16* projected;
  const __nv_bfloat16* dy;  // adjoint only
  const float* cos;
  const float* sin;
  float* partials;          // [systems][chunks][partial_floats]
  float* de_partials;       // [systems][chunks*2*dblocks] (adjoint only)
  int batch, tokens, heads, head_dim, width, rotary_rows;
  int chunks, chunk_tokens, dblocks;
  int partial_floats;
  // per-head core, computed by the spare CTAs blockIdx.x == chunks (forward only, optional)
  const float* base_raw;
  const float* eta_raw;
  float* eta;
  float* eta_slope;
  float* core_map;
  int* core_info;
  int complement;
};

template <int R, bool GRAD, bool ROT>
struct StatsSmem {
  static constexpr int A_BYTES = kTileTokens * R * 2;
  static constexpr int X_BYTES = kTileTokens * kChanBlock * 2;
  static constexpr int T_BYTES = kTileTokens * 32 * 4;
  static constexpr int STAGE = A_BYTES + X_BYTES + (GRAD ? X_BYTES : 0) + (ROT ? 2 * T_BYTES : 0);
  static constexpr int STAGES = GRAD ? 2 : 3;
  static constexpr int PIPE = STAGE * STAGES + (ROT ? X_BYTES : 0);
  static constexpr int RED = StatsCfg<R>::KS * R * ((GRAD ? 0 : R) + kChanBlock) * 4;
  static constexpr int CORE = GRAD ? 0 : (int)core_forward_smem_bytes(R);
  static constexpr int BODY = PIPE > RED ? PIPE : RED;
  static constexpr int TOTAL = (BODY > CORE ? BODY : CORE) + 128;
};

template <int R, bool GRAD, bool ROT, bool ALIGNED>
__global__ void __launch_bounds__(StatsCfg<R>::MS * StatsCfg<R>::KS * 32)
stats_kernel(const StatsParams p) {
  using Cfg = StatsCfg<R>;
  using Sm = StatsSmem<R, GRAD, ROT>;
  constexpr int MT = Cfg::MT, MS = Cfg::MS, KS = Cfg::KS;
  constexpr int NT = MS * KS * 32;
  constexpr int KSTEPS = 4 / KS;     // 16-token slices per warp per tile
  constexpr int NG = R / 8;          // Gram n-tiles
  constexpr int STAGES = Sm::STAGES;

  extern __shared__ unsigned char smem_raw[];
  const uint32_t smem = (smem_u32(smem_raw) + 127u) & ~127u;
  unsigned char* smem_gen = smem_raw + (smem - smem_u32(smem_raw));

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wm = warp % MS, wk = warp / MS;
  const int chunk = blockIdx.x, sys = blockIdx.y, dblk = blockIdx.z;
  grid_dependency_wait();
  if (!GRAD && chunk == p.chunks) {
    // spare column of the grid: the per-head core runs beside the token reduction
    if (dblk == 0 && sys < p.heads)
      core_forward_device<R, NT>(p.base_raw, p.eta_raw, sys, p.complement, p.eta, p.eta_slope, p.core_map,
                                 p.core_info, smem_gen, tid);
    return;
  }
  const int b = sys / p.heads, h = sys - b * p.heads;
  const int d0 = dblk * kChanBlock;
  const int dvalid = min(kChanBlock, p.head_dim - d0);
  const int tok0 = chunk * p.chunk_tokens;
  const int tok1 = min(p.tokens, tok0 + p.chunk_tokens);
  const int ntiles = (tok1 - tok0 + kTileTokens - 1) / kTileTokens;
  const bool do_gram = !GRAD && dblk == 0;

  const __nv_bfloat16* rowbase = p.projected + (long)b * p.tokens * p.width;
  const __nv_bfloat16* a_src = rowbase + h * R;
  const __nv_bfloat16* c_src = rowbase + p.heads * R + h * p.head_dim + d0;
  const int dmodel = p.heads * p.head_dim;
  const __nv_bfloat16* y_src = GRAD ? p.dy + (long)b * p.tokens * dmodel + h * p.head_dim + d0 : nullptr;
  const int half = p.head_dim >> 1;
  const long tab_b = (p.rotary_rows > 1) ? (long)b * p.tokens * half : 0;
  const float* cos_src = ROT ? p.cos + tab_b + (d0 >> 1) : nullptr;
  const float* sin_src = ROT ? p.sin + tab_b + (d0 >> 1) : nullptr;

  auto stage_base = [&](int s) { return smem + s * Sm::STAGE; };
  const uint32_t lo_tile = smem + STAGES * Sm::STAGE;

  auto issue = [&](int t, int s) {
    const int tk = tok0 + t * kTileTokens;
    const int rows = min(kTileTokens, tok1 - tk);
    uint32_t base = stage_base(s);
    load_tile_bf16<ALIGNED>(base, kTileTokens, R, a_src + (long)tk * p.width, p.width, rows, R, tid, NT);
    base += Sm::A_BYTES;
    if (GRAD) {
      load_tile_bf16<ALIGNED>(base, kTileTokens, kChanBlock, y_src + (long)tk * dmodel, dmodel, rows, dvalid, tid, NT);
      base += Sm::X_BYTES;
    }
    load_tile_bf16<ALIGNED>(base, kTileTokens, kChanBlock, c_src + (long)tk * p.width, p.width, rows, dvalid, tid, NT);
    base += Sm::X_BYTES;
    if (ROT) {
      load_tile_f32<ALIGNED>(base, cos_src + (long)tk * half, half, rows, dvalid >> 1, tid, NT);
      load_tile_f32<ALIGNED>(base + Sm::T_BYTES, sin_src + (long)tk * half, half, rows, dvalid >> 1, tid, NT);
    }
  };

  float accG[GRAD ? 1 : MT][GRAD ? 1 : NG][4];
  float accQ[MT][8][4];
#pragma unroll
  for (int i = 0; i < (GRAD ? 1 : MT); ++i)
#pragma unroll
    for (int j = 0; j < (GRAD ? 1 : NG); ++j)
#pragma unroll
      for (int k = 0; k < 4; ++k) accG[i][j][k] = 0.f;
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int k = 0; k < 4; ++k) accQ[i][j][k] = 0.f;
  float de_acc = 0.f;

#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < ntiles) issue(s, s);
    cp_async_commit();
  }

  for (int t = 0; t < ntiles; ++t) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();
    {
      const int tn = t + STAGES - 1;
      if (tn < ntiles) issue(tn, tn % STAGES);
      cp_async_commit();
    }
    const uint32_t a_tile = stage_base(t % STAGES);
    // operand that is contracted with A: dY (adjoint) or C (forward)
    const uint32_t x_tile = a_tile + Sm::A_BYTES;
    const uint32_t c_tile = GRAD ? x_tile + Sm::X_BYTES : x_tile;
    const uint32_t cos_tile = c_tile + Sm::X_BYTES;
    const uint32_t sin_tile = cos_tile + Sm::T_BYTES;

    if (ROT || GRAD) {
      // elementwise pass over the 64 x 64 tile, one 16-byte chunk (8 channels) at a time
      for (int i = tid; i < kTileTokens * 8; i += NT) {
        const int row = i >> 3, c = i & 7;
        const uint32_t off = swz(row * 128 + c * 16);
        uint4 xv = ld_shared_v4(x_tile + off);
        if (GRAD) {
          uint4 cv = ld_shared_v4(c_tile + off);
          const uint32_t xs[4] = {xv.x, xv.y, xv.z, xv.w};
          const uint32_t cs[4] = {cv.x, cv.y, cv.z, cv.w};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            float2 xf = bf2_to_f2(xs[k]), cf = bf2_to_f2(cs[k]);
            de_acc = fmaf(xf.x, cf.x, de_acc);
            de_acc = fmaf(xf.y, cf.y, de_acc);
          }
        }
        if (ROT) {
          float4 cc = ld_shared_f4(cos_tile + row * 128 + c * 16);
          float4 ss = ld_shared_f4(sin_tile + row * 128 + c * 16);
          const uint32_t xs[4] = {xv.x, xv.y, xv.z, xv.w};
          const float cf[4] = {cc.x, cc.y, cc.z, cc.w};
          const float sf[4] = {ss.x, ss.y, ss.z, ss.w};
          uint32_t hi[4], lo[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            float2 v = bf2_to_f2(xs[k]);
            float2 r = rot_pair(v.x, v.y, cf[k], sf[k]);
            split2(r.x, r.y, hi[k], lo[k]);
          }
          st_shared_v4(x_tile + off, make_uint4(hi[0], hi[1], hi[2], hi[3]));
          st_shared_v4(lo_tile + off, make_uint4(lo[0], lo[1], lo[2], lo[3]));
        }
      }
      if (ROT) __syncthreads();
    }

    const int mi = lane >> 3, mr = lane & 7;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
      const int trow = (wk * KSTEPS + kk) * 16;
      uint32_t af[MT][4];
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const int mt = wm * MT + m;
        // A^T as the row operand: stored [token][rank], transposed on load
        const int row = trow + mr + 8 * (mi >> 1);
        const int col = mt * 16 + 8 * (mi & 1);
        ldsm_x4_t(af[m], a_tile + swz(row * (R * 2) + col * 2));
      }
      if (!GRAD) {
        if (do_gram) {
#pragma unroll
          for (int n2 = 0; n2 < NG / 2; ++n2) {
            uint32_t bf[4];
            const int row = trow + mr + 8 * (mi & 1);
            const int col = n2 * 16 + 8 * (mi >> 1);
            ldsm_x4_t(bf, a_tile + swz(row * (R * 2) + col * 2));
#pragma unroll
            for (int m = 0; m < MT; ++m) {
              mma_bf16(accG[m][2 * n2], af[m], bf[0], bf[1]);
              mma_bf16(accG[m][2 * n2 + 1], af[m], bf[2], bf[3]);
            }
          }
        }
      }
#pragma unroll
      for (int n2 = 0; n2 < 4; ++n2) {
        const int row = trow + mr + 8 * (mi & 1);
        const int col = n2 * 16 + 8 * (mi >> 1);
        const uint32_t off = swz(row * 128 + col * 2);
        uint32_t bf[4];
        if (ROT) {
          // residual word first, dominant word last
          ldsm_x4_t(bf, lo_tile + off);
#pragma unroll
          for (int m = 0; m < MT; ++m) {
            mma_bf16(accQ[m][2 * n2], af[m], bf[0], bf[1]);
            mma_bf16(accQ[m][2 * n2 + 1], af[m], bf[2], bf[3]);
          }
        }
        ldsm_x4_t(bf, x_tile + off);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          mma_bf16(accQ[m][2 * n2], af[m], bf[0], bf[1]);
          mma_bf16(accQ[m][2 * n2 + 1], af[m], bf[2], bf[3]);
        }
      }
    }
  }
  cp_async_wait<0>();
  grid_launch_dependents();   // the next kernel may become resident while the partial is reduced and written
  __syncthreads();

  // ---- combine the KS token-slices of the CTA, then write one partial -----------------
  constexpr int RCOLS = (GRAD ? 0 : R) + kChanBlock;
  float* red = reinterpret_cast<float*>(smem_gen);
  {
    const int g = lane >> 2, tq = lane & 3;
    float* mine = red + (size_t)wk * R * RCOLS;
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      const int r0 = (wm * MT + m) * 16 + g;
      if (!GRAD) {
#pragma unroll
        for (int n = 0; n < NG; ++n) {
          const int col = n * 8 + 2 * tq;
          *reinterpret_cast<float2*>(mine + r0 * RCOLS + col) = make_float2(accG[m][n][0], accG[m][n][1]);
          *reinterpret_cast<float2*>(mine + (r0 + 8) * RCOLS + col) = make_float2(accG[m][n][2], accG[m][n][3]);
        }
      }
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        const int col = (GRAD ? 0 : R) + n * 8 + 2 * tq;
        *reinterpret_cast<float2*>(mine + r0 * RCOLS + col) = make_float2(accQ[m][n][0], accQ[m][n][1]);
        *reinterpret_cast<float2*>(mine + (r0 + 8) * RCOLS + col) = make_float2(accQ[m][n][2], accQ[m][n][3]);
      }
    }
  }
  __syncthreads();
  float* out = p.partials + ((size_t)sys * p.chunks + chunk) * p.partial_floats;
  const int gfloats = GRAD ? 0 : R * R;
  for (int i = tid; i < R * RCOLS; i += NT) {
    const int row = i / RCOLS, col = i - row * RCOLS;
    float v = 0.f;
#pragma unroll
    for (int k = 0; k < KS; ++k) v += red[(size_t)k * R * RCOLS + i];
    if (!GRAD && col < R) {
      if (do_gram) out[row * R + col] = v;
    } else {
      const int ch = col - (GRAD ? 0 : R);
      if (ch < dvalid) out[gfloats + row * p.head_dim + d0 + ch] = v;
    }
  }

  if (GRAD) {
    // <dY, C> of this CTA: warp shuffle, then a fixed-order sum over the warps
    __syncthreads();
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) de_acc += __shfl_xor_sync(0xffffffffu, de_acc, o);
    if (lane == 0) red[warp] = de_acc;
    __syncthreads();
    if (tid == 0) {
      float v = 0.f;
      for (int w = 0; w < NT / 32; ++w) v += red[w];
      // two slots per 64-channel block (the 32-channel TMA kernel fills both)
      float* de = p.de_partials + ((size_t)sys * p.chunks + chunk) * (2 * p.dblocks);
      de[2 * dblk] = v;
      de[2 * dblk + 1] = 0.f;
    }
  }
}

int launch_stats_tma(const ms_shape& s, const Plan& plan, bool grad, const void* projected, const void* dy,
                     const float* cos, const float* sin, float* partials, float* de_partials,
                     const float* base_raw, const float* eta_raw, const ms_tape* core_tape, cudaStream_t st);

// Sum partials in chunk order and apply 1/n (Gram) and 1/sqrt(n) (moment) with IEEE rounding.
// packed forward:  [systems][r*r + r*d]      packed adjoint: [systems][r*d] then [systems] de
__global__ void pack_stats_kernel(const float* __restrict__ partials, const float* __restrict__ de_partials,
                                  const float* __restrict__ counts, float* __restrict__ packed,
                                  int heads, int tokens, int chunks, int de_slots, int gram_floats,
                                  int partial_floats, int systems, int grad) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int sys = blockIdx.y;
  const int b = sys / heads;
  const float n = counts ? counts[b] : (float)tokens;
  const float inv_n = inv_rn(n), inv_s = inv_sqrt_rn(n);
  const float* src = partials + (size_t)sys * chunks * partial_floats;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < partial_floats; i += gridDim.x * blockDim.x) {
    // chunk order is kept; eight loads are in flight at a time
    float v = 0.f;
    int c = 0;
    for (; c + 8 <= chunks; c += 8) {
      float t[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) t[u] = src[(size_t)(c + u) * partial_floats + i];
#pragma unroll
      for (int u = 0; u < 8; ++u) v += t[u];
    }
    for (; c < chunks; ++c) v += src[(size_t)c * partial_floats + i];
    packed[(size_t)sys * partial_floats + i] = v * (i < gram_floats ? inv_n : inv_s);
  }
  if (grad && blockIdx.x == 0 && threadIdx.x == 0) {
    float v = 0.f;
    for (int c = 0; c < chunks * de_slots; ++c) v += de_partials[(size_t)sys * chunks * de_slots + c];
    packed[(size_t)systems * partial_floats + sys] = v;
  }
}

template <int R, bool GRAD, bool ROT, bool ALIGNED>
static int launch_one(const StatsParams& p, dim3 grid, cudaStream_t st) {
  using Sm = StatsSmem<R, GRAD, ROT>;
  auto kern = stats_kernel<R, GRAD, ROT, ALIGNED>;
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(kern), Sm::TOTAL) != MS_OK) return MS_ERR_LAUNCH;
  launch_kernel(kern, grid, dim3(StatsCfg<R>::MS * StatsCfg<R>::KS * 32), Sm::TOTAL, st, p);
  return cudaGetLastError() == cudaSuccess ? MS_OK : MS_ERR_LAUNCH;
}

template <int R, bool GRAD>
static int launch_rank(const StatsParams& p, dim3 grid, bool rot, bool aligned, cudaStream_t st) {
  if (rot) return aligned ? launch_one<R, GRAD, true, true>(p, grid, st) : launch_one<R, GRAD, true, false>(p, grid, st);
  return aligned ? launch_one<R, GRAD, false, true>(p, grid, st) : launch_one<R, GRAD, false, false>(p, grid, st);
}

int launch_stats_tc(const ms_shape& s, const Plan& plan, bool grad, const void* projected, const void* dy,
                    const float* cos, const float* sin, float* partials, float* de_partials, const float* base_raw,
                    const float* eta_raw, const ms_tape* core_tape, cudaStream_t st);

int launch_stats(const ms_shape& s, const Plan& plan, bool grad, const void* projected, const void* dy,
                 const float* cos, const float* sin, float* partials, float* de_partials,
                 const float* base_raw, const float* eta_raw, const ms_tape* core_tape, cudaStream_t st) {
  if (plan.tc) {
    const int r = launch_stats_tc(s, plan, grad, projected, dy, cos, sin, partials, de_partials, base_raw, eta_raw,
                                  core_tape, st);
    if (r != -1) return r;
  }
  if (plan.tma) {
    const int r = launch_stats_tma(s, plan, grad, projected, dy, cos, sin, partials, de_partials, base_raw, eta_raw,
                                   core_tape, st);
    if (r != -1) return r;
  }
  StatsParams p;
  const bool fuse_core = !grad && core_tape != nullptr;
  p.base_raw = base_raw;
  p.eta_raw = eta_raw;
  p.eta = fuse_core ? core_tape->eta : nullptr;
  p.eta_slope = fuse_core ? core_tape->eta_slope : nullptr;
  p.core_map = fuse_core ? core_tape->core_map : nullptr;
  p.core_info = fuse_core ? core_tape->core_info : nullptr;
  p.complement = s.complement;
  p.projected = static_cast<const __nv_bfloat16*>(projected);
  p.dy = static_cast<const __nv_bfloat16*>(dy);
  p.cos = cos;
  p.sin = sin;
  p.partials = partials;
  p.de_partials = de_partials;
  p.batch = s.batch; p.tokens = s.tokens; p.heads = s.heads; p.head_dim = s.head_dim;
  p.width = s.heads * (s.rank + s.head_dim);
  p.rotary_rows = s.rotary_rows;
  p.chunks = plan.chunks; p.chunk_tokens = plan.chunk_tokens; p.dblocks = plan.dblocks;
  p.partial_floats = (int)(grad ? plan.bwd_partial_floats : plan.fwd_partial_floats);
  dim3 grid(plan.chunks + (fuse_core ? 1 : 0), plan.systems, plan.dblocks);
  const bool rot = s.rotary_rows > 0;
  switch (s.rank) {
    case 16: return grad ? launch_rank<16, true>(p, grid, rot, plan.aligned, st) : launch_rank<16, false>(p, grid, rot, plan.aligned, st);
    case 32: return grad ? launch_rank<32, true>(p, grid, rot, plan.aligned, st) : launch_rank<32, false>(p, grid, rot, plan.aligned, st);
    case 48: return grad ? launch_rank<48, true>(p, grid, rot, plan.aligned, st) : launch_rank<48, false>(p, grid, rot, plan.aligned, st);
    case 64: return grad ? launch_rank<64, true>(p, grid, rot, plan.aligned, st) : launch_rank<64, false>(p, grid, rot, plan.aligned, st);
  }
  return MS_ERR_UNSUPPORTED_RANK;
}

int launch_pack_stats(const ms_shape& s, const Plan& plan, bool grad, const float* partials,
                      const float* de_partials, const float* counts, float* packed, cudaStream_t st) {
  const int pf = (int)(grad ? plan.bwd_partial_floats : plan.fwd_partial_floats);
  dim3 grid((pf + 255) / 256, plan.systems);
  launch_kernel(pack_stats_kernel, grid, dim3(256), 0, st, partials, de_partials, counts, packed, s.heads, s.tokens,
                plan.chunks, plan.de_slots, grad ? 0 : s.rank * s.rank, pf, plan.systems, grad ? 1 : 0);
  return cudaGetLastError() == cudaSuccess ? MS_OK : MS_ERR_LAUNCH;
}

}  // namespace ms
