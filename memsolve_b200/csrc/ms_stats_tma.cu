// Token reductions -- TMA / independent-warp version.
//
//   forward:  G += A^T A,  Q += A^T rot(C)            adjoint:  E += A^T rot(dY),  de += <dY, C>
//
// Same arithmetic as stats_kernel in ms_stats.cu (the reference's `_statistics` /
// `_chunk_statistics`, memsolve/ball/cuda.py:1542-1667, 1925-2046).  Used when the head
// dimension is a multiple of 64, the pointers are 16-byte aligned and the accumulators of one
// warp fit its registers (forward: rank 16 or 32; adjoint: rank 16, 32 or 64).
//
// A CTA owns one (system, token chunk, 64-channel block) and produces one partial, exactly like
// the generic kernel, but its warps (eight to twelve) never meet at a barrier while streaming: warp w
// of W takes the 16-token slices w, w + W, ... of the chunk, lane 0 brings the slice's relation / content /
// gradient boxes and its rotary table rows into the warp's own ring of shared-memory stages
// with TMA (one mbarrier per stage), the warp rotates the content in FP32, splits it into two
// BF16 words and feeds mma.sync with the full r x (r + 64) accumulator held in registers.
// At the end the warps' accumulators are added in warp order through shared memory.
// SOLO variant (many short sequences, see solo_shape): four-warp CTAs, several per SM; warp w of CTA x
// owns system 4 x + w, streams all its slices and stores its accumulator fragments as the partial.
#include "ms_core.cuh"
#include "ms_tma.cuh"

namespace ms {


// CB: channels of one CTA (64, or 32 so that two CTAs with half the accumulators share an SM; the
// Gram columns are then divided between the first two channel blocks of a head).
template <int R, bool GRAD, bool ROT, int CB, int STAGES_, int WARPS_, bool SOLO = false>
struct StatsTmaCfg {
  static constexpr int kStWarps = WARPS_;
  static constexpr int A_SLICE = 16 * R * 2;
  static constexpr int X_BYTES = 16 * CB * 2;
  static constexpr int T_BYTES = 16 * (CB / 2) * 4;   // one table (cos or sin), 16 rows x CB/2 floats
  static constexpr int RAW = X_BYTES + (GRAD ? X_BYTES : 0) + (ROT ? 2 * T_BYTES : 0) + A_SLICE;
  static constexpr int STAGE = ((RAW + 1023) / 1024) * 1024;
  static constexpr int STAGES = STAGES_;
  static constexpr int LO = ROT ? X_BYTES : 0;
  static constexpr int WARP_BYTES = STAGES * STAGE + ((LO + 1023) / 1024) * 1024;
  static constexpr int RING = kStWarps * WARP_BYTES;
  static constexpr int GP = (CB == 32 && R >= 32) ? 2 : 1;            // channel blocks sharing the Gram columns
  static constexpr int GCOLS = GRAD ? 0 : R / GP;
  static constexpr int RCOLS = GCOLS + CB;
  static constexpr int RED = SOLO ? 0 : kStWarps * R * RCOLS * 4;
  static constexpr int CORE = GRAD ? 0 : (int)core_forward_smem_bytes(R);
  static constexpr int BODY = RING > RED ? (RING > CORE ? RING : CORE) : (RED > CORE ? RED : CORE);
  static constexpr int BARS = kStWarps * STAGES * 8;
  static constexpr int TOTAL = 1024 + BODY + BARS + 64;
};

struct StatsTmaParams {
  float* partials;
  float* de_partials;
  int* error;
  int tokens, heads, head_dim, rotary_rows, chunks, chunk_tokens, de_slots, partial_floats;
  int systems, work_ctas;   // warp-per-system variant: B*H and the CTAs that stream (the rest run the core)
  const float* base_raw;
  const float* eta_raw;
  float* eta;
  float* eta_slope;
  float* core_map;
  int* core_info;
  int complement;
};

template <int R, bool GRAD, bool ROT, int CB, int STAGES_, int WARPS_, bool SOLO = false, int MINB = 1>
__global__ void __launch_bounds__(WARPS_ * 32, MINB)
stats_tma_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_c,
                 const __grid_constant__ CUtensorMap map_y, const __grid_constant__ CUtensorMap map_cos,
                 const __grid_constant__ CUtensorMap map_sin, const StatsTmaParams p) {
  using Cfg = StatsTmaCfg<R, GRAD, ROT, CB, STAGES_, WARPS_, SOLO>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int kStWarps = WARPS_;
  constexpr int MT = R / 16, NG = Cfg::GCOLS / 8, NQ = CB / 8;
  constexpr int NT = kStWarps * 32;
  constexpr int XP = CB * 2;   // row pitch in bytes of the content / gradient / table tiles
  extern __shared__ unsigned char smem_raw[];
  const uint32_t smem = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* smem_gen = smem_raw + (smem - smem_u32(smem_raw));

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // SOLO: warp w of CTA x owns system x * WARPS + w and streams all its tokens (many short sequences);
  // otherwise the CTA owns (system, token chunk) and its warps share the slices of the chunk
  const int chunk = SOLO ? 0 : blockIdx.x, dblk = blockIdx.z;
  const int sys_raw = SOLO ? (int)blockIdx.x * kStWarps + warp : (int)blockIdx.y;
  const bool spare = SOLO ? (int)blockIdx.x >= p.work_ctas : (!GRAD && chunk == p.chunks);
  if (spare) {
    grid_launch_dependents();
    grid_dependency_wait();
    // spare CTAs of the grid: the per-head core runs beside the token reduction
    const int head = SOLO ? (int)blockIdx.x - p.work_ctas : sys_raw;
    if (!GRAD && dblk == 0 && head < p.heads)
      core_forward_device<R, NT>(p.base_raw, p.eta_raw, head, p.complement, p.eta, p.eta_slope, p.core_map,
                                 p.core_info, smem_gen, tid);
    return;
  }
  const bool active = !SOLO || sys_raw < p.systems;
  const int sys = active ? sys_raw : 0;
  const int b = sys / p.heads, h = sys - b * p.heads;
  const int d0 = dblk * CB;
  const int tok0 = chunk * p.chunk_tokens;
  const int tok1 = min(p.tokens, tok0 + p.chunk_tokens);
  const int slice0 = tok0 >> 4;
  const int nslices = (tok1 - tok0 + 15) >> 4;
  const int first_slice = SOLO ? 0 : warp, slice_step = SOLO ? 1 : kStWarps;
  const int n_items = SOLO ? (active ? nslices : 0)
                           : (nslices > warp ? (nslices - warp + kStWarps - 1) / kStWarps : 0);
  const bool do_gram = !GRAD && dblk < Cfg::GP;
  const int gcol0 = dblk * Cfg::GCOLS;   // first Gram column of this CTA (when do_gram)
  const int tab_b = p.rotary_rows > 1 ? b : 0;

  const uint32_t ring = smem + warp * Cfg::WARP_BYTES;
  const uint32_t lo_tile = ring + STAGES * Cfg::STAGE;
  const uint32_t bars = smem + Cfg::BODY;
  const uint32_t mybar = bars + warp * STAGES * 8;

  if (tid == 0) {
    for (int i = 0; i < kStWarps * STAGES; ++i) mbar_init(bars + i * 8, 1);
    mbar_fence_init();
  }
  __syncthreads();
  grid_dependency_wait();

  // stage layout: [X: dY (adjoint) or C][C (adjoint only)][cos][sin][A]
  constexpr int OFF_C = Cfg::X_BYTES;
  constexpr int OFF_T = Cfg::X_BYTES + (GRAD ? Cfg::X_BYTES : 0);
  constexpr int OFF_A = OFF_T + (ROT ? 2 * Cfg::T_BYTES : 0);
  constexpr uint32_t TX = Cfg::X_BYTES + (GRAD ? Cfg::X_BYTES : 0) + (ROT ? 2 * Cfg::T_BYTES : 0) + Cfg::A_SLICE;

  // item k of this warp refills ring stage k % STAGES
  auto issue = [&](int k, int stage) {
    const int row = (slice0 + first_slice + k * slice_step) * 16;
    const uint32_t st = ring + stage * Cfg::STAGE;
    const uint32_t bar = mybar + stage * 8;
    mbar_expect_tx(bar, TX);
    const int ccol = p.heads * R + h * p.head_dim + d0;
    if (GRAD) {
      tma_load_3d(st, &map_y, h * p.head_dim + d0, row, b, bar);
      tma_load_3d(st + OFF_C, &map_c, ccol, row, b, bar);
    } else {
      tma_load_3d(st, &map_c, ccol, row, b, bar);
    }
    if (ROT) {
      tma_load_3d(st + OFF_T, &map_cos, d0 >> 1, row, tab_b, bar);
      tma_load_3d(st + OFF_T + Cfg::T_BYTES, &map_sin, d0 >> 1, row, tab_b, bar);
    }
    tma_load_3d(st + OFF_A, &map_a, h * R, row, b, bar);
  };

  float accG[GRAD ? 1 : MT][GRAD ? 1 : NG][4];
  float accQ[MT][NQ][4];
#pragma unroll
  for (int i = 0; i < (GRAD ? 1 : MT); ++i)
#pragma unroll
    for (int j = 0; j < (GRAD ? 1 : NG); ++j)
#pragma unroll
      for (int q = 0; q < 4; ++q) accG[i][j][q] = 0.f;
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < NQ; ++j)
#pragma unroll
      for (int q = 0; q < 4; ++q) accQ[i][j][q] = 0.f;
  float de_part[4] = {0.f, 0.f, 0.f, 0.f};

  if (lane == 0) {
    for (int k = 0; k < STAGES && k < n_items; ++k) issue(k, k);
  }
  bool ok = true;
  const int mi = lane >> 3, mr = lane & 7;

  int stage = 0;
  uint32_t parity = 0;
  for (int k = 0; k < n_items; ++k) {
    const uint32_t st = ring + stage * Cfg::STAGE;
    const uint32_t x_tile = st;
    const uint32_t c_tile = st + OFF_C;
    const uint32_t cos_tile = st + OFF_T;
    const uint32_t sin_tile = cos_tile + Cfg::T_BYTES;
    const uint32_t a_tile = st + OFF_A;
    ok = mbar_wait(mybar + stage * 8, parity);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) break;

    if (ROT || GRAD) {
      // elementwise pass over the 16 x CB slice, one 16-byte chunk (8 channels) at a time
#pragma unroll
      for (int it = 0; it < CB / 16; ++it) {
        const int i = lane + it * 32;
        const int row = i / (CB / 8), c = i % (CB / 8);
        const uint32_t off = swz_rows<XP>(row * XP + c * 16);
        const uint4 xv = ld_shared_v4(x_tile + off);
        const uint32_t xs[4] = {xv.x, xv.y, xv.z, xv.w};
        if (GRAD) {
          const uint4 cv = ld_shared_v4(c_tile + off);
          const uint32_t cs[4] = {cv.x, cv.y, cv.z, cv.w};
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float2 xf = bf2_to_f2(xs[q]), cf = bf2_to_f2(cs[q]);
            de_part[q] = fmaf(xf.x, cf.x, de_part[q]);   // four independent chains
            de_part[q] = fmaf(xf.y, cf.y, de_part[q]);
          }
        }
        if (ROT) {
          const float4 cc = ld_shared_f4(cos_tile + row * XP + c * 16);
          const float4 ss = ld_shared_f4(sin_tile + row * XP + c * 16);
          const float cf[4] = {cc.x, cc.y, cc.z, cc.w};
          const float sf[4] = {ss.x, ss.y, ss.z, ss.w};
          uint32_t hi[4], lo[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float2 v = bf2_to_f2(xs[q]);
            const float2 r = rot_pair(v.x, v.y, cf[q], sf[q]);
            split2(r.x, r.y, hi[q], lo[q]);
          }
          st_shared_v4(x_tile + off, make_uint4(hi[0], hi[1], hi[2], hi[3]));
          st_shared_v4(lo_tile + off, make_uint4(lo[0], lo[1], lo[2], lo[3]));
        }
      }
      if (ROT) __syncwarp();
    }

    uint32_t af[MT][4];
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      // A^T as the row operand: stored [token][rank], transposed on load
      ldsm_x4_t(af[m], a_tile + swz_rows<R * 2>((mr + 8 * (mi >> 1)) * (R * 2) + (m * 16 + 8 * (mi & 1)) * 2));
    }
    if (!GRAD) {
      if (do_gram) {
#pragma unroll
        for (int n2 = 0; n2 < NG / 2; ++n2) {
          uint32_t bf[4];
          ldsm_x4_t(bf, a_tile + swz_rows<R * 2>((mr + 8 * (mi & 1)) * (R * 2) +
                                                 (gcol0 + n2 * 16 + 8 * (mi >> 1)) * 2));
#pragma unroll
          for (int m = 0; m < MT; ++m) {
            mma_bf16(accG[m][2 * n2], af[m], bf[0], bf[1]);
            mma_bf16(accG[m][2 * n2 + 1], af[m], bf[2], bf[3]);
          }
        }
      }
    }
#pragma unroll
    for (int n2 = 0; n2 < NQ / 2; ++n2) {
      const uint32_t off = swz_rows<XP>((mr + 8 * (mi & 1)) * XP + (n2 * 16 + 8 * (mi >> 1)) * 2);
      uint32_t bf[4];
      if (ROT) {
        ldsm_x4_t(bf, lo_tile + off);   // residual word first, dominant word last
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
    // refill this stage: order the warp's shared-memory accesses before the async-proxy write
    if (k + STAGES < n_items) {
      fence_async_shared();
      __syncwarp();
      if (lane == 0) issue(k + STAGES, stage);
    }
    if (++stage == STAGES) {
      stage = 0;
      parity ^= 1u;
    }
  }
  if (!ok && lane == 0) atomicExch(p.error, kErrBarrierTimeout);
  grid_launch_dependents();
  if (SOLO) {
    // the warp holds the whole sum of its system: store the accumulator fragments as they are
    if (!active) return;
    const int g = lane >> 2, tq = lane & 3;
    float* out = p.partials + (size_t)sys * p.partial_floats;
    float* outq = out + (GRAD ? 0 : R * R) + d0;
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      const int r0 = m * 16 + g;
      if (!GRAD && do_gram) {
#pragma unroll
        for (int n = 0; n < NG; ++n) {
          const int col = gcol0 + n * 8 + 2 * tq;
          *reinterpret_cast<float2*>(out + r0 * R + col) = make_float2(accG[m][n][0], accG[m][n][1]);
          *reinterpret_cast<float2*>(out + (r0 + 8) * R + col) = make_float2(accG[m][n][2], accG[m][n][3]);
        }
      }
#pragma unroll
      for (int n = 0; n < NQ; ++n) {
        const int col = n * 8 + 2 * tq;
        *reinterpret_cast<float2*>(outq + r0 * p.head_dim + col) = make_float2(accQ[m][n][0], accQ[m][n][1]);
        *reinterpret_cast<float2*>(outq + (r0 + 8) * p.head_dim + col) = make_float2(accQ[m][n][2], accQ[m][n][3]);
      }
    }
    if (GRAD) {
      float de_acc = (de_part[0] + de_part[1]) + (de_part[2] + de_part[3]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) de_acc += __shfl_xor_sync(0xffffffffu, de_acc, o);
      if (lane == 0) {
        float* de = p.de_partials + (size_t)sys * p.de_slots;
        de[2 * dblk] = de_acc;
        de[2 * dblk + 1] = 0.f;
      }
    }
    return;
  }
  __syncthreads();

  // ---- add the warp accumulators in warp order, write one partial ---------------------
  constexpr int RCOLS = Cfg::RCOLS;
  float* red = reinterpret_cast<float*>(smem_gen);
  {
    const int g = lane >> 2, tq = lane & 3;
    float* mine = red + (size_t)warp * R * RCOLS;
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      const int r0 = m * 16 + g;
      if (!GRAD) {
#pragma unroll
        for (int n = 0; n < NG; ++n) {
          const int col = n * 8 + 2 * tq;
          *reinterpret_cast<float2*>(mine + r0 * RCOLS + col) = make_float2(accG[m][n][0], accG[m][n][1]);
          *reinterpret_cast<float2*>(mine + (r0 + 8) * RCOLS + col) = make_float2(accG[m][n][2], accG[m][n][3]);
        }
      }
#pragma unroll
      for (int n = 0; n < NQ; ++n) {
        const int col = Cfg::GCOLS + n * 8 + 2 * tq;
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
    for (int w = 0; w < kStWarps; ++w) v += red[(size_t)w * R * RCOLS + i];
    if (col < Cfg::GCOLS) {
      if (do_gram) out[row * R + gcol0 + col] = v;
    } else {
      out[gfloats + row * p.head_dim + d0 + col - Cfg::GCOLS] = v;
    }
  }
  if (GRAD) {
    __syncthreads();
    float de_acc = (de_part[0] + de_part[1]) + (de_part[2] + de_part[3]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) de_acc += __shfl_xor_sync(0xffffffffu, de_acc, o);
    if (lane == 0) red[warp] = de_acc;
    __syncthreads();
    if (tid == 0) {
      float v = 0.f;
      for (int w = 0; w < kStWarps; ++w) v += red[w];
      // de slots: two per 64-channel block
      float* de = p.de_partials + ((size_t)sys * p.chunks + chunk) * p.de_slots;
      if (CB == 32) {
        de[dblk] = v;
      } else {
        de[2 * dblk] = v;
        de[2 * dblk + 1] = 0.f;
      }
    }
  }
}

template <int R, bool GRAD, bool ROT, int CB, int STAGES, int WARPS>
static int launch_stats_tma_one(const ms_shape& s, const Plan& plan, const CUtensorMap* maps, const StatsTmaParams& p,
                                bool fuse_core, cudaStream_t st) {
  using Cfg = StatsTmaCfg<R, GRAD, ROT, CB, STAGES, WARPS>;
  auto kern = stats_tma_kernel<R, GRAD, ROT, CB, STAGES, WARPS>;
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(kern), Cfg::TOTAL)) return MS_ERR_LAUNCH;
  dim3 grid(plan.chunks + (fuse_core ? 1 : 0), plan.systems, s.head_dim / CB);
  launch_kernel(kern, grid, dim3(WARPS * 32), Cfg::TOTAL, st, maps[0], maps[1], maps[2], maps[3], maps[4], p);
  return cudaGetLastError() == cudaSuccess ? MS_OK : MS_ERR_LAUNCH;
}

// Many short sequences (one chunk per system, see solo_shape): four-warp CTAs, several per SM, in which
// every warp reduces one whole system and writes its partial itself.
constexpr int kSoloWarps = 4;

template <int R, bool GRAD, bool ROT>
static int launch_stats_tma_solo(const ms_shape& s, const Plan& plan, const CUtensorMap* maps, StatsTmaParams p,
                                 bool fuse_core, cudaStream_t st) {
  constexpr int MINB = GRAD ? 2 : 3;
  using Cfg = StatsTmaCfg<R, GRAD, ROT, 64, 2, kSoloWarps, true>;
  auto kern = stats_tma_kernel<R, GRAD, ROT, 64, 2, kSoloWarps, true, MINB>;
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(kern), Cfg::TOTAL)) return MS_ERR_LAUNCH;
  p.systems = plan.systems;
  p.work_ctas = (plan.systems + kSoloWarps - 1) / kSoloWarps;
  dim3 grid(p.work_ctas + (fuse_core ? s.heads : 0), 1, s.head_dim / 64);
  launch_kernel(kern, grid, dim3(kSoloWarps * 32), Cfg::TOTAL, st, maps[0], maps[1], maps[2], maps[3], maps[4], p);
  return cudaGetLastError() == cudaSuccess ? MS_OK : MS_ERR_LAUNCH;
}

// Worth it when the warps that stream (one per system) fill the machine: four systems per SM, or one
// per SM when a system is so short that a twelve-warp CTA would mostly add up its warps' accumulators.
static bool solo_shape(const ms_shape& s, const Plan& plan) {
  if (plan.chunks != 1 || s.tokens > 1024) return false;
  return plan.systems >= 4 * sm_count() || (plan.systems >= sm_count() && s.tokens <= 256);
}

template <int R, bool GRAD, int CB, int STAGES, int WARPS = 8>
static int launch_stats_tma_r(const ms_shape& s, const Plan& plan, const void* projected, const void* dy,
                              const float* cos, const float* sin, StatsTmaParams& p, bool fuse_core,
                              cudaStream_t st) {
  const int d = s.head_dim, width = s.heads * (R + d), dmodel = s.heads * d;
  CUtensorMap maps[5];
  {
    const uint64_t dims[3] = {(uint64_t)width, (uint64_t)s.tokens, (uint64_t)s.batch};
    const uint64_t str[2] = {(uint64_t)width * 2, (uint64_t)s.tokens * width * 2};
    const uint32_t box_a[3] = {(uint32_t)R, 16, 1};
    const uint32_t box_c[3] = {(uint32_t)CB, 16, 1};
    if (encode_tensor_map(&maps[0], const_cast<void*>(projected), 2, 3, dims, str, box_a, swizzle_for_rows<R * 2>()))
      return MS_ERR_LAUNCH;
    if (encode_tensor_map(&maps[1], const_cast<void*>(projected), 2, 3, dims, str, box_c, swizzle_for_rows<CB * 2>()))
      return MS_ERR_LAUNCH;
  }
  maps[2] = maps[1];
  if (GRAD) {
    const uint64_t dims[3] = {(uint64_t)dmodel, (uint64_t)s.tokens, (uint64_t)s.batch};
    const uint64_t str[2] = {(uint64_t)dmodel * 2, (uint64_t)s.tokens * dmodel * 2};
    const uint32_t box[3] = {(uint32_t)CB, 16, 1};
    if (encode_tensor_map(&maps[2], const_cast<void*>(dy), 2, 3, dims, str, box, swizzle_for_rows<CB * 2>()))
      return MS_ERR_LAUNCH;
  }
  maps[3] = maps[1];
  maps[4] = maps[1];
  const bool rot = s.rotary_rows > 0;
  if (rot) {
    const int half = d / 2;
    const uint64_t dims[3] = {(uint64_t)half, (uint64_t)s.tokens, (uint64_t)s.rotary_rows};
    const uint64_t str[2] = {(uint64_t)half * 4, (uint64_t)s.tokens * half * 4};
    const uint32_t box[3] = {(uint32_t)(CB / 2), 16, 1};
    if (encode_tensor_map(&maps[3], const_cast<float*>(cos), 4, 3, dims, str, box, Swizzle::None)) return MS_ERR_LAUNCH;
    if (encode_tensor_map(&maps[4], const_cast<float*>(sin), 4, 3, dims, str, box, Swizzle::None)) return MS_ERR_LAUNCH;
  }
  if (CB == 64 && (GRAD || R <= 32) && solo_shape(s, plan))
    return rot ? launch_stats_tma_solo<R, GRAD, true>(s, plan, maps, p, fuse_core, st)
               : launch_stats_tma_solo<R, GRAD, false>(s, plan, maps, p, fuse_core, st);
  return rot ? launch_stats_tma_one<R, GRAD, true, CB, STAGES, WARPS>(s, plan, maps, p, fuse_core, st)
             : launch_stats_tma_one<R, GRAD, false, CB, STAGES, WARPS>(s, plan, maps, p, fuse_core, st);
}

// MS_OK / error, or -1 when the shape is outside this kernel's envelope.
int launch_stats_tma(const ms_shape& s, const Plan& plan, bool grad, const void* projected, const void* dy,
                     const float* cos, const float* sin, float* partials, float* de_partials,
                     const float* base_raw, const float* eta_raw, const ms_tape* core_tape, cudaStream_t st) {
  if (!plan.aligned || (s.head_dim % 64) != 0) return -1;
  if ((plan.chunk_tokens % 16) != 0) return -1;
  StatsTmaParams p;
  p.partials = partials; p.de_partials = de_partials;
  p.error = device_error_word();
  if (!p.error) return MS_ERR_LAUNCH;
  p.tokens = s.tokens; p.heads = s.heads; p.head_dim = s.head_dim; p.rotary_rows = s.rotary_rows;
  p.chunks = plan.chunks; p.chunk_tokens = plan.chunk_tokens; p.de_slots = plan.de_slots;
  p.partial_floats = (int)(grad ? plan.bwd_partial_floats : plan.fwd_partial_floats);
  const bool fuse_core = !grad && core_tape != nullptr;
  p.base_raw = base_raw; p.eta_raw = eta_raw;
  p.eta = fuse_core ? core_tape->eta : nullptr;
  p.eta_slope = fuse_core ? core_tape->eta_slope : nullptr;
  p.core_map = fuse_core ? core_tape->core_map : nullptr;
  p.core_info = fuse_core ? core_tape->core_info : nullptr;
  p.complement = s.complement;
  p.systems = plan.systems; p.work_ctas = 0;
  if (grad) {
    switch (s.rank) {
      case 16: return launch_stats_tma_r<16, true, 64, 2>(s, plan, projected, dy, cos, sin, p, false, st);
      case 32: return launch_stats_tma_r<32, true, 64, 2>(s, plan, projected, dy, cos, sin, p, false, st);
      case 64: return launch_stats_tma_r<64, true, 64, 2>(s, plan, projected, dy, cos, sin, p, false, st);
    }
    return -1;
  }
  switch (s.rank) {
    case 16: return launch_stats_tma_r<16, false, 64, 3>(s, plan, projected, dy, cos, sin, p, fuse_core, st);
    // rank 32: twelve warps with two stages each fit the register file and hide more latency
    case 32: return launch_stats_tma_r<32, false, 64, 2, 12>(s, plan, projected, dy, cos, sin, p, fuse_core, st);
  }
  return -1;
}

}  // namespace ms
