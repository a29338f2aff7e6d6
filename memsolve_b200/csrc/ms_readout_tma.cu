// Readout  Y = eta*C + rot^-1(A_raw W)/sqrt(n)  -- TMA / persistent-warp version.
//
// Used when the head dimension is a multiple of 64, the rank is 16, 32 or 64 and all pointers
// are 16-byte aligned; other shapes take readout_kernel in ms_token.cu.  Same arithmetic as
// that kernel (the reference's `_readout`, memsolve/ball/cuda.py:1670-1764).
//
// Layout of the work: a CTA serves one sample and one group of heads.  The coefficient
// matrices W (two BF16 words) of all heads of the group are brought into shared memory once
// with TMA and stay there.  Each warp then walks over its own contiguous range of
// (16-token slice, head, 64-channel block) items: lane 0 issues the TMA loads of the slice's
// relation and content boxes into the warp's private ring of buffers (mbarrier per stage, two
// items of prefetch), the warp multiplies with mma.sync, applies the inverse rotation and the
// eta*C term in registers, writes the BF16 result over the content box and lane 0 sends it out
// with a TMA store.  There is no CTA-wide barrier after the prologue, no per-thread copy
// instruction, and out-of-range tokens are clipped by the 3-D tensor maps.
#include "ms_tma.cuh"

namespace ms {

constexpr int kRtSmemLimit = 227 * 1024;   // dynamic shared memory available to one CTA

// WARPS independent warps per CTA, each with a ring of STAGES buffers of which PRE are in flight
// ahead of the one being computed (STAGES - PRE - 1 buffers may still be read by earlier stores).
template <int R, int WARPS_, int STAGES_, int PRE_>
struct ReadoutTmaCfg {
  static constexpr int WARPS = WARPS_;
  static constexpr int STAGES = STAGES_;
  static constexpr int PRE = PRE_;
  static constexpr int A_SLICE = 16 * R * 2;
  static constexpr int C_SLICE = 16 * 128;
  static constexpr int STAGE = ((A_SLICE + C_SLICE + 1023) / 1024) * 1024;
  static constexpr int W_BYTES = R * 128;  // one word of one (head, 64-channel block)
  static constexpr int RING = WARPS * STAGES * STAGE;
  static_assert(PRE >= 1 && PRE < STAGES, "prefetch depth");
};

struct ReadoutTmaParams {
  const float* cos;
  const float* sin;
  const float* counts;
  const float* eta;
  int* error;
  int tokens, heads, head_dim, rotary_rows, dblocks;
  int group_heads;   // heads per CTA group
  int slices;        // ceil(tokens / 16)
};

template <int R, bool ROT, class Cfg>
__global__ void __launch_bounds__(Cfg::WARPS * 32)
readout_tma_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_c,
                   const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_y,
                   const ReadoutTmaParams p) {
  constexpr int STAGES = Cfg::STAGES;
  constexpr int PRE = Cfg::PRE;
  constexpr int kRtWarps = Cfg::WARPS;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t smem = (smem_u32(smem_raw) + 1023u) & ~1023u;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  grid_launch_dependents();
  const int b = blockIdx.y;
  const int h0 = blockIdx.z * p.group_heads;
  const int gh = min(p.group_heads, p.heads - h0);
  const int mats = gh * p.dblocks;                  // (head, block) pairs resident in this CTA
  const uint32_t w_base = smem;
  const uint32_t ring = smem + p.group_heads * p.dblocks * 2 * Cfg::W_BYTES + warp * STAGES * Cfg::STAGE;
  const uint32_t bars = smem + p.group_heads * p.dblocks * 2 * Cfg::W_BYTES + Cfg::RING;
  const uint32_t wbar = bars + kRtWarps * STAGES * 8;
  const uint32_t mybar = bars + warp * STAGES * 8;

  if (tid == 0) {
    for (int i = 0; i < kRtWarps * STAGES + 1; ++i) mbar_init(bars + i * 8, 1);
    mbar_fence_init();
  }
  __syncthreads();
  // contiguous item range of this warp; item = (slice, head-in-group, block)
  const int total = p.slices * mats;
  const int nwarps = gridDim.x * kRtWarps;
  const int per = (total + nwarps - 1) / nwarps;
  const int it0 = min(total, (blockIdx.x * kRtWarps + warp) * per);
  const int n_items = min(total, it0 + per) - it0;

  const int d = p.head_dim, half = d >> 1;
  const float n = p.counts ? p.counts[b] : (float)p.tokens;
  const float inv_s = inv_sqrt_rn(n);
  const long tab_b = p.rotary_rows > 1 ? (long)b * p.tokens : 0;
  const int g = lane >> 2, tq = lane & 3;
  const int mi = lane >> 3, mr = lane & 7;

  // position of an item: (slice, head in group, channel block); advanced without divisions
  struct Cursor {
    int slice, hl, jb, stage;
  };
  auto advance = [&](Cursor& c) {
    if (++c.jb == p.dblocks) {
      c.jb = 0;
      if (++c.hl == gh) {
        c.hl = 0;
        ++c.slice;
      }
    }
    c.stage = c.stage + 1 == STAGES ? 0 : c.stage + 1;
  };
  Cursor ahead;   // next item to load
  ahead.slice = it0 / mats;
  ahead.hl = (it0 - ahead.slice * mats) / p.dblocks;
  ahead.jb = it0 - ahead.slice * mats - ahead.hl * p.dblocks;
  ahead.stage = 0;
  Cursor cur = ahead;   // item being computed
  uint32_t parity = 0;

  auto issue = [&](const Cursor& c) {
    const int h = h0 + c.hl;
    const uint32_t st = ring + c.stage * Cfg::STAGE;
    const uint32_t bar = mybar + c.stage * 8;
    mbar_expect_tx(bar, Cfg::A_SLICE + Cfg::C_SLICE);
    tma_load_3d(st, &map_c, p.heads * R + h * d + c.jb * 64, c.slice * 16, b, bar);
    tma_load_3d(st + Cfg::C_SLICE, &map_a, h * R, c.slice * 16, b, bar);
  };

  for (int k = 0; k < PRE && k < n_items; ++k) {
    if (lane == 0) issue(ahead);
    advance(ahead);
  }
  // The token boxes above were requested before this point on purpose: `projected` and the counts were complete before the
  // kernel ahead of the previous one started, so a chained launch may fetch them while the previous kernel
  // (which produces the coefficient matrices) is still draining.
  grid_dependency_wait();
  if (tid == 0) {
    mbar_expect_tx(wbar, (uint32_t)(mats * 2 * Cfg::W_BYTES));
    for (int m = 0; m < mats; ++m) {
      const int hl = m / p.dblocks, jb = m - hl * p.dblocks;
      const int row = ((b * p.heads + h0 + hl) * 2) * R;
      tma_load_2d(w_base + (m * 2) * Cfg::W_BYTES, &map_w, jb * 64, row, wbar);
      tma_load_2d(w_base + (m * 2 + 1) * Cfg::W_BYTES, &map_w, jb * 64, row + R, wbar);
    }
  }
  bool ok = mbar_wait(wbar, 0);
  ok = __all_sync(0xffffffffu, ok);

  float tc[8][2], ts[8][2];
  int tab_slice = -1, tab_jb = -1;

  for (int k = 0; k < n_items && ok; ++k) {
    if (k + PRE < n_items) {
      if (lane == 0) {
        // the buffer being refilled was the source of the store of item k + PRE - STAGES
        tma_store_wait_read<STAGES - PRE - 1>();
        issue(ahead);
      }
      advance(ahead);
    }
    const int slice = cur.slice, hl = cur.hl, jb = cur.jb;
    const int m = hl * p.dblocks + jb;
    const int h = h0 + hl;
    const uint32_t c_tile = ring + cur.stage * Cfg::STAGE;
    const uint32_t a_tile = c_tile + Cfg::C_SLICE;
    const uint32_t wh_tile = w_base + (m * 2) * Cfg::W_BYTES;
    const uint32_t wl_tile = wh_tile + Cfg::W_BYTES;

    if (ROT && (slice != tab_slice || jb != tab_jb)) {
      const int row0 = slice * 16;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
          const int row = row0 + g + 8 * kk;
          float cv = 1.f, sv = 0.f;
          if (row < p.tokens) {
            const long idx = (tab_b + row) * half + jb * 32 + 4 * j + tq;
            cv = __ldg(p.cos + idx);
            sv = __ldg(p.sin + idx);
          }
          tc[j][kk] = cv * inv_s;    // the 1/sqrt(n) of the correction rides on the rotary factors
          ts[j][kk] = -sv * inv_s;   // inverse rotation
        }
      }
      tab_slice = slice;
      tab_jb = jb;
    }
    const float eta = __ldg(p.eta + h);

    ok = mbar_wait(mybar + cur.stage * 8, parity);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) break;

    float acc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[j][q] = 0.f;
#pragma unroll
    for (int ks = 0; ks < R / 16; ++ks) {
      uint32_t af[4];
      ldsm_x4(af, a_tile + swz_rows<R * 2>((mr + 8 * (mi & 1)) * (R * 2) + (ks * 16 + 8 * (mi >> 1)) * 2));
#pragma unroll
      for (int n2 = 0; n2 < 4; ++n2) {
        const uint32_t off = swz_rows<128>((ks * 16 + mr + 8 * (mi & 1)) * 128 + (n2 * 16 + 8 * (mi >> 1)) * 2);
        uint32_t bf[4];
        ldsm_x4_t(bf, wl_tile + off);   // residual word first, dominant word last
        mma_bf16(acc[2 * n2], af, bf[0], bf[1]);
        mma_bf16(acc[2 * n2 + 1], af, bf[2], bf[3]);
        ldsm_x4_t(bf, wh_tile + off);
        mma_bf16(acc[2 * n2], af, bf[0], bf[1]);
        mma_bf16(acc[2 * n2 + 1], af, bf[2], bf[3]);
      }
    }
    // the content box as row-operand fragments: the same (row, channel pair) per thread as the
    // accumulators, four ldmatrix instead of sixteen 4-byte loads
    uint32_t craw[4][4];
#pragma unroll
    for (int ks = 0; ks < 4; ++ks)
      ldsm_x4(craw[ks], c_tile + swz_rows<128>((mr + 8 * (mi & 1)) * 128 + (ks * 16 + 8 * (mi >> 1)) * 2));
    __syncwarp();   // every lane has read the box before the result is written over it
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {
        const uint32_t addr = c_tile + swz_rows<128>((g + 8 * kk) * 128 + (8 * j + 2 * tq) * 2);
        float2 corr = make_float2(acc[j][2 * kk], acc[j][2 * kk + 1]);
        if (ROT) corr = rot_pair(corr.x, corr.y, tc[j][kk], ts[j][kk]);
        else corr = make_float2(corr.x * inv_s, corr.y * inv_s);
        const float2 cv = bf2_to_f2(craw[j >> 1][2 * (j & 1) + kk]);
        st_shared_u32(addr, f2_to_bf2(fmaf(eta, cv.x, corr.x), fmaf(eta, cv.y, corr.y)));
      }
    }
    fence_async_shared();
    __syncwarp();
    if (lane == 0) {
      tma_store_3d(&map_y, h * d + jb * 64, slice * 16, b, c_tile);
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
static int launch_readout_tma_cfg(const ms_shape& s, const Plan& plan, const void* projected, const float* cos,
                                  const float* sin, const float* counts, const ms_tape& t, void* mixed,
                                  cudaStream_t st) {
  constexpr int WARPS = Cfg::WARPS;
  const int d = s.head_dim, heads = s.heads, width = heads * (R + d), dmodel = heads * d;
  const int per_head = plan.dblocks * 2 * Cfg::W_BYTES;
  const int fixed = 1024 + Cfg::RING + (WARPS * Cfg::STAGES + 1) * 8;
  int group = (kRtSmemLimit - fixed) / per_head;   // heads whose coefficients stay resident in one CTA
  if (group < 1) return -1;
  if (group > heads) group = heads;
  const int groups = (heads + group - 1) / group;
  group = (heads + groups - 1) / groups;           // balance the groups

  CUtensorMap map_a, map_c, map_w, map_y;
  {
    const uint64_t dims[3] = {(uint64_t)width, (uint64_t)s.tokens, (uint64_t)s.batch};
    const uint64_t str[2] = {(uint64_t)width * 2, (uint64_t)s.tokens * width * 2};
    const uint32_t box_a[3] = {(uint32_t)R, 16, 1};
    const uint32_t box_c[3] = {64, 16, 1};
    if (encode_tensor_map(&map_a, const_cast<void*>(projected), 2, 3, dims, str, box_a, swizzle_for_rows<R * 2>()))
      return MS_ERR_LAUNCH;
    if (encode_tensor_map(&map_c, const_cast<void*>(projected), 2, 3, dims, str, box_c, Swizzle::B128))
      return MS_ERR_LAUNCH;
  }
  {
    const uint64_t dims[2] = {(uint64_t)plan.dpad, (uint64_t)plan.systems * 2 * R};
    const uint64_t str[1] = {(uint64_t)plan.dpad * 2};
    const uint32_t box[2] = {64, (uint32_t)R};
    if (encode_tensor_map(&map_w, t.coeff, 2, 2, dims, str, box, Swizzle::B128)) return MS_ERR_LAUNCH;
  }
  {
    const uint64_t dims[3] = {(uint64_t)dmodel, (uint64_t)s.tokens, (uint64_t)s.batch};
    const uint64_t str[2] = {(uint64_t)dmodel * 2, (uint64_t)s.tokens * dmodel * 2};
    const uint32_t box[3] = {64, 16, 1};
    if (encode_tensor_map(&map_y, mixed, 2, 3, dims, str, box, Swizzle::B128)) return MS_ERR_LAUNCH;
  }

  ReadoutTmaParams p;
  p.cos = cos; p.sin = sin; p.counts = counts; p.eta = t.eta;
  p.error = device_error_word();
  if (!p.error) return MS_ERR_LAUNCH;
  p.tokens = s.tokens; p.heads = heads; p.head_dim = d; p.rotary_rows = s.rotary_rows;
  p.dblocks = plan.dblocks; p.group_heads = group; p.slices = (s.tokens + 15) / 16;

  const long total = (long)p.slices * group * plan.dblocks;
  long ctas = sm_count() / ((long)s.batch * groups);
  if (ctas < 1) ctas = 1;
  const long need = (total + WARPS * 6 - 1) / (WARPS * 6);   // at least ~6 items per warp
  if (ctas > need) ctas = need < 1 ? 1 : need;
  dim3 grid((unsigned)ctas, s.batch, groups);
  const int smem_bytes = fixed + group * per_head;
  const bool rot = s.rotary_rows > 0;
  if (rot) {
    auto kern = readout_tma_kernel<R, true, Cfg>;
    if (ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem_bytes)) return MS_ERR_LAUNCH;
    launch_kernel(kern, grid, dim3(WARPS * 32), smem_bytes, st, map_a, map_c, map_w, map_y, p);
  } else {
    auto kern = readout_tma_kernel<R, false, Cfg>;
    if (ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem_bytes)) return MS_ERR_LAUNCH;
    launch_kernel(kern, grid, dim3(WARPS * 32), smem_bytes, st, map_a, map_c, map_w, map_y, p);
  }
  return cudaGetLastError() == cudaSuccess ? MS_OK : MS_ERR_LAUNCH;
}

template <int R>
static int launch_readout_tma_r(const ms_shape& s, const Plan& plan, const void* projected, const float* cos,
                                const float* sin, const float* counts, const ms_tape& t, void* mixed,
                                cudaStream_t st) {
  // sixteen warps hide the fixed latencies of the epilogue; rank 64 keeps eight (its coefficient
  // matrices take twice the shared memory)
  if (R == 64)
    return launch_readout_tma_cfg<R, ReadoutTmaCfg<R, 8, 3, 1>>(s, plan, projected, cos, sin, counts, t, mixed, st);
  return launch_readout_tma_cfg<R, ReadoutTmaCfg<R, 16, 3, 1>>(s, plan, projected, cos, sin, counts, t, mixed, st);
}

// Returns MS_OK / an error, or -1 when the shape is outside this kernel's envelope (the caller
// then uses the generic kernel).
int launch_readout_tma(const ms_shape& s, const Plan& plan, const void* projected, const float* cos,
                       const float* sin, const float* counts, const ms_tape& t, void* mixed, cudaStream_t st) {
  if (!plan.aligned || (s.head_dim % 64) != 0) return -1;
  if ((reinterpret_cast<uintptr_t>(t.coeff) & 15u) != 0) return -1;
  switch (s.rank) {
    case 16: return launch_readout_tma_r<16>(s, plan, projected, cos, sin, counts, t, mixed, st);
    case 32: return launch_readout_tma_r<32>(s, plan, projected, cos, sin, counts, t, mixed, st);
    case 64: return launch_readout_tma_r<64>(s, plan, projected, cos, sin, counts, t, mixed, st);
  }
  return -1;
}

}  // namespace ms
