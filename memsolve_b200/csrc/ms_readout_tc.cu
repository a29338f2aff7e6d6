// Readout  Y = eta*C + rot^-1(A_raw W)/sqrt(n)  on the fifth-generation tensor cores (tcgen05), for long
// sequences: head dimension 64, rank 16/32/64, aligned pointers, at least kRoMinTokens tokens per sample
// (other shapes take the mma.sync kernels in ms_readout_tma.cu / ms_token.cu).  Same arithmetic as those
// kernels (the reference's `_readout`, memsolve/ball/cuda.py:1670-1764): W carried as two BF16 words, both
// products accumulated in FP32, inverse rotation and the eta*C term in FP32, one BF16 rounding.
//
// Work item = (128-token tile, head).  A CTA serves one sample and one group of heads whose coefficient
// matrices stay in shared memory (all twelve heads at rank 32), and walks over its items:
//
//   warp 16 (one thread)  TMA: content boxes in, and the finished rows -- which the compute warps write over
//                         the content box -- out to `mixed`.
//   warp 19 (one thread)  TMA: relation boxes, a ring of their own (free again once the MMAs have read them).
//   warp 18 (one thread)  TMA: the cos / sin rows of the next token tile.
//   warp 17               issues the tcgen05 MMAs (A W_low + A W_high, 128 x 64 FP32 accumulator in tensor
//                         memory, two accumulators in flight).
//   warps 0-7 / 8-15      one group per accumulator, half a token row per thread: read the accumulator, apply
//                         the inverse rotation and eta*C, write BF16.
//
// Every wait is bounded; after a timeout the error word is set and the CTA drains.
#include "ms_tc.cuh"

namespace ms {

constexpr int kRoComputeWarps = 16;
constexpr int kRoThreads = (kRoComputeWarps + 4) * 32;
constexpr int kRoGroupThreads = 256;
constexpr int kRoTile = 128;
constexpr int kRoMinTokens = 512;

template <int R>
struct ReadoutTcCfg {
  static constexpr int A_ROW = R * 2;
  static constexpr int A_TILE = kRoTile * A_ROW;
  static constexpr int C_TILE = 16384;
  static constexpr int C_STAGES = 4;
  static constexpr int A_STAGES = 3;
  static constexpr int TABLE_BYTES = 32768;
  static constexpr int W_BYTES = R * 128;
  static constexpr int HEAD_BYTES = 2 * W_BYTES;   // W high / low
  static constexpr int BAR_BYTES = (2 * C_STAGES + 2 * A_STAGES + 8) * 8 + 16;
  static constexpr int RING_BYTES = C_STAGES * C_TILE + A_STAGES * A_TILE;
  static constexpr int MAX_SMEM = 227 * 1024;
  static constexpr int RESIDENT_BUDGET = MAX_SMEM - 1024 - RING_BYTES - TABLE_BYTES - BAR_BYTES;
  static constexpr int SLOT_COLS = 64, TMEM_COLS = 128;
};

struct ReadoutTcParams {
  const float* counts;
  const float* eta;
  float* debug;   // optional FP32 copy of `mixed` before the BF16 rounding ([B, N, H*64]), or null
  int* error;
  int tokens, heads, rotary_rows, group_heads, tiles, work_ctas;
};

__device__ __forceinline__ void ro_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool ro_wait(uint32_t bar, uint32_t parity) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity));
}

template <int R, bool ROT, bool DEBUG>
__global__ void __launch_bounds__(kRoThreads, 1)
readout_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_c,
                  const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_y,
                  const __grid_constant__ CUtensorMap map_cos, const __grid_constant__ CUtensorMap map_sin,
                  const ReadoutTcParams p) {
  using Cfg = ReadoutTcCfg<R>;
  constexpr int SC = Cfg::C_STAGES, SA = Cfg::A_STAGES;
  constexpr int kContentWarp = kRoComputeWarps, kMmaWarp = kRoComputeWarps + 1, kTableWarp = kRoComputeWarps + 2,
                kRelationWarp = kRoComputeWarps + 3;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t smem = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  grid_launch_dependents();

  const int b = blockIdx.y;
  const int h0 = blockIdx.z * p.group_heads;
  const int gh = min(p.group_heads, p.heads - h0);
  const uint32_t res_base = smem;
  const uint32_t c_ring = smem + p.group_heads * Cfg::HEAD_BYTES;
  const uint32_t a_ring = c_ring + SC * Cfg::C_TILE;
  const uint32_t tab_buf = a_ring + SA * Cfg::A_TILE;
  const uint32_t bar_cfull = tab_buf + Cfg::TABLE_BYTES;
  const uint32_t bar_out = bar_cfull + 8 * SC;
  const uint32_t bar_afull = bar_out + 8 * SC;
  const uint32_t bar_afree = bar_afull + 8 * SA;
  const uint32_t bar_m = bar_afree + 8 * SA;        // accumulator complete, per slot
  const uint32_t bar_free = bar_m + 16;             // accumulator read, per slot
  const uint32_t bar_res = bar_free + 16;
  const uint32_t bar_tab_full = bar_res + 8, bar_tab_free = bar_tab_full + 8;
  const uint32_t tslot = bar_tab_free + 8;

  if (tid == 0) {
    for (int i = 0; i < SC; ++i) {
      mbar_init(bar_cfull + 8 * i, 1);
      mbar_init(bar_out + 8 * i, kRoGroupThreads);
    }
    for (int i = 0; i < SA; ++i) {
      mbar_init(bar_afull + 8 * i, 1);
      mbar_init(bar_afree + 8 * i, kRoGroupThreads);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_m + 8 * i, 1);
      mbar_init(bar_free + 8 * i, kRoGroupThreads);
    }
    mbar_init(bar_res, 1);
    mbar_init(bar_tab_full, 1);
    mbar_init(bar_tab_free, 2 * kRoGroupThreads);
    mbar_fence_init();
  }
  __syncthreads();
  if (warp == kMmaWarp) tc::tmem_alloc(tslot, Cfg::TMEM_COLS);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = ld_shared_u32(tslot);

  const int total = p.tiles * gh;
  const int per = (total + p.work_ctas - 1) / p.work_ctas;
  const int it0 = min(total, (int)blockIdx.x * per);
  const int n_items = min(total, it0 + per) - it0;
  const int tile0 = it0 / gh;
  const int n_tiles = n_items > 0 ? (it0 + n_items - 1) / gh - tile0 + 1 : 0;
  bool ok = true;

  if (warp == kContentWarp) {
    // ---------------------------------------------------------------- content boxes in, finished rows out
    if (lane == 0) {
      auto issue_load = [&](int i) {
        const int idx = it0 + i, tile = idx / gh, h = h0 + (idx - tile * gh);
        const uint32_t bar = bar_cfull + 8 * (i % SC);
        mbar_expect_tx(bar, Cfg::C_TILE);
        tma_load_3d(c_ring + (i % SC) * Cfg::C_TILE, &map_c, p.heads * R + h * 64, tile * kRoTile, b, bar);
      };
      // `projected` was complete before the kernel ahead of this one started (that kernel only forms the
      // coefficients), so a chained launch may fetch token boxes before the dependency wait
      for (int k = 0; k < SC && k < n_items; ++k) issue_load(k);
      grid_dependency_wait();
      mbar_expect_tx(bar_res, (uint32_t)(gh * Cfg::HEAD_BYTES));
      for (int hl = 0; hl < gh; ++hl) {
        const int sys = b * p.heads + h0 + hl;
        const uint32_t hb = res_base + hl * Cfg::HEAD_BYTES;
        tma_load_2d(hb, &map_w, 0, (sys * 2) * R, bar_res);
        tma_load_2d(hb + Cfg::W_BYTES, &map_w, 0, (sys * 2 + 1) * R, bar_res);
      }
      for (int i = 0; i < n_items; ++i) {
        ok = mbar_wait(bar_out + 8 * (i % SC), (i / SC) & 1);
        if (!ok) break;
        const int idx = it0 + i, tile = idx / gh, h = h0 + (idx - tile * gh);
        tma_store_3d(&map_y, h * 64, tile * kRoTile, b, c_ring + (i % SC) * Cfg::C_TILE);
        tma_store_commit();
        if (i + SC < n_items) {
          tma_store_wait_read<0>();
          issue_load(i + SC);
        }
      }
      tma_store_wait_all<0>();
      if (!ok) atomicExch(p.error, kErrBarrierTimeout);
    }
  } else if (warp == kRelationWarp) {
    // ---------------------------------------------------------------- relation boxes
    if (lane == 0) {
      for (int j = 0; j < n_items; ++j) {
        if (j >= SA) {
          ok = mbar_wait(bar_afree + 8 * (j % SA), ((j / SA) - 1) & 1);
          if (!ok) break;
        }
        const int idx = it0 + j, tile = idx / gh, h = h0 + (idx - tile * gh);
        mbar_expect_tx(bar_afull + 8 * (j % SA), Cfg::A_TILE);
        tma_load_3d(a_ring + (j % SA) * Cfg::A_TILE, &map_a, h * R, tile * kRoTile, b, bar_afull + 8 * (j % SA));
      }
      if (!ok) atomicExch(p.error, kErrBarrierTimeout);
    }
  } else if (warp == kTableWarp) {
    // ---------------------------------------------------------------- table producer
    if (ROT && lane == 0) {
      const int tab_b = p.rotary_rows > 1 ? b : 0;
      for (int k = 0; k < n_tiles; ++k) {
        if (k > 0) {
          ok = mbar_wait(bar_tab_free, (k - 1) & 1);
          if (!ok) break;
        }
        mbar_expect_tx(bar_tab_full, Cfg::TABLE_BYTES);
        tma_load_3d(tab_buf, &map_cos, 0, (tile0 + k) * kRoTile, tab_b, bar_tab_full);
        tma_load_3d(tab_buf + 16384, &map_sin, 0, (tile0 + k) * kRoTile, tab_b, bar_tab_full);
      }
      if (!ok) atomicExch(p.error, kErrBarrierTimeout);
    }
  } else if (warp == kMmaWarp) {
    // ---------------------------------------------------------------- MMA issuer (whole warp, uniform control flow)
    constexpr uint32_t IDESC = tc::idesc_bf16(128, 64, true);   // B = W stored [r][64]
    constexpr uint32_t HI_A = tc::desc_hi_k_major(Cfg::A_ROW), HI_N = tc::desc_hi_n_major_128();
    constexpr uint32_t N_MAJOR_LBO = ((1024u >> 4) - 1u) << 16;
    grid_dependency_wait();
    ok = ro_wait(bar_res, 0);
    const uint32_t res_lo = tc::desc_lo_k_major(res_base) + N_MAJOR_LBO;
    const uint32_t aring_lo = tc::desc_lo_k_major(a_ring);
    for (int i = 0; i < n_items && ok; ++i) {
      const int slot = i & 1;
      ok = ro_wait(bar_afull + 8 * (i % SA), (i / SA) & 1);
      if (ok && i >= 2) ok = ro_wait(bar_free + 8 * slot, ((i >> 1) - 1) & 1);
      if (!ok) break;
      tc::fence_after_sync();
      const int idx = it0 + i, tile = idx / gh;
      const uint32_t a_lo = aring_lo + (uint32_t)((i % SA) * (Cfg::A_TILE >> 4));
      const uint32_t wh = res_lo + (uint32_t)((idx - tile * gh) * (Cfg::HEAD_BYTES >> 4)), wl = wh + (Cfg::W_BYTES >> 4);
      const uint32_t tb = tmem + slot * Cfg::SLOT_COLS;
      if (tc::elect_one()) {
#pragma unroll
        for (int word = 0; word < 2; ++word) {
#pragma unroll
          for (int ks = 0; ks < R / 16; ++ks)
            tc::mma_ss_raw<HI_A, HI_N, IDESC>(tb, a_lo + ks * 2, (word == 0 ? wl : wh) + ks * 128, (word | ks) != 0);
        }
        tc::mma_commit_raw(bar_m + 8 * slot);
      }
      __syncwarp();
    }
    if (!ok && lane == 0) atomicExch(p.error, kErrBarrierTimeout);
  } else {
    // ---------------------------------------------------------------- compute warps
    const int g = warp >> 3, q = warp & 3, half = (warp >> 2) & 1, row = q * 32 + lane;
    const uint32_t lane_base = tmem + ((uint32_t)(q * 32) << 16) + g * Cfg::SLOT_COLS;
    grid_dependency_wait();
    const float n = p.counts ? p.counts[b] : (float)p.tokens;
    const float inv_s = inv_sqrt_rn(n);
    const int dmodel = p.heads * 64;
    float cs[16], sn[16];
    int tab_next = 0;
    bool owe_table = false;   // this thread holds the rows of a tile and has not yet released the buffer
    auto take_tables = [&](int k) {
      bool good = true;
      while (tab_next <= k && good) {
        good = ro_wait(bar_tab_full, tab_next & 1);
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
          // A tile whose rows were copied is handed back only after they have been USED (in the epilogue below):
          // ld.shared merely issues the reads, and an arrive right behind it can let the next bulk copy land first.
          if (tab_next == k) owe_table = true;
          else ro_arrive(bar_tab_free);
        }
        ++tab_next;
      }
      return good;
    };

    for (int i = g; i < n_items && ok; i += 2) {
      const int idx = it0 + i, tile = idx / gh, h = h0 + (idx - tile * gh);
      const uint32_t c_tile = c_ring + (i % SC) * Cfg::C_TILE;
      const int tok = tile * kRoTile + row;
      const bool valid = tok < p.tokens;
      const float eta = __ldg(p.eta + h);
      if (ROT && tile - tile0 >= tab_next) {
        ok = take_tables(tile - tile0);
        if (!ok) break;
      }
      ok = ro_wait(bar_m + 8 * g, (i >> 1) & 1);
      if (!ok) break;
      tc::fence_after_sync();
      ro_arrive(bar_afree + 8 * (i % SA));   // the MMAs that read the relation box have completed
      uint32_t acc[32];
      tc::tmem_ld16(lane_base + half * 32, *reinterpret_cast<uint32_t(*)[16]>(&acc[0]));
      tc::tmem_ld16(lane_base + half * 32 + 16, *reinterpret_cast<uint32_t(*)[16]>(&acc[16]));
      ok = ro_wait(bar_cfull + 8 * (i % SC), (i / SC) & 1);
      if (!ok) break;
      tc::wait_ld();
      tc::fence_before_sync();
      ro_arrive(bar_free + 8 * g);            // the accumulator is in registers
      float* dbg = (DEBUG && valid) ? p.debug + ((size_t)b * p.tokens + tok) * dmodel + h * 64 + half * 32 : nullptr;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint32_t addr = c_tile + row * 128 + (((half * 4 + c) ^ (row & 7)) << 4);
        const uint4 cv = ld_shared_v4(addr);
        const uint32_t cw[4] = {cv.x, cv.y, cv.z, cv.w};
        uint32_t ow[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int j = c * 4 + k;
          float2 corr = make_float2(__uint_as_float(acc[2 * j]), __uint_as_float(acc[2 * j + 1]));
          if (ROT) corr = rot_pair(corr.x, corr.y, cs[j], -sn[j]);
          const float2 cc = bf2_to_f2(cw[k]);
          const float o0 = fmaf(corr.x, inv_s, eta * cc.x), o1 = fmaf(corr.y, inv_s, eta * cc.y);
          ow[k] = f2_to_bf2(o0, o1);
          if (DEBUG && dbg) {
            dbg[2 * j] = o0;
            dbg[2 * j + 1] = o1;
          }
        }
        st_shared_v4(addr, make_uint4(ow[0], ow[1], ow[2], ow[3]));
      }
      if (ROT && owe_table) {   // every cos / sin register has been consumed by an instruction issued above
        ro_arrive(bar_tab_free);
        owe_table = false;
      }
      fence_async_shared();
      ro_arrive(bar_out + 8 * (i % SC));
    }
    while (ROT && ok && tab_next < n_tiles) {
      ok = ro_wait(bar_tab_full, tab_next & 1);
      if (ok) ro_arrive(bar_tab_free);
      ++tab_next;
    }
    if (!ok && lane == 0) atomicExch(p.error, kErrBarrierTimeout);
  }

  tc::fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarp) tc::tmem_free(tmem, Cfg::TMEM_COLS);
}

template <int R>
static int launch_readout_tc_r(const ms_shape& s, const Plan& plan, const void* projected, const float* cos,
                               const float* sin, const float* counts, const ms_tape& t, void* mixed, float* debug,
                               cudaStream_t st) {
  using Cfg = ReadoutTcCfg<R>;
  const int heads = s.heads, width = heads * (R + 64), dmodel = heads * 64;
  int group = Cfg::RESIDENT_BUDGET / Cfg::HEAD_BYTES;
  if (group < 1) return -1;
  if (group > heads) group = heads;
  const int groups = (heads + group - 1) / group;
  group = (heads + groups - 1) / groups;

  CUtensorMap map_a, map_c, map_w, map_y;
  {
    const uint64_t dims[3] = {(uint64_t)width, (uint64_t)s.tokens, (uint64_t)s.batch};
    const uint64_t str[2] = {(uint64_t)width * 2, (uint64_t)s.tokens * width * 2};
    const uint32_t box_a[3] = {(uint32_t)R, kRoTile, 1};
    const uint32_t box_c[3] = {64, kRoTile, 1};
    if (encode_tensor_map(&map_a, const_cast<void*>(projected), 2, 3, dims, str, box_a, swizzle_for_rows<R * 2>())) return MS_ERR_LAUNCH;
    if (encode_tensor_map(&map_c, const_cast<void*>(projected), 2, 3, dims, str, box_c, Swizzle::B128)) return MS_ERR_LAUNCH;
  }
  {
    const uint64_t dims[3] = {(uint64_t)dmodel, (uint64_t)s.tokens, (uint64_t)s.batch};
    const uint64_t str[2] = {(uint64_t)dmodel * 2, (uint64_t)s.tokens * dmodel * 2};
    const uint32_t box[3] = {64, kRoTile, 1};
    if (encode_tensor_map(&map_y, mixed, 2, 3, dims, str, box, Swizzle::B128)) return MS_ERR_LAUNCH;
  }
  {
    const uint64_t dims[2] = {64, (uint64_t)plan.systems * 2 * R};
    const uint64_t str[1] = {128};
    const uint32_t box[2] = {64, (uint32_t)R};
    if (encode_tensor_map(&map_w, t.coeff, 2, 2, dims, str, box, Swizzle::B128)) return MS_ERR_LAUNCH;
  }
  CUtensorMap map_cos = map_a, map_sin = map_a;   // placeholders when there is no rotation
  if (s.rotary_rows > 0) {
    const uint64_t dims[3] = {32, (uint64_t)s.tokens, (uint64_t)s.rotary_rows};
    const uint64_t str[2] = {128, (uint64_t)s.tokens * 128};
    const uint32_t box[3] = {32, kRoTile, 1};
    if (encode_tensor_map(&map_cos, const_cast<float*>(cos), 4, 3, dims, str, box, Swizzle::B128)) return MS_ERR_LAUNCH;
    if (encode_tensor_map(&map_sin, const_cast<float*>(sin), 4, 3, dims, str, box, Swizzle::B128)) return MS_ERR_LAUNCH;
  }

  ReadoutTcParams p;
  p.counts = counts; p.eta = t.eta; p.debug = debug;
  p.error = device_error_word();
  if (!p.error) return MS_ERR_LAUNCH;
  p.tokens = s.tokens; p.heads = heads; p.rotary_rows = s.rotary_rows; p.group_heads = group;
  p.tiles = (s.tokens + kRoTile - 1) / kRoTile;
  const long total = (long)p.tiles * group;
  long ctas = sm_count() / ((long)s.batch * groups);
  if (ctas < 1) ctas = 1;
  const long need = (total + 3) / 4;
  if (ctas > need) ctas = need < 1 ? 1 : need;
  p.work_ctas = (int)ctas;
  dim3 grid((unsigned)ctas, s.batch, groups);
  const int smem_bytes = 1024 + group * Cfg::HEAD_BYTES + Cfg::RING_BYTES + Cfg::TABLE_BYTES + Cfg::BAR_BYTES;
  void (*kern)(CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, ReadoutTcParams);
  if (s.rotary_rows > 0) kern = debug ? readout_tc_kernel<R, true, true> : readout_tc_kernel<R, true, false>;
  else kern = debug ? readout_tc_kernel<R, false, true> : readout_tc_kernel<R, false, false>;
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem_bytes)) return MS_ERR_LAUNCH;
  launch_kernel(kern, grid, dim3(kRoThreads), smem_bytes, st, map_a, map_c, map_w, map_y, map_cos, map_sin, p);
  return cudaGetLastError() == cudaSuccess ? MS_OK : MS_ERR_LAUNCH;
}

// MS_OK / error, or -1 when the shape is outside this kernel's envelope.  `debug` (FP32 [B, N, H*64], or null)
// receives the values before the BF16 rounding; with `debug` set shapes below kRoMinTokens are taken too.
int launch_readout_tc(const ms_shape& s, const Plan& plan, const void* projected, const float* cos, const float* sin,
                      const float* counts, const ms_tape& t, void* mixed, float* debug, cudaStream_t st) {
  if (!plan.aligned || s.head_dim != 64) return -1;
  if (s.tokens < kRoMinTokens && !debug) return -1;
  if (s.batch > 65535) return -1;
  if ((reinterpret_cast<uintptr_t>(t.coeff) & 15u) != 0) return -1;
  switch (s.rank) {
    case 16: return launch_readout_tc_r<16>(s, plan, projected, cos, sin, counts, t, mixed, debug, st);
    case 32: return launch_readout_tc_r<32>(s, plan, projected, cos, sin, counts, t, mixed, debug, st);
    case 64: return launch_readout_tc_r<64>(s, plan, projected, cos, sin, counts, t, mixed, debug, st);
  }
  return -1;
}

}  // namespace ms
