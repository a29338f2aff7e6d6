// Register-fragment helpers shared by the token-parallel kernels (mma.sync.m16n8k16 layouts).
// A warp owns 16 token rows; "row operand" fragments hold (row g | g+8, channel pair) per
// thread, which is also the accumulator layout, so the rotary rotation of adjacent channel
// pairs is thread-local.
#pragma once

#include "ms_common.cuh"

namespace ms {

// rotary entries for the accumulator / row-operand fragment of one warp:
// n-tile j (8 channels) -> pair 4j + (lane&3); rows lane>>2 and lane>>2 + 8
struct TableFrag {
  float c[8][2];
  float s[8][2];
};

__device__ __forceinline__ void load_table_frag(TableFrag& f, const float* __restrict__ cos,
                                                const float* __restrict__ sin, long row0, int rows_left,
                                                int half, int pair0, int pairs_valid, int lane) {
  const int g = lane >> 2, tq = lane & 3;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int pr = 4 * j + tq;
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int row = g + 8 * k;
      float cv = 1.f, sv = 0.f;
      if (row < rows_left && pr < pairs_valid) {
        cv = __ldg(cos + (row0 + row) * half + pair0 + pr);
        sv = __ldg(sin + (row0 + row) * half + pair0 + pr);
      }
      f.c[j][k] = cv;
      f.s[j][k] = sv;
    }
  }
}

// acc[n] += X * B^T for a 16 x 64 row operand held as fragments xf[4] and a matrix stored
// [R rows = output columns][64 = contraction] (pitch 128 bytes, 128-byte swizzle)
template <int R>
__device__ __forceinline__ void mma_rows_by_stored_nk(float (&acc)[R / 8][4], const uint32_t (&xf)[4][4],
                                                      uint32_t tile, int lane) {
  const int mi = lane >> 3, mr = lane & 7;
#pragma unroll
  for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
    for (int n2 = 0; n2 < R / 16; ++n2) {
      uint32_t bf[4];
      ldsm_x4(bf, tile + swz((n2 * 16 + mr + 8 * (mi >> 1)) * 128 + (ks * 16 + 8 * (mi & 1)) * 2));
      mma_bf16(acc[2 * n2], xf[ks], bf[0], bf[1]);
      mma_bf16(acc[2 * n2 + 1], xf[ks], bf[2], bf[3]);
    }
  }
}

// load the 16 x 64 row operand of a warp (4 k-steps) from a 128-byte-pitch tile; `warp`
// selects the 16-row band inside the tile
__device__ __forceinline__ void load_row_frags(uint32_t (&xf)[4][4], uint32_t tile, int warp, int lane) {
  const int mi = lane >> 3, mr = lane & 7;
#pragma unroll
  for (int ks = 0; ks < 4; ++ks)
    ldsm_x4(xf[ks], tile + swz((warp * 16 + mr + 8 * (mi & 1)) * 128 + (ks * 16 + 8 * (mi >> 1)) * 2));
}

// rotate a row operand in registers and split it into two BF16 words
__device__ __forceinline__ void rotate_split(const uint32_t (&raw)[4][4], const TableFrag& tab,
                                             uint32_t (&hi)[4][4], uint32_t (&lo)[4][4]) {
#pragma unroll
  for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int j = 2 * ks + (q >> 1), k = q & 1;   // q: (row g|g+8) x (cols 0-7 | 8-15)
      const float2 v = bf2_to_f2(raw[ks][q]);
      const float2 r = rot_pair(v.x, v.y, tab.c[j][k], tab.s[j][k]);
      split2(r.x, r.y, hi[ks][q], lo[ks][q]);
    }
  }
}

}  // namespace ms
