// Rank-space (r x r and r x d) stages of the MemSolve mixer, forward and adjoint.
//
//   compact_forward   per (b,h):  G,Q (sum of partials) -> T = chol(I+G)^-1, Z = T Q,
//                                 W = T^T (F - eta I) Z  (written as two BF16 words)
//   compact_backward  per (b,h):  U = T E, H = U Z^T, dQ = T^T M^T U,
//                                 dG = T^T symlow(-M H^T - M^T H) T
//   core_forward / core_backward kernels: one CTA per head around the device functions of
//                                 ms_core.cuh (also run from spare CTAs of the streaming kernels)
//
// Replaces the reference's native Cholesky-inverse (csrc/ball/solvers.cuh:34-217) and its
// Triton compact kernels (memsolve/ball/cuda.py:2530-2768).  These kernels run on one CTA per
// (sample, head) and are bound by latency, not by throughput, so each stage is shaped for a
// short dependency chain: the partial sums of the token reductions are fetched with bulk
// asynchronous copies into shared memory while the per-head matrices are set up and are then
// added in chunk order (order-deterministic); the Cholesky factor is computed by the whole
// CTA (FP32, the diagonal carried in FP64, like the reference's native kernel) with one
// barrier per elimination step; the r x d and r x r products are FP32 FMA on 4 x 2 register
// tiles with vector loads from shared memory.
#include "ms_core.cuh"
#include "ms_tma.cuh"

namespace ms {

constexpr int kCompactThreads = 256;
constexpr int kQP = 68;   // pitch in floats of the r x 64 blocks: rows 16-byte aligned, 4-bank skew

// Threads per CTA of the compact kernels: rank 64 takes 512 (its 64 x 64 products and the 64 elimination steps are
// what a sequence-parallel step waits for on every rank; twice the threads halve the work per thread and step).
// Rank 32 does the same when few systems are in flight (one resident CTA per SM; the four-CTA variant for many
// systems keeps 256 threads for its register budget).
template <int R, int MINB = 1>
constexpr int compact_threads() { return (R == 64 || (R == 32 && MINB == 1)) ? 512 : kCompactThreads; }

template <int R, int MINB = 1>
struct CompactDims {
  static constexpr int NT = compact_threads<R, MINB>();
  // threads per matrix row in the factorisation
  static constexpr int TPR = R <= 16 ? 16 : (R == 32 ? (NT == 512 ? 16 : 8) : (R == 64 ? 8 : 4));
  static constexpr int CPT = R / TPR;                            // columns per thread
  static constexpr int RP = R + 4;                               // pitch in floats of the r x r matrices
  static_assert(R * TPR <= NT && CPT * TPR == R, "factorisation layout");
};

// ---------------------------------------------------------------------------------------
// Cholesky inverse factor with the whole CTA
// ---------------------------------------------------------------------------------------
// gs: G (FP32, pitch R).  Writes T = chol(I + sym(G))^-1 (lower triangular, FP32) to ts (row
// major, pitch RP) and its transpose to tT.  Gaussian elimination applies the unit-lower factor
// to the identity in place; a final row scaling by the inverse square roots of the pivots turns
// it into the Cholesky inverse.  The bulk is FP32; each row's diagonal entry (its future pivot)
// is carried in FP64, as the reference's native Cholesky does.
// Row i lives in the registers of TPR neighbouring threads (columns q, q+TPR, ...).  Per step
// the owners of the pivot row and of the pivot column publish them (double buffered) and one
// CTA barrier separates the steps, so a step costs one barrier, a handful of shared-memory
// reads and CPT FMAs per thread instead of a whole row per lane.
template <int R, int MINB>
__device__ __forceinline__ void cholesky_inverse_cta(const float* gs, float* ts, float* tT, float* rowbuf,
                                                     float* colbuf, double* dscale, int tid) {
  using D = CompactDims<R, MINB>;
  constexpr int TPR = D::TPR, CPT = D::CPT, RP = D::RP;
  const int i = tid / TPR, q = tid % TPR;
  const bool active = i < R;
  const bool diag_owner = active && (i % TPR) == q;
  float a[CPT];
#pragma unroll
  for (int c = 0; c < CPT; ++c) {
    const int j = q + TPR * c;
    a[c] = active ? 0.5f * (gs[i * R + j] + gs[j * R + i]) + (i == j ? 1.0f : 0.0f) : 0.f;
  }
  double diag = diag_owner ? 1.0 + (double)gs[i * R + i] : 1.0;

  // publish row k and, from the register `colv` of its owners, column k (below the diagonal) as
  // they stand after the steps before k
  auto publish = [&](int k, int buf, float colv) {
    if (!active) return;
    if (i == k) {
#pragma unroll
      for (int c = 0; c < CPT; ++c) rowbuf[buf * (R + 1) + q + TPR * c] = a[c];
      if (diag_owner) {
        // reciprocal of the pivot: hardware approximation plus one FP32 Newton step (this value sits
        // on the dependency chain of every step, the FP64 diagonal keeps the pivot itself accurate)
        const float df = (float)diag;
        float r0;
        asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r0) : "f"(df));
        rowbuf[buf * (R + 1) + R] = fmaf(r0, fmaf(-df, r0, 1.0f), r0);
      }
    }
    if (i > k && q == k % TPR) colbuf[buf * R + i] = colv;
  };
  publish(0, 0, a[0]);
  // step K = cK * TPR + qK; the outer index is unrolled so that every register index is a constant
#pragma unroll
  for (int cK = 0; cK < CPT; ++cK) {
    for (int qK = 0; qK < TPR; ++qK) {
      const int K = cK * TPR + qK;
      __syncthreads();
      const int buf = K & 1;
      if (active && i > K) {
        const float* rb = rowbuf + buf * (R + 1);
        const float f = colbuf[buf * R + i] * rb[R];
        if (diag_owner) diag = fma(-(double)f, (double)rb[i], diag);
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
          const float upd = fmaf(-f, rb[q + TPR * c], a[c]);
          a[c] = (c == cK && q == qK) ? -f : upd;
        }
      }
      if (K + 1 < R) publish(K + 1, buf ^ 1, (qK + 1 < TPR) ? a[cK] : a[cK + 1 < CPT ? cK + 1 : cK]);
    }
  }
  if (diag_owner) dscale[i] = rsqrt(diag);
  __syncthreads();
  if (active) {
    const double sc = dscale[i];
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
      const int j = q + TPR * c;
      float v = 0.f;
      if (j < i) v = (float)((double)a[c] * sc);
      else if (j == i) v = (float)sc;
      ts[i * RP + j] = v;
      tT[j * RP + i] = v;
    }
  }
}

// ---------------------------------------------------------------------------------------
// small FP32 products on shared-memory operands, 4 x 2 register tiles
// ---------------------------------------------------------------------------------------
// acc[r][c] += sum_{k0 <= k < k1} At[k][i0 + r] * B[k][j0 + c]      (both operands k-major)
__device__ __forceinline__ void mm_tn(float (&acc)[4][2], const float* At, int lda, const float* B, int ldb,
                                      int i0, int j0, int k0, int k1) {
#pragma unroll 4
  for (int k = k0; k < k1; ++k) {
    const float4 a = *reinterpret_cast<const float4*>(At + k * lda + i0);
    const float2 b = *reinterpret_cast<const float2*>(B + k * ldb + j0);
    acc[0][0] = fmaf(a.x, b.x, acc[0][0]); acc[0][1] = fmaf(a.x, b.y, acc[0][1]);
    acc[1][0] = fmaf(a.y, b.x, acc[1][0]); acc[1][1] = fmaf(a.y, b.y, acc[1][1]);
    acc[2][0] = fmaf(a.z, b.x, acc[2][0]); acc[2][1] = fmaf(a.z, b.y, acc[2][1]);
    acc[3][0] = fmaf(a.w, b.x, acc[3][0]); acc[3][1] = fmaf(a.w, b.y, acc[3][1]);
  }
}

// acc[r][c] += sum_{k < K} X[i0 + r][k] * Y[j(c)][k],  j(0) = j0, j(1) = j1   (both operands row-major)
template <int K>
__device__ __forceinline__ void mm_nt(float (&acc)[4][2], const float* X, int ldx, const float* Y, int ldy,
                                      int i0, int j0, int j1) {
#pragma unroll 2
  for (int k = 0; k < K; k += 4) {
    float4 x[4], y[2];
#pragma unroll
    for (int r = 0; r < 4; ++r) x[r] = *reinterpret_cast<const float4*>(X + (i0 + r) * ldx + k);
    y[0] = *reinterpret_cast<const float4*>(Y + j0 * ldy + k);
    y[1] = *reinterpret_cast<const float4*>(Y + j1 * ldy + k);
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        acc[r][c] = fmaf(x[r].x, y[c].x, acc[r][c]);
        acc[r][c] = fmaf(x[r].y, y[c].y, acc[r][c]);
        acc[r][c] = fmaf(x[r].z, y[c].z, acc[r][c]);
        acc[r][c] = fmaf(x[r].w, y[c].w, acc[r][c]);
      }
  }
}

__device__ __forceinline__ void zero_tile(float (&acc)[4][2]) {
#pragma unroll
  for (int r = 0; r < 4; ++r) acc[r][0] = acc[r][1] = 0.f;
}

// two adjacent values as (dominant, residual) BF16 words
__device__ __forceinline__ void store_split2(__nv_bfloat16* hi, __nv_bfloat16* lo, size_t idx, float v0, float v1) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(v0, v1);
  *reinterpret_cast<__nv_bfloat162*>(hi + idx) = h;
  *reinterpret_cast<__nv_bfloat162*>(lo + idx) =
      __floats2bfloat162_rn(v0 - __low2float(h), v1 - __high2float(h));
}
__device__ __forceinline__ void store_split(__nv_bfloat16* hi, __nv_bfloat16* lo, size_t idx, float v) {
  const __nv_bfloat16 hv = __float2bfloat16_rn(v);
  hi[idx] = hv;
  lo[idx] = __float2bfloat16_rn(v - __bfloat162float(hv));
}

// ---------------------------------------------------------------------------------------
// staging of the partial sums
// ---------------------------------------------------------------------------------------
// One thread copies `chunks` partials of `floats` floats each (contiguous in global memory) into
// shared memory with bulk asynchronous copies on one mbarrier; the CTA then adds them in chunk
// order from shared memory.  The copy needs 16-byte aligned addresses and sizes; the launcher
// checks that and the size, and otherwise the kernel adds the partials straight from global
// memory.
__device__ __forceinline__ void stage_partials(uint32_t dst, const float* src, int chunks, int stride_floats,
                                               int first, int floats, uint32_t bar) {
  mbar_expect_tx(bar, (uint32_t)chunks * (uint32_t)floats * 4u);
  for (int c = 0; c < chunks; ++c) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(dst + ((uint32_t)c * (uint32_t)stride_floats + (uint32_t)first) * 4u),
                   "l"(reinterpret_cast<uint64_t>(src + (size_t)c * stride_floats + first)),
                   "r"((uint32_t)floats * 4u), "r"(bar)
                 : "memory");
  }
}

// acc[e] = sum over chunks, in chunk order, of src[c * stride + off[e]] for four entries at a time
// (independent chains, pointers advanced by the stride); entries with ok[e] false give zero.  DEPTH chunks
// are fetched per round: two from shared memory, eight from global memory, where a round costs a trip to L2
// and a long sequence leaves some twenty chunks per system (the additions keep their chunk order either way).
template <int DEPTH, class T>
__device__ __forceinline__ void sum_chunks4(const T* src, int stride, int nch, const int (&off)[4],
                                            const bool (&ok)[4], float (&acc)[4]) {
  const T* ptr[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    ptr[e] = src + (ok[e] ? off[e] : 0);
    acc[e] = 0.f;
  }
  int c = 0;
  for (; c + DEPTH <= nch; c += DEPTH) {
    float v[DEPTH][4];
#pragma unroll
    for (int k = 0; k < DEPTH; ++k)
#pragma unroll
      for (int e = 0; e < 4; ++e) v[k][e] = ptr[e][(size_t)k * stride];
#pragma unroll
    for (int e = 0; e < 4; ++e) ptr[e] += (size_t)DEPTH * stride;
#pragma unroll
    for (int k = 0; k < DEPTH; ++k)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[e] += v[k][e];
  }
  if (c < nch) {
    float v[DEPTH][4];
#pragma unroll
    for (int k = 0; k < DEPTH; ++k)
#pragma unroll
      for (int e = 0; e < 4; ++e) v[k][e] = c + k < nch ? ptr[e][(size_t)k * stride] : 0.f;
#pragma unroll
    for (int k = 0; k < DEPTH; ++k)
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (c + k < nch) acc[e] += v[k][e];
  }
#pragma unroll
  for (int e = 0; e < 4; ++e) acc[e] = ok[e] ? acc[e] : 0.f;
}

// acc[r][c] += sum_{k0 <= k < k1} At[k][i0 + r] * B[k][j(c)],  j(0) = j0, j(1) = j1
__device__ __forceinline__ void mm_tn_s(float (&acc)[4][2], const float* At, int lda, const float* B, int ldb,
                                        int i0, int j0, int j1, int k0, int k1) {
#pragma unroll 4
  for (int k = k0; k < k1; ++k) {
    const float4 a = *reinterpret_cast<const float4*>(At + k * lda + i0);
    const float b0 = B[k * ldb + j0], b1 = B[k * ldb + j1];
    acc[0][0] = fmaf(a.x, b0, acc[0][0]); acc[0][1] = fmaf(a.x, b1, acc[0][1]);
    acc[1][0] = fmaf(a.y, b0, acc[1][0]); acc[1][1] = fmaf(a.y, b1, acc[1][1]);
    acc[2][0] = fmaf(a.z, b0, acc[2][0]); acc[2][1] = fmaf(a.z, b1, acc[2][1]);
    acc[3][0] = fmaf(a.w, b0, acc[3][0]); acc[3][1] = fmaf(a.w, b1, acc[3][1]);
  }
}

// ---------------------------------------------------------------------------------------
// compact forward per (b,h)
// ---------------------------------------------------------------------------------------
struct CompactFwdParams {
  const float* partials;   // [systems][chunks][pf] or packed [systems][pf] when chunks == 0
  const float* counts;
  const float* eta;
  const float* core_map;
  float* inverse;
  float* state;
  __nv_bfloat16* coeff;
  int* error;
  int heads, tokens, head_dim, dpad, dblocks, chunks, pf, complement;
  int staged;     // the partials of one system fit the staging area and are 16-byte aligned
  int pair_ok;    // the BF16 outputs are 4-byte aligned (paired stores)
};

// floats of shared memory before the staging area
template <int R>
constexpr int compact_fwd_fixed_floats() {
  return R * R + 3 * R * CompactDims<R>::RP + 2 * R * kQP + 2 * (R + 4) + 2 * R + 2 * R + 4;
}

// MINB > 1: register budget for that many resident CTAs per SM (many systems: throughput instead of latency)
template <int R, int MINB = 1>
__global__ void __launch_bounds__(compact_threads<R, MINB>(), MINB)
compact_forward_kernel(const CompactFwdParams p) {
  using D = CompactDims<R, MINB>;
  constexpr int RP = D::RP, NT = D::NT;
  extern __shared__ __align__(16) unsigned char csm[];
  float* gs = reinterpret_cast<float*>(csm);   // R*R      G
  float* ts = gs + R * R;                      // R*RP     T
  float* tT = ts + R * RP;                     // R*RP     T^T
  float* mT = tT + R * RP;                     // R*RP     (F - eta I)^T
  float* qs = mT + R * RP;                     // R*kQP    Q block -> scratch
  float* mid = qs + R * kQP;                   // R*kQP
  float* rowbuf = mid + R * kQP;               // 2*(R+4)  pivot rows (double buffered)
  float* colbuf = rowbuf + 2 * (R + 4);        // 2*R      pivot columns
  double* dscale = reinterpret_cast<double*>(colbuf + 2 * R);   // R
  uint64_t* bar = reinterpret_cast<uint64_t*>(dscale + R);      // 2 words
  float* stage = reinterpret_cast<float*>(bar + 2);             // chunks * pf when staged

  grid_dependency_wait();
  const int tid = threadIdx.x;
  const int sys = blockIdx.x;
  const int b = sys / p.heads, h = sys - b * p.heads;
  const bool packed = p.chunks == 0;
  const int nch = packed ? 1 : p.chunks;
  const float n = p.counts ? p.counts[b] : (float)p.tokens;
  const float inv_n = packed ? 1.f : inv_rn(n);
  const float inv_s = packed ? 1.f : inv_sqrt_rn(n);
  const float* src = p.partials + (size_t)sys * nch * p.pf;
  const float eta = p.eta ? p.eta[h] : 0.f;   // null: the short-sequence path adds the eta term in token space
  const int d = p.head_dim;
  const bool staged = p.staged != 0;

  if (staged) {
    const uint32_t bar_addr = smem_u32(bar);
    if (tid == 0) {
      mbar_init(bar_addr, 1);
      mbar_init(bar_addr + 8, 1);
      mbar_fence_init();
    }
    __syncthreads();
    if (tid == 0) {
      // Gram partials first (their own barrier): the factorisation starts while the moments land
      stage_partials(smem_u32(stage), src, nch, p.pf, 0, R * R, bar_addr);
      stage_partials(smem_u32(stage), src, nch, p.pf, R * R, p.pf - R * R, bar_addr + 8);
    }
  }
  for (int i = tid; i < R * R; i += NT) {
    const int row = i / R, col = i - row * R;
    float f = p.complement ? 0.f : p.core_map[(size_t)h * R * R + i];
    if (row == col) f -= eta;
    mT[col * RP + row] = f;
  }
  bool ok = true;
  if (staged) ok = mbar_wait(smem_u32(bar), 0);
  for (int i0 = tid; i0 < R * R; i0 += 4 * NT) {
    int off[4];
    bool valid[4];
    float acc[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      off[e] = i0 + e * NT;
      valid[e] = off[e] < R * R;
    }
    if (staged) sum_chunks4<2>(stage, p.pf, nch, off, valid, acc);
    else sum_chunks4<(MINB == 1 ? 8 : 1)>(src, p.pf, nch, off, valid, acc);
#pragma unroll
    for (int e = 0; e < 4; ++e)
      if (valid[e]) gs[off[e]] = acc[e] * inv_n;
  }
  __syncthreads();
  cholesky_inverse_cta<R, MINB>(gs, ts, tT, rowbuf, colbuf, dscale, tid);
  __syncthreads();
  grid_launch_dependents();
  for (int i = tid; i < R * R; i += NT) {
    const int row = i / R, col = i - row * R;
    p.inverse[(size_t)sys * R * R + i] = ts[row * RP + col];
  }

  constexpr int TILES = (R / 4) * 32;   // 4 x 2 tiles of an r x 64 block
  for (int jb = 0; jb < p.dblocks; ++jb) {
    const int d0 = jb * 64, dv = min(64, d - d0);
    if (staged && jb == 0) ok = mbar_wait(smem_u32(bar) + 8, 0) && ok;
    for (int i0 = tid; i0 < R * 64; i0 += 4 * NT) {
      int off[4];
      bool valid[4];
      float acc[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = i0 + e * NT, row = i >> 6, c = i & 63;
        valid[e] = c < dv;
        off[e] = R * R + row * d + d0 + (valid[e] ? c : 0);
      }
      if (staged) sum_chunks4<2>(stage, p.pf, nch, off, valid, acc);
      else sum_chunks4<(MINB == 1 ? 8 : 1)>(src, p.pf, nch, off, valid, acc);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = i0 + e * NT;
        qs[(i >> 6) * kQP + (i & 63)] = acc[e] * inv_s;
      }
    }
    __syncthreads();
    // Z = T Q   (T lower triangular: the inner index stops at the row)
    for (int tile = tid; tile < TILES; tile += NT) {
      const int i0 = (tile >> 5) * 4, j0 = (tile & 31) * 2;
      float acc[4][2];
      zero_tile(acc);
      mm_tn(acc, tT, RP, qs, kQP, i0, j0, 0, i0 + 4);
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        *reinterpret_cast<float2*>(mid + (i0 + r) * kQP + j0) = make_float2(acc[r][0], acc[r][1]);
        float* st = p.state + ((size_t)sys * R + i0 + r) * d + d0 + j0;
        if (j0 < dv) st[0] = acc[r][0];
        if (j0 + 1 < dv) st[1] = acc[r][1];
      }
    }
    __syncthreads();
    // (F - eta I) Z -> qs
    for (int tile = tid; tile < TILES; tile += NT) {
      const int i0 = (tile >> 5) * 4, j0 = (tile & 31) * 2;
      float acc[4][2];
      zero_tile(acc);
      mm_tn(acc, mT, RP, mid, kQP, i0, j0, 0, R);
#pragma unroll
      for (int r = 0; r < 4; ++r)
        *reinterpret_cast<float2*>(qs + (i0 + r) * kQP + j0) = make_float2(acc[r][0], acc[r][1]);
    }
    __syncthreads();
    // W = T^T (F - eta I) Z   (the inner index starts at the row), two BF16 words
    __nv_bfloat16* hi = p.coeff + (size_t)sys * 2 * R * p.dpad;
    __nv_bfloat16* lo = hi + (size_t)R * p.dpad;
    const int cend = min(64, p.dpad - d0);
    for (int tile = tid; tile < TILES; tile += NT) {
      const int i0 = (tile >> 5) * 4, j0 = (tile & 31) * 2;
      float acc[4][2];
      zero_tile(acc);
      mm_tn(acc, ts, RP, qs, kQP, i0, j0, i0, R);
      if (j0 < cend) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const size_t idx = (size_t)(i0 + r) * p.dpad + d0 + j0;
          const float v0 = j0 < dv ? acc[r][0] : 0.f, v1 = j0 + 1 < dv ? acc[r][1] : 0.f;
          if (p.pair_ok) {
            store_split2(hi, lo, idx, v0, v1);
          } else {
            store_split(hi, lo, idx, v0);
            store_split(hi, lo, idx + 1, v1);
          }
        }
      }
    }
    __syncthreads();
  }
  if (!ok && tid == 0) atomicExch(p.error, kErrBarrierTimeout);
}

// ---------------------------------------------------------------------------------------
// compact adjoint per (b,h)
// ---------------------------------------------------------------------------------------
struct CompactBwdParams {
  const float* partials;     // E partials [systems][chunks][r*d] or packed when chunks == 0
  const float* de_partials;  // [systems][chunks*de_slots]; unused when packed
  const float* counts;
  const float* eta;
  const float* core_map;
  const float* inverse;
  const float* state;
  float* hmat;               // [systems][r*r]   H = U Z^T
  float* de_sys;             // [systems]
  __nv_bfloat16* gram_grad;  // [systems][2][r][r]
  __nv_bfloat16* cross_grad; // [systems][2][r][dpad]
  int* error;
  int heads, tokens, head_dim, dpad, dblocks, chunks, pf, complement, systems, de_slots;
  int staged, pair_ok;
};

template <int R>
constexpr int compact_bwd_fixed_floats() {
  return 5 * R * CompactDims<R>::RP + 3 * R * kQP + 4;
}

template <int R, int MINB = 1>
__global__ void __launch_bounds__(compact_threads<R, MINB>(), MINB)
compact_backward_kernel(const CompactBwdParams p) {
  using D = CompactDims<R, MINB>;
  constexpr int RP = D::RP, NT = D::NT;
  extern __shared__ __align__(16) unsigned char csm[];
  float* ts = reinterpret_cast<float*>(csm);   // T
  float* tT = ts + R * RP;                     // T^T
  float* mm = tT + R * RP;                     // M = F - eta I
  float* mT = mm + R * RP;                     // M^T
  float* hm = mT + R * RP;                     // H
  float* es = hm + R * RP;                     // E block / dZ / sym(X)
  float* us = es + R * kQP;                    // U block / Y
  float* zs = us + R * kQP;                    // Z block
  uint64_t* bar = reinterpret_cast<uint64_t*>(zs + R * kQP);
  float* stage = reinterpret_cast<float*>(bar + 2);

  grid_dependency_wait();
  const int tid = threadIdx.x;
  const int sys = blockIdx.x;
  const int b = sys / p.heads, h = sys - b * p.heads;
  const bool packed = p.chunks == 0;
  const int nch = packed ? 1 : p.chunks;
  const float n = p.counts ? p.counts[b] : (float)p.tokens;
  const float inv_s = packed ? 1.f : inv_sqrt_rn(n);
  const float* src = p.partials + (size_t)sys * nch * p.pf;
  const float eta = p.eta ? p.eta[h] : 0.f;   // null: the short-sequence path adds the eta term in token space
  const int d = p.head_dim;
  const bool staged = p.staged != 0;

  if (staged) {
    const uint32_t bar_addr = smem_u32(bar);
    if (tid == 0) {
      mbar_init(bar_addr, 1);
      mbar_fence_init();
    }
    __syncthreads();
    if (tid == 0) stage_partials(smem_u32(stage), src, nch, p.pf, 0, p.pf, bar_addr);
  }
  for (int i = tid; i < R * R; i += NT) {
    const int row = i / R, col = i - row * R;
    const float t = p.inverse[(size_t)sys * R * R + i];
    ts[row * RP + col] = t;
    tT[col * RP + row] = t;
    float f = p.complement ? 0.f : p.core_map[(size_t)h * R * R + i];
    if (row == col) f -= eta;
    mm[row * RP + col] = f;
    mT[col * RP + row] = f;
  }
  if (tid < 32) {
    // <dY, C> of this system: lane-strided sums in index order, then a shuffle tree
    float v = 0.f;
    if (packed) {
      if (tid == 0) v = p.partials[(size_t)p.systems * p.pf + sys];
    } else {
      const int cnt = p.chunks * p.de_slots;
      for (int c = tid; c < cnt; c += 32) v += p.de_partials[(size_t)sys * cnt + c];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (tid == 0) p.de_sys[sys] = v;
  }
  bool ok = true;
  if (staged) ok = mbar_wait(smem_u32(bar), 0);

  constexpr int TILES = (R / 4) * 32;          // 4 x 2 tiles of an r x 64 block
  constexpr int RTILES = (R / 4) * (R / 2);    // 4 x 2 tiles of an r x r matrix, columns j and j + r/2
  constexpr int RT_PER = (RTILES + NT - 1) / NT;
  float hacc[RT_PER][4][2];                    // H = sum over channel blocks of U Z^T, kept in registers
#pragma unroll
  for (int e = 0; e < RT_PER; ++e) zero_tile(hacc[e]);

  for (int jb = 0; jb < p.dblocks; ++jb) {
    const int d0 = jb * 64, dv = min(64, d - d0);
    for (int i0 = tid; i0 < R * 64; i0 += 4 * NT) {
      int off[4];
      bool valid[4];
      float acc[4], zv[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = i0 + e * NT, row = i >> 6, c = i & 63;
        valid[e] = c < dv;
        off[e] = row * d + d0 + (valid[e] ? c : 0);
        zv[e] = valid[e] ? p.state[(size_t)sys * R * d + off[e]] : 0.f;
      }
      if (staged) sum_chunks4<2>(stage, p.pf, nch, off, valid, acc);
      else sum_chunks4<(MINB == 1 ? 8 : 1)>(src, p.pf, nch, off, valid, acc);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = i0 + e * NT;
        es[(i >> 6) * kQP + (i & 63)] = acc[e] * inv_s;
        zs[(i >> 6) * kQP + (i & 63)] = zv[e];
      }
    }
    __syncthreads();
    // U = T E
    for (int tile = tid; tile < TILES; tile += NT) {
      const int i0 = (tile >> 5) * 4, j0 = (tile & 31) * 2;
      float acc[4][2];
      zero_tile(acc);
      mm_tn(acc, tT, RP, es, kQP, i0, j0, 0, i0 + 4);
#pragma unroll
      for (int r = 0; r < 4; ++r)
        *reinterpret_cast<float2*>(us + (i0 + r) * kQP + j0) = make_float2(acc[r][0], acc[r][1]);
    }
    __syncthreads();
    // H += U Z^T   (r x r, contraction over the 64 channels)
#pragma unroll
    for (int e = 0; e < RT_PER; ++e) {
      const int tile = tid + e * NT;
      if (tile < RTILES) {
        const int i0 = (tile / (R / 2)) * 4, j0 = tile % (R / 2);
        mm_nt<64>(hacc[e], us, kQP, zs, kQP, i0, j0, j0 + R / 2);
      }
    }
    // dZ = M^T U -> es
    for (int tile = tid; tile < TILES; tile += NT) {
      const int i0 = (tile >> 5) * 4, j0 = (tile & 31) * 2;
      float acc[4][2];
      zero_tile(acc);
      mm_tn(acc, mm, RP, us, kQP, i0, j0, 0, R);
#pragma unroll
      for (int r = 0; r < 4; ++r)
        *reinterpret_cast<float2*>(es + (i0 + r) * kQP + j0) = make_float2(acc[r][0], acc[r][1]);
    }
    __syncthreads();
    // dQ = T^T dZ, two BF16 words
    __nv_bfloat16* hi = p.cross_grad + (size_t)sys * 2 * R * p.dpad;
    __nv_bfloat16* lo = hi + (size_t)R * p.dpad;
    const int cend = min(64, p.dpad - d0);
    for (int tile = tid; tile < TILES; tile += NT) {
      const int i0 = (tile >> 5) * 4, j0 = (tile & 31) * 2;
      float acc[4][2];
      zero_tile(acc);
      mm_tn(acc, ts, RP, es, kQP, i0, j0, i0, R);
      if (j0 < cend) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const size_t idx = (size_t)(i0 + r) * p.dpad + d0 + j0;
          const float v0 = j0 < dv ? acc[r][0] : 0.f, v1 = j0 + 1 < dv ? acc[r][1] : 0.f;
          if (p.pair_ok) {
            store_split2(hi, lo, idx, v0, v1);
          } else {
            store_split(hi, lo, idx, v0);
            store_split(hi, lo, idx + 1, v1);
          }
        }
      }
    }
    __syncthreads();
  }

  grid_launch_dependents();
  // H to shared memory and to global (for the per-head sum over the batch)
#pragma unroll
  for (int e = 0; e < RT_PER; ++e) {
    const int tile = tid + e * NT;
    if (tile < RTILES) {
      const int i0 = (tile / (R / 2)) * 4, j0 = tile % (R / 2), j1 = j0 + R / 2;
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        hm[(i0 + r) * RP + j0] = hacc[e][r][0];
        hm[(i0 + r) * RP + j1] = hacc[e][r][1];
        p.hmat[(size_t)sys * R * R + (i0 + r) * R + j0] = hacc[e][r][0];
        p.hmat[(size_t)sys * R * R + (i0 + r) * R + j1] = hacc[e][r][1];
      }
    }
  }
  __syncthreads();
  // X = -M H^T - M^T H;  sym = low + low^T with low = tril(X,-1)/2 + diag(X)/4, i.e.
  // sym[r][k] = X[max(r,k)][min(r,k)] / 2, written to both triangles from the lower one
  float* sym = es;
  float* ys = us;
  for (int tile = tid; tile < RTILES; tile += NT) {
    const int i0 = (tile / (R / 2)) * 4, j0 = tile % (R / 2), j1 = j0 + R / 2;
    float acc[4][2];
    zero_tile(acc);
    mm_nt<R>(acc, mm, RP, hm, RP, i0, j0, j1);
    mm_tn_s(acc, mm, RP, hm, RP, i0, j0, j1, 0, R);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int i = i0 + r;
      if (i >= j0) sym[i * RP + j0] = sym[j0 * RP + i] = -0.5f * acc[r][0];
      if (i >= j1) sym[i * RP + j1] = sym[j1 * RP + i] = -0.5f * acc[r][1];
    }
  }
  __syncthreads();
  // Y = sym T  (T lower triangular: row k of T is zero beyond column k)
  for (int tile = tid; tile < RTILES; tile += NT) {
    const int i0 = (tile / (R / 2)) * 4, j0 = tile % (R / 2), j1 = j0 + R / 2;
    float acc[4][2];
    zero_tile(acc);
    mm_tn_s(acc, sym, RP, ts, RP, i0, j0, j1, j0, R);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      ys[(i0 + r) * RP + j0] = acc[r][0];
      ys[(i0 + r) * RP + j1] = acc[r][1];
    }
  }
  __syncthreads();
  // dG = T^T Y ;  stored as s (dG + dG^T) (dG is symmetric, s = 1/sqrt(n): the factor the token pass would
  // otherwise apply to the product A (dG + dG^T) before adding the other two products) in two BF16 words
  const float s_tok = inv_sqrt_rn(n);
  __nv_bfloat16* ghi = p.gram_grad + (size_t)sys * 2 * R * R;
  __nv_bfloat16* glo = ghi + R * R;
  for (int tile = tid; tile < RTILES; tile += NT) {
    const int i0 = (tile / (R / 2)) * 4, j0 = tile % (R / 2), j1 = j0 + R / 2;
    float acc[4][2];
    zero_tile(acc);
    mm_tn_s(acc, ts, RP, ys, RP, i0, j0, j1, i0, R);
    mm_tn_s(acc, ys, RP, ts, RP, i0, j0, j1, j0, R);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      store_split(ghi, glo, (size_t)(i0 + r) * R + j0, acc[r][0] * s_tok);
      store_split(ghi, glo, (size_t)(i0 + r) * R + j1, acc[r][1] * s_tok);
    }
  }
  if (!ok && tid == 0) atomicExch(p.error, kErrBarrierTimeout);
}

// ---------------------------------------------------------------------------------------
// per-head core kernels (stand-alone launches; the mixer drivers run the same device
// functions from spare CTAs of the statistics / token-backward grids instead)
// ---------------------------------------------------------------------------------------
template <int R>
__global__ void __launch_bounds__(kCompactThreads)
core_forward_kernel(const float* __restrict__ base_raw, const float* __restrict__ eta_raw, int complement,
                    float* __restrict__ eta_out, float* __restrict__ slope_out, float* __restrict__ core_map,
                    int* __restrict__ core_info) {
  extern __shared__ __align__(16) double dsm[];
  grid_launch_dependents();
  grid_dependency_wait();
  core_forward_device<R, kCompactThreads>(base_raw, eta_raw, blockIdx.x, complement, eta_out, slope_out, core_map,
                                          core_info, reinterpret_cast<unsigned char*>(dsm), threadIdx.x);
}

__global__ void __launch_bounds__(kCompactThreads)
core_backward_kernel(const float* __restrict__ base_raw, const float* __restrict__ hmat,
                     const float* __restrict__ de_sys, const float* __restrict__ slope,
                     const float* __restrict__ core_map, int r, int heads, int batch, int complement,
                     float grad_scale, float* __restrict__ d_base, float* __restrict__ d_eta_raw) {
  extern __shared__ double dsm[];
  grid_launch_dependents();
  grid_dependency_wait();
  core_backward_device(base_raw, hmat, de_sys, slope, core_map, r, blockIdx.x, heads, batch, complement,
                       grad_scale, d_base, d_eta_raw, reinterpret_cast<unsigned char*>(dsm), threadIdx.x,
                       kCompactThreads);
}

// ---------------------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------------------
template <class K>
static int set_smem(K kern, size_t bytes) {
  if (bytes > 48 * 1024) {
    if (ensure_dynamic_smem(reinterpret_cast<const void*>(kern), (int)bytes) != MS_OK) return MS_ERR_LAUNCH;
  }
  return MS_OK;
}

template <int R>
static int launch_core_fwd_r(const ms_shape& s, const float* base_raw, const float* eta_raw, const ms_tape& t,
                             cudaStream_t st) {
  const size_t bytes = core_forward_smem_bytes(R);
  if (set_smem(core_forward_kernel<R>, bytes)) return MS_ERR_LAUNCH;
  launch_kernel(core_forward_kernel<R>, dim3(s.heads), dim3(kCompactThreads), bytes, st, base_raw, eta_raw, s.complement, t.eta,
                                                                 t.eta_slope, t.core_map, t.core_info);
  return cudaGetLastError() == cudaSuccess ? MS_OK : MS_ERR_LAUNCH;
}

int launch_core_forward(const ms_shape& s, const float* base_raw, const float* eta_raw, const ms_tape& t,
                        cudaStream_t st) {
  switch (s.rank) {
    case 16: return launch_core_fwd_r<16>(s, base_raw, eta_raw, t, st);
    case 32: return launch_core_fwd_r<32>(s, base_raw, eta_raw, t, st);
    case 48: return launch_core_fwd_r<48>(s, base_raw, eta_raw, t, st);
    case 64: return launch_core_fwd_r<64>(s, base_raw, eta_raw, t, st);
  }
  return MS_ERR_UNSUPPORTED_RANK;
}

constexpr size_t kCompactSmemLimit = 227 * 1024;

// bytes of the staging area for `chunks` partials of `floats` floats, or 0 when they do not fit
// beside `fixed_floats` or the source is not 16-byte aligned
static size_t staging_bytes(const float* partials, int chunks, size_t floats, size_t fixed_floats) {
  const size_t need = (size_t)chunks * floats * sizeof(float);
  if ((reinterpret_cast<uintptr_t>(partials) & 15u) != 0 || (floats & 3u) != 0) return 0;
  if (need >= (1u << 20)) return 0;   // one mbarrier phase counts less than 2^20 bytes
  return fixed_floats * sizeof(float) + need <= kCompactSmemLimit ? need : 0;
}

template <int R>
static int launch_compact_fwd_r(CompactFwdParams& p, int systems, cudaStream_t st) {
  const size_t fixed = compact_fwd_fixed_floats<R>();
  const int nch = p.chunks == 0 ? 1 : p.chunks;
  // many systems: more CTAs per SM (a smaller register budget, a single partial read straight from global
  // memory) matter more than the latency of one system
  const bool many = R <= 32 && nch == 1 && systems >= 2 * sm_count();
  const size_t stage = many ? 0 : staging_bytes(p.partials, nch, (size_t)p.pf, fixed);
  p.staged = stage != 0;
  const size_t bytes = fixed * sizeof(float) + stage;
  if constexpr (R <= 32) {
    if (many) {
      if (set_smem(compact_forward_kernel<R, 4>, bytes)) return MS_ERR_LAUNCH;
      launch_kernel(compact_forward_kernel<R, 4>, dim3(systems), dim3(compact_threads<R, 4>()), bytes, st, p);
      return cudaGetLastError() == cudaSuccess ? MS_OK : MS_ERR_LAUNCH;
    }
  }
  if (set_smem(compact_forward_kernel<R>, bytes)) return MS_ERR_LAUNCH;
  launch_kernel(compact_forward_kernel<R>, dim3(systems), dim3(compact_threads<R>()), bytes, st, p);
  return cudaGetLastError() == cudaSuccess ? MS_OK : MS_ERR_LAUNCH;
}

int launch_compact_forward(const ms_shape& s, const Plan& plan, const float* counts, const float* partials,
                           bool packed, const ms_tape& t, cudaStream_t st) {
  CompactFwdParams p;
  p.partials = partials; p.counts = counts; p.eta = t.eta; p.core_map = t.core_map;
  p.inverse = t.inverse; p.state = t.state; p.coeff = static_cast<__nv_bfloat16*>(t.coeff);
  p.error = device_error_word();
  if (!p.error) return MS_ERR_LAUNCH;
  p.heads = s.heads; p.tokens = s.tokens; p.head_dim = s.head_dim; p.dpad = plan.dpad;
  p.dblocks = plan.dblocks; p.chunks = packed ? 0 : plan.chunks; p.pf = (int)plan.fwd_partial_floats;
  p.complement = s.complement;
  p.staged = 0;
  p.pair_ok = (reinterpret_cast<uintptr_t>(t.coeff) & 3u) == 0;
  switch (s.rank) {
    case 16: return launch_compact_fwd_r<16>(p, plan.systems, st);
    case 32: return launch_compact_fwd_r<32>(p, plan.systems, st);
    case 48: return launch_compact_fwd_r<48>(p, plan.systems, st);
    case 64: return launch_compact_fwd_r<64>(p, plan.systems, st);
  }
  return MS_ERR_UNSUPPORTED_RANK;
}

template <int R>
static int launch_compact_bwd_r(CompactBwdParams& p, int systems, cudaStream_t st) {
  const size_t fixed = compact_bwd_fixed_floats<R>();
  const int nch = p.chunks == 0 ? 1 : p.chunks;
  const bool many = R <= 32 && nch == 1 && systems >= 2 * sm_count();   // as in the forward launcher
  const size_t stage = many ? 0 : staging_bytes(p.partials, nch, (size_t)p.pf, fixed);
  p.staged = stage != 0;
  const size_t bytes = fixed * sizeof(float) + stage;
  if constexpr (R <= 32) {
    if (many) {
      if (set_smem(compact_backward_kernel<R, 4>, bytes)) return MS_ERR_LAUNCH;
      launch_kernel(compact_backward_kernel<R, 4>, dim3(systems), dim3(compact_threads<R, 4>()), bytes, st, p);
      return cudaGetLastError() == cudaSuccess ? MS_OK : MS_ERR_LAUNCH;
    }
  }
  if (set_smem(compact_backward_kernel<R>, bytes)) return MS_ERR_LAUNCH;
  launch_kernel(compact_backward_kernel<R>, dim3(systems), dim3(compact_threads<R>()), bytes, st, p);
  return cudaGetLastError() == cudaSuccess ? MS_OK : MS_ERR_LAUNCH;
}

int launch_compact_backward(const ms_shape& s, const Plan& plan, const float* counts, const float* partials,
                            const float* de_partials, bool packed, const ms_tape& t, float* hmat,
                            float* de_sys, void* gram_grad, void* cross_grad, cudaStream_t st) {
  CompactBwdParams p;
  p.partials = partials; p.de_partials = de_partials; p.counts = counts; p.eta = t.eta;
  p.core_map = t.core_map; p.inverse = t.inverse; p.state = t.state; p.hmat = hmat; p.de_sys = de_sys;
  p.gram_grad = static_cast<__nv_bfloat16*>(gram_grad);
  p.cross_grad = static_cast<__nv_bfloat16*>(cross_grad);
  p.error = device_error_word();
  if (!p.error) return MS_ERR_LAUNCH;
  p.heads = s.heads; p.tokens = s.tokens; p.head_dim = s.head_dim; p.dpad = plan.dpad;
  p.dblocks = plan.dblocks; p.chunks = packed ? 0 : plan.chunks; p.pf = (int)plan.bwd_partial_floats;
  p.de_slots = plan.de_slots;
  p.complement = s.complement; p.systems = plan.systems;
  p.staged = 0;
  p.pair_ok = (reinterpret_cast<uintptr_t>(cross_grad) & 3u) == 0;
  switch (s.rank) {
    case 16: return launch_compact_bwd_r<16>(p, plan.systems, st);
    case 32: return launch_compact_bwd_r<32>(p, plan.systems, st);
    case 48: return launch_compact_bwd_r<48>(p, plan.systems, st);
    case 64: return launch_compact_bwd_r<64>(p, plan.systems, st);
  }
  return MS_ERR_UNSUPPORTED_RANK;
}

int launch_core_backward(const ms_shape& s, const float* base_raw, const float* hmat, const float* de_sys,
                         const ms_tape& t, float grad_scale, float* d_base, float* d_eta_raw,
                         cudaStream_t st) {
  const size_t bytes = core_backward_smem_bytes(s.rank);
  if (set_smem(core_backward_kernel, bytes)) return MS_ERR_LAUNCH;
  launch_kernel(core_backward_kernel, dim3(s.heads), dim3(kCompactThreads), bytes, st, base_raw, hmat, de_sys, t.eta_slope,
                                                               t.core_map, s.rank, s.heads, s.batch,
                                                               s.complement, grad_scale, d_base, d_eta_raw);
  return cudaGetLastError() == cudaSuccess ? MS_OK : MS_ERR_LAUNCH;
}

}  // namespace ms
