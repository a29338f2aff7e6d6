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
// Triton compact kernels (memsolve/ball/cuda.py:2530-2768).  The Cholesky factor is computed
// with one matrix row per lane in registers (FP32, the diagonal carried in FP64, like the
// reference's native kernel) while the other warps already sum the partial moments; the
// r x d and r x r products are FP32 FMA on shared-memory operands with several independent
// accumulation chains per thread.  Partial sums of the token reductions are added in chunk order with
// several independent loads in flight, so the result is order-deterministic and the kernel is
// not bound by load latency.
#include "ms_core.cuh"

namespace ms {

constexpr int kCompactThreads = 256;

// ---------------------------------------------------------------------------------------
// Cholesky inverse factor, one matrix row per lane, FP64 registers
// ---------------------------------------------------------------------------------------
// gs: G (FP32, pitch R) in shared memory.  Writes T = chol(I + sym(G))^-1 (lower triangular,
// FP32, pitch R+1) to ts.  Executed by the first ceil(R/32) warps.  Gaussian elimination
// applies the unit-lower factor to the identity in place; a final row scaling by the inverse
// square roots of the pivots turns it into the Cholesky inverse.
// One elimination step per template instance, so that every register index is a constant.
// The bulk is FP32; each row's diagonal entry (its future pivot) is carried in FP64, as the
// reference's native Cholesky does.
template <int R, int K>
__device__ __forceinline__ void cholesky_eliminate(float (&a)[R], double& diag, float* rowbuf, int i, bool live) {
  if constexpr (K < R) {
    constexpr int NW = (R + 31) / 32;
    float* rb = rowbuf + (K & 1) * R;
    if (i == K) {
      const float inv0 = __frcp_rn((float)diag);
      const double inv = (double)inv0 * fma(-diag, (double)inv0, 2.0);   // one Newton step in FP64
      rb[K] = (float)inv;
#pragma unroll
      for (int j = K + 1; j < R; ++j) rb[j] = a[j];
#pragma unroll
      for (int j = 0; j < K; ++j) rb[j] = a[j];
    }
    if (NW == 1) __syncwarp();
    else asm volatile("bar.sync 1, %0;\n" ::"n"(NW * 32));
    if (live && i > K) {
      const float f = a[K] * rb[K];
      diag = fma(-(double)f, (double)rb[i], diag);
#pragma unroll
      for (int j = 0; j < R; ++j) {
        if (j != K) a[j] = fmaf(-f, rb[j], a[j]);
      }
      a[K] = -f;
    }
    cholesky_eliminate<R, K + 1>(a, diag, rowbuf, i, live);
  }
}

template <int R>
__device__ __noinline__ void cholesky_inverse_rows(const float* gs, float* ts, float* rowbuf, int tid) {
  constexpr int NW = (R + 31) / 32;
  if (tid >= NW * 32) return;
  const int i = tid;
  const bool live = i < R;
  float a[R];
#pragma unroll
  for (int j = 0; j < R; ++j) a[j] = live ? 0.5f * (gs[i * R + j] + gs[j * R + i]) + (i == j ? 1.0f : 0.0f) : 0.f;
  double diag = live ? 1.0 + (double)gs[i * R + i] : 1.0;
  cholesky_eliminate<R, 0>(a, diag, rowbuf, i, live);
  if (live) {
    const double sc = rsqrt(diag);
#pragma unroll
    for (int j = 0; j < R; ++j) {
      float v = 0.f;
      if (j < i) v = (float)((double)a[j] * sc);
      else if (j == i) v = (float)sc;
      ts[i * (R + 1) + j] = v;
    }
  }
}

// ---------------------------------------------------------------------------------------
// helpers
// ---------------------------------------------------------------------------------------
// out[i][c] = sum_j lhs(i,j) * rhs[j][c] for i < R, c < 64 (rhs/out pitch 65); jlo/jhi bound
// the inner index (triangular factors).
// Each thread owns one column and R/4 interleaved rows: one load of the right-hand side feeds R/4
// independent FMA chains.  Triangular left factors hold explicit zeros, so the inner index runs
// over the full range (the bounds jlo/jhi are accepted for documentation only).
template <int R, class LHS, class LO, class HI>
__device__ __forceinline__ void small_mm(LHS lhs, LO, HI, const float* rhs, float* out, int tid) {
  constexpr int ROWS = R / (kCompactThreads / 64);
  const int c = tid & 63, rg = tid >> 6;
  float acc[ROWS];
#pragma unroll
  for (int k = 0; k < ROWS; ++k) acc[k] = 0.f;
#pragma unroll 4
  for (int j = 0; j < R; ++j) {
    const float r = rhs[j * 65 + c];
#pragma unroll
    for (int k = 0; k < ROWS; ++k) acc[k] = fmaf(lhs(rg + (kCompactThreads / 64) * k, j), r, acc[k]);
  }
#pragma unroll
  for (int k = 0; k < ROWS; ++k) out[(rg + (kCompactThreads / 64) * k) * 65 + c] = acc[k];
}

// acc[e] = sum over chunks (in chunk order) of src[c*stride + off[e]] for PER entries of this
// thread; four chunks x PER entries of loads are issued before any of them is consumed.
template <int PER>
__device__ __forceinline__ void sum_partials(const float* __restrict__ src, size_t stride, int nch,
                                             const size_t (&off)[PER], const bool (&ok)[PER], float (&acc)[PER]) {
#pragma unroll
  for (int e = 0; e < PER; ++e) acc[e] = 0.f;
  int c = 0;
  for (; c + 4 <= nch; c += 4) {
    float v[4][PER];
#pragma unroll
    for (int k = 0; k < 4; ++k)
#pragma unroll
      for (int e = 0; e < PER; ++e) v[k][e] = ok[e] ? __ldg(src + (size_t)(c + k) * stride + off[e]) : 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k)
#pragma unroll
      for (int e = 0; e < PER; ++e) acc[e] += v[k][e];
  }
  for (; c < nch; ++c) {
    float v[PER];
#pragma unroll
    for (int e = 0; e < PER; ++e) v[e] = ok[e] ? __ldg(src + (size_t)c * stride + off[e]) : 0.f;
#pragma unroll
    for (int e = 0; e < PER; ++e) acc[e] += v[e];
  }
}

// Sum, in chunk order, one R x 64 block of a partial r x d matrix (first element at `base`,
// row pitch d, columns [d0, d0+dv)) with NT cooperating threads (t = 0..NT-1) and write it,
// scaled, to dst (pitch 65; columns >= dv become zero).
template <int R, int NT>
__device__ __forceinline__ void sum_block(const float* __restrict__ src, size_t stride, int nch, size_t base, int d,
                                          int d0, int dv, float scale, float* dst, int t) {
  constexpr int PER = (R * 64 + NT - 1) / NT;
  size_t off[PER];
  bool ok[PER];
  float acc[PER];
#pragma unroll
  for (int e = 0; e < PER; ++e) {
    const int i = t + e * NT;
    const int row = i >> 6, c = i & 63;
    ok[e] = i < R * 64 && c < dv;
    off[e] = ok[e] ? base + (size_t)row * d + d0 + c : 0;
  }
  sum_partials<PER>(src, stride, nch, off, ok, acc);
#pragma unroll
  for (int e = 0; e < PER; ++e) {
    const int i = t + e * NT;
    if (i < R * 64) dst[(i >> 6) * 65 + (i & 63)] = acc[e] * scale;
  }
}

__device__ __forceinline__ void store_split(__nv_bfloat16* hi, __nv_bfloat16* lo, size_t idx, float v) {
  const __nv_bfloat16 hv = __float2bfloat16_rn(v);
  hi[idx] = hv;
  lo[idx] = __float2bfloat16_rn(v - __bfloat162float(hv));
}

// r x r products spread over the CTA: thread t owns entries t, t+256, ... (kRRPer<R> of them) and
// advances all of their dot products together, so the FMA chains are independent.
template <int R>
constexpr int kRRPer = (R * R + kCompactThreads - 1) / kCompactThreads;

template <int R, class INIT>
__device__ __forceinline__ void rr_init(float (&acc)[kRRPer<R>], INIT init, int tid) {
#pragma unroll
  for (int e = 0; e < kRRPer<R>; ++e) {
    const int i = tid + e * kCompactThreads;
    acc[e] = i < R * R ? init(i / R, i % R) : 0.f;
  }
}

// acc[e] += sum_k fa(row_e, k) * fb(k, col_e)
template <int R, int KLEN, class FA, class FB>
__device__ __forceinline__ void rr_accumulate(float (&acc)[kRRPer<R>], FA fa, FB fb, int tid) {
  int row[kRRPer<R>], col[kRRPer<R>];
#pragma unroll
  for (int e = 0; e < kRRPer<R>; ++e) {
    const int i = min(tid + e * kCompactThreads, R * R - 1);
    row[e] = i / R;
    col[e] = i % R;
  }
#pragma unroll 4
  for (int k = 0; k < KLEN; ++k) {
#pragma unroll
    for (int e = 0; e < kRRPer<R>; ++e) acc[e] = fmaf(fa(row[e], k), fb(k, col[e]), acc[e]);
  }
}

template <int R, class STORE>
__device__ __forceinline__ void rr_store(const float (&acc)[kRRPer<R>], STORE store, int tid) {
#pragma unroll
  for (int e = 0; e < kRRPer<R>; ++e) {
    const int i = tid + e * kCompactThreads;
    if (i < R * R) store(i / R, i % R, i, acc[e]);
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
  int heads, tokens, head_dim, dpad, dblocks, chunks, pf, complement;
};

template <int R>
__global__ void __launch_bounds__(kCompactThreads)
compact_forward_kernel(const CompactFwdParams p) {
  extern __shared__ float fsm[];
  float* gs = fsm;                      // R*R            G
  float* ts = gs + R * R;               // R*(R+1)        T
  float* ms_ = ts + R * (R + 1);        // R*(R+1)        F - eta I
  float* qs = ms_ + R * (R + 1);        // R*65           Q block -> scratch
  float* mid = qs + R * 65;             // R*65
  float* rowbuf = mid + R * 65;         // 2*R floats (pivot-row broadcast, double buffered)

  const int tid = threadIdx.x;
  const int sys = blockIdx.x;
  const int b = sys / p.heads, h = sys - b * p.heads;
  const bool packed = p.chunks == 0;
  const int nch = packed ? 1 : p.chunks;
  const float n = p.counts ? p.counts[b] : (float)p.tokens;
  const float inv_n = packed ? 1.f : inv_rn(n);
  const float inv_s = packed ? 1.f : inv_sqrt_rn(n);
  const float* src = p.partials + (size_t)sys * nch * p.pf;
  const float eta = p.eta[h];
  const int d = p.head_dim;
  MS_TICK(0);

  {
    constexpr int PER = (R * R + kCompactThreads - 1) / kCompactThreads;
    size_t off[PER];
    bool ok[PER];
    float acc[PER];
#pragma unroll
    for (int e = 0; e < PER; ++e) {
      const int i = tid + e * kCompactThreads;
      ok[e] = i < R * R;
      off[e] = ok[e] ? i : 0;
    }
    sum_partials<PER>(src, p.pf, nch, off, ok, acc);
#pragma unroll
    for (int e = 0; e < PER; ++e) {
      const int i = tid + e * kCompactThreads;
      if (i < R * R) {
        gs[i] = acc[e] * inv_n;
        const int row = i / R, col = i - row * R;
        float f = p.complement ? 0.f : p.core_map[(size_t)h * R * R + i];
        if (row == col) f -= eta;
        ms_[row * (R + 1) + col] = f;
      }
    }
  }
  __syncthreads();
  MS_TICK(1);
  // the factorisation occupies the first warp(s); the other warps meanwhile sum the partial
  // moments of the first channel block
  constexpr int CHOL_THREADS = ((R + 31) / 32) * 32;
  if (tid < CHOL_THREADS) {
    cholesky_inverse_rows<R>(gs, ts, rowbuf, tid);
  } else {
    sum_block<R, kCompactThreads - CHOL_THREADS>(src, p.pf, nch, (size_t)R * R, d, 0, min(64, d), inv_s, qs,
                                                  tid - CHOL_THREADS);
  }
  __syncthreads();
  MS_TICK(2);
  for (int i = tid; i < R * R; i += kCompactThreads) {
    const int row = i / R, col = i - row * R;
    p.inverse[(size_t)sys * R * R + i] = ts[row * (R + 1) + col];
  }

  for (int jb = 0; jb < p.dblocks; ++jb) {
    const int d0 = jb * 64, dv = min(64, d - d0);
    if (jb > 0) {
      sum_block<R, kCompactThreads>(src, p.pf, nch, (size_t)R * R, d, d0, dv, inv_s, qs, tid);
      __syncthreads();
    }
    MS_TICK(3);
    // Z = T Q   (T lower triangular)
    small_mm<R>([&](int i, int j) { return ts[i * (R + 1) + j]; }, [](int) { return 0; },
                [](int i) { return i + 1; }, qs, mid, tid);
    __syncthreads();
    MS_TICK(4);
    for (int i = tid; i < R * 64; i += kCompactThreads) {
      const int row = i >> 6, c = i & 63;
      if (c < dv) p.state[((size_t)sys * R + row) * d + d0 + c] = mid[row * 65 + c];
    }
    // (F - eta I) Z -> qs
    small_mm<R>([&](int i, int j) { return ms_[i * (R + 1) + j]; }, [](int) { return 0; },
                [](int) { return R; }, mid, qs, tid);
    __syncthreads();
    // W = T^T (F - eta I) Z -> mid
    small_mm<R>([&](int i, int j) { return ts[j * (R + 1) + i]; }, [](int i) { return i; },
                [](int) { return R; }, qs, mid, tid);
    __syncthreads();
    MS_TICK(5);
    __nv_bfloat16* hi = p.coeff + (size_t)sys * 2 * R * p.dpad;
    __nv_bfloat16* lo = hi + (size_t)R * p.dpad;
    const int cend = min(64, p.dpad - d0);
    for (int i = tid; i < R * 64; i += kCompactThreads) {
      const int row = i >> 6, c = i & 63;
      if (c < cend) store_split(hi, lo, (size_t)row * p.dpad + d0 + c, c < dv ? mid[row * 65 + c] : 0.f);
    }
    __syncthreads();
    MS_TICK(6);
  }
}

// ---------------------------------------------------------------------------------------
// compact adjoint per (b,h)
// ---------------------------------------------------------------------------------------
struct CompactBwdParams {
  const float* partials;     // E partials [systems][chunks][r*d] or packed when chunks == 0
  const float* de_partials;  // [systems][chunks*dblocks]; unused when packed
  const float* counts;
  const float* eta;
  const float* core_map;
  const float* inverse;
  const float* state;
  float* hmat;               // [systems][r*r]   H = U Z^T
  float* de_sys;             // [systems]
  __nv_bfloat16* gram_grad;  // [systems][2][r][r]
  __nv_bfloat16* cross_grad; // [systems][2][r][dpad]
  int heads, tokens, head_dim, dpad, dblocks, chunks, pf, complement, systems;
};

template <int R>
__global__ void __launch_bounds__(kCompactThreads)
compact_backward_kernel(const CompactBwdParams p) {
  extern __shared__ float fsm[];
  constexpr int P = R + 1;
  float* ts = fsm;             // T
  float* mm = ts + R * P;      // M = F - eta I
  float* hm = mm + R * P;      // H accumulator
  float* es = hm + R * P;      // E block / scratch, R*65
  float* us = es + R * 65;     // U block
  float* zs = us + R * 65;     // Z block / scratch

  const int tid = threadIdx.x;
  const int sys = blockIdx.x;
  const int b = sys / p.heads, h = sys - b * p.heads;
  const bool packed = p.chunks == 0;
  const int nch = packed ? 1 : p.chunks;
  const float n = p.counts ? p.counts[b] : (float)p.tokens;
  const float inv_s = packed ? 1.f : inv_sqrt_rn(n);
  const float* src = p.partials + (size_t)sys * nch * p.pf;
  const float eta = p.eta[h];
  const int d = p.head_dim;
  MS_TICK(9);

  for (int i = tid; i < R * R; i += kCompactThreads) {
    const int row = i / R, col = i - row * R;
    ts[row * P + col] = p.inverse[(size_t)sys * R * R + i];
    float f = p.complement ? 0.f : p.core_map[(size_t)h * R * R + i];
    if (row == col) f -= eta;
    mm[row * P + col] = f;
    hm[row * P + col] = 0.f;
  }
  if (tid < 32) {
    // <dY, C> of this system: lane-strided sums in index order, then a shuffle tree
    float v = 0.f;
    if (packed) {
      if (tid == 0) v = p.partials[(size_t)p.systems * p.pf + sys];
    } else {
      const int cnt = p.chunks * p.dblocks;
      for (int c = tid; c < cnt; c += 32) v += p.de_partials[(size_t)sys * cnt + c];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (tid == 0) p.de_sys[sys] = v;
  }
  __syncthreads();

  MS_TICK(10);
  for (int jb = 0; jb < p.dblocks; ++jb) {
    const int d0 = jb * 64, dv = min(64, d - d0);
    {
      constexpr int PER = R * 64 / kCompactThreads;
      size_t off[PER];
      bool ok[PER];
      float acc[PER];
#pragma unroll
      for (int e = 0; e < PER; ++e) {
        const int i = tid + e * kCompactThreads;
        const int row = i >> 6, c = i & 63;
        ok[e] = c < dv;
        off[e] = (size_t)row * d + d0 + (ok[e] ? c : 0);
      }
      sum_partials<PER>(src, p.pf, nch, off, ok, acc);
#pragma unroll
      for (int e = 0; e < PER; ++e) {
        const int i = tid + e * kCompactThreads;
        const int row = i >> 6, c = i & 63;
        es[row * 65 + c] = acc[e] * inv_s;
        zs[row * 65 + c] = ok[e] ? p.state[(size_t)sys * R * d + off[e]] : 0.f;
      }
    }
    __syncthreads();
    MS_TICK(11);
    // U = T E
    small_mm<R>([&](int i, int j) { return ts[i * P + j]; }, [](int) { return 0; },
                [](int i) { return i + 1; }, es, us, tid);
    __syncthreads();
    MS_TICK(12);
    // H += U Z^T   (r x r, contraction over the 64 channels)
    {
      float acc[kRRPer<R>];
      rr_init<R>(acc, [&](int row, int col) { return hm[row * P + col]; }, tid);
      rr_accumulate<R, 64>(acc, [&](int row, int c) { return us[row * 65 + c]; },
                           [&](int c, int col) { return zs[col * 65 + c]; }, tid);
      rr_store<R>(acc, [&](int row, int col, int, float v) { hm[row * P + col] = v; }, tid);
    }
    MS_TICK(13);
    // dZ = M^T U -> es
    small_mm<R>([&](int i, int j) { return mm[j * P + i]; }, [](int) { return 0; },
                [](int) { return R; }, us, es, tid);
    __syncthreads();
    MS_TICK(14);
    // dQ = T^T dZ -> zs
    small_mm<R>([&](int i, int j) { return ts[j * P + i]; }, [](int i) { return i; },
                [](int) { return R; }, es, zs, tid);
    __syncthreads();
    __nv_bfloat16* hi = p.cross_grad + (size_t)sys * 2 * R * p.dpad;
    __nv_bfloat16* lo = hi + (size_t)R * p.dpad;
    const int cend = min(64, p.dpad - d0);
    for (int i = tid; i < R * 64; i += kCompactThreads) {
      const int row = i >> 6, c = i & 63;
      if (c < cend) store_split(hi, lo, (size_t)row * p.dpad + d0 + c, c < dv ? zs[row * 65 + c] : 0.f);
    }
    __syncthreads();
  }

  MS_TICK(16);
  // H to global for the per-head sum; X = -M H^T - M^T H
  float* xs = es;   // R*P fits in R*65
  float* ys = us;
  {
    float acc[kRRPer<R>];
    rr_init<R>(acc, [&](int, int) { return 0.f; }, tid);
    rr_accumulate<R, R>(acc, [&](int row, int k) { return -mm[row * P + k]; },
                        [&](int k, int col) { return hm[col * P + k]; }, tid);
    rr_accumulate<R, R>(acc, [&](int row, int k) { return -mm[k * P + row]; },
                        [&](int k, int col) { return hm[k * P + col]; }, tid);
    rr_store<R>(acc, [&](int row, int col, int i, float v) {
      p.hmat[(size_t)sys * R * R + i] = hm[row * P + col];
      xs[row * P + col] = v;
    }, tid);
  }
  __syncthreads();
  MS_TICK(17);
  // sym = low + low^T with low = tril(X,-1)/2 + diag(X)/4, i.e. sym[r][k] = X[max(r,k)][min(r,k)]/2;
  // Y = sym T  (T lower triangular with explicit zeros above the diagonal)
  {
    float acc[kRRPer<R>];
    rr_init<R>(acc, [&](int, int) { return 0.f; }, tid);
    rr_accumulate<R, R>(acc, [&](int row, int k) { return 0.5f * (row >= k ? xs[row * P + k] : xs[k * P + row]); },
                        [&](int k, int col) { return ts[k * P + col]; }, tid);
    rr_store<R>(acc, [&](int row, int col, int, float v) { ys[row * P + col] = v; }, tid);
  }
  __syncthreads();
  MS_TICK(18);
  // dG = T^T Y ;  stored as dG + dG^T (dG is symmetric) in two BF16 words
  __nv_bfloat16* ghi = p.gram_grad + (size_t)sys * 2 * R * R;
  __nv_bfloat16* glo = ghi + R * R;
  {
    float acc[kRRPer<R>];
    rr_init<R>(acc, [&](int, int) { return 0.f; }, tid);
    rr_accumulate<R, R>(acc, [&](int row, int k) { return ts[k * P + row]; },
                        [&](int k, int col) { return ys[k * P + col]; }, tid);
    rr_accumulate<R, R>(acc, [&](int row, int k) { return ys[k * P + row]; },
                        [&](int k, int col) { return ts[k * P + col]; }, tid);
    rr_store<R>(acc, [&](int, int, int i, float v) { store_split(ghi, glo, i, v); }, tid);
  }
  MS_TICK(19);
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
  extern __shared__ double dsm[];
  core_forward_device<R>(base_raw, eta_raw, blockIdx.x, complement, eta_out, slope_out, core_map, core_info,
                         reinterpret_cast<unsigned char*>(dsm), threadIdx.x, kCompactThreads);
}

__global__ void __launch_bounds__(kCompactThreads)
core_backward_kernel(const float* __restrict__ base_raw, const float* __restrict__ hmat,
                     const float* __restrict__ de_sys, const float* __restrict__ slope,
                     const float* __restrict__ core_map, int r, int heads, int batch, int complement,
                     float grad_scale, float* __restrict__ d_base, float* __restrict__ d_eta_raw) {
  extern __shared__ double dsm[];
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
  core_forward_kernel<R><<<s.heads, kCompactThreads, bytes, st>>>(base_raw, eta_raw, s.complement, t.eta,
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

template <int R>
static int launch_compact_fwd_r(const CompactFwdParams& p, int systems, cudaStream_t st) {
  const size_t bytes = (R * R + 2 * R * (R + 1) + 2 * R * 65) * sizeof(float) + 2 * R * sizeof(double) + 16;
  if (set_smem(compact_forward_kernel<R>, bytes)) return MS_ERR_LAUNCH;
  compact_forward_kernel<R><<<systems, kCompactThreads, bytes, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? MS_OK : MS_ERR_LAUNCH;
}

int launch_compact_forward(const ms_shape& s, const Plan& plan, const float* counts, const float* partials,
                           bool packed, const ms_tape& t, cudaStream_t st) {
  CompactFwdParams p;
  p.partials = partials; p.counts = counts; p.eta = t.eta; p.core_map = t.core_map;
  p.inverse = t.inverse; p.state = t.state; p.coeff = static_cast<__nv_bfloat16*>(t.coeff);
  p.heads = s.heads; p.tokens = s.tokens; p.head_dim = s.head_dim; p.dpad = plan.dpad;
  p.dblocks = plan.dblocks; p.chunks = packed ? 0 : plan.chunks; p.pf = (int)plan.fwd_partial_floats;
  p.complement = s.complement;
  switch (s.rank) {
    case 16: return launch_compact_fwd_r<16>(p, plan.systems, st);
    case 32: return launch_compact_fwd_r<32>(p, plan.systems, st);
    case 48: return launch_compact_fwd_r<48>(p, plan.systems, st);
    case 64: return launch_compact_fwd_r<64>(p, plan.systems, st);
  }
  return MS_ERR_UNSUPPORTED_RANK;
}

template <int R>
static int launch_compact_bwd_r(const CompactBwdParams& p, int systems, cudaStream_t st) {
  const size_t bytes = (3 * R * (R + 1) + 3 * R * 65) * sizeof(float);
  if (set_smem(compact_backward_kernel<R>, bytes)) return MS_ERR_LAUNCH;
  compact_backward_kernel<R><<<systems, kCompactThreads, bytes, st>>>(p);
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
  p.heads = s.heads; p.tokens = s.tokens; p.head_dim = s.head_dim; p.dpad = plan.dpad;
  p.dblocks = plan.dblocks; p.chunks = packed ? 0 : plan.chunks; p.pf = (int)plan.bwd_partial_floats;
  p.complement = s.complement; p.systems = plan.systems;
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
  core_backward_kernel<<<s.heads, kCompactThreads, bytes, st>>>(base_raw, hmat, de_sys, t.eta_slope,
                                                               t.core_map, s.rank, s.heads, s.batch,
                                                               s.complement, grad_scale, d_base, d_eta_raw);
  return cudaGetLastError() == cudaSuccess ? MS_OK : MS_ERR_LAUNCH;
}

}  // namespace ms
