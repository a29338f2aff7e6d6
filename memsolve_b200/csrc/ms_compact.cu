// Rank-space (r x r and r x d) stages of the MemSolve mixer, forward and adjoint.
//
//   core_forward      per head:   eta, d eta/d eta_raw, J = L L^T + Omega, F = (I+J)^-1 (I-J)
//   compact_forward   per (b,h):  G,Q (sum of partials) -> T = chol(I+G)^-1, Z = T Q,
//                                 W = T^T (F - eta I) Z  (written as two BF16 words)
//   compact_backward  per (b,h):  U = T E, H = U Z^T, dQ = T^T M^T U,
//                                 dG = T^T symlow(-M H^T - M^T H) T
//   core_backward     per head:   dF = sum_b H, d eta_raw, V = (I+J)^-T dF, dJ = -V (F+I)^T,
//                                 d base_raw
//
// Replaces the reference's native solvers (csrc/ball/solvers.cuh:34-560) and its Triton
// compact kernels (memsolve/ball/cuda.py:2281-2360, 2517-2768).  The factorisations run in
// FP64 (Cholesky: one matrix row per lane in registers; Cayley solve: pivoted Gauss-Jordan in
// shared memory); the r x d products are FP32 FMA.
#include "ms_common.cuh"

namespace ms {

constexpr double kSoftplusShift = 0.54132485461291810;  // log(expm1(1))
constexpr int kCompactThreads = 256;

// ---------------------------------------------------------------------------------------
// per-head core
// ---------------------------------------------------------------------------------------
// L = tril(U,-1) + diag(softplus(diag U + c0));  J = L L^T + triu(U,1) - triu(U,1)^T
// Writes J into jm (pitch r+1, FP64) and L into lc (pitch r+1, FP64).
__device__ void build_generator(const float* __restrict__ base, int r, double* lc, double* jm,
                                int tid, int nthreads) {
  const int p = r + 1;
  for (int i = tid; i < r * r; i += nthreads) {
    const int row = i / r, col = i - row * r;
    double v = 0.0;
    if (row > col) {
      v = (double)base[i];
    } else if (row == col) {
      const double x = (double)base[i] + kSoftplusShift;
      v = x > 30.0 ? x : log1p(exp(x));
    }
    lc[row * p + col] = v;
  }
  __syncthreads();
  for (int i = tid; i < r * r; i += nthreads) {
    const int row = i / r, col = i - row * r;
    const int kmax = row < col ? row : col;
    double acc = 0.0;
    for (int k = 0; k <= kmax; ++k) acc = fma(lc[row * p + k], lc[col * p + k], acc);
    if (row < col) acc += (double)base[row * r + col];
    if (row > col) acc -= (double)base[col * r + row];
    jm[row * p + col] = acc;
  }
  __syncthreads();
}

// Solve A X = B in place (X overwrites B) by Gauss-Jordan elimination with partial pivoting.
// A, B: r x r FP64 in shared memory, pitch r+1.  Returns 0 or k+1 for an exactly zero pivot.
__device__ int gauss_jordan(double* am, double* bm, int r, int* s_piv, int tid, int nthreads) {
  const int p = r + 1;
  int info = 0;
  for (int k = 0; k < r; ++k) {
    if (tid < 32) {
      // arg-max of |A[i][k]|, i >= k, first index wins ties
      double best = -1.0;
      int bi = k;
      for (int i = k + tid; i < r; i += 32) {
        const double v = fabs(am[i * p + k]);
        if (v > best) { best = v; bi = i; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const double ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
      }
      if (tid == 0) { s_piv[0] = bi; s_piv[1] = (best == 0.0) ? 1 : 0; }
    }
    __syncthreads();
    const int piv = s_piv[0];
    if (s_piv[1] && info == 0) info = k + 1;
    if (piv != k) {
      for (int j = tid; j < 2 * r; j += nthreads) {
        double* m = j < r ? am : bm;
        const int c = j < r ? j : j - r;
        const double t = m[k * p + c];
        m[k * p + c] = m[piv * p + c];
        m[piv * p + c] = t;
      }
    }
    __syncthreads();
    const double pv = am[k * p + k];
    const double ip = pv != 0.0 ? 1.0 / pv : 0.0;
    // multipliers first (column k is overwritten below)
    double* fcol = am + r * p;  // one spare row of r doubles after the matrix
    for (int i = tid; i < r; i += nthreads) fcol[i] = (i == k) ? 0.0 : am[i * p + k] * ip;
    __syncthreads();
    for (int idx = tid; idx < r * 2 * r; idx += nthreads) {
      const int i = idx / (2 * r), j = idx - i * 2 * r;
      if (i == k) continue;
      const double f = fcol[i];
      if (j < r) {
        if (j > k) am[i * p + j] = fma(-f, am[k * p + j], am[i * p + j]);
      } else {
        const int c = j - r;
        bm[i * p + c] = fma(-f, bm[k * p + c], bm[i * p + c]);
      }
    }
    __syncthreads();
  }
  for (int idx = tid; idx < r * r; idx += nthreads) {
    const int i = idx / r, c = idx - i * r;
    const double pv = am[i * p + i];
    bm[i * p + c] = pv != 0.0 ? bm[i * p + c] / pv : 0.0;
  }
  __syncthreads();
  return info;
}

__device__ __forceinline__ void eta_maps(float raw, float& eta, float& slope) {
  const double scale = 1.0 - 1.1920928955078125e-7;  // 1 - FP32 epsilon
  const double x = (double)raw;
  eta = (float)(scale * tanh(x));
  const double q = exp(-2.0 * fabs(x));
  slope = (float)(scale * 4.0 * q / ((1.0 + q) * (1.0 + q)));
}

__global__ void __launch_bounds__(kCompactThreads)
core_forward_kernel(const float* __restrict__ base_raw, const float* __restrict__ eta_raw, int r,
                    int complement, float* __restrict__ eta_out, float* __restrict__ slope_out,
                    float* __restrict__ core_map, int* __restrict__ core_info) {
  extern __shared__ double dsm[];
  __shared__ int s_piv[2];
  const int h = blockIdx.x, tid = threadIdx.x;
  if (tid == 0) {
    float e, s;
    eta_maps(eta_raw[h], e, s);
    eta_out[h] = e;
    slope_out[h] = s;
    core_info[h] = 0;
  }
  if (complement) return;
  const int p = r + 1;
  double* am = dsm;                  // (r+1) rows: last row is elimination scratch
  double* bm = am + (r + 1) * p;
  double* lc = bm + r * p;
  build_generator(base_raw + (size_t)h * r * r, r, lc, bm, tid, kCompactThreads);  // bm <- J
  for (int i = tid; i < r * r; i += kCompactThreads) {
    const int row = i / r, col = i - row * r;
    const double j = bm[row * p + col];
    const double id = row == col ? 1.0 : 0.0;
    am[row * p + col] = id + j;
    bm[row * p + col] = id - j;
  }
  __syncthreads();
  const int info = gauss_jordan(am, bm, r, s_piv, tid, kCompactThreads);
  for (int i = tid; i < r * r; i += kCompactThreads) {
    const int row = i / r, col = i - row * r;
    core_map[(size_t)h * r * r + i] = (float)bm[row * p + col];
  }
  if (tid == 0 && info) core_info[h] = info;
}

// ---------------------------------------------------------------------------------------
// Cholesky inverse factor, one matrix row per lane, FP64 registers
// ---------------------------------------------------------------------------------------
// gs: symmetric-part source G (FP32, pitch R) in shared memory.  Writes T = chol(I+G)^-1
// (lower triangular, FP32, pitch R+1) to ts.  Executed by the first ceil(R/32) warps; the
// elimination is Gaussian (unit-lower factor applied to the identity, in place), followed by
// a row scaling with the inverse square roots of the pivots.
template <int R, int K>
__device__ __forceinline__ void cholesky_eliminate(double (&a)[R], double* rowbuf, int i, bool live) {
  // one elimination step per template instance so that every register index is a constant
  if constexpr (K < R) {
    constexpr int NW = (R + 31) / 32;
    double* rb = rowbuf + (K & 1) * R;
    if (i == K) {
#pragma unroll
      for (int j = 0; j < R; ++j) rb[j] = a[j];
    }
    if (NW == 1) __syncwarp();
    else asm volatile("bar.sync 1, %0;\n" ::"n"(NW * 32));
    if (live && i > K) {
      const double f = a[K] / rb[K];
#pragma unroll
      for (int j = 0; j < R; ++j) {
        if (j != K) a[j] = fma(-f, rb[j], a[j]);
      }
      a[K] = -f;
    }
    cholesky_eliminate<R, K + 1>(a, rowbuf, i, live);
  }
}

template <int R>
__device__ __forceinline__ void cholesky_inverse_rows(const float* gs, float* ts, double* rowbuf, int tid) {
  constexpr int NW = (R + 31) / 32;
  if (tid >= NW * 32) return;
  const int i = tid;
  const bool live = i < R;
  double a[R];
#pragma unroll
  for (int j = 0; j < R; ++j) {
    double v = 0.0;
    if (live) v = 0.5 * ((double)gs[i * R + j] + (double)gs[j * R + i]) + (i == j ? 1.0 : 0.0);
    a[j] = v;
  }
  cholesky_eliminate<R, 0>(a, rowbuf, i, live);
  if (live) {
    // pivot of row i sits at a[i]; select it without a dynamic register index
    double piv = 1.0;
#pragma unroll
    for (int j = 0; j < R; ++j) piv = (j == i) ? a[j] : piv;
    const double sc = 1.0 / sqrt(piv);
#pragma unroll
    for (int j = 0; j < R; ++j) {
      float v = 0.f;
      if (j < i) v = (float)(a[j] * sc);
      else if (j == i) v = (float)sc;
      ts[i * (R + 1) + j] = v;
    }
  }
}

// ---------------------------------------------------------------------------------------
// small FP32 products on shared-memory operands: out[i][c] = sum_j lhs(i,j) * rhs[j][c]
// for i < R, c < 64 (rhs/out pitch 65).  jlo/jhi bound the inner index (triangular factors).
// ---------------------------------------------------------------------------------------
template <int R, class LHS, class LO, class HI>
__device__ __forceinline__ void small_mm(LHS lhs, LO jlo, HI jhi, const float* rhs, float* out, int tid) {
  const int c = tid & 63;
  for (int i = tid >> 6; i < R; i += kCompactThreads / 64) {
    float acc = 0.f;
    const int j1 = jhi(i);
    for (int j = jlo(i); j < j1; ++j) acc = fmaf(lhs(i, j), rhs[j * 65 + c], acc);
    out[i * 65 + c] = acc;
  }
}

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
  float* gs = fsm;                      // R*R            symmetric-part source
  float* ts = gs + R * R;               // R*(R+1)        T
  float* ms_ = ts + R * (R + 1);        // R*(R+1)        F - eta I
  float* qs = ms_ + R * (R + 1);        // R*65           Q block -> Z block
  float* mid = qs + R * 65;             // R*65
  double* rowbuf = reinterpret_cast<double*>(mid + R * 65);  // 2*R doubles

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

  for (int i = tid; i < R * R; i += kCompactThreads) {
    float v = 0.f;
    for (int c = 0; c < nch; ++c) v += src[(size_t)c * p.pf + i];
    gs[i] = v * inv_n;
    const int row = i / R, col = i - row * R;
    float f = p.complement ? 0.f : p.core_map[(size_t)h * R * R + i];
    if (row == col) f -= eta;
    ms_[row * (R + 1) + col] = f;
  }
  __syncthreads();
  cholesky_inverse_rows<R>(gs, ts, rowbuf, tid);
  __syncthreads();
  for (int i = tid; i < R * R; i += kCompactThreads) {
    const int row = i / R, col = i - row * R;
    p.inverse[(size_t)sys * R * R + i] = ts[row * (R + 1) + col];
  }

  const int d = p.head_dim;
  for (int jb = 0; jb < p.dblocks; ++jb) {
    const int d0 = jb * 64, dv = min(64, d - d0);
    for (int i = tid; i < R * 64; i += kCompactThreads) {
      const int row = i >> 6, c = i & 63;
      float v = 0.f;
      if (c < dv) {
        const size_t off = (size_t)R * R + (size_t)row * d + d0 + c;
        for (int k = 0; k < nch; ++k) v += src[(size_t)k * p.pf + off];
        v *= inv_s;
      }
      qs[row * 65 + c] = v;
    }
    __syncthreads();
    // Z = T Q   (T lower triangular)
    small_mm<R>([&](int i, int j) { return ts[i * (R + 1) + j]; }, [](int) { return 0; },
                [](int i) { return i + 1; }, qs, mid, tid);
    __syncthreads();
    for (int i = tid; i < R * 64; i += kCompactThreads) {
      const int row = i >> 6, c = i & 63;
      if (c < dv) p.state[((size_t)sys * R + row) * d + d0 + c] = mid[row * 65 + c];
    }
    // mid2 = (F - eta I) Z  -> qs
    small_mm<R>([&](int i, int j) { return ms_[i * (R + 1) + j]; }, [](int) { return 0; },
                [](int) { return R; }, mid, qs, tid);
    __syncthreads();
    // W = T^T mid2 -> mid
    small_mm<R>([&](int i, int j) { return ts[j * (R + 1) + i]; }, [](int i) { return i; },
                [](int) { return R; }, qs, mid, tid);
    __syncthreads();
    // split into two BF16 words, pitch dpad, zero padding
    __nv_bfloat16* hi = p.coeff + (size_t)sys * 2 * R * p.dpad;
    __nv_bfloat16* lo = hi + (size_t)R * p.dpad;
    const int cend = min(64, p.dpad - d0);
    for (int i = tid; i < R * 64; i += kCompactThreads) {
      const int row = i >> 6, c = i & 63;
      if (c < cend) {
        const float v = c < dv ? mid[row * 65 + c] : 0.f;
        const __nv_bfloat16 hv = __float2bfloat16_rn(v);
        hi[(size_t)row * p.dpad + d0 + c] = hv;
        lo[(size_t)row * p.dpad + d0 + c] = __float2bfloat16_rn(v - __bfloat162float(hv));
      }
    }
    __syncthreads();
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

  for (int i = tid; i < R * R; i += kCompactThreads) {
    const int row = i / R, col = i - row * R;
    ts[row * P + col] = p.inverse[(size_t)sys * R * R + i];
    float f = p.complement ? 0.f : p.core_map[(size_t)h * R * R + i];
    if (row == col) f -= eta;
    mm[row * P + col] = f;
    hm[row * P + col] = 0.f;
  }
  if (tid == 0) {
    float v = 0.f;
    if (packed) {
      v = p.partials[(size_t)p.systems * p.pf + sys];
    } else {
      for (int c = 0; c < p.chunks * p.dblocks; ++c) v += p.de_partials[(size_t)sys * p.chunks * p.dblocks + c];
    }
    p.de_sys[sys] = v;
  }
  __syncthreads();

  for (int jb = 0; jb < p.dblocks; ++jb) {
    const int d0 = jb * 64, dv = min(64, d - d0);
    for (int i = tid; i < R * 64; i += kCompactThreads) {
      const int row = i >> 6, c = i & 63;
      float v = 0.f, z = 0.f;
      if (c < dv) {
        const size_t off = (size_t)row * d + d0 + c;
        for (int k = 0; k < nch; ++k) v += src[(size_t)k * p.pf + off];
        v *= inv_s;
        z = p.state[(size_t)sys * R * d + off];
      }
      es[row * 65 + c] = v;
      zs[row * 65 + c] = z;
    }
    __syncthreads();
    // U = T E
    small_mm<R>([&](int i, int j) { return ts[i * P + j]; }, [](int) { return 0; },
                [](int i) { return i + 1; }, es, us, tid);
    __syncthreads();
    // H += U Z^T   (r x r, contraction over the 64 channels)
    for (int i = tid; i < R * R; i += kCompactThreads) {
      const int row = i / R, col = i - row * R;
      float acc = hm[row * P + col];
#pragma unroll 8
      for (int c = 0; c < 64; ++c) acc = fmaf(us[row * 65 + c], zs[col * 65 + c], acc);
      hm[row * P + col] = acc;
    }
    // dZ = M^T U -> es
    small_mm<R>([&](int i, int j) { return mm[j * P + i]; }, [](int) { return 0; },
                [](int) { return R; }, us, es, tid);
    __syncthreads();
    // dQ = T^T dZ -> zs
    small_mm<R>([&](int i, int j) { return ts[j * P + i]; }, [](int i) { return i; },
                [](int) { return R; }, es, zs, tid);
    __syncthreads();
    __nv_bfloat16* hi = p.cross_grad + (size_t)sys * 2 * R * p.dpad;
    __nv_bfloat16* lo = hi + (size_t)R * p.dpad;
    const int cend = min(64, p.dpad - d0);
    for (int i = tid; i < R * 64; i += kCompactThreads) {
      const int row = i >> 6, c = i & 63;
      if (c < cend) {
        const float v = c < dv ? zs[row * 65 + c] : 0.f;
        const __nv_bfloat16 hv = __float2bfloat16_rn(v);
        hi[(size_t)row * p.dpad + d0 + c] = hv;
        lo[(size_t)row * p.dpad + d0 + c] = __float2bfloat16_rn(v - __bfloat162float(hv));
      }
    }
    __syncthreads();
  }

  // H to global for the per-head sum; X = -M H^T - M^T H
  float* xs = es;   // R*P fits in R*65
  float* ys = us;
  for (int i = tid; i < R * R; i += kCompactThreads) {
    const int row = i / R, col = i - row * R;
    p.hmat[(size_t)sys * R * R + i] = hm[row * P + col];
    float acc = 0.f;
    for (int k = 0; k < R; ++k) {
      acc = fmaf(-mm[row * P + k], hm[col * P + k], acc);
      acc = fmaf(-mm[k * P + row], hm[k * P + col], acc);
    }
    xs[row * P + col] = acc;
  }
  __syncthreads();
  // sym = low + low^T with low = tril(X,-1)/2 + diag(X)/4;   Y = sym T
  for (int i = tid; i < R * R; i += kCompactThreads) {
    const int row = i / R, col = i - row * R;
    float acc = 0.f;
    for (int k = col; k < R; ++k) {
      float s;
      if (row > k) s = 0.5f * xs[row * P + k];
      else if (row < k) s = 0.5f * xs[k * P + row];
      else s = 0.5f * xs[row * P + row];
      acc = fmaf(s, ts[k * P + col], acc);
    }
    ys[row * P + col] = acc;
  }
  __syncthreads();
  // dG = T^T Y ;  stored as dG + dG^T (dG is symmetric) in two BF16 words
  __nv_bfloat16* ghi = p.gram_grad + (size_t)sys * 2 * R * R;
  __nv_bfloat16* glo = ghi + R * R;
  for (int i = tid; i < R * R; i += kCompactThreads) {
    const int row = i / R, col = i - row * R;
    float acc = 0.f, acct = 0.f;
    for (int k = row; k < R; ++k) acc = fmaf(ts[k * P + row], ys[k * P + col], acc);
    for (int k = col; k < R; ++k) acct = fmaf(ts[k * P + col], ys[k * P + row], acct);
    const float v = acc + acct;
    const __nv_bfloat16 hv = __float2bfloat16_rn(v);
    ghi[i] = hv;
    glo[i] = __float2bfloat16_rn(v - __bfloat162float(hv));
  }
}

// ---------------------------------------------------------------------------------------
// per-head core adjoint
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kCompactThreads)
core_backward_kernel(const float* __restrict__ base_raw, const float* __restrict__ hmat,
                     const float* __restrict__ de_sys, const float* __restrict__ slope,
                     const float* __restrict__ core_map, int r, int heads, int batch, int complement,
                     float grad_scale, float* __restrict__ d_base, float* __restrict__ d_eta_raw) {
  extern __shared__ double dsm[];
  __shared__ int s_piv[2];
  __shared__ double s_red[kCompactThreads / 32];
  const int h = blockIdx.x, tid = threadIdx.x;
  const int p = r + 1;
  double* am = dsm;                 // (r+1) rows
  double* bm = am + (r + 1) * p;    // dF -> V
  double* lc = bm + r * p;          // L
  double* jm = lc + r * p;          // J, later dJ

  // dF = sum over the batch, fixed order
  double tr = 0.0;
  for (int i = tid; i < r * r; i += kCompactThreads) {
    const int row = i / r, col = i - row * r;
    float acc = 0.f;
    for (int b = 0; b < batch; ++b) acc += hmat[((size_t)b * heads + h) * r * r + i];
    bm[row * p + col] = (double)acc;
    if (row == col) tr += (double)acc;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) tr += __shfl_xor_sync(0xffffffffu, tr, o);
  if ((tid & 31) == 0) s_red[tid >> 5] = tr;
  __syncthreads();
  if (tid == 0) {
    double t = 0.0;
    for (int w = 0; w < kCompactThreads / 32; ++w) t += s_red[w];
    float de = 0.f;
    for (int b = 0; b < batch; ++b) de += de_sys[(size_t)b * heads + h];
    d_eta_raw[h] = (float)(((double)de - t) * (double)slope[h]) * grad_scale;
  }
  if (complement) return;

  build_generator(base_raw + (size_t)h * r * r, r, lc, jm, tid, kCompactThreads);
  for (int i = tid; i < r * r; i += kCompactThreads) {
    const int row = i / r, col = i - row * r;
    am[row * p + col] = (row == col ? 1.0 : 0.0) + jm[col * p + row];  // (I + J)^T
  }
  __syncthreads();
  gauss_jordan(am, bm, r, s_piv, tid, kCompactThreads);  // bm <- V
  // dJ = -V (F + I)^T
  for (int i = tid; i < r * r; i += kCompactThreads) {
    const int row = i / r, col = i - row * r;
    double acc = 0.0;
    for (int k = 0; k < r; ++k) {
      const double f = (double)core_map[(size_t)h * r * r + col * r + k] + (col == k ? 1.0 : 0.0);
      acc = fma(bm[row * p + k], f, acc);
    }
    jm[row * p + col] = -acc;
  }
  __syncthreads();
  // dL = (dJ + dJ^T) L ;  d base = tril(dL,-1) + diag(dL)*sigmoid + triu(dJ - dJ^T, 1)
  for (int i = tid; i < r * r; i += kCompactThreads) {
    const int row = i / r, col = i - row * r;
    double out;
    if (row < col) {
      out = jm[row * p + col] - jm[col * p + row];
    } else {
      double acc = 0.0;
      for (int k = col; k < r; ++k) acc = fma(jm[row * p + k] + jm[k * p + row], lc[k * p + col], acc);
      if (row == col) {
        const double x = (double)base_raw[(size_t)h * r * r + i] + kSoftplusShift;
        acc *= 1.0 / (1.0 + exp(-x));
      }
      out = acc;
    }
    d_base[(size_t)h * r * r + i] = (float)out * grad_scale;
  }
}

// ---------------------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------------------
static size_t core_smem_bytes(int r, bool backward) {
  const size_t p = r + 1;
  return ((r + 1) * p + r * p * (backward ? 3 : 2)) * sizeof(double);
}

template <class K>
static int set_smem(K kern, size_t bytes) {
  if (bytes > 48 * 1024) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) != cudaSuccess)
      return MS_ERR_LAUNCH;
  }
  return MS_OK;
}

int launch_core_forward(const ms_shape& s, const float* base_raw, const float* eta_raw, const ms_tape& t,
                        cudaStream_t st) {
  const size_t bytes = core_smem_bytes(s.rank, false);
  if (set_smem(core_forward_kernel, bytes)) return MS_ERR_LAUNCH;
  core_forward_kernel<<<s.heads, kCompactThreads, bytes, st>>>(base_raw, eta_raw, s.rank, s.complement,
                                                              t.eta, t.eta_slope, t.core_map, t.core_info);
  return cudaGetLastError() == cudaSuccess ? MS_OK : MS_ERR_LAUNCH;
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
  const size_t bytes = core_smem_bytes(s.rank, true);
  if (set_smem(core_backward_kernel, bytes)) return MS_ERR_LAUNCH;
  core_backward_kernel<<<s.heads, kCompactThreads, bytes, st>>>(base_raw, hmat, de_sys, t.eta_slope,
                                                               t.core_map, s.rank, s.heads, s.batch,
                                                               s.complement, grad_scale, d_base, d_eta_raw);
  return cudaGetLastError() == cudaSuccess ? MS_OK : MS_ERR_LAUNCH;
}

}  // namespace ms
