// Per-head core of the MemSolve mixer as device functions, usable from a kernel of their own
// or from spare CTAs of a streaming kernel's grid.
//
//   forward:  eta = (1-eps) tanh(eta_raw), slope = d eta / d eta_raw,
//             L = tril(U,-1) + diag(softplus(diag U + c0)),  J = L L^T + triu(U,1) - triu(U,1)^T,
//             F = (I+J)^-1 (I-J) = 2 (I+J)^-1 - I
//   backward: dF = sum_b H_b, d eta_raw = (sum_b de_b - tr dF) * slope,
//             V = (I+J)^-T dF with (I+J)^-1 = (F+I)/2,  dJ = -V (F+I)^T,
//             dL = (dJ + dJ^T) L,  dU = tril(dL,-1) + diag(dL) sigmoid(diag U + c0) + triu(dJ - dJ^T, 1)
//
// Replaces the reference's `complement`, `core_forward`, `compact_lu`, `compact_getrs`,
// `eta_trace` and `core_backward` (memsolve/ball/cuda.py:2281-2360, 2517-2527;
// csrc/ball/solvers.cuh:227-560).  The inverse of I+J is a Gauss-Jordan elimination with partial
// pivoting in FP32, one matrix row per lane held in registers (rows are never moved between
// lanes, the pivot order is recorded instead), polished by two Newton-Schulz steps
// X <- X + X (I - A X) in FP64 carried out by the whole CTA; the generator J itself is FP64.
#pragma once

#include "ms_common.cuh"

namespace ms {

constexpr float kSoftplusShiftF = 0.5413248546129181f;  // log(expm1(1))

__device__ __forceinline__ double softplus_shifted(float u) {
  const float x = u + kSoftplusShiftF;
  return (double)(x > 20.f ? x : log1pf(expf(x)));
}

// L -> lc, J -> jm (FP64, pitch r+1).  All threads of the CTA take part.
__device__ __forceinline__ void build_generator(const float* __restrict__ base, int r, double* lc, double* jm,
                                                int tid, int nthreads) {
  const int p = r + 1;
  for (int i = tid; i < r * r; i += nthreads) {
    const int row = i / r, col = i - row * r;
    double v = 0.0;
    if (row > col) v = (double)base[i];
    else if (row == col) v = softplus_shifted(base[i]);
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

__device__ __forceinline__ void eta_maps(float raw, float& eta, float& slope) {
  const float scale = 1.0f - 1.1920928955078125e-7f;  // 1 - FP32 epsilon
  eta = scale * tanhf(raw);
  const float q = expf(-2.0f * fabsf(raw));
  slope = scale * 4.0f * q / ((1.0f + q) * (1.0f + q));
}

struct GjShared {
  float* rowbuf;    // 2 * R floats
  float* cand_v;    // 2 floats    (cross-warp pivot candidates)
  int* cand_i;      // 2 ints
  int* piv;         // R ints      pivot lane of step k
};

// Run-time loop over the elimination steps; the row registers are rotated by one after every
// step, so the pivot column is always register 0 and all register indices stay compile-time
// constants while the loop body fits the instruction cache.
template <int R>
__device__ __forceinline__ void gj_eliminate(float (&a)[R], const GjShared& sh, int lane_id, bool live, bool& used,
                                             int& my_step, int& info) {
  constexpr int NW = (R + 31) / 32;
#pragma unroll 1
  for (int K = 0; K < R; ++K) {
    float v = (live && !used) ? fabsf(a[0]) : -1.0f;
    int best = lane_id;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int ob = __shfl_xor_sync(0xffffffffu, best, o);
      if (ov > v || (ov == v && ob < best)) { v = ov; best = ob; }
    }
    if (NW > 1) {
      const int w = lane_id >> 5;
      if ((lane_id & 31) == 0) { sh.cand_v[w] = v; sh.cand_i[w] = best; }
      asm volatile("bar.sync 1, %0;\n" ::"n"(NW * 32));
      const float v0 = sh.cand_v[0], v1 = sh.cand_v[1];
      const int i0 = sh.cand_i[0], i1 = sh.cand_i[1];
      if (v1 > v0) { v = v1; best = i1; } else { v = v0; best = i0; }
    }
    if (v == 0.0f && info == 0) info = K + 1;
    float* rb = sh.rowbuf + (K & 1) * R;
    if (lane_id == best) {
      const float inv = __frcp_rn(a[0]);
      a[0] = 1.0f;
#pragma unroll
      for (int j = 0; j < R; ++j) {
        a[j] *= inv;
        rb[j] = a[j];
      }
      used = true;
      my_step = K;
      sh.piv[K] = lane_id;
    }
    if (NW == 1) __syncwarp();
    else asm volatile("bar.sync 1, %0;\n" ::"n"(NW * 32));
    if (live && lane_id != best) {
      const float f = a[0];
      a[0] = 0.0f;
#pragma unroll
      for (int j = 0; j < R; ++j) a[j] = fmaf(-f, rb[j], a[j]);
    }
    const float first = a[0];
#pragma unroll
    for (int j = 0; j + 1 < R; ++j) a[j] = a[j + 1];
    a[R - 1] = first;
  }
}

// Approximate (FP32) inverse of the R x R matrix `src` (FP64, pitch R+1) into `dst` (FP64, pitch
// R+1); run by the first ceil(R/32) warps of the CTA (the other threads return at once).
// Returns 0, or k+1 when the k-th pivot was exactly zero.
template <int R>
__device__ __noinline__ int gj_inverse(const double* src, double* dst, const GjShared sh, int tid) {
  constexpr int NW = (R + 31) / 32;
  if (tid >= NW * 32) return 0;
  const bool live = tid < R;
  float a[R];
#pragma unroll
  for (int j = 0; j < R; ++j) a[j] = live ? (float)src[tid * (R + 1) + j] : 0.0f;
  bool used = false;
  int my_step = 0, info = 0;
  gj_eliminate<R>(a, sh, tid, live, used, my_step, info);
  if (NW == 1) __syncwarp();
  else asm volatile("bar.sync 1, %0;\n" ::"n"(NW * 32));
  // this lane holds row `my_step` of (P A)^-1; column k of it is column piv[k] of A^-1
  if (live) {
#pragma unroll
    for (int k = 0; k < R; ++k) dst[my_step * (R + 1) + sh.piv[k]] = (double)a[k];
  }
  return info;
}

__host__ __device__ constexpr size_t core_forward_smem_bytes(int r) {
  // A = I+J, X, residual (FP64) + row buffers + pivot bookkeeping
  return (size_t)(3 * r * (r + 1)) * sizeof(double) + (size_t)(2 * r + 2) * sizeof(float) +
         (size_t)(r + 2) * sizeof(int) + 32;
}

// One CTA computes one head.  `smem` must provide core_forward_smem_bytes(R), 8-byte aligned.
template <int R>
__device__ __forceinline__ void core_forward_device(const float* __restrict__ base_raw,
                                                    const float* __restrict__ eta_raw, int h, int complement,
                                                    float* __restrict__ eta_out, float* __restrict__ slope_out,
                                                    float* __restrict__ core_map, int* __restrict__ core_info,
                                                    unsigned char* smem, int tid, int nthreads) {
  if (tid == nthreads - 1) {
    float e, s;
    eta_maps(eta_raw[h], e, s);
    eta_out[h] = e;
    slope_out[h] = s;
    core_info[h] = 0;
  }
  if (complement) return;
  constexpr int P = R + 1;
  double* am = reinterpret_cast<double*>(smem);  // I + J
  double* xm = am + R * P;                       // L, then the inverse
  double* rm = xm + R * P;                       // Newton-Schulz residual
  GjShared sh;
  sh.rowbuf = reinterpret_cast<float*>(rm + R * P);
  sh.cand_v = sh.rowbuf + 2 * R;
  sh.cand_i = reinterpret_cast<int*>(sh.cand_v + 2);
  sh.piv = sh.cand_i + 2;
  MS_TICK(20);
  build_generator(base_raw + (size_t)h * R * R, R, xm, am, tid, nthreads);
  for (int i = tid; i < R; i += nthreads) am[i * P + i] += 1.0;   // I + J
  __syncthreads();
  MS_TICK(21);
  const int info = gj_inverse<R>(am, xm, sh, tid);   // xm <- FP32-accurate inverse
  __syncthreads();
  MS_TICK(22);
#pragma unroll 1
  for (int sweep = 0; sweep < 2; ++sweep) {
    // residual = I - A X
    for (int i = tid; i < R * R; i += nthreads) {
      const int row = i / R, col = i - row * R;
      double acc = row == col ? 1.0 : 0.0;
      for (int k = 0; k < R; ++k) acc = fma(-am[row * P + k], xm[k * P + col], acc);
      rm[row * P + col] = acc;
    }
    __syncthreads();
    // X <- X + X residual   (each thread keeps its entries until all reads of X are done)
    constexpr int PER = (R * R + 127) / 128;   // callers run at least 128 threads
    double upd[PER];
#pragma unroll
    for (int e = 0; e < PER; ++e) {
      const int i = tid + e * nthreads;
      double acc = 0.0;
      if (i < R * R) {
        const int row = i / R, col = i - row * R;
        acc = xm[row * P + col];
        for (int k = 0; k < R; ++k) acc = fma(xm[row * P + k], rm[k * P + col], acc);
      }
      upd[e] = acc;
    }
    __syncthreads();
#pragma unroll
    for (int e = 0; e < PER; ++e) {
      const int i = tid + e * nthreads;
      if (i < R * R) xm[(i / R) * P + (i % R)] = upd[e];
    }
    __syncthreads();
  }
  MS_TICK(23);
  for (int i = tid; i < R * R; i += nthreads) {
    const int row = i / R, col = i - row * R;
    core_map[(size_t)h * R * R + i] = (float)(2.0 * xm[row * P + col] - (row == col ? 1.0 : 0.0));
  }
  if (tid == 0 && info) core_info[h] = info;
}

__host__ __device__ constexpr size_t core_backward_smem_bytes(int r) {
  return (size_t)(4 * r * (r + 1)) * sizeof(double) + 64 * sizeof(double);
}

// One CTA computes the parameter gradients of one head.  `smem`: core_backward_smem_bytes(r).
__device__ __forceinline__ void core_backward_device(const float* __restrict__ base_raw,
                                                     const float* __restrict__ hmat,
                                                     const float* __restrict__ de_sys,
                                                     const float* __restrict__ slope,
                                                     const float* __restrict__ core_map, int r, int h, int heads,
                                                     int batch, int complement, float grad_scale,
                                                     float* __restrict__ d_base, float* __restrict__ d_eta_raw,
                                                     unsigned char* smem, int tid, int nthreads) {
  const int p = r + 1;
  double* pm = reinterpret_cast<double*>(smem);  // F + I
  double* dfm = pm + r * p;                      // dF, later dJ
  double* t1 = dfm + r * p;                      // (F+I)^T dF
  double* lc = t1 + r * p;                       // L
  double* red = lc + r * p;                      // 64 doubles

  // dF = sum over the batch in fixed order; trace; <dY, C>
  double tr = 0.0;
  for (int i = tid; i < r * r; i += nthreads) {
    const int row = i / r, col = i - row * r;
    float acc = 0.f;
    for (int b = 0; b < batch; ++b) acc += hmat[((size_t)b * heads + h) * r * r + i];
    dfm[row * p + col] = (double)acc;
    if (row == col) tr += (double)acc;
    if (!complement) {
      pm[row * p + col] = (double)core_map[(size_t)h * r * r + i] + (row == col ? 1.0 : 0.0);
      double v = 0.0;
      if (row > col) v = (double)base_raw[(size_t)h * r * r + i];
      else if (row == col) v = softplus_shifted(base_raw[(size_t)h * r * r + i]);
      lc[row * p + col] = v;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) tr += __shfl_xor_sync(0xffffffffu, tr, o);
  if ((tid & 31) == 0) red[tid >> 5] = tr;
  __syncthreads();
  if (tid < 32) {
    // fixed-order sum of de over the batch: lane-strided partial sums, then a shuffle tree
    float de = 0.f;
    for (int b = tid; b < batch; b += 32) de += de_sys[(size_t)b * heads + h];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) de += __shfl_xor_sync(0xffffffffu, de, o);
    if (tid == 0) {
      double t = 0.0;
      for (int w = 0; w < (nthreads >> 5); ++w) t += red[w];
      d_eta_raw[h] = (float)(((double)de - t) * (double)slope[h]) * grad_scale;
    }
  }
  if (complement) return;

  // t1 = (F+I)^T dF ;  dJ = -1/2 t1 (F+I)^T
  for (int i = tid; i < r * r; i += nthreads) {
    const int row = i / r, col = i - row * r;
    double acc = 0.0;
    for (int k = 0; k < r; ++k) acc = fma(pm[k * p + row], dfm[k * p + col], acc);
    t1[row * p + col] = acc;
  }
  __syncthreads();
  for (int i = tid; i < r * r; i += nthreads) {
    const int row = i / r, col = i - row * r;
    double acc = 0.0;
    for (int k = 0; k < r; ++k) acc = fma(t1[row * p + k], pm[col * p + k], acc);
    dfm[row * p + col] = -0.5 * acc;   // dJ
  }
  __syncthreads();
  for (int i = tid; i < r * r; i += nthreads) {
    const int row = i / r, col = i - row * r;
    double out;
    if (row < col) {
      out = dfm[row * p + col] - dfm[col * p + row];
    } else {
      double acc = 0.0;
      for (int k = col; k < r; ++k) acc = fma(dfm[row * p + k] + dfm[k * p + row], lc[k * p + col], acc);
      if (row == col) {
        const float x = base_raw[(size_t)h * r * r + i] + kSoftplusShiftF;
        acc *= (double)(1.0f / (1.0f + expf(-x)));
      }
      out = acc;
    }
    d_base[(size_t)h * r * r + i] = (float)out * grad_scale;
  }
}

}  // namespace ms
