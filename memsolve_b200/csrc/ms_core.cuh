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
// csrc/ball/solvers.cuh:227-560).  The inverse of I+J is a Gauss-Jordan elimination in FP32 by the
// whole CTA (no pivoting: the symmetric part of I+J is positive definite), polished by one
// Newton-Schulz step X <- X + X (I - A X) in FP64; the generator J itself is FP64.  All matrix
// products run on 4 x 2 register tiles with vector loads from shared memory.
#pragma once

#include "ms_common.cuh"

namespace ms {

constexpr float kSoftplusShiftF = 0.5413248546129181f;  // log(expm1(1))

__device__ __forceinline__ double softplus_shifted(float u) {
  const float x = u + kSoftplusShiftF;
  return (double)(x > 20.f ? x : log1pf(expf(x)));
}

__device__ __forceinline__ void eta_maps(float raw, float& eta, float& slope) {
  const float scale = 1.0f - 1.1920928955078125e-7f;  // 1 - FP32 epsilon
  eta = scale * tanhf(raw);
  const float q = expf(-2.0f * fabsf(raw));
  slope = scale * 4.0f * q / ((1.0f + q) * (1.0f + q));
}

// ---------------------------------------------------------------------------------------
// small products on shared-memory operands, 4 x 2 register tiles, FP64 accumulation
// ---------------------------------------------------------------------------------------
// acc[r][c] += sum_{k < K} X[i0 + r][k] * Y[j(c)][k],  j(0) = j0, j(1) = j1   (K even)
template <class TY>
__device__ __forceinline__ void core_mm_nt(double (&acc)[4][2], const double* X, int ldx, const TY* Y, int ldy,
                                           int i0, int j0, int j1, int K) {
#pragma unroll 2
  for (int k = 0; k < K; k += 2) {
    double2 x[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) x[r] = *reinterpret_cast<const double2*>(X + (i0 + r) * ldx + k);
    double y0[2], y1[2];
    y0[0] = (double)Y[j0 * ldy + k]; y0[1] = (double)Y[j0 * ldy + k + 1];
    y1[0] = (double)Y[j1 * ldy + k]; y1[1] = (double)Y[j1 * ldy + k + 1];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      acc[r][0] = fma(x[r].x, y0[0], acc[r][0]);
      acc[r][0] = fma(x[r].y, y0[1], acc[r][0]);
      acc[r][1] = fma(x[r].x, y1[0], acc[r][1]);
      acc[r][1] = fma(x[r].y, y1[1], acc[r][1]);
    }
  }
}

// acc[r][c] += sum_{k < K} At[k][i0 + r] * B[k][j0 + c]     (At FP32, B FP64)
__device__ __forceinline__ void core_mm_tn(double (&acc)[4][2], const float* At, int lda, const double* B, int ldb,
                                           int i0, int j0, int K) {
#pragma unroll 4
  for (int k = 0; k < K; ++k) {
    const float4 a = *reinterpret_cast<const float4*>(At + k * lda + i0);
    const double2 b = *reinterpret_cast<const double2*>(B + k * ldb + j0);
    const double av[4] = {(double)a.x, (double)a.y, (double)a.z, (double)a.w};
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      acc[r][0] = fma(av[r], b.x, acc[r][0]);
      acc[r][1] = fma(av[r], b.y, acc[r][1]);
    }
  }
}

// acc[a][b] += sum_{k < r} A(i0 + a, k) B(k, j0 + b js) for FP64 matrices in shared memory with element strides
// (sai, sak) and (sbk, sbj): either operand may be read transposed
__device__ __forceinline__ void core_mm44(double (&acc)[4][4], const double* A, int sai, int sak, const double* B,
                                          int sbk, int sbj, int i0, int j0, int js, int r) {
#pragma unroll 2
  for (int k = 0; k < r; ++k) {
    double a[4], b[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      a[e] = A[(i0 + e) * sai + k * sak];
      b[e] = B[k * sbk + (j0 + e * js) * sbj];
    }
#pragma unroll
    for (int x = 0; x < 4; ++x)
#pragma unroll
      for (int y = 0; y < 4; ++y) acc[x][y] = fma(a[x], b[y], acc[x][y]);
  }
}

// layout of the core forward: NT threads, TPR neighbouring threads share one matrix row
template <int R, int NT>
struct CoreDims {
  static constexpr int Q = NT / R;
  static constexpr int TPR = Q >= 16 ? 16 : (Q >= 8 ? 8 : (Q >= 4 ? 4 : (Q >= 2 ? 2 : 1)));
  static constexpr int CPT = R / TPR;
  static constexpr int P2 = R + 2;    // pitch in doubles of the FP64 matrices (16-byte aligned rows)
  static constexpr int RP = R + 4;    // pitch in floats of the FP32 matrix
  static_assert(R * TPR <= NT && CPT * TPR == R, "core layout");
};

__host__ __device__ constexpr size_t core_forward_smem_bytes(int r) {
  // A = I+J and one scratch matrix (FP64), the FP32 inverse, two pivot rows, the pivot flag
  return (size_t)(2 * r * (r + 2)) * sizeof(double) + (size_t)(r * (r + 4) + 2 * (r + 4) + 4) * sizeof(float);
}

// In-place Gauss-Jordan inverse in FP32 by the whole CTA, without pivoting: I + J has a positive
// definite symmetric part (I + L L^T), for which elimination in the natural order is stable.
// Row i lives in the registers of TPR neighbouring lanes (columns q, q + TPR, ...).  Per step the
// owners of the pivot row scale and publish it (double buffered, one CTA barrier per step); the
// entry of each row in the next pivot column reaches the row's lanes by a shuffle inside the
// group, which also hands the next pivot to the owners of the next pivot row.
// a[] holds (I+J) on entry and its inverse on return; *zero_pivot is set to k+1 if pivot k is zero.
template <int R, int NT>
__device__ __forceinline__ void gj_inverse_cta(float (&a)[CoreDims<R, NT>::CPT], float* rowbuf, int* zero_pivot,
                                               int tid) {
  using D = CoreDims<R, NT>;
  constexpr int TPR = D::TPR, CPT = D::CPT;
  const int i = tid / TPR, q = tid % TPR;
  const bool active = i < R;
  const int lane = tid & 31;
  const int group_base = lane & ~(TPR - 1);

  // scale and publish pivot row k: `pivot` is the row's entry in column k
  auto publish = [&](int k, int cK, int buf, float pivot) {
    if (active && i == k) {
      if (pivot == 0.0f) atomicMin(zero_pivot, k + 1);
      float r0;
      asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r0) : "f"(pivot));
      const float inv = fmaf(r0, fmaf(-pivot, r0, 1.0f), r0);
#pragma unroll
      for (int c = 0; c < CPT; ++c) {
        a[c] = (c == cK && q == k % TPR) ? inv : a[c] * inv;
        rowbuf[buf * (R + 4) + q + TPR * c] = a[c];
      }
    }
  };
  float f = __shfl_sync(0xffffffffu, a[0], group_base);   // entry of this row in column 0
  publish(0, 0, 0, f);
#pragma unroll
  for (int cK = 0; cK < CPT; ++cK) {
    for (int qK = 0; qK < TPR; ++qK) {
      const int K = cK * TPR + qK;
      __syncthreads();
      const float* rb = rowbuf + (K & 1) * (R + 4);
      if (active && i != K) {
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
          const float rv = rb[q + TPR * c];
          a[c] = (c == cK && q == qK) ? -f * rv : fmaf(-f, rv, a[c]);
        }
      }
      if (K + 1 < R) {
        const float sel = (qK + 1 < TPR) ? a[cK] : a[cK + 1 < CPT ? cK + 1 : cK];
        f = __shfl_sync(0xffffffffu, sel, group_base + (qK + 1) % TPR);
        publish(K + 1, (qK + 1 < TPR) ? cK : cK + 1, (K + 1) & 1, f);
      }
    }
  }
}

// One CTA of NT threads computes one head.  `smem` must provide core_forward_smem_bytes(R),
// 16-byte aligned.
template <int R, int NT>
__device__ __forceinline__ void core_forward_device(const float* __restrict__ base_raw,
                                                    const float* __restrict__ eta_raw, int h, int complement,
                                                    float* __restrict__ eta_out, float* __restrict__ slope_out,
                                                    float* __restrict__ core_map, int* __restrict__ core_info,
                                                    unsigned char* smem, int tid) {
  using D = CoreDims<R, NT>;
  constexpr int P2 = D::P2, RP = D::RP, TPR = D::TPR, CPT = D::CPT;
  if (tid == NT - 1) {
    float e, s;
    eta_maps(eta_raw[h], e, s);
    eta_out[h] = e;
    slope_out[h] = s;
  }
  if (complement) {
    if (tid == 0) core_info[h] = 0;
    return;
  }
  double* am = reinterpret_cast<double*>(smem);   // I + J
  double* rm = am + R * P2;                       // L, then the Newton-Schulz residual
  float* xt = reinterpret_cast<float*>(rm + R * P2);   // transpose of the FP32 inverse
  float* rowbuf = xt + R * RP;                    // 2 * (R + 4)
  int* zero_pivot = reinterpret_cast<int*>(rowbuf + 2 * (R + 4));
  const float* base = base_raw + (size_t)h * R * R;

  // L = tril(U,-1) + diag(softplus(diag U + c0))
  for (int idx = tid; idx < R * R; idx += NT) {
    const int row = idx / R, col = idx - row * R;
    double v = 0.0;
    if (row > col) v = (double)base[idx];
    else if (row == col) v = softplus_shifted(base[idx]);
    rm[row * P2 + col] = v;
  }
  if (tid == 0) *zero_pivot = R + 1;
  __syncthreads();
  // A = I + L L^T + triu(U,1) - triu(U,1)^T
  constexpr int RTILES = (R / 4) * (R / 2);
  for (int tile = tid; tile < RTILES; tile += NT) {
    const int i0 = (tile / (R / 2)) * 4, j0 = tile % (R / 2), j1 = j0 + R / 2;
    double acc[4][2] = {};
    // L is lower triangular: the inner index stops at the smaller of row and column
    const int kend = min(R, (min(i0 + 3, j1) + 2) & ~1);
    core_mm_nt(acc, rm, P2, rm, P2, i0, j0, j1, kend);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int row = i0 + r;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int col = c == 0 ? j0 : j1;
        double v = acc[r][c];
        if (row < col) v += (double)base[row * R + col];
        if (row > col) v -= (double)base[col * R + row];
        if (row == col) v += 1.0;
        am[row * P2 + col] = v;
      }
    }
  }
  __syncthreads();

  // FP32 inverse
  {
    const int i = tid / TPR, q = tid % TPR;
    float a[CPT];
#pragma unroll
    for (int c = 0; c < CPT; ++c) a[c] = i < R ? (float)am[i * P2 + q + TPR * c] : 0.f;
    gj_inverse_cta<R, NT>(a, rowbuf, zero_pivot, tid);
    if (i < R) {
#pragma unroll
      for (int c = 0; c < CPT; ++c) xt[(q + TPR * c) * RP + i] = a[c];
    }
  }
  __syncthreads();

  // one Newton-Schulz step in FP64:  X <- X + X (I - A X)
  for (int tile = tid; tile < RTILES; tile += NT) {
    const int i0 = (tile / (R / 2)) * 4, j0 = tile % (R / 2), j1 = j0 + R / 2;
    double acc[4][2] = {};
    core_mm_nt(acc, am, P2, xt, RP, i0, j0, j1, R);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      rm[(i0 + r) * P2 + j0] = (i0 + r == j0 ? 1.0 : 0.0) - acc[r][0];
      rm[(i0 + r) * P2 + j1] = (i0 + r == j1 ? 1.0 : 0.0) - acc[r][1];
    }
  }
  __syncthreads();
  for (int tile = tid; tile < RTILES; tile += NT) {
    const int i0 = (tile / (R / 2)) * 4, j0 = (tile % (R / 2)) * 2;
    double acc[4][2] = {};
    core_mm_tn(acc, xt, RP, rm, P2, i0, j0, R);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int row = i0 + r, col = j0 + c;
        const double x = (double)xt[col * RP + row] + acc[r][c];
        core_map[(size_t)h * R * R + row * R + col] = (float)(2.0 * x - (row == col ? 1.0 : 0.0));
      }
    }
  }
  if (tid == 0) core_info[h] = *zero_pivot <= R ? *zero_pivot : 0;
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
  // (four consecutive entries per thread; eight samples in flight, their sums combined in a fixed tree, so
  // that a large batch costs batch / 8 round trips to L2 instead of batch)
  double tr = 0.0;
  for (int q = tid; q < (r * r) / 4; q += nthreads) {
    const float4* src = reinterpret_cast<const float4*>(hmat + (size_t)h * r * r) + q;
    const size_t step = (size_t)heads * r * r / 4;
    float4 part[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) part[u] = make_float4(0.f, 0.f, 0.f, 0.f);
    int b = 0;
    for (; b + 8 <= batch; b += 8) {
      float4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = src[(size_t)(b + u) * step];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        part[u].x += v[u].x; part[u].y += v[u].y; part[u].z += v[u].z; part[u].w += v[u].w;
      }
    }
    for (; b < batch; ++b) {
      const float4 v = src[(size_t)b * step];
      part[0].x += v.x; part[0].y += v.y; part[0].z += v.z; part[0].w += v.w;
    }
    float sum4[4];
    sum4[0] = ((part[0].x + part[1].x) + (part[2].x + part[3].x)) + ((part[4].x + part[5].x) + (part[6].x + part[7].x));
    sum4[1] = ((part[0].y + part[1].y) + (part[2].y + part[3].y)) + ((part[4].y + part[5].y) + (part[6].y + part[7].y));
    sum4[2] = ((part[0].z + part[1].z) + (part[2].z + part[3].z)) + ((part[4].z + part[5].z) + (part[6].z + part[7].z));
    sum4[3] = ((part[0].w + part[1].w) + (part[2].w + part[3].w)) + ((part[4].w + part[5].w) + (part[6].w + part[7].w));
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = 4 * q + e, row = i / r, col = i - row * r;
      dfm[row * p + col] = (double)sum4[e];
      if (row == col) tr += (double)sum4[e];
    }
  }
  for (int i = tid; i < r * r; i += nthreads) {
    const int row = i / r, col = i - row * r;
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

  // t1 = (F+I)^T dF ;  dJ = -1/2 t1 (F+I)^T ;  then L's gradient from S = dJ + dJ^T: FP64 products on 4 x 4
  // register tiles (rows i0 .. i0 + 3, columns tj + b r/4: the lanes of a warp read neighbouring columns)
  const int q4 = r / 4, ntiles = q4 * q4;
  for (int tile = tid; tile < ntiles; tile += nthreads) {
    const int i0 = (tile / q4) * 4, tj = tile % q4;
    double acc[4][4] = {};
    core_mm44(acc, pm, 1, p, dfm, p, 1, i0, tj, q4, r);
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b) t1[(i0 + a) * p + tj + b * q4] = acc[a][b];
  }
  __syncthreads();
  for (int tile = tid; tile < ntiles; tile += nthreads) {
    const int i0 = (tile / q4) * 4, tj = tile % q4;
    double acc[4][4] = {};
    core_mm44(acc, t1, p, 1, pm, 1, p, i0, tj, q4, r);
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b) dfm[(i0 + a) * p + tj + b * q4] = -0.5 * acc[a][b];   // dJ
  }
  __syncthreads();
  for (int i = tid; i < r * r; i += nthreads) {
    const int row = i / r, col = i - row * r;
    t1[row * p + col] = dfm[row * p + col] + dfm[col * p + row];   // S
  }
  __syncthreads();
  for (int tile = tid; tile < ntiles; tile += nthreads) {
    const int i0 = (tile / q4) * 4, tj = tile % q4;
    double acc[4][4] = {};
    // L is lower triangular with zeros stored above the diagonal: the full inner range adds nothing for k < col
    core_mm44(acc, t1, p, 1, lc, p, 1, i0, tj, q4, r);
#pragma unroll
    for (int a = 0; a < 4; ++a) {
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const int row = i0 + a, col = tj + b * q4;
        double out;
        if (row < col) {
          out = dfm[row * p + col] - dfm[col * p + row];
        } else {
          out = acc[a][b];
          if (row == col) {
            const float x = base_raw[(size_t)h * r * r + row * r + col] + kSoftplusShiftF;
            out *= (double)(1.0f / (1.0f + expf(-x)));
          }
        }
        d_base[(size_t)h * r * r + row * r + col] = (float)out * grad_scale;
      }
    }
  }
}

}  // namespace ms
