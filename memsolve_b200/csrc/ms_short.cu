// Sequences with no more tokens than the rank (N <= r <= 64): token-space evaluation of the eta term.
//
// With A = A_raw / sqrt(n), C' = rot(C) and S = I_N + A A^T (N x N), the layer's output in the rotated domain is
//
//   Y' = eta S^-1 C' + A Wc,     Wc = T^T F Z                      (Y = rot^-1 Y')
//
// because A (I + A^T A)^-1 A^T = I - S^-1.  The rank-space kernels evaluate the same thing as
// eta C' + A T^T (F - eta I) Z, i.e. eta (C' - P P^T C') as a difference; when N < r and the relations are strong
// P P^T is close to the identity on the token space and that difference -- and d_eta = <dY, C> - tr dF in the
// backward -- cancels catastrophically.  The reference switches to the token-space system for N <= r for the same
// reason (memsolve/ball/cuda.py:3230-3926: `short_stats`, `short_readout`, `short_bwd_*`).  Here the rank-space
// statistics and compact kernels still produce T, Z and the core part (they are run with eta = 0, so that
// W = Wc, dQ, dG carry the core part only); the two kernels below replace readout and token backward:
//
//   forward   X = S^-1 C' (Cholesky of S and two triangular solves in FP64), Y' = eta X + A Wc
//   backward  Xd = S^-1 rot(dY);  d_eta = <rot(dY), X>;  dC' = eta Xd + A dQ;
//             dA_raw = s ( A_raw S' + rot(dY) Wc^T + C' dQ^T - eta (Xd X^T + X Xd^T) A )
//
// One CTA per (sample, head); everything lives in shared memory (N, r <= 64; channels in blocks of 64).  These
// shapes are tiny: the kernels are written for accuracy and clarity, not for bandwidth.
#include "ms_common.cuh"

namespace ms {

constexpr int kShortThreads = 256;
constexpr int kSP = 65;   // pitch of the 64 x 64 shared-memory matrices

struct ShortParams {
  const __nv_bfloat16* projected;
  const __nv_bfloat16* dy;
  const float* cos;
  const float* sin;
  const float* counts;
  const float* eta;
  const __nv_bfloat16* coeff;       // [systems][2][r][dpad]   Wc (two words)
  const __nv_bfloat16* gram_grad;   // [systems][2][r][r]      s (dG + dG^T)
  const __nv_bfloat16* cross_grad;  // [systems][2][r][dpad]   dQ
  __nv_bfloat16* out;               // mixed [B, N, H*d] or dprojected [B, N, H*(r+d)]
  float* de_short;                  // [systems]  <rot(dY), X>
  int tokens, heads, rank, head_dim, dpad, rotary_rows;
};

__device__ __forceinline__ float bf16_at(const __nv_bfloat16* p, size_t i) { return __bfloat162float(p[i]); }

// A (scaled relation rows) and the Cholesky factor L of S = I + A A^T, lower triangular, in FP64
__device__ void short_setup(const ShortParams& p, int b, int h, float s, float* A, double* L, int tid) {
  const int N = p.tokens, r = p.rank, width = p.heads * (p.rank + p.head_dim);
  for (int idx = tid; idx < N * r; idx += kShortThreads) {
    const int i = idx / r, k = idx - i * r;
    A[i * kSP + k] = s * bf16_at(p.projected, ((size_t)b * N + i) * width + h * r + k);
  }
  __syncthreads();
  for (int idx = tid; idx < N * N; idx += kShortThreads) {
    const int i = idx / N, j = idx - i * N;
    double acc = i == j ? 1.0 : 0.0;
    for (int k = 0; k < r; ++k) acc = fma((double)A[i * kSP + k], (double)A[j * kSP + k], acc);
    L[i * kSP + j] = acc;
  }
  __syncthreads();
  for (int j = 0; j < N; ++j) {
    if (tid == 0) L[j * kSP + j] = sqrt(L[j * kSP + j]);
    __syncthreads();
    const double piv = L[j * kSP + j];
    for (int i = j + 1 + tid; i < N; i += kShortThreads) L[i * kSP + j] /= piv;
    __syncthreads();
    const int m = N - j - 1;   // trailing block
    for (int idx = tid; idx < m * m; idx += kShortThreads) {
      const int i = j + 1 + idx / m, k = j + 1 + idx % m;
      if (k <= i) L[i * kSP + k] = fma(-L[i * kSP + j], L[k * kSP + j], L[i * kSP + k]);
    }
    __syncthreads();
  }
}

// column c of B (N rows, pitch kSP) <- S^-1 column, by forward and backward substitution with L
__device__ void short_solve_column(const double* L, float* B, int N, int c) {
  for (int i = 0; i < N; ++i) {
    double v = B[i * kSP + c];
    for (int k = 0; k < i; ++k) v = fma(-L[i * kSP + k], (double)B[k * kSP + c], v);
    B[i * kSP + c] = (float)(v / L[i * kSP + i]);
  }
  for (int i = N - 1; i >= 0; --i) {
    double v = B[i * kSP + c];
    for (int k = i + 1; k < N; ++k) v = fma(-L[k * kSP + i], (double)B[k * kSP + c], v);
    B[i * kSP + c] = (float)(v / L[i * kSP + i]);
  }
}

// rows of a 64-channel block of `src` (row pitch `pitch` elements, first column col0), rotated, into dst
__device__ void short_load_rotated(const ShortParams& p, const __nv_bfloat16* src, size_t pitch, size_t col0, int b, int d0,
                                   int dv, float* dst, int tid) {
  const int N = p.tokens, half = p.head_dim / 2;
  const bool rot = p.rotary_rows > 0;
  const size_t tab_b = p.rotary_rows > 1 ? (size_t)b * N : 0;
  for (int idx = tid; idx < N * 32; idx += kShortThreads) {
    const int i = idx >> 5, j = idx & 31, c = 2 * j;
    float ev = 0.f, od = 0.f;
    if (c < dv) ev = bf16_at(src, ((size_t)b * N + i) * pitch + col0 + d0 + c);
    if (c + 1 < dv) od = bf16_at(src, ((size_t)b * N + i) * pitch + col0 + d0 + c + 1);
    if (rot && c + 1 < dv) {
      const float cv = p.cos[(tab_b + i) * half + d0 / 2 + j], sv = p.sin[(tab_b + i) * half + d0 / 2 + j];
      const float2 r = rot_pair(ev, od, cv, sv);
      ev = r.x;
      od = r.y;
    }
    dst[i * kSP + c] = ev;
    dst[i * kSP + c + 1] = od;
  }
}

// dst (global BF16 rows) <- rot^-1 of the block in `val`
__device__ void short_store_unrotated(const ShortParams& p, const float* val, __nv_bfloat16* dst, size_t pitch, size_t col0, int b,
                                      int d0, int dv, int tid) {
  const int N = p.tokens, half = p.head_dim / 2;
  const bool rot = p.rotary_rows > 0;
  const size_t tab_b = p.rotary_rows > 1 ? (size_t)b * N : 0;
  for (int idx = tid; idx < N * 32; idx += kShortThreads) {
    const int i = idx >> 5, j = idx & 31, c = 2 * j;
    if (c >= dv) continue;
    float ev = val[i * kSP + c], od = val[i * kSP + c + 1];
    if (rot && c + 1 < dv) {
      const float cv = p.cos[(tab_b + i) * half + d0 / 2 + j], sv = p.sin[(tab_b + i) * half + d0 / 2 + j];
      const float2 r = rot_pair(ev, od, cv, -sv);
      ev = r.x;
      od = r.y;
    }
    __nv_bfloat16* o = dst + ((size_t)b * N + i) * pitch + col0 + d0 + c;
    o[0] = __float2bfloat16(ev);
    if (c + 1 < dv) o[1] = __float2bfloat16(od);
  }
}

// a two-word compact matrix block [r][64 columns from d0] -> FP32
__device__ void short_load_words(const __nv_bfloat16* words, int r, int dpad, int d0, int dv, float* dst, int tid) {
  for (int idx = tid; idx < r * 64; idx += kShortThreads) {
    const int k = idx >> 6, c = idx & 63;
    float v = 0.f;
    if (c < dv) v = bf16_at(words, (size_t)k * dpad + d0 + c) + bf16_at(words, (size_t)(r + k) * dpad + d0 + c);
    dst[k * kSP + c] = v;
  }
}

__global__ void __launch_bounds__(kShortThreads) short_readout_kernel(const ShortParams p) {
  extern __shared__ __align__(16) unsigned char ssm[];
  double* L = reinterpret_cast<double*>(ssm);
  float* A = reinterpret_cast<float*>(L + 64 * kSP);
  float* Cb = A + 64 * kSP;
  float* Wb = Cb + 64 * kSP;
  float* Yb = Wb + 64 * kSP;
  grid_launch_dependents();
  grid_dependency_wait();
  const int tid = threadIdx.x, sys = blockIdx.x, b = sys / p.heads, h = sys - b * p.heads;
  const int N = p.tokens, r = p.rank, d = p.head_dim;
  const float n = p.counts ? p.counts[b] : (float)N;
  const float s = inv_sqrt_rn(n), eta = p.eta[h];
  const size_t width = (size_t)p.heads * (r + d), dmodel = (size_t)p.heads * d;
  short_setup(p, b, h, s, A, L, tid);
  for (int d0 = 0; d0 < d; d0 += 64) {
    const int dv = min(64, d - d0);
    short_load_rotated(p, p.projected, width, (size_t)p.heads * r + (size_t)h * d, b, d0, dv, Cb, tid);
    short_load_words(p.coeff + (size_t)sys * 2 * r * p.dpad, r, p.dpad, d0, dv, Wb, tid);
    __syncthreads();
    if (tid < 64) short_solve_column(L, Cb, N, tid);
    __syncthreads();
    for (int idx = tid; idx < N * 64; idx += kShortThreads) {
      const int i = idx >> 6, c = idx & 63;
      float acc = eta * Cb[i * kSP + c];
      for (int k = 0; k < r; ++k) acc = fmaf(A[i * kSP + k], Wb[k * kSP + c], acc);
      Yb[i * kSP + c] = acc;
    }
    __syncthreads();
    short_store_unrotated(p, Yb, p.out, dmodel, (size_t)h * d, b, d0, dv, tid);
    __syncthreads();
  }
}

__global__ void __launch_bounds__(kShortThreads) short_backward_kernel(const ShortParams p) {
  extern __shared__ __align__(16) unsigned char ssm[];
  double* L = reinterpret_cast<double*>(ssm);
  double* Km = L + 64 * kSP;                      // sum over channels of Xd X^T + X Xd^T
  float* A = reinterpret_cast<float*>(Km + 64 * kSP);
  float* dAacc = A + 64 * kSP;                    // rot(dY) Wc^T + C' dQ^T
  float* Cb = dAacc + 64 * kSP;                   // C'
  float* Gb = Cb + 64 * kSP;                      // rot(dY)
  float* Xb = Gb + 64 * kSP;                      // S^-1 C'
  float* Xd = Xb + 64 * kSP;                      // S^-1 rot(dY)
  float* Wb = Xd + 64 * kSP;                      // Wc block
  float* Qb = Wb + 64 * kSP;                      // dQ block
  __shared__ float red[kShortThreads / 32];
  grid_launch_dependents();
  grid_dependency_wait();
  const int tid = threadIdx.x, sys = blockIdx.x, b = sys / p.heads, h = sys - b * p.heads;
  const int N = p.tokens, r = p.rank, d = p.head_dim;
  const float n = p.counts ? p.counts[b] : (float)N;
  const float s = inv_sqrt_rn(n), eta = p.eta[h];
  const size_t width = (size_t)p.heads * (r + d), dmodel = (size_t)p.heads * d;
  short_setup(p, b, h, s, A, L, tid);
  for (int idx = tid; idx < 64 * kSP; idx += kShortThreads) {
    Km[idx] = 0.0;
    dAacc[idx] = 0.f;
  }
  float de = 0.f;
  __syncthreads();
  for (int d0 = 0; d0 < d; d0 += 64) {
    const int dv = min(64, d - d0);
    short_load_rotated(p, p.projected, width, (size_t)p.heads * r + (size_t)h * d, b, d0, dv, Cb, tid);
    short_load_rotated(p, p.dy, dmodel, (size_t)h * d, b, d0, dv, Gb, tid);
    short_load_words(p.coeff + (size_t)sys * 2 * r * p.dpad, r, p.dpad, d0, dv, Wb, tid);
    short_load_words(p.cross_grad + (size_t)sys * 2 * r * p.dpad, r, p.dpad, d0, dv, Qb, tid);
    __syncthreads();
    for (int idx = tid; idx < N * 64; idx += kShortThreads) {
      const int i = idx >> 6, c = idx & 63;
      Xb[i * kSP + c] = Cb[i * kSP + c];
      Xd[i * kSP + c] = Gb[i * kSP + c];
    }
    __syncthreads();
    if (tid < 64) short_solve_column(L, Xb, N, tid);
    else if (tid < 128) short_solve_column(L, Xd, N, tid - 64);
    __syncthreads();
    // d_eta, dC' = eta Xd + A dQ (into Cb's place after its last use below), the two accumulations over channels
    for (int idx = tid; idx < N * 64; idx += kShortThreads) {
      const int i = idx >> 6, c = idx & 63;
      de = fmaf(Gb[i * kSP + c], Xb[i * kSP + c], de);
    }
    for (int idx = tid; idx < N * r; idx += kShortThreads) {
      const int i = idx / r, k = idx - i * r;
      float acc = dAacc[i * kSP + k];
      for (int c = 0; c < 64; ++c) acc = fmaf(Gb[i * kSP + c], Wb[k * kSP + c], fmaf(Cb[i * kSP + c], Qb[k * kSP + c], acc));
      dAacc[i * kSP + k] = acc;
    }
    for (int idx = tid; idx < N * N; idx += kShortThreads) {
      const int i = idx / N, j = idx - i * N;
      double acc = Km[i * kSP + j];
      for (int c = 0; c < 64; ++c)
        acc += (double)Xd[i * kSP + c] * (double)Xb[j * kSP + c] + (double)Xb[i * kSP + c] * (double)Xd[j * kSP + c];
      Km[i * kSP + j] = acc;
    }
    __syncthreads();
    for (int idx = tid; idx < N * 64; idx += kShortThreads) {
      const int i = idx >> 6, c = idx & 63;
      float acc = eta * Xd[i * kSP + c];
      for (int k = 0; k < r; ++k) acc = fmaf(A[i * kSP + k], Qb[k * kSP + c], acc);
      Cb[i * kSP + c] = acc;
    }
    __syncthreads();
    short_store_unrotated(p, Cb, p.out, width, (size_t)p.heads * r + (size_t)h * d, b, d0, dv, tid);
    __syncthreads();
  }
  // dA_raw = s ( A_raw S' + dAacc - eta Km A )
  const __nv_bfloat16* sg = p.gram_grad + (size_t)sys * 2 * r * r;
  for (int idx = tid; idx < N * r; idx += kShortThreads) {
    const int i = idx / r, k = idx - i * r;
    double acc = dAacc[i * kSP + k];
    for (int j = 0; j < r; ++j)
      acc += (double)(A[i * kSP + j] / s) * (double)(bf16_at(sg, (size_t)j * r + k) + bf16_at(sg, (size_t)(r + j) * r + k));
    double corr = 0.0;
    for (int j = 0; j < N; ++j) corr = fma(Km[i * kSP + j], (double)A[j * kSP + k], corr);
    acc -= (double)eta * corr;
    p.out[((size_t)b * N + i) * width + (size_t)h * r + k] = __float2bfloat16((float)(acc * (double)s));
  }
  // <rot(dY), X> of this system: fixed shuffle tree, then the warps in order
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) de += __shfl_xor_sync(0xffffffffu, de, o);
  if ((tid & 31) == 0) red[tid >> 5] = de;
  __syncthreads();
  if (tid == 0) {
    float v = 0.f;
    for (int w = 0; w < kShortThreads / 32; ++w) v += red[w];
    p.de_short[sys] = v;
  }
}

// d_eta_raw[h] = grad_scale * slope[h] * sum over the batch (in order) of <rot(dY), X>
__global__ void short_eta_kernel(const float* __restrict__ de_short, const float* __restrict__ slope, int batch, int heads,
                                 float grad_scale, float* __restrict__ d_eta_raw) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int h = blockIdx.x * blockDim.x + threadIdx.x;
  if (h >= heads) return;
  float v = 0.f;
  for (int b = 0; b < batch; ++b) v += de_short[(size_t)b * heads + h];
  d_eta_raw[h] = v * slope[h] * grad_scale;
}

static ShortParams short_params(const ms_shape& s, const Plan& plan, const void* projected, const void* dy, const float* cos,
                                const float* sin, const float* counts, const ms_tape& t) {
  ShortParams p;
  p.projected = static_cast<const __nv_bfloat16*>(projected);
  p.dy = static_cast<const __nv_bfloat16*>(dy);
  p.cos = cos; p.sin = sin; p.counts = counts; p.eta = t.eta;
  p.coeff = static_cast<const __nv_bfloat16*>(t.coeff);
  p.gram_grad = nullptr; p.cross_grad = nullptr; p.out = nullptr; p.de_short = nullptr;
  p.tokens = s.tokens; p.heads = s.heads; p.rank = s.rank; p.head_dim = s.head_dim; p.dpad = plan.dpad;
  p.rotary_rows = s.rotary_rows;
  return p;
}

int launch_short_readout(const ms_shape& s, const Plan& plan, const void* projected, const float* cos, const float* sin,
                         const float* counts, const ms_tape& t, void* mixed, cudaStream_t st) {
  ShortParams p = short_params(s, plan, projected, nullptr, cos, sin, counts, t);
  p.out = static_cast<__nv_bfloat16*>(mixed);
  const int bytes = 64 * kSP * (int)sizeof(double) + 4 * 64 * kSP * (int)sizeof(float);
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(short_readout_kernel), bytes)) return MS_ERR_LAUNCH;
  launch_kernel(short_readout_kernel, dim3(plan.systems), dim3(kShortThreads), bytes, st, p);
  return cudaGetLastError() == cudaSuccess ? MS_OK : MS_ERR_LAUNCH;
}

int launch_short_backward(const ms_shape& s, const Plan& plan, const void* projected, const void* dy, const float* cos,
                          const float* sin, const float* counts, const ms_tape& t, const void* gram_grad,
                          const void* cross_grad, void* dprojected, float* de_short, float grad_scale, float* d_eta_raw,
                          cudaStream_t st) {
  ShortParams p = short_params(s, plan, projected, dy, cos, sin, counts, t);
  p.gram_grad = static_cast<const __nv_bfloat16*>(gram_grad);
  p.cross_grad = static_cast<const __nv_bfloat16*>(cross_grad);
  p.out = static_cast<__nv_bfloat16*>(dprojected);
  p.de_short = de_short;
  const int bytes = 2 * 64 * kSP * (int)sizeof(double) + 8 * 64 * kSP * (int)sizeof(float);
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(short_backward_kernel), bytes)) return MS_ERR_LAUNCH;
  launch_kernel(short_backward_kernel, dim3(plan.systems), dim3(kShortThreads), bytes, st, p);
  if (cudaGetLastError() != cudaSuccess) return MS_ERR_LAUNCH;
  launch_kernel(short_eta_kernel, dim3((s.heads + 63) / 64), dim3(64), 0, st, (const float*)de_short,
                (const float*)t.eta_slope, s.batch, s.heads, grad_scale, d_eta_raw);
  return cudaGetLastError() == cudaSuccess ? MS_OK : MS_ERR_LAUNCH;
}

}  // namespace ms
