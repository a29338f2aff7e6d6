// Sequence-parallel exchange of the token statistics through peer memory.
//
// One launch does what the sequence-parallel path otherwise does in three steps (reduce the
// per-chunk partials of the local tokens, all-reduce over the ranks, hand the result to the
// compact stage): every rank reduces its partials into its own exchange area, tells its peers,
// waits for theirs and adds the values of all ranks in rank order, so that every rank gets the
// same bits.  The reference uses one NCCL all-reduce for this step
// (integrations/distributed.py:47-50 of the reference, called from memsolve/ball/cuda.py:3165-3215).
//
// Exchange area of one rank (device memory that every peer can address, e.g. a symmetric-memory
// allocation; all ranks use the same layout):
//
//   float    data[2][capacity]            values of this rank, double buffered by call parity
//   uint32   flags[kMaxRanks][kCtas]      flags[r][c] = number of the last call whose slice c rank r has published
//   uint32   call, done                   number of completed calls; thread blocks finished in this call
//
// Thread block c owns slice c of the value vector on every rank, so blocks of one GPU never wait
// for each other: block c publishes its slice, raises flags[me][c] on every peer (after a
// system-wide fence), waits until its own flags[r][c] have reached this call's number for every
// peer r and then reads slice c of every peer with loads that bypass the caches.  The wait is bounded
// by wall-clock time (peer_wait_ns(), 20 s unless ms_set_peer_wait_ms or MEMSOLVE_PEER_WAIT_MS says
// otherwise): a block whose peer has not arrived by then sets the library's error word to 0x200 and
// writes NaN instead of sums, so a late or dead rank can never turn into plausible-looking numbers.  Double buffering makes one
// barrier per call sufficient: a rank can only publish call k+2 into the buffer of call k after
// all peers have raised their flags of call k+1, i.e. after their kernels of call k have ended.
// All loads of peer memory are plain loads; no multicast object, no TMA.
#include "ms_common.cuh"

namespace ms {

constexpr int kExCtas = 128;         // thread blocks = slices of the value vector (one vector of four per thread at rank 64)
constexpr int kExThreads = 256;
constexpr int kExMaxRanks = 8;
constexpr int kErrPeerTimeout = 0x200;

int* device_error_word();
unsigned long long peer_wait_ns();   // ms_api.cu: the limit set by ms_set_peer_wait_ms / MEMSOLVE_PEER_WAIT_MS

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

struct ExchangeParams {
  const float* partials;
  const float* de_partials;
  const float* counts;
  float* out;
  float* areas[kExMaxRanks];
  int* error;
  unsigned long long wait_ns;
  int world, rank, capacity;
  int heads, tokens, chunks, de_slots, gram_floats, pf, systems, grad, total;
};

__device__ __forceinline__ unsigned ld_flag(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_flag(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Polls `flag` until it has reached `call`; false when `wait_ns` nanoseconds went by first.  The clock is
// read once per 64 polls.
__device__ __forceinline__ bool wait_flag(const unsigned* flag, unsigned call, unsigned long long wait_ns) {
  if ((int)(ld_flag(flag) - call) >= 0) return true;
  const unsigned long long t0 = global_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if ((int)(ld_flag(flag) - call) >= 0) return true;
    if (global_ns() - t0 > wait_ns) return false;
  }
}
__device__ __forceinline__ float4 ld_peer4(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p));
  return v;
}

// value vector in units of four floats: [systems * pf / 4] statistics, then the <dY, C> sums
// (adjoint only), padded with zeros to a multiple of four
__device__ __forceinline__ float4 reduce_partials4(const ExchangeParams& p, int i4) {
  const int i = 4 * i4, body = p.systems * p.pf;
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  if (i < body) {
    // pf and the size of the Gram part are multiples of four: one scale per vector
    const int sys = i / p.pf, e = i - sys * p.pf;
    const float n = p.counts ? p.counts[sys / p.heads] : (float)p.tokens;
    const float4* src = reinterpret_cast<const float4*>(p.partials + (size_t)sys * p.chunks * p.pf + e);
    const int stride4 = p.pf >> 2;
    // chunk order is kept; eight loads are in flight at a time (a trip to L2 per round: with the twenty-odd
    // partials of a long sequence the rounds are what this kernel waits for)
    int k = 0;
    for (; k + 8 <= p.chunks; k += 8) {
      float4 t[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) t[u] = __ldg(src + (size_t)(k + u) * stride4);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        v.x += t[u].x; v.y += t[u].y; v.z += t[u].z; v.w += t[u].w;
      }
    }
    if (k < p.chunks) {
      float4 t[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        t[u] = k + u < p.chunks ? __ldg(src + (size_t)(k + u) * stride4) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (k + u < p.chunks) {
          v.x += t[u].x; v.y += t[u].y; v.z += t[u].z; v.w += t[u].w;
        }
      }
    }
    const float scale = e < p.gram_floats ? inv_rn(n) : inv_sqrt_rn(n);
    v.x *= scale; v.y *= scale; v.z *= scale; v.w *= scale;
  } else {
    float out[4] = {0.f, 0.f, 0.f, 0.f};
    const int cnt = p.chunks * p.de_slots;
    for (int q = 0; q < 4; ++q) {
      const int sys = i + q - body;
      if (sys < p.systems) {
        // index order is kept; eight loads in flight at a time (one thread adds a system's few dozen values, and
        // one load per trip to L2 made this the longest path of the adjoint exchange)
        const float* src = p.de_partials + (size_t)sys * cnt;
        int k = 0;
        for (; k + 8 <= cnt; k += 8) {
          float t[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) t[u] = __ldg(src + k + u);
#pragma unroll
          for (int u = 0; u < 8; ++u) out[q] += t[u];
        }
        for (; k < cnt; ++k) out[q] += __ldg(src + k);
      }
    }
    v = make_float4(out[0], out[1], out[2], out[3]);
  }
  return v;
}

constexpr int kExVecs = 2;   // vectors of four values per thread and pass

__global__ void __launch_bounds__(kExThreads) exchange_kernel(const ExchangeParams p) {
  __shared__ int s_ok;
  const int tid = threadIdx.x, c = blockIdx.x;
  float* mine = p.areas[p.rank];
  unsigned* my_flags = reinterpret_cast<unsigned*>(mine + 2 * (size_t)p.capacity);
  unsigned* state = my_flags + kExMaxRanks * kExCtas;   // [0] = completed calls, [1] = finished blocks
  const unsigned call = *reinterpret_cast<volatile unsigned*>(state) + 1u;
  const size_t buf = (size_t)(call & 1u) * p.capacity;

  // slice of this block in vectors of four values
  const int total4 = (p.total + 3) >> 2;
  const int per = (total4 + kExCtas - 1) / kExCtas;
  const int lo = min(total4, c * per), hi = min(total4, lo + per);

  // 1. reduce the partials of the local tokens (chunk order) and scale: 1/n for the Gram part,
  //    1/sqrt(n) for the moments; the <dY, C> sums follow the moments of all systems
  for (int i4 = lo + tid; i4 < hi; i4 += kExThreads)
    *reinterpret_cast<float4*>(mine + buf + 4 * (size_t)i4) = reduce_partials4(p, i4);
  if (tid == 0) s_ok = 1;
  __syncthreads();

  // 2. publish: flags[me][c] = call on every peer (the release store orders the block's values,
  //    which this thread has observed through the barrier, before the flag); then wait for the
  //    peers' slices
  if (tid < p.world && tid != p.rank) {
    unsigned* theirs = reinterpret_cast<unsigned*>(p.areas[tid] + 2 * (size_t)p.capacity);
    st_flag(theirs + p.rank * kExCtas + c, call);
    if (!wait_flag(my_flags + tid * kExCtas + c, call, p.wait_ns)) s_ok = 0;
  }
  __syncthreads();
  const bool arrived = s_ok != 0;
  if (!arrived && tid == 0) atomicExch(p.error, kErrPeerTimeout);
  const float poison = __int_as_float(0x7fc00000);

  // 3. add the slices of all ranks in rank order; all peer loads of a pass are in flight together
  for (int base = lo + tid; base < hi; base += kExThreads * kExVecs) {
    float4 vals[kExVecs][kExMaxRanks];
#pragma unroll
    for (int v = 0; v < kExVecs; ++v) {
      const int i4 = base + v * kExThreads;
#pragma unroll
      for (int r = 0; r < kExMaxRanks; ++r) {
        vals[v][r] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i4 < hi && r < p.world) {
          const float* src = p.areas[r] + buf + 4 * (size_t)i4;
          vals[v][r] = r == p.rank ? *reinterpret_cast<const float4*>(src) : ld_peer4(src);
        }
      }
    }
#pragma unroll
    for (int v = 0; v < kExVecs; ++v) {
      const int i4 = base + v * kExThreads;
      if (i4 < hi) {
        float4 acc = vals[v][0];
#pragma unroll
        for (int r = 1; r < kExMaxRanks; ++r) {
          if (r < p.world) {
            acc.x += vals[v][r].x; acc.y += vals[v][r].y; acc.z += vals[v][r].z; acc.w += vals[v][r].w;
          }
        }
        if (!arrived) acc = make_float4(poison, poison, poison, poison);   // a peer never published this slice
        float* dst = p.out + 4 * (size_t)i4;
        if (4 * i4 + 3 < p.total) {
          *reinterpret_cast<float4*>(dst) = acc;
        } else {
          const float a[4] = {acc.x, acc.y, acc.z, acc.w};
          for (int q = 0; q < 4 && 4 * i4 + q < p.total; ++q) dst[q] = a[q];
        }
      }
    }
  }

  // 4. the last block of this call advances the call number
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(state + 1, 1u) == gridDim.x - 1) {
      state[1] = 0u;
      __threadfence();
      *reinterpret_cast<volatile unsigned*>(state) = call;
    }
  }
}

// ---------------------------------------------------------------------------------------
// in-place SUM of a vector over the ranks (parameter gradients of the replicated weights)
// ---------------------------------------------------------------------------------------
// Same areas and flag protocol as above, two rounds per call: the vector is cut into `world`
// slices, rank r adds slice r of all ranks (round 1) and every rank then collects the summed slices
// from their owners (round 2), so each value crosses NVLink twice instead of world-1 times.
// Thread block c handles portion c of every slice on every rank.  Area layout for this use:
//
//   float   data[2][capacity]      this rank's values                 (double buffered by call parity)
//   float   summed[2][capacity]    slice `rank` after round 1, at its position in the vector
//   uint32  flags[2][kMaxRanks][kSumCtas], call, done
// few thread blocks, many loads in flight per thread: the SUM runs beside GEMMs that want every SM
constexpr int kSumCtas = 16;
constexpr int kSumBatch = 8;   // vectors per thread whose peer loads are in flight together

struct PeerSumParams {
  float* values;
  float* areas[kExMaxRanks];
  int* error;
  unsigned long long wait_ns;
  int world, rank, capacity, total4;   // total4: vector length in units of four values
};

__device__ __forceinline__ bool flag_round(const PeerSumParams& p, unsigned* my_flags, int round, unsigned call, int c,
                                           int tid, int* s_ok) {
  // values written by the block before this point are published by the release store of the flag
  __syncthreads();
  if (tid < p.world && tid != p.rank) {
    unsigned* theirs = reinterpret_cast<unsigned*>(p.areas[tid] + 4 * (size_t)p.capacity) +
                       round * kExMaxRanks * kSumCtas;
    st_flag(theirs + p.rank * kSumCtas + c, call);
    // after a first timeout the later rounds do not wait again
    if (*s_ok && !wait_flag(my_flags + round * kExMaxRanks * kSumCtas + tid * kSumCtas + c, call, p.wait_ns))
      *s_ok = 0;
  }
  __syncthreads();
  return *s_ok != 0;
}

__global__ void __launch_bounds__(kExThreads) peer_sum_kernel(const PeerSumParams p) {
  __shared__ int s_ok;
  const int tid = threadIdx.x, c = blockIdx.x;
  float* mine = p.areas[p.rank];
  unsigned* my_flags = reinterpret_cast<unsigned*>(mine + 4 * (size_t)p.capacity);
  unsigned* state = my_flags + 2 * kExMaxRanks * kSumCtas;
  const unsigned call = *reinterpret_cast<volatile unsigned*>(state) + 1u;
  const size_t data = (size_t)(call & 1u) * p.capacity;
  const size_t summed = (size_t)(2 + (call & 1u)) * p.capacity;
  if (tid == 0) s_ok = 1;

  // slice s = vectors [s * slice4, (s+1) * slice4); portion c of a slice = [c * part4, (c+1) * part4) within it
  const int slice4 = (p.total4 + p.world - 1) / p.world;
  const int part4 = (slice4 + kSumCtas - 1) / kSumCtas;
  const int plo = min(slice4, c * part4), phi = min(slice4, plo + part4);

  // 0. copy this rank's values into its area
  for (int s = 0; s < p.world; ++s) {
    for (int j = plo + tid; j < phi; j += kExThreads) {
      const int i4 = s * slice4 + j;
      if (i4 < p.total4)
        *reinterpret_cast<float4*>(mine + data + 4 * (size_t)i4) =
            *reinterpret_cast<const float4*>(p.values + 4 * (size_t)i4);
    }
  }
  flag_round(p, my_flags, 0, call, c, tid, &s_ok);

  // 1. slice `rank`: add the values of all ranks in rank order (kSumBatch vectors per thread at a time)
  for (int base = plo + tid; base < phi; base += kExThreads * kSumBatch) {
    float4 acc[kSumBatch];
#pragma unroll
    for (int v = 0; v < kSumBatch; ++v) acc[v] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < p.world; ++r) {
      float4 t[kSumBatch];
#pragma unroll
      for (int v = 0; v < kSumBatch; ++v) {
        const int j = base + v * kExThreads, i4 = p.rank * slice4 + j;
        t[v] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (j < phi && i4 < p.total4) {
          const float* src = p.areas[r] + data + 4 * (size_t)i4;
          t[v] = r == p.rank ? *reinterpret_cast<const float4*>(src) : ld_peer4(src);
        }
      }
#pragma unroll
      for (int v = 0; v < kSumBatch; ++v) {
        acc[v].x += t[v].x; acc[v].y += t[v].y; acc[v].z += t[v].z; acc[v].w += t[v].w;
      }
    }
#pragma unroll
    for (int v = 0; v < kSumBatch; ++v) {
      const int j = base + v * kExThreads, i4 = p.rank * slice4 + j;
      if (j < phi && i4 < p.total4) {
        *reinterpret_cast<float4*>(mine + summed + 4 * (size_t)i4) = acc[v];
        *reinterpret_cast<float4*>(p.values + 4 * (size_t)i4) = acc[v];
      }
    }
  }
  flag_round(p, my_flags, 1, call, c, tid, &s_ok);
  if (!s_ok && tid == 0) atomicExch(p.error, kErrPeerTimeout);

  // 2. collect the other slices from their owners
  for (int s = 0; s < p.world; ++s) {
    if (s == p.rank) continue;
    for (int base = plo + tid; base < phi; base += kExThreads * kSumBatch) {
      float4 t[kSumBatch];
#pragma unroll
      for (int v = 0; v < kSumBatch; ++v) {
        const int j = base + v * kExThreads, i4 = s * slice4 + j;
        if (j < phi && i4 < p.total4) t[v] = ld_peer4(p.areas[s] + summed + 4 * (size_t)i4);
      }
#pragma unroll
      for (int v = 0; v < kSumBatch; ++v) {
        const int j = base + v * kExThreads, i4 = s * slice4 + j;
        if (j < phi && i4 < p.total4) *reinterpret_cast<float4*>(p.values + 4 * (size_t)i4) = t[v];
      }
    }
  }

  if (!s_ok) {
    // a peer did not arrive in time: this block's part of every slice becomes NaN instead of a partial sum
    const float poison = __int_as_float(0x7fc00000);
    for (int s = 0; s < p.world; ++s)
      for (int j = plo + tid; j < phi; j += kExThreads) {
        const int i4 = s * slice4 + j;
        if (i4 < p.total4)
          *reinterpret_cast<float4*>(p.values + 4 * (size_t)i4) = make_float4(poison, poison, poison, poison);
      }
  }

  __syncthreads();
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(state + 1, 1u) == gridDim.x - 1) {
      state[1] = 0u;
      __threadfence();
      *reinterpret_cast<volatile unsigned*>(state) = call;
    }
  }
}

size_t peer_sum_area_bytes(size_t capacity_floats) {
  return (4 * capacity_floats + 2 * (size_t)kExMaxRanks * kSumCtas + 4) * sizeof(float);
}

int launch_peer_sum(float* values, size_t count, void* const* areas, size_t area_bytes, int world, int rank,
                    cudaStream_t st) {
  if (world < 1 || world > kExMaxRanks || rank < 0 || rank >= world || !areas || !values) return MS_ERR_INVALID_ARGUMENT;
  if ((count & 3u) != 0 || (reinterpret_cast<uintptr_t>(values) & 15u) != 0) return MS_ERR_INVALID_ARGUMENT;
  const size_t fixed = peer_sum_area_bytes(0);
  if (area_bytes < fixed + 64) return MS_ERR_WORKSPACE;
  const size_t capacity = ((area_bytes - fixed) / (4 * sizeof(float))) & ~size_t(3);
  if (count > capacity || count > 0x7ffffff0u) return MS_ERR_WORKSPACE;
  PeerSumParams p;
  p.values = values;
  for (int r = 0; r < kExMaxRanks; ++r) p.areas[r] = r < world ? static_cast<float*>(areas[r]) : nullptr;
  for (int r = 0; r < world; ++r)
    if (!p.areas[r] || (reinterpret_cast<uintptr_t>(p.areas[r]) & 15u)) return MS_ERR_INVALID_ARGUMENT;
  p.error = device_error_word();
  if (!p.error) return MS_ERR_LAUNCH;
  p.world = world; p.rank = rank; p.capacity = (int)capacity; p.total4 = (int)(count >> 2);
  p.wait_ns = peer_wait_ns();
  if (count == 0) return MS_OK;
  peer_sum_kernel<<<kSumCtas, kExThreads, 0, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? MS_OK : MS_ERR_LAUNCH;
}

size_t exchange_area_bytes(size_t capacity_floats) {
  return (2 * capacity_floats + (size_t)kExMaxRanks * kExCtas + 4) * sizeof(float);
}

int launch_exchange(const ms_shape& s, const Plan& plan, bool grad, const float* partials, const float* de_partials,
                    const float* counts, void* const* areas, int world, int rank, size_t capacity_floats,
                    float* out, cudaStream_t st) {
  if (world < 1 || world > kExMaxRanks || rank < 0 || rank >= world || !areas) return MS_ERR_INVALID_ARGUMENT;
  ExchangeParams p;
  p.partials = partials; p.de_partials = de_partials; p.counts = counts; p.out = out;
  for (int r = 0; r < kExMaxRanks; ++r) p.areas[r] = r < world ? static_cast<float*>(areas[r]) : nullptr;
  for (int r = 0; r < world; ++r)
    if (!p.areas[r] || (reinterpret_cast<uintptr_t>(p.areas[r]) & 15u)) return MS_ERR_INVALID_ARGUMENT;
  p.error = device_error_word();
  if (!p.error) return MS_ERR_LAUNCH;
  p.world = world; p.rank = rank;
  p.wait_ns = peer_wait_ns();
  p.heads = s.heads; p.tokens = s.tokens; p.chunks = plan.chunks; p.de_slots = plan.de_slots;
  p.gram_floats = grad ? 0 : s.rank * s.rank;
  p.pf = (int)(grad ? plan.bwd_partial_floats : plan.fwd_partial_floats);
  p.systems = plan.systems; p.grad = grad ? 1 : 0;
  const size_t total = (size_t)plan.systems * p.pf + (grad ? plan.systems : 0);
  if (total > capacity_floats || total > 0x7fffffffu) return MS_ERR_WORKSPACE;
  p.total = (int)total; p.capacity = (int)capacity_floats;
  exchange_kernel<<<kExCtas, kExThreads, 0, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? MS_OK : MS_ERR_LAUNCH;
}

}  // namespace ms
