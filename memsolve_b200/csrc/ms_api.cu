// extern "C" entry points of memsolve_equilibrium_sm100.so (declared in include/memsolve_b200.h):
// argument checking, launch planning and the order of kernel launches.  No allocation, no
// host synchronisation; every launch goes to the caller's stream.
#include <atomic>
#include <cstdlib>
#include <mutex>
#include <vector>

#include "ms_tma.cuh"

namespace ms {

int launch_stats(const ms_shape&, const Plan&, bool grad, const void* projected, const void* dy,
                 const float* cos, const float* sin, float* partials, float* de_partials,
                 const float* base_raw, const float* eta_raw, const ms_tape* core_tape, cudaStream_t);
size_t exchange_area_bytes(size_t capacity_floats);
size_t peer_sum_area_bytes(size_t capacity_floats);
int launch_peer_sum(float* values, size_t count, void* const* areas, size_t area_bytes, int world, int rank,
                    cudaStream_t);
int launch_exchange(const ms_shape&, const Plan&, bool grad, const float* partials, const float* de_partials,
                    const float* counts, void* const* areas, int world, int rank, size_t capacity_floats,
                    float* out, cudaStream_t);
int launch_pack_stats(const ms_shape&, const Plan&, bool grad, const float* partials, const float* de_partials,
                      const float* counts, float* packed, cudaStream_t);
int launch_core_forward(const ms_shape&, const float* base_raw, const float* eta_raw, const ms_tape&, cudaStream_t);
int launch_compact_forward(const ms_shape&, const Plan&, const float* counts, const float* partials, bool packed,
                           const ms_tape&, cudaStream_t);
int launch_compact_backward(const ms_shape&, const Plan&, const float* counts, const float* partials,
                            const float* de_partials, bool packed, const ms_tape&, float* hmat, float* de_sys,
                            void* gram_grad, void* cross_grad, cudaStream_t);
int launch_core_backward(const ms_shape&, const float* base_raw, const float* hmat, const float* de_sys,
                         const ms_tape&, float grad_scale, float* d_base, float* d_eta_raw, cudaStream_t);
int launch_readout(const ms_shape&, const Plan&, const void* projected, const float* cos, const float* sin,
                   const float* counts, const ms_tape&, void* mixed, cudaStream_t);
int launch_token_backward(const ms_shape&, const Plan&, const void* projected, const void* dy, const float* cos,
                          const float* sin, const float* counts, const ms_tape&, const void* gram_grad,
                          const void* cross_grad, void* dprojected, const CoreAdjoint* core, cudaStream_t);
int stats_tc_group_heads(int rank);
int launch_linear_tc(long rows, int in_features, int out_features, const void* x, const void* weight, const float* bias,
                     const unsigned char* input_mask, const unsigned char* output_mask, void* out, cudaStream_t);
int launch_short_readout(const ms_shape&, const Plan&, const void* projected, const float* cos, const float* sin,
                         const float* counts, const ms_tape&, void* mixed, cudaStream_t);
int launch_short_backward(const ms_shape&, const Plan&, const void* projected, const void* dy, const float* cos,
                          const float* sin, const float* counts, const ms_tape&, const void* gram_grad,
                          const void* cross_grad, void* dprojected, float* de_short, float grad_scale, float* d_eta_raw,
                          cudaStream_t);
int launch_linear_input_grad_tc(long rows, int in_features, int out_features, const void* dy, const void* weight,
                                const unsigned char* input_mask, const unsigned char* output_mask, void* dx, cudaStream_t);
size_t linear_wgrad_workspace_bytes(long rows, int in_features, int out_features);
int launch_linear_wgrad_tc(long rows, int in_features, int out_features, const void* x, const void* dy, float* dw, float* db,
                           void* workspace, size_t workspace_bytes, cudaStream_t);
int launch_readout_tc(const ms_shape&, const Plan&, const void* projected, const float* cos, const float* sin,
                      const float* counts, const ms_tape&, void* mixed, float* debug, cudaStream_t);
int launch_token_backward_tc(const ms_shape&, const Plan&, const void* projected, const void* dy, const float* cos,
                             const float* sin, const float* counts, const ms_tape&, const void* gram_grad,
                             const void* cross_grad, void* dprojected, const CoreAdjoint* core, float* debug,
                             cudaStream_t);

static std::atomic<int> g_sm_count[64];

int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  int v = g_sm_count[dev].load(std::memory_order_relaxed);
  if (v > 0) return v;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) {
    cudaGetLastError();
    return 148;
  }
  g_sm_count[dev].store(v, std::memory_order_relaxed);
  return v;
}

thread_local bool g_chain_launches = false;

bool chaining_allowed() {
  static const bool allowed = [] {
    const char* v = std::getenv("MEMSOLVE_NO_CHAIN");
    return !(v && v[0] == '1');
  }();
  return allowed;
}

int ensure_dynamic_smem(const void* kernel, int bytes) {
  struct Entry { const void* kernel; int device; int bytes; };
  static std::mutex mu;
  static std::vector<Entry> done;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return MS_ERR_DEVICE;
  std::lock_guard<std::mutex> lock(mu);
  for (const Entry& e : done)
    if (e.kernel == kernel && e.device == dev && e.bytes >= bytes) return MS_OK;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) {
    cudaGetLastError();
    return MS_ERR_LAUNCH;
  }
  done.push_back({kernel, dev, bytes});
  return MS_OK;
}

// ---- TMA tensor maps (driver entry point resolved at run time; libcuda is not linked) ----------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static std::atomic<void*> cached{nullptr};
  void* fn = cached.load(std::memory_order_acquire);
  if (fn) return reinterpret_cast<EncodeTiledFn>(fn);
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess || !fn) {
    cudaGetLastError();
    return nullptr;
  }
  cached.store(fn, std::memory_order_release);
  return reinterpret_cast<EncodeTiledFn>(fn);
}

int encode_tensor_map(CUtensorMap* out, void* base, int elem_bytes, int rank, const uint64_t* dims,
                      const uint64_t* strides_bytes, const uint32_t* box, Swizzle swizzle) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return MS_ERR_LAUNCH;
  cuuint64_t gdim[3], gstr[2];
  cuuint32_t bx[3], es[3];
  for (int i = 0; i < rank; ++i) { gdim[i] = dims[i]; bx[i] = box[i]; es[i] = 1; }
  for (int i = 0; i + 1 < rank; ++i) gstr[i] = strides_bytes[i];
  const CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_NONE;
  if (swizzle == Swizzle::B32) sw = CU_TENSOR_MAP_SWIZZLE_32B;
  if (swizzle == Swizzle::B64) sw = CU_TENSOR_MAP_SWIZZLE_64B;
  if (swizzle == Swizzle::B128) sw = CU_TENSOR_MAP_SWIZZLE_128B;
  const CUresult r = fn(out, dt, (cuuint32_t)rank, base, gdim, gstr, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? MS_OK : MS_ERR_LAUNCH;
}

// Longest time, in nanoseconds, a peer-memory exchange kernel waits for another rank.
static std::atomic<long long> g_peer_wait_ms{-1};
unsigned long long peer_wait_ns() {
  long long ms = g_peer_wait_ms.load(std::memory_order_relaxed);
  if (ms < 0) {
    ms = 20000;
    if (const char* v = std::getenv("MEMSOLVE_PEER_WAIT_MS")) {
      const long long parsed = std::atoll(v);
      if (parsed > 0) ms = parsed;
    }
    g_peer_wait_ms.store(ms, std::memory_order_relaxed);
  }
  return (unsigned long long)ms * 1000000ull;
}

__device__ int g_error_word = 0;

int* device_error_word() {
  static std::atomic<int*> cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  int* p = cached[dev].load(std::memory_order_acquire);
  if (p) return p;
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_error_word) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  cached[dev].store(p, std::memory_order_release);
  return p;
}

static int device_status() {
  static std::atomic<int> cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return MS_ERR_DEVICE;
  int v = cached[dev].load(std::memory_order_relaxed);
  if (v == 1) return MS_OK;
  int major = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return MS_ERR_DEVICE;
  if (major != 10 && major != 11) return MS_ERR_DEVICE;
  cached[dev].store(1, std::memory_order_relaxed);
  return MS_OK;
}

int check_shape(const ms_shape* s) {
  if (!s) return MS_ERR_INVALID_ARGUMENT;
  if (s->batch <= 0 || s->tokens <= 0 || s->heads <= 0 || s->head_dim <= 0) return MS_ERR_INVALID_ARGUMENT;
  if (s->rank != 16 && s->rank != 32 && s->rank != 48 && s->rank != 64) return MS_ERR_UNSUPPORTED_RANK;
  if (s->rotary_rows != 0 && s->rotary_rows != 1 && s->rotary_rows != s->batch) return MS_ERR_INVALID_ARGUMENT;
  if (s->rotary_rows != 0 && (s->head_dim & 1)) return MS_ERR_ODD_HEAD_DIM;
  if (s->reserved != 0) return MS_ERR_INVALID_ARGUMENT;
  // the (sample, head) systems ride on gridDim.y of several kernels: refuse what the grid cannot hold instead of
  // failing at launch
  if ((long long)s->batch * s->heads > 65535LL) return MS_ERR_INVALID_ARGUMENT;
  return MS_OK;
}

static size_t round64(size_t v) { return (v + 63) & ~size_t(63); }

Plan make_plan(const ms_shape& s) {
  Plan p;
  p.systems = s.batch * s.heads;
  p.dblocks = (s.head_dim + kChanBlock - 1) / kChanBlock;
  p.dpad = (s.head_dim + 7) & ~7;
  const int tiles = (s.tokens + kTileTokens - 1) / kTileTokens;
  static const bool no_tma_env = [] {
    const char* v = std::getenv("MEMSOLVE_NO_TMA");
    return v && v[0] == '1';
  }();
  // the TMA statistics kernels (rank 16/32, head dimension a multiple of 64) run one CTA of eight
  // to twelve warps per SM; the generic kernels two 4-warp CTAs
  const bool wide_ctas = !no_tma_env && (s.head_dim % 64) == 0 && (s.rank == 16 || s.rank == 32);
  p.de_slots = 2 * p.dblocks;
  const long want = (wide_ctas ? 1L : 2L) * sm_count();
  long per = (long)p.systems * p.dblocks;
  // rounded down so that the whole grid (plus the per-head CTAs that ride along with the forward
  // statistics) is resident in one wave
  long chunks = (want - s.heads) / per;
  if (chunks < 1) chunks = 1;
  if (chunks > tiles) chunks = tiles;
  const int tiles_per_chunk = (int)((tiles + chunks - 1) / chunks);
  p.chunk_tokens = tiles_per_chunk * kTileTokens;
  p.chunks = (s.tokens + p.chunk_tokens - 1) / p.chunk_tokens;
  {
    // adjoint reduction: every SM streams (no CTAs for the per-head core in that grid)
    long cb = want / per;
    if (cb < 1) cb = 1;
    if (cb > tiles) cb = tiles;
    const int per_chunk = (int)((tiles + cb - 1) / cb);
    p.chunk_tokens_bwd = per_chunk * kTileTokens;
    p.chunks_bwd = (s.tokens + p.chunk_tokens_bwd - 1) / p.chunk_tokens_bwd;
  }
  static const bool no_tc_env = [] {
    const char* v = std::getenv("MEMSOLVE_NO_TCGEN05");
    return v && v[0] == '1';
  }();
  // The tcgen05 statistics kernel (long samples, head dimension 64, rank 16/32/64) gives a CTA one head and a chunk
  // of 128-token tiles.  Rank 64 takes it (the mma.sync kernels keep a rank-64 accumulator tile in registers only
  // for the adjoint, and the forward falls back to the generic loader) and so does rank 32: alone it is faster
  // there (30.0 / 31.6 us against 31.8 / 35.8 us at 32768 tokens), inside the chained launches the two are level
  // (145.7 us either way).  At rank 16 the mma.sync kernels stay ahead inside the chain (124.2 against 125.7 us).
  // MEMSOLVE_STATS_TCGEN05=1 selects the tcgen05 kernel at every rank, =0 at rank 64 only.
  static const int tc_env = [] {
    const char* v = std::getenv("MEMSOLVE_STATS_TCGEN05");
    return !v ? -1 : (v[0] == '1' ? 1 : 0);
  }();
  p.stats_tc = !no_tma_env && !no_tc_env && s.head_dim == 64 && s.tokens >= 1024 &&
               (s.rank == 64 || (s.rank == 32 && tc_env != 0) || (s.rank == 16 && tc_env == 1));
  if (p.stats_tc) {
    const int gsize = stats_tc_group_heads(s.rank);
    const long groups = (long)s.batch * ((s.heads + gsize - 1) / gsize);
    const int tiles128 = (s.tokens + 127) / 128;
    auto size_chunks = [&](long ctas, int& n_chunks, int& chunk_tokens) {
      long c = ctas / groups;
      if (c < 1) c = 1;
      if (c > tiles128) c = tiles128;
      const int per_chunk = (int)((tiles128 + c - 1) / c);
      chunk_tokens = per_chunk * 128;
      n_chunks = (s.tokens + chunk_tokens - 1) / chunk_tokens;
    };
    // forward: the per-head core rides in spare CTAs of the same grid
    const long core_slabs = (s.heads + groups - 1) / groups;
    size_chunks(sm_count() - core_slabs * groups > groups ? sm_count() - core_slabs * groups : groups, p.chunks, p.chunk_tokens);
    size_chunks(sm_count(), p.chunks_bwd, p.chunk_tokens_bwd);
  }
  p.aligned = (s.head_dim % 8) == 0;
  static const bool no_tma = [] {
    const char* v = std::getenv("MEMSOLVE_NO_TMA");
    return v && v[0] == '1';
  }();
  p.tma = !no_tma;
  static const bool no_tc = [] {
    const char* v = std::getenv("MEMSOLVE_NO_TCGEN05");
    return v && v[0] == '1';
  }();
  p.tc = p.tma && !no_tc;
  p.fwd_partial_floats = (size_t)s.rank * s.rank + (size_t)s.rank * s.head_dim;
  p.bwd_partial_floats = (size_t)s.rank * s.head_dim;
  {
    const size_t fwd = (size_t)p.chunks * p.fwd_partial_floats, bwd = (size_t)p.chunks_bwd * p.bwd_partial_floats;
    p.ws_partials = round64((size_t)p.systems * (fwd > bwd ? fwd : bwd));
    p.ws_de = round64((size_t)p.systems * (p.chunks_bwd > p.chunks ? p.chunks_bwd : p.chunks) * p.de_slots);
  }
  p.ws_hmat = round64((size_t)p.systems * s.rank * s.rank);
  p.ws_de_sys = round64((size_t)p.systems);
  p.ws_packed = round64((size_t)p.systems * (p.fwd_partial_floats + 1));
  // Rank 64 with the tcgen05 statistics: a system's partials (twelve of 32 KB at 32768 tokens) do not fit the
  // staging area of the compact kernels, whose twelve CTAs then add them from global memory at ~26 GB/s each
  // (6.6 + 8.6 us forward, 9.4 us backward); a launch of its own over all SMs does it in ~2 us and the compact
  // kernels read one reduced vector (mix core at 32768 tokens: 236 -> 220 us).  At rank 16/32 the staged sums are
  // cheaper than the extra launch (145.7 against 150.4 us).  MEMSOLVE_PACK=1 / 0 forces either.
  static const int pack_env = [] {
    const char* v = std::getenv("MEMSOLVE_PACK");
    return !v ? -1 : (v[0] == '1' ? 1 : 0);
  }();
  p.pack = p.stats_tc && (pack_env < 0 ? s.rank == 64 : pack_env == 1);
  p.ws_total_bytes = (p.ws_partials + p.ws_de + p.ws_hmat + p.ws_de_sys + p.ws_packed) * sizeof(float);
  return p;
}

struct Workspace {
  float* partials;
  float* de_partials;
  float* hmat;
  float* de_sys;
  float* packed;
};

static Workspace carve(void* ws, const Plan& p) {
  Workspace w;
  w.partials = static_cast<float*>(ws);
  w.de_partials = w.partials + p.ws_partials;
  w.hmat = w.de_partials + p.ws_de;
  w.de_sys = w.hmat + p.ws_hmat;
  w.packed = w.de_sys + p.ws_de_sys;
  return w;
}

static bool is16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
// no more tokens than the rank: ms_mix_forward / ms_mix_backward evaluate the eta term in token space
static bool short_sequence(const ms_shape& s) { return s.tokens <= s.rank; }

}  // namespace ms

using namespace ms;

#define MS_TRY(expr)            \
  do {                          \
    int _st = (expr);           \
    if (_st != MS_OK) return _st; \
  } while (0)

extern "C" {

int ms_abi_version(void) { return MS_ABI_VERSION; }

int ms_supported_architectures(int32_t* out, int capacity) {
  if (out && capacity > 0) out[0] = 100;
  return 1;
}

const char* ms_status_string(int status) {
  switch (status) {
    case MS_OK: return "ok";
    case MS_ERR_INVALID_ARGUMENT: return "invalid argument (null pointer, non-positive size or bad rotary_rows)";
    case MS_ERR_UNSUPPORTED_RANK: return "the CUDA fast path supports rank in {16,32,48,64}";
    case MS_ERR_WORKSPACE: return "workspace is null or smaller than ms_workspace_bytes()";
    case MS_ERR_LAUNCH: return "a CUDA kernel launch failed";
    case MS_ERR_DEVICE: return "the current CUDA device is not an sm_100-class GPU";
    case MS_ERR_ODD_HEAD_DIM: return "rotary content requires an even head dimension";
    case MS_ERR_LINEAR_SHAPE:
      return "the tcgen05 projection kernels take in_features a multiple of 64 (128 for the gradients), out_features a "
             "multiple of 128 (64 for the input gradient) and 16-byte aligned pointers";
    case MS_ERR_DEBUG_SHAPE:
      return "the FP32 debug entry points cover the tensor-core (tcgen05) kernels only: head dimension 64, rank 16, "
             "32 or 64, 16-byte aligned pointers";
    case MS_ERR_STATIC_SCRATCH:
      return "this shape needs more scratch than the built-in static buffer of ms_stats_forward_static holds "
             "(MS_STATIC_SCRATCH_FLOATS); use ms_stats_forward with a caller-provided workspace";
  }
  return "unknown status";
}

int ms_padded_head_dim(int head_dim) { return (head_dim + 7) & ~7; }

int ms_device_error(void) {
  int* word = device_error_word();
  if (!word) return -1;
  int value = 0;
  if (cudaMemcpy(&value, word, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (value != 0) cudaMemset(word, 0, sizeof(int));
  return value;
}

int ms_linear_forward(int64_t rows, int32_t in_features, int32_t out_features, const void* x, const void* weight,
                      const float* bias, const uint8_t* input_mask, const uint8_t* output_mask, void* out,
                      void* stream) {
  MS_TRY(device_status());
  if (!x || !weight || !out || rows <= 0 || in_features <= 0 || out_features <= 0) return MS_ERR_INVALID_ARGUMENT;
  const int r = launch_linear_tc((long)rows, in_features, out_features, x, weight, bias, input_mask, output_mask, out,
                                 static_cast<cudaStream_t>(stream));
  return r == -1 ? MS_ERR_LINEAR_SHAPE : r;
}

int ms_linear_input_grad(int64_t rows, int32_t in_features, int32_t out_features, const void* dy, const void* weight,
                         const uint8_t* input_mask, const uint8_t* output_mask, void* dx, void* stream) {
  MS_TRY(device_status());
  if (!dy || !weight || !dx || rows <= 0 || in_features <= 0 || out_features <= 0) return MS_ERR_INVALID_ARGUMENT;
  const int r = launch_linear_input_grad_tc((long)rows, in_features, out_features, dy, weight, input_mask, output_mask, dx,
                                            static_cast<cudaStream_t>(stream));
  return r == -1 ? MS_ERR_LINEAR_SHAPE : r;
}

size_t ms_linear_weight_grad_workspace(int64_t rows, int32_t in_features, int32_t out_features) {
  return linear_wgrad_workspace_bytes((long)rows, in_features, out_features);
}

int ms_linear_weight_grad(int64_t rows, int32_t in_features, int32_t out_features, const void* x, const void* dy,
                          float* dweight, float* dbias, void* workspace, size_t workspace_bytes, void* stream) {
  MS_TRY(device_status());
  if (!x || !dy || !dweight || rows <= 0 || in_features <= 0 || out_features <= 0) return MS_ERR_INVALID_ARGUMENT;
  const int r = launch_linear_wgrad_tc((long)rows, in_features, out_features, x, dy, dweight, dbias, workspace,
                                       workspace_bytes, static_cast<cudaStream_t>(stream));
  return r == -1 ? MS_ERR_LINEAR_SHAPE : r;
}

int ms_set_peer_wait_ms(int milliseconds) {
  if (milliseconds <= 0) return MS_ERR_INVALID_ARGUMENT;
  g_peer_wait_ms.store(milliseconds, std::memory_order_relaxed);
  return MS_OK;
}

size_t ms_workspace_bytes(const ms_shape* shape) {
  if (check_shape(shape) != MS_OK) return 0;
  return make_plan(*shape).ws_total_bytes;
}

size_t ms_packed_stats_floats(const ms_shape* shape, int backward) {
  if (check_shape(shape) != MS_OK) return 0;
  const size_t sys = (size_t)shape->batch * shape->heads;
  const size_t rd = (size_t)shape->rank * shape->head_dim;
  return backward ? sys * (rd + 1) : sys * ((size_t)shape->rank * shape->rank + rd);
}

int ms_core_forward(const ms_shape* shape, const float* base_raw, const float* eta_raw, const ms_tape* tape,
                    void* stream) {
  MS_TRY(check_shape(shape));
  MS_TRY(device_status());
  if (!eta_raw || !tape || !tape->eta || !tape->eta_slope || !tape->core_info) return MS_ERR_INVALID_ARGUMENT;
  if (!shape->complement && (!base_raw || !tape->core_map)) return MS_ERR_INVALID_ARGUMENT;
  return launch_core_forward(*shape, base_raw, eta_raw, *tape, static_cast<cudaStream_t>(stream));
}

int ms_stats_forward(const ms_shape* shape, const void* projected, const float* cos, const float* sin,
                     const float* counts, void* workspace, size_t workspace_bytes, float* packed, void* stream) {
  MS_TRY(check_shape(shape));
  MS_TRY(device_status());
  if (!projected) return MS_ERR_INVALID_ARGUMENT;
  if (shape->rotary_rows && (!cos || !sin)) return MS_ERR_INVALID_ARGUMENT;
  Plan plan = make_plan(*shape);
  if (!workspace || !is16(workspace) || workspace_bytes < plan.ws_total_bytes) return MS_ERR_WORKSPACE;
  plan.aligned = plan.aligned && is16(projected) && (!shape->rotary_rows || (is16(cos) && is16(sin)));
  const Workspace w = carve(workspace, plan);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MS_TRY(launch_stats(*shape, plan, false, projected, nullptr, cos, sin, w.partials, nullptr, nullptr, nullptr,
                      nullptr, st));
  if (packed) MS_TRY(launch_pack_stats(*shape, plan, false, w.partials, nullptr, counts, packed, st));
  return MS_OK;
}

// Scratch of ms_stats_forward_static: lives in the library image, one copy per GPU that loads it.
static __device__ __align__(256) float g_static_scratch[MS_STATIC_SCRATCH_FLOATS];

// Device address of g_static_scratch on the current device.  In host code the symbol's name is
// only a handle, so the address is asked for once per device (with that device current) and kept.
static float* static_scratch_address() {
  static std::atomic<float*> cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  float* p = cached[dev].load(std::memory_order_acquire);
  if (p) return p;
  void* addr = nullptr;
  if (cudaGetSymbolAddress(&addr, g_static_scratch) != cudaSuccess || !addr) {
    cudaGetLastError();
    return nullptr;
  }
  p = static_cast<float*>(addr);
  cached[dev].store(p, std::memory_order_release);
  return p;
}

int ms_stats_forward_static(const ms_shape* shape, const void* projected, const float* cos, const float* sin,
                            const float* counts, float* packed, void* stream) {
  MS_TRY(check_shape(shape));
  MS_TRY(device_status());
  if (!projected || !packed) return MS_ERR_INVALID_ARGUMENT;
  if (shape->rotary_rows && (!cos || !sin)) return MS_ERR_INVALID_ARGUMENT;
  Plan plan = make_plan(*shape);
  if (plan.ws_partials > (size_t)MS_STATIC_SCRATCH_FLOATS) return MS_ERR_STATIC_SCRATCH;
  float* scratch = static_scratch_address();
  if (!scratch) return MS_ERR_LAUNCH;
  plan.aligned = plan.aligned && is16(projected) && (!shape->rotary_rows || (is16(cos) && is16(sin)));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // every partial of the launched grid is written in full before it is read, so nothing in the
  // shared scratch needs clearing between calls
  MS_TRY(launch_stats(*shape, plan, false, projected, nullptr, cos, sin, scratch, nullptr, nullptr, nullptr,
                      nullptr, st));
  return launch_pack_stats(*shape, plan, false, scratch, nullptr, counts, packed, st);
}

int ms_compact_forward(const ms_shape* shape, const float* counts, const void* workspace, size_t workspace_bytes,
                       const float* packed, const ms_tape* tape, void* stream) {
  MS_TRY(check_shape(shape));
  MS_TRY(device_status());
  if (!tape || !tape->eta || !tape->inverse || !tape->state || !tape->coeff) return MS_ERR_INVALID_ARGUMENT;
  if (!shape->complement && !tape->core_map) return MS_ERR_INVALID_ARGUMENT;
  const Plan plan = make_plan(*shape);
  const float* src = packed;
  if (!packed) {
    if (!workspace || !is16(workspace) || workspace_bytes < plan.ws_total_bytes) return MS_ERR_WORKSPACE;
    src = static_cast<const float*>(workspace);
  }
  return launch_compact_forward(*shape, plan, counts, src, packed != nullptr, *tape,
                                static_cast<cudaStream_t>(stream));
}

int ms_readout(const ms_shape* shape, const void* projected, const float* cos, const float* sin,
               const float* counts, const ms_tape* tape, void* mixed, void* stream) {
  MS_TRY(check_shape(shape));
  MS_TRY(device_status());
  if (!projected || !mixed || !tape || !tape->eta || !tape->coeff) return MS_ERR_INVALID_ARGUMENT;
  if (shape->rotary_rows && (!cos || !sin)) return MS_ERR_INVALID_ARGUMENT;
  Plan plan = make_plan(*shape);
  plan.aligned = plan.aligned && is16(projected) && is16(mixed);
  return launch_readout(*shape, plan, projected, cos, sin, counts, *tape, mixed, static_cast<cudaStream_t>(stream));
}

int ms_readout_short(const ms_shape* shape, const void* projected, const float* cos, const float* sin,
                     const float* counts, const ms_tape* tape, void* mixed, void* stream) {
  MS_TRY(check_shape(shape));
  MS_TRY(device_status());
  if (!projected || !mixed || !tape || !tape->eta || !tape->coeff) return MS_ERR_INVALID_ARGUMENT;
  if (shape->rotary_rows && (!cos || !sin)) return MS_ERR_INVALID_ARGUMENT;
  if (!short_sequence(*shape)) return MS_ERR_INVALID_ARGUMENT;
  const Plan plan = make_plan(*shape);
  return launch_short_readout(*shape, plan, projected, cos, sin, counts, *tape, mixed,
                              static_cast<cudaStream_t>(stream));
}

int ms_readout_debug(const ms_shape* shape, const void* projected, const float* cos, const float* sin,
                     const float* counts, const ms_tape* tape, void* mixed, float* mixed_f32, void* stream) {
  MS_TRY(check_shape(shape));
  MS_TRY(device_status());
  if (!projected || !mixed || !mixed_f32 || !tape || !tape->eta || !tape->coeff) return MS_ERR_INVALID_ARGUMENT;
  if (shape->rotary_rows && (!cos || !sin)) return MS_ERR_INVALID_ARGUMENT;
  Plan plan = make_plan(*shape);
  plan.aligned = plan.aligned && is16(projected) && is16(mixed) && (!shape->rotary_rows || (is16(cos) && is16(sin)));
  const int r = launch_readout_tc(*shape, plan, projected, cos, sin, counts, *tape, mixed, mixed_f32,
                                  static_cast<cudaStream_t>(stream));
  return r == -1 ? MS_ERR_DEBUG_SHAPE : r;
}

int ms_mix_forward(const ms_shape* shape, const void* projected, const float* base_raw, const float* eta_raw,
                   const float* cos, const float* sin, const float* counts, void* workspace,
                   size_t workspace_bytes, const ms_tape* tape, void* mixed, void* stream) {
  MS_TRY(check_shape(shape));
  MS_TRY(device_status());
  if (!projected || !mixed || !eta_raw || !tape || !tape->eta || !tape->eta_slope || !tape->core_info ||
      !tape->inverse || !tape->state || !tape->coeff)
    return MS_ERR_INVALID_ARGUMENT;
  if (!shape->complement && (!base_raw || !tape->core_map)) return MS_ERR_INVALID_ARGUMENT;
  if (shape->rotary_rows && (!cos || !sin)) return MS_ERR_INVALID_ARGUMENT;
  Plan plan = make_plan(*shape);
  if (!workspace || !is16(workspace) || workspace_bytes < plan.ws_total_bytes) return MS_ERR_WORKSPACE;
  const bool tables16 = !shape->rotary_rows || (is16(cos) && is16(sin));
  const Workspace w = carve(workspace, plan);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Plan stats_plan = plan;
  stats_plan.aligned = plan.aligned && is16(projected) && tables16;
  // the per-head core (eta, F) is computed by spare CTAs of the statistics grid
  MS_TRY(launch_stats(*shape, stats_plan, false, projected, nullptr, cos, sin, w.partials, nullptr, base_raw,
                      eta_raw, tape, st));
  if (short_sequence(*shape)) {
    // no more tokens than the rank: the compact stage keeps the core part only (eta = 0) and the eta term is
    // evaluated in token space, where it does not cancel (see ms_short.cu)
    ms_tape core_only = *tape;
    core_only.eta = nullptr;
    MS_TRY(launch_compact_forward(*shape, plan, counts, w.partials, false, core_only, st));
    return launch_short_readout(*shape, plan, projected, cos, sin, counts, *tape, mixed, st);
  }
  // the launches below start while the kernel ahead of them drains (see launch_kernel)
  ChainScope chain(chaining_allowed());
  if (plan.pack) {
    MS_TRY(launch_pack_stats(*shape, plan, false, w.partials, nullptr, counts, w.packed, st));
    MS_TRY(launch_compact_forward(*shape, plan, counts, w.packed, true, *tape, st));
  } else {
    MS_TRY(launch_compact_forward(*shape, plan, counts, w.partials, false, *tape, st));
  }
  Plan read_plan = plan;
  read_plan.aligned = plan.aligned && is16(projected) && is16(mixed);
  return launch_readout(*shape, read_plan, projected, cos, sin, counts, *tape, mixed, st);
}

int ms_stats_backward(const ms_shape* shape, const void* projected, const void* dy, const float* cos,
                      const float* sin, const float* counts, void* workspace, size_t workspace_bytes,
                      float* packed, void* stream) {
  MS_TRY(check_shape(shape));
  MS_TRY(device_status());
  if (!projected || !dy) return MS_ERR_INVALID_ARGUMENT;
  if (shape->rotary_rows && (!cos || !sin)) return MS_ERR_INVALID_ARGUMENT;
  Plan plan = backward_plan(make_plan(*shape));
  if (!workspace || !is16(workspace) || workspace_bytes < plan.ws_total_bytes) return MS_ERR_WORKSPACE;
  plan.aligned = plan.aligned && is16(projected) && is16(dy) && (!shape->rotary_rows || (is16(cos) && is16(sin)));
  const Workspace w = carve(workspace, plan);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MS_TRY(launch_stats(*shape, plan, true, projected, dy, cos, sin, w.partials, w.de_partials, nullptr, nullptr,
                      nullptr, st));
  if (packed) MS_TRY(launch_pack_stats(*shape, plan, true, w.partials, w.de_partials, counts, packed, st));
  return MS_OK;
}

int ms_compact_backward(const ms_shape* shape, const float* counts, void* workspace, size_t workspace_bytes,
                        const float* packed, const ms_tape* tape, const float* base_raw, const float* eta_raw,
                        float grad_scale, void* gram_grad, void* cross_grad, float* d_base_raw,
                        float* d_eta_raw, void* stream) {
  MS_TRY(check_shape(shape));
  MS_TRY(device_status());
  (void)eta_raw;
  if (!tape || !tape->eta || !tape->eta_slope || !tape->inverse || !tape->state) return MS_ERR_INVALID_ARGUMENT;
  if (!gram_grad || !cross_grad) return MS_ERR_INVALID_ARGUMENT;
  const bool with_core = d_eta_raw != nullptr;
  if (with_core && !shape->complement && (!base_raw || !tape->core_map || !d_base_raw)) return MS_ERR_INVALID_ARGUMENT;
  const Plan plan = backward_plan(make_plan(*shape));
  if (!workspace || !is16(workspace) || workspace_bytes < plan.ws_total_bytes) return MS_ERR_WORKSPACE;
  const Workspace w = carve(workspace, plan);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MS_TRY(launch_compact_backward(*shape, plan, counts, packed ? packed : w.partials, w.de_partials,
                                 packed != nullptr, *tape, w.hmat, w.de_sys, gram_grad, cross_grad, st));
  if (!with_core) return MS_OK;
  return launch_core_backward(*shape, base_raw, w.hmat, w.de_sys, *tape, grad_scale, d_base_raw, d_eta_raw, st);
}

int ms_token_backward_core(const ms_shape* shape, const void* projected, const void* dy, const float* cos,
                           const float* sin, const float* counts, const ms_tape* tape, const void* gram_grad,
                           const void* cross_grad, void* dprojected, const float* base_raw, void* workspace,
                           size_t workspace_bytes, float grad_scale, float* d_base_raw, float* d_eta_raw,
                           void* stream) {
  MS_TRY(check_shape(shape));
  MS_TRY(device_status());
  if (!projected || !dy || !dprojected || !gram_grad || !cross_grad || !tape || !tape->eta || !tape->coeff ||
      !tape->eta_slope || !d_eta_raw)
    return MS_ERR_INVALID_ARGUMENT;
  if (!shape->complement && (!base_raw || !tape->core_map || !d_base_raw)) return MS_ERR_INVALID_ARGUMENT;
  if (shape->rotary_rows && (!cos || !sin)) return MS_ERR_INVALID_ARGUMENT;
  Plan plan = make_plan(*shape);
  if (!workspace || !is16(workspace) || workspace_bytes < plan.ws_total_bytes) return MS_ERR_WORKSPACE;
  const Workspace w = carve(workspace, plan);
  plan.aligned = plan.aligned && is16(projected) && is16(dy) && is16(dprojected);
  CoreAdjoint core{base_raw, w.hmat, w.de_sys, d_base_raw, d_eta_raw, grad_scale};
  return launch_token_backward(*shape, plan, projected, dy, cos, sin, counts, *tape, gram_grad, cross_grad,
                               dprojected, &core, static_cast<cudaStream_t>(stream));
}

int ms_stats_forward_core(const ms_shape* shape, const void* projected, const float* base_raw,
                          const float* eta_raw, const float* cos, const float* sin, const float* counts,
                          void* workspace, size_t workspace_bytes, float* packed, const ms_tape* tape,
                          void* stream) {
  MS_TRY(check_shape(shape));
  MS_TRY(device_status());
  if (!projected || !eta_raw || !tape || !tape->eta || !tape->eta_slope || !tape->core_info)
    return MS_ERR_INVALID_ARGUMENT;
  if (!shape->complement && (!base_raw || !tape->core_map)) return MS_ERR_INVALID_ARGUMENT;
  if (shape->rotary_rows && (!cos || !sin)) return MS_ERR_INVALID_ARGUMENT;
  Plan plan = make_plan(*shape);
  if (!workspace || !is16(workspace) || workspace_bytes < plan.ws_total_bytes) return MS_ERR_WORKSPACE;
  plan.aligned = plan.aligned && is16(projected) && (!shape->rotary_rows || (is16(cos) && is16(sin)));
  const Workspace w = carve(workspace, plan);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MS_TRY(launch_stats(*shape, plan, false, projected, nullptr, cos, sin, w.partials, nullptr, base_raw, eta_raw,
                      tape, st));
  if (packed) MS_TRY(launch_pack_stats(*shape, plan, false, w.partials, nullptr, counts, packed, st));
  return MS_OK;
}

static size_t exchange_capacity(const ms_shape* shape) {
  const size_t fwd = ms_packed_stats_floats(shape, 0), bwd = ms_packed_stats_floats(shape, 1);
  return ((fwd > bwd ? fwd : bwd) + 3) & ~size_t(3);
}

size_t ms_exchange_area_bytes(const ms_shape* shape) {
  if (check_shape(shape) != MS_OK) return 0;
  return exchange_area_bytes(exchange_capacity(shape));
}

int ms_stats_exchange(const ms_shape* shape, int backward, const void* workspace, size_t workspace_bytes,
                      const float* counts, void* const* areas, size_t area_bytes, int world_size, int rank,
                      float* packed, void* stream) {
  MS_TRY(check_shape(shape));
  MS_TRY(device_status());
  if (!packed || !areas) return MS_ERR_INVALID_ARGUMENT;
  const Plan plan = backward != 0 ? backward_plan(make_plan(*shape)) : make_plan(*shape);
  if (!workspace || !is16(workspace) || workspace_bytes < plan.ws_total_bytes) return MS_ERR_WORKSPACE;
  // the layout of an area follows from its size: the largest capacity (a multiple of four values)
  // whose area fits; every rank must pass the same size
  const size_t fixed = exchange_area_bytes(0);
  if (area_bytes < fixed + 32) return MS_ERR_WORKSPACE;
  const size_t capacity = ((area_bytes - fixed) / (2 * sizeof(float))) & ~size_t(3);
  const Workspace w = carve(const_cast<void*>(workspace), plan);
  return launch_exchange(*shape, plan, backward != 0, w.partials, w.de_partials, counts, areas, world_size, rank,
                         capacity, packed, static_cast<cudaStream_t>(stream));
}

size_t ms_peer_sum_area_bytes(size_t count) { return peer_sum_area_bytes((count + 3) & ~size_t(3)) + 64; }

int ms_peer_sum(float* values, size_t count, void* const* areas, size_t area_bytes, int world_size, int rank,
                void* stream) {
  MS_TRY(device_status());
  return launch_peer_sum(values, count, areas, area_bytes, world_size, rank, static_cast<cudaStream_t>(stream));
}

int ms_token_backward(const ms_shape* shape, const void* projected, const void* dy, const float* cos,
                      const float* sin, const float* counts, const ms_tape* tape, const void* gram_grad,
                      const void* cross_grad, void* dprojected, void* stream) {
  MS_TRY(check_shape(shape));
  MS_TRY(device_status());
  if (!projected || !dy || !dprojected || !gram_grad || !cross_grad || !tape || !tape->eta || !tape->coeff)
    return MS_ERR_INVALID_ARGUMENT;
  if (shape->rotary_rows && (!cos || !sin)) return MS_ERR_INVALID_ARGUMENT;
  Plan plan = make_plan(*shape);
  plan.aligned = plan.aligned && is16(projected) && is16(dy) && is16(dprojected);
  return launch_token_backward(*shape, plan, projected, dy, cos, sin, counts, *tape, gram_grad, cross_grad,
                               dprojected, nullptr, static_cast<cudaStream_t>(stream));
}

int ms_token_backward_debug(const ms_shape* shape, const void* projected, const void* dy, const float* cos,
                            const float* sin, const float* counts, const ms_tape* tape, const void* gram_grad,
                            const void* cross_grad, void* dprojected, float* dprojected_f32, void* stream) {
  MS_TRY(check_shape(shape));
  MS_TRY(device_status());
  if (!projected || !dy || !dprojected || !dprojected_f32 || !gram_grad || !cross_grad || !tape || !tape->eta ||
      !tape->coeff)
    return MS_ERR_INVALID_ARGUMENT;
  if (shape->rotary_rows && (!cos || !sin)) return MS_ERR_INVALID_ARGUMENT;
  Plan plan = make_plan(*shape);
  plan.aligned = plan.aligned && is16(projected) && is16(dy) && is16(dprojected) &&
                 (!shape->rotary_rows || (is16(cos) && is16(sin)));
  const int r = launch_token_backward_tc(*shape, plan, projected, dy, cos, sin, counts, *tape, gram_grad, cross_grad,
                                         dprojected, nullptr, dprojected_f32, static_cast<cudaStream_t>(stream));
  return r == -1 ? MS_ERR_DEBUG_SHAPE : r;
}

int ms_mix_backward(const ms_shape* shape, const void* projected, const void* dy, const float* base_raw,
                    const float* eta_raw, const float* cos, const float* sin, const float* counts,
                    void* workspace, size_t workspace_bytes, const ms_tape* tape, void* gram_grad,
                    void* cross_grad, void* dprojected, float* d_base_raw, float* d_eta_raw, void* stream) {
  MS_TRY(ms_stats_backward(shape, projected, dy, cos, sin, counts, workspace, workspace_bytes, nullptr, stream));
  (void)eta_raw;
  if (!tape || !tape->eta || !tape->eta_slope || !tape->inverse || !tape->state) return MS_ERR_INVALID_ARGUMENT;
  if (!gram_grad || !cross_grad || !d_eta_raw) return MS_ERR_INVALID_ARGUMENT;
  if (!shape->complement && (!base_raw || !tape->core_map || !d_base_raw)) return MS_ERR_INVALID_ARGUMENT;
  const Plan plan = backward_plan(make_plan(*shape));
  const Workspace w = carve(workspace, plan);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (short_sequence(*shape)) {
    if (!projected || !dy || !dprojected || !tape->coeff) return MS_ERR_INVALID_ARGUMENT;
    ms_tape core_only = *tape;
    core_only.eta = nullptr;
    MS_TRY(launch_compact_backward(*shape, plan, counts, w.partials, w.de_partials, false, core_only, w.hmat,
                                   w.de_sys, gram_grad, cross_grad, st));
    // d_base from the core part; its d_eta_raw is replaced by the token-space one below
    MS_TRY(launch_core_backward(*shape, base_raw, w.hmat, w.de_sys, *tape, 1.0f, d_base_raw, d_eta_raw, st));
    return launch_short_backward(*shape, plan, projected, dy, cos, sin, counts, *tape, gram_grad, cross_grad,
                                 dprojected, w.de_partials, 1.0f, d_eta_raw, st);
  }
  ChainScope chain(chaining_allowed());
  if (plan.pack) {
    MS_TRY(launch_pack_stats(*shape, plan, true, w.partials, w.de_partials, counts, w.packed, st));
    MS_TRY(launch_compact_backward(*shape, plan, counts, w.packed, nullptr, true, *tape, w.hmat, w.de_sys, gram_grad,
                                   cross_grad, st));
  } else {
    MS_TRY(launch_compact_backward(*shape, plan, counts, w.partials, w.de_partials, false, *tape, w.hmat,
                                   w.de_sys, gram_grad, cross_grad, st));
  }
  // the token pass needs only dG and dQ; the per-head core adjoint rides in spare CTAs of its grid
  if (!projected || !dy || !dprojected) return MS_ERR_INVALID_ARGUMENT;
  Plan token_plan = plan;
  token_plan.aligned = plan.aligned && is16(projected) && is16(dy) && is16(dprojected);
  CoreAdjoint core{base_raw, w.hmat, w.de_sys, d_base_raw, d_eta_raw, 1.0f};
  return launch_token_backward(*shape, token_plan, projected, dy, cos, sin, counts, *tape, gram_grad, cross_grad,
                               dprojected, &core, st);
}

}  // extern "C"
