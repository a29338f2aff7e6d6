/*
 * memsolve_b200.h -- C ABI of the B200 (sm_100a) MemSolve mixer kernels.
 *
 * One shared library, `memsolve_equilibrium_sm100.so`, exports exactly the symbols
 * declared here.  Signatures use plain pointers and integers only (no torch types).
 * Every pointer named `d_*`/documented as "device" is a device pointer owned by the
 * caller; nothing here allocates or frees device memory, synchronises the host, or
 * keeps a pointer after returning, so calls may be captured into a CUDA graph.
 * `stream` is a `cudaStream_t` passed as `void*`.
 *
 * All functions returning `int` return an `ms_status` (0 on success).
 *
 * Reference interfaces replaced (paths inside the reference project):
 *   - csrc/ball/binding.cpp:314-321  TORCH_LIBRARY(memsolve_equilibrium) op set
 *   - memsolve/ball/cuda.py:2121-2247 `_no_frame_statistics`      -> ms_stats_forward / ms_stats_backward
 *   - memsolve/ball/cuda.py:2798-2880 core forward + `_no_frame_compact` -> ms_core_forward, ms_compact_forward
 *   - memsolve/ball/cuda.py:2990-3050 `_run_readout`              -> ms_readout
 *   - memsolve/ball/cuda.py:2883-2987 `_no_frame_compact_backward` -> ms_compact_backward, ms_core_backward
 *   - memsolve/ball/cuda.py:3053-3109 `_run_token_backward`       -> ms_token_backward
 *   - memsolve/ball/cuda.py:3112-3227 `_no_frame_forward` / `_NoFrameMix` -> ms_mix_forward / ms_mix_backward
 *
 * Tensor layouts (row-major, innermost last):
 *   projected   bf16 [B, N, H*r + H*d]   head h: relation cols [h*r,(h+1)*r), content cols [H*r+h*d, H*r+(h+1)*d)
 *   mixed, dy   bf16 [B, N, H*d]
 *   cos, sin    f32  [rotary_rows, N, d/2]  (rotary_rows = 1 or B; adjacent-pair layout)
 *   counts      f32  [B]                  max(valid tokens, 1); NULL means N
 *   base_raw    f32  [H, r, r]            ignored when shape.complement != 0
 *   eta_raw     f32  [H]
 *   tape tensors: see ms_tape below.
 */
#ifndef MEMSOLVE_B200_H_
#define MEMSOLVE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MS_ABI_VERSION 1

typedef enum ms_status {
  MS_OK = 0,
  MS_ERR_INVALID_ARGUMENT = 1, /* null pointer, non-positive size, bad rotary_rows ...          */
  MS_ERR_UNSUPPORTED_RANK = 2, /* rank not in {16, 32, 48, 64}                                  */
  MS_ERR_WORKSPACE = 3,        /* workspace null, not 16-byte aligned, or < ms_workspace_bytes() */
  MS_ERR_LAUNCH = 4,           /* a kernel launch reported a CUDA error                         */
  MS_ERR_DEVICE = 5,           /* current device is not sm_100-class                            */
  MS_ERR_ODD_HEAD_DIM = 6,     /* rotary tables given with an odd head dimension                */
  MS_ERR_STATIC_SCRATCH = 7,   /* shape too large for the built-in scratch of ms_stats_forward_static */
  MS_ERR_DEBUG_SHAPE = 8,      /* an FP32 debug entry point was called with a shape its kernel does not take */
  MS_ERR_LINEAR_SHAPE = 9      /* ms_linear_*: feature counts or alignment outside the tcgen05 kernels' envelope */
} ms_status;

/* Capacity, in floats, of the scratch buffer compiled into the library for
 * ms_stats_forward_static (16 MiB per GPU that loads the library, held until process exit). */
#define MS_STATIC_SCRATCH_FLOATS (4 * 1024 * 1024)

/* Problem shape shared by every call. */
typedef struct ms_shape {
  int32_t batch;       /* B; B*H <= 65535 */
  int32_t tokens;      /* N (local tokens of this rank under sequence parallelism)  */
  int32_t heads;       /* H */
  int32_t rank;        /* r in {16,32,48,64} */
  int32_t head_dim;    /* d >= 1 */
  int32_t complement;  /* nonzero: complement mode (F = 0, no base_raw)             */
  int32_t rotary_rows; /* 0: no rotary; 1: one table for all samples; B: per sample */
  int32_t reserved;    /* must be 0 */
} ms_shape;

/*
 * Compact tape written by the forward and read by the backward.  All device
 * pointers, caller-allocated (sizes in elements):
 *   eta        f32  [H]            (1 - 2^-23) * tanh(eta_raw)
 *   eta_slope  f32  [H]            d eta / d eta_raw (exponential form)
 *   core_map   f32  [H, r, r]      F = (I+J)^-1 (I-J); untouched in complement mode
 *   core_info  i32  [H]            0, or k+1 if LU pivot k was exactly zero
 *   inverse    f32  [B, H, r, r]   T = chol(I+G)^-1, lower triangular
 *   state      f32  [B, H, r, d]   Z = T Q
 *   coeff      bf16 [B, H, 2, r, dp] readout coefficients W = T^T (F - eta I) Z split into a
 *                                  high BF16 word ([..,0,..]) and the BF16 residual ([..,1,..]);
 *                                  dp = ms_padded_head_dim(d), padding columns are zero
 */
typedef struct ms_tape {
  float* eta;
  float* eta_slope;
  float* core_map;
  int32_t* core_info;
  float* inverse;
  float* state;
  void* coeff;
} ms_tape;

/* Replaces torch.ops.memsolve_equilibrium.contract_version (csrc/ball/binding.cpp:315). */
int ms_abi_version(void);

/* Replaces supported_architectures (csrc/ball/binding.cpp:316): writes up to `capacity`
 * SM numbers (e.g. 100) compiled into this library, returns how many exist. */
int ms_supported_architectures(int32_t* out, int capacity);

/* Human-readable text for a status code (static storage). */
const char* ms_status_string(int status);

/* Row pitch, in elements, of the split coefficient tensors: d rounded up to a multiple of 8. */
int ms_padded_head_dim(int head_dim);

/* Diagnostic (synchronises the device): reads and clears the library's device-side error word of
 * the current device.  0 = no error; 0x100 = a kernel gave up waiting on a shared-memory barrier
 * (its bounded wait ran out) and returned early, so the last results are incomplete; 0x200 = a
 * peer-memory exchange (ms_stats_exchange, ms_peer_sum) gave up waiting for another rank and wrote
 * NaN in place of the sums it could not form; -1 = the word could not be read.  No counterpart in
 * the reference, whose kernels have no such waits. */
int ms_device_error(void);

/* Longest time a peer-memory exchange kernel waits for another rank before it gives up (error word
 * 0x200, NaN results).  Default 20000 ms, or the value of the environment variable
 * MEMSOLVE_PEER_WAIT_MS read at the first exchange; applies to launches made after the call.  The
 * NCCL all-reduce this path replaces (integrations/distributed.py:47-50 of the reference) waits
 * without a limit; a kernel that spins forever would hang the GPU for every other user of it. */
int ms_set_peer_wait_ms(int milliseconds);

/*
 * Projection with the reference's fused epilogue (memsolve/ball/cuda.py:418-708 `_biased_gemm` / `_wide_gemm`,
 * forward of `tensor_core_linear`, memsolve/ball/reference.py:191-269):
 *   out[m, n] = output_mask[m] ? (input_mask[m] ? sum_k x[m, k] weight[n, k] : 0) + bias[n] : 0
 * x bf16 [rows, in_features], weight bf16 [out_features, in_features] (row-major, as nn.Linear stores it),
 * bias f32 [out_features] or NULL, masks one byte per row (0 = masked) or NULL, out bf16 [rows, out_features].
 * BF16 products, FP32 accumulation, FP32 bias, one BF16 rounding; masked input rows may hold anything (NaN
 * included), masked output rows are exactly zero.  tcgen05 GEMM (TMA-staged operands, accumulators in tensor
 * memory); returns MS_ERR_LINEAR_SHAPE for shapes it does not take.
 */
int ms_linear_forward(int64_t rows, int32_t in_features, int32_t out_features, const void* x, const void* weight,
                      const float* bias, const uint8_t* input_mask, const uint8_t* output_mask, void* out,
                      void* stream);

/*
 * Input gradient of the projection (memsolve/ball/cuda.py:959-1041, backward of `tensor_core_linear`):
 *   dx[m, k] = (input_mask[m] && output_mask[m]) ? sum_n dy[m, n] weight[n, k] : 0        (one BF16 rounding)
 * dy bf16 [rows, out_features], weight bf16 [out_features, in_features] as in ms_linear_forward (read in place, no
 * transposed copy), masks as there or NULL, dx bf16 [rows, in_features].  Envelope: out_features a multiple of 64,
 * in_features a multiple of 128, 16-byte aligned pointers; otherwise MS_ERR_LINEAR_SHAPE.
 */
int ms_linear_input_grad(int64_t rows, int32_t in_features, int32_t out_features, const void* dy, const void* weight,
                         const uint8_t* input_mask, const uint8_t* output_mask, void* dx, void* stream);

/*
 * Weight and bias gradients of the projection in one pass over dy and x (the reference's fused dW + db GEMM,
 * csrc/ball/binding.cpp:114-196):
 *   dweight[n, k] = sum_m dy[m, n] x[m, k]        dbias[n] = sum_m dy[m, n]        (FP32 sums and results)
 * x bf16 [rows, in_features], dy bf16 [rows, out_features], dweight f32 [out_features, in_features], dbias f32
 * [out_features] or NULL.  The rows are split over several CTAs per output tile; the partial tiles go through
 * `workspace` (ms_linear_weight_grad_workspace bytes, 16-byte aligned) and are added in a fixed order, so the result
 * is the same bits on every run.  No row masks: mask the operands first.  Envelope: in_features and out_features
 * multiples of 128; otherwise MS_ERR_LINEAR_SHAPE (and a workspace size of 0).
 */
size_t ms_linear_weight_grad_workspace(int64_t rows, int32_t in_features, int32_t out_features);
int ms_linear_weight_grad(int64_t rows, int32_t in_features, int32_t out_features, const void* x, const void* dy,
                          float* dweight, float* dbias, void* workspace, size_t workspace_bytes, void* stream);

/* Bytes of scratch the stats/compact calls need for this shape (partials of the token
 * reduction and backward intermediates).  Same workspace serves forward and backward; it must be
 * 16-byte aligned. */
size_t ms_workspace_bytes(const ms_shape* shape);

/* Number of floats in the packed, reduced forward statistics (per rank):
 * B*H*(r*r + r*d).  Backward: B*H*(r*d + 1).  Used for the sequence-parallel all-reduce. */
size_t ms_packed_stats_floats(const ms_shape* shape, int backward);

/*
 * Per-head core: eta, eta_slope, F.  Replaces `complement`, `core_forward`, `compact_lu`,
 * `compact_getrs` (memsolve/ball/cuda.py:2798-2814; csrc/ball/solvers.cuh:227-560).
 * Only tape->eta, eta_slope, core_map, core_info are written.
 */
int ms_core_forward(const ms_shape* shape, const float* base_raw, const float* eta_raw,
                    const ms_tape* tape, void* stream);

/*
 * Token reduction G = A^T A / n, Q = A^T rot(C) / sqrt(n).
 * Writes per-chunk partial sums into `workspace`.  If `packed` is non-null the partials are
 * also summed (fixed order) and scaled into packed[B*H][r*r + r*d] (G then Q per system) --
 * the buffer a sequence-parallel caller all-reduces before ms_compact_forward.
 */
int ms_stats_forward(const ms_shape* shape, const void* projected, const float* cos,
                     const float* sin, const float* counts, void* workspace,
                     size_t workspace_bytes, float* packed, void* stream);

/*
 * ms_stats_forward for callers that have no way to hand over scratch memory.  (This entry point has
 * no counterpart in the reference, whose Python layer always allocates its partial buffers itself.)
 *
 * Who needs it: code that drives the kernels from a place where device allocation is off the
 * table -- a plugin running inside a host application that owns the allocator and hands out only
 * the input and output buffers, a real-time or signal-handler-like context where cudaMalloc's
 * implicit synchronisation is not acceptable, or a caller replaying fixed buffers that cannot grow
 * a workspace after start-up.  Such a caller still passes `projected`, the tables, `counts` and the
 * output `packed`; the per-chunk partial sums go to a buffer that is part of the library image
 * (MS_STATIC_SCRATCH_FLOATS floats, 16 MiB on every GPU that loads the library, for the life of the
 * process).  The call performs no cudaMalloc/cudaFree and calls no allocating library routine.
 *
 * Result: packed[B*H][r*r + r*d] exactly as ms_stats_forward writes it with a non-null `packed`
 * (same kernels, same summation order, so bit-identical).  `packed` must not be null.
 *
 * Limits and rules:
 *  - shapes whose partial sums exceed the built-in buffer return MS_ERR_STATIC_SCRATCH and launch
 *    nothing (one sequence of 32768 tokens with 12 heads needs 3.7 MB at rank 32 and 9.8 MB at rank 64);
 *  - the first call on each device looks up the buffer's device address (cudaGetSymbolAddress, with
 *    that device current) and keeps it; make that first call before starting any stream capture;
 *  - all calls on a device share the one buffer: two calls whose kernels can overlap on the GPU
 *    (different streams, or graphs launched concurrently) race on it -- serialise them.  The buffer
 *    keeps the previous call's partial sums, which is harmless because every partial the new grid
 *    reads is first written in full by that grid.
 */
int ms_stats_forward_static(const ms_shape* shape, const void* projected, const float* cos,
                            const float* sin, const float* counts, float* packed, void* stream);

/*
 * Per (b,h): T, Z, W from the statistics.  `packed` null: read the partials left in
 * `workspace` by ms_stats_forward (reduced here, fixed order).  `packed` non-null: read the
 * already reduced + scaled statistics from it.  Needs tape->eta and tape->core_map
 * (ms_core_forward).  Writes tape->inverse, state, coeff.
 */
int ms_compact_forward(const ms_shape* shape, const float* counts, const void* workspace,
                       size_t workspace_bytes, const float* packed, const ms_tape* tape,
                       void* stream);

/* mixed = eta*C + rot^-1(A_raw W)/sqrt(n).  Reads tape->eta, tape->coeff. */
int ms_readout(const ms_shape* shape, const void* projected, const float* cos, const float* sin,
               const float* counts, const ms_tape* tape, void* mixed, void* stream);

/* ms_readout that also writes its results before the BF16 rounding (mixed_f32: FP32 [B, N, H*d]); test
 * instrument like ms_token_backward_debug below, same shape envelope and status codes. */
int ms_readout_debug(const ms_shape* shape, const void* projected, const float* cos, const float* sin,
                     const float* counts, const ms_tape* tape, void* mixed, float* mixed_f32, void* stream);

/*
 * Readout for a sequence with no more tokens than the rank (N <= r), after ms_mix_forward on the same shape:
 * mixed = rot^-1(eta S^-1 rot(C) + A_raw Wc / sqrt(n)) with S = I_N + A_raw A_raw^T / n, the token-space form of
 * the eta term (reference: memsolve/ball/cuda.py:3230-3926, its `short_*` kernels).  For such shapes
 * ms_mix_forward leaves the core part Wc = T^T F Z in tape->coeff (not T^T (F - eta I) Z), which is what this
 * entry point and ms_mix_backward expect; ms_readout on that tape would miss the eta term.  Other shapes:
 * MS_ERR_INVALID_ARGUMENT.
 */
int ms_readout_short(const ms_shape* shape, const void* projected, const float* cos, const float* sin,
                     const float* counts, const ms_tape* tape, void* mixed, void* stream);

/*
 * Whole forward on one rank: core + stats + compact + readout (no collective).  With tokens <= rank the eta
 * term is evaluated in token space (see ms_readout_short): in rank space it is a difference of nearly equal
 * quantities when the relations are strong.
 */
int ms_mix_forward(const ms_shape* shape, const void* projected, const float* base_raw,
                   const float* eta_raw, const float* cos, const float* sin, const float* counts,
                   void* workspace, size_t workspace_bytes, const ms_tape* tape, void* mixed,
                   void* stream);

/*
 * Adjoint token reduction E = A^T rot(dy)/sqrt(n), de = <dy, C> per (b,h).
 * Same partial / packed convention as ms_stats_forward; packed[B*H][r*d] then [B*H] de.
 */
int ms_stats_backward(const ms_shape* shape, const void* projected, const void* dy,
                      const float* cos, const float* sin, const float* counts, void* workspace,
                      size_t workspace_bytes, float* packed, void* stream);

/*
 * Compact adjoint per (b,h) and per head.  Inputs: E/de (workspace partials or `packed`),
 * the forward tape, base_raw, eta_raw.  Outputs (device, caller-allocated):
 *   gram_grad  bf16 [B,H,2,r,r]   (dG + dG^T) / sqrt(n), split high/residual (n = counts[b], or N)
 *   cross_grad bf16 [B,H,2,r,dp]  dQ, split high/residual
 *   d_base_raw f32  [H,r,r]       (not written in complement mode)
 *   d_eta_raw  f32  [H]
 * `grad_scale` multiplies d_base_raw and d_eta_raw (1/world_size under sequence parallelism,
 * memsolve/ball/cuda.py:3221-3226).  With d_eta_raw == NULL only the per-(b,h) part runs and the
 * per-head sums stay in `workspace` for ms_token_backward_core.
 */
int ms_compact_backward(const ms_shape* shape, const float* counts, void* workspace,
                        size_t workspace_bytes, const float* packed, const ms_tape* tape,
                        const float* base_raw, const float* eta_raw, float grad_scale,
                        void* gram_grad, void* cross_grad, float* d_base_raw, float* d_eta_raw,
                        void* stream);

/* dprojected from the token pass (dA_raw | dC), same packed layout as `projected`. */
int ms_token_backward(const ms_shape* shape, const void* projected, const void* dy,
                      const float* cos, const float* sin, const float* counts,
                      const ms_tape* tape, const void* gram_grad, const void* cross_grad,
                      void* dprojected, void* stream);

/*
 * ms_token_backward that also writes its results before the BF16 rounding: dprojected_f32 is FP32
 * [B, N, H*r + H*d] in the layout of dprojected.  Test instrument for the FP32 accuracy of the token
 * pass on identical BF16 inputs (the reference checks its FP32 path the same way, stage by stage,
 * tests/cuda/test_fast_path.py:2122-2123); it always runs the tcgen05 kernel and returns
 * MS_ERR_DEBUG_SHAPE for shapes that kernel does not take (head_dim != 64, rank 48, unaligned).
 */
int ms_token_backward_debug(const ms_shape* shape, const void* projected, const void* dy,
                            const float* cos, const float* sin, const float* counts,
                            const ms_tape* tape, const void* gram_grad, const void* cross_grad,
                            void* dprojected, float* dprojected_f32, void* stream);

/*
 * Sequence-parallel building blocks that keep the per-head core off the critical path (same work
 * as the separate calls, fewer launches): the statistics launch also computes eta / F in spare
 * CTAs, and the token-backward launch also computes d_base_raw / d_eta_raw in spare CTAs.
 *   ms_stats_forward_core   = ms_core_forward + ms_stats_forward   (cuda.py:2798-2840 + 2121-2247)
 *   ms_token_backward_core  = ms_token_backward + the per-head half of ms_compact_backward; call
 *                             ms_compact_backward first with d_eta_raw == NULL (it then leaves the
 *                             per-head sums H and de in `workspace` and skips the core adjoint).
 */
int ms_stats_forward_core(const ms_shape* shape, const void* projected, const float* base_raw,
                          const float* eta_raw, const float* cos, const float* sin,
                          const float* counts, void* workspace, size_t workspace_bytes, float* packed,
                          const ms_tape* tape, void* stream);
int ms_token_backward_core(const ms_shape* shape, const void* projected, const void* dy,
                           const float* cos, const float* sin, const float* counts,
                           const ms_tape* tape, const void* gram_grad, const void* cross_grad,
                           void* dprojected, const float* base_raw, void* workspace,
                           size_t workspace_bytes, float grad_scale, float* d_base_raw,
                           float* d_eta_raw, void* stream);

/* Whole backward on one rank: adjoint stats + compact adjoint + token pass (no collective). */
int ms_mix_backward(const ms_shape* shape, const void* projected, const void* dy,
                    const float* base_raw, const float* eta_raw, const float* cos,
                    const float* sin, const float* counts, void* workspace,
                    size_t workspace_bytes, const ms_tape* tape, void* gram_grad,
                    void* cross_grad, void* dprojected, float* d_base_raw, float* d_eta_raw,
                    void* stream);

/*
 * Sequence-parallel exchange of the token statistics through peer memory: reduces the per-chunk
 * partials that ms_stats_forward / ms_stats_backward left in `workspace` (pass packed == NULL
 * there), publishes them in this rank's exchange area, waits for the peers and writes the SUM over
 * all ranks, added in rank order (bit-identical on every rank), to `packed` in the layout of
 * ms_packed_stats_floats.  It replaces pack + all-reduce + unpack of the collective path: the
 * reference issues one NCCL all-reduce here (integrations/distributed.py:47-50, called from
 * memsolve/ball/cuda.py:3165-3215).
 *
 * areas[r], r < world_size <= 8: device address, valid on THIS GPU, of rank r's exchange area
 * (peer-accessible memory of `area_bytes` bytes, e.g. one symmetric-memory allocation per rank;
 * same size on all ranks; >= ms_exchange_area_bytes(shape); 16-byte aligned).  The areas must be
 * zero before the first call and must only be touched by this function afterwards; every rank
 * has to make the same sequence of calls.  A peer that does not arrive within the limit of
 * ms_set_peer_wait_ms sets the device error word (ms_device_error) and turns the affected sums into
 * NaN instead of hanging the GPU.  Only plain peer loads and
 * stores are used.
 */
size_t ms_exchange_area_bytes(const ms_shape* shape);
int ms_stats_exchange(const ms_shape* shape, int backward, const void* workspace,
                      size_t workspace_bytes, const float* counts, void* const* areas,
                      size_t area_bytes, int world_size, int rank, float* packed, void* stream);

/*
 * In-place SUM of `count` FP32 values (count a multiple of 4, `values` 16-byte aligned) over the
 * ranks through peer memory, bit-identical on every rank: reduce-scatter and all-gather in one
 * kernel with plain peer loads, two flag rounds.  It serves the SUM of the replicated parameters'
 * gradients that the reference does with one NCCL all-reduce (`SequenceParallel.reduce_gradients_`,
 * integrations/distributed.py:77-99).  `areas` as for ms_stats_exchange, but areas of their own
 * (the two functions lay their areas out differently): ms_peer_sum_area_bytes(count) bytes or
 * more, the same size on all ranks, zero before the first call.
 */
size_t ms_peer_sum_area_bytes(size_t count);
int ms_peer_sum(float* values, size_t count, void* const* areas, size_t area_bytes, int world_size,
                int rank, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MEMSOLVE_B200_H_ */
