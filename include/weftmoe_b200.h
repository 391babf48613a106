/* weftmoe_b200 — C ABI of the B200 (sm_100a) routed-MoE expert operator.
 *
 * Plain C linkage, plain pointers and sizes, no C++ or torch types.  Every function returns an
 * int status (WM_OK = 0); wm_last_error() returns the calling thread's last message.  Device
 * pointers are CUDA device addresses on the current device; `stream` is a cudaStream_t passed as
 * void*.  Together these calls replace the native object behind the reference's Python Tensor
 * API (`TensorRuntime.native`, weftmoe/runtime.py:277-464; its pybind surface is
 * src/python/runtime.cpp:870-953 and, on Blackwell, the Python class weftmoe/blackwell.py:51-178).
 *
 * Tensor contract (weftmoe/runtime.py:243-275, docs/usage.md:63-69):
 *   x[T,H] bf16, routes[T,K] int32 global expert ids (ids outside [0,E) mean "no route"),
 *   gates[T,K] fp32, w1[E_local,2I,H] bf16 (rows 0..I-1 gate, I..2I-1 up), w2[E_local,H,I] bf16,
 *   all contiguous device memory; y[T,H] bf16; dx bf16, dgates[T,K] fp32, dw1/dw2 bf16.
 * Expert e lives on rank e / (E / world) (src/python/runtime.cpp:175-176).
 */
#ifndef WEFTMOE_B200_H_
#define WEFTMOE_B200_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define WM_API __attribute__((visibility("default")))
#else
#define WM_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes.  Contract violations (-> ValueError) are distinct from runtime failures
 * (-> RuntimeError), as in the reference's NotifyErrorCode (include/weftmoe/api/errors.hpp:12-31). */
enum {
  WM_OK = 0,
  WM_ERR_INVALID = 2,  /* argument / shape / alignment contract violated                       */
  WM_ERR_CUDA = 3,     /* a CUDA call failed                                                    */
  WM_ERR_TIMEOUT = 4,  /* a bounded device wait ran out (reference: TransportTimeout)           */
  WM_ERR_ROUTE = 5,    /* reserved: route id rejected (reference: ExpertOutOfRange)             */
  WM_ERR_CAPACITY = 6, /* rows or tokens exceed the prepared capacity (CapacityExceeded)        */
  WM_ERR_STATE = 7     /* call not valid in this state (runtime closed, peers not imported ...) */
};

WM_API const char* wm_last_error(void);

/* ------------------------------------------------------------------------------------------
 * Runtime: one persistent workspace per EP group member.
 * Replaces Runtime.__init__ / BlackwellRuntime.__init__ (src/python/runtime.cpp:113-240,
 * weftmoe/blackwell.py:54-82) and the symmetric workspace (weftmoe/blackwell_cutlass.py:179-218,
 * src/cuda/blackwell/fused_host.cpp:32-55). */
typedef struct wm_runtime wm_runtime;

typedef struct wm_config {
  int32_t rank;         /* this process' rank in the EP group                                   */
  int32_t world;        /* EP group size: 1, 2, 4 or 8                                          */
  int32_t experts;      /* global expert count E, E % world == 0                                */
  int32_t top_k;        /* 1..32                                                                */
  int32_t hidden;       /* H, multiple of 256                                                   */
  int32_t intermediate; /* I, multiple of 128                                                   */
  int32_t max_tokens;   /* token capacity of this rank                                          */
  int32_t max_rows;     /* routed rows this rank may receive as an expert owner                 */
  int32_t training;     /* non-zero: backward buffers are allocated                             */
  int32_t reserved;     /* precision: 0 BF16, 1 blockwise FP8 (E4M3), 2 NVFP4 (intermediate % 256 == 0)  */
} wm_config;

typedef struct wm_sizes {
  int64_t arena_bytes;   /* peer-mapped arena                                                   */
  int64_t scratch_bytes; /* private device scratch                                              */
  int64_t tape_bytes;    /* bytes the caller must provide per saved forward (training cache)    */
  int32_t row_capacity;  /* padded row capacity of the owner-side buffers                       */
  int32_t ipc_handle_bytes;
} wm_sizes;

/* Allocates the arena and scratch on the current device (cudaMalloc).  Not capturable. */
WM_API int wm_runtime_create(const wm_config* config, wm_runtime** out);
WM_API int wm_runtime_sizes(const wm_runtime* rt, wm_sizes* out);
/* CUDA-IPC handle of this rank's arena (ipc_handle_bytes bytes).  The caller moves the handles
 * between ranks (the Python layer uses all_gather_object, as weftmoe/runtime.py:191-196 does for
 * the bootstrap id; the reference's own IPC exchange is src/cuda/activation_transport.cu:1355-1498). */
WM_API int wm_runtime_export_handle(wm_runtime* rt, void* handle_out, size_t bytes);
/* handles: world * ipc_handle_bytes bytes, rank-major.  world == 1 needs no call. */
WM_API int wm_runtime_import_peers(wm_runtime* rt, const void* handles, size_t bytes);
/* Collective teardown step: unmap peers (reference: retire_peer_mappings, weftmoe/runtime.py:450-464). */
WM_API int wm_runtime_retire_peers(wm_runtime* rt);
WM_API int wm_runtime_destroy(wm_runtime* rt);

/* Forward (reference: BlackwellRuntime._run, weftmoe/blackwell.py:84-127; fused kernel
 * src/cuda/blackwell/fused/impls/routed_bf16.cuh:22-1312).  Enqueues on `stream`, no host sync.
 * tape: NULL for inference, else tape_bytes of device memory that receives the training cache
 * (reference: checkpoint(), weftmoe/blackwell_backward.py:29-52).  All EP ranks must call in the
 * same order. */
WM_API int wm_forward(wm_runtime* rt, const void* x, const int32_t* routes, const float* gates,
                      const void* w1, const void* w2, int32_t tokens, void* y, void* tape,
                      void* stream);

/* Backward (reference: gradients(), weftmoe/blackwell_backward.py:252-285).  `tape` is the cache a
 * previous wm_forward filled for the same `tokens`; w1/w2 are the same weights. */
WM_API int wm_backward(wm_runtime* rt, const void* tape, const void* dy, const void* w1,
                       const void* w2, int32_t tokens, void* dx, float* dgates, void* dw1, void* dw2,
                       void* stream);

/* Quantised inference forward (reference: inference_fp8 / forward_fp8 without a tape,
 * weftmoe/runtime.py:303-352,387-415; NVFP4 inference, weftmoe/nvfp4.py:252-278).  The runtime must have
 * been created with precision 1 or 2.  x stays BF16 and is quantised online at the source rank
 * (1 x 128 power-of-two FP32 scales, or block-16 E4M3 scales with layer scale x_scale); weights are
 * pre-quantised and their scale factors pre-packed in 512-byte tensor-core chunks:
 *   FP8   w1 [E_local][2I][H] E4M3, w1_sf = wm_fp8_pack_weight_scales(scales [E_local*2I/128][H/128]);
 *   NVFP4 w1 [E_local][2I][H/2],    w1_sf = chunked scales of wm_nvfp4_quantize over [E_local*2I, H];
 * w2 likewise over [E_local][H][I].  NVFP4: accumulators are scaled by x_scale*w1_scale and rounded to
 * BF16, u = silu(a)*b*prob is quantised with u_scale, FC2 is scaled by u_scale*w2_scale. */
typedef struct wm_quant_weights {
  const void* w1;
  const void* w1_sf;
  const void* w2;
  const void* w2_sf;
  float x_scale, w1_scale, u_scale, w2_scale; /* NVFP4 layer scales; ignored for FP8 */
  float dy_scale, dab_scale;                   /* NVFP4 backward only: layer scales of dY and d(gate,up) */
  /* Blockwise FP8 only, optional (NULL = quantise the BF16 source online): the source rows already
   * quantised 1 x 128 by wm_fp8_quantize (E4M3 bytes [tokens][H] and FP32 scales [tokens][H/128]); x in
   * wm_forward_quantized, dY in wm_backward_quantized.  The BF16 pointer is then ignored and the result has
   * the bits of the online path (reference: FP8Tensor sources, tests/torchrun_fp8.py:133-157). */
  const void* source_q;
  const float* source_scales;
  /* Blockwise FP8 only, optional (NULL = every block scale of that weight is a power of two): the FP32
   * 128 x 128 block scales of w1 / w2 as given, [E_local * rows / 128][K / 128], for weights whose scales carry
   * mantissas (imported checkpoints, reference: tests/torchrun_fp8.py:235-255).  The bytes are used as they
   * are: the MMA applies each scale's exponent (the packed chunks) and the kernel promotes every K128 block
   * in FP32 by the mantissas (reference: src/cuda/fp8/gemm.cuh:68-70). */
  const float* w1_scales;
  const float* w2_scales;
  /* wm_backward_quantized, blockwise FP8 only: non-zero = dw1 / dw2 are FP32 buffers and receive the
   * unrounded FP32 accumulators (FP32 master parameters; reference: weight_grad_dtype of forward_fp8,
   * weftmoe/runtime.py:303-352); zero = BF16. */
  int32_t wgrad_f32;
} wm_quant_weights;
WM_API int wm_forward_quantized(wm_runtime* rt, const void* x, const int32_t* routes, const float* gates,
                                const wm_quant_weights* weights, int32_t tokens, void* y, void* tape,
                                void* stream);
/* Backward of the quantised layer; `tape` was filled by wm_forward_quantized on a runtime created with
 * training = 1 and the same precision.
 *
 * NVFP4 (reference: weftmoe/nvfp4_backward.py:59-112): `transposed` holds W1^T [E_local][H][2I/2] and
 * W2^T [E_local][I][H/2] quantised along their new last axis with the same weight scales, plus all six
 * layer scales.  dY rows are quantised along H (dy_scale) for dU = dY W2, dAB rows along 2I (dab_scale)
 * for dX = dAB W1; for the weight gradients dAB, the saved X (dequantised NVFP4 rows), dY and the
 * recomputed U are re-quantised block-16 ALONG THE ROWS (each contraction's reduction axis) with
 * dab_scale, x_scale, dy_scale, u_scale, and contracted per expert.  SwiGLU backward runs in FP32 on the
 * saved BF16 gate/up rows.  Outputs as in wm_backward.
 *
 * Blockwise FP8 (reference: forward_fp8 + backward, weftmoe/runtime.py:303-367; dataflow
 * docs/usage.md:216-252).  `tape` (tape_bytes, same size as the BF16 tape) was filled by
 * wm_forward_quantized on an FP8 runtime created with training = 1; `transposed` holds the prepared
 * W1^T [E_local][H][2I] and W2^T [E_local][I][H] bytes with their packed scale chunks.  dY is quantised
 * 1 x 128 at the source; dU and dX run in FP8; dW1/dW2 are BF16 contractions of the dequantised saved X
 * and dY rows (a stated simplification: no column-wise re-quantisation), returned as BF16. */
WM_API int wm_backward_quantized(wm_runtime* rt, const void* tape, const void* dy,
                                 const wm_quant_weights* transposed, int32_t tokens, void* dx,
                                 float* dgates, void* dw1, void* dw2, void* stream);
/* scales [rows/128][kblocks] FP32 (128 x 128 blocks of a [rows][K] weight, experts stacked along rows)
 * -> UE8M0 chunks [rows/128][kblocks][512 bytes]. */
WM_API int wm_fp8_pack_weight_scales(const float* scales, int32_t rows, int32_t kblocks, void* out,
                                     void* stream);

/* Reads (and clears) the device status word; synchronises `stream`.  *code receives a WM_ERR_* value
 * (reference: TransportDeviceStatus surfaced through profile_inference, src/python/runtime.cpp:295-331). */
WM_API int wm_status_poll(wm_runtime* rt, int32_t* code, void* stream);

/* ------------------------------------------------------------------------------------------
 * Instrumentation (reference: always-on device clocks surfaced as profile_inference /
 * BackwardMegaKernelTimings, src/python/runtime.cpp:295-331, include/weftmoe/cuda/backward.hpp:48-61).
 * wm_launch_count: kernels this library launched in this process so far.
 * Timing: when enabled, every forward/backward brackets each stage with a CUDA event pair on the
 * caller's stream; wm_runtime_read_timing waits for the recorded events and returns, per stage,
 * the summed milliseconds and the number of calls (arrays of wm_stage_count() entries). */
WM_API long long wm_launch_count(void);
WM_API int wm_stage_count(void);
WM_API const char* wm_stage_name(int stage);
WM_API int wm_runtime_enable_timing(wm_runtime* rt, int enable);
WM_API int wm_runtime_read_timing(wm_runtime* rt, double* total_ms, long long* calls, int reset);

/* ------------------------------------------------------------------------------------------
 * Stand-alone route planning for tests and tools (reference: build_rank_local_histogram /
 * materialize_rank_metadata, include/weftmoe/api/notify_dispatch.hpp:49-114).  Two phases, so a
 * single GPU can play every rank in turn:
 *   phase 0 (local): fills sorted_slot, sorted_expert, local_offset-independent arrays and row
 *           `rank` of count_matrix[world*experts];
 *   phase 1 (global): with every row of count_matrix present, fills the remaining outputs.
 * All pointers are device pointers; the call allocates and frees temporary device scratch. */
typedef struct wm_route_out {
  int32_t* sorted_slot;   /* [T*K] original slot at combine position j                          */
  int32_t* sorted_expert; /* [T*K] expert at combine position j, -1 = no route                  */
  int32_t* local_offset;  /* [T*K] by original slot; -1 = no route                              */
  int32_t* dst_rank;      /* [T*K]                                                              */
  int32_t* dst_row;       /* [T*K] canonical (unpadded) row inside the owner                    */
  int32_t* dst_prow;      /* [T*K] physical row in the owner's 128-padded layout                */
  int32_t* expert_total;  /* [E]                                                                */
  int32_t* expert_base;   /* [E] unpadded first row inside the owner                            */
  int32_t* expert_pbase;  /* [E] padded first row inside the owner                              */
  int32_t* padded_start;  /* [E/world + 1] this rank as owner                                   */
  int32_t* tile_group;    /* [row_capacity/128]                                                 */
  int32_t* num_tiles;     /* [1]                                                                */
  int32_t* padded_rows;   /* [1]                                                                */
  int32_t* dst_primary;   /* [T*K] optional (NULL = skip): dst_prow of the token's first route (lowest
                             combine position) to the same owner rank; equal to dst_prow for that route.
                             At world > 1 only such rows are pulled over NVLink, the others are copied
                             from them inside the owner.  -1 = no route                               */
} wm_route_out;

WM_API int wm_route_plan(int32_t phase, int32_t world, int32_t rank, int32_t experts, int32_t top_k,
                         int32_t tokens, int32_t cap, int32_t row_capacity, const int32_t* routes,
                         int32_t* count_matrix, const wm_route_out* out, void* stream);

/* ------------------------------------------------------------------------------------------
 * Blockwise FP8 (E4M3) quantisation.  Replaces the reference's fp8 bindings
 * (src/python/fp8.hpp:61-174: fp8_quantize, fp8_quantize_weight, fp8_transpose_weight) with the same
 * byte and scale results (src/cuda/fp8/quantization.cuh:35-81): power-of-two FP32 scales, zero block
 * -> 1, non-finite block -> NaN scale.  dtype: 0 = BF16, 1 = FP32 input.  x is [batches][rows][cols].
 * wm_fp8_quantize: block_rows 1 (1 x 128 along the last dimension) or 128 (128 x 128); transpose != 0
 *   quantises x^T.  Output q is [batches][m][ceil128(k)] bytes (padding bytes written), scales
 *   [batches][ceil(m / block_rows)][ceil(k / 128)] with (m, k) = transpose ? (cols, rows) : (rows, cols).
 * wm_fp8_quantize_weight: one read of each 128 x 128 block, emits W (q, s) and W^T (qt, st) with the
 *   same bytes and scales.  Operands must not alias; FP8 outputs must be 4-byte aligned.
 * wm_fp8_transpose_weight: byte transpose of a 128 x 128-quantised weight, bits preserved. */
WM_API int wm_fp8_quantize(const void* x, int32_t dtype, int32_t batches, int32_t rows, int32_t cols,
                           int32_t block_rows, int32_t transpose, void* q, float* scales, void* stream);
WM_API int wm_fp8_quantize_weight(const void* x, int32_t dtype, int32_t batches, int32_t rows,
                                  int32_t cols, void* q, float* s, void* qt, float* st, void* stream);
WM_API int wm_fp8_transpose_weight(const void* q, const float* s, int32_t batches, int32_t rows,
                                   int32_t cols, void* qt, float* st, void* stream);

/* Diagnostic FP8 GEMM out[m,n] (+)= A[m,k] * B[n,k]^T on the block-scaled tensor-core path
 * (reference: fp8_gemm, weftmoe/fp8.py:129-153).  aq/bq: E4M3 bytes with rows padded to ceil128(k);
 * as/bs: FP32 power-of-two scales per [block_rows x 128] block; out FP32 or BF16; accumulate needs an
 * existing FP32 output.  Synchronises `stream`; allocates temporary device memory. */
WM_API int wm_fp8_gemm(const void* aq, const float* as, const void* bq, const float* bs, void* out,
                       int32_t m, int32_t n, int32_t k, int32_t a_block_rows, int32_t b_block_rows,
                       int32_t out_is_f32, int32_t accumulate, void* stream);

/* ------------------------------------------------------------------------------------------
 * NVFP4 (E2M1 with an E4M3 scale per 16 elements and an FP32 layer scale).
 * wm_nvfp4_quantize: x BF16 [rows][cols] -> data [rows][cols/2] bytes (even element in the low nibble)
 *   and scale bytes, row-major [rows][cols/16] (chunked = 0; reference activation layout,
 *   weftmoe/nvfp4.py:61-63) or in 512-byte tensor-core chunks (chunked = 1; reference weight/backward
 *   layout, weftmoe/nvfp4.py:58-60, src/cuda/blackwell/nvfp4_quantize.cuh:48-51).  Same results as the
 *   reference's `_encode_row` (weftmoe/nvfp4.py:14-31) / `quantize_blocks` (nvfp4_quantize.cuh:53-125).
 * wm_nvfp4_gemm: diagnostic out[m,n] = alpha * A[m,k] * B[n,k]^T on the block-scaled tensor-core path
 *   with row-major scale bytes (reference oracle: tests/torchrun_sm100_nvfp4.py:30-33). */
WM_API int wm_nvfp4_quantize(const void* x, int32_t rows, int32_t cols, float layer_scale, void* data,
                             void* scales, int32_t chunked, void* stream);
WM_API int wm_nvfp4_gemm(const void* a, const void* a_sf, const void* b, const void* b_sf, void* out,
                         int32_t m, int32_t n, int32_t k, float alpha, int32_t out_is_f32, void* stream);

/* Route planning for callers that must not allocate.  It has no counterpart in the reference.
 * Same arguments, outputs (dst_primary included) and phases as wm_route_plan, but no
 * cudaMalloc/cudaFree: the temporaries live in a fixed 1 MiB __device__ array inside the library
 * (held by every GPU that loads it until the process exits).  Meant for hosts whose own pool owns all free HBM, and for latency-critical
 * paths where cudaMalloc's device-wide synchronisation would stall every stream.
 * Limits: tokens * top_k <= 131072, experts <= 512, row_capacity <= 262144; larger requests return
 * WM_ERR_CAPACITY with a message that names the limit.  The first call on a device looks up the
 * array's device address (cudaGetSymbolAddress); make that first call before any stream capture.
 * Every call, like wm_route_plan, ends by synchronising `stream` and reading the device status word
 * on the host.  All calls on a device share the array, so calls whose GPU work overlaps race:
 * serialise them. */
WM_API int wm_route_plan_noalloc(int32_t phase, int32_t world, int32_t rank, int32_t experts,
                                 int32_t top_k, int32_t tokens, int32_t cap, int32_t row_capacity,
                                 const int32_t* routes, int32_t* count_matrix, const wm_route_out* out,
                                 void* stream);

/* ------------------------------------------------------------------------------------------
 * Serving-adapter helpers (reference: the SGLang staging kernels sanitize_routes / stage_inputs /
 * scatter_output, weftmoe/_sglang_kernels.py:21-99).  Every rank holds the same [tokens][hidden] BF16
 * activations and [tokens][top_k] ids / FP32 weights; rank r works on rows [start, start + valid_rows).
 * wm_stage_inputs: staged_x[local_rows][hidden], routes[local_rows][top_k] int32, gates FP32 = that slice,
 *   padded with zero rows whose routes are -1; negative ids stay -1 ("no route") and get gate 0.  Strides
 *   are in elements; ids are int32 or (ids_are_int64) int64.
 * wm_scatter_output: result[tokens][hidden] = zeros with rows [start, start + valid_rows) = output[0..). */
WM_API int wm_stage_inputs(const void* x, int64_t x_row_stride, const void* ids, int32_t ids_are_int64,
                           int64_t id_row_stride, const float* weights, int64_t weight_row_stride,
                           int32_t start, int32_t valid_rows, int32_t local_rows, int32_t hidden,
                           int32_t top_k, void* staged_x, int32_t* routes, float* gates, void* stream);
WM_API int wm_scatter_output(const void* output, int32_t tokens, int32_t start, int32_t valid_rows,
                             int32_t hidden, void* result, void* stream);

/* Diagnostic: one grouped GEMM on caller buffers (synchronises `stream`).
 * kind 0: out[rows,n]   = a[rows,k] * b[g][n,k]^T          (FC2 form)
 * kind 1: out[rows,n]   = a[rows,k] * b[g][k,n]            (dU / dX form)
 * kind 2: out[g][m,n]   = sum_r a[r,m] * b[r,n]            (dW form; k_or_m = m)
 * kind 3: out=u[rows,n] = swiglu(a[rows,k] * b[g][2n,k]^T) * row_prob, aux_out = ab[rows,2n] or NULL
 * group_rows_host[g] = rows of expert g (multiples of 128).  Plays the role of the reference's
 * diagnostic fp8_gemm binding (src/python/fp8.hpp:61-174). */
WM_API int wm_debug_grouped_gemm(int kind, const void* a, const void* b, void* out, void* aux_out,
                                 const float* row_prob, const int* group_rows_host, int groups, int n,
                                 int k_or_m, int* status_dev, void* stream);

/* Diagnostic: pin the grouped-GEMM kernel choice for this process: -1 automatic (default), 0 the
 * one-CTA kernel, 1 the CTA-pair (cta_group::2) kernel.  No counterpart in the reference, whose
 * tile heuristic lives in weftmoe/blackwell_cutlass.py:80-88. */
WM_API void wm_debug_force_gemm_pairs(int mode);

/* Diagnostics of the bounded cross-rank waits (reference: the transport deadline,
 * ActivationTransportRunOptions.deadline_after -> NotifyErrorCode::TransportTimeout,
 * include/weftmoe/cuda/activation_transport.hpp:169-175, src/cuda/activation_transport/execution.cuh:1243-1250).
 * wm_debug_set_wait_budget: process-wide budget, in SM clock cycles, of every wait on a generation flag
 *   (cycles <= 0 restores the default of about two seconds).  Applies to launches made afterwards.
 * wm_debug_wait_flag: enqueue one flag wait of `rt` on a caller-owned device word: the kernel returns
 *   when *flag_word >= target or when the budget runs out; in that case the runtime's status word is
 *   set and the next wm_status_poll reports WM_ERR_TIMEOUT (and clears it).  Nothing traps or spins on. */
WM_API int wm_debug_set_wait_budget(long long cycles);
WM_API int wm_debug_wait_flag(wm_runtime* rt, const int32_t* flag_word, int32_t target, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* WEFTMOE_B200_H_ */
