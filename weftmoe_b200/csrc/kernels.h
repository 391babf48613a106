// Internal C++ interface between the host runtime (runtime.cu, the C ABI) and the kernel
// translation units.  Nothing here is exported; the public surface is include/weftmoe_b200.h.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "route.h"
#include "status.h"

namespace wm {

constexpr int kMaxPeers = 8;

// ------------------------------------------------------------------ error plumbing
void set_error(const char* fmt, ...);
const char* last_error();
// Process-wide count of kernels this library has launched (read through wm_launch_count()).
void count_launch(int n = 1);
long long launch_count();
// Kernel choice override for tests and A/B runs: -1 automatic, 0 one-CTA kernel, 1 CTA-pair kernel.
void force_gemm_pairs(int mode);

#define WM_CUDA(expr)                                                                 \
  do {                                                                                \
    cudaError_t e_ = (expr);                                                          \
    if (e_ != cudaSuccess) {                                                          \
      ::wm::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e_), __FILE__, \
                      __LINE__);                                                      \
      return 3;                                                                       \
    }                                                                                 \
  } while (0)

// Function attributes belong to a device: opt a kernel in to `bytes` of dynamic shared memory once per
// device of this process (`done` is one static table per kernel instantiation).
struct PerDeviceOnce {
  bool done[64] = {};
};
template <class Kernel>
inline int opt_in_dynamic_smem(Kernel kernel, int bytes, PerDeviceOnce& once) {
  int device = 0;
  WM_CUDA(cudaGetDevice(&device));
  if (device < 0 || device >= 64 || !once.done[device]) {
    WM_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    if (device >= 0 && device < 64) once.done[device] = true;
  }
  return 0;
}

// ------------------------------------------------------------------ tensor maps
// 2-D BF16 (elem_bytes = 2) or 8-bit (elem_bytes = 1) row-major tensor, 128-byte swizzle.
// box_inner * elem_bytes must be 128.  Returns 0 on success.
int make_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner, uint64_t outer,
                 uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer);

// ------------------------------------------------------------------ grouped GEMM launchers
struct Schedule {
  const int* split;            // device [kSplitWords]: tile / pair / row chunk boundaries (route.h)
  const int* tile_group;       // device [max tiles]
  const int* group_row_start;  // device [groups + 1]
  int groups;
  int row_capacity;            // rows addressable in the row-indexed operands
  const int* pair_tiles;       // device [2 * pairs]: CTA-pair work items (two tiles of one expert)
  bool many_rows_per_expert;   // host estimate: experts average >= 1024 rows (long K loops, few odd tiles)
  int chunk;                   // which chunk of the M-grouped work to run (kWhole = all of it)
  const int* group_live_rows = nullptr;  // device [groups], optional: unpadded rows per expert (K-grouped)
  const int* group_order = nullptr;      // device [groups], optional: experts by descending rows (K-grouped walk)
};

struct PushTarget {
  __nv_bfloat16* mailbox[kMaxPeers];
  const int* origin;
  int cap;
  int top_k;
};

// FC1: u[rows, I] = swiglu(x[rows, H] * w1[e][2I, H]^T) * prob ; ab optional [rows, 2I].
int launch_fc1(const Schedule& s, const __nv_bfloat16* x, const __nv_bfloat16* w1, __nv_bfloat16* u,
               __nv_bfloat16* ab, const float* row_prob, int hidden, int inter, int* status,
               int sms, cudaStream_t stream);
// M-grouped, B K-major: out[rows, n] = a[rows, k] * b[e][n, k]^T  (store) or pushed to mailboxes.
int launch_mgrouped_nt(const Schedule& s, const __nv_bfloat16* a, const __nv_bfloat16* b,
                       __nv_bfloat16* out, const PushTarget* push, int n, int k, int* status,
                       int sms, cudaStream_t stream);
// M-grouped, B MN-major: out[rows, n] = a[rows, k] * b[e][k, n]  (store) or pushed to mailboxes.
int launch_mgrouped_nn(const Schedule& s, const __nv_bfloat16* a, const __nv_bfloat16* b,
                       __nv_bfloat16* out, const PushTarget* push, int n, int k, int* status,
                       int sms, cudaStream_t stream);
// dU = dY rows * W2[e] (B MN-major, N = I, K = H) with the SwiGLU backward fused into the epilogue of
// the one-CTA kernel (eight epilogue warps): writes U [rows, I], dAB [rows, 2I] and the dprob partials
// [I / 128][row_capacity] instead of dU.  Needs I % 256 == 0; returns -1 (nothing launched) where the
// CTA-pair kernel is the better choice for the shape, and the caller runs the two-kernel form.
int launch_du_swiglu_backward(const Schedule& s, const __nv_bfloat16* dy_rows, const __nv_bfloat16* w2,
                              const __nv_bfloat16* ab, const float* row_prob, __nv_bfloat16* u,
                              __nv_bfloat16* dab, float* dprob_part, int inter, int hidden, int* status,
                              int sms, cudaStream_t stream);
// K-grouped: out[e][m, n] = sum over the expert's rows r of a[r, m] * b[r, n]; out is BF16, or FP32
// (the accumulators unrounded) with out_is_f32.
int launch_kgrouped_tn(const Schedule& s, const __nv_bfloat16* a, const __nv_bfloat16* b,
                       void* out, int m, int n, int* status, int sms,
                       cudaStream_t stream, bool out_is_f32 = false);

}  // namespace wm
