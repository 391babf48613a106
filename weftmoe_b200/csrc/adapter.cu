// Serving-adapter helpers: staging of a rank's slice of replicated inputs and the scatter of its result rows.
// Same jobs as the reference's Triton kernels for SGLang (weftmoe/_sglang_kernels.py:21-99: sanitize_routes,
// stage_inputs, scatter_output), as two HBM-bound copy kernels.  Masked top-k entries (negative ids) are legal
// route ids in this library ("no route"), so sanitising only clears their gates.
#include "../../include/weftmoe_b200.h"
#include "kernels.h"

using namespace wm;

namespace {

// One warp per staged row.  Rows below valid_rows copy x[start + row] (16-byte words), their ids (clamped to
// int32, negative -> -1) and gates (0 where the id is negative); the padding rows are zero with routes -1.
template <class Id>
__global__ void stage_inputs_kernel(const __nv_bfloat16* __restrict__ x, long long x_stride,
                                    const Id* __restrict__ ids, long long id_stride,
                                    const float* __restrict__ weights, long long weight_stride, int start,
                                    int valid_rows, int local_rows, int hidden, int top_k,
                                    __nv_bfloat16* __restrict__ staged, int* __restrict__ routes,
                                    float* __restrict__ gates) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int vecs = hidden / 8;
  for (int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < local_rows; row += warps) {
    uint4* dst = reinterpret_cast<uint4*>(staged + static_cast<size_t>(row) * hidden);
    const bool live = row < valid_rows;
    if (live) {
      const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(start + row) * x_stride);
      for (int c = lane; c < vecs; c += 32) dst[c] = src[c];
    } else {
      for (int c = lane; c < vecs; c += 32) dst[c] = make_uint4(0, 0, 0, 0);
    }
    for (int k = lane; k < top_k; k += 32) {
      int id = -1;
      float gate = 0.0f;
      if (live) {
        const Id raw = ids[static_cast<size_t>(start + row) * id_stride + k];
        id = raw < 0 ? -1 : static_cast<int>(raw);
        gate = id >= 0 ? weights[static_cast<size_t>(start + row) * weight_stride + k] : 0.0f;
      }
      routes[static_cast<size_t>(row) * top_k + k] = id;
      gates[static_cast<size_t>(row) * top_k + k] = gate;
    }
  }
}

// result[tokens][hidden] = 0 except rows [start, start + valid_rows) = output[0 .. valid_rows).
__global__ void scatter_output_kernel(const uint4* __restrict__ output, long long first, long long count,
                                      long long total, uint4* __restrict__ result) {
  const long long step = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += step) {
    const long long local = i - first;
    result[i] = (local >= 0 && local < count) ? output[local] : make_uint4(0, 0, 0, 0);
  }
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

extern "C" int wm_stage_inputs(const void* x, int64_t x_row_stride, const void* ids, int32_t ids_are_int64,
                               int64_t id_row_stride, const float* weights, int64_t weight_row_stride,
                               int32_t start, int32_t valid_rows, int32_t local_rows, int32_t hidden,
                               int32_t top_k, void* staged_x, int32_t* routes, float* gates, void* stream_) {
  if (local_rows < 0 || valid_rows < 0 || valid_rows > local_rows || start < 0 || hidden <= 0 || hidden % 8 ||
      top_k < 1 || x_row_stride % 8 || (local_rows > 0 && (!staged_x || !routes || !gates)) ||
      (valid_rows > 0 && (!x || !ids || !weights)) || !aligned16(x) || !aligned16(staged_x)) {
    set_error("wm_stage_inputs: bad argument (hidden and the row stride must be multiples of 8 elements, "
              "rows 16-byte aligned)");
    return WM_ERR_INVALID;
  }
  if (local_rows == 0) return WM_OK;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int blocks = (local_rows + 7) / 8 < 1184 ? (local_rows + 7) / 8 : 1184;
  auto* xs = static_cast<const __nv_bfloat16*>(x);
  auto* out = static_cast<__nv_bfloat16*>(staged_x);
  if (ids_are_int64)
    stage_inputs_kernel<long long><<<blocks, 256, 0, stream>>>(xs, x_row_stride, static_cast<const long long*>(ids),
                                                               id_row_stride, weights, weight_row_stride, start,
                                                               valid_rows, local_rows, hidden, top_k, out, routes, gates);
  else
    stage_inputs_kernel<int><<<blocks, 256, 0, stream>>>(xs, x_row_stride, static_cast<const int*>(ids), id_row_stride,
                                                         weights, weight_row_stride, start, valid_rows, local_rows,
                                                         hidden, top_k, out, routes, gates);
  count_launch();
  WM_CUDA(cudaGetLastError());
  return WM_OK;
}

extern "C" int wm_scatter_output(const void* output, int32_t tokens, int32_t start, int32_t valid_rows,
                                 int32_t hidden, void* result, void* stream_) {
  if (tokens < 0 || start < 0 || valid_rows < 0 || hidden <= 0 || hidden % 8 ||
      static_cast<long long>(start) + valid_rows > tokens || (tokens > 0 && !result) ||
      (valid_rows > 0 && !output) || !aligned16(output) || !aligned16(result)) {
    set_error("wm_scatter_output: bad argument");
    return WM_ERR_INVALID;
  }
  if (tokens == 0) return WM_OK;
  const long long vecs = hidden / 8;
  const long long total = static_cast<long long>(tokens) * vecs;
  const int blocks = static_cast<int>((total + 255) / 256 < 2368 ? (total + 255) / 256 : 2368);
  scatter_output_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      static_cast<const uint4*>(output), static_cast<long long>(start) * vecs,
      static_cast<long long>(valid_rows) * vecs, total, static_cast<uint4*>(result));
  count_launch();
  WM_CUDA(cudaGetLastError());
  return WM_OK;
}
