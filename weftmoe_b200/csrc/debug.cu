// Diagnostic C entry point: run one grouped GEMM variant on caller-provided device buffers.
// It plays the role of the reference's diagnostic fp8_gemm op (src/python/fp8.hpp:61-174):
// a way to check a single contraction against a dense oracle without running the layer.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "../../include/weftmoe_b200.h"
#include "kernels.h"

using namespace wm;

extern "C" int wm_debug_grouped_gemm(int kind, const void* a, const void* b, void* out, void* aux_out,
                                     const float* row_prob, const int* group_rows_host, int groups,
                                     int n, int k_or_m, int* status_dev, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (groups <= 0 || !group_rows_host) {
    set_error("wm_debug_grouped_gemm: groups must be positive");
    return WM_ERR_INVALID;
  }
  std::vector<int> starts(groups + 1, 0), tile_group, pairs;
  for (int g = 0; g < groups; ++g) {
    if (group_rows_host[g] % 128) {
      set_error("wm_debug_grouped_gemm: group rows must be multiples of 128");
      return WM_ERR_INVALID;
    }
    starts[g + 1] = starts[g] + group_rows_host[g];
    const int first = static_cast<int>(tile_group.size()), tiles = group_rows_host[g] / 128;
    for (int t = 0; t < tiles; ++t) tile_group.push_back(g);
    for (int j = 0; j < (tiles + 1) / 2; ++j) {
      pairs.push_back(first + 2 * j);
      pairs.push_back(2 * j + 1 < tiles ? first + 2 * j + 1 : -1);
    }
  }
  const int num_pairs = static_cast<int>(pairs.size() / 2);
  pairs.push_back(-1);
  const int rows = starts[groups];
  const int num_tiles = static_cast<int>(tile_group.size());
  tile_group.push_back(0);
  int *d_num = nullptr, *d_tiles = nullptr, *d_starts = nullptr, *d_pairs = nullptr;
  int split[kSplitWords];
  fill_whole_split(split, num_tiles, num_pairs, rows, groups);
  WM_CUDA(cudaMalloc(&d_pairs, pairs.size() * sizeof(int)));
  WM_CUDA(cudaMemcpyAsync(d_pairs, pairs.data(), pairs.size() * sizeof(int), cudaMemcpyHostToDevice, stream));
  WM_CUDA(cudaMalloc(&d_num, sizeof(split)));
  WM_CUDA(cudaMalloc(&d_tiles, tile_group.size() * sizeof(int)));
  WM_CUDA(cudaMalloc(&d_starts, starts.size() * sizeof(int)));
  WM_CUDA(cudaMemcpyAsync(d_num, split, sizeof(split), cudaMemcpyHostToDevice, stream));
  WM_CUDA(cudaMemcpyAsync(d_tiles, tile_group.data(), tile_group.size() * sizeof(int),
                          cudaMemcpyHostToDevice, stream));
  WM_CUDA(cudaMemcpyAsync(d_starts, starts.data(), starts.size() * sizeof(int),
                          cudaMemcpyHostToDevice, stream));
  int sms = 0, dev = 0;
  WM_CUDA(cudaGetDevice(&dev));
  WM_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  Schedule s{d_num, d_tiles, d_starts, groups, rows, d_pairs, rows >= 1024 * groups, kWhole};
  auto A = static_cast<const __nv_bfloat16*>(a);
  auto B = static_cast<const __nv_bfloat16*>(b);
  auto O = static_cast<__nv_bfloat16*>(out);
  int rc = 0;
  // WM_DEBUG_GEMM_REPEAT=n launches the same GEMM n times (for timing runs of this diagnostic entry).
  const char* repeat_env = std::getenv("WM_DEBUG_GEMM_REPEAT");
  const int repeat = repeat_env ? std::max(1, std::atoi(repeat_env)) : 1;
  for (int it = 0; it < repeat && rc == 0; ++it)
  switch (kind) {
    case 0: rc = launch_mgrouped_nt(s, A, B, O, nullptr, n, k_or_m, status_dev, sms, stream); break;
    case 1: rc = launch_mgrouped_nn(s, A, B, O, nullptr, n, k_or_m, status_dev, sms, stream); break;
    case 2: rc = launch_kgrouped_tn(s, A, B, O, k_or_m, n, status_dev, sms, stream); break;
    case 3:
      rc = launch_fc1(s, A, B, O, static_cast<__nv_bfloat16*>(aux_out), row_prob, k_or_m, n,
                      status_dev, sms, stream);
      break;
    default:
      set_error("wm_debug_grouped_gemm: unknown kind %d", kind);
      rc = WM_ERR_INVALID;
  }
  cudaError_t e = cudaStreamSynchronize(stream);
  cudaFree(d_num);
  cudaFree(d_tiles);
  cudaFree(d_starts);
  cudaFree(d_pairs);
  if (rc) return rc;
  if (e != cudaSuccess) {
    set_error("wm_debug_grouped_gemm: %s", cudaGetErrorString(e));
    return WM_ERR_CUDA;
  }
  return WM_OK;
}

extern "C" const char* wm_last_error(void) { return wm::last_error(); }

extern "C" void wm_debug_force_gemm_pairs(int mode) { wm::force_gemm_pairs(mode); }
