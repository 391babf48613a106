// Blockwise FP8 (E4M3) quantisation for the routed-MoE path.
//
// Numerics contract (reference: src/cuda/fp8/quantization.cuh:35-81, tests/test_fp8.py:20-63):
//   scale = 2^ceil(log2(amax / 448)), never below the smallest normal FP32; an all-zero block
//   has scale 1; a block that holds a non-finite value has a NaN scale (and NaN codes);
//   q = e4m3_rn_satfinite(x * 2^-e) — exact, because the multiplier is a power of two.
//   Blocks are 1 x 128 along K (activations, dY) or 128 x 128 (weights).  The last dimension of
//   the byte tensor is padded to a multiple of 128 with zero bytes.
// All kernels are HBM-bound byte work: algorithmic bytes = input bytes + output bytes + scales.
#include <cuda_fp8.h>

#include "../../include/weftmoe_b200.h"
#include "kernels.h"

using namespace wm;

namespace {

__device__ __forceinline__ float block_scale(float amax, bool invalid) {
  if (invalid || !isfinite(amax)) return __int_as_float(0x7fc00000);
  if (amax == 0.0f) return 1.0f;
  const unsigned bits = __float_as_uint(amax);
  // 448 = 1.75 * 2^8: amax / 448 rounds up to 2^(exponent-8), or one more above mantissa 1.75.
  int exponent = static_cast<int>(bits >> 23) - 8 + ((bits & 0x7fffffu) > 0x600000u);
  exponent = exponent < 1 ? 1 : exponent;
  return __uint_as_float(static_cast<unsigned>(exponent) << 23);
}
// Exact reciprocal of a power-of-two scale (NaN stays NaN).
__device__ __forceinline__ float inverse_scale(float scale) {
  return scale != scale ? scale : __uint_as_float(0x7f000000u - __float_as_uint(scale));
}
__device__ __forceinline__ unsigned char to_e4m3(float v) {
  return static_cast<unsigned char>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ unsigned pack4(float a, float b, float c, float d) {
  const unsigned lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const unsigned hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int d = 16; d; d >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, d));
  return v;
}

enum Mode { kRows = 0, kRowsOfTranspose = 1, kBlock = 2 };

// One CTA per 128 x 128 tile of the INPUT matrix.  The tile is staged in shared memory as FP32
// (zero outside the matrix) and then quantised along rows, along columns, or as one block.
//   kRows            : q [rows][colsP],  s [rows][cblocks]                     (1 x 128 along columns)
//   kRowsOfTranspose : qt[cols][rowsP],  st[cols][rblocks]                     (1 x 128 of x^T)
//   kBlock           : q/s and/or qt/st with one scale for the tile            (128 x 128)
template <class T>
__global__ void quantize_tile_kernel(const T* __restrict__ x, int rows, int cols, int mode,
                                     unsigned char* __restrict__ q, float* __restrict__ s,
                                     unsigned char* __restrict__ qt, float* __restrict__ st) {
  extern __shared__ float tile[];  // [128][129]
  constexpr int kPitch = 129;
  const int cblocks = (cols + 127) / 128, rblocks = (rows + 127) / 128;
  const int colsP = cblocks * 128, rowsP = rblocks * 128;
  const int c0 = blockIdx.x * 128, r0 = blockIdx.y * 128;
  const size_t batch = blockIdx.z;
  const T* xb = x + batch * static_cast<size_t>(rows) * cols;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  float amax = 0.0f;
  int invalid = 0;
  for (int i = threadIdx.x; i < 128 * 128; i += blockDim.x) {
    const int r = i >> 7, c = i & 127;
    float v = 0.0f;
    if (r0 + r < rows && c0 + c < cols) v = static_cast<float>(xb[static_cast<size_t>(r0 + r) * cols + c0 + c]);
    tile[r * kPitch + c] = v;
    invalid |= !isfinite(v);
    amax = fmaxf(amax, fabsf(v));
  }
  __shared__ float warp_amax[8];
  __shared__ float tile_scale;
  const int tile_invalid = __syncthreads_or(invalid);
  if (mode == kBlock) {
    amax = warp_max(amax);
    if (lane == 0) warp_amax[warp] = amax;
    __syncthreads();
    if (threadIdx.x == 0) {
      float m = 0.0f;
      for (int w = 0; w < 8; ++w) m = fmaxf(m, warp_amax[w]);
      tile_scale = block_scale(m, tile_invalid != 0);
      if (s) s[(batch * rblocks + blockIdx.y) * cblocks + blockIdx.x] = tile_scale;
      if (st) st[(batch * cblocks + blockIdx.x) * rblocks + blockIdx.y] = tile_scale;
    }
    __syncthreads();
  }
  // ---- row-major output: each warp takes rows w, w+8, ...; a lane owns 4 consecutive columns
  if (q != nullptr && (mode == kRows || mode == kBlock)) {
    unsigned char* qb = q + batch * static_cast<size_t>(rows) * colsP;
    for (int r = warp; r < 128 && r0 + r < rows; r += 8) {
      const float* p = tile + r * kPitch + lane * 4;
      const float v0 = p[0], v1 = p[1], v2 = p[2], v3 = p[3];
      float scale;
      if (mode == kRows) {
        const bool bad = __any_sync(0xffffffffu, !isfinite(v0) || !isfinite(v1) || !isfinite(v2) || !isfinite(v3));
        const float m = warp_max(fmaxf(fmaxf(fabsf(v0), fabsf(v1)), fmaxf(fabsf(v2), fabsf(v3))));
        scale = block_scale(m, bad);
        if (lane == 0) s[(batch * rows + r0 + r) * cblocks + blockIdx.x] = scale;
      } else {
        scale = tile_scale;
      }
      const float inv = inverse_scale(scale);
      *reinterpret_cast<unsigned*>(qb + static_cast<size_t>(r0 + r) * colsP + c0 + lane * 4) =
          pack4(v0 * inv, v1 * inv, v2 * inv, v3 * inv);
    }
  }
  // ---- transposed output: each warp takes tile columns w, w+8, ...; a lane owns 4 consecutive rows
  if (qt != nullptr && (mode == kRowsOfTranspose || mode == kBlock)) {
    unsigned char* qb = qt + batch * static_cast<size_t>(cols) * rowsP;
    for (int c = warp; c < 128 && c0 + c < cols; c += 8) {
      const float* p = tile + (lane * 4) * kPitch + c;
      const float v0 = p[0], v1 = p[kPitch], v2 = p[2 * kPitch], v3 = p[3 * kPitch];
      float scale;
      if (mode == kRowsOfTranspose) {
        const bool bad = __any_sync(0xffffffffu, !isfinite(v0) || !isfinite(v1) || !isfinite(v2) || !isfinite(v3));
        const float m = warp_max(fmaxf(fmaxf(fabsf(v0), fabsf(v1)), fmaxf(fabsf(v2), fabsf(v3))));
        scale = block_scale(m, bad);
        if (lane == 0) st[(batch * cols + c0 + c) * rblocks + blockIdx.y] = scale;
      } else {
        scale = tile_scale;
      }
      const float inv = inverse_scale(scale);
      *reinterpret_cast<unsigned*>(qb + static_cast<size_t>(c0 + c) * rowsP + r0 + lane * 4) =
          pack4(v0 * inv, v1 * inv, v2 * inv, v3 * inv);
    }
  }
}

// Hot path: BF16 activations [rows][cols], cols % 128 == 0, 16-byte aligned rows.  Sixteen lanes
// own one 1 x 128 block, eight consecutive values per lane (one 16-byte load, one 8-byte store).
__global__ void quantize_rows_bf16_kernel(const uint4* __restrict__ x, long long blocks, int cblocks,
                                          uint2* __restrict__ q, float* __restrict__ s) {
  const long long half_warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 4;
  const int sub = threadIdx.x & 15;
  const unsigned mask = 0xffffu << (threadIdx.x & 16);
  for (long long b = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 4; b < blocks;
       b += half_warps) {
    const uint4 raw = x[b * 16 + sub];
    const unsigned w[4] = {raw.x, raw.y, raw.z, raw.w};
    float v[8];
    float m = 0.0f;
    bool bad = false;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[2 * j] = __uint_as_float(w[j] << 16);
      v[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
      m = fmaxf(m, fmaxf(fabsf(v[2 * j]), fabsf(v[2 * j + 1])));
      bad |= !isfinite(v[2 * j]) || !isfinite(v[2 * j + 1]);
    }
#pragma unroll
    for (int d = 8; d; d >>= 1) {
      m = fmaxf(m, __shfl_xor_sync(mask, m, d, 16));
      bad |= __shfl_xor_sync(mask, static_cast<int>(bad), d, 16) != 0;
    }
    const float scale = block_scale(m, bad);
    const float inv = inverse_scale(scale);
    uint2 out;
    out.x = pack4(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv);
    out.y = pack4(v[4] * inv, v[5] * inv, v[6] * inv, v[7] * inv);
    q[b * 16 + sub] = out;
    if (sub == 0) s[b] = scale;
  }
  (void)cblocks;
}

// Byte transpose of 128 x 128-quantised weights: bits and scales are preserved.
__global__ void transpose_weight_kernel(const unsigned char* __restrict__ q, const float* __restrict__ s,
                                        int rows, int cols, unsigned char* __restrict__ qt,
                                        float* __restrict__ st) {
  __shared__ unsigned char tile[32][33];
  const int cblocks = (cols + 127) / 128, rblocks = (rows + 127) / 128;
  const int colsP = cblocks * 128, rowsP = rblocks * 128;
  const size_t batch = blockIdx.z;
  const unsigned char* qb = q + batch * static_cast<size_t>(rows) * colsP;
  unsigned char* ob = qt + batch * static_cast<size_t>(cols) * rowsP;
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int r = r0 + j, c = c0 + threadIdx.x;
    tile[j][threadIdx.x] = (r < rows && c < colsP) ? qb[static_cast<size_t>(r) * colsP + c] : 0;
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int c = c0 + j, r = r0 + threadIdx.x;
    if (c < cols && r < rowsP) ob[static_cast<size_t>(c) * rowsP + r] = tile[threadIdx.x][j];
  }
  if (blockIdx.x == 0 && blockIdx.y == 0)
    for (int i = threadIdx.y * blockDim.x + threadIdx.x; i < rblocks * cblocks; i += blockDim.x * blockDim.y) {
      const int rb = i / cblocks, cb = i - rb * cblocks;
      st[(batch * cblocks + cb) * rblocks + rb] = s[batch * rblocks * cblocks + i];
    }
}

template <class T>
int launch_tile(const void* x, int batches, int rows, int cols, int mode, void* q, float* s, void* qt,
                float* st, cudaStream_t stream) {
  if (batches == 0 || rows == 0 || cols == 0) return WM_OK;
  constexpr int smem = 128 * 129 * sizeof(float);
  static PerDeviceOnce configured;  // one table per template instantiation
  if (int rc = opt_in_dynamic_smem(quantize_tile_kernel<T>, smem, configured)) return rc;
  dim3 grid((cols + 127) / 128, (rows + 127) / 128, batches);
  quantize_tile_kernel<T><<<grid, 256, smem, stream>>>(static_cast<const T*>(x), rows, cols, mode,
                                                       static_cast<unsigned char*>(q), s,
                                                       static_cast<unsigned char*>(qt), st);
  WM_CUDA(cudaGetLastError());
  count_launch();
  return WM_OK;
}

bool overlap(const void* a, size_t an, const void* b, size_t bn) {
  const auto pa = reinterpret_cast<uintptr_t>(a), pb = reinterpret_cast<uintptr_t>(b);
  return a && b && an && bn && pa < pb + bn && pb < pa + an;
}

int check_common(const char* what, const void* x, int dtype, int batches, int rows, int cols) {
  if ((dtype != 0 && dtype != 1) || batches < 0 || rows < 0 || cols < 0 || batches > 65535 ||
      (static_cast<long long>(batches) * rows * cols > 0 && !x)) {
    set_error("%s: input must be BF16 (0) or FP32 (1), batch <= 65535, non-negative shape", what);
    return WM_ERR_INVALID;
  }
  return WM_OK;
}

}  // namespace

namespace wm {
// BF16 [rows][cols] (cols % 128 == 0, 16-byte aligned) -> E4M3 bytes + FP32 scales [rows][cols/128].
int fp8_quantize_rows(const void* x, long long rows, int cols, void* q, float* scales, int sms,
                      cudaStream_t stream) {
  const long long blocks = rows * (cols / 128);
  if (blocks == 0) return 0;
  const long long want = (blocks * 16 + 255) / 256;
  const int grid = static_cast<int>(want < sms * 16LL ? want : sms * 16LL);
  quantize_rows_bf16_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint4*>(x), blocks, cols / 128,
                                                      static_cast<uint2*>(q), scales);
  WM_CUDA(cudaGetLastError());
  count_launch();
  return 0;
}
}  // namespace wm

extern "C" int wm_fp8_quantize(const void* x, int32_t dtype, int32_t batches, int32_t rows,
                               int32_t cols, int32_t block_rows, int32_t transpose, void* q,
                               float* scales, void* stream_) {
  if (int rc = check_common("wm_fp8_quantize", x, dtype, batches, rows, cols)) return rc;
  if (block_rows != 1 && block_rows != 128) {
    set_error("wm_fp8_quantize: block_rows must be 1 or 128");
    return WM_ERR_INVALID;
  }
  if (reinterpret_cast<uintptr_t>(q) % 4) {
    set_error("wm_fp8_quantize: FP8 output data must be 4-byte aligned");
    return WM_ERR_INVALID;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const long long elements = static_cast<long long>(batches) * rows * cols;
  if (elements == 0) return WM_OK;
  if (!q || !scales) {
    set_error("wm_fp8_quantize: null output");
    return WM_ERR_INVALID;
  }
  if (block_rows == 1 && !transpose && dtype == 0 && cols % 128 == 0 &&
      reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(q) % 8 == 0) {
    const long long blocks = elements / 128;
    int sms = 0, dev = 0;
    WM_CUDA(cudaGetDevice(&dev));
    WM_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const long long want = (blocks * 16 + 255) / 256;
    const int grid = static_cast<int>(want < sms * 16LL ? want : sms * 16LL);
    quantize_rows_bf16_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint4*>(x), blocks, cols / 128,
                                                        static_cast<uint2*>(q), scales);
    WM_CUDA(cudaGetLastError());
    count_launch();
    return WM_OK;
  }
  // x^T with 128 x 128 blocks is the transposed output of the block mode.
  const int mode = block_rows == 128 ? kBlock : (transpose ? kRowsOfTranspose : kRows);
  void* qa = transpose ? nullptr : q;
  float* sa = transpose ? nullptr : scales;
  void* qb = transpose ? q : nullptr;
  float* sb = transpose ? scales : nullptr;
  return dtype == 0 ? launch_tile<__nv_bfloat16>(x, batches, rows, cols, mode, qa, sa, qb, sb, stream)
                    : launch_tile<float>(x, batches, rows, cols, mode, qa, sa, qb, sb, stream);
}

extern "C" int wm_fp8_quantize_weight(const void* x, int32_t dtype, int32_t batches, int32_t rows,
                                      int32_t cols, void* q, float* s, void* qt, float* st,
                                      void* stream_) {
  if (int rc = check_common("wm_fp8_quantize_weight", x, dtype, batches, rows, cols)) return rc;
  const size_t rb = (rows + 127) / 128, cb = (cols + 127) / 128;
  const size_t qn = static_cast<size_t>(batches) * rows * cb * 128, qtn = static_cast<size_t>(batches) * cols * rb * 128;
  const size_t sn = static_cast<size_t>(batches) * rb * cb * sizeof(float);
  const size_t xn = static_cast<size_t>(batches) * rows * cols * (dtype == 0 ? 2 : 4);
  const void* ptrs[5] = {x, q, s, qt, st};
  const size_t sizes[5] = {xn, qn, sn, qtn, sn};
  for (int i = 1; i < 5; ++i)
    for (int j = 0; j < i; ++j)
      if (overlap(ptrs[i], sizes[i], ptrs[j], sizes[j])) {
        set_error("wm_fp8_quantize_weight: operands alias");
        return WM_ERR_INVALID;
      }
  if (reinterpret_cast<uintptr_t>(q) % 4 || reinterpret_cast<uintptr_t>(qt) % 4) {
    set_error("wm_fp8_quantize_weight: FP8 weight output data must be 4-byte aligned");
    return WM_ERR_INVALID;
  }
  if (xn == 0) return WM_OK;
  if (!q || !s || !qt || !st) {
    set_error("wm_fp8_quantize_weight: null output");
    return WM_ERR_INVALID;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  return dtype == 0 ? launch_tile<__nv_bfloat16>(x, batches, rows, cols, kBlock, q, s, qt, st, stream)
                    : launch_tile<float>(x, batches, rows, cols, kBlock, q, s, qt, st, stream);
}

extern "C" int wm_fp8_transpose_weight(const void* q, const float* s, int32_t batches, int32_t rows,
                                       int32_t cols, void* qt, float* st, void* stream_) {
  if (batches < 0 || rows < 0 || cols < 0 || batches > 65535) {
    set_error("wm_fp8_transpose_weight: bad shape");
    return WM_ERR_INVALID;
  }
  if (static_cast<long long>(batches) * rows * cols == 0) return WM_OK;
  if (!q || !s || !qt || !st) {
    set_error("wm_fp8_transpose_weight: null tensor");
    return WM_ERR_INVALID;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int colsP = (cols + 127) / 128 * 128, rowsP = (rows + 127) / 128 * 128;
  dim3 grid((colsP + 31) / 32, (rowsP + 31) / 32, batches);
  transpose_weight_kernel<<<grid, dim3(32, 8), 0, stream>>>(static_cast<const unsigned char*>(q), s, rows,
                                                            cols, static_cast<unsigned char*>(qt), st);
  WM_CUDA(cudaGetLastError());
  count_launch();
  return WM_OK;
}
