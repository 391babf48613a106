// NVFP4: block-16 E2M1 operands with one E4M3 scale per 16 elements and an FP32 layer scale.
//
// Numerics contract (reference: weftmoe/nvfp4.py:14-31 `_encode_row`, tests/torchrun_sm100_nvfp4.py:13-27):
//   sf   = e4m3_rn( min( amax / (6 s), 448 ) )                     (FP32 division, s = layer scale)
//   code = e2m1_rn_even( v / (sf * s) ), 0 when sf == 0            (FP32 division)
//   two codes per byte, even element in the low nibble.
// Scale bytes are written either row-major ([rows][cols/16], the activation layout of the reference,
// weftmoe/nvfp4.py:61-63) or straight into the 512-byte chunks the tensor core's scale-factor copy
// consumes: chunk (row tile, 64-column group) holds word (r%32)*4 + (r%128)/32 for row r, byte g%4
// for 16-column group g (the reference's weight layout, weftmoe/nvfp4.py:58-60, and its backward
// operand layout, src/cuda/blackwell/nvfp4_quantize.cuh:48-51).
// HBM-bound: reads 2 B and writes 0.5625 B per element.
#include <cuda_fp8.h>

#include "../../include/weftmoe_b200.h"
#include "kernels.h"
#include "gemm_bs.cuh"

using namespace wm;

namespace wm {

__device__ __forceinline__ unsigned e2m1x2(float hi, float lo) {
  unsigned short r;
  asm("{ .reg .b8 p; cvt.rn.satfinite.e2m1x2.f32 p, %1, %2; cvt.u16.u8 %0, p; }" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}

// Quantise 16 consecutive values: returns 8 packed bytes and the E4M3 scale byte.
__device__ __forceinline__ uint2 nvfp4_encode16(const float (&v)[16], float six_s, float s, unsigned char* sf_byte) {
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
  const float unrounded = fminf(__fdiv_rn(amax, six_s), 448.0f);
  const unsigned char sb = static_cast<unsigned char>(__nv_cvt_float_to_fp8(unrounded, __NV_SATFINITE, __NV_E4M3));
  const float sf = __half2float(__half(__nv_cvt_fp8_to_halfraw(sb, __NV_E4M3)));
  const float divisor = sf * s;
  unsigned bytes[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float lo = divisor > 0.0f ? __fdiv_rn(v[2 * i], divisor) : 0.0f;
    const float hi = divisor > 0.0f ? __fdiv_rn(v[2 * i + 1], divisor) : 0.0f;
    bytes[i] = e2m1x2(hi, lo);
  }
  *sf_byte = sb;
  uint2 out;
  out.x = bytes[0] | (bytes[1] << 8) | (bytes[2] << 16) | (bytes[3] << 24);
  out.y = bytes[4] | (bytes[5] << 8) | (bytes[6] << 16) | (bytes[7] << 24);
  return out;
}

// Byte address of the scale of (row r, 16-column group g) in the chunked layout with `k64` 64-column
// groups per row tile.
__device__ __forceinline__ size_t nvfp4_sf_chunk_offset(int r, int g, int k64) {
  return ((static_cast<size_t>(r >> 7) * k64 + (g >> 2)) * 128 + (r & 31) * 4 + ((r & 127) >> 5)) * 4 + (g & 3);
}

}  // namespace wm

namespace {

// One lane per 16-element block; a warp covers 512 consecutive columns of one row.
__global__ void nvfp4_quantize_kernel(const __nv_bfloat16* __restrict__ x, int rows, int cols, float six_s,
                                      float s, uint2* __restrict__ data, unsigned char* __restrict__ sf,
                                      int chunked, const int* __restrict__ live_rows) {
  if (live_rows != nullptr) rows = min(rows, *live_rows);  // rows behind the live ones are never read
  const int groups = cols / 16;
  const long long total = static_cast<long long>(rows) * groups;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / groups), g = static_cast<int>(i - static_cast<long long>(r) * groups);
    const uint4* p = reinterpret_cast<const uint4*>(x + static_cast<size_t>(r) * cols + g * 16);
    const uint4 a = p[0], b = p[1];
    const unsigned w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    float v[16];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      v[2 * j] = __uint_as_float(w[j] << 16);
      v[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
    }
    unsigned char sb;
    data[i] = nvfp4_encode16(v, six_s, s, &sb);
    sf[chunked ? nvfp4_sf_chunk_offset(r, g, cols / 64) : static_cast<size_t>(i)] = sb;
  }
}

// [rows][cols] values -> NVFP4 of the TRANSPOSE: packed codes [cols][rows / 2] with block 16 along the
// rows, scales in the chunked layout of a [cols][rows] operand (the weight-gradient operands of the
// NVFP4 backward, reference: src/cuda/blackwell/nvfp4_quantize.cuh:48-51).  A warp serves 64 rows x 64
// columns: lane l holds columns c = 2l and 2l+1 and ends up with 64 consecutive codes of each of its two
// output rows (32 bytes, one sector) plus their four scale bytes (one word of the chunk).  Same values as
// transposing first and quantising the rows after (the blocks are the same 16 consecutive rows), without
// the two extra passes.  `word_at(i)` returns the BF16 pair (columns c, c + 1) of row r0 + i.
template <class WordAt>
__device__ __forceinline__ void nvfp4_encode_columns(WordAt word_at, int r0, int c, int rows, float six_s, float s,
                                                     uint8_t* __restrict__ data, uint8_t* __restrict__ sf) {
  uint2 codes[2][4];
  unsigned scale_word[2] = {0u, 0u};
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    float lo[16], hi[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const unsigned w = word_at(16 * g + i);
      lo[i] = __uint_as_float(w << 16);
      hi[i] = __uint_as_float(w & 0xffff0000u);
    }
    unsigned char sb;
    codes[0][g] = nvfp4_encode16(lo, six_s, s, &sb);
    scale_word[0] |= static_cast<unsigned>(sb) << (8 * g);
    codes[1][g] = nvfp4_encode16(hi, six_s, s, &sb);
    scale_word[1] |= static_cast<unsigned>(sb) << (8 * g);
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    uint4* dst = reinterpret_cast<uint4*>(data + static_cast<size_t>(c + h) * (rows / 2) + r0 / 2);
    dst[0] = make_uint4(codes[h][0].x, codes[h][0].y, codes[h][1].x, codes[h][1].y);
    dst[1] = make_uint4(codes[h][2].x, codes[h][2].y, codes[h][3].x, codes[h][3].y);
    *reinterpret_cast<unsigned*>(sf + nvfp4_sf_chunk_offset(c + h, r0 / 16, rows / 64)) = scale_word[h];
  }
}

// Source = BF16 [rows][cols]: every load instruction of the warp is one 128-byte row segment.
__global__ void nvfp4_quantize_cols_kernel(const __nv_bfloat16* __restrict__ x, int rows, int cols, float six_s,
                                           float s, uint8_t* __restrict__ data, uint8_t* __restrict__ sf,
                                           const int* __restrict__ live_rows) {
  const int lane = threadIdx.x & 31;
  const int col_blocks = cols / 64;
  // rows behind the live ones (a multiple of 64) are never read by the contraction: left out
  const long long units = static_cast<long long>((live_rows ? min(rows, *live_rows) : rows) / 64) * col_blocks;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const size_t pitch = static_cast<size_t>(cols) / 2;  // words per input row
  for (long long unit = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5; unit < units;
       unit += warps) {
    const int rb = static_cast<int>(unit / col_blocks), cb = static_cast<int>(unit - static_cast<long long>(rb) * col_blocks);
    const int r0 = rb * 64, c = cb * 64 + 2 * lane;
    const unsigned* src = reinterpret_cast<const unsigned*>(x + static_cast<size_t>(r0) * cols + c);
    nvfp4_encode_columns([&](int i) { return src[i * pitch]; }, r0, c, rows, six_s, s, data, sf);
  }
}

// Source = rows stored as NVFP4 (packed E2M1 [rows][cols / 2] + chunked E4M3 scales, layer scale s_in): the
// values a dequantisation to BF16 rows would hold (code * block scale * s_in, rounded to BF16), without
// that copy.  Lane l first decodes rows l and 32 + l of the warp's 64 x 64 block (32 bytes of codes and
// one scale word each) into the warp's shared-memory tile (33-word row pitch: conflict-free both ways),
// then the lanes read the tile column-wise as above.
constexpr int kRequantWarps = 4;
__global__ void __launch_bounds__(32 * kRequantWarps)
nvfp4_requantize_cols_kernel(const uint8_t* __restrict__ xq, const uint8_t* __restrict__ xsf, float s_in, int rows,
                             int cols, float six_s, float s, uint8_t* __restrict__ data,
                             uint8_t* __restrict__ sf, const int* __restrict__ live_rows) {
  __shared__ unsigned tiles[kRequantWarps][64 * 33];
  __shared__ float e2m1[16];  // value of each code: sign bit 3, magnitudes 0, 0.5, 1, 1.5, 2, 3, 4, 6
  const int lane = threadIdx.x & 31;
  if (threadIdx.x < 16) {
    const unsigned mag = threadIdx.x & 7u;
    const float m = mag < 2 ? 0.5f * mag : (mag & 1 ? 1.5f : 1.0f) * static_cast<float>(1 << ((mag >> 1) - 1));
    e2m1[threadIdx.x] = threadIdx.x & 8u ? -m : m;
  }
  __syncthreads();
  unsigned* tile = tiles[threadIdx.x >> 5];
  const int col_blocks = cols / 64;
  const long long units = static_cast<long long>((live_rows ? min(rows, *live_rows) : rows) / 64) * col_blocks;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long unit = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5; unit < units;
       unit += warps) {
    const int rb = static_cast<int>(unit / col_blocks), cb = static_cast<int>(unit - static_cast<long long>(rb) * col_blocks);
    const int r0 = rb * 64, c0 = cb * 64;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int row = r0 + 32 * half + lane;
      const uint4* src = reinterpret_cast<const uint4*>(xq + static_cast<size_t>(row) * (cols / 2) + c0 / 2);
      const uint4 d0 = src[0], d1 = src[1];
      const unsigned scales = *reinterpret_cast<const unsigned*>(xsf + nvfp4_sf_chunk_offset(row, c0 / 16, cols / 64));
      const unsigned words[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
      unsigned* out = tile + (32 * half + lane) * 33;
#pragma unroll
      for (int g = 0; g < 4; ++g) {  // 16 columns = 8 bytes = words 2g, 2g+1
        const unsigned char sb = static_cast<unsigned char>(scales >> (8 * g));
        const float scale = __half2float(__half(__nv_cvt_fp8_to_halfraw(sb, __NV_E4M3))) * s_in;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const unsigned byte = (words[2 * g + (j >> 2)] >> (8 * (j & 3))) & 0xffu;
          out[8 * g + j] = pack_bf16x2(e2m1[byte & 0xfu] * scale, e2m1[byte >> 4] * scale);
        }
      }
    }
    __syncwarp();
    nvfp4_encode_columns([&](int i) { return tile[i * 33 + lane]; }, r0, c0 + 2 * lane, rows, six_s, s, data, sf);
    __syncwarp();
  }
}

// Row-major scale bytes [rows][k/16] -> chunked layout (rows beyond `rows` and groups beyond k get 0).
__global__ void nvfp4_pack_scales_kernel(const unsigned char* __restrict__ sf, int rows, int groups, int k64,
                                         unsigned char* __restrict__ out, int tiles) {
  const long long total = static_cast<long long>(tiles) * 128 * k64 * 4;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int g = static_cast<int>(i % (k64 * 4));
    const int r = static_cast<int>(i / (k64 * 4));
    out[nvfp4_sf_chunk_offset(r, g, k64)] = (r < rows && g < groups) ? sf[static_cast<size_t>(r) * groups + g] : 0;
  }
}

}  // namespace

namespace wm {
int nvfp4_quantize_rows(const void* x, int rows, int cols, float layer_scale, void* data, void* scales,
                        int chunked, cudaStream_t stream, const int* live_rows) {
  const long long total = static_cast<long long>(rows) * (cols / 16);
  if (total == 0) return 0;
  if (chunked) {
    const size_t bytes = static_cast<size_t>((rows + 127) / 128) * (cols / 64) * 512;
    WM_CUDA(cudaMemsetAsync(scales, 0, bytes, stream));
  }
  const int grid = static_cast<int>((total + 255) / 256 < 8192 ? (total + 255) / 256 : 8192);
  nvfp4_quantize_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), rows, cols,
                                                  static_cast<float>(6.0 * static_cast<double>(layer_scale)),
                                                  layer_scale, static_cast<uint2*>(data),
                                                  static_cast<unsigned char*>(scales), chunked, live_rows);
  WM_CUDA(cudaGetLastError());
  count_launch();
  return 0;
}
static int check_cols_shape(int rows, int cols, uint8_t* scales, cudaStream_t stream) {
  if (rows % 64 || cols % 64) {
    set_error("nvfp4_quantize_cols: rows and columns must be multiples of 64");
    return WM_ERR_INVALID;
  }
  if (cols % 128)  // the last 128-row tile of the output is half empty: its scale words must read as zero
    WM_CUDA(cudaMemsetAsync(scales, 0, static_cast<size_t>((cols + 127) / 128) * (rows / 64) * 512, stream));
  return 0;
}
int nvfp4_quantize_cols(const __nv_bfloat16* x, int rows, int cols, float layer_scale, uint8_t* data,
                        uint8_t* scales, const int* live_rows, int sms, cudaStream_t stream) {
  if (rows == 0 || cols == 0) return 0;
  if (int rc = check_cols_shape(rows, cols, scales, stream)) return rc;
  nvfp4_quantize_cols_kernel<<<sms * 8, 256, 0, stream>>>(
      x, rows, cols, static_cast<float>(6.0 * static_cast<double>(layer_scale)), layer_scale, data, scales,
      live_rows);
  WM_CUDA(cudaGetLastError());
  count_launch();
  return 0;
}
int nvfp4_requantize_cols(const uint8_t* xq, const uint8_t* sf_chunks, int rows, int cols, float layer_scale,
                          uint8_t* data, uint8_t* scales, const int* live_rows, int sms, cudaStream_t stream) {
  if (rows == 0 || cols == 0) return 0;
  if (int rc = check_cols_shape(rows, cols, scales, stream)) return rc;
  nvfp4_requantize_cols_kernel<<<sms * 6, 32 * kRequantWarps, 0, stream>>>(
      xq, sf_chunks, layer_scale, rows, cols, static_cast<float>(6.0 * static_cast<double>(layer_scale)), layer_scale,
      data, scales, live_rows);
  WM_CUDA(cudaGetLastError());
  count_launch();
  return 0;
}
}  // namespace wm

extern "C" int wm_nvfp4_quantize(const void* x, int32_t rows, int32_t cols, float layer_scale, void* data,
                                 void* scales, int32_t chunked, void* stream_) {
  if (rows < 0 || cols < 0 || cols % 16 || (chunked && cols % 64) || !(layer_scale > 0.0f) ||
      !isfinite(layer_scale)) {
    set_error("wm_nvfp4_quantize: columns must be a multiple of 16 (64 for the chunked scale layout) and "
              "the layer scale finite and positive");
    return WM_ERR_INVALID;
  }
  if (static_cast<long long>(rows) * cols == 0) return WM_OK;
  if (!x || !data || !scales || reinterpret_cast<uintptr_t>(x) % 16 || reinterpret_cast<uintptr_t>(data) % 8) {
    set_error("wm_nvfp4_quantize: null or misaligned tensor");
    return WM_ERR_INVALID;
  }
  return nvfp4_quantize_rows(x, rows, cols, layer_scale, data, scales, chunked,
                             static_cast<cudaStream_t>(stream_), nullptr);
}

// Diagnostic: out[m,n] = alpha * (A[m,k] * B[n,k]^T) with NVFP4 operands; scales row-major bytes.
extern "C" int wm_nvfp4_gemm(const void* a, const void* a_sf, const void* b, const void* b_sf, void* out,
                             int32_t m, int32_t n, int32_t k, float alpha, int32_t out_is_f32, void* stream_) {
  if (m < 0 || n < 0 || k <= 0 || k % 64) {
    set_error("wm_nvfp4_gemm: K must be a positive multiple of 64");
    return WM_ERR_INVALID;
  }
  if (m == 0 || n == 0) return WM_OK;
  if (!a || !a_sf || !b || !b_sf || !out || reinterpret_cast<uintptr_t>(a) % 16 ||
      reinterpret_cast<uintptr_t>(b) % 16 || (k / 2) % 16) {
    set_error("wm_nvfp4_gemm: null or misaligned operand (rows of K/2 bytes must be 16-byte multiples)");
    return WM_ERR_INVALID;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int k_stages = (k + 255) / 256, k64 = k_stages * 4;
  const int m_tiles = (m + 127) / 128, n_tiles = (n + 127) / 128;
  const size_t sfa_bytes = static_cast<size_t>(m_tiles) * k64 * 512, sfb_bytes = static_cast<size_t>(n_tiles) * k64 * 512;
  const size_t sched_bytes = (static_cast<size_t>(m_tiles) + 16) * sizeof(int);
  uint8_t* tmp = nullptr;
  WM_CUDA(cudaMalloc(&tmp, sfa_bytes + sfb_bytes + sched_bytes));
  uint8_t* sfa = tmp;
  uint8_t* sfb = tmp + sfa_bytes;
  int* sched = reinterpret_cast<int*>(tmp + sfa_bytes + sfb_bytes);
  int rc = 0;
  if (cudaMemsetAsync(sched, 0, sched_bytes, stream) != cudaSuccess ||
      cudaMemcpyAsync(sched, &m_tiles, sizeof(int), cudaMemcpyHostToDevice, stream) != cudaSuccess ||
      cudaMemcpyAsync(sched + 1, &m_tiles, sizeof(int), cudaMemcpyHostToDevice, stream) != cudaSuccess)
    rc = WM_ERR_CUDA;
  if (!rc) {
    nvfp4_pack_scales_kernel<<<1024, 256, 0, stream>>>(static_cast<const unsigned char*>(a_sf), m, k / 16, k64, sfa, m_tiles);
    nvfp4_pack_scales_kernel<<<1024, 256, 0, stream>>>(static_cast<const unsigned char*>(b_sf), n, k / 16, k64, sfb, n_tiles);
    if (cudaGetLastError() != cudaSuccess) rc = WM_ERR_CUDA;
    count_launch(2);
  }
  CUtensorMap ta, tb;
  if (!rc) rc = make_tmap_2d(&ta, a, 1, k / 2, m, k / 2, 128, 128);
  if (!rc) rc = make_tmap_2d(&tb, b, 1, k / 2, n, k / 2, 128, 128);
  int sms = 0, dev = 0;
  if (!rc && (cudaGetDevice(&dev) != cudaSuccess ||
              cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess))
    rc = WM_ERR_CUDA;
  if (!rc) {
    BsArgs args{};
    args.base.tile_begin = sched + 6;
    args.base.tile_end = sched + 1;
    args.base.tile_group = sched + 8;
    args.base.n_tiles = n_tiles;
    args.base.k_total = k;
    args.base.b_group_rows = n;
    args.base.status = sched + 7;
    args.sfa = SfLayout{sfa, 0, 512ll * k64, 2048, 512};
    args.sfb = SfLayout{sfb, 0, 512ll * k64, 2048, 512};
    EpilogueBounded epi{out, m, n, n, out_is_f32, 0, alpha};
    rc = launch_bs<kKindNvfp4>(ta, tb, args, epi, sms, stream);
  }
  int status = 0;
  if (!rc && cudaMemcpyAsync(&status, sched + 7, sizeof(int), cudaMemcpyDeviceToHost, stream) != cudaSuccess)
    rc = WM_ERR_CUDA;
  cudaError_t e = cudaStreamSynchronize(stream);
  cudaFree(tmp);
  if (rc) return rc;
  if (e != cudaSuccess) {
    set_error("wm_nvfp4_gemm: %s", cudaGetErrorString(e));
    return WM_ERR_CUDA;
  }
  if (status) {
    set_error("wm_nvfp4_gemm: device status %d", status);
    return WM_ERR_TIMEOUT;
  }
  return WM_OK;
}
