// Diagnostic FP8 GEMM  out[M,N] (+)= A[M,K] * B[N,K]^T  on the block-scaled tcgen05 path, and the
// scale-factor packer that feeds it.  Plays the role of the reference's standalone fp8_gemm
// (weftmoe/fp8.py:129-153, src/cuda/fp8/gemm.cuh:17-98): a way to check the quantised contraction
// against a dequantised FP64 product without running the layer.
#include <vector>

#include "../../include/weftmoe_b200.h"
#include "kernels.h"
#include "gemm_bs.cuh"

using namespace wm;

namespace {

// FP32 power-of-two scales -> UE8M0 bytes in the 4 x 32 chunk order of tcgen05.cp.32x128b.warpx4.
// scales: [ceil(rows / block_rows)][kblocks]; out: [ceil(rows/128)][kblocks][128 words].  A row's word
// repeats its scale byte four times (one byte per 32-element group of the 128-wide block).
__global__ void pack_fp8_scales_kernel(const float* __restrict__ scales, int rows, int kblocks,
                                       int block_rows, uint32_t* __restrict__ out, int tiles) {
  const long long total = static_cast<long long>(tiles) * kblocks * 128;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int word = static_cast<int>(i & 127);
    const long long chunk = i >> 7;
    const int kb = static_cast<int>(chunk % kblocks);
    const int tile = static_cast<int>(chunk / kblocks);
    const int r = tile * 128 + (word >> 2) + 32 * (word & 3);
    uint32_t byte = 127;  // scale 1 for rows beyond the matrix (their data is zero)
    if (r < rows) {
      const float s = scales[static_cast<size_t>(r / block_rows) * kblocks + kb];
      byte = (__float_as_uint(s) >> 23) & 0xffu;  // biased exponent == UE8M0 code; NaN scale -> 0xff
    }
    out[i] = byte * 0x01010101u;
  }
}

// flag |= 1 when any of the n scales has a non-empty mantissa field (is not a power of two).
__global__ void scales_have_mantissa_kernel(const float* __restrict__ scales, long long n, int* __restrict__ flag) {
  bool any = false;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    any |= (__float_as_uint(scales[i]) & 0x007fffffu) != 0;
  if (any) atomicOr(flag, 1);
}

}  // namespace

namespace wm {

// (declared in quant_path.h)
int pack_fp8_scales(const float* scales, int rows, int kblocks, int block_rows, void* out,
                    cudaStream_t stream) {
  const int tiles = (rows + 127) / 128;
  if (tiles == 0 || kblocks == 0) return 0;
  const long long total = static_cast<long long>(tiles) * kblocks * 128;
  const int grid = static_cast<int>((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
  pack_fp8_scales_kernel<<<grid, 256, 0, stream>>>(scales, rows, kblocks, block_rows,
                                                   static_cast<uint32_t*>(out), tiles);
  WM_CUDA(cudaGetLastError());
  count_launch();
  return 0;
}

}  // namespace wm

extern "C" int wm_fp8_gemm(const void* aq, const float* as, const void* bq, const float* bs, void* out,
                           int32_t m, int32_t n, int32_t k, int32_t a_block_rows, int32_t b_block_rows,
                           int32_t out_is_f32, int32_t accumulate, void* stream_) {
  if (m < 0 || n < 0 || k < 0 || (a_block_rows != 1 && a_block_rows != 128) ||
      (b_block_rows != 1 && b_block_rows != 128) || (accumulate && !out_is_f32)) {
    set_error("wm_fp8_gemm: FP8 GEMM requires [M,K], [N,K], block rows 1/128; accumulation needs an FP32 output");
    return WM_ERR_INVALID;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (m == 0 || n == 0) return WM_OK;
  if (!out) {
    set_error("wm_fp8_gemm: null output");
    return WM_ERR_INVALID;
  }
  if (k == 0) {
    if (!accumulate) WM_CUDA(cudaMemsetAsync(out, 0, static_cast<size_t>(m) * n * (out_is_f32 ? 4 : 2), stream));
    return WM_OK;
  }
  if (!aq || !as || !bq || !bs || reinterpret_cast<uintptr_t>(aq) % 16 || reinterpret_cast<uintptr_t>(bq) % 16) {
    set_error("wm_fp8_gemm: null or misaligned operand (16-byte alignment required)");
    return WM_ERR_INVALID;
  }
  const int kblocks = (k + 127) / 128, kp = kblocks * 128;
  const int m_tiles = (m + 127) / 128, n_tiles = (n + 127) / 128;
  // Temporary device memory (diagnostic entry): packed scales, schedule words, status.
  const size_t sfa_bytes = static_cast<size_t>(m_tiles) * kblocks * 512;
  const size_t sfb_bytes = static_cast<size_t>(n_tiles) * kblocks * 512;
  const size_t sched_bytes = (static_cast<size_t>(m_tiles) + 16) * sizeof(int);
  uint8_t* tmp = nullptr;
  WM_CUDA(cudaMalloc(&tmp, sfa_bytes + sfb_bytes + sched_bytes));
  uint8_t* sfa = tmp;
  uint8_t* sfb = tmp + sfa_bytes;
  int* sched = reinterpret_cast<int*>(tmp + sfa_bytes + sfb_bytes);
  std::vector<int> host(m_tiles + 16, 0);
  const int split[8] = {m_tiles, m_tiles, 0, 0, 0, 0, 0, 0};
  for (int i = 0; i < 8; ++i) host[i] = split[i];
  int rc = 0;
  cudaError_t e = cudaMemcpyAsync(sched, host.data(), sched_bytes, cudaMemcpyHostToDevice, stream);
  if (e != cudaSuccess) rc = WM_ERR_CUDA;
  // Scales with mantissas (imported checkpoints) take the promotion form of the kernel; words 4 and 5 of
  // the schedule block are free and hold the two findings.
  const int a_scale_rows = (m + a_block_rows - 1) / a_block_rows, b_scale_rows = (n + b_block_rows - 1) / b_block_rows;
  int mantissa[2] = {0, 0};
  if (!rc) {
    scales_have_mantissa_kernel<<<64, 256, 0, stream>>>(as, static_cast<long long>(a_scale_rows) * kblocks, sched + 4);
    scales_have_mantissa_kernel<<<64, 256, 0, stream>>>(bs, static_cast<long long>(b_scale_rows) * kblocks, sched + 5);
    count_launch(2);
    if (cudaGetLastError() != cudaSuccess ||
        cudaMemcpyAsync(mantissa, sched + 4, sizeof(mantissa), cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
        cudaStreamSynchronize(stream) != cudaSuccess)
      rc = WM_ERR_CUDA;
  }
  const bool promote = mantissa[0] || mantissa[1];
  if (!rc && promote && b_block_rows != 128) {
    cudaFree(tmp);
    set_error("wm_fp8_gemm: scales that are not powers of two need 128 x 128 blocks on the second operand");
    return WM_ERR_INVALID;
  }
  if (!rc) rc = pack_fp8_scales(as, m, kblocks, a_block_rows, sfa, stream);
  if (!rc) rc = pack_fp8_scales(bs, n, kblocks, b_block_rows, sfb, stream);
  CUtensorMap ta, tb;
  if (!rc) rc = make_tmap_2d(&ta, aq, 1, kp, m, kp, 128, 128);
  if (!rc) rc = make_tmap_2d(&tb, bq, 1, kp, n, kp, 128, 128);
  int sms = 0, dev = 0;
  if (!rc && (cudaGetDevice(&dev) != cudaSuccess ||
              cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess))
    rc = WM_ERR_CUDA;
  if (!rc) {
    BsArgs args{};
    args.base.tile_begin = sched + 6;
    args.base.tile_end = sched + 1;
    args.base.tile_group = sched + 8;  // all zero: one group
    args.base.n_tiles = n_tiles;
    args.base.k_total = kp;
    args.base.b_group_rows = n;
    args.base.status = sched + 7;
    args.sfa = SfLayout{sfa, 0, 512ll * kblocks, 512, 512};
    args.sfb = SfLayout{sfb, 0, 512ll * kblocks, 512, 512};
    args.a_scales = as;
    args.a_block_rows = a_block_rows;
    args.a_scale_rows = a_scale_rows;
    args.b_scales = bs;
    EpilogueBounded epi{out, m, n, n, out_is_f32, accumulate, 1.0f};
    rc = promote ? launch_bs<kKindFp8, false, true>(ta, tb, args, epi, sms, stream)
                 : launch_bs<kKindFp8>(ta, tb, args, epi, sms, stream);
  }
  int status = 0;
  if (!rc && cudaMemcpyAsync(&status, sched + 7, sizeof(int), cudaMemcpyDeviceToHost, stream) != cudaSuccess)
    rc = WM_ERR_CUDA;
  e = cudaStreamSynchronize(stream);
  cudaFree(tmp);
  if (rc) return rc;
  if (e != cudaSuccess) {
    set_error("wm_fp8_gemm: %s", cudaGetErrorString(e));
    return WM_ERR_CUDA;
  }
  if (status) {
    set_error("wm_fp8_gemm: device status %d", status);
    return WM_ERR_TIMEOUT;
  }
  return WM_OK;
}
