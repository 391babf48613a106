// Host interface of the quantised forward path (quant_path.cu) and the types it shares with the
// block-scaled GEMM kernel (gemm_bs.cuh).
#pragma once
#include <stdint.h>

#include "kernels.h"
#include "route.h"

namespace wm {

enum BlockScaledKind { kKindFp8 = 0, kKindNvfp4 = 1 };

// Where the 512-byte scale-factor chunks of an operand live: chunk (group, tile, k stage, c) is at
// base + group*group_stride + tile*tile_stride + kstage*kstage_stride + c*chunk_stride (bytes).
struct SfLayout {
  const uint8_t* base;
  long long group_stride, tile_stride, kstage_stride, chunk_stride;
};

struct PeerBytes { const uint8_t* p[kMaxWorld]; };

// fp8.cu / nvfp4.cu / fp8_gemm.cu
int fp8_quantize_rows(const void* x, long long rows, int cols, void* q, float* scales, int sms,
                      cudaStream_t stream);
// `live_rows` (optional device scalar): only rows below it are quantised (the owner's padded rows; what lies
// behind them in a row buffer is never read by a contraction).
int nvfp4_quantize_rows(const void* x, int rows, int cols, float layer_scale, void* data, void* scales,
                        int chunked, cudaStream_t stream, const int* live_rows = nullptr);
// BF16 [rows][cols] -> NVFP4 of the transpose ([cols][rows / 2] codes, block 16 along the rows, chunked scales).
int nvfp4_quantize_cols(const __nv_bfloat16* x, int rows, int cols, float layer_scale, uint8_t* data,
                        uint8_t* scales, const int* live_rows, int sms, cudaStream_t stream);
// The same for rows that are stored as NVFP4 (packed codes + chunked scales along the columns, the saved X
// of the training cache): re-quantised along the rows without a BF16 copy in between.
int nvfp4_requantize_cols(const uint8_t* xq, const uint8_t* sf_chunks, int rows, int cols, float layer_scale,
                          uint8_t* data, uint8_t* scales, const int* live_rows, int sms, cudaStream_t stream);
int pack_fp8_scales(const float* scales, int rows, int kblocks, int block_rows, void* out,
                    cudaStream_t stream);

// quant_path.cu
int gather_q_rows(const OwnerRows& o, int rank, int e_local, int world, int cap, int top_k, int kind, int hidden,
                  const PeerBytes& stage, size_t sf_offset, const int* meta_origin, const float* meta_prob,
                  uint8_t* rows_out, uint32_t* sfa_out, int* origin_out, float* prob_out, int by_origin,
                  int ctas, cudaStream_t stream);
// FP8 backward helpers over a device-side row range: BF16 rows -> E4M3 + chunked UE8M0 scales, and back.
int fp8_quantize_rows_chunked(DeviceRange rows, const __nv_bfloat16* x, int cols, uint8_t* q,
                              uint32_t* sfa_out, int sms, cudaStream_t stream);
int fp8_dequantize_rows(DeviceRange rows, const uint8_t* q, const uint32_t* sfa, int cols,
                        __nv_bfloat16* out, int sms, cudaStream_t stream);
// BF16 rows -> E4M3 of the transpose [cols][row_capacity], 1 x 128 along the rows, chunked UE8M0 scales
// (chunk = (cols / 128 tile, 128-row block)): the operand layout of a block-scaled weight gradient.
int fp8_quantize_cols_chunked(DeviceRange rows, const __nv_bfloat16* x, int cols, int row_capacity,
                              uint8_t* qt, uint32_t* sf_out, int sms, cudaStream_t stream);
// out[e] [m, n] = alpha * A[:, rows of e] * B[:, rows of e]^T, operands K-major over the padded rows.
int launch_block_scaled_kgrouped(int kind, const Schedule& s, const void* a, const SfLayout& sfa, const void* b,
                                 const SfLayout& sfb, __nv_bfloat16* out, int m, int n, float alpha,
                                 int* status, int sms, cudaStream_t stream);
int swiglu_quantize(DeviceRange rows, const __nv_bfloat16* ab, const float* prob, int inter, int kind,
                    float layer_scale, uint8_t* uq, uint32_t* sfa_out, int sms, cudaStream_t stream);
// out[rows, n] = alpha * A[rows, k] * B[e][n, k]^T with quantised operands; `push` != nullptr sends the
// rows to the source ranks' mailboxes instead of storing them.  `b_scales` (FP8 only, optional): the FP32
// 128 x 128 block scales of B, [groups * n / 128][k / 128], when they are not powers of two -- the kernel then
// promotes every K128 block in FP32 by the scales' mantissas.
int launch_block_scaled(int kind, const Schedule& s, const void* a, const SfLayout& sfa, const void* b,
                        const SfLayout& sfb, __nv_bfloat16* out, const PushTarget* push, int n, int k,
                        float alpha, int* status, int sms, cudaStream_t stream, const float* b_scales = nullptr);

}  // namespace wm
