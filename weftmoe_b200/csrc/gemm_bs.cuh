// Block-scaled grouped GEMM for sm_100a (one CTA per tile): quantised operands with per-block
// scale factors applied inside the tensor core.
//
//   kind FP8  : E4M3 operands, `tcgen05.mma.kind::mxf8f6f4.block_scale`, one UE8M0 scale per 32 K
//               elements.  The path's blockwise-FP8 scales are powers of two (reference:
//               src/cuda/fp8/quantization.cuh:35-43) over 1 x 128 (activations) or 128 x 128 (weights)
//               blocks, so each scale is exactly representable as UE8M0 and is repeated for the four
//               32-element groups of its block.  This replaces the reference's per-K128 FP32
//               promotion (src/cuda/fp8/gemm.cuh:68-70) by the same sum evaluated in the MMA.
//   kind NVFP4: packed E2M1 operands, `kind::mxf4nvf4.block_scale.scale_vec::4X`, one UE4M3 scale per
//               16 elements (reference: src/cuda/blackwell/fused/ptx/tcgen05.cuh:89-108).
//
// FP8 scales that are NOT powers of two (imported checkpoints; reference: tests/torchrun_fp8.py:235-255) take
// the PROMOTE form of the kernel: the MMA applies the power-of-two part of every scale as before, each K128
// block is accumulated into a fresh TMEM buffer, and the epilogue warps add it into FP32 registers times the
// mantissas of the block's scales -- the per-K128 FP32 promotion of the reference's kernel
// (src/cuda/fp8/gemm.cuh:68-70) with the exponents already applied.  The quantised bytes are used as they are.
//
// Per stage a CTA loads 128 rows x 128 bytes of A, 128 rows x 128 bytes of B (TMA, 128-byte swizzle)
// and the scale-factor chunks of both (1-D bulk copies of 512 bytes: 128 rows x 4 bytes in the
// 4 x 32 order that `tcgen05.cp.32x128b.warpx4` expects: word (r%32)*4 + r/32 holds row r).  The MMA
// thread copies the chunks into TMEM and issues four MMAs per stage.  Accumulators: 2 x 128 columns.
#pragma once
#include "gemm.cuh"
#include "quant_path.h"

namespace wm {

template <int KIND>
struct BsConfig {
  static constexpr int kBlockN = 128;
  static constexpr int kRowBytes = 128;                          // bytes of K per stage and row
  static constexpr int kElemsPerStage = KIND == kKindFp8 ? 128 : 256;
  static constexpr int kMmaK = KIND == kKindFp8 ? 32 : 64;       // elements per MMA (32 bytes either way)
  static constexpr int kSfChunks = KIND == kKindFp8 ? 1 : 4;     // 512-byte chunks per operand and stage
  static constexpr int kABytes = kBlockM * kRowBytes;
  static constexpr int kBBytes = kBlockN * kRowBytes;
  static constexpr int kSfBytes = kSfChunks * 512;
  static constexpr int kStageBytes = kABytes + kBBytes + 2 * kSfBytes;
  static constexpr int kStages = 5;
  static constexpr int kStagingBytes = 4 * 32 * 256;
  static constexpr int kTotal = kStages * kStageBytes + kStagingBytes + 256 + 1024;
  static constexpr uint32_t kTmemSfa = 2 * kBlockN;              // first scale-factor column
  static constexpr uint32_t kTmemSfb = kTmemSfa + 4 * kSfChunks;
  static constexpr uint32_t kTmemResult = 384;                   // PROMOTE: the finished sums, 128 columns
  static constexpr uint32_t kTmemCols = 512;
};

struct BsArgs {
  GemmArgs base;   // M-grouped schedule; k_total in ELEMENTS; b_group_rows = N_total
  SfLayout sfa;    // tile = 128-row tile of A (group_stride unused)
  SfLayout sfb;    // group = expert, tile = 128-row tile of that expert's B
  // PROMOTE only: the FP32 scales themselves, [scale rows][K / 128]; their mantissas are applied per K128
  // block by the epilogue warps.  a_scales may be null (activations quantised online have power-of-two
  // scales); one scale row covers a_block_rows (1 or 128) rows of A, and 128 rows of B.
  const float* a_scales;
  int a_block_rows;
  int a_scale_rows;
  const float* b_scales;
};

// The factor of an FP32 scale that its biased exponent (the UE8M0 code the MMA applies) leaves out.
__device__ __forceinline__ float scale_mantissa(float s) {
  return __uint_as_float((__float_as_uint(s) & 0x007fffffu) | 0x3f800000u);
}

// K_GROUPED (weight gradients): out[e] = A[:, rows_e]  x  B[:, rows_e]^T with both operands stored
// K-major over the rank's padded rows (A [M, row_capacity], B [N, row_capacity]); expert e reduces over
// its own row segment [row0_e, row0_e + rows_e), rows_e a multiple of 128.  An NVFP4 stage spans 256
// rows: when only 128 remain, half of the stage's MMAs are issued.
template <int KIND, bool K_GROUPED, class Epilogue, bool PROMOTE = false>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bs_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const BsArgs bs, const Epilogue epilogue) {
  using C = BsConfig<KIND>;
  constexpr int kStages = C::kStages;
  static_assert(!PROMOTE || (KIND == kKindFp8 && !K_GROUPED), "promotion is the FP8 M-grouped form");
  const GemmArgs& args = bs.base;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* staging = smem + kStages * C::kStageBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(staging + C::kStagingBytes);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full = empty_bar + kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar + s, 1);
      mbar_init(empty_bar + s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(tmem_full + s, 1);
      mbar_init(tmem_empty + s, 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  int first_tile = 0, total_tiles;
  if constexpr (K_GROUPED) {
    total_tiles = args.groups * args.m_tiles_per_group * args.n_tiles;
  } else {
    first_tile = __ldg(args.tile_begin) * args.n_tiles;
    total_tiles = __ldg(args.tile_end) * args.n_tiles;
  }
  // Stages and 64-element MMA groups of a tile's K loop, and the element its K range starts at.
  constexpr int kElemsPerMma = C::kElemsPerStage / 4;
  auto k_groups_of = [&](const TileCoord& t) {
    return K_GROUPED ? t.num_kb * kBlockK / kElemsPerMma : (args.k_total + kElemsPerMma - 1) / kElemsPerMma;
  };

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = first_tile + blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        const TileCoord t = decode_tile<K_GROUPED>(args, tile);
        const int k_stages = (k_groups_of(t) + 3) / 4;
        // K-grouped: the K range starts at the expert's first row; its scale chunks follow suit.
        const int k0 = K_GROUPED ? t.row0 : 0;
        const int k0_bytes = KIND == kKindFp8 ? k0 : k0 / 2;
        const long long sf_k0 = static_cast<long long>(k0 / (C::kElemsPerStage / C::kSfChunks)) * 512;
        const uint8_t* sfa = bs.sfa.base + t.m_tile * bs.sfa.tile_stride + (K_GROUPED ? sf_k0 : 0);
        const uint8_t* sfb = bs.sfb.base + (K_GROUPED ? sf_k0 : t.group * bs.sfb.group_stride) +
                             t.n_tile * bs.sfb.tile_stride;
        const int b_row = K_GROUPED ? t.n_tile * C::kBlockN : t.group * args.b_group_rows + t.n_tile * C::kBlockN;
        for (int kb = 0; kb < k_stages; ++kb) {
          ok = mbar_wait(empty_bar + stage, phase ^ 1, abort_flag, args.status, kStatusTimeoutSmemEmpty);
          if (!ok) break;
          uint8_t* sa = smem + stage * C::kStageBytes;
          uint8_t* sb = sa + C::kABytes;
          uint8_t* ssfa = sb + C::kBBytes;
          uint8_t* ssfb = ssfa + C::kSfBytes;
          mbar_expect_tx(full_bar + stage, C::kStageBytes);
          tma_load_2d(sa, &tmap_a, full_bar + stage, k0_bytes + kb * C::kRowBytes, t.m_tile * kBlockM);
          tma_load_2d(sb, &tmap_b, full_bar + stage, k0_bytes + kb * C::kRowBytes, b_row);
#pragma unroll
          for (int c = 0; c < C::kSfChunks; ++c) {
            bulk_load_1d(ssfa + c * 512, sfa + kb * bs.sfa.kstage_stride + c * bs.sfa.chunk_stride, 512,
                         full_bar + stage);
            bulk_load_1d(ssfb + c * 512, sfb + kb * bs.sfb.kstage_stride + c * bs.sfb.chunk_stride, 512,
                         full_bar + stage);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = first_tile + blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        int k_groups = 0;
        if constexpr (K_GROUPED) {
          const TileCoord t = decode_tile<true>(args, tile);
          k_groups = k_groups_of(t);
        } else {
          k_groups = (args.k_total + kElemsPerMma - 1) / kElemsPerMma;
        }
        const int k_stages = (k_groups + 3) / 4;
        if constexpr (!PROMOTE) {
          ok = mbar_wait(tmem_empty + acc, acc_phase ^ 1, abort_flag, args.status, kStatusTimeoutTmemEmpty);
          if (!ok) break;
          tc_fence_after();
        }
        uint32_t tmem_d = tmem_base + acc * C::kBlockN;
        for (int kb = 0; kb < k_stages; ++kb) {
          if constexpr (PROMOTE) {  // every K128 block gets a fresh accumulator buffer
            ok = mbar_wait(tmem_empty + acc, acc_phase ^ 1, abort_flag, args.status, kStatusTimeoutTmemEmpty);
            if (!ok) break;
            tmem_d = tmem_base + acc * C::kBlockN;
          }
          ok = mbar_wait(full_bar + stage, phase, abort_flag, args.status, kStatusTimeoutSmemFull);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * C::kStageBytes);
          const uint32_t sb = sa + C::kABytes;
          const uint32_t ssfa = sb + C::kBBytes;
          const uint32_t ssfb = ssfa + C::kSfBytes;
#pragma unroll
          for (int c = 0; c < C::kSfChunks; ++c) {
            tmem_cp_32x128b_warpx4(tmem_base + C::kTmemSfa + 4 * c, umma_desc_noswizzle(ssfa + c * 512, 128));
            tmem_cp_32x128b_warpx4(tmem_base + C::kTmemSfb + 4 * c, umma_desc_noswizzle(ssfb + c * 512, 128));
          }
          const uint64_t da = umma_desc_sw128(sa, 0, 1024);
          const uint64_t db = umma_desc_sw128(sb, 0, 1024);
          const int mmas = K_GROUPED ? min(4, k_groups - 4 * kb) : 4;  // a half-filled last NVFP4 stage
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            if (K_GROUPED && k >= mmas) break;
            const uint32_t accumulate = ((PROMOTE ? 0 : kb) | k) != 0 ? 1u : 0u;
            if constexpr (KIND == kKindFp8) {
              // one chunk per stage: byte k of each row's word is the scale of 32-element group k
              const uint32_t idesc = umma_idesc_block_scaled(0u, 1u, kBlockM, C::kBlockN, k, k);
              umma_mxf8_block_scaled(tmem_d, da + 2 * k, db + 2 * k, idesc, accumulate,
                                     tmem_base + C::kTmemSfa, tmem_base + C::kTmemSfb);
            } else {
              // one chunk per MMA: the four bytes of a row's word scale its four 16-element groups
              const uint32_t idesc = umma_idesc_block_scaled(1u, 0u, kBlockM, C::kBlockN, 0u, 0u);
              umma_nvf4_block_scaled(tmem_d, da + 2 * k, db + 2 * k, idesc, accumulate,
                                     tmem_base + C::kTmemSfa + 4 * k, tmem_base + C::kTmemSfb + 4 * k);
            }
          }
          umma_commit(empty_bar + stage);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
          if constexpr (PROMOTE) {
            umma_commit(tmem_full + acc);
            if (++acc == 2) { acc = 0; acc_phase ^= 1; }
          }
        }
        if (!ok) break;
        if constexpr (!PROMOTE) {
          umma_commit(tmem_full + acc);
          if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
      }
    }
  } else {
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = first_tile + blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
      const TileCoord t = decode_tile<K_GROUPED>(args, tile);
      const int k_stages = (k_groups_of(t) + 3) / 4;
      if constexpr (PROMOTE) {
        const uint32_t lanes = static_cast<uint32_t>(q * 32) << 16;
        const int kblocks = args.k_total / 128;
        const int a_row = (t.m_tile * kBlockM + q * 32 + lane) / bs.a_block_rows;
        const float* a_scale = bs.a_scales != nullptr && a_row < bs.a_scale_rows
                                   ? bs.a_scales + static_cast<size_t>(a_row) * kblocks : nullptr;
        const float* b_scale = bs.b_scales +
            (static_cast<size_t>(t.group) * args.b_group_rows / 128 + t.n_tile) * kblocks;
        float sum[C::kBlockN];
#pragma unroll
        for (int j = 0; j < C::kBlockN; ++j) sum[j] = 0.0f;
        for (int kb = 0; kb < k_stages; ++kb) {
          ok = mbar_wait(tmem_full + acc, acc_phase, abort_flag, args.status, kStatusTimeoutTmemFull);
          if (!ok) break;
          tc_fence_after();
          const float factor = scale_mantissa(__ldg(b_scale + kb)) *
                               (a_scale != nullptr ? scale_mantissa(__ldg(a_scale + kb)) : 1.0f);
#pragma unroll
          for (int c = 0; c < C::kBlockN / 32; ++c) {
            uint32_t v[32];
            tmem_ld_32x32(tmem_base + lanes + acc * C::kBlockN + c * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) sum[c * 32 + j] = fmaf(factor, __uint_as_float(v[j]), sum[c * 32 + j]);
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(tmem_empty + acc);
          if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
        if (!ok) break;
        // The finished sums go back to TMEM (columns no accumulator uses; each warp its own lanes), so that
        // the epilogues read them exactly as they read an accumulator.
#pragma unroll
        for (int c = 0; c < C::kBlockN / 32; ++c) {
          uint32_t v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(sum[c * 32 + j]);
          tmem_st_32x32(tmem_base + lanes + C::kTmemResult + c * 32, v);
        }
        tmem_st_wait();
        epilogue(tmem_base + lanes + C::kTmemResult, t, q, lane, k_stages == 0, staging + (warp - 2) * (32 * 256));
        continue;
      }
      ok = mbar_wait(tmem_full + acc, acc_phase, abort_flag, args.status, kStatusTimeoutTmemFull);
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * C::kBlockN;
      epilogue(taddr, t, q, lane, k_stages == 0, staging + (warp - 2) * (32 * 256));
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty + acc);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// Diagnostic epilogue: bounds-checked FP32 or BF16 store of a 128 x 128 tile, optional accumulate
// into an existing FP32 output, optional constant factor (NVFP4 tensor scales).
struct EpilogueBounded {
  void* out;
  int rows, cols, ld;
  int out_is_f32, accumulate;
  float alpha;

  __device__ __forceinline__ void operator()(uint32_t taddr, const TileCoord& t, int q, int lane, bool zero,
                                             uint8_t*) const {
    const int row = t.m_tile * kBlockM + q * 32 + lane;
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t v[32];
      if (!zero) {
        tmem_ld_32x32(taddr + c * 32, v);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = 0;
      }
      if (row < rows) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int col = t.n_tile * 128 + c * 32 + j;
          if (col < cols) {
            float x = __uint_as_float(v[j]) * alpha;
            const size_t at = static_cast<size_t>(row) * ld + col;
            if (out_is_f32) {
              float* o = static_cast<float*>(out);
              o[at] = accumulate ? o[at] + x : x;
            } else {
              static_cast<__nv_bfloat16*>(out)[at] = __float2bfloat16_rn(x);
            }
          }
        }
      }
    }
  }
};

// Host launcher (needs kernels.h for WM_CUDA / count_launch; include it before this header).
#ifdef WM_CUDA
template <int KIND, bool K_GROUPED = false, bool PROMOTE = false, class Epi>
int launch_bs(const CUtensorMap& ta, const CUtensorMap& tb, const BsArgs& args, const Epi& epi, int sms,
              cudaStream_t stream) {
  auto kernel = gemm_bs_kernel<KIND, K_GROUPED, Epi, PROMOTE>;
  constexpr int smem = BsConfig<KIND>::kTotal;
  static PerDeviceOnce configured;  // one table per template instantiation
  if (int rc = opt_in_dynamic_smem(kernel, smem, configured)) return rc;
  kernel<<<sms, kGemmThreads, smem, stream>>>(ta, tb, args, epi);
  WM_CUDA(cudaGetLastError());
  count_launch();
  return 0;
}

#endif

}  // namespace wm
