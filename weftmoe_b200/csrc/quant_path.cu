// Quantised forward path (blockwise FP8 and NVFP4): staging of quantised source packets, the
// owner-side pull of quantised rows with their scale factors laid out for the tensor core, the
// SwiGLU + re-quantisation stage between FC1 and FC2, and the block-scaled grouped GEMM launchers.
//
// Reference dataflow: FP8 — docs/usage.md:116-125,207-224 (source packets FP8[H] + FP32[H/128]; FC1;
// SwiGLU; Z quantised 1 x 128; FC2; BF16 contributions).  NVFP4 — weftmoe/nvfp4.py:145-159,252-278 and
// tests/torchrun_sm100_nvfp4.py:36-47: accumulators scaled by sx*s1 and rounded to BF16, u = silu(a)*b*prob
// quantised block-16 with layer scale sm, FC2 scaled by sm*s2, BF16 contributions.
// All kernels here are HBM-bound byte work; the GEMMs are gemm_bs.cuh.
#include <cuda_fp8.h>

#include "../../include/weftmoe_b200.h"
#include "kernels.h"
#include "gemm_bs.cuh"
#include "quant_path.h"

namespace wm {

namespace {

__device__ __forceinline__ unsigned e2m1x2_local(float hi, float lo) {
  unsigned short r;
  asm("{ .reg .b8 p; cvt.rn.satfinite.e2m1x2.f32 p, %1, %2; cvt.u16.u8 %0, p; }" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ uint2 encode16(const float (&v)[16], float six_s, float s, unsigned char* sf_byte) {
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
    bytes[i] = e2m1x2_local(hi, lo);
  }
  *sf_byte = sb;
  return make_uint2(bytes[0] | (bytes[1] << 8) | (bytes[2] << 16) | (bytes[3] << 24),
                    bytes[4] | (bytes[5] << 8) | (bytes[6] << 16) | (bytes[7] << 24));
}
__device__ __forceinline__ float fp8_block_scale(float amax, bool invalid) {
  if (invalid || !isfinite(amax)) return __int_as_float(0x7fc00000);
  if (amax == 0.0f) return 1.0f;
  const unsigned bits = __float_as_uint(amax);
  int exponent = static_cast<int>(bits >> 23) - 8 + ((bits & 0x7fffffu) > 0x600000u);
  exponent = exponent < 1 ? 1 : exponent;
  return __uint_as_float(static_cast<unsigned>(exponent) << 23);
}
__device__ __forceinline__ unsigned pack4_e4m3(float a, float b, float c, float d) {
  const unsigned lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const unsigned hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}
// Word index of row r inside a 128-row scale-factor chunk.
__device__ __forceinline__ int chunk_word(int r) { return (r & 31) * 4 + ((r & 127) >> 5); }

// ------------------------------------------------------------------ owner-side pull
// One warp per padded row: copy the quantised row from its source rank's staging buffer and write
// its scale words into the chunked layout; padding rows get zero data and neutral scales.
// by_origin != 0 (backward): `meta_origin` is the saved origin array (-1 on padding rows) and nothing is
// written to origin_out / prob_out.
__global__ void gather_q_kernel(OwnerRows o, int rank, int e_local, int world, int cap, int top_k, int kind,
                                int hidden,
                                PeerBytes stage, size_t sf_offset, const int* __restrict__ meta_origin,
                                const float* __restrict__ meta_prob, uint8_t* __restrict__ rows_out,
                                uint32_t* __restrict__ sfa_out, int* __restrict__ origin_out,
                                float* __restrict__ prob_out, int by_origin) {
  const int rows = *o.rows.end;
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int row_bytes = kind == kKindFp8 ? hidden : hidden / 2;
  const int sf_words = kind == kKindFp8 ? hidden / 128 : hidden / 64;
  const int vecs = row_bytes / 16;
  for (int r = *o.rows.begin + ((blockIdx.x * blockDim.x + threadIdx.x) >> 5); r < rows; r += warps) {
    bool live;
    if (by_origin) {
      live = meta_origin[r] >= 0;
    } else {
      const int l = o.tile_group[r >> 7];
      live = r - o.padded_start[l] < o.expert_total[rank * e_local + l];
    }
    uint4* dst = reinterpret_cast<uint4*>(rows_out + static_cast<size_t>(r) * row_bytes);
    uint32_t* sf_dst = sfa_out + static_cast<size_t>(r >> 7) * sf_words * 128 + chunk_word(r);
    // An origin outside [0, world * cap * top_k) is a word its source never wrote: treat the row as padding.
    const int org = live ? meta_origin[r] : -1;
    if (live && org >= 0 && org < world * cap * top_k) {
      const int src = org / (cap * top_k);
      const int token = (org - src * cap * top_k) / top_k;
      const uint8_t* base = stage.p[src];
      const uint4* from = reinterpret_cast<const uint4*>(base + static_cast<size_t>(token) * row_bytes);
      for (int c = lane; c < vecs; c += 32) dst[c] = from[c];
      for (int j = lane; j < sf_words; j += 32) {
        uint32_t word;
        if (kind == kKindFp8) {
          const float s = reinterpret_cast<const float*>(base + sf_offset)[static_cast<size_t>(token) * sf_words + j];
          word = ((__float_as_uint(s) >> 23) & 0xffu) * 0x01010101u;
        } else {
          word = reinterpret_cast<const uint32_t*>(base + sf_offset)[static_cast<size_t>(token) * sf_words + j];
        }
        sf_dst[static_cast<size_t>(j) * 128] = word;
      }
      if (lane == 0 && !by_origin) {
        origin_out[r] = org;
        prob_out[r] = meta_prob[r];
      }
    } else {
      for (int c = lane; c < vecs; c += 32) dst[c] = make_uint4(0, 0, 0, 0);
      for (int j = lane; j < sf_words; j += 32) sf_dst[static_cast<size_t>(j) * 128] = kind == kKindFp8 ? 0x7f7f7f7fu : 0u;
      if (lane == 0 && !by_origin) {
        origin_out[r] = -1;
        prob_out[r] = 0.0f;
      }
    }
  }
}

// ------------------------------------------------------------------ SwiGLU + re-quantisation
// One warp per row, one lane per 16 intermediate columns.  a and b are the BF16-rounded gate and up
// accumulators; u = silu(a) * b * prob in FP32 is quantised without an intermediate BF16 rounding.
__global__ void swiglu_quantize_kernel(DeviceRange range, const __nv_bfloat16* __restrict__ ab,
                                       const float* __restrict__ prob, int inter, int kind, float six_s,
                                       float s, uint8_t* __restrict__ uq, uint32_t* __restrict__ sfa_out) {
  const int rows = *range.end;
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int groups = inter / 16;
  for (int r = *range.begin + ((blockIdx.x * blockDim.x + threadIdx.x) >> 5); r < rows; r += warps) {
    const float p = prob[r];
    const __nv_bfloat16* row = ab + static_cast<size_t>(r) * 2 * inter;
    for (int g = lane; g < groups; g += 32) {
      const uint4* pa = reinterpret_cast<const uint4*>(row + g * 16);
      const uint4* pb = reinterpret_cast<const uint4*>(row + inter + g * 16);
      const uint4 a0 = pa[0], a1 = pa[1], b0 = pb[0], b1 = pb[1];
      const unsigned wa[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const unsigned wb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
      float u[16];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const float a = __uint_as_float(h ? (wa[j] & 0xffff0000u) : (wa[j] << 16));
          const float b = __uint_as_float(h ? (wb[j] & 0xffff0000u) : (wb[j] << 16));
          u[2 * j + h] = (a / (1.0f + expf(-a))) * b * p;
        }
      }
      if (kind == kKindNvfp4) {
        unsigned char sb;
        const uint2 packed = encode16(u, six_s, s, &sb);
        *reinterpret_cast<uint2*>(uq + static_cast<size_t>(r) * (inter / 2) + g * 8) = packed;
        const int k64 = inter / 64;
        reinterpret_cast<uint8_t*>(sfa_out)[((static_cast<size_t>(r >> 7) * k64 + (g >> 2)) * 128 + chunk_word(r)) * 4 + (g & 3)] = sb;
      } else {
        // a 1 x 128 block spans eight consecutive lanes
        float amax = 0.0f;
        bool bad = false;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          amax = fmaxf(amax, fabsf(u[j]));
          bad |= !isfinite(u[j]);
        }
        const unsigned mask = 0xffu << (lane & 24);
#pragma unroll
        for (int d = 4; d; d >>= 1) {
          amax = fmaxf(amax, __shfl_xor_sync(mask, amax, d, 8));
          bad |= __shfl_xor_sync(mask, static_cast<int>(bad), d, 8) != 0;
        }
        const float scale = fp8_block_scale(amax, bad);
        const float inv = scale != scale ? scale : __uint_as_float(0x7f000000u - __float_as_uint(scale));
        uint4 out;
        out.x = pack4_e4m3(u[0] * inv, u[1] * inv, u[2] * inv, u[3] * inv);
        out.y = pack4_e4m3(u[4] * inv, u[5] * inv, u[6] * inv, u[7] * inv);
        out.z = pack4_e4m3(u[8] * inv, u[9] * inv, u[10] * inv, u[11] * inv);
        out.w = pack4_e4m3(u[12] * inv, u[13] * inv, u[14] * inv, u[15] * inv);
        *reinterpret_cast<uint4*>(uq + static_cast<size_t>(r) * inter + g * 16) = out;
        if ((lane & 7) == 0) {
          const int kb = g >> 3, kblocks = inter / 128;
          sfa_out[(static_cast<size_t>(r >> 7) * kblocks + kb) * 128 + chunk_word(r)] =
              ((__float_as_uint(scale) >> 23) & 0xffu) * 0x01010101u;
        }
      }
    }
  }
}

// ------------------------------------------------------------------ FP8 helpers of the backward pass
// BF16 rows -> E4M3 bytes + UE8M0 scale words in the chunked layout (1 x 128 blocks): sixteen lanes per
// block, eight values per lane, over a device-side row range.
__global__ void fp8_quantize_rows_chunked_kernel(DeviceRange range, const __nv_bfloat16* __restrict__ x,
                                                 int cols, uint8_t* __restrict__ q,
                                                 uint32_t* __restrict__ sfa_out) {
  const int row0 = *range.begin, rows = *range.end;
  const int kblocks = cols / 128;
  const long long blocks = static_cast<long long>(rows - row0) * kblocks;
  const long long half_warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 4;
  const int sub = threadIdx.x & 15;
  const unsigned mask = 0xffffu << (threadIdx.x & 16);
  for (long long b = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 4; b < blocks; b += half_warps) {
    const int r = row0 + static_cast<int>(b / kblocks), kb = static_cast<int>(b % kblocks);
    const uint4 raw = reinterpret_cast<const uint4*>(x + static_cast<size_t>(r) * cols + kb * 128)[sub];
    const unsigned w[4] = {raw.x, raw.y, raw.z, raw.w};
    float v[8], m = 0.0f;
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
    const float scale = fp8_block_scale(m, bad);
    const float inv = scale != scale ? scale : __uint_as_float(0x7f000000u - __float_as_uint(scale));
    uint2 out;
    out.x = pack4_e4m3(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv);
    out.y = pack4_e4m3(v[4] * inv, v[5] * inv, v[6] * inv, v[7] * inv);
    reinterpret_cast<uint2*>(q + static_cast<size_t>(r) * cols + kb * 128)[sub] = out;
    if (sub == 0)
      sfa_out[(static_cast<size_t>(r >> 7) * kblocks + kb) * 128 + chunk_word(r)] =
          ((__float_as_uint(scale) >> 23) & 0xffu) * 0x01010101u;
  }
}

// E4M3 rows + chunked UE8M0 scales -> BF16 rows (exact: the scale is a power of two).
__global__ void fp8_dequantize_rows_kernel(DeviceRange range, const uint8_t* __restrict__ q,
                                           const uint32_t* __restrict__ sfa, int cols,
                                           __nv_bfloat16* __restrict__ out) {
  const int row0 = *range.begin, rows = *range.end;
  const int kblocks = cols / 128;
  const long long blocks = static_cast<long long>(rows - row0) * kblocks;
  const long long half_warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 4;
  const int sub = threadIdx.x & 15;
  for (long long b = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 4; b < blocks; b += half_warps) {
    const int r = row0 + static_cast<int>(b / kblocks), kb = static_cast<int>(b % kblocks);
    const uint2 raw = reinterpret_cast<const uint2*>(q + static_cast<size_t>(r) * cols + kb * 128)[sub];
    const unsigned e8 = sfa[(static_cast<size_t>(r >> 7) * kblocks + kb) * 128 + chunk_word(r)] & 0xffu;
    const float scale = e8 == 0xffu ? __int_as_float(0x7fc00000) : __uint_as_float(e8 << 23);
    const unsigned words[2] = {raw.x, raw.y};
    unsigned o[4];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      float f[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>((words[j] >> (8 * i)) & 0xffu), __NV_E4M3);
        f[i] = __half2float(__half(h)) * scale;
      }
      o[2 * j] = pack_bf16x2(f[0], f[1]);
      o[2 * j + 1] = pack_bf16x2(f[2], f[3]);
    }
    reinterpret_cast<uint4*>(out + static_cast<size_t>(r) * cols + kb * 128)[sub] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

template <int KIND>
int launch_bs_grouped(const Schedule& s, const void* a, const SfLayout& sfa, const void* b, const SfLayout& sfb,
                      __nv_bfloat16* out, const PushTarget* push, int n, int k, float alpha, int* status,
                      int sms, cudaStream_t stream, const float* b_scales) {
  const int kbytes = KIND == kKindFp8 ? k : k / 2;
  CUtensorMap ta, tb;
  if (int rc = make_tmap_2d(&ta, a, 1, kbytes, s.row_capacity, kbytes, 128, 128)) return rc;
  if (int rc = make_tmap_2d(&tb, b, 1, kbytes, static_cast<uint64_t>(s.groups) * n, kbytes, 128, 128)) return rc;
  BsArgs args{};
  const DeviceRange tiles = split_range(s.split, 0, s.chunk);
  args.base.tile_begin = tiles.begin;
  args.base.tile_end = tiles.end;
  args.base.tile_group = s.tile_group;
  args.base.n_tiles = n / 128;
  args.base.k_total = k;
  args.base.b_group_rows = n;
  args.base.status = status;
  args.sfa = sfa;
  args.sfb = sfb;
  args.a_block_rows = 1;
  args.b_scales = b_scales;
  // FP8 weight scales with mantissas: the promotion form of the kernel (gemm_bs.cuh).
  constexpr bool kCanPromote = KIND == kKindFp8;
  if (push) {
    EpiloguePushScaled<128> epi{};
    for (int r = 0; r < kMaxPeers; ++r) epi.push.mailbox[r] = push->mailbox[r];
    epi.push.origin = push->origin;
    epi.push.cap = push->cap;
    epi.push.top_k = push->top_k;
    epi.push.ld = n;
    epi.alpha = alpha;
    if constexpr (kCanPromote)
      if (b_scales != nullptr) return launch_bs<KIND, false, true>(ta, tb, args, epi, sms, stream);
    return launch_bs<KIND>(ta, tb, args, epi, sms, stream);
  }
  EpilogueStoreScaled<128> epi{out, n, alpha, 0};
  if constexpr (kCanPromote)
    if (b_scales != nullptr) return launch_bs<KIND, false, true>(ta, tb, args, epi, sms, stream);
  return launch_bs<KIND>(ta, tb, args, epi, sms, stream);
}

// Weight gradient: out[e] [m, n] = alpha * A[:, rows_e] * B[:, rows_e]^T, operands stored K-major
// over the padded rows (A [m, row_capacity], B [n, row_capacity] elements).
template <int KIND>
int launch_bs_kgrouped(const Schedule& s, const void* a, const SfLayout& sfa, const void* b, const SfLayout& sfb,
                       __nv_bfloat16* out, int m, int n, float alpha, int* status, int sms, cudaStream_t stream) {
  const int kbytes = KIND == kKindFp8 ? s.row_capacity : s.row_capacity / 2;
  CUtensorMap ta, tb;
  if (int rc = make_tmap_2d(&ta, a, 1, kbytes, m, kbytes, 128, 128)) return rc;
  if (int rc = make_tmap_2d(&tb, b, 1, kbytes, n, kbytes, 128, 128)) return rc;
  BsArgs args{};
  args.base.group_row_start = s.group_row_start;
  args.base.groups = s.groups;
  args.base.m_tiles_per_group = m / 128;
  args.base.n_tiles = n / 128;
  args.base.status = status;
  args.sfa = sfa;
  args.sfb = sfb;
  EpilogueStoreScaled<128> epi{out, n, alpha, static_cast<long long>(m) * n};
  return launch_bs<KIND, true>(ta, tb, args, epi, sms, stream);
}

// BF16 rows [rows, cols] -> E4M3 of the TRANSPOSE, qt [cols][row_capacity], quantised 1 x 128 along the
// rows (the reduction axis of a weight gradient; reference: column re-quantisation, docs/usage.md:122-125),
// with the UE8M0 scale words in the chunked layout of a K-major operand whose rows are the columns of x:
// chunk (cols/128 tile, 128-row block).  One warp per (128-row block, 64 columns): two columns per lane,
// first the column maxima, then sixteen rows at a time.
__global__ void fp8_quantize_cols_chunked_kernel(DeviceRange range, const __nv_bfloat16* __restrict__ x,
                                                 int cols, int row_capacity, uint8_t* __restrict__ qt,
                                                 uint32_t* __restrict__ sf_out) {
  const int row0 = *range.begin, rows = *range.end;
  const int rblocks = (rows - row0) >> 7, cgroups = cols / 64, rblocks_total = row_capacity >> 7;
  const long long units = static_cast<long long>(rblocks) * cgroups;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  for (long long unit = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; unit < units;
       unit += warps) {
    const int rb = static_cast<int>(unit / cgroups), cg = static_cast<int>(unit % cgroups);
    const int r_first = row0 + rb * 128, c = cg * 64 + lane * 2;
    const unsigned* src = reinterpret_cast<const unsigned*>(x + static_cast<size_t>(r_first) * cols + c);
    const size_t pitch = static_cast<size_t>(cols) / 2;  // in 32-bit words
    float m0 = 0.0f, m1 = 0.0f;
    bool bad0 = false, bad1 = false;  // a non-finite value poisons only its own column's block
#pragma unroll 8
    for (int r = 0; r < 128; ++r) {
      const unsigned w = src[r * pitch];
      const float a = __uint_as_float(w << 16), b = __uint_as_float(w & 0xffff0000u);
      m0 = fmaxf(m0, fabsf(a));
      m1 = fmaxf(m1, fabsf(b));
      bad0 |= !isfinite(a);
      bad1 |= !isfinite(b);
    }
    const float s0 = fp8_block_scale(m0, bad0), s1 = fp8_block_scale(m1, bad1);
    const float i0 = s0 != s0 ? s0 : __uint_as_float(0x7f000000u - __float_as_uint(s0));
    const float i1 = s1 != s1 ? s1 : __uint_as_float(0x7f000000u - __float_as_uint(s1));
    uint8_t* dst0 = qt + static_cast<size_t>(c) * row_capacity + r_first;
    uint8_t* dst1 = dst0 + row_capacity;
#pragma unroll 1
    for (int g = 0; g < 8; ++g) {
      float a[16], b[16];
#pragma unroll
      for (int r = 0; r < 16; ++r) {
        const unsigned w = src[(g * 16 + r) * pitch];
        a[r] = __uint_as_float(w << 16) * i0;
        b[r] = __uint_as_float(w & 0xffff0000u) * i1;
      }
      uint4 oa, ob;
      oa.x = pack4_e4m3(a[0], a[1], a[2], a[3]);   oa.y = pack4_e4m3(a[4], a[5], a[6], a[7]);
      oa.z = pack4_e4m3(a[8], a[9], a[10], a[11]); oa.w = pack4_e4m3(a[12], a[13], a[14], a[15]);
      ob.x = pack4_e4m3(b[0], b[1], b[2], b[3]);   ob.y = pack4_e4m3(b[4], b[5], b[6], b[7]);
      ob.z = pack4_e4m3(b[8], b[9], b[10], b[11]); ob.w = pack4_e4m3(b[12], b[13], b[14], b[15]);
      *reinterpret_cast<uint4*>(dst0 + g * 16) = oa;
      *reinterpret_cast<uint4*>(dst1 + g * 16) = ob;
    }
    const int kb = (r_first >> 7);
    uint32_t* chunk = sf_out + (static_cast<size_t>(c >> 7) * rblocks_total + kb) * 128;
    chunk[chunk_word(c)] = ((__float_as_uint(s0) >> 23) & 0xffu) * 0x01010101u;
    chunk[chunk_word(c + 1)] = ((__float_as_uint(s1) >> 23) & 0xffu) * 0x01010101u;
  }
}

}  // namespace

int gather_q_rows(const OwnerRows& o, int rank, int e_local, int world, int cap, int top_k, int kind, int hidden,
                  const PeerBytes& stage, size_t sf_offset, const int* meta_origin, const float* meta_prob,
                  uint8_t* rows_out, uint32_t* sfa_out, int* origin_out, float* prob_out, int by_origin,
                  int ctas, cudaStream_t stream) {
  gather_q_kernel<<<ctas, 256, 0, stream>>>(o, rank, e_local, world, cap, top_k, kind, hidden, stage, sf_offset,
                                            meta_origin, meta_prob, rows_out, sfa_out, origin_out, prob_out,
                                            by_origin);
  WM_CUDA(cudaGetLastError());
  count_launch();
  return 0;
}

int swiglu_quantize(DeviceRange rows, const __nv_bfloat16* ab, const float* prob, int inter, int kind,
                    float layer_scale, uint8_t* uq, uint32_t* sfa_out, int sms, cudaStream_t stream) {
  swiglu_quantize_kernel<<<sms * 8, 256, 0, stream>>>(rows, ab, prob, inter, kind,
                                                      static_cast<float>(6.0 * static_cast<double>(layer_scale)),
                                                      layer_scale, uq, sfa_out);
  WM_CUDA(cudaGetLastError());
  count_launch();
  return 0;
}

int fp8_quantize_rows_chunked(DeviceRange rows, const __nv_bfloat16* x, int cols, uint8_t* q,
                              uint32_t* sfa_out, int sms, cudaStream_t stream) {
  fp8_quantize_rows_chunked_kernel<<<sms * 16, 256, 0, stream>>>(rows, x, cols, q, sfa_out);
  WM_CUDA(cudaGetLastError());
  count_launch();
  return 0;
}

int fp8_dequantize_rows(DeviceRange rows, const uint8_t* q, const uint32_t* sfa, int cols,
                        __nv_bfloat16* out, int sms, cudaStream_t stream) {
  fp8_dequantize_rows_kernel<<<sms * 16, 256, 0, stream>>>(rows, q, sfa, cols, out);
  WM_CUDA(cudaGetLastError());
  count_launch();
  return 0;
}

int fp8_quantize_cols_chunked(DeviceRange rows, const __nv_bfloat16* x, int cols, int row_capacity,
                              uint8_t* qt, uint32_t* sf_out, int sms, cudaStream_t stream) {
  fp8_quantize_cols_chunked_kernel<<<sms * 8, 256, 0, stream>>>(rows, x, cols, row_capacity, qt, sf_out);
  WM_CUDA(cudaGetLastError());
  count_launch();
  return 0;
}

int launch_block_scaled_kgrouped(int kind, const Schedule& s, const void* a, const SfLayout& sfa, const void* b,
                                 const SfLayout& sfb, __nv_bfloat16* out, int m, int n, float alpha,
                                 int* status, int sms, cudaStream_t stream) {
  if (m % 128 || n % 128 || s.row_capacity % 128) {
    set_error("block-scaled weight gradient needs M, N and the row capacity to be multiples of 128 "
              "(M=%d, N=%d, rows=%d)", m, n, s.row_capacity);
    return 2;
  }
  return kind == kKindFp8
             ? launch_bs_kgrouped<kKindFp8>(s, a, sfa, b, sfb, out, m, n, alpha, status, sms, stream)
             : launch_bs_kgrouped<kKindNvfp4>(s, a, sfa, b, sfb, out, m, n, alpha, status, sms, stream);
}

int launch_block_scaled(int kind, const Schedule& s, const void* a, const SfLayout& sfa, const void* b,
                        const SfLayout& sfb, __nv_bfloat16* out, const PushTarget* push, int n, int k,
                        float alpha, int* status, int sms, cudaStream_t stream, const float* b_scales) {
  if (n % 128 || k % (kind == kKindFp8 ? 128 : 256)) {
    set_error("block-scaled grouped GEMM needs N %% 128 == 0 and K %% %d == 0 (N=%d, K=%d)",
              kind == kKindFp8 ? 128 : 256, n, k);
    return 2;
  }
  return kind == kKindFp8
             ? launch_bs_grouped<kKindFp8>(s, a, sfa, b, sfb, out, push, n, k, alpha, status, sms, stream, b_scales)
             : launch_bs_grouped<kKindNvfp4>(s, a, sfa, b, sfb, out, push, n, k, alpha, status, sms, stream, nullptr);
}

}  // namespace wm
