// Epilogues shared by the one-CTA (gemm.cuh) and CTA-pair (gemm2.cuh) grouped GEMM kernels.
// Include after TileCoord / kBlockM are defined.
#pragma once
#include "ptx.cuh"

namespace wm {

// 32 packed BF16 columns (16 words) of row `lane` into chunk group c32 (0..3) of the staging block.
__device__ __forceinline__ void stage_put32(uint8_t* stage, int lane, int c32, const uint32_t (&w)[16]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int pos = (c32 * 4 + j) ^ (lane & 15);
    *reinterpret_cast<uint4*>(stage + lane * 256 + pos * 16) =
        make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
  }
}
// Accumulator columns [col, col+32) of this thread's row, rounded to BF16 and packed.
__device__ __forceinline__ void load_pack32(uint32_t taddr, bool zero, uint32_t (&w)[16]) {
  if (zero) {
#pragma unroll
    for (int j = 0; j < 16; ++j) w[j] = 0;
    return;
  }
  uint32_t v[32];
  tmem_ld_32x32(taddr, v);
  tmem_ld_wait();
#pragma unroll
  for (int j = 0; j < 16; ++j)
    w[j] = pack_bf16x2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
}
// One step of a software-pipelined read-out in 64-column groups: wait for the group whose load is in
// flight in `v`, round it to BF16 into `w`, and (when `next_taddr` != 0) start the load of the next
// group into `v`, so that its latency overlaps whatever the caller does with `w`.
__device__ __forceinline__ void take_pack64(uint32_t (&v)[64], uint32_t (&w)[32], uint32_t next_taddr) {
  tmem_ld_wait();
#pragma unroll
  for (int j = 0; j < 32; ++j)
    w[j] = pack_bf16x2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
  if (next_taddr != 0) tmem_ld_32x64(next_taddr, v);
}
// 64 packed BF16 columns (32 words) of row `lane` into chunk groups 2*c64, 2*c64+1 of the staging block.
__device__ __forceinline__ void stage_put64(uint8_t* stage, int lane, int c64, const uint32_t (&w)[32]) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int pos = (c64 * 8 + j) ^ (lane & 15);
    *reinterpret_cast<uint4*>(stage + lane * 256 + pos * 16) =
        make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
  }
}
// Write the staged 32 x 128 block: half-warp h handles row 2*it + h, lane&15 picks the 16-byte
// chunk.  `row_dst(r)` returns the global address of column 0 of the block in row r (or nullptr
// to skip the row).
template <class RowDst>
__device__ __forceinline__ void stage_flush(const uint8_t* stage, int lane, RowDst row_dst) {
  const int c = lane & 15;
#pragma unroll 4
  for (int it = 0; it < 16; ++it) {
    const int r = 2 * it + (lane >> 4);
    const uint4 v = *reinterpret_cast<const uint4*>(stage + r * 256 + ((c ^ (r & 15)) << 4));
    __nv_bfloat16* dst = row_dst(r);
    if (dst != nullptr) *reinterpret_cast<uint4*>(dst + c * 8) = v;
  }
}

// Plain BF16 store: out[(group_base) + row, col] with leading dimension ld.
//   M-grouped: row = m_tile*128 + r.   K-grouped: out + group*group_stride, row = m_tile*128 + r.
template <int BLOCK_N>
struct EpilogueStore {
  __nv_bfloat16* out;
  long long group_stride;  // elements between experts (K-grouped), 0 for M-grouped
  int ld;

  __device__ __forceinline__ void operator()(uint32_t taddr, const TileCoord& t, int q, int lane,
                                             bool zero, uint8_t* stage) const {
    const long long row0 = static_cast<long long>(t.m_tile) * kBlockM + q * 32;
    __nv_bfloat16* base = out + group_stride * t.group + row0 * ld + t.n_tile * BLOCK_N;
#pragma unroll 1
    for (int half = 0; half < BLOCK_N / 128; ++half) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t w[16];
        load_pack32(taddr + half * 128 + c * 32, zero, w);
        stage_put32(stage, lane, c, w);
      }
      __syncwarp();
      __nv_bfloat16* block = base + half * 128;
      const int ldl = ld;
      stage_flush(stage, lane, [block, ldl](int r) { return block + static_cast<long long>(r) * ldl; });
      __syncwarp();
    }
  }
};

// Plain BF16 store through TMA: each warp packs its 32 rows into two 128-byte-swizzled boxes
// (32 rows x 64 columns, 4 KB each) and one lane issues a bulk tensor store per box, so the warp
// spends no instructions on reading the staging back and writing global memory.  `out` is described by
// a 2-D tensor map over [all rows][ld] with box {64, 32}; K-grouped outputs stack the experts along
// the rows (row = group * rows_per_group + m_tile * 128 + r).  A box is reused once the store issued
// from it one half earlier has finished reading it.
template <int BLOCK_N>
struct EpilogueStoreTma {
  alignas(64) CUtensorMap tmap;
  int rows_per_group;  // K-grouped: M (rows of one expert's output); 0 for M-grouped

  __device__ __forceinline__ void operator()(uint32_t taddr, const TileCoord& t, int q, int lane,
                                             bool zero, uint8_t* stage) const {
    const int row0 = t.group * rows_per_group + t.m_tile * kBlockM + q * 32;
    const int col0 = t.n_tile * BLOCK_N;
    constexpr int kUnits = BLOCK_N / 64;
    // Software pipeline over the 64-column units: the TMEM load of unit u+1 is issued as soon as unit
    // u's registers are packed, so its latency overlaps the shared-memory writes and the store issue of
    // unit u instead of standing in front of every unit.
    uint32_t v[64];
    if (!zero) tmem_ld_32x64(taddr, v);
#pragma unroll
    for (int unit = 0; unit < kUnits; ++unit) {
      uint32_t w[32];
      if (zero) {
#pragma unroll
        for (int j = 0; j < 32; ++j) w[j] = 0;
      } else {
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j)
          w[j] = pack_bf16x2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
        if (unit + 1 < kUnits) tmem_ld_32x64(taddr + (unit + 1) * 64, v);
      }
      uint8_t* box = stage + (unit & 1) * 4096;
      if (lane == 0) bulk_wait_group_read<1>();  // the store issued from this box two units ago
      __syncwarp();
#pragma unroll
      for (int j = 0; j < 8; ++j)
        *reinterpret_cast<uint4*>(box + lane * 128 + ((j ^ (lane & 7)) << 4)) =
            make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        tma_store_2d(&tmap, box, col0 + unit * 64, row0);
        bulk_commit_group();
      }
    }
  }
  // Before the CTA exits: every store has finished reading shared memory.
  __device__ __forceinline__ void finish(int lane) const {
    if (lane == 0) bulk_wait_group_read<0>();
  }
};

// FP32 store through TMA (weight gradients for FP32 master parameters: the accumulator leaves unrounded).
// Same scheme as EpilogueStoreTma with 32-column units: a 32 x 32 FP32 box has the same 128-byte rows, so
// the swizzle and the two alternating 4 KB boxes per warp are unchanged.  `out` is described by a 2-D map
// over [all rows][ld] FP32 with box {32, 32}.
template <int BLOCK_N>
struct EpilogueStoreTmaF32 {
  alignas(64) CUtensorMap tmap;
  int rows_per_group;  // K-grouped: M (rows of one expert's output); 0 for M-grouped

  __device__ __forceinline__ void operator()(uint32_t taddr, const TileCoord& t, int q, int lane,
                                             bool zero, uint8_t* stage) const {
    const int row0 = t.group * rows_per_group + t.m_tile * kBlockM + q * 32;
    const int col0 = t.n_tile * BLOCK_N;
    constexpr int kUnits = BLOCK_N / 32;
    uint32_t v[32];
    if (!zero) tmem_ld_32x32(taddr, v);
#pragma unroll
    for (int unit = 0; unit < kUnits; ++unit) {
      uint32_t w[32];
      if (zero) {
#pragma unroll
        for (int j = 0; j < 32; ++j) w[j] = 0;
      } else {
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) w[j] = v[j];
        if (unit + 1 < kUnits) tmem_ld_32x32(taddr + (unit + 1) * 32, v);
      }
      uint8_t* box = stage + (unit & 1) * 4096;
      if (lane == 0) bulk_wait_group_read<1>();  // the store issued from this box two units ago
      __syncwarp();
#pragma unroll
      for (int j = 0; j < 8; ++j)
        *reinterpret_cast<uint4*>(box + lane * 128 + ((j ^ (lane & 7)) << 4)) =
            make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        tma_store_2d(&tmap, box, col0 + unit * 32, row0);
        bulk_commit_group();
      }
    }
  }
  __device__ __forceinline__ void finish(int lane) const {
    if (lane == 0) bulk_wait_group_read<0>();
  }
};

// FC1 epilogue (reference: src/cuda/blackwell/fused/impls/routed_bf16.cuh:874-1027):
// accumulator columns [0,128) are gate, [128,256) are up for intermediate columns
// n_tile*128 .. +127.  gate and up are rounded to BF16 first (that rounded pair is what the
// training cache stores), then u = bf16( silu(gate) * up * prob ).
struct EpilogueSwiglu {
  __nv_bfloat16* u;         // [rows, I]
  __nv_bfloat16* ab;        // [rows, 2I] or nullptr (inference)
  const float* row_prob;    // [rows] gate probability of the routed row (0 on padding rows)
  int inter;                // I

  __device__ __forceinline__ void operator()(uint32_t taddr, const TileCoord& t, int q, int lane,
                                             bool, uint8_t* stage) const {
    const long long row0 = static_cast<long long>(t.m_tile) * kBlockM + q * 32;
    const float prob = row_prob[row0 + lane];
    const int col0 = t.n_tile * 128;
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t g[32], b[32];
      tmem_ld_32x32(taddr + c * 32, g);
      tmem_ld_32x32(taddr + 128 + c * 32, b);
      tmem_ld_wait();
      uint32_t pu[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float g0 = bf16_round(__uint_as_float(g[2 * j])), g1 = bf16_round(__uint_as_float(g[2 * j + 1]));
        const float b0 = bf16_round(__uint_as_float(b[2 * j])), b1 = bf16_round(__uint_as_float(b[2 * j + 1]));
        // __fdividef: the IEEE division falls into its slow subroutine for the zero / non-finite
        // operands that padding rows hold, which made tail tiles 2-3x slower than full ones.
        const float u0 = __fdividef(g0, 1.0f + __expf(-g0)) * b0 * prob;
        const float u1 = __fdividef(g1, 1.0f + __expf(-g1)) * b1 * prob;
        pu[j] = pack_bf16x2(u0, u1);
      }
      stage_put32(stage, lane, c, pu);
    }
    __syncwarp();
    {
      __nv_bfloat16* block = u + row0 * inter + col0;
      const int ldl = inter;
      stage_flush(stage, lane, [block, ldl](int r) { return block + static_cast<long long>(r) * ldl; });
    }
    __syncwarp();
    if (ab != nullptr) {
      // Training cache: the BF16-rounded gate and up halves, re-read from TMEM.
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t w[16];
          load_pack32(taddr + half * 128 + c * 32, false, w);
          stage_put32(stage, lane, c, w);
        }
        __syncwarp();
        __nv_bfloat16* block = ab + row0 * (2 * inter) + half * inter + col0;
        const int ldl = 2 * inter;
        stage_flush(stage, lane, [block, ldl](int r) { return block + static_cast<long long>(r) * ldl; });
        __syncwarp();
      }
    }
  }
};

// dU epilogue with the SwiGLU backward fused in (reference math: weftmoe/blackwell_backward.py:81-113),
// for the one-CTA kernel with EIGHT epilogue warps (two per TMEM lane quarter; `part` picks the half of the
// tile's 256 columns): four warps would need longer for this arithmetic than the main loop of a tile.
// The accumulator holds dU for intermediate columns n_tile*256 .. +255; it is rounded to BF16 (the value a
// separate dU buffer would have held) and combined with the saved BF16 gate/up row:
//   sig = sigmoid(a); silu = a*sig; U = bf16(silu*b*p)
//   dA = bf16(dU*p*b*sig*(1+a*(1-sig))); dB = bf16(dU*p*silu); dprob += dU*silu*b
// U, dA and dB leave one after the other through a 32-row x 32-column staging block (80-byte row pitch:
// the eight lanes of a store phase hit distinct banks); the row's partial dprob over this warp's 128
// columns goes to dprob_part[2*n_tile + part][row] and is summed in fixed order by dprob_finish.
struct EpilogueSwigluBackward {
  const __nv_bfloat16* ab;   // [rows, 2I] saved gate | up
  const float* row_prob;     // [rows]
  __nv_bfloat16* u;          // [rows, I]
  __nv_bfloat16* dab;        // [rows, 2I]
  float* dprob_part;         // [I / 128][row_capacity]
  int inter;                 // I
  int row_capacity;

  __device__ __forceinline__ void flush(const uint8_t* stage, int lane, const uint32_t (&w)[16],
                                        __nv_bfloat16* dst, long long ld) const {
    constexpr int kPitch = 80;
#pragma unroll
    for (int j = 0; j < 4; ++j)
      *reinterpret_cast<uint4*>(const_cast<uint8_t*>(stage) + lane * kPitch + j * 16) =
          make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
    __syncwarp();
    const int j = lane & 3;  // four lanes cover one 64-byte row segment: eight rows per store instruction
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int r = 8 * it + (lane >> 2);
      *reinterpret_cast<uint4*>(dst + r * ld + j * 8) = *reinterpret_cast<const uint4*>(stage + r * kPitch + j * 16);
    }
    __syncwarp();
  }

  __device__ __forceinline__ void operator()(uint32_t taddr, const TileCoord& t, int q, int lane,
                                             bool zero, uint8_t* stage, int part) const {
    const long long row0 = static_cast<long long>(t.m_tile) * kBlockM + q * 32;
    const long long row = row0 + lane;
    const float p = row_prob[row];
    const int col0 = t.n_tile * 256 + part * 128;
    const __nv_bfloat16* arow = ab + row * (2 * inter) + col0;
    float dsum = 0.0f;
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint4 va[4], vb[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        va[j] = reinterpret_cast<const uint4*>(arow + c * 32)[j];
        vb[j] = reinterpret_cast<const uint4*>(arow + inter + c * 32)[j];
      }
      uint32_t d[32];
      if (zero) {
#pragma unroll
        for (int j = 0; j < 32; ++j) d[j] = 0;
      } else {
        tmem_ld_32x32(taddr + part * 128 + c * 32, d);
        tmem_ld_wait();
      }
      const uint32_t* wa = reinterpret_cast<const uint32_t*>(va);
      const uint32_t* wb = reinterpret_cast<const uint32_t*>(vb);
      uint32_t ou[16], oa[16], ob[16];
#pragma unroll
      for (int k = 0; k < 16; ++k) {
        float ru[2], ra[2], rb[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const float a = __uint_as_float(h ? (wa[k] & 0xffff0000u) : (wa[k] << 16));
          const float b = __uint_as_float(h ? (wb[k] & 0xffff0000u) : (wb[k] << 16));
          const float du = bf16_round(__uint_as_float(d[2 * k + h]));
          const float sig = __fdividef(1.0f, 1.0f + __expf(-a));
          const float silu = a * sig;
          const float act = silu * b;
          ru[h] = act * p;
          ra[h] = du * p * b * (sig * (1.0f + a * (1.0f - sig)));
          rb[h] = du * p * silu;
          dsum += du * act;
        }
        ou[k] = pack_bf16x2(ru[0], ru[1]);
        oa[k] = pack_bf16x2(ra[0], ra[1]);
        ob[k] = pack_bf16x2(rb[0], rb[1]);
      }
      flush(stage, lane, ou, u + row0 * inter + col0 + c * 32, inter);
      flush(stage, lane, oa, dab + row0 * (2 * inter) + col0 + c * 32, 2 * inter);
      flush(stage, lane, ob, dab + row0 * (2 * inter) + inter + col0 + c * 32, 2 * inter);
    }
    dprob_part[static_cast<long long>(2 * t.n_tile + part) * row_capacity + row] = dsum;
  }
};

// Return epilogue (FC2 contributions and backward dX rows): each routed row is written as
// BF16 into the SOURCE rank's mailbox [sorted_slot][token][N], local or over NVLink through
// the peer-mapped arena (reference: routed_bf16.cuh:1028-1139 and
// weftmoe/blackwell_backward.py:116-144).  origin = src_rank*cap*K + token*K + sorted_slot,
// -1 on padding rows.
constexpr int kMaxRanks = 8;
template <int BLOCK_N>
struct EpiloguePush {
  __nv_bfloat16* mailbox[kMaxRanks];  // peer-mapped base of each rank's mailbox
  const int* origin;                  // [rows]
  int cap;                            // tokens capacity per rank
  int top_k;
  int ld;                             // N_total (hidden)

  __device__ __forceinline__ __nv_bfloat16* select_mailbox(int src) const {
    __nv_bfloat16* p = mailbox[0];
#pragma unroll
    for (int r = 1; r < kMaxRanks; ++r)
      if (src == r) p = mailbox[r];
    return p;
  }

  __device__ __forceinline__ void operator()(uint32_t taddr, const TileCoord& t, int q, int lane,
                                             bool, uint8_t* stage) const {
    const long long row = static_cast<long long>(t.m_tile) * kBlockM + q * 32 + lane;
    const int org = origin[row];
    unsigned long long my_dst = 0;  // destination of column n_tile*BLOCK_N of this thread's row
    if (org >= 0) {
      const int per_rank = cap * top_k;
      const int src = org / per_rank;
      const int rem = org - src * per_rank;
      const int token = rem / top_k, slot = rem - token * top_k;
      my_dst = reinterpret_cast<unsigned long long>(
          select_mailbox(src) + (static_cast<long long>(slot) * cap + token) * ld + t.n_tile * BLOCK_N);
    }
    // 64-column groups, read one group ahead: the load of the next group (or half) is in flight while
    // this half is staged and written out.
    constexpr int kGroups = BLOCK_N / 64;
    uint32_t v[64];
    tmem_ld_32x64(taddr, v);
#pragma unroll
    for (int half = 0; half < BLOCK_N / 128; ++half) {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int group = half * 2 + c;
        uint32_t w[32];
        take_pack64(v, w, group + 1 < kGroups ? taddr + (group + 1) * 64 : 0u);
        stage_put64(stage, lane, c, w);
      }
      __syncwarp();
      stage_flush(stage, lane, [my_dst, half](int r) {
        const unsigned long long d = __shfl_sync(0xffffffffu, my_dst, r);
        return d ? reinterpret_cast<__nv_bfloat16*>(d) + half * 128 : nullptr;
      });
      __syncwarp();
    }
  }
};

// ---------------------------------------------------------------- scaled variants (quantised paths)
// Same stores as EpilogueStore / EpiloguePush with the FP32 accumulator multiplied by a constant first
// (the product of the NVFP4 layer scales; 1 for blockwise FP8, whose scales live in the MMA).
__device__ __forceinline__ void load_pack32_scaled(uint32_t taddr, float alpha, uint32_t (&w)[16]) {
  uint32_t v[32];
  tmem_ld_32x32(taddr, v);
  tmem_ld_wait();
#pragma unroll
  for (int j = 0; j < 16; ++j)
    w[j] = pack_bf16x2(__uint_as_float(v[2 * j]) * alpha, __uint_as_float(v[2 * j + 1]) * alpha);
}

template <int BLOCK_N>
struct EpilogueStoreScaled {
  __nv_bfloat16* out;
  int ld;
  float alpha;
  long long group_stride;  // elements between experts' outputs (K-grouped), 0 for M-grouped

  __device__ __forceinline__ void operator()(uint32_t taddr, const TileCoord& t, int q, int lane, bool,
                                             uint8_t* stage) const {
    static_assert(BLOCK_N == 128, "the block-scaled kernel uses 128-wide tiles");
    const long long row0 = static_cast<long long>(t.m_tile) * kBlockM + q * 32;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t w[16];
      load_pack32_scaled(taddr + c * 32, alpha, w);
      stage_put32(stage, lane, c, w);
    }
    __syncwarp();
    __nv_bfloat16* block = out + group_stride * t.group + row0 * ld + t.n_tile * BLOCK_N;
    const int ldl = ld;
    stage_flush(stage, lane, [block, ldl](int r) { return block + static_cast<long long>(r) * ldl; });
    __syncwarp();
  }
};

template <int BLOCK_N>
struct EpiloguePushScaled {
  EpiloguePush<BLOCK_N> push;
  float alpha;

  __device__ __forceinline__ void operator()(uint32_t taddr, const TileCoord& t, int q, int lane, bool,
                                             uint8_t* stage) const {
    static_assert(BLOCK_N == 128, "the block-scaled kernel uses 128-wide tiles");
    const long long row = static_cast<long long>(t.m_tile) * kBlockM + q * 32 + lane;
    const int org = push.origin[row];
    unsigned long long my_dst = 0;
    if (org >= 0) {
      const int per_rank = push.cap * push.top_k;
      const int src = org / per_rank;
      const int rem = org - src * per_rank;
      const int token = rem / push.top_k, slot = rem - token * push.top_k;
      my_dst = reinterpret_cast<unsigned long long>(
          push.select_mailbox(src) + (static_cast<long long>(slot) * push.cap + token) * push.ld +
          t.n_tile * BLOCK_N);
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t w[16];
      load_pack32_scaled(taddr + c * 32, alpha, w);
      stage_put32(stage, lane, c, w);
    }
    __syncwarp();
    stage_flush(stage, lane, [my_dst](int r) {
      const unsigned long long d = __shfl_sync(0xffffffffu, my_dst, r);
      return d ? reinterpret_cast<__nv_bfloat16*>(d) : nullptr;
    });
    __syncwarp();
  }
};

}  // namespace wm
