// Persistent grouped GEMM for sm_100a: TMA -> shared-memory ring -> tcgen05.mma -> TMEM -> epilogue.
//
// One kernel template serves the six contractions of the routed-MoE layer
// (reference dataflow: weftmoe/blackwell_backward.py:192-249 and
// src/cuda/blackwell/fused/impls/routed_bf16.cuh:620-1139):
//
//   M-grouped (rows of one 128-row tile all belong to one expert):
//     FC1  AB = X  * W1[e]^T   A K-major, B K-major, gate/up pair tile, SwiGLU epilogue
//     FC2  Y  = U  * W2[e]^T   A K-major, B K-major
//     dU   dU = dY * W2[e]     A K-major, B MN-major
//     dX   dX = dAB* W1[e]     A K-major, B MN-major
//   K-grouped (reduction over the rows of one expert, fixed row order, no split-K):
//     dW1[e] = dAB_e^T * X_e   A MN-major, B MN-major
//     dW2[e] = dY_e^T  * U_e   A MN-major, B MN-major
//
// CTA = 192 threads: warp 0 TMA producer, warp 1 MMA issuer (+TMEM owner), warps 2-5 epilogue
// (one TMEM lane quarter each).  Tile 128 x BLOCK_N x 64, UMMA 128 x BLOCK_N x 16, two TMEM
// accumulator stages so the epilogue of tile i overlaps the MMAs of tile i+1.
//
// Batch invariance: a row's accumulator only ever sees that row of A, the K loop always
// runs k-blocks 0..K/64-1 in order with UMMA_K = 16, and the tile shape never depends on the
// batch, so an output row's bits do not depend on its position or on co-batched rows.
#pragma once
#include "ptx.cuh"

namespace wm {

constexpr int kBlockM = 128;
constexpr int kBlockK = 64;   // 64 bf16 = one 128-byte swizzle row
constexpr int kUmmaK = 16;
constexpr int kGemmThreads = 192;

struct GemmArgs {
  // ---- schedule
  const int* tile_begin;       // M-grouped: device scalars, range of live 128-row tiles to process
  const int* tile_end;
  const int* tile_group;       // M-grouped: expert of each 128-row tile
  const int* group_row_start;  // K-grouped: [groups + 1] padded row offsets (multiples of 64)
  const int* group_live_rows;  // K-grouped, optional: [groups] rows that are not padding (the rest are zero)
  const int* group_order;      // K-grouped, optional: [groups] experts in descending order of rows (tile walk order)
  int groups;                  // K-grouped: number of experts
  const int* group_begin;      // K-grouped, optional device scalars: range of expert slots to process
  const int* group_end;        //   (null = all `groups`)
  int m_tiles_per_group;       // K-grouped: M_total / 128
  int n_tiles;                 // N_total / BLOCK_N  (gate/up pair: I / 128)
  int k_total;                 // M-grouped: reduction extent in elements
  int b_group_rows;            // rows one expert occupies in B's 2-D tensor map
  int gate_up_half;            // gate/up pair: I (row offset of the "up" half inside one expert)
  int* status;                 // device status word (0 = ok)
  // Optional device timeline (diagnostics, reference idea: src/cuda/profiling/device_timeline.cuh):
  // CTA 0 stamps %globaltimer at a few points of every tile: [tile][role 0 producer / 1 MMA][4].
  unsigned long long* timeline;
  int timeline_cta;            // the CTA whose per-tile stamps are kept
};

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

template <int BLOCK_N>
struct GemmSmem {
  static constexpr int kABytes = kBlockM * kBlockK * 2;
  static constexpr int kBBytes = BLOCK_N * kBlockK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (BLOCK_N == 256) ? 4 : 6;
  // Epilogue staging: each of the 4 epilogue warps owns 32 rows x 256 B (128 BF16 columns).
  static constexpr int kStagingBytes = 4 * 32 * 256;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kTotal = kStages * kStageBytes + kStagingBytes + kBarrierBytes + 1024;  // + alignment slack
};

struct TileCoord {
  int m_tile;    // M-grouped: 128-row tile index; K-grouped: m tile inside the expert
  int n_tile;
  int group;
  int row0;      // K-grouped: first row of the expert's segment
  int num_kb;    // number of 64-wide k blocks
};

// Reduction length of a K-grouped tile in 64-row blocks: the expert's padded rows, or, when the live
// row counts are known, only the blocks that hold a live row (the padding rows behind them are zero in
// both operands, so leaving their blocks out changes no bit of the result).
__device__ __forceinline__ int kgrouped_k_blocks(const GemmArgs& a, int group, int row0) {
  const int padded = __ldg(a.group_row_start + group + 1) - row0;
  const int rows = a.group_live_rows != nullptr ? min(__ldg(a.group_live_rows + group), padded) : padded;
  return (rows + kBlockK - 1) / kBlockK;
}

template <bool K_GROUPED>
__device__ __forceinline__ TileCoord decode_tile(const GemmArgs& a, int tile) {
  TileCoord t;
  if constexpr (!K_GROUPED) {
    t.m_tile = tile / a.n_tiles;
    t.n_tile = tile - t.m_tile * a.n_tiles;
    t.group = __ldg(a.tile_group + t.m_tile);
    t.row0 = 0;
    t.num_kb = a.k_total / kBlockK;
  } else {
    const int per_group = a.m_tiles_per_group * a.n_tiles;
    const int local_slot = tile / per_group;
    const int slot = local_slot + (a.group_begin != nullptr ? __ldg(a.group_begin) : 0);
    t.group = a.group_order != nullptr ? __ldg(a.group_order + slot) : slot;
    const int rem = tile - local_slot * per_group;
    t.m_tile = rem / a.n_tiles;
    t.n_tile = rem - t.m_tile * a.n_tiles;
    t.row0 = __ldg(a.group_row_start + t.group);
    t.num_kb = kgrouped_k_blocks(a, t.group, t.row0);
  }
  return t;
}

// Epilogue functors get: the TMEM address of the accumulator for this warp's lane quarter
// (lane field already set), the tile, the lane quarter q (rows q*32 .. q*32+31 of the tile),
// the lane id, and `zero` = the K loop was empty (nothing was accumulated: result is 0).
//
// `stage` is this warp's private 8 KB of shared memory (32 rows x 256 B).
//
// Signature: void operator()(uint32_t taddr, const TileCoord& t, int q, int lane, bool zero,
//                            uint8_t* stage) const
//
// All epilogues write global memory the same way: a 32-row x 128-column BF16 block is first
// put into `stage` (thread = row, 16-byte chunks XOR-swizzled by the row so that both the
// row-wise writes and the later chunk-wise reads hit every bank once per 128 B), then written
// out with each half-warp covering one whole 256-byte row segment: fully coalesced stores,
// local or over NVLink.

// Epilogues that keep asynchronous stores in flight define finish(lane); the others need nothing.
template <class Epilogue>
__device__ __forceinline__ auto epilogue_finish(const Epilogue& e, int lane, int) -> decltype(e.finish(lane)) {
  e.finish(lane);
}
template <class Epilogue>
__device__ __forceinline__ void epilogue_finish(const Epilogue&, int, long) {}

// An epilogue may take a seventh argument, `part`: with EPI_WARPS = 8 two warps share each TMEM lane
// quarter and the warp with part 0 / 1 handles the first / second half of the tile's columns.
template <class Epilogue>
__device__ __forceinline__ auto call_epilogue(const Epilogue& e, uint32_t taddr, const TileCoord& t, int q, int lane,
                                              bool zero, uint8_t* stage, int part, int)
    -> decltype(e(taddr, t, q, lane, zero, stage, part)) {
  e(taddr, t, q, lane, zero, stage, part);
}
template <class Epilogue>
__device__ __forceinline__ void call_epilogue(const Epilogue& e, uint32_t taddr, const TileCoord& t, int q, int lane,
                                              bool zero, uint8_t* stage, int, long) {
  e(taddr, t, q, lane, zero, stage);
}

template <int BLOCK_N, bool A_MN, bool B_MN, bool GATE_UP, bool K_GROUPED, class Epilogue, int EPI_WARPS = 4>
__global__ void __launch_bounds__(64 + 32 * EPI_WARPS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
            const GemmArgs args, const __grid_constant__ Epilogue epilogue) {
  using S = GemmSmem<BLOCK_N>;
  constexpr int kStages = S::kStages;
  constexpr uint32_t kTmemCols = 2 * BLOCK_N;  // two accumulator stages (256 or 512 columns)
  static_assert(BLOCK_N == 128 || BLOCK_N == 256, "BLOCK_N");
  static_assert(!GATE_UP || (BLOCK_N == 256 && !B_MN), "gate/up pair tile is 128+128 K-major rows");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* staging = smem + kStages * S::kStageBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(staging + S::kStagingBytes);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full = empty_bar + kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    if (args.timeline) args.timeline[kTimelineTileWords + 2 * blockIdx.x] = global_timer_ns();
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar + s, 1);
      mbar_init(empty_bar + s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(tmem_full + s, 1);
      mbar_init(tmem_empty + s, EPI_WARPS);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  int total_tiles, first_tile = 0;
  if constexpr (K_GROUPED) {
    const int slots = args.group_begin != nullptr ? __ldg(args.group_end) - __ldg(args.group_begin) : args.groups;
    total_tiles = slots * args.m_tiles_per_group * args.n_tiles;
  } else {
    first_tile = __ldg(args.tile_begin) * args.n_tiles;
    total_tiles = __ldg(args.tile_end) * args.n_tiles;
  }

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      // Issues the loads of one k block of a tile.
      auto issue = [&](const TileCoord& t, int kb, uint8_t* sa, uint64_t* bar) {
        uint8_t* sb = sa + S::kABytes;
        const int k0 = kb * kBlockK;
        auto box = [&](uint8_t* dst, const CUtensorMap* map, int x, int y) { tma_load_2d(dst, map, bar, x, y); };
        if constexpr (!A_MN) {
          box(sa, &tmap_a, k0, t.m_tile * kBlockM);
        } else {
#pragma unroll
          for (int j = 0; j < kBlockM / 64; ++j)
            box(sa + j * (kBlockK * 128), &tmap_a, t.m_tile * kBlockM + j * 64, t.row0 + k0);
        }
        if constexpr (GATE_UP) {
          const int r = t.group * args.b_group_rows + t.n_tile * 128;
          box(sb, &tmap_b, k0, r);
          box(sb + 128 * kBlockK * 2, &tmap_b, k0, r + args.gate_up_half);
        } else if constexpr (!B_MN) {
          box(sb, &tmap_b, k0, t.group * args.b_group_rows + t.n_tile * BLOCK_N);
        } else {
          const int krow = K_GROUPED ? (t.row0 + k0) : (t.group * args.b_group_rows + k0);
#pragma unroll
          for (int j = 0; j < BLOCK_N / 64; ++j)
            box(sb + j * (kBlockK * 128), &tmap_b, t.n_tile * BLOCK_N + j * 64, krow);
        }
      };
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int local_tile = 0;
      for (int tile = first_tile + blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++local_tile) {
        const bool stamp = args.timeline != nullptr && blockIdx.x == args.timeline_cta && local_tile < 64;
        unsigned long long* tl = args.timeline + local_tile * kTimelineTileStamps;
        if (stamp) tl[0] = global_timer_ns();
        const TileCoord t = decode_tile<K_GROUPED>(args, tile);
        if (stamp) tl[1] = global_timer_ns();
        for (int kb = 0; kb < t.num_kb; ++kb) {
          ok = mbar_wait(empty_bar + stage, phase ^ 1, abort_flag, args.status,
                         kStatusTimeoutSmemEmpty);
          if (!ok) break;
          if (stamp && kb == 0) tl[2] = global_timer_ns();
          if (stamp && kb == t.num_kb - 1) tl[3] = global_timer_ns();
          mbar_expect_tx(full_bar + stage, S::kStageBytes);
          issue(t, kb, smem + stage * S::kStageBytes, full_bar + stage);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(1u, kBlockM, BLOCK_N, A_MN ? 1u : 0u, B_MN ? 1u : 0u);
      // K-major, 128B swizzle: 8-row groups are 1024 B apart (SBO); LBO unused.
      // MN-major, 128B swizzle: 64-element MN atoms are kBlockK*128 B apart (LBO), 8-row k groups
      // 1024 B apart (SBO).
      constexpr uint32_t kLboA = A_MN ? kBlockK * 128 : 0, kLboB = B_MN ? kBlockK * 128 : 0;
      constexpr uint32_t kAdvA = (A_MN ? kUmmaK * 128 : kUmmaK * 2) >> 4;
      constexpr uint32_t kAdvB = (B_MN ? kUmmaK * 128 : kUmmaK * 2) >> 4;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      int local_tile = 0;
      for (int tile = first_tile + blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++local_tile) {
        const bool stamp = args.timeline != nullptr && blockIdx.x == args.timeline_cta && local_tile < 64;
        unsigned long long* tl = args.timeline + local_tile * kTimelineTileStamps + 4;
        if (stamp) tl[0] = global_timer_ns();
        const TileCoord t = decode_tile<K_GROUPED>(args, tile);
        ok = mbar_wait(tmem_empty + acc, acc_phase ^ 1, abort_flag, args.status,
                       kStatusTimeoutTmemEmpty);
        if (!ok) break;
        if (stamp) tl[1] = global_timer_ns();
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BLOCK_N;
        for (int kb = 0; kb < t.num_kb; ++kb) {
          ok = mbar_wait(full_bar + stage, phase, abort_flag, args.status, kStatusTimeoutSmemFull);
          if (!ok) break;
          if (stamp && kb == 0) tl[2] = global_timer_ns();
          if (stamp && kb == t.num_kb - 1) tl[3] = global_timer_ns();
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * S::kStageBytes);
          const uint32_t sb = sa + S::kABytes;
          const uint64_t da = umma_desc_sw128(sa, kLboA, 1024);
          const uint64_t db = umma_desc_sw128(sb, kLboB, 1024);
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {
            umma_bf16(tmem_d, da + k * kAdvA, db + k * kAdvB, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(empty_bar + stage);  // frees the stage once these MMAs have read it
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(tmem_full + acc);  // accumulator complete (fires at once for an empty K loop)
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    int local_tile = 0;
    for (int tile = first_tile + blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++local_tile) {
      const bool stamp = args.timeline != nullptr && blockIdx.x == args.timeline_cta && local_tile < 64 && lane == 0;
      unsigned long long* tl = args.timeline + local_tile * kTimelineTileStamps + 8 + ((warp - 2) & 3);
      const TileCoord t = decode_tile<K_GROUPED>(args, tile);
      ok = mbar_wait(tmem_full + acc, acc_phase, abort_flag, args.status, kStatusTimeoutTmemFull);
      if (!ok) break;
      if (stamp && warp == 2) tl[0] = global_timer_ns();
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BLOCK_N;
      call_epilogue(epilogue, taddr, t, q, lane, t.num_kb == 0,
                    staging + (warp - 2) * (S::kStagingBytes / EPI_WARPS), (warp - 2) >> 2, 0);
      tc_fence_before();
      __syncwarp();
      if (stamp && warp > 2 && warp < 6) tl[0] = global_timer_ns();
      if (lane == 0) mbar_arrive(tmem_empty + acc);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    epilogue_finish(epilogue, lane, 0);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0 && args.timeline)
    args.timeline[kTimelineTileWords + 2 * blockIdx.x + 1] = global_timer_ns();
}

}  // namespace wm

#include "epilogue.cuh"
