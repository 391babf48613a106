// CTA-pair grouped GEMM for sm_100a: two CTAs (a cluster of 2, one per SM) compute one
// 256 x BLOCK_N tile with tcgen05.mma.cta_group::2.
//
// Why pairs: a 128 x 256 x 64 step of a single-CTA kernel pulls 48 KB through L2 per 4.2 MFLOP;
// at the tensor-core rate that is far more than L2 can deliver, so the one-CTA kernel (gemm.cuh)
// is L2-bound.  In a pair each CTA fetches only its own 128 rows of A and HALF of the B tile
// (BLOCK_N/2 rows), the UMMA reads both halves of B from the two CTAs' shared memory, and the
// same FLOPs cost 2/3 of the bytes per CTA; with twice the M extent the L2 traffic per FLOP halves.
// Nothing is broadcast: every CTA issues plain tiled loads for its own tiles.
//
// Roles per CTA (192 threads): warp 0 TMA producer, warp 1 MMA issuer (leader CTA only; the peer's
// warp 1 only owns its TMEM allocation), warps 2-5 epilogue.
// Barriers (all waits bounded):
//   full[s]       leader only.  The leader's producer arms it with the bytes of BOTH CTAs; both
//                 CTAs' loads credit it (the peer's loads name the leader's barrier).
//   empty[s]      one per CTA; the leader's MMA thread commits to its own and to the peer's.
//   tmem_full[a]  one per CTA; same double commit.
//   tmem_empty[a] leader only, 8 arrivals: four epilogue warps of each CTA.
// M-grouped schedules pair two 128-row tiles of the SAME expert (pair_tiles[2p], [2p+1]; the second
// is -1 for an expert with an odd tile count: that CTA re-reads the first tile and stores nothing).
#pragma once
#include "gemm.cuh"

namespace wm {

template <int BLOCK_N>
struct Gemm2Smem {
  static constexpr int kABytes = kBlockM * kBlockK * 2;          // this CTA's 128 rows
  static constexpr int kBBytes = (BLOCK_N / 2) * kBlockK * 2;    // this CTA's half of B
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (BLOCK_N == 256) ? 6 : 8;
  static constexpr int kStagingBytes = 4 * 32 * 256;
  static constexpr int kBarrierBytes = 512;
  static constexpr int kTotal = kStages * kStageBytes + kStagingBytes + kBarrierBytes + 1024;
};

struct Gemm2Args {
  GemmArgs base;
  const int* pair_begin;  // M-grouped: device scalars, range of pairs to process
  const int* pair_end;
  const int* pair_tiles;  // M-grouped: [2 * pairs] 128-row tile indices, -1 = none
};

struct PairTile {
  TileCoord t;   // m_tile = this CTA's 128-row tile (epilogue coordinates)
  int load_m;    // 128-row tile this CTA loads A from (== t.m_tile unless the slot is empty)
  bool live;     // false: this CTA has no rows in this pair (compute, store nothing)
};

template <bool K_GROUPED>
__device__ __forceinline__ PairTile decode_pair(const Gemm2Args& a, int work, int cta) {
  PairTile p;
  const GemmArgs& g = a.base;
  if constexpr (!K_GROUPED) {
    const int pair = work / g.n_tiles;
    p.t.n_tile = work - pair * g.n_tiles;
    const int first = __ldg(a.pair_tiles + 2 * pair);
    const int mine = __ldg(a.pair_tiles + 2 * pair + cta);
    p.live = mine >= 0;
    p.load_m = p.live ? mine : first;
    p.t.m_tile = p.load_m;
    p.t.group = __ldg(g.tile_group + first);
    p.t.row0 = 0;
    p.t.num_kb = g.k_total / kBlockK;
  } else {
    const int m_pairs = g.m_tiles_per_group / 2;
    const int per_group = m_pairs * g.n_tiles;
    const int local_slot = work / per_group;
    const int slot = local_slot + (g.group_begin != nullptr ? __ldg(g.group_begin) : 0);
    p.t.group = g.group_order != nullptr ? __ldg(g.group_order + slot) : slot;
    const int rem = work - local_slot * per_group;
    const int mp = rem / g.n_tiles;
    p.t.n_tile = rem - mp * g.n_tiles;
    p.t.m_tile = mp * 2 + cta;
    p.load_m = p.t.m_tile;
    p.live = true;
    p.t.row0 = __ldg(g.group_row_start + p.t.group);
    p.t.num_kb = kgrouped_k_blocks(g, p.t.group, p.t.row0);
  }
  return p;
}

template <int BLOCK_N, bool A_MN, bool B_MN, bool GATE_UP, bool K_GROUPED, class Epilogue>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm2_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
             const Gemm2Args args2, const __grid_constant__ Epilogue epilogue) {
  using S = Gemm2Smem<BLOCK_N>;
  constexpr int kStages = S::kStages;
  constexpr int kHalfN = BLOCK_N / 2;
  constexpr uint32_t kTmemCols = 2 * BLOCK_N;
  static_assert(BLOCK_N == 128 || BLOCK_N == 256, "BLOCK_N");
  static_assert(!GATE_UP || (BLOCK_N == 256 && !B_MN), "gate/up pair tile is 128+128 K-major rows");
  const GemmArgs& args = args2.base;

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
  const int cta = static_cast<int>(cluster_ctarank());  // 0 = leader
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar + s, 1);
      mbar_init(empty_bar + s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(tmem_full + s, 1);
      mbar_init(tmem_empty + s, 8);  // four epilogue warps of each CTA of the pair
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    // Each CTA takes all of its own TMEM, so both allocations start at column 0 and the pair
    // MMA can address the two accumulators with one address.
    tmem_alloc(tmem_holder, kTmemCols == 512 ? 512 : 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  int total_work, first_work = 0;
  if constexpr (K_GROUPED) {
    const int slots = args.group_begin != nullptr ? __ldg(args.group_end) - __ldg(args.group_begin) : args.groups;
    total_work = slots * (args.m_tiles_per_group / 2) * args.n_tiles;
  } else {
    first_work = __ldg(args2.pair_begin) * args.n_tiles;
    total_work = __ldg(args2.pair_end) * args.n_tiles;
  }

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int work = first_work + cluster_id; ok && work < total_work; work += num_clusters) {
        const PairTile p = decode_pair<K_GROUPED>(args2, work, cta);
        const TileCoord& t = p.t;
        for (int kb = 0; kb < t.num_kb; ++kb) {
          ok = mbar_wait_cluster(empty_bar + stage, phase ^ 1, abort_flag, args.status,
                                 kStatusTimeoutSmemEmpty);
          if (!ok) break;
          uint8_t* sa = smem + stage * S::kStageBytes;
          uint8_t* sb = sa + S::kABytes;
          const uint32_t bar = map_to_cta(smem_u32(full_bar + stage), 0);  // leader's barrier
          if (cta == 0) mbar_expect_tx(full_bar + stage, 2 * S::kStageBytes);
          const int k0 = kb * kBlockK;
          if constexpr (!A_MN) {
            tma_load_2d_pair(sa, &tmap_a, bar, k0, p.load_m * kBlockM);
          } else {
#pragma unroll
            for (int j = 0; j < kBlockM / 64; ++j)
              tma_load_2d_pair(sa + j * (kBlockK * 128), &tmap_a, bar, p.load_m * kBlockM + j * 64,
                               t.row0 + k0);
          }
          if constexpr (GATE_UP) {
            // leader holds the gate rows, the peer the up rows of the same intermediate columns
            tma_load_2d_pair(sb, &tmap_b, bar, k0,
                             t.group * args.b_group_rows + t.n_tile * 128 + cta * args.gate_up_half);
          } else if constexpr (!B_MN) {
            tma_load_2d_pair(sb, &tmap_b, bar, k0,
                             t.group * args.b_group_rows + t.n_tile * BLOCK_N + cta * kHalfN);
          } else {
            const int krow = K_GROUPED ? (t.row0 + k0) : (t.group * args.b_group_rows + k0);
#pragma unroll
            for (int j = 0; j < kHalfN / 64; ++j)
              tma_load_2d_pair(sb + j * (kBlockK * 128), &tmap_b, bar,
                               t.n_tile * BLOCK_N + cta * kHalfN + j * 64, krow);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && cta == 0) {
      constexpr uint32_t idesc = umma_idesc(1u, 2 * kBlockM, BLOCK_N, A_MN ? 1u : 0u, B_MN ? 1u : 0u);
      constexpr uint32_t kLboA = A_MN ? kBlockK * 128 : 0, kLboB = B_MN ? kBlockK * 128 : 0;
      constexpr uint32_t kAdvA = (A_MN ? kUmmaK * 128 : kUmmaK * 2) >> 4;
      constexpr uint32_t kAdvB = (B_MN ? kUmmaK * 128 : kUmmaK * 2) >> 4;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int work = first_work + cluster_id; ok && work < total_work; work += num_clusters) {
        const PairTile p = decode_pair<K_GROUPED>(args2, work, 0);
        ok = mbar_wait_cluster(tmem_empty + acc, acc_phase ^ 1, abort_flag, args.status,
                               kStatusTimeoutTmemEmpty);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BLOCK_N;
        for (int kb = 0; kb < p.t.num_kb; ++kb) {
          ok = mbar_wait_cluster(full_bar + stage, phase, abort_flag, args.status,
                                 kStatusTimeoutSmemFull);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * S::kStageBytes);
          const uint32_t sb = sa + S::kABytes;
          const uint64_t da = umma_desc_sw128(sa, kLboA, 1024);
          const uint64_t db = umma_desc_sw128(sb, kLboB, 1024);
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k)
            umma_bf16_pair(tmem_d, da + k * kAdvA, db + k * kAdvB, idesc, (kb | k) != 0 ? 1u : 0u);
          const uint32_t e = smem_u32(empty_bar + stage);
          umma_commit_pair(e);                 // frees this stage in the leader ...
          umma_commit_pair(map_to_cta(e, 1));  // ... and in the peer
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        const uint32_t f = smem_u32(tmem_full + acc);
        umma_commit_pair(f);
        umma_commit_pair(map_to_cta(f, 1));
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int work = first_work + cluster_id; ok && work < total_work; work += num_clusters) {
      const PairTile p = decode_pair<K_GROUPED>(args2, work, cta);
      ok = mbar_wait_cluster(tmem_full + acc, acc_phase, abort_flag, args.status,
                             kStatusTimeoutTmemFull);
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BLOCK_N;
      if (p.live) epilogue(taddr, p.t, q, lane, p.t.num_kb == 0, staging + (warp - 2) * (32 * 256));
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(tmem_empty + acc), 0));
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    epilogue_finish(epilogue, lane, 0);
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's shared memory and barriers stay valid until both are done
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols == 512 ? 512 : 256);
  }
}

}  // namespace wm
