// Route planning ("notify") kernels: per-token combine order, per-expert counts, stable
// per-source ordinals, count exchange through peer-mapped arenas, destination rows.
//
// Integer-only and deterministic: the same routes always give the same rows, which is what
// makes the weight-gradient reduction order and the combine order reproducible.
// Reference behaviour restated here (not its code):
//   combine order  — weftmoe/blackwell.py:10-13, src/cuda/weftmoe_pf/route_plan.cuh:29-50
//   ordinals       — weftmoe/blackwell_backward.py:20-37
//   canonical rows — src/metadata/notify_dispatch.cpp:835-906
//   counts/notify  — src/cuda/blackwell/fused/impls/routed_bf16.cuh:294-373
// All kernels are HBM/latency-bound integer work over T*K route words.
#include "kernels.h"
#include "ptx.cuh"
#include <atomic>
#include <cstdlib>

#include "route.h"

namespace wm {

constexpr int kChunk = 1024;  // routes per CTA in the counting passes (one per thread)

// ------------------------------------------------------------------ K1: per-token sort
// One warp per token; lane s < K owns original slot s.  Position = number of slots that sort
// before it under key (valid ? id : E, slot).
__global__ void sort_slots_kernel(const int* __restrict__ routes, int tokens, int top_k, int experts,
                                  int* __restrict__ sorted_slot, int* __restrict__ sorted_expert,
                                  int* __restrict__ slot_pos) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= tokens) return;
  const int id = lane < top_k ? routes[warp * top_k + lane] : experts + 1;
  const bool valid = id >= 0 && id < experts;
  const int key = lane < top_k ? (valid ? id : experts) : experts + 1;
  int pos = 0;
  for (int j = 0; j < top_k; ++j) {
    const int kj = __shfl_sync(0xffffffffu, key, j);
    pos += (kj < key) || (kj == key && j < lane);
  }
  if (lane < top_k) {
    sorted_slot[warp * top_k + pos] = lane;
    sorted_expert[warp * top_k + pos] = valid ? id : -1;
    slot_pos[warp * top_k + lane] = pos;
  }
}

// ------------------------------------------------------------------ K2a: chunk histograms
__global__ void chunk_hist_kernel(const int* __restrict__ routes, int n, int experts,
                                  int* __restrict__ chunk_hist) {
  extern __shared__ int hist[];
  for (int e = threadIdx.x; e < experts; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  const int i = blockIdx.x * kChunk + threadIdx.x;
  if (i < n) {
    const int id = routes[i];
    if (id >= 0 && id < experts) atomicAdd(&hist[id], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x)
    chunk_hist[static_cast<size_t>(blockIdx.x) * experts + e] = hist[e];
}

// ------------------------------------------------------------------ K2b: scan over chunks
// One warp per expert: exclusive prefix of the chunk counts (in place), total into
// local_count[e] and into row `rank` of every rank's count matrix (peer-mapped stores).
__global__ void chunk_scan_kernel(int* __restrict__ chunk_hist, int chunks, int experts,
                                  int* __restrict__ local_count, PeerInts count_matrix, int world,
                                  int rank) {
  const int e = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (e >= experts) return;
  int running = 0;
  for (int base = 0; base < chunks; base += 32) {
    const int c = base + lane;
    const int v = c < chunks ? chunk_hist[static_cast<size_t>(c) * experts + e] : 0;
    int incl = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += up;
    }
    if (c < chunks) chunk_hist[static_cast<size_t>(c) * experts + e] = running + incl - v;
    running += __shfl_sync(0xffffffffu, incl, 31);
  }
  if (lane == 0) local_count[e] = running;
  if (lane < world) count_matrix.p[lane][rank * experts + e] = running;
}

// ------------------------------------------------------------------ Kg: global plan
// Single CTA.  Waits for every rank's count row of this generation, then derives per expert:
// total rows, rows from lower ranks, unpadded and padded base inside the owner; and for this
// rank as owner: padded row start per local expert, the 128-row tile -> expert map, tile count.
// Publish an empty owner schedule: every later kernel of the call finds empty ranges (M-grouped work,
// copies) or zero-length reductions (K-grouped GEMMs then write zero gradients).
__device__ void publish_empty_schedule(const PlanTables& t, int e_local) {
  for (int l = threadIdx.x; l <= e_local; l += blockDim.x) t.padded_start[l] = 0;
  if (t.live_rows != nullptr)
    for (int l = threadIdx.x; l < e_local; l += blockDim.x) t.live_rows[l] = 0;
  if (t.group_order != nullptr)
    for (int l = threadIdx.x; l < e_local; l += blockDim.x) t.group_order[l] = l;
  if (threadIdx.x == 0) {
    *t.num_tiles = 0;
    *t.padded_rows = 0;
    *t.num_pairs = 0;
  }
  if (t.split != nullptr) {
    // no tiles, pairs or rows in any chunk; chunk 0 still names every local expert, so that the weight
    // gradients of an empty call are written as zeros
    for (int i = threadIdx.x; i < kSplitWords; i += blockDim.x) {
      const int row = i / kSplitStride, c = i - row * kSplitStride;
      t.split[i] = (row == 3 && c >= 1) ? e_local : 0;
    }
  }
}

// The plan itself, for one CTA whose threads have all seen every count row (callers wait for the COUNTS
// flags and synchronise the block first).  total / padded: [experts] words, pair_first: [513] words and
// flags: [1] word of shared memory.
__device__ void global_plan_body(const int* __restrict__ count_matrix, int world, int rank, int experts,
                                 int row_capacity, const PlanTables& t, int* status, int split_percent,
                                 int chunks, int* total, int* padded, int* pair_first, int* overflow) {
  const int e_local = experts / world;
  if (threadIdx.x == 0) *overflow = 0;
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    int sum = 0, before = 0;
    for (int s = 0; s < world; ++s) {
      const int c = count_matrix[s * experts + e];
      sum += c;
      if (s < rank) before += c;
    }
    total[e] = sum;
    padded[e] = (sum + 127) / 128 * 128;
    t.expert_total[e] = sum;
    t.expert_before[e] = before;
  }
  __syncthreads();
  // Per-owner exclusive prefixes (unpadded and padded).  One thread per owner; E/EP <= 512.
  if (threadIdx.x < world) {
    int base = 0, pbase = 0;
    for (int l = 0; l < e_local; ++l) {
      const int e = threadIdx.x * e_local + l;
      t.expert_base[e] = base;
      t.expert_pbase[e] = pbase;
      base += total[e];
      pbase += padded[e];
    }
    // Every rank holds the same count matrix and the same row capacity, so every rank sees every
    // owner's overflow and all of them fail the call together (the reference checks every destination
    // rank's rows on every rank too: src/metadata/notify_dispatch.cpp:2003-2035).
    if (pbase > row_capacity) *overflow = 1;
    if (threadIdx.x == rank) {
      *t.num_tiles = pbase / 128;
      *t.padded_rows = pbase;
      t.padded_start[e_local] = pbase;
    }
  }
  __syncthreads();
  if (*overflow || *t.padded_rows == 0) {
    if (*overflow && threadIdx.x == 0) atomicCAS(status, 0, kStatusRowOverflow);
    __syncthreads();
    publish_empty_schedule(t, e_local);
    return;
  }
  // CTA-pair schedule: consecutive 128-row tiles of one expert are paired; an odd last tile
  // is paired with -1.  pair_first[l] = pairs of lower local experts (sequential, E/EP <= 512).
  if (threadIdx.x == 0) {
    int p = 0;
    for (int l = 0; l < e_local; ++l) {
      pair_first[l] = p;
      p += (padded[rank * e_local + l] / 128 + 1) / 2;
    }
    *t.num_pairs = p;
    if (t.split != nullptr) {
      // Chunk c ends at the first expert boundary at or beyond c / chunks of the padded rows (with two
      // chunks: at split_percent of them).
      const int total_rows = *t.padded_rows;
      int* tiles_b = t.split;
      int* pairs_b = t.split + kSplitStride;
      int* rows_b = t.split + 2 * kSplitStride;
      int* experts_b = t.split + 3 * kSplitStride;
      tiles_b[0] = pairs_b[0] = rows_b[0] = experts_b[0] = 0;
      int rows = 0, l = 0;
      for (int c = 1; c <= kMaxChunks; ++c) {
        if (c < chunks) {
          const long long share = chunks == 2 ? split_percent : 100ll * c / chunks;
          while (l < e_local && 100ll * rows < share * total_rows) rows += padded[rank * e_local + l++];
          tiles_b[c] = rows / 128;
          pairs_b[c] = l < e_local ? pair_first[l] : p;
          rows_b[c] = rows;
          experts_b[c] = l;
        } else {
          tiles_b[c] = total_rows / 128;
          pairs_b[c] = p;
          rows_b[c] = total_rows;
          experts_b[c] = e_local;
        }
      }

    }
  }
  __syncthreads();
  for (int l = threadIdx.x; l < e_local; l += blockDim.x) {
    const int e = rank * e_local + l;
    const int start = t.expert_pbase[e];
    const int tiles = padded[e] / 128;
    t.padded_start[l] = start;
    if (t.live_rows != nullptr) t.live_rows[l] = total[e];
    if (t.group_order != nullptr) {
      // position of expert l when the experts of ITS CHUNK are sorted by rows, largest first (counting
      // sort by comparison: at most 512 local experts); without a split all experts form one chunk
      int first = 0, last = e_local;
      if (t.split != nullptr) {
        const int* experts_b = t.split + 3 * kSplitStride;
        for (int c = 0; c < kMaxChunks; ++c)
          if (l >= experts_b[c] && l < experts_b[c + 1]) {
            first = experts_b[c];
            last = experts_b[c + 1];
          }
      }
      int before = 0;
      for (int j = first; j < last; ++j) {
        const int other = total[rank * e_local + j];
        before += (other > total[e]) || (other == total[e] && j < l);
      }
      t.group_order[first + before] = l;
    }
    for (int k = 0; k < tiles; ++k) t.tile_group[start / 128 + k] = l;
    for (int j = 0; j < (tiles + 1) / 2; ++j) {
      t.pair_tiles[2 * (pair_first[l] + j)] = start / 128 + 2 * j;
      t.pair_tiles[2 * (pair_first[l] + j) + 1] = (2 * j + 1 < tiles) ? start / 128 + 2 * j + 1 : -1;
    }
  }
}

__global__ void global_plan_kernel(const int* __restrict__ count_matrix, const int* flag_counts,
                                   Gen gen, int world, int rank, int experts,
                                   int row_capacity, PlanTables t, int* status, int split_percent,
                                   int chunks, long long wait_budget) {
  extern __shared__ int sh[];
  int* total = sh;               // [experts]
  int* padded = sh + experts;    // [experts]
  __shared__ int ok, overflow;
  __shared__ int pair_first[513];
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if (threadIdx.x < world) {
    if (!wait_flag_ge(flag_counts + threadIdx.x * kFlagStride, gen.value(), status, wait_budget)) ok = 0;
  }
  __syncthreads();
  if (!ok) {  // a count row never arrived: the status word is set, nothing may be derived from the counts
    publish_empty_schedule(t, experts / world);
    return;
  }
  global_plan_body(count_matrix, world, rank, experts, row_capacity, t, status, split_percent, chunks, total,
                   padded, pair_first, &overflow);
}

// ------------------------------------------------------------------ K2c: destination rows + meta push
// One route per thread, 1024 routes per CTA in route order.  Stable ordinal inside the chunk
// = (same-expert routes in earlier warps) + (same-expert lanes below me in my warp).
__global__ void route_rows_kernel(const int* __restrict__ routes, const float* __restrict__ gates,
                                  const int* __restrict__ slot_pos, int n, int top_k, int experts,
                                  int world, int rank, int cap, const int* __restrict__ chunk_base,
                                  PlanTables t, int* __restrict__ local_offset,
                                  int* __restrict__ dst_rank, int* __restrict__ dst_row,
                                  int* __restrict__ dst_prow, PeerInts meta_origin,
                                  PeerFloats meta_prob, int row_capacity,
                                  const int* __restrict__ status) {
  extern __shared__ unsigned short warp_cnt[];  // [32][experts]
  // A failed plan (a wait that ran out, a row overflow) left no tables to read: push nothing.
  if (status != nullptr && *status != 0) return;
  for (int k = threadIdx.x; k < 32 * experts; k += blockDim.x) warp_cnt[k] = 0;
  __syncthreads();
  const int i = blockIdx.x * kChunk + threadIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int id = i < n ? routes[i] : -1;
  const bool valid = id >= 0 && id < experts;
  const int key = valid ? id : experts;
  const unsigned peers = __match_any_sync(0xffffffffu, key);
  const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
  if (valid && rank_in_warp == 0) warp_cnt[warp * experts + id] = static_cast<unsigned short>(__popc(peers));
  __syncthreads();
  if (i >= n) return;
  if (!valid) {
    local_offset[i] = dst_rank[i] = dst_row[i] = dst_prow[i] = -1;
    return;
  }
  int ordinal = chunk_base[static_cast<size_t>(blockIdx.x) * experts + id] + rank_in_warp;
  for (int w = 0; w < warp; ++w) ordinal += warp_cnt[w * experts + id];
  const int e_local = experts / world;
  const int owner = id / e_local;
  const int within = t.expert_before[id] + ordinal;
  const int prow = t.expert_pbase[id] + within;
  local_offset[i] = ordinal;
  dst_rank[i] = owner;
  dst_row[i] = t.expert_base[id] + within;
  dst_prow[i] = prow;
  if (meta_origin.p[owner] != nullptr && prow >= 0 && prow < row_capacity) {
    const int token = i / top_k;
    meta_origin.p[owner][prow] = rank * cap * top_k + token * top_k + slot_pos[i];
    meta_prob.p[owner][prow] = gates[i];
  }
}

__global__ void route_primary_kernel(const int* __restrict__ slot_pos,
                                     const int* __restrict__ dst_rank,
                                     const int* __restrict__ dst_prow, int n, int top_k,
                                     PeerInts meta_primary, int* __restrict__ per_route,
                                     int row_capacity, const int* __restrict__ status) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  if (status != nullptr && *status != 0) return;  // route_rows wrote nothing
  const int owner = dst_rank[i];
  if (owner < 0) {
    if (per_route) per_route[i] = -1;
    return;
  }
  const int base = (i / top_k) * top_k;
  int head = i, head_pos = slot_pos[i];
  for (int j = 0; j < top_k; ++j) {
    const int r = base + j;
    if (dst_rank[r] == owner && slot_pos[r] < head_pos) {
      head = r;
      head_pos = slot_pos[r];
    }
  }
  const int prow = dst_prow[i];
  if (meta_primary.p[owner] != nullptr && prow >= 0 && prow < row_capacity)
    meta_primary.p[owner][prow] = dst_prow[head];
  if (per_route) per_route[i] = dst_prow[head];
}

// ------------------------------------------------------------------ Ks: the whole plan in one CTA
// For calls of at most kSmallPlanRoutes routes (decode, small prefill): per-token sort, stable ordinals
// and counts, count exchange, global plan, destination rows, origin / prob / primary words to the
// owners and the READY hand-shake, all in ONE launch of one 1024-thread CTA instead of nine small
// launches in a row.  Every step computes exactly what the stand-alone kernels above compute.
// Shared memory: total[E], padded[E], running[E] ints and warp_cnt[32][E] shorts.
__global__ void __launch_bounds__(1024, 1) plan_small_kernel(const SmallPlan a) {
  extern __shared__ int sh[];
  const int E = a.shape.experts, K = a.shape.top_k, world = a.shape.world, rank = a.shape.rank;
  int* total = sh;
  int* padded = sh + E;
  int* running = sh + 2 * E;
  unsigned short* warp_cnt = reinterpret_cast<unsigned short*>(sh + 3 * E);  // [32][E]
  __shared__ int pair_first[513];
  __shared__ int ok, overflow;
  const int n = a.tokens * K;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int generation = a.generation.value();

  // (1) per-token combine order: one warp per token
  for (int token = warp; token < a.tokens; token += 32) {
    const int id = lane < K ? a.routes[token * K + lane] : E + 1;
    const bool valid = id >= 0 && id < E;
    const int key = lane < K ? (valid ? id : E) : E + 1;
    int pos = 0;
    for (int j = 0; j < K; ++j) {
      const int kj = __shfl_sync(0xffffffffu, key, j);
      pos += (kj < key) || (kj == key && j < lane);
    }
    if (lane < K) {
      a.local.sorted_slot[token * K + pos] = lane;
      a.local.sorted_expert[token * K + pos] = valid ? id : -1;
      a.local.slot_pos[token * K + lane] = pos;
    }
  }
  // (2) stable ordinal of every route among this rank's routes to the same expert (route order), 1024
  //     routes at a time; `running` ends as the per-expert counts
  for (int e = threadIdx.x; e < E; e += blockDim.x) running[e] = 0;
  __syncthreads();
  for (int base = 0; base < n; base += 1024) {
    for (int k = threadIdx.x; k < 16 * E; k += blockDim.x) reinterpret_cast<int*>(warp_cnt)[k] = 0;
    __syncthreads();
    const int i = base + threadIdx.x;
    const int id = i < n ? a.routes[i] : -1;
    const bool valid = id >= 0 && id < E;
    const unsigned peers = __match_any_sync(0xffffffffu, valid ? id : E);
    const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
    if (valid && rank_in_warp == 0) warp_cnt[warp * E + id] = static_cast<unsigned short>(__popc(peers));
    __syncthreads();
    if (i < n) {
      int ordinal = -1;
      if (valid) {
        ordinal = running[id] + rank_in_warp;
        for (int w = 0; w < warp; ++w) ordinal += warp_cnt[w * E + id];
      }
      a.rows.local_offset[i] = ordinal;
    }
    __syncthreads();
    if (valid && rank_in_warp == 0) atomicAdd(&running[id], __popc(peers));
    __syncthreads();
  }
  // (3) counts to every rank's matrix, then the COUNTS flag
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    a.local_count[e] = running[e];
    for (int r = 0; r < world; ++r)
      if (a.count_matrix.p[r] != nullptr) a.count_matrix.p[r][rank * E + e] = running[e];
  }
  if (a.exchange) {
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < world) st_release_sys(a.flag_counts.p[threadIdx.x] + rank * kFlagStride, generation);
  }
  if (!a.global_part) return;
  // (4) every rank's counts, the global plan
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if (a.exchange && threadIdx.x < world &&
      !wait_flag_ge(a.my_flag_counts + threadIdx.x * kFlagStride, generation, a.status, a.wait_budget))
    ok = 0;
  __syncthreads();
  if (!ok) {
    publish_empty_schedule(a.tables, E / world);
  } else {
    global_plan_body(a.my_count_matrix, world, rank, E, a.row_capacity, a.tables, a.status, a.split_percent,
                     a.chunks, total, padded, pair_first, &overflow);
  }
  __syncthreads();
  // (5) destination rows and the words the owners need; nothing on a failed plan (sticky status word)
  const bool healthy = *reinterpret_cast<volatile int*>(a.status) == 0;
  const int e_local = E / world;
  if (healthy) {
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const int id = a.routes[i];
      if (id < 0 || id >= E) {
        a.rows.dst_rank[i] = a.rows.dst_row[i] = a.rows.dst_prow[i] = -1;
        continue;
      }
      const int owner = id / e_local;
      const int within = a.tables.expert_before[id] + a.rows.local_offset[i];
      const int prow = a.tables.expert_pbase[id] + within;
      a.rows.dst_rank[i] = owner;
      a.rows.dst_row[i] = a.tables.expert_base[id] + within;
      a.rows.dst_prow[i] = prow;
      if (a.meta_origin.p[owner] != nullptr && prow >= 0 && prow < a.row_capacity) {
        a.meta_origin.p[owner][prow] = rank * a.shape.cap * K + (i / K) * K + a.local.slot_pos[i];
        a.meta_prob.p[owner][prow] = a.gates[i];
      }
    }
    __syncthreads();
    if (a.want_primary) {
      for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int owner = a.rows.dst_rank[i];
        if (owner < 0) {
          if (a.per_route_primary) a.per_route_primary[i] = -1;
          continue;
        }
        const int first = (i / K) * K;
        int head = i, head_pos = a.local.slot_pos[i];
        for (int j = 0; j < K; ++j) {
          const int r = first + j;
          if (a.rows.dst_rank[r] == owner && a.local.slot_pos[r] < head_pos) {
            head = r;
            head_pos = a.local.slot_pos[r];
          }
        }
        const int prow = a.rows.dst_prow[i];
        if (a.meta_primary.p[owner] != nullptr && prow >= 0 && prow < a.row_capacity)
          a.meta_primary.p[owner][prow] = a.rows.dst_prow[head];
        if (a.per_route_primary) a.per_route_primary[i] = a.rows.dst_prow[head];
      }
    }
  }
  // (6) READY hand-shake: my words are in the owners' arenas; wait for every source's words
  if (a.exchange) {
    __threadfence_system();
    __syncthreads();
    bool arrived = true;
    if (threadIdx.x < world) {
      st_release_sys(a.flag_ready.p[threadIdx.x] + rank * kFlagStride, generation);
      arrived = wait_flag_ge(a.my_flag_ready + threadIdx.x * kFlagStride, generation, a.status, a.wait_budget);
    }
    if (threadIdx.x < 32) {
      const bool failed = __any_sync(0xffffffffu, !arrived) || *reinterpret_cast<volatile int*>(a.status) != 0;
      if (failed && a.tables.split != nullptr)
        for (int i = threadIdx.x; i < kSplitWords; i += 32) a.tables.split[i] = 0;
    }
  }
}

// ------------------------------------------------------------------ host side
static std::atomic<long long> g_flag_wait_budget{kWaitBudgetCycles};
long long flag_wait_budget() { return g_flag_wait_budget.load(std::memory_order_relaxed); }
void set_flag_wait_budget(long long cycles) {
  g_flag_wait_budget.store(cycles > 0 ? cycles : kWaitBudgetCycles, std::memory_order_relaxed);
}

int route_primary(const RouteShape& s, int tokens, const RouteLocal& local, const RouteRows& rows,
                  const PeerInts& meta_primary, int* per_route, int row_capacity, const int* status,
                  cudaStream_t stream) {
  const int n = tokens * s.top_k;
  if (n == 0) return 0;
  route_primary_kernel<<<(n + 255) / 256, 256, 0, stream>>>(local.slot_pos, rows.dst_rank, rows.dst_prow, n,
                                                           s.top_k, meta_primary, per_route, row_capacity,
                                                           status);
  count_launch();
  WM_CUDA(cudaGetLastError());
  return 0;
}

int route_plan_small(SmallPlan plan, cudaStream_t stream) {
  static const int split_percent = [] {
    const char* v = std::getenv("WM_SPLIT_PERCENT");
    const int n = v ? std::atoi(v) : 50;
    return n >= 10 && n <= 90 ? n : 50;
  }();
  plan.split_percent = split_percent;
  plan.wait_budget = flag_wait_budget();
  plan.chunks = plan.chunks < 1 ? 1 : (plan.chunks > kMaxChunks ? kMaxChunks : plan.chunks);
  const int E = plan.shape.experts;
  const size_t smem = static_cast<size_t>(E) * (3 * sizeof(int) + 32 * sizeof(unsigned short));
  static bool configured[64] = {};
  int device = 0;
  WM_CUDA(cudaGetDevice(&device));
  if (device >= 0 && device < 64 && !configured[device]) {
    WM_CUDA(cudaFuncSetAttribute(plan_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 2048 * (3 * (int)sizeof(int) + 32 * (int)sizeof(unsigned short))));
    configured[device] = true;
  }
  plan_small_kernel<<<1, 1024, smem, stream>>>(plan);
  count_launch();
  WM_CUDA(cudaGetLastError());
  return 0;
}

int route_local(const RouteShape& s, const int* routes, int tokens, RouteLocal out,
                int* chunk_hist, int* local_count, const PeerInts& count_matrix,
                cudaStream_t stream) {
  const int n = tokens * s.top_k;
  const int chunks = (n + kChunk - 1) / kChunk;
  if (tokens > 0) {
    sort_slots_kernel<<<(tokens * 32 + 255) / 256, 256, 0, stream>>>(
        routes, tokens, s.top_k, s.experts, out.sorted_slot, out.sorted_expert, out.slot_pos);
  count_launch();
    chunk_hist_kernel<<<chunks, kChunk, s.experts * sizeof(int), stream>>>(routes, n, s.experts,
                                                                           chunk_hist);
  count_launch();
  }
  chunk_scan_kernel<<<(s.experts * 32 + 255) / 256, 256, 0, stream>>>(
      chunk_hist, chunks, s.experts, local_count, count_matrix, s.world, s.rank);
  count_launch();
  WM_CUDA(cudaGetLastError());
  return 0;
}

int route_global(const RouteShape& s, const int* count_matrix, const int* flag_counts,
                 Gen generation, int row_capacity, PlanTables t, int* status, int chunks,
                 cudaStream_t stream) {
  // With two chunks: share of the owner's rows in the first one (WM_SPLIT_PERCENT, 10..90).
  static const int split_percent = [] {
    const char* v = std::getenv("WM_SPLIT_PERCENT");
    const int n = v ? std::atoi(v) : 50;
    return n >= 10 && n <= 90 ? n : 50;
  }();
  global_plan_kernel<<<1, 1024, 2 * s.experts * sizeof(int), stream>>>(
      count_matrix, flag_counts, generation, s.world, s.rank, s.experts, row_capacity, t, status, split_percent,
      chunks < 1 ? 1 : (chunks > kMaxChunks ? kMaxChunks : chunks), flag_wait_budget());
  count_launch();
  WM_CUDA(cudaGetLastError());
  return 0;
}

int route_rows(const RouteShape& s, const int* routes, const float* gates, int tokens,
               const RouteLocal& local, const int* chunk_base, PlanTables t, RouteRows out,
               const PeerInts& meta_origin, const PeerFloats& meta_prob, int row_capacity,
               const int* status, cudaStream_t stream) {
  const int n = tokens * s.top_k;
  if (n == 0) return 0;
  const int chunks = (n + kChunk - 1) / kChunk;
  const size_t smem = 32u * s.experts * sizeof(unsigned short);
  // Opt in once per device to the largest size any accepted shape needs (64 B x 2048 experts).
  static bool configured[64] = {};
  int device = 0;
  WM_CUDA(cudaGetDevice(&device));
  if (device >= 0 && device < 64 && !configured[device]) {
    WM_CUDA(cudaFuncSetAttribute(route_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 32 * 2048 * (int)sizeof(unsigned short)));
    configured[device] = true;
  }
  route_rows_kernel<<<chunks, kChunk, smem, stream>>>(
      routes, gates, local.slot_pos, n, s.top_k, s.experts, s.world, s.rank, s.cap, chunk_base, t,
      out.local_offset, out.dst_rank, out.dst_row, out.dst_prow, meta_origin, meta_prob, row_capacity,
      status);
  count_launch();
  WM_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace wm
