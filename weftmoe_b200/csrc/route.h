// Internal structs shared by the route-planning and transport kernels and the host runtime.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace wm {

constexpr int kMaxWorld = 8;
constexpr int kFlagStride = 32;  // ints between two flags: one 128-byte line each

struct PeerInts { int* p[kMaxWorld]; };
struct PeerFloats { float* p[kMaxWorld]; };
struct PeerRows { __nv_bfloat16* p[kMaxWorld]; };
struct PeerConstRows { const __nv_bfloat16* p[kMaxWorld]; };

// A generation number that kernels read on the device: *dev + delta (dev == nullptr: just delta).
// The runtime bumps *dev with a one-thread kernel at the start of every multi-rank call, so a call
// captured in a CUDA graph advances the generation at every replay.
struct Gen {
  const int* dev = nullptr;
  int delta = 0;
  Gen operator-(int d) const { return Gen{dev, delta - d}; }
#ifdef __CUDACC__
  __device__ __forceinline__ int value() const { return (dev ? *dev : 0) + delta; }
#endif
};

struct RouteShape {
  int experts, top_k, world, rank, cap;  // cap = token capacity per rank
};

// Source-side, per token: [tokens * top_k] each.
struct RouteLocal {
  int* sorted_slot;    // original slot at combine position j
  int* sorted_expert;  // expert id at combine position j, -1 when the route is invalid
  int* slot_pos;       // combine position of original slot s
};
struct RouteRows {
  int* local_offset;  // ordinal among this rank's routes to the same expert, -1 invalid
  int* dst_rank;      // owner rank
  int* dst_row;       // canonical (unpadded) row inside the owner
  int* dst_prow;      // physical row inside the owner's 128-padded layout
};

// Global tables (identical on every rank) and this rank's owner-side schedule.
struct PlanTables {
  int* expert_total;   // [experts] rows routed to the expert over all ranks
  int* expert_before;  // [experts] rows routed to it by lower ranks than this one
  int* expert_base;    // [experts] unpadded first row inside its owner
  int* expert_pbase;   // [experts] padded first row inside its owner
  int* padded_start;   // [experts/world + 1] padded first row of each local expert
  int* tile_group;     // [row_capacity / 128] local expert of each 128-row tile
  int* num_tiles;      // scalar
  int* padded_rows;    // scalar
  int* pair_tiles;     // [2 * pairs] two 128-row tiles of one expert per CTA pair, -1 = none
  int* num_pairs;      // scalar
  // Optional [kSplitWords]: the owner's work cut at expert boundaries into up to kMaxChunks chunks, so
  // that a later chunk's transfers overlap an earlier chunk's compute.  Four rows of kMaxChunks + 1
  // boundaries (tiles, CTA pairs, padded rows, local experts): chunk c is [b[c], b[c + 1]); b[0] = 0 and
  // every boundary from the chunk count on equals the total, so unused chunks are empty.
  int* split;
  // Optional [experts/world]: unpadded rows of each local expert of this rank (the K-grouped weight
  // gradients stop their reduction at the last 64-row block that holds a live row).
  int* live_rows;
  // Optional [experts/world]: this rank's local experts, chunk by chunk, inside a chunk in descending order
  // of their rows (ties by index).  The K-grouped weight gradients walk their tiles in this order, so that
  // the round-robin deal of tiles to CTAs gives every CTA nearly the same amount of reduction work.
  int* group_order;
};

constexpr int kMaxChunks = 8;
constexpr int kSplitStride = kMaxChunks + 1;
constexpr int kSplitWords = 4 * kSplitStride;

// A [begin, end) range held in device memory (two pointers into PlanTables::split).
struct DeviceRange {
  const int* begin;
  const int* end;
};
constexpr int kWhole = -1;  // "chunk" argument: all of the owner's work
inline DeviceRange split_range(const int* split, int what /*0 tiles, 1 pairs, 2 rows, 3 experts*/, int chunk) {
  const int* b = split + what * kSplitStride;
  return chunk < 0 ? DeviceRange{b, b + kMaxChunks} : DeviceRange{b + chunk, b + chunk + 1};
}
// Host-side image of a split that has one chunk holding everything.
inline void fill_whole_split(int* words, int tiles, int pairs, int rows, int experts) {
  const int totals[4] = {tiles, pairs, rows, experts};
  for (int what = 0; what < 4; ++what) {
    words[what * kSplitStride] = 0;
    for (int c = 1; c <= kMaxChunks; ++c) words[what * kSplitStride + c] = totals[what];
  }
}

// The whole plan of a small call (at most kSmallPlanRoutes routes) in one launch: what route_local,
// route_global, route_rows and route_primary compute, plus (exchange != 0) the COUNTS and READY flag
// hand-shakes that surround them at world > 1.
constexpr int kSmallPlanRoutes = 4096;
struct SmallPlan {
  RouteShape shape;
  const int* routes;
  const float* gates;         // nullable when no owner words are pushed
  int tokens;
  RouteLocal local;
  RouteRows rows;
  PlanTables tables;
  int* local_count;           // [experts]
  PeerInts count_matrix;      // every rank's count matrix (row `rank` is written); null entries are skipped
  const int* my_count_matrix; // this rank's matrix [world][experts]
  PeerInts meta_origin;       // null entries: nothing is pushed to that owner
  PeerFloats meta_prob;
  PeerInts meta_primary;
  int* per_route_primary;     // nullable
  int want_primary;           // compute the per-owner primary rows
  int global_part;            // 0: stop after the counts (phase 0 of the stand-alone planner)
  int exchange;               // world > 1 inside a runtime: signal / wait the COUNTS and READY flags
  PeerInts flag_counts;       // COUNTS flag group of every rank
  const int* my_flag_counts;
  PeerInts flag_ready;        // READY flag group of every rank
  const int* my_flag_ready;
  Gen generation;
  int row_capacity;
  int* status;
  int chunks;
  int split_percent;          // filled by route_plan_small
  long long wait_budget;      // filled by route_plan_small
};
int route_plan_small(SmallPlan plan, cudaStream_t stream);

int route_local(const RouteShape& s, const int* routes, int tokens, RouteLocal out,
                int* chunk_hist, int* local_count, const PeerInts& count_matrix,
                cudaStream_t stream);
// `chunks` (1..kMaxChunks): how many chunks PlanTables::split cuts the owner's rows into.
int route_global(const RouteShape& s, const int* count_matrix, const int* flag_counts,
                 Gen generation, int row_capacity, PlanTables t, int* status, int chunks,
                 cudaStream_t stream);
// `status` (nullable): when the status word is already non-zero (the plan failed) nothing is written.
// Words for rows at or beyond `row_capacity` are never pushed to an owner.
int route_rows(const RouteShape& s, const int* routes, const float* gates, int tokens,
               const RouteLocal& local, const int* chunk_base, PlanTables t, RouteRows out,
               const PeerInts& meta_origin, const PeerFloats& meta_prob, int row_capacity,
               const int* status, cudaStream_t stream);

// Cycle budget of the cross-rank flag waits (default: kWaitBudgetCycles, about 2 s).  Process-wide;
// tests shorten it through wm_debug_set_wait_budget to make a wait run out quickly.
long long flag_wait_budget();
void set_flag_wait_budget(long long cycles);

// Source side, world > 1: a token routed to several experts of ONE owner rank crosses NVLink once.
// For every route, meta_primary[owner][row] = the owner row of the token's first route (lowest
// combine position) to that owner; rows whose value is their own index are pulled, the others are
// copied from that row inside the owner.
// `per_route` (nullable) also receives that row per route, in route order (-1 = no route); entries of
// meta_primary may be null (nothing is sent to that owner).
int route_primary(const RouteShape& s, int tokens, const RouteLocal& local, const RouteRows& rows,
                  const PeerInts& meta_primary, int* per_route, int row_capacity, const int* status,
                  cudaStream_t stream);

// ------------------------------------------------------------------ transport (transport.cu)
struct OwnerRows {
  const int* padded_start;  // [e_local + 1]
  const int* tile_group;    // [tiles]
  DeviceRange rows;         // padded rows to process
  const int* expert_total;  // [experts] (global ids)
};

// Wait until flags[r] >= generation for r < world (bounded); flags are kFlagStride apart.
// When a wait runs out the status word is set and, if `split_on_fail` is given, the eight words of the
// owner schedule's split are zeroed, so that every later owner-side kernel of the call finds an empty
// range and touches no row whose indices might not have arrived.
int wait_flags(const int* flags, int world, Gen generation, int* status, int* split_on_fail,
               cudaStream_t stream);
// Store `generation` into flag slot `slot` of every rank's flag group (peer-mapped).
int signal_peers(const PeerInts& flag_group, int world, int slot, Gen generation,
                 cudaStream_t stream);

// The row-copy kernels take their CTA count: 8 CTAs of 8 warps per SM when they run alone (enough
// loads in flight for HBM), 2 per SM when a half is copied beside a grouped GEMM (thread slots
// must stay free for the GEMM's CTA; NVLink needs far fewer loads in flight than HBM).
// Owner side, forward: pull every live row's activation from its source rank's staging buffer,
// copy origin/prob words from the meta mailbox to local arrays, zero the padding rows.
// meta_primary (nullable = every row is pulled) names the row a duplicate is copied from;
// primary_out (nullable) keeps it for the backward pass.  Call copy_duplicate_rows afterwards.
int gather_rows(const OwnerRows& o, int rank, int e_local, int world, int row_capacity, int cap, int top_k,
                int hidden,
                const PeerConstRows& stage, const int* meta_origin, const float* meta_prob,
                const int* meta_primary, __nv_bfloat16* rows_out, int* origin_out, float* prob_out,
                int* primary_out, int ctas, cudaStream_t stream);
// Owner side, backward: pull dY rows by the saved origins (only rows with primary[r] == r when
// `primary` is given).
int gather_by_origin(DeviceRange rows, const int* origin, const int* primary, int world, int cap, int top_k,
                     int hidden, const PeerConstRows& stage, __nv_bfloat16* rows_out, int ctas,
                     cudaStream_t stream);
// Owner side: rows_out[r] = rows_out[primary[r]] for the rows of the range with primary[r] != r.
int copy_duplicate_rows(DeviceRange rows, const int* primary, int hidden, __nv_bfloat16* rows_out,
                        int ctas, cudaStream_t stream);
// Source side: out[t] = bf16( sum over combine positions j with a live route of mailbox[j][t] ).
int combine_rows(const __nv_bfloat16* mailbox, const int* sorted_expert, int tokens, int cap,
                 int top_k, int hidden, __nv_bfloat16* out, cudaStream_t stream);
// Source side, backward: dgates[t, original slot] = dgate_box[t*K + j] for live positions, else 0.
int unpermute_dgates(const float* dgate_box, const int* sorted_slot, const int* sorted_expert,
                     int tokens, int top_k, float* dgates, cudaStream_t stream);
// Owner side, backward elementwise: from saved gate/up (ab), dU and prob compute
// U = bf16(silu(a) b p), dAB, and the per-row dprob, which is sent to the source's dgate box.
// Finish of the fused dU + SwiGLU-backward epilogue: sum the per-block dprob partials of each row in
// block order and send them to the sources' dprob boxes.
int dprob_finish(DeviceRange rows, const float* part, int blocks, int row_capacity, const int* origin, int cap,
                 int top_k, const PeerFloats& dgate_box, cudaStream_t stream);
int swiglu_backward(DeviceRange rows, const __nv_bfloat16* ab, const __nv_bfloat16* du,
                    const float* prob, const int* origin, int inter, int cap, int top_k,
                    __nv_bfloat16* u, __nv_bfloat16* dab, const PeerFloats& dgate_box, int sms,
                    cudaStream_t stream);

}  // namespace wm
