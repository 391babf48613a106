/* TEST INFRASTRUCTURE ONLY — CPU restatement of the route planning ("notify") stage.
 * Never linked into, imported by or executed from the product path; only tests/,
 * __graft_entry__.smoke() and bench.py's CPU-baseline leg may use it.
 *
 * What it restates (reference file:line):
 *   - combine order = stable sort of a token's slots by expert id, invalid ids last
 *     (weftmoe/blackwell.py:10-13 `_sorted_route_keys`; src/metadata/notify_dispatch.cpp:936-948)
 *   - per-source local offset = running count per expert in token-major, slot order
 *     (src/metadata/notify_dispatch.cpp:870-880; weftmoe/blackwell_backward.py:29-37)
 *   - canonical destination row = expert_base[e] + sum_{s<rank} count[s][e] + local_offset
 *     (src/metadata/notify_dispatch.cpp:835-906)
 *   - expert e lives on rank e / (E / EP) (src/python/runtime.cpp:175-176)
 *   - owner-side padded layout: each local expert's rows rounded up to 128
 *     (weftmoe/blackwell_backward.py:41-44; an idle expert gets no rows here)
 *   - origin word = src_rank*cap*K + token*K + sorted_slot, -1 on padding rows
 *     (src/cuda/blackwell/fused/impls/routed_bf16.cuh:540-541)
 * Pinned against the reference's own host planner (oracle/_ref/libref_route.so) in
 * tests/test_route_oracle.py and against tests/golden/route_cases.json.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define WM_ROW_ALIGN 128

static int valid_expert(int32_t id, int experts) { return id >= 0 && id < experts; }

/* Source-side plan for one rank.
 * routes [tokens*top_k]; outputs all [tokens*top_k] except local_count [experts].
 *   sorted_slot[t*K + j]   original slot at combine position j
 *   sorted_expert[t*K + j] expert id at combine position j, -1 when invalid
 *   local_offset[t*K + s]  indexed by ORIGINAL slot s; -1 when invalid                      */
void wm_oracle_local_plan(int experts, int top_k, int64_t tokens, const int32_t* routes,
                          int32_t* sorted_slot, int32_t* sorted_expert, int32_t* local_offset,
                          int32_t* local_count) {
  memset(local_count, 0, sizeof(int32_t) * (size_t)experts);
  for (int64_t t = 0; t < tokens; ++t) {
    const int32_t* r = routes + t * top_k;
    int32_t* ss = sorted_slot + t * top_k;
    for (int s = 0; s < top_k; ++s) ss[s] = s;
    /* insertion sort == stable sort; key = (valid ? id : experts) */
    for (int i = 1; i < top_k; ++i) {
      int32_t slot = ss[i];
      int32_t key = valid_expert(r[slot], experts) ? r[slot] : experts;
      int j = i - 1;
      while (j >= 0) {
        int32_t kj = valid_expert(r[ss[j]], experts) ? r[ss[j]] : experts;
        if (kj <= key) break;
        ss[j + 1] = ss[j];
        --j;
      }
      ss[j + 1] = slot;
    }
    for (int j = 0; j < top_k; ++j)
      sorted_expert[t * top_k + j] = valid_expert(r[ss[j]], experts) ? r[ss[j]] : -1;
    for (int s = 0; s < top_k; ++s) {
      if (valid_expert(r[s], experts)) local_offset[t * top_k + s] = local_count[r[s]]++;
      else local_offset[t * top_k + s] = -1;
    }
  }
}

/* Global plan from the count matrix [world][experts] (int32).
 * Per expert (global id): total rows, unpadded base inside its owner, padded base inside its owner.
 * Per owner rank: padded_rows[world] (sum of padded extents).                                  */
void wm_oracle_global_plan(int world, int experts, const int32_t* count_matrix, int32_t* expert_total,
                           int32_t* expert_base, int32_t* expert_pbase, int32_t* padded_rows) {
  const int per_rank = experts / world;
  for (int owner = 0; owner < world; ++owner) {
    int32_t base = 0, pbase = 0;
    for (int l = 0; l < per_rank; ++l) {
      const int e = owner * per_rank + l;
      int32_t total = 0;
      for (int s = 0; s < world; ++s) total += count_matrix[s * experts + e];
      expert_total[e] = total;
      expert_base[e] = base;
      expert_pbase[e] = pbase;
      base += total;
      pbase += (total + WM_ROW_ALIGN - 1) / WM_ROW_ALIGN * WM_ROW_ALIGN;
    }
    padded_rows[owner] = pbase;
  }
}

/* Destination of every route of `rank` (indexed by ORIGINAL slot): owner rank, canonical row
 * (unpadded) and physical row (padded layout); -1 for invalid routes.                         */
void wm_oracle_route_rows(int world, int experts, int top_k, int rank, int64_t tokens,
                          const int32_t* routes, const int32_t* local_offset,
                          const int32_t* count_matrix, const int32_t* expert_base,
                          const int32_t* expert_pbase, int32_t* dst_rank, int32_t* dst_row,
                          int32_t* dst_prow) {
  const int per_rank = experts / world;
  for (int64_t i = 0; i < tokens * top_k; ++i) {
    const int32_t e = routes[i];
    if (!valid_expert(e, experts)) {
      dst_rank[i] = dst_row[i] = dst_prow[i] = -1;
      continue;
    }
    int32_t before = 0;
    for (int s = 0; s < rank; ++s) before += count_matrix[s * experts + e];
    dst_rank[i] = e / per_rank;
    dst_row[i] = expert_base[e] + before + local_offset[i];
    dst_prow[i] = expert_pbase[e] + before + local_offset[i];
  }
}

/* Which row of the owner holds the only copy of the token's activation that crosses NVLink: a token
 * routed to several experts of ONE owner rank is pulled once, into the row of its first such route in
 * combine order (stable sort of the token's slots by expert id, src/cuda/weftmoe_pf/route_plan.cuh:29-50),
 * and the token's other rows in that owner are copies of it.  dst_primary[i] = dst_prow of that first
 * route (so dst_primary[i] == dst_prow[i] marks the pulled rows); -1 for invalid routes.  This is this
 * build's transport choice; the reference pulls every routed row (routed_bf16.cuh:378-557), so the
 * function is pinned by its definition only (hand-made cases in tests/test_oracle_route.py).        */
void wm_oracle_route_primary(int experts, int top_k, int64_t tokens, const int32_t* routes,
                             const int32_t* dst_rank, const int32_t* dst_prow, int32_t* dst_primary) {
  for (int64_t t = 0; t < tokens; ++t) {
    const int32_t* r = routes + t * top_k;
    for (int s = 0; s < top_k; ++s) {
      const int64_t i = t * top_k + s;
      if (!valid_expert(r[s], experts)) {
        dst_primary[i] = -1;
        continue;
      }
      int head = s;
      for (int o = 0; o < top_k; ++o) {
        if (!valid_expert(r[o], experts) || dst_rank[t * top_k + o] != dst_rank[i]) continue;
        /* earlier in the stable sort by expert id: smaller id, or equal id and smaller slot */
        if (r[o] < r[head] || (r[o] == r[head] && o < head)) head = o;
      }
      dst_primary[i] = dst_prow[t * top_k + head];
    }
  }
}

/* Owner-side tables of `owner`: padded row start of every local expert [per_rank+1], the expert of
 * every 128-row tile, and the number of tiles.  Returns the number of tiles.                   */
int wm_oracle_owner_tiles(int world, int experts, int owner, const int32_t* expert_total,
                          int32_t* padded_start, int32_t* tile_group) {
  const int per_rank = experts / world;
  int tiles = 0;
  padded_start[0] = 0;
  for (int l = 0; l < per_rank; ++l) {
    const int32_t total = expert_total[owner * per_rank + l];
    const int32_t padded = (total + WM_ROW_ALIGN - 1) / WM_ROW_ALIGN * WM_ROW_ALIGN;
    padded_start[l + 1] = padded_start[l] + padded;
    for (int t = 0; t < padded / WM_ROW_ALIGN; ++t) tile_group[tiles++] = l;
  }
  return tiles;
}
