// TEST INFRASTRUCTURE ONLY.  C-callable driver around the reference's own host route planner
// (src/metadata/notify_dispatch.cpp, entered through build_notify_dispatch_for_testing,
// src/metadata/testing_api.hpp:25-28).  It is compiled against the reference sources where they
// lie (see oracle/Makefile); no reference source is copied.  Used to pin oracle/route_oracle.c
// and to generate tests/golden/route_*.json.
#include <cstdint>
#include <cstring>
#include <exception>
#include <string>
#include <vector>

#include "metadata/testing_api.hpp"

namespace {
thread_local std::string g_error;
}

extern "C" __attribute__((visibility("default"))) const char* ref_route_error() {
  return g_error.c_str();
}

// Experts are sharded contiguously (expert e on rank e / (experts / world)), one node.
// Outputs for `calling_rank` (all preallocated by the caller):
//   source_expert_count [world * experts]   local_offset/route_dst_row/route_dst_rank/combine_order
//   [tokens(calling_rank) * top_k]          expert_row_count/expert_row_prefix [experts / world]
extern "C" __attribute__((visibility("default"))) int ref_route_plan(
    uint32_t world, uint32_t experts, uint32_t top_k, uint32_t m_tile_rows,
    const uint64_t* tokens_per_rank, const int32_t* routes_concat, uint32_t calling_rank,
    uint64_t* source_expert_count, uint64_t* local_offset, uint64_t* route_dst_row,
    uint32_t* route_dst_rank, uint32_t* combine_order, uint64_t* expert_row_count,
    uint64_t* expert_row_prefix) {
  try {
    weftmoe::RuntimeConfig config;
    config.num_experts = experts;
    config.top_k = top_k;
    config.m_tile_rows = m_tile_rows;
    config.topology.num_nodes = 1;
    config.topology.world_size = world;
    for (uint32_t r = 0; r < world; ++r) {
      config.topology.rank_to_node.push_back(0);
      config.topology.rank_to_local_rank.push_back(r);
    }
    const uint32_t per_rank = experts / world;
    for (uint32_t e = 0; e < experts; ++e) config.topology.expert_to_rank.push_back(e / per_rank);
    std::vector<weftmoe::RankRoutingInput> inputs(world);
    size_t cursor = 0;
    for (uint32_t r = 0; r < world; ++r) {
      inputs[r].num_tokens = tokens_per_rank[r];
      const size_t n = static_cast<size_t>(tokens_per_rank[r]) * top_k;
      inputs[r].selected_experts.assign(routes_concat + cursor, routes_concat + cursor + n);
      cursor += n;
    }
    auto handles = weftmoe::build_notify_dispatch_for_testing(config, inputs);
    const auto& md = handles.at(calling_rank).metadata();
    for (uint32_t s = 0; s < world; ++s)
      for (uint32_t e = 0; e < experts; ++e)
        source_expert_count[static_cast<size_t>(s) * experts + e] = md.source_expert_count[s][e];
    const auto& out = md.outgoing;
    for (size_t i = 0; i < out.expert_id.size(); ++i) {
      local_offset[i] = out.local_offset[i];
      route_dst_row[i] = out.route_dst_row[i];
      route_dst_rank[i] = out.route_dst_rank[i];
      combine_order[i] = out.combine_order[i];
    }
    for (size_t i = 0; i < md.incoming.expert_row_count.size(); ++i) {
      expert_row_count[i] = md.incoming.expert_row_count[i];
      expert_row_prefix[i] = md.incoming.expert_row_prefix[i];
    }
    return 0;
  } catch (const std::exception& e) {
    g_error = e.what();
    return 1;
  }
}
