// Host runtime behind the C ABI: arena/scratch layout, CUDA-IPC peer mapping, and the launch
// sequences of forward and backward.  One process per GPU; every call enqueues on the caller's
// stream and never synchronises (except the explicit status poll).
//
// Cross-rank protocol (world > 1).  Every collective operation (a forward or a backward) takes
// the next generation number g, identical on all ranks because all ranks call in the same order.
// Four flag groups live in each rank's arena, one 128-byte line per peer, holding the latest
// generation for which the event happened; flags only grow and are never reset:
//   COUNTS [s]  source s stored its per-expert counts into my count matrix
//   READY  [s]  source s staged its activations and pushed origin/prob words for my rows
//   PULLED [o]  owner o finished reading my staging buffer and meta words
//   CONTRIB[o]  owner o finished writing its results into my mailbox
// A source overwrites its staging buffer only after PULLED >= g-1 from every owner; an owner
// writes a mailbox only after READY >= g, which the source sends after its previous combine.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

#include "../../include/weftmoe_b200.h"
#include "kernels.h"
#include "quant_path.h"
#include "route.h"

using namespace wm;

namespace {

enum FlagGroup { kCounts = 0, kReady = 1, kPulled = 2, kContrib = 3, kFlagGroups = 4 };

// Stages timed when wm_runtime_enable_timing is on: one CUDA event pair per stage and call.
enum Stage {
  kStagePlan = 0, kStageGather, kStageFc1, kStageFc2, kStageCombine,
  kStageGatherDy, kStageDu, kStageSwigluBwd, kStageDx, kStageDw1, kStageDw2, kStageCombineDx,
  // later chunks (world > 1 only; chunks after the first are pulled on the side stream)
  kStageFc1B, kStageFc2B, kStageDuB, kStageSwigluBwdB, kStageDxB, kStageGatherB, kStageGatherDyB,
  // waits and staging copies around the kernels (they absorb the skew between ranks)
  kStageStageIn, kStageSyncReady, kStageSyncContrib, kStageStageInBwd, kStageSyncReadyBwd, kStageSyncContribBwd,
  kStageCount
};
const char* const kStageNames[kStageCount] = {
    "route_plan", "gather_rows", "fc1_swiglu", "fc2_push", "combine",
    "gather_dy", "dgrad_du", "swiglu_backward", "dgrad_dx_push", "wgrad_dw1", "wgrad_dw2",
    "combine_dx", "fc1_swiglu_b", "fc2_push_b", "dgrad_du_b", "swiglu_backward_b", "dgrad_dx_push_b",
    "gather_rows_b", "gather_dy_b", "stage_in", "sync_ready", "sync_contrib", "stage_in_bwd", "sync_ready_bwd",
    "sync_contrib_bwd"};
constexpr int kTimingRing = 32;
// One event pair per (stage, chunk) and call; created at first use.
struct TimingSlot {
  cudaEvent_t start[kStageCount][kMaxChunks] = {};
  cudaEvent_t stop[kStageCount][kMaxChunks] = {};
  bool used[kStageCount][kMaxChunks] = {};
};

constexpr size_t kAlign = 256;
size_t align_up(size_t v, size_t a = kAlign) { return (v + a - 1) / a * a; }

struct Carver {
  size_t cursor = 0;
  size_t take(size_t bytes) {
    const size_t at = cursor;
    cursor = align_up(cursor + bytes);
    return at;
  }
};

struct ArenaLayout {
  size_t flags, counts, stage, meta_origin, meta_prob, meta_primary, mailbox, dgate_box, total;
};
struct ScratchLayout {
  size_t status, sorted_slot, sorted_expert, slot_pos, local_offset, dst_rank, dst_row, dst_prow,
      chunk_hist, local_count, expert_total, expert_before, expert_base, expert_pbase, padded_start,
      tile_group, num_tiles, padded_rows, pair_tiles, num_pairs, split, origin, prob, xrows, u, recv, du,
      dab, abq, sfa_x, sfa_u, primary, wq_a, wq_b, wsf_a, wsf_b, dprob_part, gen, total;
};
// Training cache carved out of the caller's tape buffer.
struct TapeLayout {
  size_t sorted_slot, sorted_expert, padded_start, live_rows, group_order, tile_group, num_tiles, padded_rows, pair_tiles,
      num_pairs, split, origin, prob, primary, xrows, ab, total;
};

}  // namespace

struct wm_runtime {
  wm_config cfg;
  int e_local = 0, row_cap = 0, sms = 0, device = 0, generation = 0;
  ArenaLayout al{};
  ScratchLayout sl{};
  TapeLayout tl{};
  uint8_t* arena = nullptr;
  uint8_t* scratch = nullptr;
  uint8_t* peer[kMaxWorld] = {};
  bool peers_ready = false;
  // world > 1: the second half of the owner's rows is pulled on a side stream while the first
  // half is being computed (inbound NVLink beside compute and outbound pushes).
  cudaStream_t side = nullptr;
  int chunks = 1;                              // chunks the owner's rows are pipelined in (1 at world 1)
  cudaEvent_t ev_pulled[kMaxChunks] = {};      // chunk c's rows are in this rank's row buffer
  // Optional (WM_PUSH_SMS = n > 0, world > 1): the first half's push GEMM (FC2 / dX, bound by NVLink)
  // runs on n SMs of a third stream beside the second half's compute-bound kernels on the other SMs.
  cudaStream_t push_stream = nullptr;
  cudaEvent_t ev_ready[kMaxChunks] = {};       // chunk c's push GEMM may start (its input is complete)
  cudaEvent_t ev_pushed = nullptr;             // the latest push GEMM issued on push_stream has finished
  int push_sms = 0, push_sms_bwd = 0;
  // Optional per-stage device timing (CUDA events on the caller's stream).
  bool timing = false;
  int timing_slot = 0;
  cudaEvent_t ev_trace_origin = nullptr;  // recorded at the first timed call
  std::vector<TimingSlot> slots;
  double stage_ms[kStageCount] = {};
  long long stage_calls[kStageCount] = {};
};

namespace {

template <class T>
T* at(uint8_t* base, size_t off) { return reinterpret_cast<T*>(base + off); }

ArenaLayout arena_layout(const wm_config& c, int row_cap) {
  Carver k;
  ArenaLayout a{};
  a.flags = k.take(sizeof(int) * kFlagGroups * kMaxWorld * kFlagStride);
  a.counts = k.take(sizeof(int) * c.world * c.experts);
  a.stage = k.take(2ull * c.max_tokens * c.hidden);
  a.meta_origin = k.take(sizeof(int) * row_cap);
  a.meta_prob = k.take(sizeof(float) * row_cap);
  a.meta_primary = k.take(sizeof(int) * row_cap);
  a.mailbox = k.take(2ull * c.top_k * c.max_tokens * c.hidden);
  a.dgate_box = k.take(sizeof(float) * c.max_tokens * c.top_k);
  a.total = align_up(k.cursor, 1 << 16);  // 64 KiB multiple keeps large-page peer mappings
  return a;
}

ScratchLayout scratch_layout(const wm_config& c, int row_cap) {
  Carver k;
  ScratchLayout s{};
  const size_t routes = static_cast<size_t>(c.max_tokens) * c.top_k;
  const size_t chunks = (routes + 1023) / 1024 + 1;
  const int e_local = c.experts / c.world;
  s.status = k.take(sizeof(int) * 4);
  s.gen = k.take(sizeof(int));  // device copy of the call generation (bumped by a kernel per call)
  s.sorted_slot = k.take(sizeof(int) * routes);
  s.sorted_expert = k.take(sizeof(int) * routes);
  s.slot_pos = k.take(sizeof(int) * routes);
  s.local_offset = k.take(sizeof(int) * routes);
  s.dst_rank = k.take(sizeof(int) * routes);
  s.dst_row = k.take(sizeof(int) * routes);
  s.dst_prow = k.take(sizeof(int) * routes);
  s.chunk_hist = k.take(sizeof(int) * chunks * c.experts);
  s.local_count = k.take(sizeof(int) * c.experts);
  s.expert_total = k.take(sizeof(int) * c.experts);
  s.expert_before = k.take(sizeof(int) * c.experts);
  s.expert_base = k.take(sizeof(int) * c.experts);
  s.expert_pbase = k.take(sizeof(int) * c.experts);
  s.padded_start = k.take(sizeof(int) * (e_local + 1));
  s.tile_group = k.take(sizeof(int) * (row_cap / 128 + 1));
  s.num_tiles = k.take(sizeof(int));
  s.padded_rows = k.take(sizeof(int));
  s.pair_tiles = k.take(sizeof(int) * 2 * (row_cap / 128 + 1));
  s.num_pairs = k.take(sizeof(int));
  s.split = k.take(sizeof(int) * kSplitWords);
  s.origin = k.take(sizeof(int) * row_cap);
  s.prob = k.take(sizeof(float) * row_cap);
  s.primary = k.take(sizeof(int) * row_cap);
  s.xrows = k.take(2ull * row_cap * c.hidden);
  s.u = k.take(2ull * row_cap * c.intermediate);
  if (c.reserved != 0) {  // quantised precisions: BF16 gate/up rows and scale-factor chunks
    const size_t tiles = row_cap / 128;
    s.abq = k.take(4ull * row_cap * c.intermediate);
    s.sfa_x = k.take(tiles * (c.hidden / 64) * 512);
    // U chunks in the forward pass; the backward pass keeps the chunks of dAB (2I wide) here
    s.sfa_u = k.take(tiles * (c.intermediate / 64) * 512 * (c.training ? 2 : 1));
  }
  if (c.training) {
    s.recv = k.take(2ull * row_cap * c.hidden);
    s.du = k.take(2ull * row_cap * c.intermediate);
    s.dab = k.take(4ull * row_cap * c.intermediate);
    s.dprob_part = k.take(sizeof(float) * row_cap * ((c.intermediate + 127) / 128));
  }
  if (c.training && c.reserved == 1) {
    // FP8 weight gradients: both operands of each contraction, re-quantised along the rows and stored
    // transposed ([features][row_cap] bytes), plus their scale chunks (+4 chunks of slack).
    const size_t wide = c.hidden > 2 * c.intermediate ? c.hidden : 2 * c.intermediate;
    s.wq_a = k.take(static_cast<size_t>(row_cap) * wide);
    s.wq_b = k.take(static_cast<size_t>(row_cap) * c.hidden);
    s.wsf_a = k.take((wide / 128) * (row_cap / 128) * 512 + 4 * 512);
    s.wsf_b = k.take((static_cast<size_t>(c.hidden) / 128) * (row_cap / 128) * 512 + 4 * 512);
  }
  if (c.training && c.reserved == 2) {
    // NVFP4 weight gradients: both operands of the contraction quantised block-16 along the rows and
    // stored transposed ([features][row_cap / 2] bytes) with their scale chunks.
    const size_t wide = c.hidden > 2 * c.intermediate ? c.hidden : 2 * c.intermediate;
    s.wq_a = k.take(static_cast<size_t>(row_cap) / 2 * wide);
    s.wq_b = k.take(static_cast<size_t>(row_cap) / 2 * wide);
    s.wsf_a = k.take((wide / 128) * (row_cap / 64) * 512 + 4 * 512);
    s.wsf_b = k.take((wide / 128) * (row_cap / 64) * 512 + 4 * 512);
  }
  s.total = k.cursor;
  return s;
}

TapeLayout tape_layout(const wm_config& c, int row_cap) {
  Carver k;
  TapeLayout t{};
  const size_t routes = static_cast<size_t>(c.max_tokens) * c.top_k;
  const int e_local = c.experts / c.world;
  t.sorted_slot = k.take(sizeof(int) * routes);
  t.sorted_expert = k.take(sizeof(int) * routes);
  t.padded_start = k.take(sizeof(int) * (e_local + 1));
  t.live_rows = k.take(sizeof(int) * e_local);
  t.group_order = k.take(sizeof(int) * e_local);
  t.tile_group = k.take(sizeof(int) * (row_cap / 128 + 1));
  t.num_tiles = k.take(sizeof(int));
  t.padded_rows = k.take(sizeof(int));
  t.pair_tiles = k.take(sizeof(int) * 2 * (row_cap / 128 + 1));
  t.num_pairs = k.take(sizeof(int));
  t.split = k.take(sizeof(int) * kSplitWords);
  t.origin = k.take(sizeof(int) * row_cap);
  t.prob = k.take(sizeof(float) * row_cap);
  t.primary = k.take(sizeof(int) * row_cap);
  t.xrows = k.take(2ull * row_cap * c.hidden);
  t.ab = k.take(4ull * row_cap * c.intermediate);
  t.total = k.cursor;
  return t;
}

int check_config(const wm_config& c) {
  if (c.world != 1 && c.world != 2 && c.world != 4 && c.world != 8) {
    set_error("world must be 1, 2, 4 or 8 (got %d)", c.world);
    return WM_ERR_INVALID;
  }
  if (c.rank < 0 || c.rank >= c.world) {
    set_error("rank %d outside world %d", c.rank, c.world);
    return WM_ERR_INVALID;
  }
  // Shape limits follow weftmoe/runtime.py:113-118.
  if (c.experts <= 0 || c.experts % c.world || c.experts / c.world > 512 || c.experts > 2048 ||
      c.top_k < 1 || c.top_k > 32 || c.top_k > c.experts || c.hidden < 256 || c.hidden % 256 ||
      c.intermediate < 128 || c.intermediate > 4096 || c.intermediate % 128 || c.max_tokens < 0 ||
      c.max_rows < 0) {
    set_error("Unsupported expert shape or token capacity (E=%d K=%d H=%d I=%d T=%d rows=%d)",
              c.experts, c.top_k, c.hidden, c.intermediate, c.max_tokens, c.max_rows);
    return WM_ERR_INVALID;
  }
  if (c.reserved < 0 || c.reserved > 2 || (c.reserved == 2 && c.intermediate % 256)) {
    set_error("precision must be 0 (BF16), 1 (blockwise FP8) or 2 (NVFP4; needs intermediate %% 256 == 0)");
    return WM_ERR_INVALID;
  }
  const long long origin_span = 1ll * c.world * (c.max_tokens > 0 ? c.max_tokens : 1) * c.top_k;
  if (origin_span >= (1ll << 31)) {
    set_error("world * max_tokens * top_k must fit in 31 bits");
    return WM_ERR_INVALID;
  }
  return WM_OK;
}

PeerInts flag_group(const wm_runtime* rt, int group) {
  PeerInts p{};
  for (int r = 0; r < rt->cfg.world; ++r)
    p.p[r] = at<int>(rt->peer[r], rt->al.flags) + group * kMaxWorld * kFlagStride;
  return p;
}
const int* my_flags(const wm_runtime* rt, int group) {
  return at<int>(rt->arena, rt->al.flags) + group * kMaxWorld * kFlagStride;
}

int map_status(int device_code) {
  switch (device_code) {
    case 0: return WM_OK;
    case kStatusRowOverflow: return WM_ERR_CAPACITY;
    case kStatusBadRoute: return WM_ERR_ROUTE;
    default: return WM_ERR_TIMEOUT;
  }
}

int check_ready(const wm_runtime* rt, const char* what) {
  if (!rt || !rt->arena) {
    set_error("%s: runtime is closed", what);
    return WM_ERR_STATE;
  }
  if (rt->cfg.world > 1 && !rt->peers_ready) {
    set_error("%s: import the peer handles first", what);
    return WM_ERR_STATE;
  }
  return WM_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Fold the finished measurements of one ring slot into the totals (waits for its events).
void harvest(wm_runtime* rt, TimingSlot& slot) {
  // WM_DEBUG_STEP_TRACE=1: print each stage's start and end relative to the first timed call.
  static const bool trace = std::getenv("WM_DEBUG_STEP_TRACE") != nullptr;
  for (int k = 0; k < kStageCount; ++k) {
    bool any = false;
    for (int c = 0; c < kMaxChunks; ++c) {
      if (!slot.used[k][c]) continue;
      float ms = 0.0f;
      if (cudaEventSynchronize(slot.stop[k][c]) == cudaSuccess &&
          cudaEventElapsedTime(&ms, slot.start[k][c], slot.stop[k][c]) == cudaSuccess) {
        rt->stage_ms[k] += ms;   // a stage that ran once per chunk reports the sum over its chunks
        any = true;
        float at = 0.0f;
        if (trace && rt->ev_trace_origin &&
            cudaEventElapsedTime(&at, rt->ev_trace_origin, slot.start[k][c]) == cudaSuccess)
          fprintf(stderr, "[trace rank %d] %-20s c%d %9.1f %9.1f us\n", rt->cfg.rank, kStageNames[k], c, at * 1e3,
                  (at + ms) * 1e3);
      }
      slot.used[k][c] = false;
    }
    if (any) rt->stage_calls[k] += 1;
  }
}
TimingSlot* begin_timing(wm_runtime* rt, cudaStream_t stream) {
  if (!rt->timing) return nullptr;
  if (!rt->ev_trace_origin && cudaEventCreate(&rt->ev_trace_origin) == cudaSuccess)
    cudaEventRecord(rt->ev_trace_origin, stream);
  TimingSlot& slot = rt->slots[rt->timing_slot];
  rt->timing_slot = (rt->timing_slot + 1) % kTimingRing;
  harvest(rt, slot);
  return &slot;
}
struct StageScope {
  TimingSlot* slot;
  int stage, chunk;
  cudaStream_t stream;
  StageScope(TimingSlot* s, int k, cudaStream_t st, int c = 0) : slot(s), stage(k), chunk(c), stream(st) {
    if (!slot) return;
    if (!slot->start[stage][chunk] && (cudaEventCreate(&slot->start[stage][chunk]) != cudaSuccess ||
                                       cudaEventCreate(&slot->stop[stage][chunk]) != cudaSuccess)) {
      slot = nullptr;
      return;
    }
    cudaEventRecord(slot->start[stage][chunk], stream);
  }
  ~StageScope() {
    if (slot) {
      cudaEventRecord(slot->stop[stage][chunk], stream);
      slot->used[stage][chunk] = true;
    }
  }
};

}  // namespace

// =============================================================================== lifecycle
extern "C" int wm_runtime_create(const wm_config* config, wm_runtime** out) {
  if (!config || !out) {
    set_error("wm_runtime_create: null argument");
    return WM_ERR_INVALID;
  }
  if (int rc = check_config(*config)) return rc;
  wm_runtime* rt = new (std::nothrow) wm_runtime();
  if (!rt) {
    set_error("out of host memory");
    return WM_ERR_CUDA;
  }
  rt->cfg = *config;
  rt->e_local = config->experts / config->world;
  const int cap_tokens = config->max_tokens > 0 ? config->max_tokens : 1;
  rt->cfg.max_tokens = cap_tokens;
  // Each local expert's rows are padded to 128: at most 127 extra rows per live expert.
  rt->row_cap = static_cast<int>(align_up(static_cast<size_t>(config->max_rows), 128)) +
                128 * rt->e_local;
  rt->al = arena_layout(rt->cfg, rt->row_cap);
  rt->sl = scratch_layout(rt->cfg, rt->row_cap);
  rt->tl = tape_layout(rt->cfg, rt->row_cap);
  auto fail = [&](int rc) {
    if (rt->arena) cudaFree(rt->arena);
    if (rt->scratch) cudaFree(rt->scratch);
    delete rt;
    return rc;
  };
  if (cudaGetDevice(&rt->device) != cudaSuccess ||
      cudaDeviceGetAttribute(&rt->sms, cudaDevAttrMultiProcessorCount, rt->device) != cudaSuccess) {
    set_error("no CUDA device is current");
    return fail(WM_ERR_CUDA);
  }
  cudaError_t e = cudaMalloc(&rt->arena, rt->al.total);
  if (e == cudaSuccess) e = cudaMalloc(&rt->scratch, rt->sl.total);
  if (e != cudaSuccess) {
    set_error("workspace allocation failed (arena %zu B, scratch %zu B): %s", rt->al.total,
              rt->sl.total, cudaGetErrorString(e));
    return fail(WM_ERR_CUDA);
  }
  // Zero what must start at zero (flags, count matrix, status) and everything an owner may read
  // before its source wrote it when a source drops out (staging rows, origin / prob / primary words:
  // zero is a valid value for each).  Done on the legacy stream and synchronised so that peers may
  // write as soon as they have imported the handle.
  e = cudaMemset(rt->arena, 0, rt->al.mailbox);
  if (e == cudaSuccess) e = cudaMemset(rt->scratch + rt->sl.status, 0, sizeof(int) * 4);
  if (e == cudaSuccess) e = cudaMemset(rt->scratch + rt->sl.gen, 0, sizeof(int));
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    set_error("workspace initialisation failed: %s", cudaGetErrorString(e));
    return fail(WM_ERR_CUDA);
  }
  if (rt->cfg.world > 1) {
    e = cudaStreamCreateWithFlags(&rt->side, cudaStreamNonBlocking);
    for (int c = 0; c < kMaxChunks && e == cudaSuccess; ++c) {
      e = cudaEventCreateWithFlags(&rt->ev_pulled[c], cudaEventDisableTiming);
      if (e == cudaSuccess) e = cudaEventCreateWithFlags(&rt->ev_ready[c], cudaEventDisableTiming);
    }
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&rt->push_stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&rt->ev_pushed, cudaEventDisableTiming);
    // Chunks of the owner's rows: only the first chunk's pull is exposed, every later pull runs on the side
    // stream beside the GEMMs of the chunks before it (WM_CHUNKS = 2..8).  Measured at 2 and 4 ranks on the
    // headline shape: 2 chunks 2.20 / 2.43 ms per step, 3 chunks 2.49 ms (4 ranks), 4 chunks 2.35 / 2.57 ms:
    // smaller GEMM launches and more copy kernels beside them cost more than the shorter first pull saves.
    // A runtime whose capacity is a small call (at most kSmallPlanRoutes routes per rank: decode) moves too
    // few rows to gain from the pipeline and takes one chunk: fewer launches and stream hand-offs per call.
    rt->chunks = 1ll * config->max_tokens * config->top_k <= kSmallPlanRoutes ? 1 : 2;
    if (const char* v = std::getenv("WM_CHUNKS")) {
      const int n = std::atoi(v);
      if (n >= 1 && n <= kMaxChunks) rt->chunks = n;
    }
    // SMs of the push GEMM when it runs beside the next chunk's compute (forward) or beside the chunk's own
    // weight gradients (backward).  Measured on the headline shape with skewed routing: forward at 8 ranks
    // 72 SMs 2.98 ms per step, none 3.08 ms, 48 SMs 3.06 ms; at 2 ranks 48 SMs 2.15 ms against 2.22 ms with
    // none; backward (beside the weight gradients) at 2 / 4 ranks: 48 SMs 2.22 / 2.34 ms, 74 SMs 2.38 / 2.42 ms,
    // 32 SMs 2.43 ms (2 ranks), 96 SMs 2.63 ms (4 ranks), weight gradients at the end 2.29 / 2.43 ms.  At 8 ranks
    // with this pipeline: 72 / 48 SMs (forward / backward) 2.60 ms, 48 / 48 2.58 ms, 72 / 72 2.64 ms, no SM split
    // 2.72 ms, weight gradients at the end 2.88 ms, four chunks 2.77 ms.
    rt->push_sms = config->world == 8 ? 72 : 48;
    rt->push_sms_bwd = 48;
    auto knob = [&](const char* name, int* value) {
      if (const char* v = std::getenv(name)) {
        const int n = std::atoi(v);
        *value = (n >= 8 && n <= rt->sms - 8) ? (n & ~1) : 0;
      }
    };
    knob("WM_PUSH_SMS", &rt->push_sms);
    knob("WM_PUSH_SMS_BWD", &rt->push_sms_bwd);
    if (e != cudaSuccess) {
      set_error("side stream creation failed: %s", cudaGetErrorString(e));
      return fail(WM_ERR_CUDA);
    }
  }
  rt->peer[rt->cfg.rank] = rt->arena;
  rt->peers_ready = rt->cfg.world == 1;
  *out = rt;
  return WM_OK;
}

extern "C" int wm_runtime_sizes(const wm_runtime* rt, wm_sizes* out) {
  if (!rt || !out) {
    set_error("wm_runtime_sizes: null argument");
    return WM_ERR_INVALID;
  }
  out->arena_bytes = static_cast<int64_t>(rt->al.total);
  out->scratch_bytes = static_cast<int64_t>(rt->sl.total);
  out->tape_bytes = static_cast<int64_t>(rt->tl.total);
  out->row_capacity = rt->row_cap;
  out->ipc_handle_bytes = static_cast<int32_t>(sizeof(cudaIpcMemHandle_t));
  return WM_OK;
}

extern "C" int wm_runtime_export_handle(wm_runtime* rt, void* handle_out, size_t bytes) {
  if (!rt || !rt->arena || !handle_out || bytes < sizeof(cudaIpcMemHandle_t)) {
    set_error("wm_runtime_export_handle: bad argument");
    return WM_ERR_INVALID;
  }
  cudaIpcMemHandle_t h;
  WM_CUDA(cudaIpcGetMemHandle(&h, rt->arena));
  std::memcpy(handle_out, &h, sizeof(h));
  return WM_OK;
}

extern "C" int wm_runtime_import_peers(wm_runtime* rt, const void* handles, size_t bytes) {
  if (!rt || !rt->arena || !handles || bytes < sizeof(cudaIpcMemHandle_t) * rt->cfg.world) {
    set_error("wm_runtime_import_peers: bad argument");
    return WM_ERR_INVALID;
  }
  if (rt->peers_ready) return WM_OK;
  const auto* h = static_cast<const cudaIpcMemHandle_t*>(handles);
  for (int r = 0; r < rt->cfg.world; ++r) {
    if (r == rt->cfg.rank) continue;
    void* p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h[r], cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      set_error("cudaIpcOpenMemHandle for rank %d failed: %s", r, cudaGetErrorString(e));
      for (int q = 0; q < r; ++q)
        if (q != rt->cfg.rank && rt->peer[q]) {
          cudaIpcCloseMemHandle(rt->peer[q]);
          rt->peer[q] = nullptr;
        }
      return WM_ERR_CUDA;
    }
    rt->peer[r] = static_cast<uint8_t*>(p);
  }
  rt->peers_ready = true;
  return WM_OK;
}

extern "C" int wm_runtime_retire_peers(wm_runtime* rt) {
  if (!rt) return WM_OK;
  for (int r = 0; r < rt->cfg.world; ++r) {
    if (r != rt->cfg.rank && rt->peer[r]) {
      cudaIpcCloseMemHandle(rt->peer[r]);
      rt->peer[r] = nullptr;
    }
  }
  rt->peers_ready = rt->cfg.world == 1;
  return WM_OK;
}

extern "C" int wm_runtime_destroy(wm_runtime* rt) {
  if (!rt) return WM_OK;
  wm_runtime_retire_peers(rt);
  if (rt->side) cudaStreamDestroy(rt->side);
  for (int c = 0; c < kMaxChunks; ++c) {
    if (rt->ev_pulled[c]) cudaEventDestroy(rt->ev_pulled[c]);
    if (rt->ev_ready[c]) cudaEventDestroy(rt->ev_ready[c]);
  }
  if (rt->push_stream) cudaStreamDestroy(rt->push_stream);
  if (rt->ev_pushed) cudaEventDestroy(rt->ev_pushed);
  for (auto& slot : rt->slots)
    for (int k = 0; k < kStageCount; ++k)
      for (int c = 0; c < kMaxChunks; ++c) {
        if (slot.start[k][c]) cudaEventDestroy(slot.start[k][c]);
        if (slot.stop[k][c]) cudaEventDestroy(slot.stop[k][c]);
      }
  if (rt->ev_trace_origin) cudaEventDestroy(rt->ev_trace_origin);
  if (rt->arena) cudaFree(rt->arena);
  if (rt->scratch) cudaFree(rt->scratch);
  rt->arena = rt->scratch = nullptr;
  delete rt;
  return WM_OK;
}

extern "C" int wm_status_poll(wm_runtime* rt, int32_t* code, void* stream_) {
  if (int rc = check_ready(rt, "wm_status_poll")) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  int device_code = 0;
  WM_CUDA(cudaMemcpyAsync(&device_code, rt->scratch + rt->sl.status, sizeof(int),
                          cudaMemcpyDeviceToHost, stream));
  WM_CUDA(cudaStreamSynchronize(stream));
  if (device_code != 0) {
    WM_CUDA(cudaMemsetAsync(rt->scratch + rt->sl.status, 0, sizeof(int), stream));
    set_error("device status %d (%s)", device_code,
              device_code == kStatusRowOverflow ? "received rows exceed max_rows"
                                                : "a bounded device wait ran out");
  }
  if (code) *code = map_status(device_code);
  return WM_OK;
}

// Every collective call takes the next generation.  At world > 1 the number lives on the device and is
// bumped by a one-thread kernel on the call's stream, so that the flag kernels of a call captured in a
// CUDA graph see a new generation at every replay.
__global__ void bump_generation_kernel(int* gen) { *gen += 1; }
static Gen begin_generation(wm_runtime* rt, cudaStream_t stream) {
  ++rt->generation;
  if (rt->cfg.world == 1) return Gen{nullptr, rt->generation};
  int* dev = reinterpret_cast<int*>(rt->scratch + rt->sl.gen);
  bump_generation_kernel<<<1, 1, 0, stream>>>(dev);
  count_launch();
  return Gen{dev, 0};
}

// =============================================================================== forward
// Calls of at most kSmallPlanRoutes routes plan in one launch (WM_SMALL_PLAN=0 keeps the general kernels).
static bool small_plan_allowed(long long routes) {
  static const bool on = [] {
    const char* v = std::getenv("WM_SMALL_PLAN");
    return !(v && v[0] == '0');
  }();
  return on && routes <= kSmallPlanRoutes;
}

extern "C" int wm_forward(wm_runtime* rt, const void* x, const int32_t* routes, const float* gates,
                          const void* w1, const void* w2, int32_t tokens, void* y, void* tape,
                          void* stream_) {
  if (int rc = check_ready(rt, "wm_forward")) return rc;
  const wm_config& c = rt->cfg;
  if (tokens < 0 || tokens > c.max_tokens) {
    set_error("Activation shape exceeds prepared capacity (%d tokens, capacity %d)", tokens,
              c.max_tokens);
    return WM_ERR_CAPACITY;
  }
  if (!w1 || !w2 || (tokens > 0 && (!x || !routes || !gates || !y)) || !aligned16(x) ||
      !aligned16(y) || !aligned16(w1) || !aligned16(w2) || !aligned16(tape)) {
    set_error("wm_forward: null or misaligned tensor (16-byte alignment required)");
    return WM_ERR_INVALID;
  }
  if (tape && !c.training) {
    set_error("wm_forward: a training cache needs a runtime created with training=1");
    return WM_ERR_STATE;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const Gen gen = begin_generation(rt, stream);
  const int world = c.world;
  uint8_t* S = rt->scratch;
  uint8_t* T = static_cast<uint8_t*>(tape);
  int* status = at<int>(S, rt->sl.status);

  // Arrays that the backward pass needs live in the tape when one is given.
  RouteLocal local{tape ? at<int>(T, rt->tl.sorted_slot) : at<int>(S, rt->sl.sorted_slot),
                   tape ? at<int>(T, rt->tl.sorted_expert) : at<int>(S, rt->sl.sorted_expert),
                   at<int>(S, rt->sl.slot_pos)};
  PlanTables tables{};
  tables.expert_total = at<int>(S, rt->sl.expert_total);
  tables.expert_before = at<int>(S, rt->sl.expert_before);
  tables.expert_base = at<int>(S, rt->sl.expert_base);
  tables.expert_pbase = at<int>(S, rt->sl.expert_pbase);
  tables.padded_start = tape ? at<int>(T, rt->tl.padded_start) : at<int>(S, rt->sl.padded_start);
  tables.tile_group = tape ? at<int>(T, rt->tl.tile_group) : at<int>(S, rt->sl.tile_group);
  tables.num_tiles = tape ? at<int>(T, rt->tl.num_tiles) : at<int>(S, rt->sl.num_tiles);
  tables.padded_rows = tape ? at<int>(T, rt->tl.padded_rows) : at<int>(S, rt->sl.padded_rows);
  tables.pair_tiles = tape ? at<int>(T, rt->tl.pair_tiles) : at<int>(S, rt->sl.pair_tiles);
  tables.num_pairs = tape ? at<int>(T, rt->tl.num_pairs) : at<int>(S, rt->sl.num_pairs);
  tables.split = tape ? at<int>(T, rt->tl.split) : at<int>(S, rt->sl.split);
  tables.live_rows = tape ? at<int>(T, rt->tl.live_rows) : nullptr;
  tables.group_order = tape ? at<int>(T, rt->tl.group_order) : nullptr;
  int* origin = tape ? at<int>(T, rt->tl.origin) : at<int>(S, rt->sl.origin);
  float* prob = tape ? at<float>(T, rt->tl.prob) : at<float>(S, rt->sl.prob);
  // world > 1: row a duplicate of a token is copied from (the token crosses NVLink once per owner).
  int* primary = world == 1 ? nullptr : (tape ? at<int>(T, rt->tl.primary) : at<int>(S, rt->sl.primary));
  auto* xrows = tape ? at<__nv_bfloat16>(T, rt->tl.xrows) : at<__nv_bfloat16>(S, rt->sl.xrows);
  auto* ab = tape ? at<__nv_bfloat16>(T, rt->tl.ab) : nullptr;
  auto* u = at<__nv_bfloat16>(S, rt->sl.u);

  RouteShape shape{c.experts, c.top_k, world, c.rank, c.max_tokens};
  PeerInts counts{}, meta_origin{}, meta_primary{};
  PeerFloats meta_prob{};
  PeerConstRows stage{};
  PushTarget push{};
  for (int r = 0; r < world; ++r) {
    counts.p[r] = at<int>(rt->peer[r], rt->al.counts);
    meta_origin.p[r] = at<int>(rt->peer[r], rt->al.meta_origin);
    meta_prob.p[r] = at<float>(rt->peer[r], rt->al.meta_prob);
    meta_primary.p[r] = at<int>(rt->peer[r], rt->al.meta_primary);
    stage.p[r] = at<__nv_bfloat16>(rt->peer[r], rt->al.stage);
    push.mailbox[r] = at<__nv_bfloat16>(rt->peer[r], rt->al.mailbox);
  }
  push.origin = origin;
  push.cap = c.max_tokens;
  push.top_k = c.top_k;

  // Rows per local expert if routing were uniform: tokens * K * world / E (kernel choice only).
  const bool many_rows = 1ll * tokens * c.top_k * world >= 1024ll * c.experts;
  // 1. staging buffer free?  then stage x and plan locally; counts go to every rank.
  TimingSlot* timing = begin_timing(rt, stream);
  if (world == 1) {
    stage.p[0] = static_cast<const __nv_bfloat16*>(x);  // no peers: owners read x itself
  } else {
    StageScope scope(timing, kStageStageIn, stream);
    if (int rc = wait_flags(my_flags(rt, kPulled), world, gen - 1, status, nullptr, stream)) return rc;
    if (tokens > 0)
      WM_CUDA(cudaMemcpyAsync(rt->arena + rt->al.stage, x, 2ull * tokens * c.hidden,
                              cudaMemcpyDeviceToDevice, stream));
  }
  // 1b/2. local plan, count exchange, global plan (waits for all count rows), destination rows,
  //       origin/prob words to the owners.  At world > 1 the stage time includes the wait.
  RouteRows rows{at<int>(S, rt->sl.local_offset), at<int>(S, rt->sl.dst_rank), at<int>(S, rt->sl.dst_row),
                 at<int>(S, rt->sl.dst_prow)};
  if (small_plan_allowed(1ll * tokens * c.top_k)) {
    // decode and small prefill: everything above plus the COUNTS / READY hand-shakes in one launch
    StageScope scope(timing, kStagePlan, stream);
    SmallPlan plan{};
    plan.shape = shape;
    plan.routes = routes;
    plan.gates = gates;
    plan.tokens = tokens;
    plan.local = local;
    plan.rows = rows;
    plan.tables = tables;
    plan.local_count = at<int>(S, rt->sl.local_count);
    plan.count_matrix = counts;
    plan.my_count_matrix = at<int>(rt->arena, rt->al.counts);
    plan.meta_origin = meta_origin;
    plan.meta_prob = meta_prob;
    plan.meta_primary = meta_primary;
    plan.want_primary = world > 1;
    plan.global_part = 1;
    plan.exchange = world > 1;
    plan.flag_counts = flag_group(rt, kCounts);
    plan.my_flag_counts = my_flags(rt, kCounts);
    plan.flag_ready = flag_group(rt, kReady);
    plan.my_flag_ready = my_flags(rt, kReady);
    plan.generation = world > 1 ? gen : Gen{};
    plan.row_capacity = rt->row_cap;
    plan.status = status;
    plan.chunks = rt->chunks;
    if (int rc = route_plan_small(plan, stream)) return rc;
  } else {
    {
      StageScope scope(timing, kStagePlan, stream);
      if (int rc = route_local(shape, routes, tokens, local, at<int>(S, rt->sl.chunk_hist),
                               at<int>(S, rt->sl.local_count), counts, stream))
        return rc;
      if (world > 1)
        if (int rc = signal_peers(flag_group(rt, kCounts), world, c.rank, gen, stream)) return rc;
      if (int rc = route_global(shape, at<int>(rt->arena, rt->al.counts), my_flags(rt, kCounts),
                                world > 1 ? gen : Gen{}, rt->row_cap, tables, status, rt->chunks, stream))
        return rc;
      if (int rc = route_rows(shape, routes, gates, tokens, local, at<int>(S, rt->sl.chunk_hist),
                              tables, rows, meta_origin, meta_prob, rt->row_cap, status, stream))
        return rc;
      if (world > 1)
        if (int rc = route_primary(shape, tokens, local, rows, meta_primary, nullptr, rt->row_cap, status, stream))
          return rc;
    }
    if (world > 1) {
      StageScope scope(timing, kStageSyncReady, stream);
      if (int rc = signal_peers(flag_group(rt, kReady), world, c.rank, gen, stream)) return rc;
      if (int rc = wait_flags(my_flags(rt, kReady), world, gen, status, tables.split, stream)) return rc;
    }
  }
  // 3. owner side: pull rows, then the two grouped GEMMs; FC2 pushes into the sources' mailboxes.
  //    world > 1: the rows are cut at expert boundaries into rt->chunks chunks.  Chunk 0 is pulled on
  //    this stream with every SM; the later chunks are pulled on the side stream while FC1 / FC2 of the
  //    chunks before them run (inbound NVLink beside compute and pushes), so only the first pull is
  //    exposed.
  const int chunks = world > 1 ? rt->chunks : 1;
  auto owner_rows = [&](int chunk) {
    return OwnerRows{tables.padded_start, tables.tile_group, split_range(tables.split, 2, chunk),
                     tables.expert_total};
  };
  auto pull = [&](int chunk, cudaStream_t st) -> int {
    const int ctas = st == rt->side ? rt->sms * 2 : rt->sms * 8;  // the side stream copies beside a GEMM
    if (int rc = gather_rows(owner_rows(chunk), c.rank, rt->e_local, world, rt->row_cap, c.max_tokens, c.top_k,
                             c.hidden, stage,
                             at<int>(rt->arena, rt->al.meta_origin), at<float>(rt->arena, rt->al.meta_prob),
                             primary ? at<int>(rt->arena, rt->al.meta_primary) : nullptr, xrows, origin,
                             prob, primary, ctas, st))
      return rc;
    return primary ? copy_duplicate_rows(split_range(tables.split, 2, chunk), primary, c.hidden, xrows, ctas, st)
                   : 0;
  };
  auto schedule_of = [&](int chunk) {
    return Schedule{tables.split, tables.tile_group, tables.padded_start, rt->e_local, rt->row_cap,
                    tables.pair_tiles, many_rows, chunk};
  };
  auto fc1 = [&](int chunk, int sms) -> int {
    StageScope scope(timing, chunk <= 0 ? kStageFc1 : kStageFc1B, stream, chunk < 0 ? 0 : chunk);
    return launch_fc1(schedule_of(chunk), xrows, static_cast<const __nv_bfloat16*>(w1), u, ab, prob, c.hidden,
                      c.intermediate, status, sms, stream);
  };
  auto fc2 = [&](int chunk, int sms, cudaStream_t st) -> int {
    StageScope scope(timing, chunk <= 0 ? kStageFc2 : kStageFc2B, st, chunk < 0 ? 0 : chunk);
    return launch_mgrouped_nt(schedule_of(chunk), u, static_cast<const __nv_bfloat16*>(w2), nullptr, &push,
                              c.hidden, c.intermediate, status, sms, st);
  };
  if (chunks == 1) {
    {
      StageScope scope(timing, kStageGather, stream);
      if (int rc = pull(kWhole, stream)) return rc;
    }
    if (world > 1)  // every row of this call has been read from the sources' staging buffers
      if (int rc = signal_peers(flag_group(rt, kPulled), world, c.rank, gen, stream)) return rc;
    if (int rc = fc1(kWhole, rt->sms)) return rc;
    if (int rc = fc2(kWhole, rt->sms, stream)) return rc;
  } else {
    {
      StageScope scope(timing, kStageGather, stream);
      if (int rc = pull(0, stream)) return rc;
    }
    WM_CUDA(cudaEventRecord(rt->ev_pulled[0], stream));
    WM_CUDA(cudaStreamWaitEvent(rt->side, rt->ev_pulled[0], 0));
    for (int k = 1; k < chunks; ++k) {
      {
        StageScope scope(timing, kStageGatherB, rt->side, k);
        if (int rc = pull(k, rt->side)) return rc;
      }
      WM_CUDA(cudaEventRecord(rt->ev_pulled[k], rt->side));
    }
    // With push_sms > 0, FC2 of chunk k (bound by its NVLink pushes) runs on push_sms SMs of a third
    // stream beside FC1 of chunk k + 1 on the other SMs; the last chunk's FC2 gets every SM again.
    const bool beside = rt->push_sms > 0;
    for (int k = 0; k < chunks; ++k) {
      if (k > 0) WM_CUDA(cudaStreamWaitEvent(stream, rt->ev_pulled[k], 0));
      if (k == chunks - 1)  // every row of this call has been read from the sources' staging buffers
        if (int rc = signal_peers(flag_group(rt, kPulled), world, c.rank, gen, stream)) return rc;
      if (int rc = fc1(k, beside && k > 0 ? rt->sms - rt->push_sms : rt->sms)) return rc;
      if (beside && k < chunks - 1) {
        WM_CUDA(cudaEventRecord(rt->ev_ready[k], stream));
        WM_CUDA(cudaStreamWaitEvent(rt->push_stream, rt->ev_ready[k], 0));
        if (int rc = fc2(k, rt->push_sms, rt->push_stream)) return rc;
        WM_CUDA(cudaEventRecord(rt->ev_pushed, rt->push_stream));
      } else {
        if (beside) WM_CUDA(cudaStreamWaitEvent(stream, rt->ev_pushed, 0));
        if (int rc = fc2(k, rt->sms, stream)) return rc;
      }
    }
  }
  if (world > 1) {
    StageScope scope(timing, kStageSyncContrib, stream);
    if (int rc = signal_peers(flag_group(rt, kContrib), world, c.rank, gen, stream)) return rc;
    if (int rc = wait_flags(my_flags(rt, kContrib), world, gen, status, nullptr, stream)) return rc;
  }
  // 4. source side: ordered FP32 combine.
  StageScope scope(timing, kStageCombine, stream);
  return combine_rows(at<__nv_bfloat16>(rt->arena, rt->al.mailbox), local.sorted_expert, tokens,
                      c.max_tokens, c.top_k, c.hidden, static_cast<__nv_bfloat16*>(y), stream);
}

// =============================================================================== backward
extern "C" int wm_backward(wm_runtime* rt, const void* tape, const void* dy, const void* w1,
                           const void* w2, int32_t tokens, void* dx, float* dgates, void* dw1,
                           void* dw2, void* stream_) {
  if (int rc = check_ready(rt, "wm_backward")) return rc;
  const wm_config& c = rt->cfg;
  if (!c.training) {
    set_error("Backward requires a runtime prepared with training=True");
    return WM_ERR_STATE;
  }
  if (tokens < 0 || tokens > c.max_tokens) {
    set_error("Backward token count %d exceeds capacity %d", tokens, c.max_tokens);
    return WM_ERR_CAPACITY;
  }
  if (!tape || !w1 || !w2 || !dw1 || !dw2 || (tokens > 0 && (!dy || !dx || !dgates)) ||
      !aligned16(tape) || !aligned16(dy) || !aligned16(dx) || !aligned16(dw1) || !aligned16(dw2)) {
    set_error("wm_backward: null or misaligned tensor (16-byte alignment required)");
    return WM_ERR_INVALID;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const Gen gen = begin_generation(rt, stream);
  const int world = c.world;
  uint8_t* S = rt->scratch;
  const uint8_t* T = static_cast<const uint8_t*>(tape);
  auto tp = [&](size_t off) { return const_cast<uint8_t*>(T) + off; };
  int* status = at<int>(S, rt->sl.status);
  const int* sorted_slot = reinterpret_cast<const int*>(tp(rt->tl.sorted_slot));
  const int* sorted_expert = reinterpret_cast<const int*>(tp(rt->tl.sorted_expert));
  const int* padded_start = reinterpret_cast<const int*>(tp(rt->tl.padded_start));
  const int* tile_group = reinterpret_cast<const int*>(tp(rt->tl.tile_group));
  const int* pair_tiles = reinterpret_cast<const int*>(tp(rt->tl.pair_tiles));
  const int* origin = reinterpret_cast<const int*>(tp(rt->tl.origin));
  const float* prob = reinterpret_cast<const float*>(tp(rt->tl.prob));
  const auto* xrows = reinterpret_cast<const __nv_bfloat16*>(tp(rt->tl.xrows));
  const auto* ab = reinterpret_cast<const __nv_bfloat16*>(tp(rt->tl.ab));
  auto* recv = at<__nv_bfloat16>(S, rt->sl.recv);
  auto* u = at<__nv_bfloat16>(S, rt->sl.u);
  auto* du = at<__nv_bfloat16>(S, rt->sl.du);
  auto* dab = at<__nv_bfloat16>(S, rt->sl.dab);

  PeerConstRows stage{};
  PeerFloats dgate_box{};
  PushTarget push{};
  for (int r = 0; r < world; ++r) {
    stage.p[r] = at<__nv_bfloat16>(rt->peer[r], rt->al.stage);
    dgate_box.p[r] = at<float>(rt->peer[r], rt->al.dgate_box);
    push.mailbox[r] = at<__nv_bfloat16>(rt->peer[r], rt->al.mailbox);
  }
  push.origin = origin;
  push.cap = c.max_tokens;
  push.top_k = c.top_k;

  // 1. stage dY where the owners can read it.
  TimingSlot* timing = begin_timing(rt, stream);
  if (world == 1) {
    stage.p[0] = static_cast<const __nv_bfloat16*>(dy);  // no peers: owners read dY itself
  } else {
    {
      StageScope scope(timing, kStageStageInBwd, stream);
      if (int rc = wait_flags(my_flags(rt, kPulled), world, gen - 1, status, nullptr, stream)) return rc;
      if (tokens > 0)
        WM_CUDA(cudaMemcpyAsync(rt->arena + rt->al.stage, dy, 2ull * tokens * c.hidden,
                                cudaMemcpyDeviceToDevice, stream));
    }
    StageScope scope(timing, kStageSyncReadyBwd, stream);
    if (int rc = signal_peers(flag_group(rt, kReady), world, c.rank, gen, stream)) return rc;
    // (the saved split is only read by this call: emptying it on a failed wait is harmless)
    if (int rc = wait_flags(my_flags(rt, kReady), world, gen, status,
                            reinterpret_cast<int*>(tp(rt->tl.split)), stream))
      return rc;
  }
  // 2./3. owner side: pull dY rows in the saved row order; dU = dY * W2; SwiGLU backward (U, dAB,
  //       dprob -> sources); dX = dAB * W1 -> sources.  world > 1: two halves, the second half's
  //       pull runs on the side stream beside the first half's compute and pushes.
  // Rows per local expert if routing were uniform: tokens * K * world / E.
  const bool many_rows = 1ll * tokens * c.top_k * world >= 1024ll * c.experts;
  const int* split = reinterpret_cast<const int*>(tp(rt->tl.split));
  const int chunks = world > 1 ? rt->chunks : 1;
  const int* primary = world == 1 ? nullptr : reinterpret_cast<const int*>(tp(rt->tl.primary));
  auto pull = [&](int chunk, cudaStream_t st) -> int {
    const int ctas = st == rt->side ? rt->sms * 2 : rt->sms * 8;  // the side stream copies beside a GEMM
    if (int rc = gather_by_origin(split_range(split, 2, chunk), origin, primary, world, c.max_tokens, c.top_k,
                                  c.hidden, stage, recv, ctas, st))
      return rc;
    return primary ? copy_duplicate_rows(split_range(split, 2, chunk), primary, c.hidden, recv, ctas, st) : 0;
  };
  auto schedule = [&](int chunk) {
    return Schedule{split, tile_group, padded_start, rt->e_local, rt->row_cap, pair_tiles, many_rows, chunk};
  };
  // dU with the SwiGLU backward in its epilogue (no dU buffer, no separate elementwise pass) where the
  // one-CTA kernel runs dU and I is a multiple of 256; WM_FUSED_DU=0 keeps the two-kernel form.
  static const bool fused_allowed = [] {
    const char* v = std::getenv("WM_FUSED_DU");
    return !(v && v[0] == '0');
  }();
  auto* dprob_part = at<float>(S, rt->sl.dprob_part);
  auto du_and_swiglu = [&](int chunk, int sms) -> int {
    const int slot = chunk < 0 ? 0 : chunk;
    const int stage_du = chunk <= 0 ? kStageDu : kStageDuB, stage_sw = chunk <= 0 ? kStageSwigluBwd : kStageSwigluBwdB;
    if (fused_allowed) {
      int rc;
      {
        StageScope scope(timing, stage_du, stream, slot);
        rc = launch_du_swiglu_backward(schedule(chunk), recv, static_cast<const __nv_bfloat16*>(w2), ab, prob, u,
                                       dab, dprob_part, c.intermediate, c.hidden, status, sms, stream);
      }
      if (rc > 0) return rc;
      if (rc == 0) {
        StageScope scope(timing, stage_sw, stream, slot);
        return dprob_finish(split_range(split, 2, chunk), dprob_part, c.intermediate / 128, rt->row_cap, origin,
                            c.max_tokens, c.top_k, dgate_box, stream);
      }
    }
    {
      StageScope scope(timing, stage_du, stream, slot);
      if (int rc = launch_mgrouped_nn(schedule(chunk), recv, static_cast<const __nv_bfloat16*>(w2), du, nullptr,
                                      c.intermediate, c.hidden, status, sms, stream))
        return rc;
    }
    StageScope scope(timing, stage_sw, stream, slot);
    return swiglu_backward(split_range(split, 2, chunk), ab, du, prob, origin, c.intermediate, c.max_tokens,
                           c.top_k, u, dab, dgate_box, rt->sms, stream);
  };
  auto dx_push = [&](int chunk, int sms, cudaStream_t st) -> int {
    StageScope scope(timing, chunk <= 0 ? kStageDx : kStageDxB, st, chunk < 0 ? 0 : chunk);
    return launch_mgrouped_nn(schedule(chunk), dab, static_cast<const __nv_bfloat16*>(w1), nullptr, &push,
                              c.hidden, 2 * c.intermediate, status, sms, st);
  };
  static const bool ordered_wgrad = [] {  // WM_WGRAD_ORDER=0: walk the experts in index order (A/B runs)
    const char* v = std::getenv("WM_WGRAD_ORDER");
    return !(v && v[0] == '0');
  }();
  static const bool interleave_wgrad = [] {  // WM_WGRAD_INTERLEAVE=0: all weight gradients after the last chunk
    const char* v = std::getenv("WM_WGRAD_INTERLEAVE");
    return !(v && v[0] == '0');
  }();
  auto weight_gradients = [&](int chunk, int sms) -> int {
    Schedule sched = schedule(chunk);
    sched.group_live_rows = reinterpret_cast<const int*>(tp(rt->tl.live_rows));
    if (ordered_wgrad) sched.group_order = reinterpret_cast<const int*>(tp(rt->tl.group_order));
    const int slot = chunk < 0 ? 0 : chunk;
    {
      StageScope scope(timing, kStageDw1, stream, slot);
      if (int rc = launch_kgrouped_tn(sched, dab, xrows, static_cast<__nv_bfloat16*>(dw1), 2 * c.intermediate,
                                      c.hidden, status, sms, stream))
        return rc;
    }
    StageScope scope(timing, kStageDw2, stream, slot);
    return launch_kgrouped_tn(sched, recv, u, static_cast<__nv_bfloat16*>(dw2), c.hidden, c.intermediate, status,
                              sms, stream);
  };
  if (chunks == 1) {
    {
      StageScope scope(timing, kStageGatherDy, stream);
      if (int rc = pull(kWhole, stream)) return rc;
    }
    if (world > 1)
      if (int rc = signal_peers(flag_group(rt, kPulled), world, c.rank, gen, stream)) return rc;
    if (int rc = du_and_swiglu(kWhole, rt->sms)) return rc;
    if (int rc = dx_push(kWhole, rt->sms, stream)) return rc;
  } else {
    {
      StageScope scope(timing, kStageGatherDy, stream);
      if (int rc = pull(0, stream)) return rc;
    }
    WM_CUDA(cudaEventRecord(rt->ev_pulled[0], stream));
    WM_CUDA(cudaStreamWaitEvent(rt->side, rt->ev_pulled[0], 0));
    for (int k = 1; k < chunks; ++k) {
      {
        StageScope scope(timing, kStageGatherDyB, rt->side, k);
        if (int rc = pull(k, rt->side)) return rc;
      }
      WM_CUDA(cudaEventRecord(rt->ev_pulled[k], rt->side));
    }
    if (!interleave_wgrad) {
      // With push_sms_bwd > 0, dX of chunk k pushes from a few SMs on a third stream while dU and the SwiGLU
      // backward of chunk k + 1 compute on the others.
      const bool beside = rt->push_sms_bwd > 0;
      for (int k = 0; k < chunks; ++k) {
        if (k > 0) WM_CUDA(cudaStreamWaitEvent(stream, rt->ev_pulled[k], 0));
        if (k == chunks - 1)
          if (int rc = signal_peers(flag_group(rt, kPulled), world, c.rank, gen, stream)) return rc;
        if (int rc = du_and_swiglu(k, beside && k > 0 ? rt->sms - rt->push_sms_bwd : rt->sms)) return rc;
        if (beside && k < chunks - 1) {
          WM_CUDA(cudaEventRecord(rt->ev_ready[k], stream));
          WM_CUDA(cudaStreamWaitEvent(rt->push_stream, rt->ev_ready[k], 0));
          if (int rc = dx_push(k, rt->push_sms_bwd, rt->push_stream)) return rc;
          WM_CUDA(cudaEventRecord(rt->ev_pushed, rt->push_stream));
        } else {
          if (beside) WM_CUDA(cudaStreamWaitEvent(stream, rt->ev_pushed, 0));
          if (int rc = dx_push(k, rt->sms, stream)) return rc;
        }
      }
    } else {
      // Chunk by chunk: dU + SwiGLU backward on every SM, then the chunk's dX GEMM (bound by its NVLink
      // pushes) on `push` SMs of the third stream WHILE this stream computes the chunk's weight gradients
      // (no communication, pure tensor work) on the other SMs.  The weight gradients of a chunk only need
      // that chunk's rows, so they fill the time the link is the limit instead of running at the very end.
      const int push = rt->push_sms_bwd > 0 ? rt->push_sms_bwd : (rt->sms / 2) & ~1;
      for (int k = 0; k < chunks; ++k) {
        if (k > 0) WM_CUDA(cudaStreamWaitEvent(stream, rt->ev_pulled[k], 0));
        if (k == chunks - 1)
          if (int rc = signal_peers(flag_group(rt, kPulled), world, c.rank, gen, stream)) return rc;
        if (int rc = du_and_swiglu(k, rt->sms)) return rc;
        WM_CUDA(cudaEventRecord(rt->ev_ready[k], stream));
        WM_CUDA(cudaStreamWaitEvent(rt->push_stream, rt->ev_ready[k], 0));
        if (int rc = dx_push(k, push, rt->push_stream)) return rc;
        if (k == chunks - 1)  // every result row of this call is on its way: tell the sources from that stream
          if (int rc = signal_peers(flag_group(rt, kContrib), world, c.rank, gen, rt->push_stream)) return rc;
        WM_CUDA(cudaEventRecord(rt->ev_pushed, rt->push_stream));
        if (int rc = weight_gradients(k, rt->sms - push)) return rc;
      }
      WM_CUDA(cudaStreamWaitEvent(stream, rt->ev_pushed, 0));
    }
  }
  // 4. weight gradients: reductions over each expert's rows in the saved (fixed) order (chunk by chunk above
  //    when they are interleaved with the pushes).
  if (!(chunks > 1 && interleave_wgrad)) {
    if (world > 1)
      if (int rc = signal_peers(flag_group(rt, kContrib), world, c.rank, gen, stream)) return rc;
    if (int rc = weight_gradients(kWhole, rt->sms)) return rc;
  }
  // 5. source side: ordered combine of dX, dprob back to the original slots.
  if (world > 1) {
    StageScope scope(timing, kStageSyncContribBwd, stream);
    if (int rc = wait_flags(my_flags(rt, kContrib), world, gen, status, nullptr, stream)) return rc;
  }
  StageScope scope(timing, kStageCombineDx, stream);
  if (int rc = combine_rows(at<__nv_bfloat16>(rt->arena, rt->al.mailbox), sorted_expert, tokens,
                            c.max_tokens, c.top_k, c.hidden, static_cast<__nv_bfloat16*>(dx), stream))
    return rc;
  return unpermute_dgates(at<float>(rt->arena, rt->al.dgate_box), sorted_slot, sorted_expert, tokens,
                          c.top_k, dgates, stream);
}

// =============================================================================== quantised forward
extern "C" int wm_forward_quantized(wm_runtime* rt, const void* x, const int32_t* routes,
                                    const float* gates, const wm_quant_weights* weights, int32_t tokens,
                                    void* y, void* tape, void* stream_) {
  if (int rc = check_ready(rt, "wm_forward_quantized")) return rc;
  const wm_config& c = rt->cfg;
  const int kind = c.reserved == 1 ? kKindFp8 : kKindNvfp4;
  if (c.reserved == 0) {
    set_error("wm_forward_quantized: the runtime was created for BF16");
    return WM_ERR_STATE;
  }
  if (tokens < 0 || tokens > c.max_tokens) {
    set_error("Activation shape exceeds prepared capacity (%d tokens, capacity %d)", tokens, c.max_tokens);
    return WM_ERR_CAPACITY;
  }
  const bool prequantised = weights && weights->source_q != nullptr;
  if (prequantised && (c.reserved != 1 || !weights->source_scales || !aligned16(weights->source_q) ||
                       !aligned16(weights->source_scales))) {
    set_error("wm_forward_quantized: a prequantised source needs an FP8 runtime and 16-byte aligned bytes and scales");
    return WM_ERR_INVALID;
  }
  if (!weights || !weights->w1 || !weights->w1_sf || !weights->w2 || !weights->w2_sf ||
      (tokens > 0 && ((!x && !prequantised) || !routes || !gates || !y)) || !aligned16(x) || !aligned16(y) ||
      !aligned16(weights->w1) || !aligned16(weights->w2) || !aligned16(weights->w1_sf) ||
      !aligned16(weights->w2_sf)) {
    set_error("wm_forward_quantized: null or misaligned tensor (16-byte alignment required)");
    return WM_ERR_INVALID;
  }
  if (kind == kKindNvfp4 && !(weights->x_scale > 0 && weights->w1_scale > 0 && weights->u_scale > 0 &&
                              weights->w2_scale > 0)) {
    set_error("NVFP4 tensor scales must be finite and positive");
    return WM_ERR_INVALID;
  }
  if (tape && (!c.training || !aligned16(tape))) {
    set_error("a training cache needs a runtime created with training=1");
    return WM_ERR_STATE;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const Gen gen = begin_generation(rt, stream);
  const int world = c.world;
  const int H = c.hidden, I = c.intermediate;
  uint8_t* S = rt->scratch;
  uint8_t* T = static_cast<uint8_t*>(tape);
  int* status = at<int>(S, rt->sl.status);
  // With a tape, everything the backward pass needs is written into it (same layout as the BF16 tape;
  // the row section holds the E4M3 rows followed by their scale chunks).
  auto pick = [&](size_t tape_off, size_t scratch_off) { return tape ? T + tape_off : S + scratch_off; };
  RouteLocal local{reinterpret_cast<int*>(pick(rt->tl.sorted_slot, rt->sl.sorted_slot)),
                   reinterpret_cast<int*>(pick(rt->tl.sorted_expert, rt->sl.sorted_expert)),
                   at<int>(S, rt->sl.slot_pos)};
  PlanTables tables{};
  tables.expert_total = at<int>(S, rt->sl.expert_total);
  tables.expert_before = at<int>(S, rt->sl.expert_before);
  tables.expert_base = at<int>(S, rt->sl.expert_base);
  tables.expert_pbase = at<int>(S, rt->sl.expert_pbase);
  tables.padded_start = reinterpret_cast<int*>(pick(rt->tl.padded_start, rt->sl.padded_start));
  tables.tile_group = reinterpret_cast<int*>(pick(rt->tl.tile_group, rt->sl.tile_group));
  tables.num_tiles = reinterpret_cast<int*>(pick(rt->tl.num_tiles, rt->sl.num_tiles));
  tables.padded_rows = reinterpret_cast<int*>(pick(rt->tl.padded_rows, rt->sl.padded_rows));
  tables.pair_tiles = reinterpret_cast<int*>(pick(rt->tl.pair_tiles, rt->sl.pair_tiles));
  tables.num_pairs = reinterpret_cast<int*>(pick(rt->tl.num_pairs, rt->sl.num_pairs));
  tables.split = reinterpret_cast<int*>(pick(rt->tl.split, rt->sl.split));
  int* origin = reinterpret_cast<int*>(pick(rt->tl.origin, rt->sl.origin));
  float* prob = reinterpret_cast<float*>(pick(rt->tl.prob, rt->sl.prob));
  uint8_t* xq = pick(rt->tl.xrows, rt->sl.xrows);
  uint8_t* uq = at<uint8_t>(S, rt->sl.u);
  auto* abq = reinterpret_cast<__nv_bfloat16*>(pick(rt->tl.ab, rt->sl.abq));
  auto* sfa_x = tape ? reinterpret_cast<uint32_t*>(T + rt->tl.xrows + align_up(static_cast<size_t>(rt->row_cap) * H))
                     : at<uint32_t>(S, rt->sl.sfa_x);
  auto* sfa_u = at<uint32_t>(S, rt->sl.sfa_u);

  RouteShape shape{c.experts, c.top_k, world, c.rank, c.max_tokens};
  PeerInts counts{}, meta_origin{};
  PeerFloats meta_prob{};
  PeerBytes stage{};
  PushTarget push{};
  for (int r = 0; r < world; ++r) {
    counts.p[r] = at<int>(rt->peer[r], rt->al.counts);
    meta_origin.p[r] = at<int>(rt->peer[r], rt->al.meta_origin);
    meta_prob.p[r] = at<float>(rt->peer[r], rt->al.meta_prob);
    stage.p[r] = rt->peer[r] + rt->al.stage;
    push.mailbox[r] = at<__nv_bfloat16>(rt->peer[r], rt->al.mailbox);
  }
  push.origin = origin;
  push.cap = c.max_tokens;
  push.top_k = c.top_k;

  // 1. quantise this rank's tokens into the staging buffer: data rows, then the scale rows.
  const size_t row_bytes = kind == kKindFp8 ? H : H / 2;
  const size_t sf_offset = align_up(static_cast<size_t>(c.max_tokens) * row_bytes);
  if (world > 1)
    if (int rc = wait_flags(my_flags(rt, kPulled), world, gen - 1, status, nullptr, stream)) return rc;
  uint8_t* my_stage = rt->arena + rt->al.stage;
  if (tokens > 0) {
    if (prequantised) {  // the caller's bytes and scales are what the online quantiser would have written
      WM_CUDA(cudaMemcpyAsync(my_stage, weights->source_q, static_cast<size_t>(tokens) * H,
                              cudaMemcpyDeviceToDevice, stream));
      WM_CUDA(cudaMemcpyAsync(my_stage + sf_offset, weights->source_scales,
                              static_cast<size_t>(tokens) * (H / 128) * sizeof(float), cudaMemcpyDeviceToDevice,
                              stream));
    } else if (kind == kKindFp8) {
      if (int rc = fp8_quantize_rows(x, tokens, H, my_stage, reinterpret_cast<float*>(my_stage + sf_offset),
                                     rt->sms, stream))
        return rc;
    } else {
      if (int rc = nvfp4_quantize_rows(x, tokens, H, weights->x_scale, my_stage, my_stage + sf_offset, 0, stream))
        return rc;
    }
  }
  // 2. route plan (as wm_forward).
  RouteRows rows{at<int>(S, rt->sl.local_offset), at<int>(S, rt->sl.dst_rank), at<int>(S, rt->sl.dst_row),
                 at<int>(S, rt->sl.dst_prow)};
  if (small_plan_allowed(1ll * tokens * c.top_k)) {
    SmallPlan plan{};
    plan.shape = shape;
    plan.routes = routes;
    plan.gates = gates;
    plan.tokens = tokens;
    plan.local = local;
    plan.rows = rows;
    plan.tables = tables;
    plan.local_count = at<int>(S, rt->sl.local_count);
    plan.count_matrix = counts;
    plan.my_count_matrix = at<int>(rt->arena, rt->al.counts);
    plan.meta_origin = meta_origin;
    plan.meta_prob = meta_prob;
    plan.global_part = 1;
    plan.exchange = world > 1;
    plan.flag_counts = flag_group(rt, kCounts);
    plan.my_flag_counts = my_flags(rt, kCounts);
    plan.flag_ready = flag_group(rt, kReady);
    plan.my_flag_ready = my_flags(rt, kReady);
    plan.generation = world > 1 ? gen : Gen{};
    plan.row_capacity = rt->row_cap;
    plan.status = status;
    plan.chunks = 1;
    if (int rc = route_plan_small(plan, stream)) return rc;
  } else {
    if (int rc = route_local(shape, routes, tokens, local, at<int>(S, rt->sl.chunk_hist),
                             at<int>(S, rt->sl.local_count), counts, stream))
      return rc;
    if (world > 1)
      if (int rc = signal_peers(flag_group(rt, kCounts), world, c.rank, gen, stream)) return rc;
    if (int rc = route_global(shape, at<int>(rt->arena, rt->al.counts), my_flags(rt, kCounts),
                              world > 1 ? gen : Gen{}, rt->row_cap, tables, status, 1, stream))
      return rc;
    if (int rc = route_rows(shape, routes, gates, tokens, local, at<int>(S, rt->sl.chunk_hist), tables, rows,
                            meta_origin, meta_prob, rt->row_cap, status, stream))
      return rc;
    if (world > 1) {
      if (int rc = signal_peers(flag_group(rt, kReady), world, c.rank, gen, stream)) return rc;
      if (int rc = wait_flags(my_flags(rt, kReady), world, gen, status, tables.split, stream)) return rc;
    }
  }
  // 3. owner side: pull quantised rows + scale factors, FC1, SwiGLU + re-quantisation, FC2 -> mailboxes.
  OwnerRows owner{tables.padded_start, tables.tile_group, split_range(tables.split, 2, kWhole),
                  tables.expert_total};
  if (int rc = gather_q_rows(owner, c.rank, rt->e_local, world, c.max_tokens, c.top_k, kind, H, stage, sf_offset,
                             at<int>(rt->arena, rt->al.meta_origin), at<float>(rt->arena, rt->al.meta_prob),
                             xq, sfa_x, origin, prob, 0, rt->sms * 8, stream))
    return rc;
  if (world > 1)
    if (int rc = signal_peers(flag_group(rt, kPulled), world, c.rank, gen, stream)) return rc;
  Schedule sched{tables.split, tables.tile_group, tables.padded_start, rt->e_local, rt->row_cap,
                 tables.pair_tiles, false, kWhole};
  const long long chunk = 512;
  const int kx = kind == kKindFp8 ? H / 128 : H / 64;   // scale-factor chunks per row tile along K
  const int ku = kind == kKindFp8 ? I / 128 : I / 64;
  const long long stage_chunks = kind == kKindFp8 ? 1 : 4;
  const SfLayout sfa1{reinterpret_cast<const uint8_t*>(sfa_x), 0, kx * chunk, stage_chunks * chunk, chunk};
  const SfLayout sfb1{static_cast<const uint8_t*>(weights->w1_sf), (2ll * I / 128) * kx * chunk, kx * chunk,
                      stage_chunks * chunk, chunk};
  const SfLayout sfa2{reinterpret_cast<const uint8_t*>(sfa_u), 0, ku * chunk, stage_chunks * chunk, chunk};
  const SfLayout sfb2{static_cast<const uint8_t*>(weights->w2_sf), (1ll * H / 128) * ku * chunk, ku * chunk,
                      stage_chunks * chunk, chunk};
  const float alpha1 = kind == kKindFp8 ? 1.0f : weights->x_scale * weights->w1_scale;
  const float alpha2 = kind == kKindFp8 ? 1.0f : weights->u_scale * weights->w2_scale;
  // FP8 weights whose block scales carry mantissas (imported checkpoints) come with the FP32 scales as well
  const float* w1_scales = kind == kKindFp8 ? weights->w1_scales : nullptr;
  const float* w2_scales = kind == kKindFp8 ? weights->w2_scales : nullptr;
  if (int rc = launch_block_scaled(kind, sched, xq, sfa1, weights->w1, sfb1, abq, nullptr, 2 * I, H, alpha1,
                                   status, rt->sms, stream, w1_scales))
    return rc;
  if (int rc = swiglu_quantize(split_range(tables.split, 2, kWhole), abq, prob, I, kind,
                               kind == kKindFp8 ? 1.0f : weights->u_scale, uq, sfa_u, rt->sms, stream))
    return rc;
  if (int rc = launch_block_scaled(kind, sched, uq, sfa2, weights->w2, sfb2, nullptr, &push, H, I, alpha2,
                                   status, rt->sms, stream, w2_scales))
    return rc;
  if (world > 1) {
    if (int rc = signal_peers(flag_group(rt, kContrib), world, c.rank, gen, stream)) return rc;
    if (int rc = wait_flags(my_flags(rt, kContrib), world, gen, status, nullptr, stream)) return rc;
  }
  return combine_rows(at<__nv_bfloat16>(rt->arena, rt->al.mailbox), local.sorted_expert, tokens,
                      c.max_tokens, c.top_k, c.hidden, static_cast<__nv_bfloat16*>(y), stream);
}

// =============================================================================== NVFP4 backward
// Reference: weftmoe/nvfp4_backward.py:59-112.  Every contraction reads operands quantised block-16 along
// ITS reduction axis: dU and dX use row-quantised dY / dAB against the prepared W2^T / W1^T; the weight
// gradients use dAB, X, dY, U transposed and quantised along the rows, contracted by the K-grouped mode
// of the block-scaled kernel.  dY travels in BF16 (pulled by the saved origins like the BF16 backward).
static int backward_nvfp4(wm_runtime* rt, const void* tape, const void* dy, const wm_quant_weights* w,
                          int32_t tokens, void* dx, float* dgates, void* dw1, void* dw2, void* stream_) {
  const wm_config& c = rt->cfg;
  if (tokens < 0 || tokens > c.max_tokens) {
    set_error("Backward token count %d exceeds capacity %d", tokens, c.max_tokens);
    return WM_ERR_CAPACITY;
  }
  if (!tape || !w || !w->w1 || !w->w1_sf || !w->w2 || !w->w2_sf || !dw1 || !dw2 ||
      (tokens > 0 && (!dy || !dx || !dgates)) || !aligned16(tape) || !aligned16(dy) || !aligned16(dx) ||
      !aligned16(dw1) || !aligned16(dw2)) {
    set_error("wm_backward_quantized: null or misaligned tensor (16-byte alignment required)");
    return WM_ERR_INVALID;
  }
  const float scales[6] = {w->x_scale, w->w1_scale, w->u_scale, w->w2_scale, w->dy_scale, w->dab_scale};
  for (float v : scales)
    if (!(v > 0.0f) || !std::isfinite(v)) {
      set_error("NVFP4 tensor scales must be finite and positive");
      return WM_ERR_INVALID;
    }
  const int H = c.hidden, I = c.intermediate;
  if (H > 8 * I) {
    set_error("NVFP4 backward needs hidden <= 8 * intermediate (scratch sizing)");
    return WM_ERR_INVALID;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const Gen gen = begin_generation(rt, stream);
  const int world = c.world;
  uint8_t* S = rt->scratch;
  const uint8_t* T = static_cast<const uint8_t*>(tape);
  auto tp = [&](size_t off) { return const_cast<uint8_t*>(T) + off; };
  int* status = at<int>(S, rt->sl.status);
  const int* sorted_slot = reinterpret_cast<const int*>(tp(rt->tl.sorted_slot));
  const int* sorted_expert = reinterpret_cast<const int*>(tp(rt->tl.sorted_expert));
  const int* padded_start = reinterpret_cast<const int*>(tp(rt->tl.padded_start));
  const int* tile_group = reinterpret_cast<const int*>(tp(rt->tl.tile_group));
  const int* pair_tiles = reinterpret_cast<const int*>(tp(rt->tl.pair_tiles));
  const int* split = reinterpret_cast<const int*>(tp(rt->tl.split));
  const int* origin = reinterpret_cast<const int*>(tp(rt->tl.origin));
  const float* prob = reinterpret_cast<const float*>(tp(rt->tl.prob));
  const uint8_t* xq = tp(rt->tl.xrows);
  const uint8_t* sf_x = tp(rt->tl.xrows) + align_up(static_cast<size_t>(rt->row_cap) * H);
  const auto* ab = reinterpret_cast<const __nv_bfloat16*>(tp(rt->tl.ab));
  auto* recv = at<__nv_bfloat16>(S, rt->sl.recv);
  auto* u = at<__nv_bfloat16>(S, rt->sl.u);
  auto* du = at<__nv_bfloat16>(S, rt->sl.du);
  auto* dab = at<__nv_bfloat16>(S, rt->sl.dab);
  uint8_t* qrows = at<uint8_t>(S, rt->sl.abq);       // row-quantised dY, then dAB (<= row_cap * 4I bytes)
  uint8_t* sf_dy = at<uint8_t>(S, rt->sl.sfa_x);     // H / 64 chunks per row tile
  uint8_t* sf_dab = at<uint8_t>(S, rt->sl.sfa_u);    // 2I / 64 chunks per row tile
  uint8_t* qa = at<uint8_t>(S, rt->sl.wq_a);
  uint8_t* qb = at<uint8_t>(S, rt->sl.wq_b);
  uint8_t* sa = at<uint8_t>(S, rt->sl.wsf_a);
  uint8_t* sb = at<uint8_t>(S, rt->sl.wsf_b);
  const int R = rt->row_cap;

  PeerConstRows stage{};
  PeerFloats dgate_box{};
  PushTarget push{};
  for (int r = 0; r < world; ++r) {
    stage.p[r] = at<__nv_bfloat16>(rt->peer[r], rt->al.stage);
    dgate_box.p[r] = at<float>(rt->peer[r], rt->al.dgate_box);
    push.mailbox[r] = at<__nv_bfloat16>(rt->peer[r], rt->al.mailbox);
  }
  push.origin = origin;
  push.cap = c.max_tokens;
  push.top_k = c.top_k;

  // 1. stage dY (BF16) and pull its rows in the saved row order.
  if (world > 1)
    if (int rc = wait_flags(my_flags(rt, kPulled), world, gen - 1, status, nullptr, stream)) return rc;
  if (world == 1)
    stage.p[0] = static_cast<const __nv_bfloat16*>(dy);
  else if (tokens > 0)
    WM_CUDA(cudaMemcpyAsync(rt->arena + rt->al.stage, dy, 2ull * tokens * H, cudaMemcpyDeviceToDevice, stream));
  if (world > 1) {
    if (int rc = signal_peers(flag_group(rt, kReady), world, c.rank, gen, stream)) return rc;
    if (int rc = wait_flags(my_flags(rt, kReady), world, gen, status, const_cast<int*>(split), stream)) return rc;
  }
  const DeviceRange all_rows = split_range(split, 2, kWhole);
  if (int rc = gather_by_origin(all_rows, origin, nullptr, world, c.max_tokens, c.top_k, H, stage, recv, rt->sms * 8,
                                stream))
    return rc;
  if (world > 1)
    if (int rc = signal_peers(flag_group(rt, kPulled), world, c.rank, gen, stream)) return rc;
  Schedule sched{split, tile_group, padded_start, rt->e_local, R, pair_tiles, false, kWhole};
  const long long chunk = 512;
  const int kh = H / 64, ki2 = 2 * I / 64;
  // 2. dU = q(dY) W2: dY rows quantised along H against W2^T [I][H].
  if (int rc = nvfp4_quantize_rows(recv, R, H, w->dy_scale, qrows, sf_dy, 1, stream, all_rows.end)) return rc;
  const SfLayout sfa_dy{sf_dy, 0, kh * chunk, 4 * chunk, chunk};
  const SfLayout sfb_w2t{static_cast<const uint8_t*>(w->w2_sf), (1ll * I / 128) * kh * chunk, kh * chunk, 4 * chunk,
                         chunk};
  if (int rc = launch_block_scaled(kKindNvfp4, sched, qrows, sfa_dy, w->w2, sfb_w2t, du, nullptr, I, H,
                                   w->dy_scale * w->w2_scale, status, rt->sms, stream))
    return rc;
  // 3. SwiGLU backward in FP32 on the saved BF16 gate/up rows: U, dAB, dprob -> sources.
  if (int rc = swiglu_backward(all_rows, ab, du, prob, origin, I, c.max_tokens, c.top_k, u, dab, dgate_box,
                               rt->sms, stream))
    return rc;
  // 4. dX = q(dAB) W1 -> sources' mailboxes: dAB rows quantised along 2I against W1^T [H][2I].
  if (int rc = nvfp4_quantize_rows(dab, R, 2 * I, w->dab_scale, qrows, sf_dab, 1, stream, all_rows.end)) return rc;
  const SfLayout sfa_dab{sf_dab, 0, ki2 * chunk, 4 * chunk, chunk};
  const SfLayout sfb_w1t{static_cast<const uint8_t*>(w->w1_sf), (1ll * H / 128) * ki2 * chunk, ki2 * chunk,
                         4 * chunk, chunk};
  if (int rc = launch_block_scaled(kKindNvfp4, sched, qrows, sfa_dab, w->w1, sfb_w1t, nullptr, &push, H, 2 * I,
                                   w->dab_scale * w->w1_scale, status, rt->sms, stream))
    return rc;
  if (world > 1)
    if (int rc = signal_peers(flag_group(rt, kContrib), world, c.rank, gen, stream)) return rc;
  // 5. weight gradients: operands transposed, quantised along the rows, contracted per expert.
  const long long per_tile = static_cast<long long>(R / 64) * chunk;
  const SfLayout la{sa, 0, per_tile, 4 * chunk, chunk}, lb{sb, 0, per_tile, 4 * chunk, chunk};
  auto along_rows = [&](const __nv_bfloat16* rows_in, int cols, float scale, uint8_t* q, uint8_t* sf) -> int {
    return nvfp4_quantize_cols(rows_in, R, cols, scale, q, sf, all_rows.end, rt->sms, stream);
  };
  if (int rc = along_rows(dab, 2 * I, w->dab_scale, qa, sa)) return rc;
  if (int rc = nvfp4_requantize_cols(xq, sf_x, R, H, w->x_scale, qb, sb, all_rows.end, rt->sms, stream)) return rc;
  if (int rc = launch_block_scaled_kgrouped(kKindNvfp4, sched, qa, la, qb, lb, static_cast<__nv_bfloat16*>(dw1),
                                            2 * I, H, w->dab_scale * w->x_scale, status, rt->sms, stream))
    return rc;
  if (int rc = along_rows(recv, H, w->dy_scale, qa, sa)) return rc;
  if (int rc = along_rows(u, I, w->u_scale, qb, sb)) return rc;
  if (int rc = launch_block_scaled_kgrouped(kKindNvfp4, sched, qa, la, qb, lb, static_cast<__nv_bfloat16*>(dw2), H, I,
                                            w->dy_scale * w->u_scale, status, rt->sms, stream))
    return rc;
  // 6. source side: ordered combine of dX, dprob back to the original slots.
  if (world > 1)
    if (int rc = wait_flags(my_flags(rt, kContrib), world, gen, status, nullptr, stream)) return rc;
  if (int rc = combine_rows(at<__nv_bfloat16>(rt->arena, rt->al.mailbox), sorted_expert, tokens, c.max_tokens,
                            c.top_k, H, static_cast<__nv_bfloat16*>(dx), stream))
    return rc;
  return unpermute_dgates(at<float>(rt->arena, rt->al.dgate_box), sorted_slot, sorted_expert, tokens, c.top_k,
                          dgates, stream);
}

// =============================================================================== FP8 backward
// Mixed precision (stated in the header): both dgrad contractions run in blockwise FP8 against the
// prepared transposed weights, exactly like the forward GEMMs; the two weight-gradient contractions run
// in BF16 on the dequantised saved X and the dequantised dY rows (one E4M3 rounding each, no second
// column-wise re-quantisation as in the reference, docs/usage.md:122-125).
extern "C" int wm_backward_quantized(wm_runtime* rt, const void* tape, const void* dy,
                                     const wm_quant_weights* transposed, int32_t tokens, void* dx,
                                     float* dgates, void* dw1, void* dw2, void* stream_) {
  if (int rc = check_ready(rt, "wm_backward_quantized")) return rc;
  const wm_config& c = rt->cfg;
  if (!c.training || c.reserved == 0) {
    set_error("Backward requires an FP8 or NVFP4 runtime prepared with training=True");
    return WM_ERR_STATE;
  }
  if (c.reserved == 2) return backward_nvfp4(rt, tape, dy, transposed, tokens, dx, dgates, dw1, dw2, stream_);
  if (tokens < 0 || tokens > c.max_tokens) {
    set_error("Backward token count %d exceeds capacity %d", tokens, c.max_tokens);
    return WM_ERR_CAPACITY;
  }
  const bool prequantised = transposed && transposed->source_q != nullptr;
  if (prequantised && (!transposed->source_scales || !aligned16(transposed->source_q) ||
                       !aligned16(transposed->source_scales))) {
    set_error("wm_backward_quantized: a prequantised dY needs 16-byte aligned bytes and scales");
    return WM_ERR_INVALID;
  }
  if (!tape || !transposed || !transposed->w1 || !transposed->w1_sf || !transposed->w2 || !transposed->w2_sf ||
      !dw1 || !dw2 || (tokens > 0 && ((!dy && !prequantised) || !dx || !dgates)) || !aligned16(tape) || !aligned16(dy) ||
      !aligned16(dx) || !aligned16(dw1) || !aligned16(dw2)) {
    set_error("wm_backward_quantized: null or misaligned tensor (16-byte alignment required)");
    return WM_ERR_INVALID;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const Gen gen = begin_generation(rt, stream);
  const int world = c.world;
  const int H = c.hidden, I = c.intermediate;
  uint8_t* S = rt->scratch;
  const uint8_t* T = static_cast<const uint8_t*>(tape);
  auto tp = [&](size_t off) { return const_cast<uint8_t*>(T) + off; };
  int* status = at<int>(S, rt->sl.status);
  const int* sorted_slot = reinterpret_cast<const int*>(tp(rt->tl.sorted_slot));
  const int* sorted_expert = reinterpret_cast<const int*>(tp(rt->tl.sorted_expert));
  const int* padded_start = reinterpret_cast<const int*>(tp(rt->tl.padded_start));
  const int* tile_group = reinterpret_cast<const int*>(tp(rt->tl.tile_group));
  const int* pair_tiles = reinterpret_cast<const int*>(tp(rt->tl.pair_tiles));
  const int* split = reinterpret_cast<const int*>(tp(rt->tl.split));
  const int* origin = reinterpret_cast<const int*>(tp(rt->tl.origin));
  const float* prob = reinterpret_cast<const float*>(tp(rt->tl.prob));
  const uint8_t* xq = tp(rt->tl.xrows);
  const auto* sfa_x = reinterpret_cast<const uint32_t*>(tp(rt->tl.xrows) + align_up(static_cast<size_t>(rt->row_cap) * H));
  const auto* ab = reinterpret_cast<const __nv_bfloat16*>(tp(rt->tl.ab));
  // scratch: dyq rows reuse the `u`-sized + `abq` buffers is too small for H-wide rows; the BF16 row
  // buffers are: xrows (dequantised X), recv (dequantised dY); quantised rows: abq region (dY, dAB).
  auto* x_bf16 = at<__nv_bfloat16>(S, rt->sl.xrows);
  auto* dy_bf16 = at<__nv_bfloat16>(S, rt->sl.recv);
  auto* u = at<__nv_bfloat16>(S, rt->sl.u);
  auto* du = at<__nv_bfloat16>(S, rt->sl.du);
  auto* dab = at<__nv_bfloat16>(S, rt->sl.dab);
  uint8_t* qrows = at<uint8_t>(S, rt->sl.abq);          // 4*row_cap*I bytes >= row_cap*max(H, 2I)? checked below
  auto* sfa_q = at<uint32_t>(S, rt->sl.sfa_x);
  if (static_cast<size_t>(H) > 4ull * I) {
    set_error("FP8 backward needs hidden <= 4 * intermediate (scratch sizing)");
    return WM_ERR_INVALID;
  }

  PeerBytes stage{};
  PeerFloats dgate_box{};
  PushTarget push{};
  for (int r = 0; r < world; ++r) {
    stage.p[r] = rt->peer[r] + rt->al.stage;
    dgate_box.p[r] = at<float>(rt->peer[r], rt->al.dgate_box);
    push.mailbox[r] = at<__nv_bfloat16>(rt->peer[r], rt->al.mailbox);
  }
  push.origin = origin;
  push.cap = c.max_tokens;
  push.top_k = c.top_k;

  // 1. quantise dY (1 x 128) into the staging buffer, as X was in the forward pass.
  const size_t sf_offset = align_up(static_cast<size_t>(c.max_tokens) * H);
  if (world > 1)
    if (int rc = wait_flags(my_flags(rt, kPulled), world, gen - 1, status, nullptr, stream)) return rc;
  uint8_t* my_stage = rt->arena + rt->al.stage;
  if (tokens > 0 && prequantised) {
    WM_CUDA(cudaMemcpyAsync(my_stage, transposed->source_q, static_cast<size_t>(tokens) * H,
                            cudaMemcpyDeviceToDevice, stream));
    WM_CUDA(cudaMemcpyAsync(my_stage + sf_offset, transposed->source_scales,
                            static_cast<size_t>(tokens) * (H / 128) * sizeof(float), cudaMemcpyDeviceToDevice,
                            stream));
  } else if (tokens > 0) {
    if (int rc = fp8_quantize_rows(dy, tokens, H, my_stage, reinterpret_cast<float*>(my_stage + sf_offset),
                                   rt->sms, stream))
      return rc;
  }
  if (world > 1) {
    if (int rc = signal_peers(flag_group(rt, kReady), world, c.rank, gen, stream)) return rc;
    if (int rc = wait_flags(my_flags(rt, kReady), world, gen, status, const_cast<int*>(split), stream)) return rc;
  }
  // 2. owner side: pull the quantised dY rows by the saved origins.
  const DeviceRange all_rows = split_range(split, 2, kWhole);
  OwnerRows owner{padded_start, tile_group, all_rows, nullptr};
  if (int rc = gather_q_rows(owner, c.rank, rt->e_local, world, c.max_tokens, c.top_k, kKindFp8, H, stage, sf_offset,
                             origin, nullptr, qrows, sfa_q, nullptr, nullptr, 1, rt->sms * 8, stream))
    return rc;
  if (world > 1)
    if (int rc = signal_peers(flag_group(rt, kPulled), world, c.rank, gen, stream)) return rc;
  const bool many_rows = 1ll * tokens * c.top_k * world >= 1024ll * c.experts;
  Schedule sched{split, tile_group, padded_start, rt->e_local, rt->row_cap, pair_tiles, many_rows, kWhole};
  const long long chunk = 512;
  const int kh = H / 128, ki2 = 2 * I / 128;
  // 3. dU = dYq * W2 (as dYq [rows,H] x w2_t [I,H]^T); BF16 copy of dY for the weight gradient.
  const SfLayout sfa_dy{reinterpret_cast<const uint8_t*>(sfa_q), 0, kh * chunk, chunk, chunk};
  const SfLayout sfb_w2t{static_cast<const uint8_t*>(transposed->w2_sf), (1ll * I / 128) * kh * chunk, kh * chunk,
                         chunk, chunk};
  if (int rc = launch_block_scaled(kKindFp8, sched, qrows, sfa_dy, transposed->w2, sfb_w2t, du, nullptr, I, H,
                                   1.0f, status, rt->sms, stream, transposed->w2_scales))
    return rc;
  if (int rc = fp8_dequantize_rows(all_rows, qrows, sfa_q, H, dy_bf16, rt->sms, stream)) return rc;
  // 4. SwiGLU backward on the saved BF16 gate/up rows: U, dAB, dprob -> sources.
  if (int rc = swiglu_backward(all_rows, ab, du, prob, origin, I, c.max_tokens, c.top_k, u, dab, dgate_box,
                               rt->sms, stream))
    return rc;
  // 5. dX = q(dAB) * W1 (as dABq [rows,2I] x w1_t [H,2I]^T) -> sources' mailboxes.
  auto* sfa_d = at<uint32_t>(S, rt->sl.sfa_u);  // sized for 2I/128 chunks per row tile
  if (int rc = fp8_quantize_rows_chunked(all_rows, dab, 2 * I, qrows, sfa_d, rt->sms, stream)) return rc;
  const SfLayout sfa_dab{reinterpret_cast<const uint8_t*>(sfa_d), 0, ki2 * chunk, chunk, chunk};
  const SfLayout sfb_w1t{static_cast<const uint8_t*>(transposed->w1_sf), (1ll * H / 128) * ki2 * chunk,
                         ki2 * chunk, chunk, chunk};
  if (int rc = launch_block_scaled(kKindFp8, sched, qrows, sfa_dab, transposed->w1, sfb_w1t, nullptr, &push, H,
                                   2 * I, 1.0f, status, rt->sms, stream, transposed->w1_scales))
    return rc;
  if (world > 1)
    if (int rc = signal_peers(flag_group(rt, kContrib), world, c.rank, gen, stream)) return rc;
  // 6. weight gradients (fixed row order).  Default: BF16 on the dequantised saved X and dY rows.
  //    WM_FP8_WGRAD=1: the reference's recipe (docs/usage.md:122-125) - every operand re-quantised
  //    1 x 128 along the rows and the contraction run in blockwise FP8.
  if (int rc = fp8_dequantize_rows(all_rows, xq, sfa_x, H, x_bf16, rt->sms, stream)) return rc;
  static const bool fp8_wgrad = [] {
    const char* v = std::getenv("WM_FP8_WGRAD");
    return v && v[0] == '1';
  }();
  // FP32 gradients (FP32 master parameters) always take the BF16-operand contraction: its accumulators
  // leave unrounded, where the block-scaled recipe's epilogue writes BF16.
  const bool wgrad_f32 = transposed->wgrad_f32 != 0;
  if (fp8_wgrad && !wgrad_f32) {
    uint8_t* qa = at<uint8_t>(S, rt->sl.wq_a);
    uint8_t* qb = at<uint8_t>(S, rt->sl.wq_b);
    auto* sa = at<uint32_t>(S, rt->sl.wsf_a);
    auto* sb = at<uint32_t>(S, rt->sl.wsf_b);
    const long long per_tile = static_cast<long long>(rt->row_cap / 128) * chunk;
    const SfLayout la{reinterpret_cast<const uint8_t*>(sa), 0, per_tile, chunk, chunk};
    const SfLayout lb{reinterpret_cast<const uint8_t*>(sb), 0, per_tile, chunk, chunk};
    if (int rc = fp8_quantize_cols_chunked(all_rows, dab, 2 * I, rt->row_cap, qa, sa, rt->sms, stream)) return rc;
    if (int rc = fp8_quantize_cols_chunked(all_rows, x_bf16, H, rt->row_cap, qb, sb, rt->sms, stream)) return rc;
    if (int rc = launch_block_scaled_kgrouped(kKindFp8, sched, qa, la, qb, lb, static_cast<__nv_bfloat16*>(dw1),
                                              2 * I, H, 1.0f, status, rt->sms, stream))
      return rc;
    if (int rc = fp8_quantize_cols_chunked(all_rows, dy_bf16, H, rt->row_cap, qa, sa, rt->sms, stream)) return rc;
    if (int rc = fp8_quantize_cols_chunked(all_rows, u, I, rt->row_cap, qb, sb, rt->sms, stream)) return rc;
    if (int rc = launch_block_scaled_kgrouped(kKindFp8, sched, qa, la, qb, lb, static_cast<__nv_bfloat16*>(dw2), H,
                                              I, 1.0f, status, rt->sms, stream))
      return rc;
  } else {
    if (int rc = launch_kgrouped_tn(sched, dab, x_bf16, dw1, 2 * I, H, status, rt->sms, stream, wgrad_f32))
      return rc;
    if (int rc = launch_kgrouped_tn(sched, dy_bf16, u, dw2, H, I, status, rt->sms, stream, wgrad_f32)) return rc;
  }
  // 7. source side: ordered combine of dX, dprob back to the original slots.
  if (world > 1)
    if (int rc = wait_flags(my_flags(rt, kContrib), world, gen, status, nullptr, stream)) return rc;
  if (int rc = combine_rows(at<__nv_bfloat16>(rt->arena, rt->al.mailbox), sorted_expert, tokens, c.max_tokens,
                            c.top_k, c.hidden, static_cast<__nv_bfloat16*>(dx), stream))
    return rc;
  return unpermute_dgates(at<float>(rt->arena, rt->al.dgate_box), sorted_slot, sorted_expert, tokens, c.top_k,
                          dgates, stream);
}

extern "C" int wm_fp8_pack_weight_scales(const float* scales, int32_t rows, int32_t kblocks, void* out,
                                         void* stream) {
  if (rows < 0 || rows % 128 || kblocks < 0 || (static_cast<long long>(rows) * kblocks > 0 && (!scales || !out))) {
    set_error("wm_fp8_pack_weight_scales: rows must be a multiple of 128");
    return WM_ERR_INVALID;
  }
  return pack_fp8_scales(scales, rows, kblocks, 128, out, static_cast<cudaStream_t>(stream));
}

// =============================================================================== stand-alone plan
extern "C" int wm_route_plan(int32_t phase, int32_t world, int32_t rank, int32_t experts,
                             int32_t top_k, int32_t tokens, int32_t cap, int32_t row_capacity,
                             const int32_t* routes, int32_t* count_matrix, const wm_route_out* out,
                             void* stream_) {
  if (!out || !count_matrix || world < 1 || world > kMaxWorld || rank < 0 || rank >= world ||
      experts < 1 || experts % world || experts > 2048 || top_k < 1 || top_k > 32 || tokens < 0 ||
      tokens > cap || (tokens > 0 && !routes) || row_capacity < 0 || row_capacity % 128) {
    set_error("wm_route_plan: bad argument");
    return WM_ERR_INVALID;
  }
  // The planning kernel keeps one shared-memory word per local expert (at most 512), like the runtime.
  if (experts / world > 512 || top_k > experts) {
    set_error("wm_route_plan: experts / world must be <= 512 and top_k <= experts (E=%d world=%d K=%d)",
              experts, world, top_k);
    return WM_ERR_INVALID;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const size_t n = static_cast<size_t>(tokens) * top_k;
  const size_t chunks = (n + 1023) / 1024 + 1;
  Carver k;
  const size_t o_hist = k.take(sizeof(int) * chunks * experts);
  const size_t o_pos = k.take(sizeof(int) * (n + 1));
  const size_t o_cnt = k.take(sizeof(int) * experts);
  const size_t o_before = k.take(sizeof(int) * experts);
  const size_t o_status = k.take(sizeof(int));
  const size_t o_flags = k.take(sizeof(int) * kMaxWorld * kFlagStride);
  const size_t o_pairs = k.take(sizeof(int) * (2 * (row_capacity / 128 + 1) + 1));
  uint8_t* tmp = nullptr;
  WM_CUDA(cudaMalloc(&tmp, k.cursor));
  int device_code = 0;
  // Everything between the allocation and the free reports through rc, so tmp is never leaked.
  auto body = [&]() -> int {
    WM_CUDA(cudaMemsetAsync(tmp + o_status, 0, k.cursor - o_status, stream));
    RouteShape shape{experts, top_k, world, rank, cap};
    RouteLocal local{out->sorted_slot, out->sorted_expert, at<int>(tmp, o_pos)};
    PeerInts counts{};
    for (int r = 0; r < world; ++r) counts.p[r] = count_matrix;  // every "rank" shares one matrix
    PlanTables t{out->expert_total, at<int>(tmp, o_before), out->expert_base, out->expert_pbase,
                 out->padded_start, out->tile_group, out->num_tiles, out->padded_rows,
                 at<int>(tmp, o_pairs) + 1, at<int>(tmp, o_pairs)};
    RouteRows rows{out->local_offset, out->dst_rank, out->dst_row, out->dst_prow};
    if (small_plan_allowed(static_cast<long long>(n))) {
      // the single-launch planner of small calls, so that the tests of this entry cover it too
      SmallPlan plan{};
      plan.shape = shape;
      plan.routes = routes;
      plan.tokens = tokens;
      plan.local = local;
      plan.rows = rows;
      plan.tables = t;
      plan.local_count = at<int>(tmp, o_cnt);
      plan.count_matrix = counts;
      plan.my_count_matrix = count_matrix;
      plan.per_route_primary = out->dst_primary;
      plan.want_primary = out->dst_primary != nullptr;
      plan.global_part = phase == 1;
      plan.row_capacity = row_capacity;
      plan.status = at<int>(tmp, o_status);
      plan.chunks = 1;
      if (int rc = route_plan_small(plan, stream)) return rc;
      if (phase != 1) return 0;
    } else {
      if (int rc = route_local(shape, routes, tokens, local, at<int>(tmp, o_hist), at<int>(tmp, o_cnt), counts,
                               stream))
        return rc;
      if (phase != 1) return 0;
      // No exchange to wait for: generation 0 is satisfied by the zeroed flag words.
      if (int rc = route_global(shape, count_matrix, at<int>(tmp, o_flags), Gen{}, row_capacity, t,
                                at<int>(tmp, o_status), 1, stream))
        return rc;
      PeerInts no_origin{};
      PeerFloats no_prob{};
      if (int rc = route_rows(shape, routes, nullptr, tokens, local, at<int>(tmp, o_hist), t, rows, no_origin,
                              no_prob, row_capacity, at<int>(tmp, o_status), stream))
        return rc;
      if (out->dst_primary)
        if (int rc = route_primary(shape, tokens, local, rows, no_origin, out->dst_primary, row_capacity,
                                   at<int>(tmp, o_status), stream))
          return rc;
    }
    WM_CUDA(cudaMemcpyAsync(&device_code, tmp + o_status, sizeof(int), cudaMemcpyDeviceToHost, stream));
    return 0;
  };
  const int rc = body();
  cudaError_t e = cudaStreamSynchronize(stream);
  cudaFree(tmp);
  if (rc) return rc;
  if (e != cudaSuccess) {
    set_error("wm_route_plan: %s", cudaGetErrorString(e));
    return WM_ERR_CUDA;
  }
  if (device_code) {
    set_error("wm_route_plan: device status %d", device_code);
    return map_status(device_code);
  }
  return WM_OK;
}

// =============================================================================== wait diagnostics
extern "C" int wm_debug_set_wait_budget(long long cycles) {
  set_flag_wait_budget(cycles);
  return WM_OK;
}

extern "C" int wm_debug_wait_flag(wm_runtime* rt, const int32_t* flag_word, int32_t target, void* stream_) {
  if (int rc = check_ready(rt, "wm_debug_wait_flag")) return rc;
  if (!flag_word) {
    set_error("wm_debug_wait_flag: null flag word");
    return WM_ERR_INVALID;
  }
  // One flag ("world" 1) on the caller's word, this runtime's status word, the current budget.
  return wait_flags(flag_word, 1, Gen{nullptr, target}, at<int>(rt->scratch, rt->sl.status), nullptr,
                    static_cast<cudaStream_t>(stream_));
}

// =============================================================================== instrumentation
extern "C" long long wm_launch_count(void) { return wm::launch_count(); }
extern "C" int wm_stage_count(void) { return kStageCount; }
extern "C" const char* wm_stage_name(int stage) {
  return stage >= 0 && stage < kStageCount ? kStageNames[stage] : "";
}

extern "C" int wm_runtime_enable_timing(wm_runtime* rt, int enable) {
  if (int rc = check_ready(rt, "wm_runtime_enable_timing")) return rc;
  if (enable && rt->slots.empty()) rt->slots.resize(kTimingRing);  // events are created at first use
  rt->timing = enable != 0;
  return WM_OK;
}

extern "C" int wm_runtime_read_timing(wm_runtime* rt, double* total_ms, long long* calls, int reset) {
  if (int rc = check_ready(rt, "wm_runtime_read_timing")) return rc;
  for (auto& slot : rt->slots) harvest(rt, slot);
  for (int k = 0; k < kStageCount; ++k) {
    if (total_ms) total_ms[k] = rt->stage_ms[k];
    if (calls) calls[k] = rt->stage_calls[k];
    if (reset) {
      rt->stage_ms[k] = 0.0;
      rt->stage_calls[k] = 0;
    }
  }
  return WM_OK;
}
