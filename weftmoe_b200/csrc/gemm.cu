// Host launchers for the tcgen05 grouped GEMM template (gemm.cuh) and tensor-map creation.
#include <cudaTypedefs.h>
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <mutex>
#include <vector>
#include <algorithm>

#include <cstdlib>
#include <cstring>

#include "gemm.cuh"
#include "gemm2.cuh"
#include "kernels.h"

namespace wm {

// ------------------------------------------------------------------ error text (thread local)
static thread_local char g_error[512] = "";
void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}
const char* last_error() { return g_error; }

static std::atomic<long long> g_launches{0};
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
long long launch_count() { return g_launches.load(std::memory_order_relaxed); }

// ------------------------------------------------------------------ tensor maps
static PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  });
  return fn;
}

// Encoded maps are cached per thread by (base, shape, box): a training step issues the same dozen
// descriptions every call (weights, row buffers of the arena and scratch, tape sections that the
// caching allocator hands back at the same addresses), so steady-state calls encode nothing on the host.
// A map only describes addresses and extents, it holds no reference to the memory: a stale entry whose
// key matches again describes the same bytes.
namespace {
struct TmapKey {
  const void* base;
  uint64_t inner, outer, stride;
  uint32_t box_inner, box_outer;
  int elem_bytes;
  bool operator==(const TmapKey& o) const {
    return base == o.base && inner == o.inner && outer == o.outer && stride == o.stride &&
           box_inner == o.box_inner && box_outer == o.box_outer && elem_bytes == o.elem_bytes;
  }
};
struct TmapSlot {
  TmapKey key{};
  CUtensorMap map;
  bool used = false;
};
constexpr int kTmapSlots = 256;  // direct-mapped; a collision just re-encodes
}  // namespace

static int encode_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner, uint64_t outer,
                          uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer);

int make_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner, uint64_t outer,
                 uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer) {
  static thread_local TmapSlot cache[kTmapSlots];
  const TmapKey key{base, inner, outer, row_stride_bytes, box_inner, box_outer, elem_bytes};
  uint64_t h = reinterpret_cast<uintptr_t>(base) >> 4;
  h = (h ^ (inner * 0x9E3779B97F4A7C15ull) ^ (outer * 0xC2B2AE3D27D4EB4Full) ^ (box_outer * 0x165667B19E3779F9ull) ^
       (static_cast<uint64_t>(box_inner) << 7) ^ static_cast<uint64_t>(elem_bytes)) * 0xD6E8FEB86659FD93ull;
  TmapSlot& slot = cache[(h >> 40) % kTmapSlots];
  if (slot.used && slot.key == key) {
    *out = slot.map;
    return 0;
  }
  if (int rc = encode_tmap_2d(out, base, elem_bytes, inner, outer, row_stride_bytes, box_inner, box_outer)) return rc;
  slot.key = key;
  slot.map = *out;
  slot.used = true;
  return 0;
}

static int encode_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner, uint64_t outer,
                          uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer) {
  auto fn = encode_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from the CUDA driver");
    return 3;
  }
  if (box_inner * elem_bytes != 128 || box_outer > 256 || (row_stride_bytes % 16) ||
      (reinterpret_cast<uintptr_t>(base) % 16)) {
    set_error("tensor map: box %ux%u / stride %llu / base %p violate TMA rules", box_inner,
              box_outer, (unsigned long long)row_stride_bytes, base);
    return 2;
  }
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType type = elem_bytes == 2   ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                   : elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                                     : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult r = fn(out, type,
                  2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult %d (inner %llu outer %llu)", (int)r,
              (unsigned long long)inner, (unsigned long long)outer);
    return 3;
  }
  return 0;
}

// ------------------------------------------------------------------ launch helpers
// Kernel choice.  Measured on B200 (35B-A3B-like shape): with about 2048 rows per expert the
// CTA-pair kernel wins on the long-K backward contractions (dU, dX, dW1, dW2: 6 x 32 KB stages
// hide the load latency) and loses on FC1/FC2 (epilogue-heavy or short K: the extra cross-CTA
// hop costs more than it saves); with about 256 rows per expert every second pair is half
// empty and the one-CTA kernel wins everywhere.  WM_GEMM_PAIR=0/1 forces one kernel (A/B runs).
static std::atomic<int> g_forced_pairs{-2};  // -2: not read yet, -1: automatic, 0: one CTA, 1: pair
void force_gemm_pairs(int mode) { g_forced_pairs.store(mode < 0 ? -1 : (mode ? 1 : 0)); }
static int forced_pairs() {
  int value = g_forced_pairs.load();
  if (value == -2) {
    const char* v = std::getenv("WM_GEMM_PAIR");
    value = v ? (v[0] == '0' ? 0 : 1) : -1;
    g_forced_pairs.store(value);
  }
  return value;
}
// Per-contraction overrides for A/B runs: WM_PAIR_FC1, WM_PAIR_FC2, WM_PAIR_DGRAD (dU / dX), WM_PAIR_WGRAD
// (dW1 / dW2) = 0 / 1; unset = the measured default below: with about 2048 rows per expert FC1 gains 3 - 8 %
// on the pair kernel (its long K loop hides the cross-CTA hops), FC2 (K = I, a store-heavy epilogue) loses
// 15 %.  The two kernels give the same bits (tests/test_gpu_gemm.py), so the choice may follow the batch.
enum Contraction { kFc1 = 0, kFc2 = 1, kDgrad = 2, kWgrad = 3 };
static int contraction_override(Contraction c) {
  static const int values[4] = {
      [] { const char* v = std::getenv("WM_PAIR_FC1"); return v ? (v[0] != '0') : -1; }(),
      [] { const char* v = std::getenv("WM_PAIR_FC2"); return v ? (v[0] != '0') : -1; }(),
      [] { const char* v = std::getenv("WM_PAIR_DGRAD"); return v ? (v[0] != '0') : -1; }(),
      [] { const char* v = std::getenv("WM_PAIR_WGRAD"); return v ? (v[0] != '0') : -1; }()};
  return values[c];
}
static bool use_pairs(const Schedule& s, Contraction c) {
  const int forced = forced_pairs();
  if (forced >= 0) return forced == 1;
  const int override = contraction_override(c);
  if (override >= 0) return override == 1;
  return c != kFc2 && s.many_rows_per_expert;
}

template <int BLOCK_N, bool A_MN, bool B_MN, bool GATE_UP, bool K_GROUPED, class Epi, int EPI_WARPS = 4>
static int launch_single(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& args,
                         const Epi& epi, int sms, cudaStream_t stream) {
  auto kernel = gemm_kernel<BLOCK_N, A_MN, B_MN, GATE_UP, K_GROUPED, Epi, EPI_WARPS>;
  constexpr int smem = GemmSmem<BLOCK_N>::kTotal;
  static PerDeviceOnce configured;  // one table per template instantiation
  if (int rc = opt_in_dynamic_smem(kernel, smem, configured)) return rc;
  kernel<<<sms, 64 + 32 * EPI_WARPS, smem, stream>>>(ta, tb, args, epi);
  WM_CUDA(cudaGetLastError());
  count_launch();
  return 0;
}

template <int BLOCK_N, bool A_MN, bool B_MN, bool GATE_UP, bool K_GROUPED, class Epi>
static int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& args,
                       const Schedule& s, const Epi& epi, int sms, cudaStream_t stream) {
  auto kernel = gemm2_kernel<BLOCK_N, A_MN, B_MN, GATE_UP, K_GROUPED, Epi>;
  constexpr int smem = Gemm2Smem<BLOCK_N>::kTotal;
  static PerDeviceOnce configured;  // one table per template instantiation
  if (int rc = opt_in_dynamic_smem(kernel, smem, configured)) return rc;
  const DeviceRange pairs = split_range(s.split, 1, s.chunk);
  Gemm2Args a2{args, pairs.begin, pairs.end, s.pair_tiles};
  kernel<<<sms & ~1, kGemmThreads, smem, stream>>>(ta, tb, a2, epi);  // clusters of two CTAs
  WM_CUDA(cudaGetLastError());
  count_launch();
  return 0;
}

template <int BLOCK_N, bool A_MN, bool B_MN, bool GATE_UP, bool K_GROUPED, class Epi>
static int launch(bool pair, const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& args,
                  const Schedule& s, const Epi& epi, int sms, cudaStream_t stream) {
  if (pair)
    return launch_pair<BLOCK_N, A_MN, B_MN, GATE_UP, K_GROUPED>(ta, tb, args, s, epi, sms, stream);
  return launch_single<BLOCK_N, A_MN, B_MN, GATE_UP, K_GROUPED>(ta, tb, args, epi, sms, stream);
}

// Device timeline (diagnostics; the idea of the reference's src/cuda/profiling/device_timeline.cuh).
// WM_DEBUG_TIMELINE=<names> makes the named one-CTA launchers (fc1, fc2, du, dx, nt, wgrad, or
// "all") hand the kernel a stamp buffer and print it to stderr after the launch.  Printing
// synchronises the device, so this is for investigation runs only.
static unsigned long long* g_timeline = nullptr;

static void dump_timeline(const char* what) {
  cudaDeviceSynchronize();
  std::vector<unsigned long long> t(kTimelineWords);
  cudaMemcpy(t.data(), g_timeline, t.size() * sizeof(unsigned long long), cudaMemcpyDeviceToHost);
  cudaMemset(g_timeline, 0, t.size() * sizeof(unsigned long long));
  unsigned long long first = ~0ull, last_start = 0, first_end = ~0ull, last_end = 0;
  int slowest = 0, fastest = 0;
  for (int c = 0; c < 1024; ++c) {
    const unsigned long long b = t[kTimelineTileWords + 2 * c], e = t[kTimelineTileWords + 2 * c + 1];
    if (!b) continue;
    first = std::min(first, b); last_start = std::max(last_start, b);
    if (e < first_end) { first_end = e; fastest = c; }
    if (e > last_end) { last_end = e; slowest = c; }
  }
  fprintf(stderr, "[%s] CTA starts within %lld ns; first CTA (%d) done at %lld ns, last (%d) at %lld ns\n", what,
          (long long)(last_start - first), fastest, (long long)(first_end - first), slowest,
          (long long)(last_end - first));
  const unsigned long long t0 = t[0];
  fprintf(stderr, "stamps of the CTA chosen with WM_DEBUG_TIMELINE_CTA (default 0)\n");
  fprintf(stderr, "tile | producer: start decoded first_stage last_stage | mma: start got_tmem first_full "
                  "last_full | epilogue: acc_ready done_w3 done_w4 done_w5 (ns, CTA 0)\n");
  for (int i = 0; i < 24 && t[i * kTimelineTileStamps]; ++i) {
    fprintf(stderr, "%3d |", i);
    for (int j = 0; j < kTimelineTileStamps; ++j)
      fprintf(stderr, " %7lld%s", (long long)(t[i * kTimelineTileStamps + j] - t0), (j == 3 || j == 7) ? " |" : "");
    fprintf(stderr, "\n");
  }
}

struct TimelineScope {
  const char* name;
  bool on = false;
  TimelineScope(const char* launcher, GemmArgs& a) : name(launcher) {
    const char* want = std::getenv("WM_DEBUG_TIMELINE");
    if (!want || !(std::strstr(want, launcher) || std::strstr(want, "all"))) return;
    if (!g_timeline) {
      if (cudaMalloc(&g_timeline, kTimelineWords * sizeof(unsigned long long)) != cudaSuccess) return;
      cudaMemset(g_timeline, 0, kTimelineWords * sizeof(unsigned long long));
    }
    a.timeline = g_timeline;
    if (const char* cta = std::getenv("WM_DEBUG_TIMELINE_CTA")) a.timeline_cta = std::atoi(cta);
    on = true;
  }
  ~TimelineScope() {
    if (on) dump_timeline(name);
  }
};

// WM_EPILOGUE_TMA=0 keeps the plain-store epilogue of dU / dW (comparison runs).
static bool tma_epilogue() {
  static const bool on = [] {
    const char* v = std::getenv("WM_EPILOGUE_TMA");
    return !(v && v[0] == '0');
  }();
  return on;
}

static GemmArgs base_args(const Schedule& s, int* status) {
  GemmArgs a{};
  const DeviceRange tiles = split_range(s.split, 0, s.chunk);
  a.tile_begin = tiles.begin;
  a.tile_end = tiles.end;
  a.tile_group = s.tile_group;
  a.group_row_start = s.group_row_start;
  a.group_live_rows = s.group_live_rows;
  a.group_order = s.group_order;
  a.groups = s.groups;
  a.status = status;
  return a;
}

int launch_fc1(const Schedule& s, const __nv_bfloat16* x, const __nv_bfloat16* w1, __nv_bfloat16* u,
               __nv_bfloat16* ab, const float* row_prob, int hidden, int inter, int* status,
               int sms, cudaStream_t stream) {
  CUtensorMap ta, tb;
  if (int rc = make_tmap_2d(&ta, x, 2, hidden, s.row_capacity, (uint64_t)hidden * 2, 64, 128)) return rc;
  if (int rc = make_tmap_2d(&tb, w1, 2, hidden, (uint64_t)s.groups * 2 * inter, (uint64_t)hidden * 2, 64, 128))
    return rc;
  GemmArgs a = base_args(s, status);
  a.n_tiles = inter / 128;
  a.k_total = hidden;
  a.b_group_rows = 2 * inter;
  a.gate_up_half = inter;
  EpilogueSwiglu epi{u, ab, row_prob, inter};
  TimelineScope timeline("fc1", a);
  return launch<256, false, false, true, false>(use_pairs(s, kFc1), ta, tb, a, s, epi, sms, stream);
}

template <bool B_MN>
static int launch_mgrouped(const Schedule& s, const __nv_bfloat16* a_ptr, const __nv_bfloat16* b_ptr,
                           __nv_bfloat16* out, const PushTarget* push, int n, int k, int* status,
                           int sms, cudaStream_t stream) {
  CUtensorMap ta, tb;
  if (int rc = make_tmap_2d(&ta, a_ptr, 2, k, s.row_capacity, (uint64_t)k * 2, 64, 128)) return rc;
  const int bn = (n % 256 == 0) ? 256 : 128;
  if (n % 128) {
    set_error("grouped GEMM needs N %% 128 == 0, got %d", n);
    return 2;
  }
  const bool pair = use_pairs(s, B_MN ? kDgrad : kFc2);  // B MN-major = dU / dX
  if (B_MN) {
    if (int rc = make_tmap_2d(&tb, b_ptr, 2, n, (uint64_t)s.groups * k, (uint64_t)n * 2, 64, 64)) return rc;
  } else {
    // K-major B: one box is the whole N tile (one CTA) or this CTA's half of it (CTA pair)
    if (int rc = make_tmap_2d(&tb, b_ptr, 2, k, (uint64_t)s.groups * n, (uint64_t)k * 2, 64,
                              pair ? bn / 2 : bn))
      return rc;
  }
  GemmArgs a = base_args(s, status);
  a.n_tiles = n / bn;
  a.k_total = k;
  a.b_group_rows = B_MN ? k : n;
  TimelineScope timeline(B_MN ? (push ? "dx" : "du") : (push ? "fc2" : "nt"), a);
  if (push) {
    if (bn == 256) {
      EpiloguePush<256> epi{};
      for (int r = 0; r < kMaxPeers; ++r) epi.mailbox[r] = push->mailbox[r];
      epi.origin = push->origin; epi.cap = push->cap; epi.top_k = push->top_k; epi.ld = n;
      return launch<256, false, B_MN, false, false>(pair, ta, tb, a, s, epi, sms, stream);
    }
    EpiloguePush<128> epi{};
    for (int r = 0; r < kMaxPeers; ++r) epi.mailbox[r] = push->mailbox[r];
    epi.origin = push->origin; epi.cap = push->cap; epi.top_k = push->top_k; epi.ld = n;
    return launch<128, false, B_MN, false, false>(pair, ta, tb, a, s, epi, sms, stream);
  }
  if (bn == 256 && tma_epilogue()) {
    EpilogueStoreTma<256> epi{};
    if (int rc = make_tmap_2d(&epi.tmap, out, 2, n, s.row_capacity, (uint64_t)n * 2, 64, 32)) return rc;
    epi.rows_per_group = 0;
    return launch<256, false, B_MN, false, false>(pair, ta, tb, a, s, epi, sms, stream);
  }
  if (bn == 256) {
    EpilogueStore<256> epi{out, 0, n};
    return launch<256, false, B_MN, false, false>(pair, ta, tb, a, s, epi, sms, stream);
  }
  EpilogueStore<128> epi{out, 0, n};
  return launch<128, false, B_MN, false, false>(pair, ta, tb, a, s, epi, sms, stream);
}

int launch_du_swiglu_backward(const Schedule& s, const __nv_bfloat16* dy_rows, const __nv_bfloat16* w2,
                              const __nv_bfloat16* ab, const float* row_prob, __nv_bfloat16* u,
                              __nv_bfloat16* dab, float* dprob_part, int inter, int hidden, int* status,
                              int sms, cudaStream_t stream) {
  if (inter % 256 || use_pairs(s, kDgrad)) return -1;
  CUtensorMap ta, tb;
  if (int rc = make_tmap_2d(&ta, dy_rows, 2, hidden, s.row_capacity, (uint64_t)hidden * 2, 64, 128)) return rc;
  if (int rc = make_tmap_2d(&tb, w2, 2, inter, (uint64_t)s.groups * hidden, (uint64_t)inter * 2, 64, 64)) return rc;
  GemmArgs a = base_args(s, status);
  a.n_tiles = inter / 256;
  a.k_total = hidden;
  a.b_group_rows = hidden;
  TimelineScope timeline("du", a);
  EpilogueSwigluBackward epi{ab, row_prob, u, dab, dprob_part, inter, s.row_capacity};
  return launch_single<256, false, true, false, false, EpilogueSwigluBackward, 8>(ta, tb, a, epi, sms, stream);
}

int launch_mgrouped_nt(const Schedule& s, const __nv_bfloat16* a, const __nv_bfloat16* b,
                       __nv_bfloat16* out, const PushTarget* push, int n, int k, int* status,
                       int sms, cudaStream_t stream) {
  return launch_mgrouped<false>(s, a, b, out, push, n, k, status, sms, stream);
}
int launch_mgrouped_nn(const Schedule& s, const __nv_bfloat16* a, const __nv_bfloat16* b,
                       __nv_bfloat16* out, const PushTarget* push, int n, int k, int* status,
                       int sms, cudaStream_t stream) {
  return launch_mgrouped<true>(s, a, b, out, push, n, k, status, sms, stream);
}

int launch_kgrouped_tn(const Schedule& s, const __nv_bfloat16* a_ptr, const __nv_bfloat16* b_ptr,
                       void* out_any, int m, int n, int* status, int sms,
                       cudaStream_t stream, bool out_is_f32) {
  if (m % 128 || n % 128) {
    set_error("K-grouped GEMM needs M %% 128 == 0 and N %% 128 == 0, got %d x %d", m, n);
    return 2;
  }
  __nv_bfloat16* out = static_cast<__nv_bfloat16*>(out_any);
  CUtensorMap ta, tb;
  if (int rc = make_tmap_2d(&ta, a_ptr, 2, m, s.row_capacity, (uint64_t)m * 2, 64, 64)) return rc;
  if (int rc = make_tmap_2d(&tb, b_ptr, 2, n, s.row_capacity, (uint64_t)n * 2, 64, 64)) return rc;
  const int bn = (n % 256 == 0) ? 256 : 128;
  const bool pair = use_pairs(s, kWgrad) && m % 256 == 0;  // a pair covers 256 output rows
  GemmArgs a = base_args(s, status);
  a.m_tiles_per_group = m / 128;
  a.n_tiles = n / bn;
  if (s.split != nullptr && s.chunk >= 0) {  // the experts of one chunk only
    const DeviceRange experts = split_range(s.split, 3, s.chunk);
    a.group_begin = experts.begin;
    a.group_end = experts.end;
  }
  TimelineScope timeline("wgrad", a);
  if (out_is_f32) {  // FP32 master parameters: the accumulators leave unrounded
    CUtensorMap map;
    if (int rc = make_tmap_2d(&map, out_any, 4, n, (uint64_t)s.groups * m, (uint64_t)n * 4, 32, 32)) return rc;
    if (bn == 256) {
      EpilogueStoreTmaF32<256> epi{map, m};
      return launch<256, true, true, false, true>(pair, ta, tb, a, s, epi, sms, stream);
    }
    EpilogueStoreTmaF32<128> epi{map, m};
    return launch<128, true, true, false, true>(pair, ta, tb, a, s, epi, sms, stream);
  }
  if (bn == 256 && tma_epilogue()) {
    EpilogueStoreTma<256> epi{};
    if (int rc = make_tmap_2d(&epi.tmap, out, 2, n, (uint64_t)s.groups * m, (uint64_t)n * 2, 64, 32)) return rc;
    epi.rows_per_group = m;
    return launch<256, true, true, false, true>(pair, ta, tb, a, s, epi, sms, stream);
  }
  if (bn == 256) {
    EpilogueStore<256> epi{out, (long long)m * n, n};
    return launch<256, true, true, false, true>(pair, ta, tb, a, s, epi, sms, stream);
  }
  EpilogueStore<128> epi{out, (long long)m * n, n};
  return launch<128, true, true, false, true>(pair, ta, tb, a, s, epi, sms, stream);
}

}  // namespace wm
