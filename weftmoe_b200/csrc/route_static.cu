// Route planning without any allocation: wm_route_plan_noalloc.
//
// Some hosts of this library must not allocate device memory when they plan routes: an inference
// server that has already handed every free byte of HBM to its own KV-cache / tensor pool (a
// cudaMalloc there fails or fragments the pool), and any caller on a latency-critical path, because
// cudaMalloc and cudaFree synchronise the whole device and stall every stream.  wm_route_plan
// (runtime.cu) takes its temporaries from cudaMalloc on every call; this variant takes them from
// one fixed array that lives in the library image instead.
//
// The array is a file-scope __device__ object: every GPU that loads the library carries its
// 1 MiB until the process exits.  Its name is only a host-side handle, not a device address, so
// the address is looked up once per device with cudaGetSymbolAddress (with that device current)
// and that pointer is what the kernels receive.  The look-up happens in the first call made on a
// device; make that first call before any stream capture.  Every call, the first included, ends by
// synchronising `stream` and reading the device status word back on the host.
//
// All calls on a device share the array and it keeps whatever the previous call left in it.  The
// words that must start at zero (status, flag words) are cleared on the caller's stream at the
// start of every call.  Two calls whose GPU work overlaps (different streams, or different host
// threads) would overwrite each other's temporaries: run them one after the other.
#include <mutex>

#include "../../include/weftmoe_b200.h"
#include "kernels.h"
#include "route.h"

using namespace wm;

namespace {

// Limits of the no-allocation variant (the scratch array is sized for exactly these).
constexpr int kMaxRoutes = 131072;        // tokens * top_k
constexpr int kMaxExperts = 512;          // global expert count
constexpr int kMaxRowCapacity = 262144;   // padded rows of the owner-side layout

constexpr size_t align256(size_t v) { return (v + 255) / 256 * 256; }
constexpr size_t kChunks = kMaxRoutes / 1024 + 1;
constexpr size_t kOffHist = 0;
constexpr size_t kOffPos = kOffHist + align256(sizeof(int) * kChunks * kMaxExperts);
constexpr size_t kOffCount = kOffPos + align256(sizeof(int) * (kMaxRoutes + 1));
constexpr size_t kOffBefore = kOffCount + align256(sizeof(int) * kMaxExperts);
constexpr size_t kOffStatus = kOffBefore + align256(sizeof(int) * kMaxExperts);
constexpr size_t kOffFlags = kOffStatus + align256(sizeof(int));
constexpr size_t kOffPairs = kOffFlags + align256(sizeof(int) * kMaxWorld * kFlagStride);
constexpr size_t kScratchBytes = kOffPairs + align256(sizeof(int) * (2 * (kMaxRowCapacity / 128 + 1) + 1));
static_assert(kScratchBytes <= (1u << 20), "the fixed scratch array is meant to stay within 1 MiB");

static __device__ __align__(256) unsigned char g_route_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
unsigned char* g_scratch_address[kMaxDevices] = {};

// Device address of the scratch array on the current device (looked up once per device).
int scratch_for_current_device(unsigned char** out) {
  int device = 0;
  WM_CUDA(cudaGetDevice(&device));
  if (device < 0 || device >= kMaxDevices) {
    set_error("wm_route_plan_noalloc: device ordinal %d is not supported", device);
    return WM_ERR_INVALID;
  }
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_address[device] == nullptr) {
    unsigned char* address = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&address), g_route_scratch);
    if (e != cudaSuccess || address == nullptr) {
      set_error("wm_route_plan_noalloc: cudaGetSymbolAddress failed on device %d: %s", device,
                cudaGetErrorString(e));
      return WM_ERR_CUDA;
    }
    g_scratch_address[device] = address;
  }
  *out = g_scratch_address[device];
  return WM_OK;
}

template <class T>
T* at(unsigned char* base, size_t off) { return reinterpret_cast<T*>(base + off); }

}  // namespace

extern "C" int wm_route_plan_noalloc(int32_t phase, int32_t world, int32_t rank, int32_t experts,
                                     int32_t top_k, int32_t tokens, int32_t cap,
                                     int32_t row_capacity, const int32_t* routes,
                                     int32_t* count_matrix, const wm_route_out* out, void* stream_) {
  if (!out || !count_matrix || world < 1 || world > kMaxWorld || rank < 0 || rank >= world ||
      experts < 1 || experts % world || top_k < 1 || top_k > 32 || top_k > experts || tokens < 0 || tokens > cap ||
      (tokens > 0 && !routes) || row_capacity < 0 || row_capacity % 128) {
    set_error("wm_route_plan_noalloc: bad argument");
    return WM_ERR_INVALID;
  }
  if (static_cast<long long>(tokens) * top_k > kMaxRoutes || experts > kMaxExperts ||
      row_capacity > kMaxRowCapacity) {
    set_error("wm_route_plan_noalloc: %lld routes / %d experts / %d rows exceed the fixed scratch "
              "(at most %d routes, %d experts, %d rows); use wm_route_plan",
              static_cast<long long>(tokens) * top_k, experts, row_capacity, kMaxRoutes, kMaxExperts,
              kMaxRowCapacity);
    return WM_ERR_CAPACITY;
  }
  unsigned char* tmp = nullptr;
  if (int rc = scratch_for_current_device(&tmp)) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  // The array still holds the previous call's words: clear status and flag words.
  WM_CUDA(cudaMemsetAsync(tmp + kOffStatus, 0, kOffPairs - kOffStatus, stream));
  RouteShape shape{experts, top_k, world, rank, cap};
  RouteLocal local{out->sorted_slot, out->sorted_expert, at<int>(tmp, kOffPos)};
  PeerInts counts{};
  for (int r = 0; r < world; ++r) counts.p[r] = count_matrix;
  int rc = route_local(shape, routes, tokens, local, at<int>(tmp, kOffHist), at<int>(tmp, kOffCount),
                       counts, stream);
  int device_code = 0;
  if (!rc && phase == 1) {
    PlanTables t{out->expert_total, at<int>(tmp, kOffBefore), out->expert_base, out->expert_pbase,
                 out->padded_start, out->tile_group, out->num_tiles, out->padded_rows,
                 at<int>(tmp, kOffPairs) + 1, at<int>(tmp, kOffPairs)};
    rc = route_global(shape, count_matrix, at<int>(tmp, kOffFlags), Gen{}, row_capacity, t,
                      at<int>(tmp, kOffStatus), 1, stream);
    RouteRows rows{out->local_offset, out->dst_rank, out->dst_row, out->dst_prow};
    PeerInts no_origin{};
    PeerFloats no_prob{};
    if (!rc)
      rc = route_rows(shape, routes, nullptr, tokens, local, at<int>(tmp, kOffHist), t, rows, no_origin,
                      no_prob, row_capacity, at<int>(tmp, kOffStatus), stream);
    // Needs no scratch of its own: it reads the per-route arrays written just above.
    if (!rc && out->dst_primary)
      rc = route_primary(shape, tokens, local, rows, no_origin, out->dst_primary, row_capacity,
                         at<int>(tmp, kOffStatus), stream);
    if (!rc && cudaMemcpyAsync(&device_code, tmp + kOffStatus, sizeof(int), cudaMemcpyDeviceToHost,
                               stream) != cudaSuccess)
      rc = WM_ERR_CUDA;
  }
  cudaError_t e = cudaStreamSynchronize(stream);
  if (rc) return rc;
  if (e != cudaSuccess) {
    set_error("wm_route_plan_noalloc: %s", cudaGetErrorString(e));
    return WM_ERR_CUDA;
  }
  if (device_code) {
    set_error("wm_route_plan_noalloc: device status %d (%s)", device_code,
              device_code == kStatusRowOverflow ? "rows exceed row_capacity" : "a device wait ran out");
    return device_code == kStatusRowOverflow ? WM_ERR_CAPACITY : WM_ERR_TIMEOUT;
  }
  return WM_OK;
}
