// Device status codes shared by kernels and the host runtime.
#pragma once

namespace wm {

// Status codes written to the device status word (first failure wins).
enum : int {
  kStatusOk = 0,
  kStatusTimeoutSmemFull = 101,   // MMA warp waited for a TMA stage
  kStatusTimeoutSmemEmpty = 102,  // TMA warp waited for a free stage
  kStatusTimeoutTmemFull = 103,   // epilogue waited for an accumulator
  kStatusTimeoutTmemEmpty = 104,  // MMA warp waited for a drained accumulator
  kStatusTimeoutPeerFlag = 110,   // a cross-rank generation flag never arrived
  kStatusBadRoute = 120,          // route id outside [-1, experts)
  kStatusRowOverflow = 121,       // received rows exceed the prepared capacity
};

// Diagnostic timeline buffer of the one-CTA grouped GEMM: 64 tiles x 12 stamps of CTA 0 (4 of the
// TMA producer, 4 of the MMA issuer, then the epilogue: accumulator ready, and the time at which
// epilogue warps 3, 4 and 5 finished the tile), then the (start, end) time of every CTA.
constexpr int kTimelineTileStamps = 12;
constexpr int kTimelineTileWords = 64 * kTimelineTileStamps;
constexpr int kTimelineWords = kTimelineTileWords + 2 * 1024;

}  // namespace wm
