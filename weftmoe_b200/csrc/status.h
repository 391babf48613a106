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


}  // namespace wm
