// Device status word shared by every kernel that can give up on a wait.
//
// A kernel never traps and never spins without a limit.  When a bounded wait
// (mbarrier, peer flag, split-K semaphore) runs out, the kernel records ONE
// code in the status word it was handed, finishes its own teardown (in-flight
// bulk copies, TMEM) and returns.  The host reads the word after the stream (or
// the replayed graph) has completed and raises RPUBackendError.
#pragma once
#include <stdint.h>

namespace rf {

enum StatusCode : int32_t {
  kStatusOk = 0,
  kStatusTmaTimeout = 1,       // producer waited too long for a free smem stage
  kStatusMmaTimeout = 2,       // MMA issuer waited too long for a full smem stage
  kStatusEpilogueTimeout = 3,  // epilogue waited too long for the accumulator
  kStatusSplitKTimeout = 4,    // (reserved) split-K partner never arrived
  kStatusPeerTimeout = 5,      // a peer GPU's flag never reached the expected epoch
  kStatusBadArgument = 6,      // device-side argument check failed; access skipped
  kStatusBoundsCheck = 7,      // debug-build bounds check failed; access skipped
};

// Layout of the status block (int32 words) in device memory.
//   [0] first non-zero code recorded     [1] blockIdx.x of the reporter
//   [2] kernel id (see KernelTag)        [3] free-form detail (stage, rank ...)
constexpr int kStatusWords = 8;

enum KernelTag : int32_t {
  kTagGemmTc = 1,
  kTagGemmAr = 2,
  kTagAttnDecode = 3,
  kTagAttnPrefill = 4,
  kTagBarrier = 5,
  kTagMoe = 6,
  kTagW8A16 = 7,
};

}  // namespace rf
