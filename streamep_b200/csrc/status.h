// Status block every bounded device wait reports into, and the ids used in it.  Plain C++ (shared
// by host and device code).
#pragma once

namespace sep {

// Every wait in this library is bounded; when a wait gives up the kernel records why in a status
// block that the host reads after the launch, and returns normally (no trap, no hang).
enum StatusCode : int {
  kStatusOk = 0,
  kStatusTimeoutBarrier = 1,       // cross-rank flag barrier
  kStatusTimeoutMailbox = 2,       // waiting for a peer's published buffer record
  kStatusTimeoutTileGate = 3,      // pool_arrival_count never reached its target
  kStatusTimeoutTokenGate = 4,     // y_done / a_done stamp never arrived
  kStatusTimeoutPipeline = 5,      // an mbarrier inside a GEMM pipeline
  kStatusTimeoutTail = 6,          // end-of-kernel completion wait
  kStatusBadIndex = 7,             // bounds check (debug builds of the index math)
  kStatusOverflow = 8,             // capacity mode: a rank's pool layout does not fit the fixed regions
  kStatusRegionMismatch = 9,       // capacity mode: the ranks did not pick the same region for this dispatch
};

struct StatusBlock {
  int code;        // first failure wins (atomicCAS from 0)
  int kernel_id;
  int role;
  int rank;
  int where;       // tile / channel / token / peer, depending on code
  int expected;
  int observed;
  int abort;       // set together with code; every spin polls it so one failure drains all waits
};

enum KernelId : int {
  kKernelMetadata = 1, kKernelFill = 2, kKernelDispatch = 3, kKernelDispatchGrads = 4,
  kKernelCombine = 5, kKernelGemm = 6, kKernelBarrier = 7, kKernelProducer = 8,
};

}  // namespace sep
