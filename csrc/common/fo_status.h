// Status words written by device code and read back by the host runtime.
//
// Every device-side wait in this library is bounded.  When a wait gives up it
// records one of these codes (first writer wins) together with a small
// diagnostic payload, lets the kernel drain and returns, so the CUDA context
// stays usable and the host can raise a Python exception instead of hanging.
// The reference's wait kernel spins without a limit (src/wait.cuh:5-9).
#pragma once
#include <cstdint>
#include <string>

namespace fo {

enum StatusCode : int32_t {
  kStatusOk = 0,
  kStatusTimeoutSmemFull = 1,    // MMA warp gave up waiting for a TMA stage
  kStatusTimeoutSmemEmpty = 2,   // TMA warp gave up waiting for a free stage
  kStatusTimeoutTmemFull = 3,    // epilogue gave up waiting for an accumulator
  kStatusTimeoutTmemEmpty = 4,   // MMA warp gave up waiting for a free accumulator
  kStatusTimeoutGroupFlag = 5,   // reducer gave up waiting for a tile/group flag from peers
  kStatusTimeoutDoneFlag = 6,    // end-of-call handshake with peers timed out
  kStatusTimeoutStartFlag = 7,   // start-of-call handshake (staging still in use) timed out
  kStatusTimeoutWaitKernel = 8,  // standalone counting wait kernel timed out
  kStatusBadArgument = 9,
};

// Layout of the status buffer (int32 words).
constexpr int kStatusWordCode = 0;   // StatusCode, 0 when healthy
constexpr int kStatusWordArg0 = 1;   // e.g. group / tile index
constexpr int kStatusWordArg1 = 2;   // e.g. observed counter value
constexpr int kStatusWordArg2 = 3;   // e.g. expected counter value
constexpr int kStatusWords = 8;

inline const char* status_name(int32_t c) {
  switch (c) {
    case kStatusOk: return "ok";
    case kStatusTimeoutSmemFull: return "timeout: MMA warp waiting for TMA stage";
    case kStatusTimeoutSmemEmpty: return "timeout: TMA warp waiting for free stage";
    case kStatusTimeoutTmemFull: return "timeout: epilogue waiting for accumulator";
    case kStatusTimeoutTmemEmpty: return "timeout: MMA warp waiting for free accumulator";
    case kStatusTimeoutGroupFlag: return "timeout: reducer waiting for peers' tile/group flag";
    case kStatusTimeoutDoneFlag: return "timeout: end-of-call handshake with peers";
    case kStatusTimeoutStartFlag: return "timeout: start-of-call handshake with peers";
    case kStatusTimeoutWaitKernel: return "timeout: counting wait kernel";
    case kStatusBadArgument: return "bad argument";
    default: return "unknown";
  }
}

// Text of a non-zero status block, as check_status() raises it.
inline std::string status_message(const int64_t* words, int rank) {
  return std::string("flashoverlap device status: ") + status_name(static_cast<int32_t>(words[kStatusWordCode])) +
         " (args " + std::to_string(words[kStatusWordArg0]) + ", " + std::to_string(words[kStatusWordArg1]) + ", " +
         std::to_string(words[kStatusWordArg2]) + ") on rank " + std::to_string(rank);
}

}  // namespace fo
