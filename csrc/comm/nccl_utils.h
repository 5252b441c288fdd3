// NCCL bootstrap helpers: unique-id generation that can travel through Python as a list of
// int64 (reference: src/nccl_utils.cu:7-14, src/nccl_utils.h:10-19) and checked calls.
// Unlike the reference's NCCL_CHECK, which prints and exits the process, failures here
// throw, so they surface as Python exceptions.
#pragma once
#include <nccl.h>

#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

namespace fo {

// 128-byte ncclUniqueId packed into 16 int64 values.
std::vector<int64_t> generate_nccl_id();

// Inverse of generate_nccl_id(); throws if the list does not hold 16 values.
ncclUniqueId unpack_nccl_id(const std::vector<int64_t>& id);

inline void nccl_check(ncclResult_t r, const char* what, const char* file, int line) {
  if (r != ncclSuccess) {
    throw std::runtime_error(std::string("NCCL failure in ") + what + " at " + file + ":" +
                             std::to_string(line) + ": " + ncclGetErrorString(r));
  }
}

}  // namespace fo

#define FO_NCCL_CHECK(cmd) ::fo::nccl_check((cmd), #cmd, __FILE__, __LINE__)
