#include "nccl_utils.h"

#include <cstring>

namespace fo {

static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is expected to be 128 bytes");

std::vector<int64_t> generate_nccl_id() {
  ncclUniqueId uid;
  FO_NCCL_CHECK(ncclGetUniqueId(&uid));
  std::vector<int64_t> out(sizeof(ncclUniqueId) / sizeof(int64_t));
  std::memcpy(out.data(), &uid, sizeof(ncclUniqueId));
  return out;
}

ncclUniqueId unpack_nccl_id(const std::vector<int64_t>& id) {
  if (id.size() * sizeof(int64_t) != sizeof(ncclUniqueId)) {
    throw std::runtime_error("nccl id must be a list of 16 int64 values");
  }
  ncclUniqueId uid;
  std::memcpy(&uid, id.data(), sizeof(ncclUniqueId));
  return uid;
}

}  // namespace fo
