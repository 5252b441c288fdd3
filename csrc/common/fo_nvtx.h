// Named ranges around the host entry points, visible in Nsight Systems timelines next to the
// kernels they launch.  NVTX v3 is header-only and costs a few nanoseconds per call when no
// tool is attached.  (The reference has no tracing hooks; its only timeline is a screenshot,
// docs/_static/image/typical_timeline.jpeg.)
#pragma once
#include <nvtx3/nvToolsExt.h>

namespace fo {

class NvtxRange {
 public:
  explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
  ~NvtxRange() { nvtxRangePop(); }
  NvtxRange(const NvtxRange&) = delete;
  NvtxRange& operator=(const NvtxRange&) = delete;
};

}  // namespace fo
