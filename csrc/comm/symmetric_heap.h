// Symmetric device memory: buffers that exist once per rank and that every rank of the node
// can address directly, so a kernel can store partial tiles into a peer GPU's memory over
// NVLink and bump counters there.  The reference has nothing like it: all of its inter-GPU
// traffic goes through host-launched NCCL calls (src/overlap_impl.cu:250-258, :303-315).
//
// A region is one cudaMalloc per rank, exported with cudaIpcGetMemHandle, exchanged through
// the NCCL communicator the runtime already owns (an all-gather of the 64-byte handles) and
// opened by the peers with cudaIpcOpenMemHandle.  Allocation is therefore a collective:
// every rank must allocate the same sizes in the same order.
//
// "Loopback" heaps back the single-GPU emulation used by tests: all `world` copies live on
// the current device and no inter-process exchange happens.
#pragma once
#include <cuda_runtime.h>
#include <nccl.h>

#include <cstddef>
#include <memory>
#include <vector>

namespace fo {

struct SymmetricRegion {
  size_t bytes = 0;
  int rank = 0;
  std::vector<void*> ptr;  // ptr[r]: rank r's copy as addressable from this process; ptr[rank] is local
  bool loopback = false;
  bool owned = true;           // false: registered by the caller, never freed here
  void* multicast = nullptr;   // NVSwitch multicast mapping of the buffer, if any
  void* local() const { return ptr[rank]; }
  bool contains(const void* p, size_t n) const {
    const char* b = static_cast<const char*>(ptr[rank]);
    const char* q = static_cast<const char*>(p);
    return q >= b && q + n <= b + bytes;
  }
};

class SymmetricHeap {
 public:
  // comm may be null only when world == 1 or loopback is true.
  SymmetricHeap(int rank, int world, ncclComm_t comm, bool loopback);
  ~SymmetricHeap();
  SymmetricHeap(const SymmetricHeap&) = delete;
  SymmetricHeap& operator=(const SymmetricHeap&) = delete;

  // Collective.  The memory is zero-filled before any peer can see it.
  SymmetricRegion* allocate(size_t bytes, cudaStream_t stream);
  // Collective: gives a region of allocate() back.  Every rank closes its mappings of the peers'
  // copies, all ranks meet (so that nobody frees memory a peer still has mapped), then each
  // frees its own copy.  The caller guarantees that no kernel on any rank still uses the region
  // (true after a later allocate() on the same stream has returned: its handle exchange is
  // ordered after everything enqueued before it on every rank).  Regions from adopt() are only
  // forgotten.
  void release(SymmetricRegion* region, cudaStream_t stream);
  // Records a symmetric buffer that somebody else allocated and mapped.
  SymmetricRegion* adopt(size_t bytes, const std::vector<void*>& ptrs, void* multicast);
  // Region of this heap that fully contains [p, p+n), or nullptr.
  const SymmetricRegion* find(const void* p, size_t n) const;

  // The owner of the communicator is going away: no collective call may follow.
  void detach_comm() { comm_ = nullptr; }
  int rank() const { return rank_; }
  int world() const { return world_; }
  bool loopback() const { return loopback_; }

 private:
  int rank_, world_;
  ncclComm_t comm_;
  bool loopback_;
  std::vector<std::unique_ptr<SymmetricRegion>> regions_;
};

}  // namespace fo
